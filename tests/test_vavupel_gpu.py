"""Vavupel through the engine against the plain model (tests/plain_vavupel.py): each mixer
alone, prompts against token-by-token steps, portions, unequal batches, slots and pages used
again, the window's edges, the sink and keys far back with a softmax that picks single keys,
the first tokens of a sequence, long decoding, odd, narrow and wide sizes, recorded steps,
greedy generation and trace replay."""

from __future__ import annotations

import copy
import json
import math
import os
import subprocess
import sys

import pytest
import torch

import plain_vavupel as plain
from vavupel_cases import (ALONE, BROAD, CORNERS, MIXED, NARROW, ODD, SHARP, STRAIGHT, WIDE, assert_close, plain_logits, prompts,
                           random_weights, rows_that_differ)

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def make_engine(cfg, weights, dtype, **kw):
    from strata_inference_b200.config.registry import spec_from_config
    from strata_inference_b200.engine.engine import Engine
    _, spec = spec_from_config(cfg)
    kw.setdefault("max_tokens", 2048)
    kw.setdefault("max_seq_len", 1024)
    return Engine(spec, weights, dtype=dtype, **kw)


def all_rows(n):
    return list(range(n))


def run_whole(eng, tokens):
    s = eng.new_sequence()
    out = eng.step([(s, tokens)], [all_rows(len(tokens))])
    eng.end_sequence(s)
    return out


def run_portions(eng, tokens, sizes):
    """The prompt cut into steps of the given sizes (the last takes the rest)."""
    s, at, rows = eng.new_sequence(), 0, []
    for n in list(sizes) + [len(tokens)]:
        part = tokens[at:at + n]
        if not part:
            break
        rows.append(eng.step([(s, part)], [all_rows(len(part))]))
        at += len(part)
    eng.end_sequence(s)
    return torch.cat(rows)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mixer_alone(name, dtype):
    cfg = ALONE[name]
    w = random_weights(cfg, seed=11)
    eng = make_engine(cfg, w, dtype)
    for toks in prompts(cfg, [1, 2, 5, 90], seed=3):
        assert_close(run_whole(eng, toks), plain_logits(cfg, w, toks), dtype, f"{name}, {len(toks)} tokens")
    toks = prompts(cfg, [95], seed=4)[0]
    assert_close(run_portions(eng, toks, [3, 1, 1, 2, 50] + [1] * 8), plain_logits(cfg, w, toks), dtype,
                 f"{name} in portions and single tokens")


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompt_then_long_decoding(dtype):
    """A prompt in one step, then 260 single-token steps (over page borders and well past every
    window; the token steps are recorded at the second and replayed from the third), and
    token by token from the very first token."""
    cfg = MIXED
    w = random_weights(cfg, seed=5)
    eng = make_engine(cfg, w, dtype)
    toks = prompts(cfg, [300], seed=6)[0]
    ref = plain_logits(cfg, w, toks)
    assert_close(run_portions(eng, toks, [40] + [1] * 260), ref, dtype, "prompt of 40, then token by token")
    assert_close(run_portions(eng, toks[:50], [1] * 30 + [20]), ref[:50], dtype, "token by token from the first token")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [[2, 2, 2, 2], [64, 25], [63, 2, 24], [1, 24, 3, 23], [17, 17, 17, 17, 17],
                                   [7, 8, 9, 16, 1, 15, 24], [39, 1, 1, 23, 2]])
def test_portions(sizes, dtype):
    """(the windows of the mixed model are 40, 100 and 64; the last list cuts at the first one's edge,
    the one before it around the scan's chunks of 8)"""
    cfg = MIXED
    w = random_weights(cfg, seed=7)
    eng = make_engine(cfg, w, dtype)
    toks = prompts(cfg, [140], seed=8)[0]
    assert_close(run_portions(eng, toks, sizes + [20] * 8), plain_logits(cfg, w, toks), dtype, f"portions {sizes}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batch_against_each_alone(dtype):
    """Prompts of 1 to 130 tokens in one step, then single-token steps together; the
    shorter requests end earlier and a new one takes a freed slot later."""
    cfg = MIXED
    w = random_weights(cfg, seed=9)
    eng = make_engine(cfg, w, dtype)
    reqs = prompts(cfg, [21, 22, 100, 160, 35], seed=10)
    first = [1, 2, 70, 130, 5]
    refs = [plain_logits(cfg, w, t) for t in reqs]
    live = [0, 1, 2, 3]
    slots = {i: eng.new_sequence() for i in live}
    out = eng.step([(slots[i], reqs[i][:first[i]]) for i in live], [all_rows(first[i]) for i in live])
    at = 0
    for i in live:
        assert_close(out[at:at + first[i]], refs[i][:first[i]], dtype, f"batched prompt {i}")
        at += first[i]
    pos = {i: first[i] for i in live}
    step = 0
    while live:
        if step == 25:                         # the latecomer starts alone, then decodes with the rest
            slots[4] = eng.new_sequence()
            got = eng.step([(slots[4], reqs[4][:first[4]])], [all_rows(first[4])])
            assert_close(got, refs[4][:first[4]], dtype, "late prompt")
            pos[4] = first[4]
            live.append(4)
        out = eng.step([(slots[i], [reqs[i][pos[i]]]) for i in live], [[0]] * len(live))
        for k, i in enumerate(live):
            assert_close(out[k:k + 1], refs[i][pos[i]:pos[i] + 1], dtype, f"request {i}, token {pos[i]}")
            pos[i] += 1
        for i in list(live):
            if pos[i] == len(reqs[i]):
                eng.end_sequence(slots[i])
                live.remove(i)
        step += 1
    assert step > 25


@pytest.mark.parametrize("dtype", DTYPES)
def test_slots_and_pages_used_again(dtype):
    """A slot that is given back and taken again starts from nothing: state, last token and
    pages of the request before leave no trace; with few pages they are all used again."""
    cfg = MIXED
    w = random_weights(cfg, seed=12)
    eng = make_engine(cfg, w, dtype, max_tokens=256, max_seq_len=256, max_slots=2)
    a, b, c = prompts(cfg, [100, 90, 120], seed=13)
    ra, rb, rc = (plain_logits(cfg, w, t) for t in (a, b, c))
    sa = eng.new_sequence()
    assert_close(eng.step([(sa, a[:70])], [all_rows(70)]), ra[:70], dtype, "a, first part")
    sb = eng.new_sequence()
    assert_close(eng.step([(sb, b[:50])], [all_rows(50)]), rb[:50], dtype, "b, first part")
    assert_close(eng.step([(sa, a[70:])], [all_rows(30)]), ra[70:], dtype, "a, second part")
    eng.end_sequence(sa)
    sc = eng.new_sequence()
    assert sc == sa
    assert_close(eng.step([(sc, c[:110])], [all_rows(110)]), rc[:110], dtype, "c in a's slot and pages")
    out = eng.step([(sb, [b[50]]), (sc, [c[110]])], [[0], [0]])
    assert_close(out, torch.stack([rb[50], rc[110]]), dtype, "b and c together")
    assert_close(eng.step([(sb, b[51:])], [all_rows(39)]), rb[51:], dtype, "b, the rest")
    eng.end_sequence(sb)
    eng.end_sequence(sc)
    assert_close(run_whole(eng, a), ra, dtype, "a once more")


def changed(cfg, edit):
    other = copy.deepcopy(cfg)
    edit(other)
    return other


def test_window_edges_sink_and_far_keys_with_a_sharp_softmax():
    """With a large scale the softmax puts most of a row's weight on single keys, wherever in
    the window they lie.  The plain model with a window one shorter or one longer gives other
    logits in two thirds of the rows behind the windows (that is checked first: the test can
    tell them apart); the engine agrees with the right one as a prompt, in portions around
    page borders and the windows' edges, and token by token."""
    cfg, dtype = SHARP, "float32"
    w = random_weights(cfg, seed=14)
    toks = prompts(cfg, [330], seed=15)[0]
    ref = plain_logits(cfg, w, toks)

    def window(delta):
        def edit(c):
            for layer in c["layers"]:
                layer["mixer"]["mask"]["size"] += delta
        return edit
    for delta in (-1, 1):
        other = plain_logits(changed(cfg, window(delta)), w, toks)
        assert rows_that_differ(ref[160:], other[160:], 20.0) > 100, f"a window off by {delta} would not show"
    eng = make_engine(cfg, w, dtype)
    assert_close(run_whole(eng, toks), ref, dtype, "whole prompt")
    assert_close(run_portions(eng, toks, [64, 64, 64, 64]), ref, dtype, "portions of one page")
    assert_close(run_portions(eng, toks, [63, 2, 63, 1, 1, 20, 66, 60]), ref, dtype, "portions around page borders")
    assert_close(run_portions(eng, toks, [66, 1, 1, 60, 21, 1, 1, 1, 90, 60]), ref, dtype, "portions around the windows' edges")
    assert_close(run_portions(eng, toks, [200] + [1] * 130), ref, dtype, "single tokens past both windows")
    # two requests of unequal length together: the shorter one's window starts elsewhere
    a, b = toks[:250], prompts(cfg, [180], seed=16)[0]
    rb = plain_logits(cfg, w, b)
    sa, sb = eng.new_sequence(), eng.new_sequence()
    out = eng.step([(sa, a[:200]), (sb, b[:100])], [all_rows(200), all_rows(100)])
    assert_close(out, torch.cat([ref[:200], rb[:100]]), dtype, "two prompts")
    for k in range(50):
        out = eng.step([(sa, [a[200 + k]]), (sb, [b[100 + k]])], [[0], [0]])
        assert_close(out, torch.stack([ref[200 + k], rb[100 + k]]), dtype, f"two requests, token {k}")


def test_sinks_that_take_much_of_the_weight():
    """Sinks raised by 3 take a large share of every row's weight; without them every row's
    logits are others (checked first).  Prompt, portions, tokens, and a batch."""
    cfg, dtype = ALONE["latent"], "float32"
    w = {n: (t + 3.0 if n.endswith(".sink") else t) for n, t in random_weights(cfg, seed=26).items()}
    a, b = prompts(cfg, [200, 77], seed=27)
    ra, rb = plain_logits(cfg, w, a), plain_logits(cfg, w, b)
    no_sink = {n: (t - 30.0 if n.endswith(".sink") else t) for n, t in w.items()}
    assert rows_that_differ(ra, plain_logits(cfg, no_sink, a)) == 200, "a sink left out would not show"
    eng = make_engine(cfg, w, dtype)
    assert_close(run_whole(eng, a), ra, dtype, "whole prompt")
    assert_close(run_portions(eng, a, [30, 2, 50] + [1] * 100), ra, dtype, "portions and single tokens")
    sa, sb = eng.new_sequence(), eng.new_sequence()
    out = eng.step([(sa, a[:150]), (sb, b[:60])], [all_rows(150), all_rows(60)])
    assert_close(out, torch.cat([ra[:150], rb[:60]]), dtype, "two prompts")
    for k in range(17):
        out = eng.step([(sa, [a[150 + k]]), (sb, [b[60 + k]])], [[0], [0]])
        assert_close(out, torch.stack([ra[150 + k], rb[60 + k]]), dtype, f"two requests, token {k}")


def test_first_tokens_and_the_previous_token_across_steps():
    """The first token takes the bigram table's last row, every other one the row of (previous
    token, token), also when the previous token came in an earlier step or the slot held
    another request before; the plain model with another hash gives other logits."""
    cfg, dtype = STRAIGHT, "float32"
    w = random_weights(cfg, seed=24)
    toks = prompts(cfg, [40], seed=25)[0]
    ref = plain_logits(cfg, w, toks)
    other = changed(cfg, lambda c: c["embedding"]["bigram"].update(mul_prev=c["embedding"]["bigram"]["mul_prev"] + 1))
    assert rows_that_differ(ref[1:], plain_logits(other, w, toks)[1:]) > 30
    eng = make_engine(cfg, w, dtype, max_slots=1)
    assert_close(run_portions(eng, toks, [1, 1, 1, 2, 2, 5]), ref, dtype, "first tokens one by one")
    assert_close(run_portions(eng, toks[::-1], [3, 1]), plain_logits(cfg, w, toks[::-1]), dtype, "the slot again")
    assert_close(run_whole(eng, toks[:1]), ref[:1], dtype, "one token alone")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["odd", "wide", "narrow", "straight", "broad"])
def test_other_sizes(name, dtype):
    cfg = {"odd": ODD, "wide": WIDE, "narrow": NARROW, "straight": STRAIGHT, "broad": BROAD}[name]
    w = random_weights(cfg, seed=16)
    eng = make_engine(cfg, w, dtype)
    a, b = prompts(cfg, [150, 37], seed=17)
    ra, rb = plain_logits(cfg, w, a), plain_logits(cfg, w, b)
    assert_close(run_whole(eng, a), ra, dtype, f"{name}: whole prompt")
    assert_close(run_portions(eng, a, [2, 60, 30] + [1] * 20), ra, dtype, f"{name}: portions and tokens")
    sa, sb = eng.new_sequence(), eng.new_sequence()
    out = eng.step([(sa, a[:130]), (sb, b[:30])], [[0, 129], [29]])
    assert_close(out, torch.stack([ra[0], ra[129], rb[29]]), dtype, f"{name}: two prompts")
    for k in range(7):
        out = eng.step([(sa, [a[130 + k]]), (sb, [b[30 + k]])], [[0], [0]])
        assert_close(out, torch.stack([ra[130 + k], rb[30 + k]]), dtype, f"{name}: tokens {k}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CORNERS))
def test_corner_configurations(name, dtype):
    """A prompt of 330 tokens (over five pages), then 30 single tokens, and a batch of three."""
    cfg = CORNERS[name]
    w = random_weights(cfg, seed=31)
    eng = make_engine(cfg, w, dtype)
    a, b, c = prompts(cfg, [360, 3, 90], seed=32)
    ra, rb, rc = (plain_logits(cfg, w, t) for t in (a, b, c))
    assert_close(run_portions(eng, a, [330] + [1] * 30), ra, dtype, f"{name}: prompt, then tokens")
    slots = [eng.new_sequence() for _ in range(3)]
    out = eng.step([(slots[0], a[:200]), (slots[1], b[:1]), (slots[2], c[:70])], [all_rows(200), [0], all_rows(70)])
    assert_close(out, torch.cat([ra[:200], rb[:1], rc[:70]]), dtype, f"{name}: three prompts")
    for k in range(2):
        out = eng.step([(slots[0], [a[200 + k]]), (slots[1], [b[1 + k]]), (slots[2], [c[70 + k]])], [[0]] * 3)
        assert_close(out, torch.stack([ra[200 + k], rb[1 + k], rc[70 + k]]), dtype, f"{name}: three tokens {k}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_recorded_prompt_steps(dtype):
    """Prompt steps of one shape: launched, recorded, then replayed for other prompts (also
    shorter ones, filled up with rows that belong to no sequence)."""
    cfg = MIXED
    w = random_weights(cfg, seed=18)
    eng = make_engine(cfg, w, dtype)
    for n, seed in ((60, 1), (64, 2), (50, 3), (33, 4), (64, 5)):
        toks = prompts(cfg, [n], seed=seed)[0]
        s = eng.new_sequence()
        out = eng.step([(s, toks)], [[0, n - 1]])
        eng.end_sequence(s)
        ref = plain_logits(cfg, w, toks)
        assert_close(out, torch.stack([ref[0], ref[n - 1]]), dtype, f"prompt of {n}")
    assert any(g.graph is not None for g in eng._prompt_graphs.values())


def write_model(path, cfg, weights):
    from strata_inference_b200.weights.safetensors_io import write_safetensors
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(path, "model.safetensors"),
                      {n: t.to(torch.bfloat16) for n, t in weights.items()})
    return path


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_generation_engine(tmp_path, dtype):
    """Unequal prompts through generate(): every chosen token is the plain model's best (or
    within rounding of it) given the run's own history."""
    from strata_inference_b200 import GenerationConfig, GenerationEngine, SamplingConfig
    cfg = MIXED
    w = random_weights(cfg, seed=19)
    model_dir = write_model(str(tmp_path / "model"), cfg, w)
    engine = GenerationEngine.from_dir(model_dir, dtype=dtype, max_tokens=1024, ctx=256)
    reqs = prompts(cfg, [3, 40, 75], seed=20)
    outs = engine.generate(reqs, GenerationConfig(max_tokens=24, sampling=SamplingConfig(temperature=0.0)))
    tol = {"float32": 1e-4, "bfloat16": 0.15}[dtype]
    for prompt, out in zip(reqs, outs):
        assert len(out.token_ids) == 24 and out.stop_reason == "max_tokens"
        logits = plain_logits(cfg, w, list(prompt) + list(out.token_ids))
        for k, tok in enumerate(out.token_ids):
            row = logits[len(prompt) + k - 1]
            gap = (row.max() - row[tok]).item()
            assert gap <= tol * row.abs().max().item(), f"token {k} ({tok}) lies {gap:.3e} below the best"


def test_trace_replay_of_a_model_folder(tmp_path):
    cfg, dtype = ODD, "float32"
    w = random_weights(cfg, seed=21)
    model_dir = write_model(str(tmp_path / "model"), cfg, w)
    a, b = prompts(cfg, [80, 30], seed=22)
    ra, rb = plain_logits(cfg, w, a), plain_logits(cfg, w, b)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:70], "want": [0, 69]},
                                     {"id": "b", "tokens": b[:20], "want": []}], "end": []}]
    for k in range(10):
        steps.append({"step": k + 1, "entries": [{"id": "a", "tokens": [a[70 + k]], "want": [0]},
                                                 {"id": "b", "tokens": [b[20 + k]], "want": [0] if k % 2 else []}],
                      "end": ["a", "b"] if k == 9 else []})
    out = str(tmp_path / "out")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir,
                        "--dtype", dtype, "--out", out, "--max-tokens", "256"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                       timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.split("\n") if l.startswith("done")] == [f"done {k}" for k in range(11)]
    V = cfg["vocab"]

    def read(step):
        import numpy as np
        return torch.from_numpy(np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4").reshape(-1, V).copy())
    assert_close(read(0), torch.stack([ra[0], ra[69]]), dtype, "prompts")
    for k in range(10):
        want = [ra[70 + k]] + ([rb[20 + k]] if k % 2 else [])
        assert_close(read(k + 1), torch.stack(want), dtype, f"step {k + 1}")


def test_command_line_generates_from_a_model_folder(tmp_path):
    cfg = ALONE["retention_ff"]
    w = random_weights(cfg, seed=23)
    model_dir = write_model(str(tmp_path / "model"), cfg, w)
    prompt = prompts(cfg, [9], seed=24)[0]
    p = subprocess.run([sys.executable, "-m", "strata_inference_b200.cli", "-m", model_dir, "--token-ids",
                        ",".join(map(str, prompt)), "-n", "6", "--temp", "0", "--output-format", "json",
                        "--dtype", "float32"], capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert p.returncode == 0, p.stderr[-2000:]
    out = json.loads(p.stdout)
    tokens = out["output_token_ids"]
    assert len(tokens) == 6 and out["stop_reason"] == "max_tokens"
    logits = plain_logits(cfg, w, list(prompt) + list(tokens))
    for k, tok in enumerate(tokens):
        row = logits[len(prompt) + k - 1]
        assert (row.max() - row[tok]).item() <= 1e-4 * row.abs().max().item()


# ---- the mechanisms' kernels alone ---------------------------------------------------------

def _dev(t, dtype=torch.float32):
    return t.to(dtype).cuda()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [64, 100, 1032])
def test_dynamic_tanh_alone_and_around_the_add(hidden, dtype):
    from strata_inference_b200.kernels import native
    g = torch.Generator().manual_seed(hidden)
    rows = 37
    w1, b1, w2, b2 = (torch.randn(hidden, generator=g) for _ in range(4))
    a1, a2 = torch.tensor([0.7]), torch.tensor([1.3])
    x = torch.randn((rows, hidden), generator=g).to(dtype)
    h = torch.randn((rows, hidden), generator=g)
    pick = torch.tensor([5, 0, 36, 5], dtype=torch.int32)
    out = torch.empty((4, hidden), dtype=torch.float32, device="cuda")
    native.dyt_norm(_dev(x, dtype), _dev(w1), _dev(b1), _dev(a1), out, pick.cuda())
    ref = torch.from_numpy(plain.dynamic_tanh(plain.f64(x.float()), plain.f64(w1), plain.f64(b1), 0.7))[pick.long()]
    assert (out.cpu().double() - ref).abs().max().item() < 1e-5
    hd, nxt = _dev(h), torch.empty((rows, hidden), dtype=dtype, device="cuda")
    native.add_dyt_norm(_dev(x, dtype), (_dev(w1), _dev(b1), _dev(a1)), hd, (_dev(w2), _dev(b2), _dev(a2)), nxt)
    h_ref = plain.f64(h) + plain.dynamic_tanh(plain.f64(x.float()), plain.f64(w1), plain.f64(b1), 0.7)
    n_ref = plain.dynamic_tanh(h_ref, plain.f64(w2), plain.f64(b2), 1.3)
    assert (hd.cpu().double() - torch.from_numpy(h_ref)).abs().max().item() < 1e-5
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert (nxt.cpu().double() - torch.from_numpy(n_ref)).abs().max().item() < tol * max(1.0, abs(n_ref).max())
    # no norm on the way out, none on the way in: a plain add and the stream as activations
    hd2, nxt2 = _dev(h), torch.empty((rows, hidden), dtype=dtype, device="cuda")
    native.add_dyt_norm(_dev(x, dtype), None, hd2, None, nxt2)
    assert (hd2.cpu().double() - torch.from_numpy(plain.f64(h) + plain.f64(x.float()))).abs().max().item() < 1e-5


@pytest.mark.parametrize("rows", [1, 8, 12, 130, 300])
def test_relu_squared_feed_forward_alone(rows):
    """The feed-forward part alone in bfloat16 at row counts that take the weight-streaming
    product, the library's and the tensor-core one."""
    from strata_inference_b200.parts.base import Runtime, build_part
    from strata_inference_b200.parts.feed_forward import PlainMLP
    g = torch.Generator().manual_seed(rows)
    hidden, inter = 128, 264
    stored = {"up_proj.weight": torch.randn((inter, hidden), generator=g) * 0.2,
              "down_proj.weight": torch.randn((hidden, inter), generator=g) * 0.2}
    stored = {n: t.to(torch.bfloat16) for n, t in stored.items()}
    rt = Runtime("cuda:0", torch.bfloat16)
    part = build_part(PlainMLP, ({"intermediate_size": inter, "activation": "relu_squared"}, hidden),
                      {n: t.cuda() for n, t in stored.items()}, rt)
    x = (torch.randn((rows, hidden), generator=g)).to(torch.bfloat16)
    got = part.forward(x.cuda(), None).float().cpu().double()
    ref = torch.from_numpy(plain.dense_ff(plain.f64(x.float()), {n.split("_")[0]: plain.f64(t.float()) for n, t in stored.items()}))
    assert (got - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()


def _latent_reference(q, keys_of, row_seq, row_pos, sink, scale, window):
    """64-bit: every head of every row over its sequence's rows (keys that are values too)."""
    rows, heads, kw = q.shape
    out = torch.zeros((rows, heads, kw), dtype=torch.float64)
    for r in range(rows):
        c = keys_of[row_seq[r]].double()
        p = row_pos[r]
        lo = max(0, p - window + 1) if window else 0
        for h in range(heads):
            s = (c[lo:p + 1] @ q[r, h].double()) * scale
            top = max(s.max().item(), sink[h].item())
            e = torch.exp(s - top)
            out[r, h] = (e @ c[lo:p + 1]) / (e.sum() + math.exp(sink[h].item() - top))
    return out


@pytest.mark.parametrize("heads, kw, window", [(16, 512, 0), (5, 80, 77), (3, 48, 17), (20, 64, 40),
                                               (1, 16, 5), (8, 256, 300)])
def test_tensor_core_latent_attention_alone(heads, kw, window):
    """The bfloat16 kernel against a 64-bit sum over the same bfloat16 rows: prompts of unequal
    lengths in one step (rows of a tile from two sequences), then single rows over a paged
    cache whose pages lie in any order, whole and cut into runs of keys."""
    from types import SimpleNamespace
    from strata_inference_b200.kernels import native
    g = torch.Generator().manual_seed(heads * 1000 + kw)
    lens = [37, 1, 150, 5]
    scale = 2.0 / math.sqrt(kw)
    keys_of = [(torch.randn((n, kw), generator=g)).to(torch.bfloat16) for n in lens]
    sink = torch.randn(heads, generator=g)
    dev = lambda v: torch.tensor(v, dtype=torch.int32).cuda()  # noqa: E731
    # prompts
    rows = sum(lens)
    row_seq = [b for b, n in enumerate(lens) for _ in range(n)]
    row_pos = [i for n in lens for i in range(n)]
    row0 = [sum(lens[:b]) for b in range(len(lens))]
    q = torch.randn((rows, heads, kw), generator=g).to(torch.bfloat16)
    ctx = SimpleNamespace(row_pos=dev(row_pos), row_seq=dev(row_seq), seq_slot=dev([0, 1, 2, 3]),
                          seq_start=dev([0] * 4), seq_row0=dev(row0), n_seqs=4)
    out = torch.empty((rows, heads * kw), dtype=torch.bfloat16, device="cuda")
    native.attention_latent(q.reshape(rows, -1).cuda(), torch.cat(keys_of).cuda(), None, None, 16, 0, ctx, out,
                            None, sink.cuda(), heads, kw, scale, window, 1, rows_per_tile=max(1, 16 // heads))
    ref = _latent_reference(q, keys_of, row_seq, row_pos, sink, scale, window)
    err = (out.cpu().double().view(rows, heads, kw) - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item(), f"prompts: {err:.3e} of {ref.abs().max().item():.3e}"
    # single rows over the cache: sequence b's position j lies in page table[b][j // 16], cell j % 16
    page_tokens, max_pages = 16, 10
    order = torch.randperm(4 * max_pages, generator=g).view(4, max_pages)
    pool = torch.zeros((4 * max_pages, 1, page_tokens, kw), dtype=torch.bfloat16)
    for b, c in enumerate(keys_of):
        for j in range(c.shape[0]):
            pool[order[b, j // page_tokens], 0, j % page_tokens] = c[j]
    last = [n - 1 for n in lens]
    q1 = torch.randn((4, heads, kw), generator=g).to(torch.bfloat16)
    ctx = SimpleNamespace(row_pos=dev(last), row_seq=dev([0, 1, 2, 3]), seq_slot=dev([0, 1, 2, 3]),
                          seq_start=dev(last), seq_row0=dev([0, 1, 2, 3]), n_seqs=4)
    ref = _latent_reference(q1, keys_of, [0, 1, 2, 3], last, sink, scale, window)
    for splits in (1, 3, 7):
        out = torch.empty((4, heads * kw), dtype=torch.bfloat16, device="cuda")
        scratch = torch.empty(native.attention_rows_scratch_bytes(4, heads, kw, splits) + 16, dtype=torch.uint8,
                              device="cuda") if splits > 1 else None
        native.attention_latent(q1.reshape(4, -1).cuda(), None, pool.cuda(), order.to(torch.int32).cuda(),
                                page_tokens, 0, ctx, out, scratch, sink.cuda(), heads, kw, scale, window, splits)
        err = (out.cpu().double().view(4, heads, kw) - ref).abs().max().item()
        assert err <= 2e-2 * ref.abs().max().item(), f"cache, {splits} runs: {err:.3e}"


@pytest.mark.parametrize("heads, hd, window, lens", [(4, 64, 0, [200, 5, 64, 131, 300]), (5, 128, 90, [390, 130]),
                                                     (16, 256, 700, [1100, 70]), (2, 128, 0, [2000])])
def test_tcgen05_prompt_kernel_with_sinks(heads, hd, window, lens):
    """The prompt kernel with one sink per head (a term of the denominator with no key and no
    value) against a 64-bit softmax: as a grid, as a balanced list of work, and with long blocks
    split in two.  Scores are spread widely, so single keys carry a row; some sinks are far
    above the scores, some far below."""
    from strata_inference_b200.kernels import native
    g = torch.Generator().manual_seed(heads + hd)
    scale = 3.0 / math.sqrt(hd)
    sink = torch.randn(heads, generator=g) * 3.0 + 2.0
    rows, refs = [], []
    for T in lens:
        q, k, v = (torch.randn((T, heads, hd), generator=g).to(torch.bfloat16) for _ in range(3))
        s = torch.einsum("thd,jhd->htj", q.double(), k.double()) * scale
        pos = torch.arange(T)
        hidden = (pos[None, :] > pos[:, None]) | ((pos[:, None] - pos[None, :] >= window) if window else False)
        s = s.masked_fill(hidden[None], float("-inf"))
        top = torch.maximum(s.amax(-1), sink.double()[:, None])
        e = torch.exp(s - top[..., None])
        w = e / (e.sum(-1) + torch.exp(sink.double()[:, None] - top))[..., None]
        refs.append(torch.einsum("htj,jhd->thd", w, v.double()))
        rows.append(torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1))
    packed = torch.cat(rows).contiguous().cuda()
    row0 = [sum(lens[:i]) for i in range(len(lens))]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")  # noqa: E731
    ref = torch.cat(refs).reshape(sum(lens), -1)

    def run(scratch, tickets, host_lens):
        out = torch.full((sum(lens), heads * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
        native.attention_prefill_tc(packed, out, i32(row0), i32(lens), len(lens), max(lens), heads, heads, hd,
                                    scale, 0.0, window, scratch, tickets, host_lens, sink=sink.cuda())
        assert native.attention_prefill_tc_error() == 0
        err = (out.cpu().double() - ref).abs().max().item()
        assert err <= 2e-2 * ref.abs().max().item(), f"{err:.3e} of {ref.abs().max().item():.3e}"
    run(None, None, None)
    need, n_tickets = native.attention_prefill_tc_split(len(lens), max(lens), heads, heads, hd)
    if need:
        run(torch.empty(need, dtype=torch.uint8, device="cuda"), torch.zeros(n_tickets, dtype=torch.int32, device="cuda"), None)
    n_items, need, n_tickets = native.attention_prefill_tc_plan(lens, heads, heads, hd, window)
    if n_items:
        run(torch.empty(max(need, 16), dtype=torch.uint8, device="cuda"),
            torch.zeros(max(n_tickets, 1), dtype=torch.int32, device="cuda"), lens)


@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_long_prompts_through_keys_and_values_per_head_and_through_the_latent_agree(name):
    """bfloat16 prompts of more than 128 tokens make keys and values per head for the tcgen05
    prompt kernel; with that switched off they attend over the latent rows as single tokens do.
    Both agree with the plain model, and with each other more closely than either must."""
    from strata_inference_b200.parts import attention
    cfg = {"mixed": MIXED, "wide": WIDE}[name]
    w = random_weights(cfg, seed=41)
    a, b = prompts(cfg, [300, 190], seed=42)
    ref = torch.cat([plain_logits(cfg, w, a), plain_logits(cfg, w, b)])
    got = {}
    for expand in (True, False):
        attention._USE_LATENT_EXPAND = expand
        try:
            eng = make_engine(cfg, w, "bfloat16")
            sa, sb = eng.new_sequence(), eng.new_sequence()
            got[expand] = eng.step([(sa, a), (sb, b)], [all_rows(300), all_rows(190)]).cpu().double()
        finally:
            attention._USE_LATENT_EXPAND = True
        assert_close(got[expand], ref, "bfloat16", f"{name}, keys per head: {expand}")
    diff = (got[True] - got[False]).abs().amax(-1) / ref.abs().max()
    assert diff.median().item() <= 1.5e-2 and (diff > 4e-2).float().mean().item() <= 0.1, \
        f"median {diff.median().item():.3e}, worst {diff.max().item():.3e}"
