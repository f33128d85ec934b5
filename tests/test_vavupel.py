"""Vavupel without a device: the configuration and its schedule, the tensor table, and the plain
model's mechanisms against closed forms of their own."""

from __future__ import annotations

import copy

import numpy as np
import pytest

import plain_vavupel as plain
from vavupel_cases import ALONE, MIXED, ODD, STRAIGHT, latent, model, random_weights, retention

from strata_inference_b200.config.registry import spec_from_config
from strata_inference_b200.config.spec import ConfigError
from strata_inference_b200.engine.model import expected_tensors


def test_loop_becomes_a_schedule_with_a_pass_mark():
    typed, spec = spec_from_config(MIXED)
    assert typed.loop == (1, 4, 3)
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 3, 1, 2, 3, 1, 2, 3, 4]
    assert [i for i, e in enumerate(spec.schedule) if e.begins_pass] == [1, 4, 7]
    assert [(i, b) for i, b in plain.layer_runs(MIXED)] == [(e.layer, e.begins_pass) for e in spec.schedule]
    _, straight = spec_from_config(STRAIGHT)
    assert straight.pass_mix is None and not any(e.begins_pass for e in straight.schedule)
    _, odd = spec_from_config(ODD)
    assert [e.layer for e in odd.schedule] == [0, 1, 0, 1, 2, 3] and odd.schedule[0].begins_pass


def test_every_size_and_constant_comes_from_the_configuration():
    _, spec = spec_from_config(MIXED)
    la = spec.layers[3].mixer
    assert la.kind == "latent_attention" and la["window"] == 100 and la["kv_rank"] == 48
    assert la["position"].kind == "rope_interleaved" and la["position"]["rotary_dim"] == 8
    re = spec.layers[0].mixer
    assert re.kind == "retention" and tuple(re["decay"]) == (0.9, 0.97, 0.99, 0.999)
    assert re["key_scale"] == 16 ** -0.5 and re["position"].kind == "rope_neox"
    assert spec.layers[2].feed_forward is None and spec.layers[0].feed_forward["intermediate_size"] == 96
    assert spec.embedding["buckets"] == 61 and spec.head["logit_softcap"] == 20.0
    _, bare = spec_from_config(ALONE["latent_open"])
    assert bare.layers[0].mixer["window"] == 0 and bare.head["logit_softcap"] == 0.0


def test_tensor_table_matches_the_random_weights_and_tolerates_unused_norms():
    for cfg in list(ALONE.values()) + [MIXED, ODD]:
        _, spec = spec_from_config(cfg)
        exp = expected_tensors(spec)
        w = random_weights(cfg, seed=1)
        assert {n for n, d in exp.items() if not d.optional} == set(w)
        for n, t in w.items():
            assert tuple(exp[n].shape) == tuple(t.shape), n
    _, spec = spec_from_config(MIXED)
    assert expected_tensors(spec)["l2.norm2b.alpha"].optional     # (layer 2 has no feed-forward)


@pytest.mark.parametrize("edit, text", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.9]), "decay"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "dims"),
    (lambda c: c.update(loop={"start": 2, "stop": 9, "times": 2}), "loop"),
    (lambda c: c["embedding"].pop("bigram"), "bigram"),
    (lambda c: c.pop("width"), "width"),
])
def test_configuration_errors_name_the_key(edit, text):
    cfg = copy.deepcopy(MIXED)
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        spec_from_config(cfg)
    assert text in str(e.value)


def test_plain_retention_is_the_decayed_sum_over_the_past():
    """o_t = sum_{s <= t} decay^(t - s) <q_t, k_s> v_s, then the unit norm and the gate."""
    rng = np.random.default_rng(0)
    n, W, H, d, vd = 12, 16, 2, 4, 6
    m = {"heads": H, "dim": d, "vdim": vd, "decay": [0.9, 0.5], "rot": {"dims": 4, "base": 100.0}}
    w = {k: rng.normal(size=s) for k, s in (("q", (H * d, W)), ("k", (H * d, W)), ("v", (H * vd, W)),
                                             ("g", (H * vd, W)), ("o", (W, H * vd)))}
    h = rng.normal(size=(n, W))
    pos = np.arange(n)
    q = plain.rotate((h @ w["q"].T).reshape(n, H, d), pos, 4, 100.0, False)
    k = plain.rotate((h @ w["k"].T).reshape(n, H, d), pos, 4, 100.0, False) / 2.0
    v = (h @ w["v"].T).reshape(n, H, vd)
    o = np.zeros((n, H, vd))
    for a in range(H):
        for t in range(n):
            for s in range(t + 1):
                o[t, a] += m["decay"][a] ** (t - s) * (q[t, a] @ k[s, a]) * v[s, a]
    z = h @ w["g"].T
    ref = (plain.unit_rms(o, 1e-5).reshape(n, -1) * z / (1 + np.exp(-z))) @ w["o"].T
    assert np.allclose(plain.retention(h, w, m, 1e-5), ref, atol=1e-10)


def test_plain_rotations_keep_lengths_and_relative_angles():
    rng = np.random.default_rng(1)
    x = rng.normal(size=(5, 2, 8))
    for inter in (False, True):
        y = plain.rotate(x, [3, 4, 5, 6, 7], 6, 50.0, inter)
        assert np.allclose((y ** 2).sum(-1), (x ** 2).sum(-1))
        assert np.array_equal(y[..., 6:], x[..., 6:])
        # the product of two rotated vectors depends on the distance of their positions only
        a, b = rng.normal(size=(1, 1, 8)), rng.normal(size=(1, 1, 8))
        one = (plain.rotate(a, [9], 6, 50.0, inter) * plain.rotate(b, [4], 6, 50.0, inter)).sum()
        two = (plain.rotate(a, [105], 6, 50.0, inter) * plain.rotate(b, [100], 6, 50.0, inter)).sum()
        assert abs(one - two) < 1e-9
    pair = plain.rotate(np.array([[[1.0, 0.0, 0.0, 0.0]]]), [1], 4, 10.0, True)[0, 0]
    assert np.allclose(pair, [np.cos(1.0), np.sin(1.0), 0, 0])
    split = plain.rotate(np.array([[[1.0, 0.0, 0.0, 0.0]]]), [1], 4, 10.0, False)[0, 0]
    assert np.allclose(split, [np.cos(1.0), 0, np.sin(1.0), 0])


def test_plain_sink_takes_weight_and_window_hides_old_keys():
    cfg = model(32, 50, [latent(2, 8, 4, 8, 12, 5)], cap=0)
    w = {n: plain.f64(t) for n, t in random_weights(cfg, seed=3).items()}
    toks = list(range(20))
    base = plain.forward(toks, w, cfg)
    early = plain.forward([7] + toks[1:], w, cfg)
    # rows whose window (5) and bigram no longer reach the first token do not change with it
    assert np.allclose(base[6:], early[6:]) and not np.allclose(base[:5], early[:5])
    heavy = dict(w)
    heavy["l0.mix.sink"] = w["l0.mix.sink"] + 50.0       # all weight on the sink: the mixer gives (nearly) nothing
    h = np.random.default_rng(2).normal(size=(6, 32))
    mix = {k[len("l0.mix."):]: v for k, v in heavy.items() if k.startswith("l0.mix.")}
    assert np.abs(plain.latent_attention(h, mix, cfg["layers"][0]["mixer"], 1e-5)).max() < 1e-12


def test_plain_bigram_rows():
    table, big = np.eye(5), np.arange(4 * 5, dtype=float).reshape(4, 5)
    out = plain.bigram_embedding([2, 4, 4], table, big, 2.0, 3, 2, 5)
    assert np.allclose(out[0], 2 * table[2] + big[3])
    assert np.allclose(out[1], 2 * table[4] + big[(2 * 2 + 4 * 5) % 3])
    assert np.allclose(out[2], 2 * table[4] + big[(4 * 2 + 4 * 5) % 3])
