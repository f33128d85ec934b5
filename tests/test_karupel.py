"""Karupel without a device: the configuration, the tensor table, and the plain model's own
consistency (a prompt in one piece, in portions and token by token gives the same rows)."""

from __future__ import annotations

import copy

import pytest
import torch

import plain_karupel as plain
from karupel_cases import ALONE, BROAD, MIXED, NARROW, ODD, WIDE, attention, delta, mlstm, model, prompts
from strata_inference_b200.config.registry import spec_from_config
from strata_inference_b200.config.spec import ConfigError
from strata_inference_b200.engine.model import expected_tensors, resident_plan


@pytest.mark.parametrize("cfg", [MIXED, ODD, WIDE, BROAD, NARROW] + [ALONE[k] for k in sorted(ALONE)])
def test_tensor_table_is_the_design_s(cfg):
    """The names and shapes the loader expects are the ones the plain model reads."""
    _, spec = spec_from_config(cfg)
    want = plain.random_weights(cfg, seed=1)
    have = expected_tensors(spec)
    needed = {n for n, d in have.items() if not d.optional}
    assert needed <= set(want) and set(want) <= set(have)
    for n, t in want.items():
        assert tuple(have[n].shape) == tuple(t.shape), n
    resident_plan(spec)


def test_spec_layout():
    typed, spec = spec_from_config(MIXED)
    assert spec.architecture == "Karupel" and spec.hidden_size == 64 and spec.vocab_size == 200
    kinds = [l.mixer.kind for l in spec.layers]
    assert kinds == ["attention", "gated_delta", "attention", "matrix_memory", "attention", "attention",
                     "gated_delta", "attention"]
    mix = [l.mixer.params.get("value_mix") for l in spec.layers if l.mixer.kind == "attention"]
    assert mix == [None, "first", None, "mix", "mix"]
    assert [l.feed_forward is not None for l in spec.layers] == [True, False, False, True, False, True, True, False]
    a = spec.layers[4].mixer.params
    assert a["position"].params == {"theta": 50.0, "rotary_dim": 8, "scaling_factor": 1.5}
    assert spec.layers[7].mixer.params["position"].kind == "none"
    assert all(l.norms["pre_mixer"].kind == "identity" for l in spec.layers)
    assert typed.layers[1].mixer["conv"] == 3


@pytest.mark.parametrize("change, message", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["layers"][0].update(type="window"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=34), "dims"),
    (lambda c: c["layers"][1]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][3]["mixer"].update(gate_cap=0), "gate_cap"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "kind"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_config_errors_name_the_key(change, message):
    cfg = copy.deepcopy(MIXED)
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        spec_from_config(cfg)


@pytest.mark.parametrize("cfg", [MIXED, ODD])
def test_plain_model_in_portions(cfg):
    """The plain model's state handling: one piece, portions and single tokens agree."""
    w = plain.random_weights(cfg, seed=2)
    m = plain.Plain(cfg, w)
    toks = prompts(cfg, [40], seed=3)[0]
    whole = m.run(toks)
    for sizes in ([1] * 40, [2, 3, 1, 30, 4], [39, 1]):
        state, rows, at = m.new_state(), [], 0
        for n in sizes:
            rows.append(m.run(toks[at:at + n], state))
            at += n
        assert torch.allclose(torch.cat(rows), whole, rtol=0, atol=1e-9 * whole.abs().max().item())


def test_plain_mechanisms_by_hand():
    """Each plain function on a case small enough to work out by hand."""
    # short convolution: taps (1, 2, 3) on inputs 1, 1, 1, 1 -> 3, 5, 6, 6; history carries over
    st = {}
    x = torch.ones((2, 1), dtype=torch.float64)
    w = torch.tensor([[1.0, 2.0, 3.0]], dtype=torch.float64)
    y = torch.cat([plain.short_conv(x, w, st, "c"), plain.short_conv(x, w, st, "c")])
    assert y.flatten().tolist() == [3.0, 5.0, 6.0, 6.0]
    # rotation by a quarter turn of the pair (dimension 0, dimension 1) at position 1
    import math
    q = torch.tensor([[[1.0, 0.0, 5.0]]], dtype=torch.float64)
    r = plain.rotate(q, torch.tensor([1]), {"dims": 2, "base": 7.0, "scaling": {"factor": 2.0 / math.pi}})
    assert torch.allclose(r, torch.tensor([[[0.0, 1.0, 5.0]]], dtype=torch.float64), atol=1e-12)
    # root mean square
    assert torch.allclose(plain.rms_unit(torch.tensor([3.0, 4.0], dtype=torch.float64), 0.0),
                          torch.tensor([3.0, 4.0], dtype=torch.float64) / math.sqrt(12.5))


def test_value_mixing_needs_an_earlier_layer_only_from_the_second_on():
    cfg = model(32, 50, [attention(2, 1, 16, 16, v_mix=True), mlstm(1, 16, 16), delta(2, 1, 16, 16, 2)])
    _, spec = spec_from_config(cfg)
    assert spec.layers[0].mixer.params["value_mix"] == "first"
    assert expected_tensors(spec)["l0.mix.vmix"].optional
