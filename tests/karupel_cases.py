"""Small Karupel configurations for the tests, and the comparison with the plain model."""

from __future__ import annotations

from typing import Dict, List, Sequence

import torch

import plain_karupel as plain


def attention(heads, kv, dim, vdim, scale=0.2, rot=None, v_mix=False, ff=0):
    mixer = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix}
    if rot is not None:
        mixer["rot"] = rot
    return {"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def delta(heads, kv, dim, vdim, conv, ff=0):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def mlstm(heads, dim, vdim, cap=10.0, ff=0):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def model(width, vocab, layers, eps=1e-5):
    return {"architecture": "Karupel", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": list(layers)}


ROT_HALF = {"base": 10000.0, "dims": 16, "scaling": {"factor": 2.0}}
ROT_FULL = {"base": 777.0, "dims": 24}        # every dimension rotated, no scaling

# one layer of each mixer alone, with and without a feed-forward
ALONE = {
    "delta": model(64, 200, [delta(4, 2, 16, 24, 3)]),
    "delta_ff": model(64, 200, [delta(2, 2, 32, 16, 4, ff=96)]),
    "attention": model(64, 200, [attention(4, 2, 32, 16, rot=ROT_HALF)]),
    "attention_ff": model(64, 200, [attention(2, 1, 16, 48, rot=None, ff=80)]),
    "mlstm": model(64, 200, [mlstm(2, 16, 32)]),
    "mlstm_ff": model(64, 200, [mlstm(4, 32, 16, cap=4.0, ff=72)]),
}

# every mixer, grouped heads everywhere, key and value widths that differ, a mixing layer that is not
# the first attention layer, an attention layer between the mixing ones that does not mix
MIXED = model(64, 200, [
    attention(4, 2, 32, 16, rot=ROT_HALF, ff=96),
    delta(4, 2, 16, 24, 3),
    attention(4, 2, 32, 16, rot=ROT_HALF, v_mix=True),
    mlstm(2, 16, 32, ff=64),
    attention(2, 1, 16, 16, scale=0.3, rot={"base": 50.0, "dims": 8, "scaling": {"factor": 1.5}}),
    attention(4, 2, 16, 16, rot=ROT_HALF, v_mix=True, ff=64),
    delta(2, 2, 32, 16, 2, ff=48),
    attention(4, 2, 48, 16, scale=0.15, v_mix=True),
])

# sizes that are no multiples of 16 (or of 8), one head, one tap, one mixing layer only
ODD = model(72, 131, [
    attention(3, 1, 24, 40, rot=ROT_FULL, v_mix=True, ff=100),
    delta(2, 1, 40, 8, 5),
    mlstm(1, 48, 20, cap=30.0),
    delta(3, 3, 8, 12, 1, ff=36),
    attention(1, 1, 8, 8, scale=0.5),
], eps=1e-6)

# head widths that the tensor-core attention kernels and the widest recurrences take
WIDE = model(128, 300, [
    attention(4, 2, 64, 64, scale=0.125, rot={"base": 500000.0, "dims": 32, "scaling": {"factor": 8.0}},
              v_mix=True, ff=128),
    delta(2, 1, 128, 64, 4),
    mlstm(2, 64, 128),
    attention(4, 2, 128, 64, scale=0.09, rot={"base": 10000.0, "dims": 128}, v_mix=True),
    delta(1, 1, 256, 32, 4),
])

# a width, heads and a vocabulary that are multiples of 2 only
NARROW = model(100, 77, [
    delta(2, 1, 12, 10, 3),
    attention(2, 2, 12, 20, scale=0.3, rot={"base": 100.0, "dims": 6, "scaling": {"factor": 3.0}}, v_mix=True),
    mlstm(2, 10, 6, cap=6.0, ff=30),
    attention(2, 2, 18, 20, scale=0.25, v_mix=True, ff=26),
])

# recurrent matrices with more than 256 rows, heads of attention wider than 256
BROAD = model(96, 150, [
    delta(1, 1, 320, 16, 2),
    mlstm(1, 264, 8),
    attention(2, 1, 272, 24, scale=0.05, rot={"base": 1000.0, "dims": 100}, ff=40),
])

# attention alone with a scale that makes the softmax pick a few keys among hundreds
SHARP = model(64, 200, [
    attention(4, 2, 32, 16, scale=1.0, rot=ROT_HALF, v_mix=True),
    attention(4, 2, 32, 16, scale=1.0, rot=ROT_HALF, v_mix=True, ff=64),
])

# Largest |engine - plain| of a row as a fraction of the largest plain logit of the compared rows.
# 32-bit: every row.  bfloat16: a head's output is divided by its root mean square, and the matrix
# memory's by |n . q|, so a row in which one of these nearly cancels turns the rounding of its inputs
# (2^-9) into an error of any size, even a flipped sign, and a recurrent state hands the error on
# to the rows behind it; such rows lie anywhere (in 32-bit the same rows show as 3e-5 instead of
# 3e-6).  The bfloat16 runs therefore bound the typical row tightly, the number of rows above the
# tolerance and every row loosely: a wrong path, scale or state shows in most rows.  What a wrong
# key, cell or state does to a single row is the 32-bit runs' business, which take the same kernels'
# other instantiation.
REL_TOL = {"float32": 1e-4, "bfloat16": 4e-2}
BF16_MEDIAN, BF16_ROWS_OVER, BF16_WORST = 2.5e-2, 0.3, 0.9


def prompts(cfg: dict, lengths: Sequence[int], seed: int) -> List[List[int]]:
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lengths]


def plain_logits(cfg: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    return plain.Plain(cfg, weights).run(tokens)


def assert_close(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str) -> None:
    """Rows of logits against the plain model's: the largest difference as a fraction of the
    largest plain logit of the compared rows."""
    got = got.detach().to("cpu", torch.float64)
    ref = ref.to(torch.float64)
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    scale = ref.abs().max().item()
    diff = (got - ref).abs().amax(dim=-1)
    bad = (diff > REL_TOL[dtype] * scale).nonzero()
    text = (f"{what}: max |diff| {diff.max().item():.3e}, median {diff.median().item():.3e}, "
            f"{bad.numel()} of {got.shape[0]} rows over {REL_TOL[dtype]:.0e} x max|ref| {scale:.3e}"
            + (f"; first of them row {int(bad[0])}" if bad.numel() else ""))
    if dtype == "float32":
        assert bad.numel() == 0, text
    elif got.shape[0] < 8:
        assert diff.max().item() <= BF16_WORST * scale, text
    else:
        assert diff.median().item() <= BF16_MEDIAN * scale, text
        assert bad.numel() <= max(1, BF16_ROWS_OVER * got.shape[0]), text
        assert diff.max().item() <= BF16_WORST * scale, text
