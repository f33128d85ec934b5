"""Small Vavupel configurations for the tests, random weights for them, and the comparison with
the plain model (tests/plain_vavupel.py)."""

from __future__ import annotations

import math
from typing import Dict, List, Sequence

import numpy as np
import torch

import plain_vavupel as plain


def latent(heads, dim, rot_dim, vdim, rank, window, scale=0.2, rot_dims=None, base=10000.0, ff=0):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
             "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}
    if window:
        mixer["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def retention(heads, dim, vdim, decay, rot_dims=None, base=10000.0, ff=0):
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot_dims != 0:
        mixer["rot"] = {"base": base, "dims": dim if rot_dims is None else rot_dims}
    return {"type": "retention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def model(width, vocab, layers, loop=None, eps=1e-5, scale=0.7, buckets=61, mul_prev=13, mul_cur=5, cap=20.0):
    cfg = {"architecture": "Vavupel", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "embedding": {"scale": scale, "bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}},
           "layers": list(layers)}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    if cap:
        cfg["logit_softcap"] = cap
    return cfg


# one layer of each mixer alone, with and without a feed-forward, with and without a loop
ALONE = {
    "latent": model(64, 200, [latent(4, 16, 8, 24, 32, 40)]),
    "latent_ff": model(64, 200, [latent(2, 32, 16, 16, 48, 70, rot_dims=8, ff=96)], loop=(0, 1, 2)),
    "latent_open": model(64, 200, [latent(3, 16, 8, 16, 24, 0, ff=40)], cap=0),
    "retention": model(64, 200, [retention(4, 16, 24, [0.9, 0.97, 0.99, 0.999])]),
    "retention_ff": model(64, 200, [retention(2, 32, 16, [0.95, 0.995], rot_dims=16, ff=80)], loop=(0, 1, 3)),
    "retention_still": model(64, 200, [retention(2, 16, 16, [0.98, 1.0], rot_dims=0)]),
}

# both mixers, a loop in the middle that is walked three times, layers without a feed-forward, windows
# shorter and longer than a page of 64, rotated widths that differ from the rotated part's
MIXED = model(64, 200, [
    retention(4, 16, 24, [0.9, 0.97, 0.99, 0.999], ff=96),
    latent(4, 16, 8, 24, 32, 40, ff=64),
    retention(2, 32, 16, [0.96, 0.998], rot_dims=8),
    latent(2, 32, 16, 16, 48, 100, rot_dims=8, scale=0.15, ff=48),
    latent(3, 16, 8, 16, 40, 64),
], loop=(1, 4, 3))

# sizes that are no multiples of 16, 8 or 4; one head; a loop from the first layer; no cap
ODD = model(72, 131, [
    latent(3, 10, 6, 14, 21, 33, rot_dims=4, ff=100),
    retention(1, 20, 7, [0.99], rot_dims=10),
    latent(1, 7, 2, 5, 9, 5, scale=0.5),
    retention(3, 6, 9, [0.5, 0.9, 0.999], ff=36),
], loop=(0, 2, 2), eps=1e-6, buckets=7, mul_prev=1000003, mul_cur=999983, cap=0)

# a width and a vocabulary that are multiples of 2 only, the loop over the last layers, once
NARROW = model(100, 77, [
    retention(2, 12, 10, [0.9, 0.99], ff=30),
    latent(2, 12, 6, 20, 18, 50, ff=26),
    latent(2, 18, 4, 20, 30, 20),
], loop=(1, 3, 1), scale=1.0, buckets=300)

# wide heads: the widest recurrences and latent rows
WIDE = model(128, 300, [
    latent(4, 64, 32, 64, 192, 128, scale=0.09, base=500000.0, ff=128),
    retention(2, 128, 64, [0.99, 0.999]),
    latent(8, 128, 64, 128, 448, 200, scale=0.06),
    retention(1, 320, 16, [0.995], rot_dims=100),
], loop=(0, 2, 2))

# a latent row wider than 512 (the general attention kernel in both compute types)
BROAD = model(64, 100, [latent(2, 16, 32, 16, 560, 50, ff=32), retention(1, 16, 16, [0.99])])

# corners: a window of one (a row sees itself and the sink), a window longer than any request, 40 heads
# in chunks of 16, a latent of 8 with 2 rotated columns, values wider than keys, a loop of one layer walked
# four times, no feed-forward anywhere, a one-layer model whose only layer is looped
CORNERS = {
    "window_of_one": model(48, 90, [latent(2, 8, 4, 8, 12, 1), retention(2, 8, 3, [0.9, 0.99])], loop=(0, 2, 2)),
    "long_window": model(48, 90, [latent(5, 8, 4, 12, 16, 5000, ff=24)], cap=0),
    "many_heads": model(64, 90, [latent(40, 8, 8, 8, 24, 70), retention(20, 8, 8, [1.0 - 0.5 ** (i % 9 + 1) for i in range(20)])]),
    "tiny_latent": model(32, 50, [latent(7, 24, 2, 40, 8, 37, ff=20), latent(2, 4, 2, 4, 8, 9)], loop=(1, 2, 4)),
    "bare": model(40, 60, [retention(2, 8, 12, [0.97, 0.9]), latent(2, 8, 4, 8, 12, 20), retention(1, 16, 8, [0.999])],
                  loop=(0, 1, 3), scale=0.25, buckets=1, mul_prev=0, mul_cur=1),
}

# no loop at all
STRAIGHT = model(64, 150, [retention(2, 16, 16, [0.9, 0.99], ff=32), latent(2, 16, 8, 16, 24, 30, ff=32)])

# attention with a scale that makes the softmax pick a few keys among those inside the window
SHARP = model(64, 200, [
    latent(4, 16, 8, 24, 32, 150, scale=1.5),
    latent(4, 16, 8, 24, 32, 66, scale=1.5, ff=64),
])

REL_TOL = {"float32": 1e-4, "bfloat16": 4e-2}
# 32-bit: a row in which a retention head's output nearly cancels before it is divided by its root
# mean square shows the 32-bit rounding of its inputs enlarged (1e-4 where the typical row has 1e-5);
# one row in a hundred may lie above the tolerance, none above five times it.
F32_ROWS_OVER, F32_WORST = 0.01, 5.0
# bfloat16: a retention head's output is divided by its root mean square, so a row in which that
# nearly cancels turns the rounding of its inputs into an error of any size; the bfloat16 runs bound
# the typical row, the share of rows over the tolerance and every row loosely, the 32-bit runs (the
# same kernels' other instantiation) every row tightly.
BF16_MEDIAN, BF16_ROWS_OVER, BF16_WORST = 2.5e-2, 0.3, 0.9


def prompts(cfg: dict, lengths: Sequence[int], seed: int) -> List[List[int]]:
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lengths]


def random_weights(config: dict, seed: int, std: float = 0.5) -> Dict[str, torch.Tensor]:
    """Random tensors of every name the configuration asks for, rounded to bfloat16 values.
    (``std`` 0.5: a model of eleven layer runs passes a relative change of its weights on to its
    logits about 3-fold; with 0.8 it is 40- to 260-fold, and bfloat16 rounding alone moves the
    logits by a tenth of their size.)"""
    g = torch.Generator().manual_seed(seed)
    W = config["width"]

    def mat(o, i, s=1.0):
        return torch.randn((o, i), generator=g) * (s * std / math.sqrt(i))

    def vec(n, s=0.3, at=0.0):
        return torch.randn((n,), generator=g) * s + at

    out: Dict[str, torch.Tensor] = {}

    def norm(name):
        out[name], out[name + ".b"] = vec(W, 0.3, 1.0), vec(W, 0.1)
        out[name + ".alpha"] = (torch.rand((), generator=g) + 0.5)

    out["embed"] = torch.randn((config["vocab"], W), generator=g)
    out["bigram"] = torch.randn((config["embedding"]["bigram"]["buckets"] + 1, W), generator=g) * 0.7
    norm("embed.norm")
    if config.get("loop"):
        out["loop.in"] = mat(W, 2 * W, 1.5)
    for i, layer in enumerate(config["layers"]):
        m, pre = layer["mixer"], f"l{i}.mix."
        norm(f"l{i}.norm1")
        norm(f"l{i}.norm1b")
        H, D, V = m["heads"], m["dim"], m["vdim"]
        if layer["type"] == "retention":
            out[pre + "q"], out[pre + "k"] = mat(H * D, W, 2.0), mat(H * D, W, 2.0)
            out[pre + "v"], out[pre + "g"] = mat(H * V, W, 2.0), mat(H * V, W, 2.0)
            out[pre + "o"] = mat(W, H * V, 2.0)
        else:
            R, rank = m["rot_dim"], m["kv_rank"]
            out[pre + "q"], out[pre + "dkv"] = mat(H * (D + R), W, 2.0), mat(rank + R, W, 2.0)
            out[pre + "dkv.norm"] = vec(rank, 0.3, 1.0)
            out[pre + "uk"], out[pre + "uv"] = mat(H * D, rank, 2.0), mat(H * V, rank, 2.0)
            out[pre + "sink"] = vec(H, 1.0)
            out[pre + "g"], out[pre + "o"] = mat(H, W, 3.0), mat(W, H * V, 2.0)
        if layer.get("mlp"):
            F = layer["mlp"]["ff"]
            norm(f"l{i}.norm2")
            norm(f"l{i}.norm2b")
            out[f"l{i}.mlp.up"], out[f"l{i}.mlp.down"] = mat(F, W, 2.0), mat(W, F, 2.0)
    norm("final.norm")
    out["head"] = mat(config["vocab"], W, 3.0)
    return {n: t.to(torch.bfloat16).to(torch.float32) for n, t in out.items()}


def plain_logits(cfg: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    w = {n: plain.f64(t) for n, t in weights.items()}
    return torch.from_numpy(np.ascontiguousarray(plain.forward(list(tokens), w, cfg)))


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
        assert bad.numel() <= int(F32_ROWS_OVER * got.shape[0] + 0.99), text
        assert diff.max().item() <= F32_WORST * REL_TOL[dtype] * scale, text
    elif got.shape[0] < 8:
        assert diff.max().item() <= BF16_WORST * scale, text
    else:
        assert diff.median().item() <= BF16_MEDIAN * scale, text
        assert bad.numel() <= max(1, BF16_ROWS_OVER * got.shape[0]), text
        assert diff.max().item() <= BF16_WORST * scale, text


def rows_that_differ(a: torch.Tensor, b: torch.Tensor, factor: float = 100.0) -> int:
    """How many rows of two plain results differ by more than ``factor`` times the 32-bit
    tolerance: what a test needs to be able to tell the two apart."""
    scale = a.abs().max().item()
    return int(((a - b).abs().amax(dim=-1) > factor * REL_TOL["float32"] * scale).sum())
