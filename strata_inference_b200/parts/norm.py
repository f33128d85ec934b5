"""RMS norm: x * 1/sqrt(mean(x^2) + eps) * gain, statistics in 32-bit.

``unit_offset`` selects gain = 1 + weight (the convention of checkpoints
that store the weight as a deviation from one) instead of gain = weight
(the reference's convention, src/backend/cpu.rs:797-810, whose input files
already hold the effective gain).  The gain is formed once, in 32-bit, when
the weights are placed on the device.

``identity`` is the norm of a site that has none: the rows of the 32-bit stream as
activations, unchanged.  A layer whose sub-layers read the stream itself and are normed
on the way out only (x <- x + norm(sublayer(x))) names it at its two "pre" sites, so
that the block arrangements and their fused "norm, add, norm" step serve it as they are.

``dynamic_tanh`` is a norm without statistics: tanh(alpha x) * weight + b, element by
element in 32-bit, with one stored number ``alpha`` and one ``weight`` and ``b`` per
column.  Blocks fuse it into the residual add as they fuse the RMS norm (``fusable_dyt``,
csrc/norm.cu add_dyt_norm).
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..kernels import native
from ..weights.arena import Piece, Resident
from ..weights.loader import TensorDecl
from .registry import register_norm


class RMSNorm:
    fusable_rms = True

    @staticmethod
    def tensors(params: Mapping, hidden: int) -> Dict[str, TensorDecl]:
        return {"weight": TensorDecl((hidden,), init="norm")}

    @staticmethod
    def resident(params: Mapping, hidden: int) -> Dict[str, Resident]:
        return {"gain": Resident((hidden,), torch.float32, (Piece("weight"),),
                                 1.0 if params.get("unit_offset", False) else 0.0)}

    def __init__(self, params: Mapping, hidden: int, weights: Mapping[str, torch.Tensor], rt):
        self.eps = float(params["eps"])
        self.hidden = hidden
        self.rt = rt
        self.gain = weights["gain"]

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.hidden), dtype=out_dtype or self.rt.dtype, device=x.device)
        return native.rms_norm(x, self.gain, self.eps, out, rows)


class IdentityNorm:
    """No norm: rows pass as they are (in the activation type).  ``gain`` None with
    ``fusable_rms`` tells a block that the residual kernel writes the plain rows out."""

    fusable_rms = True
    gain = None
    eps = 0.0

    @staticmethod
    def tensors(params: Mapping, hidden: int) -> Dict[str, TensorDecl]:
        return {}

    @staticmethod
    def resident(params: Mapping, hidden: int) -> Dict[str, Resident]:
        return {}

    def __init__(self, params: Mapping, hidden: int, weights: Mapping[str, torch.Tensor], rt):
        self.hidden = hidden
        self.rt = rt

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        if rows is not None:
            raise ValueError("the identity norm takes whole steps, not chosen rows")
        out = torch.empty((x.shape[0], self.hidden), dtype=out_dtype or self.rt.dtype, device=x.device)
        return native.cast_rows(x, out)


class DynamicTanh:
    fusable_rms = False
    fusable_dyt = True

    @staticmethod
    def tensors(params: Mapping, hidden: int) -> Dict[str, TensorDecl]:
        return {"weight": TensorDecl((hidden,), init="norm"), "b": TensorDecl((hidden,), init="norm"),
                "alpha": TensorDecl((), init="norm")}

    @staticmethod
    def resident(params: Mapping, hidden: int) -> Dict[str, Resident]:
        return {"weight": Resident((hidden,), torch.float32, (Piece("weight"),)),
                "b": Resident((hidden,), torch.float32, (Piece("b"),)),
                "alpha": Resident((1,), torch.float32, (Piece("alpha"),))}

    def __init__(self, params: Mapping, hidden: int, weights: Mapping[str, torch.Tensor], rt):
        self.hidden = hidden
        self.rt = rt
        self.weight, self.b, self.alpha = weights["weight"], weights["b"], weights["alpha"]

    @property
    def triple(self):
        """(weight, b, alpha) as the fused residual kernel takes them."""
        return self.weight, self.b, self.alpha

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.hidden), dtype=out_dtype or self.rt.dtype, device=x.device)
        return native.dyt_norm(x, self.weight, self.b, self.alpha, out, rows)


register_norm("rms_norm", RMSNorm)
register_norm("dynamic_tanh", DynamicTanh)
register_norm("identity", IdentityNorm)
