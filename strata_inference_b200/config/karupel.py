"""Karupel: the typed configuration and its translation into a ModelSpec.

A Karupel model is a list of layers, each with one of three mixers and, optionally, a
dense gated feed-forward; config.json writes every layer out:

    {"architecture": "Karupel", "vocab": V, "width": W, "norm": {"eps": e},
     "layers": [{"type": "delta" | "attention" | "mlstm", "mixer": {...}, "mlp": {...} | null}]}

What the design fixes and config.json has no key for is stated once in
:func:`karupel_spec`: a sub-layer reads the residual stream itself and is normed on its way
out only (x <- x + norm(sublayer(x)), RMS norm with a ``1 + w`` weight); the feed-forward
is SiLU-gated; attention has biases on q, k and v, an RMS norm with a weight on q and k,
half-split rotary pairs on the first ``rot.dims`` dimensions with linearly stretched
positions, one sigmoid gate per head, and (``v_mix``) values mixed with those of the first
such layer; the logits come from the embedding table.  Tensor names: ``embed``,
``final.norm``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, require

_TYPES = ("delta", "attention", "mlstm")
# positions a sequence may reach where config.json sets no bound ("max_positions")
_DEFAULT_POSITIONS = 1 << 20


def _positive(d: Mapping[str, Any], key: str, where: str) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}.'{key}' must be a positive integer, got {v!r}")
    return v


def _number(d: Mapping[str, Any], key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}.'{key}' must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class KarupelLayer:
    type: str
    mixer: Mapping[str, Any]       # checked sizes and constants of the mixer
    ff: int                        # 0: no feed-forward


@dataclass(frozen=True)
class KarupelConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[KarupelLayer, ...]
    max_positions: int
    raw: Mapping[str, Any]

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "KarupelConfig":
        vocab, width = require(d, "vocab", int), require(d, "width", int)
        if vocab <= 0 or width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        norm = require(d, "norm")
        eps = _number(norm, "eps", "norm")
        if eps <= 0:
            raise ConfigError("config.json: norm.'eps' must be positive")
        listed = require(d, "layers")
        if not isinstance(listed, (list, tuple)) or not listed:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, l in enumerate(listed):
            where = f"layers[{i}]"
            kind = l.get("type")
            if kind not in _TYPES:
                raise ConfigError(f"config.json: {where}.'type' = {kind!r} is not one of "
                                  f"{', '.join(_TYPES)}")
            m = l.get("mixer")
            if not isinstance(m, Mapping):
                raise ConfigError(f"config.json: {where}.'mixer' is missing")
            mw = where + ".mixer"
            mixer = {"heads": _positive(m, "heads", mw), "dim": _positive(m, "dim", mw),
                     "vdim": _positive(m, "vdim", mw)}
            if kind in ("delta", "attention"):
                mixer["kv_heads"] = _positive(m, "kv_heads", mw) if m.get("kv_heads") is not None \
                    else mixer["heads"]
                if mixer["heads"] % mixer["kv_heads"]:
                    raise ConfigError(f"config.json: {mw}: {mixer['heads']} heads cannot share "
                                      f"{mixer['kv_heads']} kv_heads")
            if kind == "delta":
                mixer["conv"] = _positive(m, "conv", mw)
            elif kind == "mlstm":
                mixer["gate_cap"] = _number(m, "gate_cap", mw)
                if mixer["gate_cap"] <= 0:
                    raise ConfigError(f"config.json: {mw}.'gate_cap' must be positive")
            else:
                mixer["scale"] = _number(m, "scale", mw)
                if mixer["scale"] <= 0:
                    raise ConfigError(f"config.json: {mw}.'scale' must be positive")
                mixer["v_mix"] = bool(m.get("v_mix"))
                rot = m.get("rot")
                if rot:
                    dims = _positive(rot, "dims", mw + ".rot")
                    if dims % 2 or dims > mixer["dim"]:
                        raise ConfigError(f"config.json: {mw}.rot.'dims' = {dims} must be even and "
                                          f"at most 'dim' ({mixer['dim']})")
                    base = _number(rot, "base", mw + ".rot")
                    factor = 1.0
                    if rot.get("scaling"):
                        factor = _number(rot["scaling"], "factor", mw + ".rot.scaling")
                    if base <= 0 or factor <= 0:
                        raise ConfigError(f"config.json: {mw}.rot: 'base' and the scaling 'factor' "
                                          f"must be positive")
                    mixer["rot"] = {"dims": dims, "base": base, "factor": factor}
                else:
                    mixer["rot"] = None
            ff = 0
            mlp = l.get("mlp")
            if mlp:
                if mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.'kind' = {mlp.get('kind')!r} is not "
                                      f"supported; known: dense")
                ff = _positive(mlp, "ff", where + ".mlp")
            layers.append(KarupelLayer(kind, mixer, ff))
        shapes = {(l.mixer["kv_heads"], l.mixer["vdim"]) for l in layers
                  if l.type == "attention" and l.mixer["v_mix"]}
        if len(shapes) > 1:
            raise ConfigError("config.json: layers with 'v_mix' mix values of one shape, but their "
                              f"(kv_heads, vdim) are {sorted(shapes)}")
        most = d.get("max_positions")
        return cls(vocab=vocab, width=width, eps=eps, layers=tuple(layers),
                   max_positions=_DEFAULT_POSITIONS if most is None else _positive(d, "max_positions", ""),
                   raw=dict(d))

    def to_dict(self) -> dict:
        return dict(self.raw)


def _names(**table: str) -> Mapping[str, str]:
    return dict(table)


_DELTA_NAMES = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v",
                "q_conv.weight": "q.conv", "k_conv.weight": "k.conv", "v_conv.weight": "v.conv",
                "b_proj.weight": "b", "a_proj.weight": "a", "A_log": "A_log", "dt_bias": "dt_bias",
                "norm.weight": "norm", "g_proj.weight": "g", "o_proj.weight": "o"}
_ATTENTION_NAMES = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v",
                    "q_proj.bias": "q.b", "k_proj.bias": "k.b", "v_proj.bias": "v.b",
                    "q_norm.weight": "q.norm", "k_norm.weight": "k.norm",
                    "value_mix.weight": "vmix", "g_proj.weight": "g", "o_proj.weight": "o"}
_MEMORY_NAMES = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v",
                 "g_proj.weight": "g", "i_proj.weight": "i", "i_proj.bias": "i.b",
                 "f_proj.weight": "f", "f_proj.bias": "f.b", "norm.weight": "norm",
                 "o_proj.weight": "o"}
_MLP_NAMES = {"gate_proj.weight": "gate", "up_proj.weight": "up", "down_proj.weight": "down"}
_WHOLE = {"weight": ""}      # a norm's or the embedding's only tensor carries the site's name


def karupel_spec(cfg: KarupelConfig) -> ModelSpec:
    """Lay the configuration out as parts, layer by layer."""
    norm = PartSpec("rms_norm", {"eps": cfg.eps, "unit_offset": True})
    passes = PartSpec("identity", {})
    mixing = [i for i, l in enumerate(cfg.layers) if l.type == "attention" and l.mixer["v_mix"]]
    layers = []
    for i, l in enumerate(cfg.layers):
        m = l.mixer
        if l.type == "delta":
            mixer = PartSpec("gated_delta", {
                "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                "value_dim": m["vdim"], "conv_taps": m["conv"], "norm_eps": cfg.eps})
            names = _DELTA_NAMES
        elif l.type == "mlstm":
            mixer = PartSpec("matrix_memory", {
                "num_heads": m["heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
                "gate_cap": m["gate_cap"], "norm_eps": cfg.eps})
            names = _MEMORY_NAMES
        else:
            rot = m["rot"]
            position = PartSpec("rope_neox", {"theta": rot["base"], "rotary_dim": rot["dims"],
                                              "scaling_factor": rot["factor"]}) if rot \
                else PartSpec("none", {})
            mixer = PartSpec("attention", {
                "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                "value_dim": m["vdim"], "score_scale": m["scale"], "logit_softcap": 0.0,
                "window": 0, "position": position, "bias": True, "qk_norm": {"eps": cfg.eps},
                "value_mix": None if not m["v_mix"] else ("first" if i == mixing[0] else "mix"),
                "head_gate": True})
            names = _ATTENTION_NAMES
        ffn: Optional[PartSpec] = None
        norms = {"pre_mixer": passes, "post_mixer": norm}
        if l.ff:
            ffn = PartSpec("gated_mlp", {"intermediate_size": l.ff, "activation": "silu"})
            norms.update({"pre_feed_forward": passes, "post_feed_forward": norm})
        layers.append(LayerSpec(
            prefix=f"l{i}.", block="sandwich", mixer=mixer, feed_forward=ffn, norms=norms,
            names={"mixer": "mix.", "feed_forward": "mlp.", "pre_mixer": "", "post_mixer": "norm1",
                   "pre_feed_forward": "", "post_feed_forward": "norm2"},
            tensor_names={"mixer": names, "feed_forward": _MLP_NAMES, "post_mixer": _WHOLE,
                          "post_feed_forward": _WHOLE}))
    spec = ModelSpec(
        architecture="Karupel", hidden_size=cfg.width, vocab_size=cfg.vocab,
        max_positions=cfg.max_positions,
        embedding=PartSpec("token_embedding", {"scale": 1.0}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=norm,
        head=PartSpec("lm_head", {"tied": True, "logit_softcap": 0.0}),
        names={"embedding": "embed", "final_norm": "final.norm", "head": "head."},
        tensor_names={"embedding": _WHOLE, "final_norm": _WHOLE},
        stop_tokens=())
    spec.validate()
    return spec
