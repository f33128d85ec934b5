"""Vavupel: the typed configuration and its translation into a ModelSpec.

A Vavupel model is a list of layers that config.json writes out one by one, a part of which
may run several times in a row with the same weights:

    {"architecture": "Vavupel", "vocab": V, "width": W, "norm": {"eps": e},
     "embedding": {"scale": s, "bigram": {"buckets": B, "mul_prev": a, "mul_cur": b}},
     "layers": [{"type": "latent_attention" | "retention", "mixer": {...}, "mlp": {...} | null}],
     "loop": {"start": i, "stop": j, "times": n},        (optional)
     "logit_softcap": c}                                 (optional)

What the design fixes and config.json has no key for is stated once in
:func:`vavupel_spec`: every norm is a Dynamic Tanh (tanh(alpha x) w + b); a sub-layer is
normed on its way in and on its way out (x <- x + N'(sublayer(N(x)))); the embedding adds a
hashed bigram row to the token's row and is normed; the feed-forward is two matrices around
the square of relu; the latent attention rotates neighbouring pairs, masks with a sliding
window, has a sink per head in its softmax and a sigmoid gate per head; retention rotates
half-split pairs, scales k by dim^-1/2 and is followed by a weightless unit norm per head and
a SiLU gate; before the first layer of every pass through the loop the stream is mixed with
the embedding's output by one matrix over [x | x0]; the logits have a matrix of their own and
a tanh cap.  Tensor names: ``embed``, ``bigram``, ``embed.norm``, ``loop.in``,
``l<i>.norm1`` / ``norm1b`` / ``norm2`` / ``norm2b`` (each with ``.b`` and ``.alpha``),
``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Mapping, Optional, Tuple

from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, require

_TYPES = ("latent_attention", "retention")
# positions a sequence may reach where config.json sets no bound ("max_positions")
_DEFAULT_POSITIONS = 1 << 20


def _positive(d: Mapping[str, Any], key: str, where: str) -> int:
    v = d.get(key) if isinstance(d, Mapping) else None
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}.'{key}' must be a positive integer, got {v!r}")
    return v


def _integer(d: Mapping[str, Any], key: str, where: str) -> int:
    v = d.get(key) if isinstance(d, Mapping) else None
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config.json: {where}.'{key}' must be an integer, got {v!r}")
    return v


def _number(d: Mapping[str, Any], key: str, where: str) -> float:
    v = d.get(key) if isinstance(d, Mapping) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}.'{key}' must be a number, got {v!r}")
    return float(v)


def _rot(m: Mapping[str, Any], where: str, width: int) -> Optional[Mapping[str, Any]]:
    """The rotation of a mixer: {"dims", "base"} or None when nothing is rotated."""
    rot = m.get("rot")
    if not rot:
        return None
    dims = _positive(rot, "dims", where + ".rot")
    if dims % 2 or dims > width:
        raise ConfigError(f"config.json: {where}.rot.'dims' = {dims} must be even and at most "
                          f"the rotated width ({width})")
    base = _number(rot, "base", where + ".rot")
    if base <= 0:
        raise ConfigError(f"config.json: {where}.rot.'base' must be positive")
    return {"dims": dims, "base": base}


@dataclass(frozen=True)
class VavupelLayer:
    type: str
    mixer: Mapping[str, Any]       # checked sizes and constants of the mixer
    ff: int                        # 0: no feed-forward


@dataclass(frozen=True)
class VavupelConfig:
    vocab: int
    width: int
    eps: float
    embed_scale: float
    buckets: int
    mul_prev: int
    mul_cur: int
    layers: Tuple[VavupelLayer, ...]
    loop: Optional[Tuple[int, int, int]]     # (start, stop, times)
    logit_softcap: float                     # 0: none
    max_positions: int
    raw: Mapping[str, Any]

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "VavupelConfig":
        vocab, width = require(d, "vocab", int), require(d, "width", int)
        if vocab <= 0 or width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        eps = _number(require(d, "norm"), "eps", "norm")
        if eps <= 0:
            raise ConfigError("config.json: norm.'eps' must be positive")
        emb = require(d, "embedding")
        scale = _number(emb, "scale", "embedding")
        big = emb.get("bigram") if isinstance(emb, Mapping) else None
        if not isinstance(big, Mapping):
            raise ConfigError("config.json: embedding.'bigram' is missing")
        buckets = _positive(big, "buckets", "embedding.bigram")
        mul_prev = _integer(big, "mul_prev", "embedding.bigram")
        mul_cur = _integer(big, "mul_cur", "embedding.bigram")
        listed = require(d, "layers")
        if not isinstance(listed, (list, tuple)) or not listed:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers: List[VavupelLayer] = []
        for i, l in enumerate(listed):
            where = f"layers[{i}]"
            kind = l.get("type") if isinstance(l, Mapping) else None
            if kind not in _TYPES:
                raise ConfigError(f"config.json: {where}.'type' = {kind!r} is not one of "
                                  f"{', '.join(_TYPES)}")
            m = l.get("mixer")
            if not isinstance(m, Mapping):
                raise ConfigError(f"config.json: {where}.'mixer' is missing")
            mw = where + ".mixer"
            mixer = {"heads": _positive(m, "heads", mw), "dim": _positive(m, "dim", mw),
                     "vdim": _positive(m, "vdim", mw)}
            if kind == "retention":
                decay = m.get("decay")
                if not isinstance(decay, (list, tuple)) or len(decay) != mixer["heads"] or any(
                        isinstance(x, bool) or not isinstance(x, (int, float)) for x in decay):
                    raise ConfigError(f"config.json: {mw}.'decay' must list one number per head "
                                      f"({mixer['heads']})")
                mixer["decay"] = tuple(float(x) for x in decay)
                mixer["rot"] = _rot(m, mw, mixer["dim"])
            else:
                mixer["rot_dim"] = _positive(m, "rot_dim", mw)
                mixer["kv_rank"] = _positive(m, "kv_rank", mw)
                mixer["scale"] = _number(m, "scale", mw)
                if mixer["scale"] <= 0:
                    raise ConfigError(f"config.json: {mw}.'scale' must be positive")
                mask = m.get("mask")
                mixer["window"] = _positive(mask, "size", mw + ".mask") if mask else 0
                mixer["rot"] = _rot(m, mw, mixer["rot_dim"])
            ff = 0
            mlp = l.get("mlp")
            if mlp:
                if mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.'kind' = {mlp.get('kind')!r} is not "
                                      f"supported; known: dense")
                ff = _positive(mlp, "ff", where + ".mlp")
            layers.append(VavupelLayer(kind, mixer, ff))
        loop = None
        if d.get("loop"):
            lp = d["loop"]
            start, stop = _integer(lp, "start", "loop"), _integer(lp, "stop", "loop")
            times = _positive(lp, "times", "loop")
            if not 0 <= start < stop <= len(layers):
                raise ConfigError(f"config.json: loop: layers {start} to {stop} - 1 of {len(layers)}")
            loop = (start, stop, times)
        cap = d.get("logit_softcap")
        cap = 0.0 if not cap else _number(d, "logit_softcap", "")
        if cap < 0:
            raise ConfigError("config.json: 'logit_softcap' must be positive")
        most = d.get("max_positions")
        return cls(vocab=vocab, width=width, eps=eps, embed_scale=scale, buckets=buckets,
                   mul_prev=mul_prev, mul_cur=mul_cur, layers=tuple(layers), loop=loop,
                   logit_softcap=cap,
                   max_positions=_DEFAULT_POSITIONS if most is None else _positive(d, "max_positions", ""),
                   raw=dict(d))

    def to_dict(self) -> dict:
        return dict(self.raw)


_NORM_NAMES = {"weight": "", "b": ".b", "alpha": ".alpha"}
_RETENTION_NAMES = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v",
                    "g_proj.weight": "g", "o_proj.weight": "o"}
_LATENT_NAMES = {"q_proj.weight": "q", "dkv_proj.weight": "dkv", "dkv_norm.weight": "dkv.norm",
                 "uk_proj.weight": "uk", "uv_proj.weight": "uv", "sink": "sink",
                 "g_proj.weight": "g", "o_proj.weight": "o"}
_MLP_NAMES = {"up_proj.weight": "up", "down_proj.weight": "down"}
_NORM_SITES = {"pre_mixer": "norm1", "post_mixer": "norm1b", "pre_feed_forward": "norm2",
               "post_feed_forward": "norm2b"}


def vavupel_spec(cfg: VavupelConfig) -> ModelSpec:
    """Lay the configuration out as parts, layer by layer, and the loop as a schedule in
    which the looped layers appear once per pass (same weights, a cache of their own)."""
    norm = PartSpec("dynamic_tanh", {})
    layers, tolerated = [], []
    for i, l in enumerate(cfg.layers):
        m = l.mixer
        rot = m["rot"]
        if l.type == "retention":
            position = PartSpec("rope_neox", {"theta": rot["base"], "rotary_dim": rot["dims"],
                                              "frequencies": "float64"}) if rot else PartSpec("none", {})
            mixer = PartSpec("retention", {
                "num_heads": m["heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
                "decay": m["decay"], "key_scale": m["dim"] ** -0.5, "norm_eps": cfg.eps,
                "position": position})
            names = _RETENTION_NAMES
        else:
            position = PartSpec("rope_interleaved", {"theta": rot["base"], "rotary_dim": rot["dims"],
                                                     "frequencies": "float64"}) if rot \
                else PartSpec("none", {})
            mixer = PartSpec("latent_attention", {
                "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"],
                "value_dim": m["vdim"], "kv_rank": m["kv_rank"], "score_scale": m["scale"],
                "window": m["window"], "norm_eps": cfg.eps, "position": position,
                "sink": True, "head_gate": True})
            names = _LATENT_NAMES
        ffn: Optional[PartSpec] = None
        norms = {"pre_mixer": norm, "post_mixer": norm}
        if l.ff:
            ffn = PartSpec("mlp", {"intermediate_size": l.ff, "activation": "relu_squared"})
            norms.update({"pre_feed_forward": norm, "post_feed_forward": norm})
        else:
            # a folder may still hold the norms of the sub-layer that is not there
            tolerated += [f"l{i}.{site}{tail}" for site in ("norm2", "norm2b") for tail in _NORM_NAMES.values()]
        sites = {"mixer": "mix.", "feed_forward": "mlp."}
        sites.update(_NORM_SITES)
        tensor_names = {"mixer": names, "feed_forward": _MLP_NAMES}
        tensor_names.update({site: _NORM_NAMES for site in _NORM_SITES})
        layers.append(LayerSpec(prefix=f"l{i}.", block="sandwich", mixer=mixer, feed_forward=ffn,
                                norms=norms, names=sites, tensor_names=tensor_names))
    n = len(layers)
    if cfg.loop:
        start, stop, times = cfg.loop
        schedule = [ScheduleEntry(i) for i in range(start)]
        for _ in range(times):
            schedule += [ScheduleEntry(i, begins_pass=(i == start)) for i in range(start, stop)]
        schedule += [ScheduleEntry(i) for i in range(stop, n)]
        pass_mix: Optional[PartSpec] = PartSpec("stream_mix", {})
    else:
        schedule = [ScheduleEntry(i) for i in range(n)]
        pass_mix = None
    spec = ModelSpec(
        architecture="Vavupel", hidden_size=cfg.width, vocab_size=cfg.vocab,
        max_positions=cfg.max_positions,
        embedding=PartSpec("bigram_embedding", {
            "scale": cfg.embed_scale, "buckets": cfg.buckets, "mul_prev": cfg.mul_prev,
            "mul_cur": cfg.mul_cur, "norm": norm}),
        layers=tuple(layers), schedule=tuple(schedule), final_norm=norm,
        head=PartSpec("lm_head", {"tied": False, "logit_softcap": cfg.logit_softcap}),
        names={"embedding": "", "final_norm": "final.norm", "head": "head", "pass_mix": "loop."},
        tensor_names={"embedding": {"weight": "embed", "bigram.weight": "bigram",
                                    "norm.weight": "embed.norm", "norm.b": "embed.norm.b",
                                    "norm.alpha": "embed.norm.alpha"},
                      "final_norm": _NORM_NAMES, "head": {"weight": ""},
                      "pass_mix": {"weight": "in"}},
        pass_mix=pass_mix, tolerated=tuple(tolerated), stop_tokens=())
    spec.validate()
    return spec
