"""A plain, slow Karupel: one function per mechanism, straight from the equations, on the
CPU in 64-bit.  It shares no code with the package and is what the tests compare with.

Notation.  T tokens of one sequence, W the model width.  ``p`` maps a layer's local tensor
names to tensors, ``m`` is the layer's mixer configuration.  Every mechanism takes the
tokens it is given plus what earlier tokens of the sequence left behind (``state``, a
dictionary that it updates), so a prompt can be fed in one piece, in portions or token by
token and must give the same rows.

    layer:      x <- x + N1(mixer(x));  x <- x + N2(ff(x))  (the second only with a feed-forward)
    N(y)      = y / sqrt(mean(y^2) + eps) * (1 + w)
    logits    = E . Nf(x)           (E: the embedding table)
"""

from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional, Sequence

import torch

F = torch.float64


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.log1p(torch.exp(-x.abs())) + torch.clamp(x, min=0)


def log_sigmoid(x: torch.Tensor) -> torch.Tensor:
    return -softplus(-x)


def short_conv(x: torch.Tensor, w: torch.Tensor, state: Dict, key: str) -> torch.Tensor:
    """y[t, c] = sum_j w[c, j] * x[t - (taps - 1) + j, c], zeros before the sequence's start;
    the last taps - 1 inputs are carried in ``state[key]``."""
    taps = w.shape[1]
    past = state.get(key)
    if past is None:
        past = torch.zeros((taps - 1, x.shape[1]), dtype=F)
    full = torch.cat([past, x], dim=0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + full[j:j + x.shape[0]] * w[:, j]
    state[key] = full[full.shape[0] - (taps - 1):].clone()
    return y


def delta_mixer(h: torch.Tensor, p: Mapping[str, torch.Tensor], m: Mapping, eps: float,
                state: Dict) -> torch.Tensor:
    """Gated delta rule.  Per head, with unit q (times dim^-1/2) and unit k:
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ p["q"].T, p["q.conv"], state, "q")).view(T, G, D)
    k = silu(short_conv(h @ p["k"].T, p["k.conv"], state, "k")).view(T, G, D)
    v = silu(short_conv(h @ p["v"].T, p["v.conv"], state, "v")).view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ p["b"].T)                                          # [T, H]
    g = torch.exp(-torch.exp(p["A_log"]) * softplus(h @ p["a"].T + p["dt_bias"]))   # [T, H]
    gate = silu(h @ p["g"].T).view(T, H, V)
    S = state.get("S")
    if S is None:
        S = torch.zeros((H, D, V), dtype=F)
    out = torch.zeros((T, H, V), dtype=F)
    for t in range(T):
        for hd in range(H):
            kv = hd // (H // G)
            S[hd] = g[t, hd] * S[hd]
            u = beta[t, hd] * (v[t, hd] - S[hd].T @ k[t, kv])
            S[hd] = S[hd] + torch.outer(k[t, kv], u)
            out[t, hd] = S[hd].T @ q[t, kv]
    state["S"] = S
    out = rms_unit(out, eps) * p["norm"] * gate
    return out.reshape(T, H * V) @ p["o"].T


def rotate(x: torch.Tensor, pos: torch.Tensor, rot: Mapping) -> torch.Tensor:
    """Rotary positions on the first ``dims`` dimensions of each head of x[T, heads, dim];
    dimension i is paired with i + dims/2; angle = pos * base^(-2i/dims) / factor."""
    dims = int(rot["dims"])
    half = dims // 2
    factor = float((rot.get("scaling") or {}).get("factor", 1.0))
    i = torch.arange(half, dtype=F)
    freq = float(rot["base"]) ** (-2.0 * i / dims) / factor
    ang = pos.to(F)[:, None] * freq[None, :]                 # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def attention_mixer(h: torch.Tensor, p: Mapping[str, torch.Tensor], m: Mapping, eps: float,
                    state: Dict, shared: Dict, first_mix: bool) -> torch.Tensor:
    """Softmax attention over all earlier positions and the own one.  ``shared`` carries the
    first value-mixing layer's values of the same tokens from layer to layer."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    start = state.get("n", 0)
    pos = torch.arange(start, start + T)
    q = (h @ p["q"].T + p["q.b"]).view(T, H, D)
    k = (h @ p["k"].T + p["k.b"]).view(T, G, D)
    v = (h @ p["v"].T + p["v.b"]).view(T, G, V)
    q = rms_unit(q, eps) * p["q.norm"]
    k = rms_unit(k, eps) * p["k.norm"]
    if m.get("rot"):
        q, k = rotate(q, pos, m["rot"]), rotate(k, pos, m["rot"])
    if m.get("v_mix"):
        if first_mix:
            shared["v_first"] = v
        else:
            lam = p["vmix"]
            v = (1 - lam) * v + lam * shared["v_first"]
    K = torch.cat([state["k"], k]) if "k" in state else k
    Vv = torch.cat([state["v"], v]) if "v" in state else v
    state["k"], state["v"], state["n"] = K, Vv, start + T
    gate = torch.sigmoid(h @ p["g"].T)                       # [T, H]
    out = torch.zeros((T, H, V), dtype=F)
    for hd in range(H):
        kv = hd // (H // G)
        s = (q[:, hd] @ K[:, kv].T) * float(m["scale"])      # [T, keys]
        keys = torch.arange(K.shape[0])
        s = s.masked_fill(keys[None, :] > pos[:, None], float("-inf"))
        out[:, hd] = torch.softmax(s, dim=-1) @ Vv[:, kv]
    out = out * gate[:, :, None]
    return out.reshape(T, H * V) @ p["o"].T


def mlstm_mixer(h: torch.Tensor, p: Mapping[str, torch.Tensor], m: Mapping, eps: float,
                state: Dict) -> torch.Tensor:
    """Matrix memory with a running maximum mx (0 at the start):
    mx' = max(f + mx, i);  S' = e^(f + mx - mx') S + e^(i - mx') k v^T;  n' likewise with k;
    o = S'^T q / (max(|n' . q|, e^-mx') + 1e-6)."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    cap = float(m["gate_cap"])
    q = (h @ p["q"].T).view(T, H, D) * D ** -0.5
    k = (h @ p["k"].T).view(T, H, D)
    v = (h @ p["v"].T).view(T, H, V)
    ig = cap * torch.tanh((h @ p["i"].T + p["i.b"]) / cap)
    fg = log_sigmoid(cap * torch.tanh((h @ p["f"].T + p["f.b"]) / cap))
    S = state.get("S")
    if S is None:
        S = torch.zeros((H, D, V), dtype=F)
        state["n"] = torch.zeros((H, D), dtype=F)
        state["m"] = torch.zeros((H,), dtype=F)
    n, mx = state["n"], state["m"]
    out = torch.zeros((T, H, V), dtype=F)
    for t in range(T):
        for hd in range(H):
            new = torch.maximum(fg[t, hd] + mx[hd], ig[t, hd])
            keep, take = torch.exp(fg[t, hd] + mx[hd] - new), torch.exp(ig[t, hd] - new)
            S[hd] = keep * S[hd] + take * torch.outer(k[t, hd], v[t, hd])
            n[hd] = keep * n[hd] + take * k[t, hd]
            mx[hd] = new
            den = torch.maximum((n[hd] @ q[t, hd]).abs(), torch.exp(-new)) + 1e-6
            out[t, hd] = S[hd].T @ q[t, hd] / den
    state["S"], state["n"], state["m"] = S, n, mx
    out = rms_unit(out, eps).reshape(T, H * V) * p["norm"] * torch.sigmoid(h @ p["g"].T)
    return out @ p["o"].T


def dense_ff(h: torch.Tensor, p: Mapping[str, torch.Tensor]) -> torch.Tensor:
    return (silu(h @ p["gate"].T) * (h @ p["up"].T)) @ p["down"].T


def layer_tensors(weights: Mapping[str, torch.Tensor], i: int, part: str) -> Dict[str, torch.Tensor]:
    pre = f"l{i}.{part}."
    return {n[len(pre):]: t.to(F) for n, t in weights.items() if n.startswith(pre)}


class Plain:
    """The whole model; ``new_state()`` per sequence, ``run(tokens, state)`` continues it."""

    def __init__(self, config: Mapping, weights: Mapping[str, torch.Tensor]):
        self.cfg = config
        self.w = weights
        self.eps = float(config["norm"]["eps"])
        self.embed = weights["embed"].to(F)
        mixing = [i for i, l in enumerate(config["layers"])
                  if l["type"] == "attention" and l["mixer"].get("v_mix")]
        self.first_mix = mixing[0] if mixing else -1

    def new_state(self) -> List[Dict]:
        return [dict() for _ in self.cfg["layers"]]

    def norm(self, y: torch.Tensor, name: str) -> torch.Tensor:
        return rms_unit(y, self.eps) * (1 + self.w[name].to(F))

    def run(self, tokens: Sequence[int], state: Optional[List[Dict]] = None, layers_out=None):
        """Logits [len(tokens), vocab] of the given tokens, continuing ``state``."""
        state = self.new_state() if state is None else state
        x = self.embed[torch.tensor(list(tokens), dtype=torch.long)]
        shared: Dict = {}
        for i, layer in enumerate(self.cfg["layers"]):
            p, m = layer_tensors(self.w, i, "mix"), layer["mixer"]
            if layer["type"] == "delta":
                y = delta_mixer(x, p, m, self.eps, state[i])
            elif layer["type"] == "attention":
                y = attention_mixer(x, p, m, self.eps, state[i], shared, i == self.first_mix)
            elif layer["type"] == "mlstm":
                y = mlstm_mixer(x, p, m, self.eps, state[i])
            else:
                raise ValueError(layer["type"])
            x = x + self.norm(y, f"l{i}.norm1")
            if layer.get("mlp"):
                x = x + self.norm(dense_ff(x, layer_tensors(self.w, i, "mlp")), f"l{i}.norm2")
            if layers_out is not None:
                layers_out.append(x.clone())
        return self.norm(x, "final.norm") @ self.embed.T


def random_weights(config: Mapping, seed: int, std: float = 0.5) -> Dict[str, torch.Tensor]:
    """Random tensors of every name the configuration asks for, rounded to bfloat16 values:
    matrices ~ N(0, std^2 / inputs), small norm weights, decays and gates in a lively range."""
    g = torch.Generator().manual_seed(seed)
    W = config["width"]

    def mat(o, i, s=1.0):
        return torch.randn((o, i), generator=g) * (s * std / math.sqrt(i))

    def vec(n, s=0.3, at=0.0):
        return torch.randn((n,), generator=g) * s + at

    out = {"embed": torch.randn((config["vocab"], W), generator=g), "final.norm": vec(W)}
    for i, layer in enumerate(config["layers"]):
        m, pre = layer["mixer"], f"l{i}.mix."
        out[f"l{i}.norm1"] = vec(W)
        if layer["type"] == "delta":
            H, G, D, V, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for n, rows in (("q", G * D), ("k", G * D), ("v", H * V)):
                out[pre + n] = mat(rows, W, 3.0)
                out[pre + n + ".conv"] = torch.randn((rows, taps), generator=g) * 0.6
            out[pre + "b"], out[pre + "a"] = mat(H, W, 3.0), mat(H, W, 3.0)
            out[pre + "A_log"], out[pre + "dt_bias"] = vec(H, 0.5, -1.0), vec(H, 0.5)
            out[pre + "norm"] = vec(V, 0.3, 1.0)
            out[pre + "g"], out[pre + "o"] = mat(H * V, W, 3.0), mat(W, H * V, 2.0)
        elif layer["type"] == "attention":
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for n, rows in (("q", H * D), ("k", G * D), ("v", G * V)):
                out[pre + n] = mat(rows, W, 2.0)
                out[pre + n + ".b"] = vec(rows, 0.2)
            out[pre + "q.norm"], out[pre + "k.norm"] = vec(D, 0.3, 1.0), vec(D, 0.3, 1.0)
            if m.get("v_mix"):
                out[pre + "vmix"] = torch.rand((), generator=g) * 0.6 + 0.2
            out[pre + "g"], out[pre + "o"] = mat(H, W, 3.0), mat(W, H * V, 2.0)
        elif layer["type"] == "mlstm":
            H, D, V = m["heads"], m["dim"], m["vdim"]
            out[pre + "q"], out[pre + "k"], out[pre + "v"] = mat(H * D, W, 2.0), mat(H * D, W, 2.0), mat(H * V, W, 2.0)
            out[pre + "i"], out[pre + "f"] = mat(H, W, 4.0), mat(H, W, 4.0)
            out[pre + "i.b"], out[pre + "f.b"] = vec(H, 0.5), vec(H, 0.5, 2.0)
            out[pre + "norm"] = vec(H * V, 0.3, 1.0)
            out[pre + "g"], out[pre + "o"] = mat(H * V, W, 3.0), mat(W, H * V, 2.0)
        if layer.get("mlp"):
            ff = layer["mlp"]["ff"]
            out[f"l{i}.norm2"] = vec(W)
            out[f"l{i}.mlp.gate"], out[f"l{i}.mlp.up"] = mat(ff, W, 2.0), mat(ff, W, 2.0)
            out[f"l{i}.mlp.down"] = mat(W, ff, 2.0)
    return {n: t.to(torch.bfloat16).to(torch.float32) for n, t in out.items()}
