"""A plain, slow Vavupel in 64-bit numpy: one function per mechanism, whole sequences only.

Nothing here is shared with the package: no cache, no state, no steps.  A sequence is
worked on as a whole, every position from the sequence's first token, so that what the
package does with pages, rings, slots and recorded steps has something independent to be
compared with.

Notation: n tokens, width W; x[t] is row t.  Weights are stored [out, in].
"""

from __future__ import annotations

import numpy as np


def f64(t) -> np.ndarray:
    """A stored tensor (torch or numpy, any float type) as 64-bit numpy."""
    if hasattr(t, "detach"):
        t = t.detach().to("cpu").double().numpy() if t.dtype.is_floating_point else t.cpu().numpy()
    return np.asarray(t, dtype=np.float64)


def dynamic_tanh(x, w, b, alpha):
    """Element by element: tanh(alpha x) w + b.  No mean, no variance."""
    return np.tanh(float(alpha) * x) * w + b


def unit_rms(x, eps):
    """Rows of the last axis divided by their root mean square (eps inside the root)."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def bigram_embedding(tokens, table, bigram, scale, buckets, mul_prev, mul_cur):
    """Row of the token times ``scale`` plus a row of the bigram table picked by a hash of
    (previous token, token); the first token takes the table's last row."""
    out = np.zeros((len(tokens), table.shape[1]))
    for t, tok in enumerate(tokens):
        row = buckets if t == 0 else (int(tokens[t - 1]) * mul_prev + int(tok) * mul_cur) % buckets
        out[t] = table[int(tok)] * scale + bigram[row]
    return out


def rotate(x, positions, dims, base, interleaved):
    """Rotary positions on the first ``dims`` entries of the last axis of x[n, heads, d].
    Pair i is (2i, 2i+1) when ``interleaved`` else (i, i + dims/2); its angle at position p
    is p * base^(-2i/dims)."""
    y = x.copy()
    half = dims // 2
    for i in range(half):
        a, b = (2 * i, 2 * i + 1) if interleaved else (i, i + half)
        ang = np.asarray(positions, dtype=np.float64) * base ** (-2.0 * i / dims)
        c, s = np.cos(ang)[:, None], np.sin(ang)[:, None]
        u, v = x[..., a], x[..., b]
        y[..., a] = u * c - v * s
        y[..., b] = v * c + u * s
    return y


def latent_attention(h, w, m, eps):
    """h[n, W] -> [n, W].  ``w``: the mixer's tensors by their short names (q, dkv, dkv.norm,
    uk, uv, sink, g, o); ``m``: its sizes (heads, dim, rot_dim, vdim, kv_rank, scale,
    mask.size, rot.base).  Keys and values are made from the latent for every position and
    every head; the window and the sink enter a plain softmax over the visible keys."""
    n = h.shape[0]
    H, d, r, vd, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    window = m["mask"]["size"] if m.get("mask") else n      # (no mask: every earlier position)
    pos = np.arange(n)
    q = (h @ w["q"].T).reshape(n, H, d + r)
    down = h @ w["dkv"].T
    c = unit_rms(down[:, :rank], eps) * w["dkv.norm"]
    k_rot = rotate(down[:, None, rank:], pos, m["rot"]["dims"], m["rot"]["base"], True)[:, 0]
    q_rot = rotate(q[:, :, d:], pos, m["rot"]["dims"], m["rot"]["base"], True)
    k = (c @ w["uk"].T).reshape(n, H, d)
    v = (c @ w["uv"].T).reshape(n, H, vd)
    gate = 1.0 / (1.0 + np.exp(-(h @ w["g"].T)))          # [n, H]
    out = np.zeros((n, H, vd))
    for t in range(n):
        lo = max(0, t - window + 1)
        for a in range(H):
            s = (k[lo:t + 1, a] @ q[t, a, :d] + k_rot[lo:t + 1] @ q_rot[t, a]) * m["scale"]
            top = max(s.max(), w["sink"][a])
            e = np.exp(s - top)
            out[t, a] = (e @ v[lo:t + 1, a]) / (e.sum() + np.exp(w["sink"][a] - top))
    out = out * gate[:, :, None]
    return out.reshape(n, H * vd) @ w["o"].T


def retention(h, w, m, eps):
    """h[n, W] -> [n, W].  Per head S <- decay S + k v^T, o = S^T q, token by token."""
    n = h.shape[0]
    H, d, vd = m["heads"], m["dim"], m["vdim"]
    pos = np.arange(n)
    q, k = (h @ w["q"].T).reshape(n, H, d), (h @ w["k"].T).reshape(n, H, d)
    if m.get("rot"):
        q = rotate(q, pos, m["rot"]["dims"], m["rot"]["base"], False)
        k = rotate(k, pos, m["rot"]["dims"], m["rot"]["base"], False)
    k = k * d ** -0.5
    v = (h @ w["v"].T).reshape(n, H, vd)
    o = np.zeros((n, H, vd))
    for a in range(H):
        S = np.zeros((d, vd))
        for t in range(n):
            S = m["decay"][a] * S + np.outer(k[t, a], v[t, a])
            o[t, a] = S.T @ q[t, a]
    o = unit_rms(o, eps).reshape(n, H * vd)
    z = h @ w["g"].T
    return (o * (z / (1.0 + np.exp(-z)))) @ w["o"].T


def dense_ff(h, w):
    up = np.maximum(h @ w["up"].T, 0.0)
    return (up * up) @ w["down"].T


def _norm(x, weights, name):
    return dynamic_tanh(x, weights[name], weights[name + ".b"], weights[name + ".alpha"])


def layer_runs(config):
    """The order in which layers run: those of the loop ``times`` times in a row.  Each item
    is (layer index, whether a pass begins with it)."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, i == 0) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(start)]
    for _ in range(times):
        order += [(i, i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, n)]


def forward(tokens, weights, config, return_layers=False):
    """Logits [n, vocab] of one sequence from its first token on.  ``weights``: every stored
    tensor by its full name, as 64-bit numpy."""
    eps = config["norm"]["eps"]
    emb = config["embedding"]
    x = bigram_embedding(tokens, weights["embed"], weights["bigram"], emb["scale"],
                         emb["bigram"]["buckets"], emb["bigram"]["mul_prev"], emb["bigram"]["mul_cur"])
    x = _norm(x, weights, "embed.norm")
    x0 = x
    after = []
    for i, begins in layer_runs(config):
        layer = config["layers"][i]
        p = f"l{i}."
        if begins and config.get("loop"):
            x = np.concatenate([x, x0], axis=1) @ weights["loop.in"].T
        mix = {k[len(p + "mix."):]: v for k, v in weights.items() if k.startswith(p + "mix.")}
        fn = latent_attention if layer["type"] == "latent_attention" else retention
        x = x + _norm(fn(_norm(x, weights, p + "norm1"), mix, layer["mixer"], eps), weights, p + "norm1b")
        if layer.get("mlp"):
            ff = {k[len(p + "mlp."):]: v for k, v in weights.items() if k.startswith(p + "mlp.")}
            x = x + _norm(dense_ff(_norm(x, weights, p + "norm2"), ff), weights, p + "norm2b")
        after.append(x)
    y = _norm(x, weights, "final.norm") @ weights["head"].T
    cap = config.get("logit_softcap")
    if cap:
        y = cap * np.tanh(y / cap)
    return (y, np.stack(after)) if return_layers else y
