"""The Gotulorn decoder, plain and slow: float64 NumPy over whole sequences, one function per
mechanism, no cache, no batching, nothing shared with the engine.

``cfg`` is the configuration as a dictionary (the keys of config.json), ``W`` maps tensor names
to float64 arrays.  A sequence is a list of token ids; position t is its index.

Notation: T tokens, E the width, H query heads, G key/value heads, D the query/key size per head,
Dv the value size per head, R the latent's rank, Dr the rotated size.
"""
from __future__ import annotations

import math

import numpy as np


def dyt(x, w, b, alpha):
    """Dynamic tanh norm: tanh(alpha x) w + b, element by element (no mean, no variance)."""
    return np.tanh(float(alpha) * x) * w + b


def rms_unit(x, eps):
    """x over its root mean square along the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def softmax_rows(s, visible):
    """Row-wise softmax of s over the entries where ``visible`` is true; zeros elsewhere."""
    s = np.where(visible, s, -np.inf)
    m = s.max(axis=-1, keepdims=True)
    e = np.where(visible, np.exp(s - m), 0.0)
    return e / e.sum(axis=-1, keepdims=True)


def causal(T):
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return j <= i


def window_with_first(T, size, keep_first):
    """Position i sees j <= i when it is one of the last ``size`` (i - j < size) or one of the first
    ``keep_first`` tokens of the sequence."""
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def rotate_interleaved(x, base, dims, positions):
    """Rotary positions on the first ``dims`` entries of the last axis of x [T, ..., n]: the pair
    (2i, 2i + 1) turns by positions * base^(-2i / dims)."""
    out = x.copy()
    half = dims // 2
    f = np.array([float(base) ** (-2.0 * i / dims) for i in range(half)])
    a = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]        # [T, half]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (half,)
    c, s = np.cos(a).reshape(shape), np.sin(a).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def differential_attention(h, W, p, m, eps, kv=None):
    """The 'attention' mixer.  h [T, E].  ``kv``: (k, v) of the layer whose keys and values this one
    borrows, or None to project its own.  Returns (out [T, E], (k, v))."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + ".q"].T).reshape(T, H, 2, D)
    if kv is None:
        k = (h @ W[p + ".k"].T).reshape(T, G, 2, D)
        v = (h @ W[p + ".v"].T).reshape(T, G, Dv)
    else:
        k, v = kv
    see = window_with_first(T, m["mask"]["size"], m["mask"]["keep_first"]) if m.get("mask") else causal(T)
    lam = math.exp(float(np.sum(W[p + ".lq1"] * W[p + ".lk1"]))) - math.exp(float(np.sum(W[p + ".lq2"] * W[p + ".lk2"]))) + m["diff"]
    out = np.zeros((T, H, Dv))
    for hd in range(H):
        g = hd // (H // G)
        a = []
        for mp in range(2):
            s = (q[:, hd, mp, :] @ k[:, g, mp, :].T) * m["scale"]
            a.append(softmax_rows(s, see) @ v[:, g, :])
        o = a[0] - lam * a[1]
        out[:, hd, :] = rms_unit(o, eps) * (1.0 - m["diff"])
    return out.reshape(T, H * Dv) @ W[p + ".o"].T, (k, v)


def latent_attention(h, W, p, m, eps):
    """The 'latent_attention' mixer: keys and values of every head come from one latent c [T, R] and
    one rotated key part [T, Dr] shared by the heads."""
    T = h.shape[0]
    H, D, Dr, Dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(T)
    q = (h @ W[p + ".q"].T).reshape(T, H, D + Dr)
    q_plain, q_rot = q[:, :, :D], rotate_interleaved(q[:, :, D:], m["rot"]["base"], m["rot"]["dims"], pos)
    down = h @ W[p + ".dkv"].T
    c = rms_unit(down[:, :R], eps) * W[p + ".dkv.norm"]
    k_rot = rotate_interleaved(down[:, R:], m["rot"]["base"], m["rot"]["dims"], pos)           # [T, Dr]
    k_plain = (c @ W[p + ".uk"].T).reshape(T, H, D)
    v = (c @ W[p + ".uv"].T).reshape(T, H, Dv)
    see = causal(T)
    out = np.zeros((T, H, Dv))
    for hd in range(H):
        s = (q_plain[:, hd, :] @ k_plain[:, hd, :].T + q_rot[:, hd, :] @ k_rot.T) * m["scale"]
        out[:, hd, :] = softmax_rows(s, see) @ v[:, hd, :]
    return out.reshape(T, H * Dv) @ W[p + ".o"].T


def dense_ff(h, W, p, f):
    """g = min(W_gate h, limit), u = clamp(W_up h, +-limit); W_down (g sigmoid(1.702 g) (u + 1))."""
    lim = f["limit"]
    g = np.minimum(h @ W[p + ".gate"].T, lim)
    u = np.clip(h @ W[p + ".up"].T, -lim, lim)
    return (g / (1.0 + np.exp(-1.702 * g)) * (u + 1.0)) @ W[p + ".down"].T


def routed_ff(h, W, p, f, gaps=None):
    """Every token goes through its ``top`` experts with the largest router logits; their weights are
    the softmax over those logits alone.  ``gaps`` (a list) receives, per token, how far the last
    chosen logit lies above the first one left out (infinite when every expert is chosen)."""
    n_exp, top = f["router"]["experts"], f["router"]["top"]
    z = h @ W[p + ".router"].T + W[p + ".router.b"]
    out = np.zeros((h.shape[0], W[p + ".e0.down"].shape[0]))
    if gaps is not None:
        ranked = -np.sort(-z, axis=1)
        gaps.append(ranked[:, top - 1] - ranked[:, top] if top < n_exp else np.full(h.shape[0], np.inf))
    for t in range(h.shape[0]):
        chosen = np.argsort(-z[t], kind="stable")[:top]
        w = np.exp(z[t, chosen] - z[t, chosen].max())
        w = w / w.sum()
        for e, we in zip(chosen, w):
            a = h[t] @ W[f"{p}.e{e}.gate"].T
            y = (a / (1.0 + np.exp(-a))) * (h[t] @ W[f"{p}.e{e}.up"].T)
            out[t] += we * (y @ W[f"{p}.e{e}.down"].T)
    return out


def norm_of(W, name, x):
    return dyt(x, W[name], W[name + ".b"], W[name + ".alpha"])


def forward(cfg, W, tokens, return_layers=False, router_gaps=None):
    """Logits [T, vocab] of a whole sequence (and, on request, the residual stream after every layer;
    ``router_gaps``, a list, receives one array per routed layer: see ``routed_ff``)."""
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    x = norm_of(W, "embed.norm", x)
    kept = {}
    layers = []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}", layer["mixer"]
        h = norm_of(W, p + ".norm1", x)
        if layer["type"] == "attention":
            src = m.get("kv_from")
            d, kv = differential_attention(h, W, p + ".mix", m, eps, kv=None if src is None else kept[src])
            kept[i] = kv
        elif layer["type"] == "latent_attention":
            d = latent_attention(h, W, p + ".mix", m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + d
        f = layer.get("mlp")
        if f is not None:
            h = norm_of(W, p + ".norm2", x)
            x = x + (dense_ff(h, W, p + ".mlp", f) if f["kind"] == "dense" else routed_ff(h, W, p + ".mlp", f, router_gaps))
        layers.append(x.copy())
    logits = norm_of(W, "final.norm", x) @ W["head"].T
    return (logits, layers) if return_layers else logits
