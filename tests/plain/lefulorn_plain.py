"""A plain, slow Lefulorn in float64 on the host: one function per mechanism, written from the
design's equations, sharing nothing with the engine.  Tests compare the engine against it.

Notation: T tokens of one sequence at positions 0 .. T-1 (or ``pos0`` .. for a continuation),
E the model width.  ``w`` maps tensor names to float64 tensors.  Linear weights are [out, in].
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def rms_norm(x, weight, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def relu_squared_ff(h, up, up_b, down, down_b):
    a = torch.relu(h @ up.T + up_b)
    return (a * a) @ down.T + down_b


def query_temperature(positions, coef, every):
    """1 + coef * ln(floor((p + 1) / every) + 1) per position."""
    steps = torch.div(positions + 1, every, rounding_mode="floor").to(F64)
    return 1.0 + coef * torch.log(steps + 1.0)


def distance_slopes(n_heads):
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / n_heads) for h in range(n_heads)], dtype=F64)


def sink_attention(q, k, v, sink, scale, window: Optional[int], slopes):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] of one whole sequence -> [T, H, Dv].  Query i sees
    keys j with 0 <= i - j < window; score (q.k) scale - slope_h (i - j); the softmax's denominator
    also holds exp(sink_h), which has no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = 0 if window is None else max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            dist = torch.arange(i - lo, -1, -1, dtype=F64)          # i - j for j = lo .. i
            s = s - slopes[h] * dist
            m = max(float(s.max()), float(sink[h]))
            e = torch.exp(s - m)
            den = e.sum() + math.exp(float(sink[h]) - m)
            out[i, h] = (e / den) @ v[lo:i + 1, g]
    return out


def attention_mixer(h, w, pre, spec, positions, v_first):
    """The attention mixer on one whole sequence.  Returns (delta [T, E], the values it cached
    [T, G, Dv]).  ``v_first``: the values of the first value-mixing layer (None in that layer
    and in layers that do not mix)."""
    H, G, D, Dv = spec["heads"], spec["kv_heads"], spec["dim"], spec["vdim"]
    T = h.shape[0]
    q = (h @ w[pre + "q"].T + w[pre + "q.b"]).view(T, H, D)
    k = (h @ w[pre + "k"].T + w[pre + "k.b"]).view(T, G, D)
    v = (h @ w[pre + "v"].T + w[pre + "v.b"]).view(T, G, Dv)
    qt = spec.get("q_temp")
    if qt:
        q = q * query_temperature(positions, qt["coef"], qt["every"])[:, None, None]
    if v_first is not None:
        lam = w[pre + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    mask = spec.get("mask")
    o = sink_attention(q, k, v, w[pre + "sink"], spec["scale"], mask["size"] if mask else None, distance_slopes(H))
    gate = torch.sigmoid(h @ w[pre + "g"].T)
    return (o.reshape(T, H * Dv) * gate) @ w[pre + "o"].T, v


def causal_conv_silu(x, taps_w):
    """x [T, C]; taps_w [C, taps], the last column weighs the current token; zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F64), x], 0)
    y = torch.zeros(T, C, dtype=F64)
    for i in range(taps):
        y = y + padded[i:i + T] * taps_w[:, i]
    return y * torch.sigmoid(y)


def gated_delta_rule(q, k, v, beta, decay):
    """One head.  q, k, decay [T, D]; v [T, Dv]; beta [T].  S [D, Dv] starts at zero:
    S <- decay_t * S (row-wise); u = beta_t (v_t - S^T k_t); S <- S + k_t u^T; o_t = S^T q_t."""
    T, D = q.shape
    S = torch.zeros(D, v.shape[1], dtype=F64)
    out = torch.zeros(T, v.shape[1], dtype=F64)
    for t in range(T):
        S = decay[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def channel_delta_mixer(h, w, pre, spec, eps):
    H, G, D, Dv = spec["heads"], spec["kv_heads"], spec["dim"], spec["vdim"]
    T = h.shape[0]
    q = causal_conv_silu(h @ w[pre + "q"].T, w[pre + "q.conv"]).view(T, G, D)
    k = causal_conv_silu(h @ w[pre + "k"].T, w[pre + "k.conv"]).view(T, G, D)
    v = causal_conv_silu(h @ w[pre + "v"].T, w[pre + "v.conv"]).view(T, H, Dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[pre + "b"].T)                                   # [T, H]
    a = (h @ w[pre + "a1"].T) @ w[pre + "a2"].T + w[pre + "dt_bias"]            # [T, H D]
    rate = torch.exp(w[pre + "A_log"])                                         # [H]
    decay = torch.exp(-rate[None, :, None] * torch.nn.functional.softplus(a.view(T, H, D)))
    gate = torch.sigmoid((h @ w[pre + "g1"].T) @ w[pre + "g2"].T).view(T, H, Dv)
    out = torch.zeros(T, H, Dv, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        o = gated_delta_rule(q[:, g], k[:, g], v[:, hd], beta[:, hd], decay[:, hd])
        o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * w[pre + "norm"]
        out[:, hd] = o * gate[:, hd]
    return out.reshape(T, H * Dv) @ w[pre + "o"].T


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens: List[int], want_layers: bool = False):
    """Logits [T, vocab] of one whole sequence (and the residual stream after every layer)."""
    w = {n: t.to(F64) for n, t in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    positions = torch.arange(len(tokens))
    v_first = None
    seen_mix = False
    after = []
    for i, layer in enumerate(config["layers"]):
        pre = f"l{i}."
        hin = rms_norm(x, w[pre + "norm1"], eps)
        if layer["type"] == "attention":
            mixes = bool(layer["mixer"].get("v_mix"))
            delta, v = attention_mixer(hin, w, pre + "mix.", layer["mixer"], positions, v_first if (mixes and seen_mix) else None)
            if mixes and not seen_mix:
                v_first, seen_mix = v, True
        elif layer["type"] == "channel_delta":
            delta = channel_delta_mixer(hin, w, pre + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + delta
        if layer.get("mlp"):
            hin = rms_norm(x, w[pre + "norm2"], eps)
            x = x + relu_squared_ff(hin, w[pre + "mlp.up"], w[pre + "mlp.up.b"], w[pre + "mlp.down"], w[pre + "mlp.down.b"])
        after.append(x.clone())
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T * config["logit_scale"]
    return (logits, torch.stack(after)) if want_layers else logits
