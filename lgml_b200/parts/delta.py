"""The gated delta rule with a decay per key channel ("channel delta") as a mixer.

Per token, from the mixer's input h (H value heads on G query/key heads; head h reads
query/key head h // (H / G)):

    q, k, v   = silu(conv(W h))           short causal convolutions over time, one filter per channel
    q         = q / |q| * D^-1/2,  k = k / |k|                     |x| = sqrt(sum x^2 + 1e-6), per head
    beta      = sigmoid(W_b h)                                      one per head
    g         = exp(-exp(A_log) * softplus(W_a2 W_a1 h + dt_bias))   one per head and key channel
    S        <- g * S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q          per head, S [D, Dv]
    out       = W_o (o / rms(o) * w_norm * sigmoid(W_g2 W_g1 h))

What a request carries from token to token is one float32 vector in its state slot: S of
every head, then the last taps - 1 inputs of the convolutions.  The four wide projections of h
are one product, the two narrow ones (into the low ranks) another.
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache import FixedState
from ..weights import VECTOR, TensorSpec
from .base import Part, register_part


class ChannelDelta(Part):
    graph_safe = True

    def __init__(self, width: int, n_heads: int, n_kv_heads: int, head_dim: int, v_head_dim: int, taps: int, rank_a: int,
                 rank_g: int, eps: float):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads are no multiple of {n_kv_heads} key heads")
        self.width, self.n_heads, self.n_kv_heads = width, n_heads, n_kv_heads
        self.head_dim, self.v_head_dim, self.taps = head_dim, v_head_dim, int(taps)
        self.rank_a, self.rank_g, self.eps = int(rank_a), int(rank_g), float(eps)
        self.channels = 2 * n_kv_heads * head_dim + n_heads * v_head_dim
        self.state_floats = n_heads * head_dim * v_head_dim            # S of every head; the convolutions' inputs follow
        self.w_in = self.w_low = self.w_a2 = self.w_g2 = self.wo = self.conv_w = self.a_log = self.dt_bias = self.norm_w = None

    def cache_spec(self):
        return FixedState((self.state_floats + (self.taps - 1) * self.channels,), torch.float32)

    def tensor_specs(self, prefix):
        H, G, D, Dv, E = self.n_heads, self.n_kv_heads, self.head_dim, self.v_head_dim, self.width
        return [
            TensorSpec(prefix + ".q", (G * D, E)), TensorSpec(prefix + ".q.conv", (G * D, self.taps), VECTOR, init=(0.0, 10.0)),
            TensorSpec(prefix + ".k", (G * D, E)), TensorSpec(prefix + ".k.conv", (G * D, self.taps), VECTOR, init=(0.0, 10.0)),
            TensorSpec(prefix + ".v", (H * Dv, E)), TensorSpec(prefix + ".v.conv", (H * Dv, self.taps), VECTOR, init=(0.0, 10.0)),
            TensorSpec(prefix + ".b", (H, E)), TensorSpec(prefix + ".A_log", (H,), VECTOR),
            TensorSpec(prefix + ".norm", (Dv,), VECTOR, init=(1.0, 1.0)),
            TensorSpec(prefix + ".a1", (self.rank_a, E)), TensorSpec(prefix + ".a2", (H * D, self.rank_a)),
            TensorSpec(prefix + ".dt_bias", (H * D,), VECTOR),
            TensorSpec(prefix + ".g1", (self.rank_g, E)), TensorSpec(prefix + ".g2", (H * Dv, self.rank_g)),
            TensorSpec(prefix + ".o", (E, H * Dv)),
        ]

    def bind(self, prefix, tensors, rt):
        t = lambda n: tensors[prefix + n]
        self.w_in = torch.cat([t(".q"), t(".k"), t(".v"), t(".b")], dim=0).contiguous()
        self.w_low = torch.cat([t(".a1"), t(".g1")], dim=0).contiguous()
        self.w_a2, self.w_g2, self.wo = t(".a2"), t(".g2"), t(".o")
        self.conv_w = torch.cat([t(".q.conv"), t(".k.conv"), t(".v.conv")], dim=0).float().contiguous()
        self.a_log, self.dt_bias, self.norm_w = t(".A_log"), t(".dt_bias"), t(".norm")

    def first_weights(self):
        return [self.w_in]

    def forward(self, rt, h, batch, cache):
        H, G, D, Dv = self.n_heads, self.n_kv_heads, self.head_dim, self.v_head_dim
        proj = rt.linear(h, self.w_in, out_dtype=torch.float32)
        low = rt.linear(h, self.w_low)
        a_pre = rt.linear(low[:, :self.rank_a], self.w_a2, out_dtype=torch.float32)
        g_pre = rt.linear(low[:, self.rank_a:], self.w_g2, out_dtype=torch.float32)
        qkv_c, gb = ops.delta_prepare(proj, a_pre, self.conv_w, cache.state, self.state_floats, batch.seq_of_token,
                                      batch.seq_start, batch.slots, self.a_log, self.dt_bias, H, G, D, Dv)
        o = ops.delta_scan(qkv_c, gb, cache.state, batch.seq_start, batch.slots, H, G, D, Dv)
        y = ops.delta_output(o, self.norm_w, g_pre, self.eps, rt.dtype, H)
        return rt.linear(y, self.wo, partials_ok=True)


register_part("mixer", "channel_delta", ChannelDelta)
