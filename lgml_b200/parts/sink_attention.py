"""Attention with a sink, a distance bias, a window, a temperature on the queries, mixed
values and an output gate; keys and values have head sizes of their own.

For query head h of a token at position i (H heads on G key/value heads, head h reads
key/value head h // (H / G)):

    q, k, v = W h + b                 one fused product, with the gate's rows behind them
    q      <- q * (1 + coef * ln(floor((i + 1) / every) + 1))                  (``temperature``)
    v      <- (1 - lambda) v + lambda v_first                                  (``v_mix`` = "mix")
    s_j     = (q . k_j) * scale - slope_h * (i - j),  slope_h = 2^(-slope_base (h + 1) / H)
    w_j     = exp(s_j) / (exp(sink_h) + sum_j' exp(s_j'))      over 0 <= i - j < window
    out     = W_o ((sum_j w_j v_j) * sigmoid(W_g h))

``v_first`` is what the layer built with ``v_mix`` = "keep" computed for the same token in the
same step: that layer leaves its values in the step's ``shared`` table under ``v_mix_key`` and
the mixing layers read them there; the mixed values are what the cache holds.  The sink is a
learned number per head that only adds to the softmax's denominator.  Each constant is a
constructor argument; ``slope_base`` None, ``sink`` False, ``gate`` False, ``temperature`` None
switch a mechanism off.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import ops
from ..cache import PagedKV
from ..weights import VECTOR, TensorSpec
from .base import Part, register_part


class SinkAttention(Part):
    graph_safe = True

    def __init__(self, width: int, n_heads: int, n_kv_heads: int, head_dim: int, v_head_dim: int, scale: float,
                 window: Optional[int] = None, temperature: Optional[Tuple[float, int]] = None, slope_base: Optional[float] = 8.0,
                 sink: bool = True, gate: bool = True, bias: bool = True, v_mix: Optional[str] = None, v_mix_key: str = "v_first"):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads are no multiple of {n_kv_heads} KV heads")
        if v_mix not in (None, "keep", "mix"):
            raise ValueError(f"v_mix must be None, 'keep' or 'mix', not {v_mix!r}")
        self.width, self.n_heads, self.n_kv_heads = width, n_heads, n_kv_heads
        self.head_dim, self.v_head_dim = head_dim, v_head_dim
        self.scale = float(scale)
        self.window = int(window) if window else None
        self.temp_coef, self.temp_every = (float(temperature[0]), int(temperature[1])) if temperature else (0.0, 1)
        self.slope_base = slope_base
        self.has_sink, self.has_gate, self.bias = bool(sink), bool(gate), bool(bias)
        self.v_mix, self.v_mix_key = v_mix, v_mix_key
        self.w_in = self.b_in = self.wo = self.sinks = self.slopes = self.lam = None

    def cache_spec(self):
        return PagedKV(self.n_kv_heads, self.head_dim, self.window, self.v_head_dim)

    def tensor_specs(self, prefix):
        H, G, D, Dv, E = self.n_heads, self.n_kv_heads, self.head_dim, self.v_head_dim, self.width
        specs = [TensorSpec(prefix + ".q", (H * D, E)), TensorSpec(prefix + ".k", (G * D, E)), TensorSpec(prefix + ".v", (G * Dv, E)),
                 TensorSpec(prefix + ".o", (E, H * Dv))]
        if self.bias:
            specs += [TensorSpec(prefix + ".q.b", (H * D,), VECTOR), TensorSpec(prefix + ".k.b", (G * D,), VECTOR),
                      TensorSpec(prefix + ".v.b", (G * Dv,), VECTOR)]
        if self.has_gate:
            specs.append(TensorSpec(prefix + ".g", (H * Dv, E)))
        if self.has_sink:
            specs.append(TensorSpec(prefix + ".sink", (H,), VECTOR))
        # only a mixing layer reads the weight; the layer that keeps its values may carry one unread
        specs.append(TensorSpec(prefix + ".vmix", (), VECTOR, optional=self.v_mix != "mix", init=(0.5, 1.0)))
        return specs

    def bind(self, prefix, tensors, rt):
        H, Dv = self.n_heads, self.v_head_dim
        mats = [tensors[prefix + ".q"], tensors[prefix + ".k"], tensors[prefix + ".v"]]
        if self.has_gate:
            mats.append(tensors[prefix + ".g"])
        self.w_in = torch.cat(mats, dim=0).contiguous()
        if self.bias:
            vecs = [tensors[prefix + ".q.b"], tensors[prefix + ".k.b"], tensors[prefix + ".v.b"]]
            if self.has_gate:
                vecs.append(torch.zeros(H * Dv, dtype=torch.float32, device=vecs[0].device))
            self.b_in = torch.cat(vecs, dim=0).contiguous()
        self.wo = tensors[prefix + ".o"]
        self.sinks = tensors[prefix + ".sink"].contiguous() if self.has_sink else None
        if self.slope_base is not None:
            self.slopes = torch.tensor([2.0 ** (-float(self.slope_base) * (h + 1) / H) for h in range(H)], dtype=torch.float64) \
                .to(torch.float32).to(rt.device)
        if self.v_mix == "mix":
            self.lam = tensors[prefix + ".vmix"].reshape(1).contiguous()

    def first_weights(self):
        return [self.w_in]

    def forward(self, rt, h, batch, cache):
        H, G, D, Dv = self.n_heads, self.n_kv_heads, self.head_dim, self.v_head_dim
        n = h.shape[0]
        proj = rt.linear(h, self.w_in, bias=self.b_in, out_dtype=torch.float32)
        v_mode, kept = 0, None
        if self.v_mix == "keep":
            kept = batch.shared[self.v_mix_key] = torch.empty((n, G * Dv), dtype=torch.float32, device=h.device)
            v_mode = 1
        elif self.v_mix == "mix":
            kept = batch.shared.get(self.v_mix_key)
            if kept is None:
                raise RuntimeError("a value-mixing layer ran before the layer that keeps the values")
            v_mode = 2
        q = ops.sink_qkv_store(proj, batch.positions, batch.seq_of_token, cache.block_table, cache.k, cache.v, H, rt.status,
                               temp_coef=self.temp_coef, temp_every=self.temp_every, v_mode=v_mode, v_keep=kept, v_lambda=self.lam,
                               write_kv=cache.writable)
        lo = H * D + G * (D + Dv)
        gate = proj[:, lo:lo + H * Dv] if self.has_gate else None
        o = torch.empty((n, H * Dv), dtype=h.dtype, device=h.device)
        rt.sink_attention(q, batch, cache, o, H, self.scale, self.window or 0, self.slopes, self.sinks, gate)
        return rt.linear(o, self.wo, partials_ok=True)


register_part("mixer", "sink_attention", SinkAttention)
