"""Differential attention: every head holds two attention maps over the same values and outputs
their difference, normed per head.

For query head h (H heads on G key/value heads; head h reads key/value head h // (H / G)):

    q1 | q2 = W_q h   (2 D per head),   k1 | k2 = W_k h   (2 D per key head),   v = W_v h   (Dv per key head)
    a_m     = softmax_j((q_m . k_m,j) * scale) v_j        over the visible j, m = 1, 2
    lambda  = exp(lq1 . lk1) - exp(lq2 . lk2) + diff       one number for the layer
    o       = a_1 - lambda a_2;   o <- o / sqrt(mean(o^2) + eps) * (1 - diff)
    out     = W_o [o of every head]

Visible: j <= i and (i - j < ``window`` or j < ``keep_first``); without a window every j <= i.  No
position encoding.  The two maps are two key heads of one value head: the cache holds keys as
2 G heads of D and values as G heads of Dv, the queries run as 2 H heads in the order (key head, map,
head of the group), so that the masked attention kernels see plain grouped heads, and a small kernel
combines the maps.  A layer built with ``own_kv`` False has no key and value projections: it reads
the cache another layer wrote (``cache.writable`` False), with its own queries and mask.

``cache_window`` / ``cache_keep_first``: what the cache has to keep when other layers with wider
masks read it (default: this layer's own mask).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import ops
from ..cache import PagedKV
from ..weights import VECTOR, TensorSpec
from .base import Part, register_part

_OWN = object()


class DifferentialAttention(Part):
    graph_safe = True

    def __init__(self, width: int, n_heads: int, n_kv_heads: int, head_dim: int, v_head_dim: int, scale: float, diff: float, eps: float,
                 window: Optional[int] = None, keep_first: int = 0, own_kv: bool = True, cache_window=_OWN, cache_keep_first=_OWN):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads are no multiple of {n_kv_heads} KV heads")
        self.width, self.n_heads, self.n_kv_heads = width, n_heads, n_kv_heads
        self.head_dim, self.v_head_dim = head_dim, v_head_dim
        self.scale, self.diff, self.eps = float(scale), float(diff), float(eps)
        self.window = int(window) if window else None
        self.keep_first = int(keep_first) if self.window else 0
        self.own_kv = bool(own_kv)
        self.cache_window = self.window if cache_window is _OWN else (int(cache_window) if cache_window else None)
        self.cache_keep_first = self.keep_first if cache_keep_first is _OWN else int(cache_keep_first or 0)
        self.w_in = self.wo = None
        self.lam = 0.0

    def cache_spec(self):
        if not self.own_kv:
            return None
        return PagedKV(2 * self.n_kv_heads, self.head_dim, self.cache_window, self.v_head_dim,
                       keep_first=self.cache_keep_first if self.cache_window else 0, v_heads=self.n_kv_heads)

    def tensor_specs(self, prefix):
        H, G, D, Dv, E = self.n_heads, self.n_kv_heads, self.head_dim, self.v_head_dim, self.width
        specs = [TensorSpec(prefix + ".q", (H * 2 * D, E)), TensorSpec(prefix + ".o", (E, H * Dv))]
        if self.own_kv:
            specs += [TensorSpec(prefix + ".k", (G * 2 * D, E)), TensorSpec(prefix + ".v", (G * Dv, E))]
        specs += [TensorSpec(prefix + "." + n, (D,), VECTOR) for n in ("lq1", "lk1", "lq2", "lk2")]
        return specs

    def bind(self, prefix, tensors, rt):
        H, G, D, E = self.n_heads, self.n_kv_heads, self.head_dim, self.width
        per = H // G
        # query rows (head, map, d) -> (key head, map, head of the group, d)
        wq = tensors[prefix + ".q"].view(G, per, 2, D, E).permute(0, 2, 1, 3, 4).reshape(H * 2 * D, E)
        mats = [wq] + ([tensors[prefix + ".k"], tensors[prefix + ".v"]] if self.own_kv else [])
        self.w_in = torch.cat(mats, dim=0).contiguous()
        self.wo = tensors[prefix + ".o"]
        l = {n: tensors[prefix + "." + n].double().cpu() for n in ("lq1", "lk1", "lq2", "lk2")}
        self.lam = math.exp(float((l["lq1"] * l["lk1"]).sum())) - math.exp(float((l["lq2"] * l["lk2"]).sum())) + self.diff

    def first_weights(self):
        return [self.w_in]

    def forward(self, rt, h, batch, cache):
        H, G, Dv = self.n_heads, self.n_kv_heads, self.v_head_dim
        if cache.writable != self.own_kv:
            raise RuntimeError("a differential attention layer without projections of its own needs another layer's cache, and one with them its own")
        n = h.shape[0]
        proj = rt.linear(h, self.w_in, out_dtype=torch.float32)
        q = ops.sink_qkv_store(proj, batch.positions, batch.seq_of_token, cache.block_table, cache.k, cache.v, 2 * H, rt.status,
                               write_kv=cache.writable)
        maps = torch.empty((n, 2 * H * Dv), dtype=torch.float32, device=h.device)
        rt.sink_attention(q, batch, cache, maps, 2 * H, self.scale, self.window or 0, None, None, None, keep_first=self.keep_first)
        o = torch.empty((n, H * Dv), dtype=h.dtype, device=h.device)
        ops.diff_combine(maps, o, H, G, self.lam, self.eps, 1.0 - self.diff)
        return rt.linear(o, self.wo, partials_ok=True)


register_part("mixer", "differential_attention", DifferentialAttention)
