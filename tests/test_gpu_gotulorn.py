"""Gotulorn in the engine against the plain implementation: every mechanism alone, then whole models
under every way of cutting the work.

The models are small and differ from each other in every size and option (grouped heads, sizes that
are no multiple of 8, windows of 1 to 130 with 0 to 70 kept first tokens, layers that read another
layer's keys under a wider or a narrower mask, 1 to 8 experts with 1 to all of them chosen, layers
without a feed-forward).  Weights and, in the kernel tests, inputs are made so that the mechanism
under test decides the result: the keys at a window's edge and at the edge of the kept first tokens
carry the largest scores, a far key outweighs hundreds of near ones.
"""
import json
import math
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests import gotulorn_helpers as L
from tests import helpers as H
from tests.plain import gotulorn_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = Path(__file__).resolve().parent.parent
F64 = torch.float64
TOL = {"float32": dict(atol=3e-5, rtol=2e-4), "bfloat16": dict(atol=3e-2, rtol=8e-2)}


# ---------------------------------------------------------------------------------------------
# kernels alone
# ---------------------------------------------------------------------------------------------

def paged(T, Hk, D, Hv, Dv, dtype, seed=0):
    """Empty pages for one request of T tokens whose block table is a shuffle, so that a page lookup
    that ignores the table reads another page."""
    n_blocks = -(-T // 64)
    g = torch.Generator().manual_seed(seed)
    order = torch.randperm(n_blocks + 3, generator=g)[:n_blocks]
    k = torch.zeros(n_blocks + 3, Hk, 64, D, dtype=dtype, device=DEV)
    v = torch.zeros(n_blocks + 3, Hv, 64, Dv, dtype=dtype, device=DEV)
    return k, v, order.to(torch.int32).view(1, -1).contiguous().to(DEV)


def plain_masked(q, k, v, scale, window, keep_first):
    """q [T, Hq, D], k [T, Hk, D], v [T, Hv, Dv] -> [T, Hq, Dv]; query head h reads key head h // (Hq / Hk),
    key head g reads value head g // (Hk / Hv)."""
    T, Hq, _ = q.shape
    Hk, Hv = k.shape[1], v.shape[1]
    see = P.window_with_first(T, window, keep_first) if window else P.causal(T)
    out = np.zeros((T, Hq, v.shape[2]))
    for h in range(Hq):
        g = h // (Hq // Hk)
        s = (q[:, h].numpy() @ k[:, g].numpy().T) * scale
        out[:, h] = P.softmax_rows(s, see) @ v[:, g // (Hk // Hv)].numpy()
    return torch.from_numpy(out)


def run_masked(q, k, v, scale, window, keep_first, dtype, form="general", out_dtype=None):
    """The same through sink_qkv_store and one form of the masked attention kernels."""
    from lgml_b200 import ops

    T, Hq, D = q.shape
    Hk, Hv, Dv = k.shape[1], v.shape[1], v.shape[2]
    proj = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], 1).float().to(DEV).contiguous()
    kp, vp, table = paged(T, Hk, D, Hv, Dv, dtype)
    positions = torch.arange(T, dtype=torch.int32, device=DEV)
    seq = torch.zeros(T, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    qd = ops.sink_qkv_store(proj, positions, seq, table, kp, vp, Hq, status)
    out = torch.empty(T, Hq * Dv, dtype=out_dtype or dtype, device=DEV)
    if form == "split":
        ops.sink_decode(qd, positions, seq, table, kp, vp, out, Hq, scale, window or 0, status, 3, keep_first=keep_first)
    elif form == "mma":
        tiles = torch.tensor([[0, r0, min(64, T - r0), 0] for r0 in range(0, T, 64)], dtype=torch.int32, device=DEV)
        ops.sink_attention_mma(qd, positions, tiles, table, kp, vp, out, Hq, scale, window or 0, status, keep_first=keep_first)
    else:
        ops.sink_attention(qd, positions, seq, table, kp, vp, out, Hq, scale, window or 0, status, keep_first=keep_first)
    assert int(status.item()) == 0
    return out.double().cpu().view(T, Hq, Dv)


FORMS = [(torch.float32, "general"), (torch.bfloat16, "general"), (torch.bfloat16, "mma"), (torch.bfloat16, "split")]


@pytest.mark.parametrize("dtype,form", FORMS)
@pytest.mark.parametrize("window,keep", [(None, 0), (1, 1), (5, 2), (64, 64), (70, 3), (129, 70), (20, 0)])
@pytest.mark.parametrize("sizes", [(24, 10), (64, 32)])
def test_masked_attention_edges_of_the_window_and_of_the_kept_tokens(dtype, form, window, keep, sizes):
    """6 query heads on 2 key heads on 1 value head, D != Dv, 260 tokens on shuffled pages.  For every
    query the key at distance window - 1 (the last one inside) and the one at distance window (the first
    one outside) get scores far above the rest, and so do the last kept token and the first one that is
    not kept; without a window key 3 outweighs the hundreds after it."""
    torch.manual_seed(1)
    T, Hq, Hk, Hv, (D, Dv) = 260, 6, 2, 1, sizes
    q = torch.randn(T, Hq, D, dtype=F64) * 0.3
    k = torch.randn(T, Hk, D, dtype=F64) * 0.3
    v = torch.randn(T, Hv, Dv, dtype=F64)
    q[:, :, 0] = 1.0          # channel 0 of key j says how much every query likes it
    k[:, :, 0] = 0.0
    if window is None:
        k[3, :, 0] = 40.0
    else:
        for j in range(T):    # a sawtooth over a key's age as the last query sees it: the window's edge ranks highest
            k[j, :, 0] = 20.0 * ((T - 1 - j) % (window + 1)) / (window + 1)
        if keep:
            k[keep - 1, :, 0] = 21.0
        k[keep, :, 0] = 22.0
    if dtype == torch.bfloat16:
        q, k, v = (t.to(torch.bfloat16).double() for t in (q, k, v))
    got = run_masked(q, k, v, 0.7, window, keep, dtype, form)
    want = plain_masked(q, k, v, 0.7, window, keep)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert float((got - want).abs().max()) < tol, float((got - want).abs().max())
    if window not in (None, 1):
        # the test has teeth: one key more or less, in the window or among the kept, moves the result by far more
        for w2, k2 in ((window + 1, keep), (window - 1, keep), (window, keep + 1)) + (((window, keep - 1),) if keep else ()):
            other = plain_masked(q, k, v, 0.7, w2, k2)
            assert float((other - want).abs().max()) > 5 * tol, (w2, k2)


@pytest.mark.parametrize("D,Dv", [(40, 24), (300, 288)])
def test_masked_attention_float32_output_and_values_inside_the_key_cells(D, Dv):
    """bfloat16 keys with a float32 result, and values that are the first Dv entries of the key cells; also at
    cell sizes beyond what the split and tensor-core forms take."""
    from lgml_b200 import ops

    torch.manual_seed(3)
    T, Hq = 150, 3
    q = (torch.randn(T, Hq, D, dtype=F64) * 0.4 * (40 / D) ** 0.5).to(torch.bfloat16).double()
    k = (torch.randn(T, 1, D, dtype=F64)).to(torch.bfloat16).double()
    for dtype in (torch.float32, torch.bfloat16):
        kp, _, table = paged(T, 1, D, 1, 1, dtype)
        positions = torch.arange(T, dtype=torch.int32, device=DEV)
        seq = torch.zeros(T, dtype=torch.int32, device=DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        for t in range(T):
            kp[int(table[0, t // 64]), 0, t % 64] = k[t, 0].to(dtype).to(DEV)
        out = torch.empty(T, Hq * Dv, dtype=torch.float32, device=DEV)
        ops.sink_attention(q.reshape(T, -1).to(dtype).to(DEV), positions, seq, table, kp, kp[..., :Dv], out, Hq, 0.3, 0, status)
        assert int(status.item()) == 0
        want = plain_masked(q, k, k[:, :, :Dv], 0.3, None, 0)
        assert float((out.double().cpu().view(T, Hq, Dv) - want).abs().max()) < (2e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hh,G,Dv", [(4, 2, 24), (1, 1, 12), (6, 1, 130), (5, 5, 64)])
def test_diff_combine(dtype, Hh, G, Dv):
    from lgml_b200 import ops

    torch.manual_seed(4)
    T, lam, eps, diff = 37, 0.83, 1e-5, 0.3
    a = torch.randn(T, Hh, 2, Dv, dtype=F64)                         # (head, map)
    per = Hh // G
    # the kernel's order: (key head, map, head of the group)
    packed = a.view(T, G, per, 2, Dv).permute(0, 1, 3, 2, 4).reshape(T, 2 * Hh * Dv).float().contiguous().to(DEV)
    out = torch.empty(T, Hh * Dv, dtype=dtype, device=DEV)
    ops.diff_combine(packed, out, Hh, G, lam, eps, 1.0 - diff)
    o = a[:, :, 0].float().double() - lam * a[:, :, 1].float().double()
    want = torch.from_numpy(P.rms_unit(o.numpy(), eps)) * (1.0 - diff)
    assert float((out.double().cpu().view(T, Hh, Dv) - want).abs().max()) < (1e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(3, 16, 8, 12, 24, 8), (1, 12, 2, 20, 10, 2), (2, 24, 12, 20, 40, 8), (4, 32, 32, 32, 96, 32)])
def test_latent_attention_through_its_kernels(dtype, shape):
    """The latent's norm, the rotation of the shared key part and of the queries, both products per head
    and attention over the cached [c | r] cells, against the plain form that builds keys and values of
    every head; the portion starts at position 4,990 (angles of thousands of radians) after a first
    portion of 4,990 tokens was cached (only its last cells matter: the far keys are made to show)."""
    from lgml_b200 import ops

    Hh, D, Dr, Dv, R, dims = shape
    torch.manual_seed(5)
    E, T = 48, 200
    m = {"heads": Hh, "dim": D, "rot_dim": Dr, "vdim": Dv, "kv_rank": R, "scale": 0.3, "rot": {"base": 1000.0, "dims": dims}}
    bf = lambda t: t.to(torch.bfloat16).double()
    W = {"x.q": bf(torch.randn(Hh * (D + Dr), E, dtype=F64) * 0.15), "x.dkv": bf(torch.randn(R + Dr, E, dtype=F64) * 0.3),
         "x.dkv.norm": bf(1.0 + 0.2 * torch.randn(R, dtype=F64)), "x.uk": bf(torch.randn(Hh * D, R, dtype=F64) * 0.3),
         "x.uv": bf(torch.randn(Hh * Dv, R, dtype=F64) * 0.3), "x.o": torch.eye(Hh * Dv, dtype=F64)}
    h = bf(torch.randn(T, E, dtype=F64))
    eps = 1e-5
    want = torch.from_numpy(P.latent_attention(h.numpy(), {n: t.numpy() for n, t in W.items()}, "x", m, eps))
    tol = 3e-5 if dtype == torch.float32 else 2e-2 * (1.0 + float(want.abs().max()))

    def chain(pos0_of_portion):
        kp, _, table = paged(T, 1, R + Dr, 1, 1, dtype, seed=2)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        exact = torch.tensor([1000.0 ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
        hi = exact.float()
        inv_freq = torch.stack([hi, (exact - hi.double()).float()]).contiguous().to(DEV)
        outs = []
        for a, b in pos0_of_portion:
            n = b - a
            positions = torch.arange(a, b, dtype=torch.int32, device=DEV)
            seq = torch.zeros(n, dtype=torch.int32, device=DEV)
            hp = h[a:b].float().to(DEV)
            qp = (hp @ W["x.q"].float().to(DEV).T).contiguous()
            dk = (hp @ W["x.dkv"].float().to(DEV).T).contiguous()
            q_plain, q_full = ops.latent_prepare(qp, dk, W["x.dkv.norm"].float().to(DEV), eps, inv_freq, dims, positions, seq, table, kp, Hh, D,
                                                 Dr, R, status)
            ops.head_linear(q_plain, W["x.uk"].view(Hh, D, R).transpose(1, 2).contiguous().to(dtype).to(DEV), q_full, D, R + Dr)
            mix = torch.empty(n, Hh * R, dtype=dtype, device=DEV)
            ops.sink_attention(q_full, positions, seq, table, kp, kp[..., :R], mix, Hh, 0.3, 0, status)
            o = torch.empty(n, Hh * Dv, dtype=dtype, device=DEV)
            ops.head_linear(mix, W["x.uv"].view(Hh, Dv, R).contiguous().to(dtype).to(DEV), o, R, Dv)
            outs.append(o.double().cpu())
        assert int(status.item()) == 0
        return torch.cat(outs)

    assert float((chain([(0, T)]) - want).abs().max()) < tol
    assert float((chain([(0, 3), (3, 5), (5, 130), (130, T)]) - want).abs().max()) < tol


def test_rotation_far_from_the_start_keeps_its_angle():
    """Positions in the thousands: the rotated parts of the cell and of the queries against float64 angles."""
    from lgml_b200 import ops

    torch.manual_seed(6)
    Hh, D, Dr, R, dims, T, pos0 = 2, 8, 16, 8, 12, 40, 70000
    qp = torch.randn(T, Hh * (D + Dr), dtype=torch.float32, device=DEV)
    dk = torch.randn(T, R + Dr, dtype=torch.float32, device=DEV)
    n_blocks = (pos0 + T) // 64 + 1
    kp = torch.zeros(2, 1, 64, R + Dr, dtype=torch.float32, device=DEV)
    table = torch.full((1, n_blocks), -1, dtype=torch.int32, device=DEV)
    table[0, pos0 // 64], table[0, pos0 // 64 + 1] = 1, 0
    positions = torch.arange(pos0, pos0 + T, dtype=torch.int32, device=DEV)
    seq = torch.zeros(T, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    exact = torch.tensor([50000.0 ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    hi = exact.float()
    inv_freq = torch.stack([hi, (exact - hi.double()).float()]).contiguous().to(DEV)
    _, q_full = ops.latent_prepare(qp, dk, torch.ones(R, device=DEV), 1e-5, inv_freq, dims, positions, seq, table, kp, Hh, D, Dr, R, status)
    assert int(status.item()) == 0
    pos = np.arange(pos0, pos0 + T)
    want_q = P.rotate_interleaved(qp.double().cpu().view(T, Hh, D + Dr)[:, :, D:].numpy(), 50000.0, dims, pos)
    got_q = q_full.double().cpu().view(T, Hh, R + Dr)[:, :, R:].numpy()
    assert np.abs(got_q - want_q).max() < 3e-6
    want_k = P.rotate_interleaved(dk.double().cpu()[:, R:].numpy(), 50000.0, dims, pos)
    got_k = np.stack([kp[int(table[0, p // 64]), 0, p % 64, R:].double().cpu().numpy() for p in pos])
    assert np.abs(got_k - want_k).max() < 3e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dynamic_tanh_and_clamped_gate(dtype):
    from lgml_b200 import ops

    torch.manual_seed(7)
    for width in (36, 64, 1001):
        x = torch.randn(19, width, dtype=torch.float32, device=DEV) * 3
        d = torch.randn(19, width, dtype=torch.float32, device=DEV).to(dtype)
        w, b = torch.randn(width, device=DEV), torch.randn(width, device=DEV)
        alpha = torch.tensor([0.37], device=DEV)
        want_sum = x.double() + d.double()
        want = torch.from_numpy(P.dyt(2.5 * want_sum.cpu().numpy(), w.double().cpu().numpy(), b.double().cpu().numpy(), 0.37))
        out = torch.empty(19, width, dtype=dtype, device=DEV)
        x2 = x.clone()
        ops.dyt_norm(x2, w, b, alpha, out, delta=d, pre_scale=2.5)
        assert float((x2.double() - want_sum).abs().max()) < 1e-6                    # the sum stays in x
        assert float((out.double().cpu() - want).abs().max()) < (2e-6 if dtype == torch.float32 else 3e-2)
        rows = torch.tensor([5, 0, 18], dtype=torch.int32, device=DEV)
        out3 = torch.empty(3, width, dtype=torch.float32, device=DEV)
        ops.dyt_norm(x.clone(), w, b, alpha, out3, delta=d, rows=rows, pre_scale=2.5)
        assert float((out3.double().cpu() - want[[5, 0, 18]]).abs().max()) < 2e-6
    gu = (torch.randn(23, 2 * 50, device=DEV) * 3).to(dtype)
    act = torch.empty(23, 50, dtype=dtype, device=DEV)
    ops.glu_clamped(gu, act, 1.702, 1.5)
    g, u = gu[:, :50].double().cpu().clamp(max=1.5), gu[:, 50:].double().cpu().clamp(-1.5, 1.5)
    want = g * torch.sigmoid(1.702 * g) * (u + 1)
    assert float((act.double().cpu() - want).abs().max()) < (1e-5 if dtype == torch.float32 else 3e-2)
    assert float((gu.double().abs() > 1.5).double().mean()) > 0.3          # the clamp was at work


@pytest.mark.parametrize("M", [1, 7, 64, 65, 300])
def test_clamped_gate_in_the_products_epilogue(M):
    """The gate|up product with the clamped activation in its epilogue against the plain formula; both
    orientations of the product's tile and the pairs of CTAs (1 to 300 tokens)."""
    from lgml_b200 import ops

    torch.manual_seed(9 + M)
    K, F = 192, 136
    x = torch.randn(M, K, dtype=F64).to(torch.bfloat16)
    wg, wu = (torch.randn(F, K, dtype=F64) * 0.2).to(torch.bfloat16), (torch.randn(F, K, dtype=F64) * 0.2).to(torch.bfloat16)
    pairs = torch.stack([wg, wu], dim=1).reshape(2 * F, K).contiguous().to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    act = ops.gemm_bf16_glu_clamped(x.to(DEV), pairs, 1.702, 1.5, status)
    assert int(status.item()) == 0
    g, u = (x.double() @ wg.double().T).clamp(max=1.5), (x.double() @ wu.double().T).clamp(-1.5, 1.5)
    want = g * torch.sigmoid(1.702 * g) * (u + 1)
    assert float((act.double().cpu() - want).abs().max()) < 3e-2
    assert float(((x.double() @ wu.double().T).abs() > 1.5).double().mean()) > 0.2          # the clamp was at work


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("X,top,E,F", [(5, 2, 64, 24), (1, 1, 36, 20), (4, 4, 40, 12), (12, 3, 96, 40), (40, 6, 128, 64), (3, 2, 256, 520)])
def test_router_and_experts(dtype, X, top, E, F):
    """The chosen experts are those of the plain router (logits kept apart), ties go to the lower index, and
    the weighted sum of the experts' outputs is the plain one; 300 tokens, so that the grouped form runs too."""
    from lgml_b200 import ops

    torch.manual_seed(8)
    T = 300
    bf = lambda t: t.to(torch.bfloat16).double()
    W = {"f.router": bf(torch.randn(X, E, dtype=F64)), "f.router.b": bf(torch.randn(X, dtype=F64))}
    for e in range(X):
        W[f"f.e{e}.gate"], W[f"f.e{e}.up"], W[f"f.e{e}.down"] = (bf(torch.randn(F, E, dtype=F64) * 0.3), bf(torch.randn(F, E, dtype=F64) * 0.3),
                                                                 bf(torch.randn(E, F, dtype=F64) * 0.3))
    h = bf(torch.randn(T, E, dtype=F64))
    f = {"router": {"experts": X, "top": top}}
    want = torch.from_numpy(P.routed_ff(h.numpy(), {n: t.numpy() for n, t in W.items()}, "f", f))
    hd = h.to(dtype).to(DEV)
    ids, wts = ops.moe_router(hd, W["f.router"].float().to(DEV), W["f.router.b"].float().to(DEV), top)
    z = h @ W["f.router"].T + W["f.router.b"]
    assert torch.equal(ids.cpu().long(), torch.argsort(-z, dim=1, stable=True)[:, :top])
    w_gu = torch.stack([torch.stack([W[f"f.e{e}.gate"], W[f"f.e{e}.up"]], dim=1).reshape(2 * F, E) for e in range(X)]).to(dtype).to(DEV)
    w_down = torch.stack([W[f"f.e{e}.down"] for e in range(X)]).to(dtype).to(DEV)
    tol = (3e-5 if dtype == torch.float32 else 2e-2) * (1.0 + float(want.abs().max()))
    out = ops.moe_experts_rows(hd, ids, wts, w_gu, w_down)
    assert float((out.double().cpu() - want).abs().max()) < tol
    if dtype == torch.bfloat16 and ops.moe_grouped_supports(hd, w_gu):
        out2 = ops.moe_experts_grouped(hd, ids, wts, w_gu, w_down)
        assert float((out2.double().cpu() - want).abs().max()) < tol
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        out3 = ops.moe_experts_tcgen05(hd, ids, wts, w_gu, w_down, status)
        assert int(status.item()) == 0
        assert float((out3.double().cpu() - want).abs().max()) < tol
    # ties: equal logits go to the lower index
    ids2, wts2 = ops.moe_router(torch.zeros(3, E, dtype=dtype, device=DEV), W["f.router"].float().to(DEV), None, top)
    assert torch.equal(ids2.cpu(), torch.arange(top, dtype=torch.int32).expand(3, top))
    assert float((wts2 - 1.0 / top).abs().max()) < 1e-6


# ---------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------

@pytest.fixture(scope="module", params=sorted(L.CONFIGS))
def model(request, tmp_path_factory):
    cfg = L.CONFIGS[request.param]
    made = {}
    # float32 runs see attention sharpened (a wrong key moves the logits far past the tolerance);
    # bfloat16's own rounding of q and k would be amplified alike, so its models are left as drawn
    for dtype, sharpen in (("float32", 2.0), ("bfloat16", 1.0)):
        weights = L.random_weights(cfg, seed=11, sharpen=sharpen)
        made[dtype] = (weights, L.write_folder(tmp_path_factory.mktemp(f"{request.param}_{dtype}"), cfg, weights))
    return request.param, cfg, made


def make_runner(folder, dtype, n_pages, slots=4, **kw):
    from lgml_b200.engine.engine import parse_dtype
    from lgml_b200.engine.runner import ModelRunner

    return ModelRunner.from_folder(folder, parse_dtype(dtype), DEV, n_pages=n_pages, max_slots=slots, max_step_tokens=n_pages * 64, **kw)


def sequences(cfg, lens, seed=50, weights=None):
    """Random requests; with ``weights`` (the bfloat16 runs) such that no router decides by a close call."""
    if weights is not None:
        return {f"r{i}": L.clear_ids(cfg, weights, n, seed + i) for i, n in enumerate(lens)}
    return {f"r{i}": H.random_ids(n, cfg["vocab"], seed + i) for i, n in enumerate(lens)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_all_cuttings_match_the_plain_model(model, dtype):
    """Whole; the last 32 tokens one by one; portions down to two tokens; and up to three live requests
    with so few pages that pages are used again."""
    name, cfg, made = model
    weights, folder = made[dtype]
    seqs = sequences(cfg, [1, 5, 23, 64, 65, 97, 150, 201], weights=weights if dtype == "bfloat16" else None)
    results = {}
    for kind, trace in (("whole", H.trace_whole(seqs)), ("tail", H.trace_tail(seqs)), ("portions", H.trace_portions(seqs))):
        runner = make_runner(folder, dtype, n_pages=4)
        results[kind] = H.run_trace(runner, trace)
        assert all(g.pool.n_held == 0 for g in runner.cache.groups)
    trace = H.trace_mixed(seqs, max_tokens=64 * 7, seed=5, max_live=3)
    assert max(len(st["entries"]) for st in trace) >= 3
    runner = make_runner(folder, dtype, n_pages=7, slots=3)
    results["mixed"] = H.run_trace(runner, trace)
    assert all(g.pool.taken_total > g.pool.n_pages for g in runner.cache.groups if g.spec.window is None), "no page was used twice"
    for kind, got in results.items():
        worst = L.compare(got, cfg, weights, seqs, **TOL[dtype])
        print(f"{name} {dtype} {kind}: max |diff| {worst:.3g}")
    if dtype == "float32":
        for kind in ("tail", "portions", "mixed"):
            for key, row in results["whole"].items():
                assert torch.equal(row, results[kind][key]), f"float32 {kind} differs from whole at {key}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_then_long_decoding_over_every_window(model, dtype):
    """Three tokens of prompt, then 230 tokens one by one (through captured steps): every window of the
    models (1 to 130) passes over decoded tokens while the kept first tokens stay, also where they fill
    more than a page."""
    name, cfg, made = model
    weights, folder = made[dtype]
    seqs = sequences(cfg, [233], seed=70, weights=weights if dtype == "bfloat16" else None)
    runner = make_runner(folder, dtype, n_pages=4)
    got = H.run_trace(runner, H.trace_tail(seqs, tail=230))
    assert runner.graph_replays > 100
    L.compare(got, cfg, weights, seqs, **TOL[dtype])


def test_a_window_gives_its_pages_back_but_not_those_of_the_kept_tokens(model):
    name, cfg, made = model
    weights, folder = made["float32"]
    runner = make_runner(folder, "float32", n_pages=12)
    seqs = sequences(cfg, [700], seed=75)
    req = runner.open("a")
    ids = seqs["r0"]
    for a in range(0, 700, 50):
        runner.step([(req, ids[a:a + 50], [])])
    for g, table in zip(runner.cache.groups, req.tables):
        if g.spec.window is None:
            assert all(p >= 0 for p in table)
            continue
        kept = -(-g.spec.keep_first // 64)
        first = max(0, 700 - g.spec.window + 1) // 64
        assert all(p >= 0 for p in table[:kept]) and all(p < 0 for p in table[kept:first]) and all(p >= 0 for p in table[max(kept, first):])
    row = runner.step([(req, [ids[0]], [0])])
    want = L.oracle_logits(cfg, weights, ids + [ids[0]])[-1]
    assert float((row[0].double().cpu() - want).abs().max()) < 3e-5 + 2e-4 * float(want.abs().max())
    runner.close(req)
    runner.cache.check()


def test_batch_of_unequal_requests_equals_each_alone(model):
    name, cfg, made = model
    weights, folder = made["float32"]
    seqs = sequences(cfg, [90, 3, 41, 1], seed=120)
    runner = make_runner(folder, "float32", n_pages=8)
    alone = H.run_trace(runner, H.trace_whole(seqs))
    together = H.run_trace(runner, [{"step": 0, "entries": [{"id": r, "tokens": ids, "want": list(range(len(ids)))} for r, ids in seqs.items()],
                                     "end": list(seqs)}])
    for key, row in alone.items():
        assert torch.equal(row, together[key])
    L.compare(together, cfg, weights, seqs, **TOL["float32"])


def test_many_tokens_take_the_grouped_experts_and_the_tensor_core_attention(model):
    """A portion of 290 tokens beside a decoded token, bfloat16: the step's experts run in the grouped form and
    its attention on tensor cores where the head sizes allow; then the same request goes on token by token."""
    name, cfg, made = model
    weights, folder = made["bfloat16"]
    seqs = sequences(cfg, [320, 80], seed=140, weights=weights)
    runner = make_runner(folder, "bfloat16", n_pages=16)
    a, b = runner.open("r0"), runner.open("r1")
    got = {}
    rows = runner.step([(b, seqs["r1"][:70], [69])]).float().cpu()
    got[("r1", 69)] = rows[0]
    rows = runner.step([(a, seqs["r0"][:290], list(range(0, 290, 7))), (b, seqs["r1"][70:71], [0])]).float().cpu()
    for i, p in enumerate(range(0, 290, 7)):
        got[("r0", p)] = rows[i]
    got[("r1", 70)] = rows[-1]
    for p in range(290, 320):
        q = 71 + p - 290
        entries = [(a, [seqs["r0"][p]], [0])] + ([(b, [seqs["r1"][q]], [0])] if q < 80 else [])
        rows = runner.step(entries).float().cpu()
        got[("r0", p)] = rows[0]
        if len(entries) > 1:
            got[("r1", q)] = rows[1]
    runner.rt.check_status()
    L.compare(got, cfg, weights, seqs, **TOL["bfloat16"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(model, dtype):
    """Engine.generate (scheduler, portions of 16 prompt tokens, sampling on the device, steps run ahead)
    and Engine.greedy against greedy decoding with the plain model."""
    import lgml_b200

    name, cfg, made = model
    weights, folder = made[dtype]
    prompts = [L.clear_ids(cfg, weights, n, 200 + n) if dtype == "bfloat16" else H.random_ids(n, cfg["vocab"], 200 + n) for n in (37, 5, 70)]
    eng = lgml_b200.Engine(str(folder), dtype=dtype, n_ctx=256, slots=2, ubatch=16)
    outs = eng.generate(prompts, max_tokens=10, temperature=0.0, stop=[])
    solo, _ = eng.greedy(prompts[0], 10)
    for prompt, got in zip(prompts, outs):
        assert len(got) == 10
        checked = 0
        for i, tok in enumerate(got):
            if dtype == "bfloat16":
                # a generated token may bring a close call between two experts, which bfloat16 may decide the other way: stop there
                gaps = []
                P.forward(cfg, L.as_numpy(weights), prompt + got[:i], router_gaps=gaps)
                if gaps and float(np.min(np.stack(gaps))) < 0.3:
                    break
            row = L.oracle_logits(cfg, weights, prompt + got[:i])[-1]
            gap = float(row.max() - row[tok])
            bound = 0.0 if dtype == "float32" and gap > 1e-4 else (1e-4 if dtype == "float32" else 5e-2 * float(row.abs().max()))
            assert gap <= bound, f"{dtype}: token {i} is {tok}, the plain model prefers {int(row.argmax())} by {gap:.3g}"
            checked += 1
        assert checked >= 1
    if dtype == "float32":
        assert solo == outs[0]


@pytest.mark.parametrize("variant", ["float32", "bfloat16-switches"])
def test_trace_run_as_a_process(model, tmp_path, variant):
    """bin/trace_run as a process on a mixed trace; in bfloat16 with the older of each pair of implementations switched on
    (the experts' tiles on mma.sync, the clamped gate as a kernel of its own)."""
    import os

    name, cfg, made = model
    dtype = variant.split("-")[0]
    weights, folder = made[dtype]
    seqs = sequences(cfg, [70, 20, 131], seed=300, weights=weights if dtype == "bfloat16" else None)
    trace = H.trace_mixed(seqs, max_tokens=64 * 4, seed=2, max_live=2)
    out = tmp_path / "out"
    env = dict(os.environ)
    if variant.endswith("switches"):
        env.update(LGML_MOE_GROUPED="mma", LGML_GLU_FUSED="0")
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out),
                           "--max-tokens", str(64 * 4)], input="\n".join(json.dumps(s) for s in trace) + "\n", text=True,
                          capture_output=True, timeout=600, env=env)
    assert proc.returncode == 0, proc.stderr[-2000:]
    done = [ln for ln in proc.stdout.splitlines() if ln.startswith("done ")]
    assert done == [f"done {s['step']}" for s in trace]
    got, fed = {}, {r: 0 for r in seqs}
    for st in trace:
        rows = np.fromfile(out / f"{st['step']}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
        r = 0
        for e in st["entries"]:
            for i in e["want"]:
                got[(e["id"], fed[e["id"]] + i)] = torch.from_numpy(rows[r].copy())
                r += 1
            fed[e["id"]] += len(e["tokens"])
        assert r == rows.shape[0]
    L.compare(got, cfg, weights, seqs, **TOL[dtype])


def test_command_line_generates_with_the_folders_architecture(model):
    name, cfg, made = model
    weights, folder = made["float32"]
    prompt = H.random_ids(19, cfg["vocab"], 400)
    proc = subprocess.run([sys.executable, "-m", "lgml_b200", "-m", str(folder), "--dtype", "float32", "--prompt-ids", ",".join(map(str, prompt)),
                           "-n", "5", "--temperature", "0", "--repeat-stop", "0"], capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert proc.returncode == 0, proc.stderr[-2000:]
    got = [int(t) for t in proc.stdout.strip().splitlines()[-1].split(",")]
    assert len(got) == 5
    for i, tok in enumerate(got):
        row = L.oracle_logits(cfg, weights, prompt + got[:i])[-1]
        assert float(row.max() - row[tok]) <= 1e-4
