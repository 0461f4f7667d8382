"""Lefulorn in the engine against the plain implementation: every mechanism alone, then whole
models under every way of cutting the work.

The models are small and differ from each other in every size and option (grouped heads, key
and value sizes that are no multiple of 8, windows below a page, across pages and none, a
value-mixing chain that starts in the middle, layers with and without a feed-forward, filters
of one to five taps).  Weights and, in the kernel tests, inputs are made so that the mechanism
under test decides the result: a key just inside a window and one just outside it carry the
largest scores, a far key outweighs hundreds of near ones, the sink holds a visible share.
"""
import json
import math
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from tests import helpers as H
from tests import lefulorn_helpers as L
from tests.plain import lefulorn_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = Path(__file__).resolve().parent.parent
F64 = torch.float64
TOL = {"float32": dict(atol=3e-5, rtol=2e-4), "bfloat16": dict(atol=3e-2, rtol=5e-2)}


# ---------------------------------------------------------------------------------------------
# kernels alone
# ---------------------------------------------------------------------------------------------

def paged(T, G, D, Dv, dtype, seed=0):
    """Empty pages for one request of T tokens whose block table is a shuffle, so that a page
    lookup that ignores the table reads another page."""
    n_blocks = -(-T // 64)
    g = torch.Generator().manual_seed(seed)
    order = torch.randperm(n_blocks + 3, generator=g)[:n_blocks]
    k = torch.zeros(n_blocks + 3, G, 64, D, dtype=dtype, device=DEV)
    v = torch.zeros(n_blocks + 3, G, 64, Dv, dtype=dtype, device=DEV)
    table = order.to(torch.int32).view(1, -1).contiguous().to(DEV)
    return k, v, table


def run_sink_attention(q, k, v, sink, scale, window, dtype, temp=None, gate=None, keep_mode=0, kept=None, lam=None, pos0=0, mma=False):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] (float64) through sink_qkv_store and sink_attention."""
    from lgml_b200 import ops

    T, Hh, D = q.shape
    G, Dv = k.shape[1], v.shape[2]
    proj = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], 1).float().to(DEV).contiguous()
    kp, vp, table = paged(pos0 + T, G, D, Dv, dtype)
    positions = torch.arange(pos0, pos0 + T, dtype=torch.int32, device=DEV)
    seq = torch.zeros(T, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    qd = ops.sink_qkv_store(proj, positions, seq, table, kp, vp, Hh, status, temp_coef=temp[0] if temp else 0.0,
                            temp_every=temp[1] if temp else 1, v_mode=keep_mode, v_keep=kept, v_lambda=lam)
    out = torch.empty(T, Hh * Dv, dtype=dtype, device=DEV)
    slopes = P.distance_slopes(Hh).float().to(DEV)
    if mma == "split":      # the split form for decoding, here on every token of the run
        ops.sink_decode(qd, positions, seq, table, kp, vp, out, Hh, scale, window or 0, status, 3, slopes=slopes,
                        sinks=sink.float().to(DEV), gate=gate)
    elif mma == "twin":      # the two-tile tcgen05 form: tiles of 2 x (128 rows / heads of a KV head) tokens
        tt = ops.prefill_twin_tile_tokens(Hh, G)
        tiles = torch.tensor([[0, r0, min(tt, T - r0), 0] for r0 in range(0, T, tt)], dtype=torch.int32, device=DEV)
        assert ops.sink_twin_supports(qd, out, kp, vp, gate)
        ops.sink_attention_twin(qd, positions, tiles, table, kp, vp, out, Hh, scale, window or 0, status, slopes=slopes,
                                sinks=sink.float().to(DEV), gate=gate)
    elif mma:     # the tensor-core form: tiles of at most 64 tokens, here 64, 64, ..., and the rest
        tiles = torch.tensor([[0, r0, min(64, T - r0), 0] for r0 in range(0, T, 64)], dtype=torch.int32, device=DEV)
        ops.sink_attention_mma(qd, positions, tiles, table, kp, vp, out, Hh, scale, window or 0, status, slopes=slopes,
                               sinks=sink.float().to(DEV), gate=gate)
    else:
        ops.sink_attention(qd, positions, seq, table, kp, vp, out, Hh, scale, window or 0, status, slopes=slopes,
                           sinks=sink.float().to(DEV), gate=gate)
    assert int(status.item()) == 0
    return out.double().cpu().view(T, Hh, Dv)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, "mma", "split"])
@pytest.mark.parametrize("window", [None, 1, 5, 64, 70, 129])
@pytest.mark.parametrize("sizes", [(24, 10), (64, 32)])
def test_sink_attention_edges_of_the_window_and_far_keys(dtype, window, sizes):
    """Grouped heads, D != Dv, 200 tokens on shuffled pages.  For every query the key at distance
    window - 1 (the last one inside) and the one at distance window (the first one outside) get
    scores far above the rest; without a window, key 3 outweighs the hundreds after it."""
    torch.manual_seed(1)
    mma, dtype = (dtype if isinstance(dtype, str) else False), (torch.bfloat16 if isinstance(dtype, str) else dtype)
    T, Hh, G, (D, Dv) = 200, 6, 2, sizes        # (64, 32): sizes the tensor-core decode form takes; (24, 10): its plain twin
    q = torch.randn(T, Hh, D, dtype=F64) * 0.3
    k = torch.randn(T, G, D, dtype=F64) * 0.3
    v = torch.randn(T, G, Dv, dtype=F64)
    # channel 0 of q is 1 everywhere; channel 0 of key j says how much every query likes it
    q[:, :, 0] = 1.0
    k[:, :, 0] = 0.0
    if window is None:
        k[3, :, 0] = 40.0
    else:
        # a sawtooth that grows with a key's age as the last query sees it and drops after window + 1
        # keys: for that query the oldest key inside the window and the one just outside it rank highest
        for j in range(T):
            k[j, :, 0] = 20.0 * ((T - 1 - j) % (window + 1)) / (window + 1)
    if dtype == torch.bfloat16:
        q, k, v = (t.to(torch.bfloat16).double() for t in (q, k, v))
    sink = torch.tensor([0.5, -1.0, 2.0, 0.0, 1.0, -0.5], dtype=F64)
    got = run_sink_attention(q, k, v, sink, 0.7, window, dtype, mma=mma)
    want = P.sink_attention(q, k, v, sink, 0.7, window, P.distance_slopes(Hh))
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert float((got - want).abs().max()) < tol, float((got - want).abs().max())
    if window not in (None, 1):
        # the test has teeth: seeing one key more or one key less moves the result by far more than the tolerance
        one_more = P.sink_attention(q, k, v, sink, 0.7, window + 1, P.distance_slopes(Hh))
        one_less = P.sink_attention(q, k, v, sink, 0.7, window - 1, P.distance_slopes(Hh))
        assert float((one_more - want).abs().max()) > 5 * tol and float((one_less - want).abs().max()) > 5 * tol


@pytest.mark.parametrize("window", [None, 1, 5, 64, 70, 129, 200])
@pytest.mark.parametrize("shape", [(6, 2, 64), (5, 5, 128), (12, 1, 64)])
def test_sink_attention_on_tcgen05_edges_sink_and_gate(window, shape):
    """The two-tile tcgen05 form (keys and values of one head size, 64 or 128; groups of 3, 1 and 12
    heads): 330 tokens that start at position 21, the keys at a window's edge (or key 3 without one)
    ranking highest, sinks from small to as large as the largest score, the gate read from a column slice."""
    torch.manual_seed(8)
    Hh, G, D = shape
    T, pos0 = 330, 21
    q = torch.randn(T, Hh, D, dtype=F64) * 0.2
    k = torch.randn(T, G, D, dtype=F64) * 0.2
    v = torch.randn(T, G, D, dtype=F64)
    q[:, :, 0] = 1.0
    k[:, :, 0] = 0.0
    if window is None:
        k[3, :, 0] = 40.0
    else:
        for j in range(T):
            k[j, :, 0] = 20.0 * ((T - 1 - j) % (window + 1)) / (window + 1)
    q, k, v = (t.to(torch.bfloat16).double() for t in (q, k, v))
    sink = torch.linspace(-2.0, 12.0, Hh, dtype=F64)        # the last head's sink stands beside the edge keys' scores
    wide = torch.randn(T, Hh * D + 8, dtype=torch.float32, device=DEV)
    gate = wide[:, 4:4 + Hh * D]
    got = run_sink_attention(q, k, v, sink, 0.6, window, torch.bfloat16, pos0=pos0, gate=gate, mma="twin")
    # the cells before the portion are zero keys and values: score 0 minus the distance bias
    z = lambda t: torch.cat([torch.zeros(pos0, *t.shape[1:], dtype=F64), t])
    want = P.sink_attention(z(q), z(k), z(v), sink, 0.6, window, P.distance_slopes(Hh))[pos0:]
    want = want * torch.sigmoid(gate.double().cpu()).view(T, Hh, D)
    assert float((got - want).abs().max()) < 2e-2, float((got - want).abs().max())
    if window not in (None, 1):
        one_more = P.sink_attention(z(q), z(k), z(v), sink, 0.6, window + 1, P.distance_slopes(Hh))[pos0:] * torch.sigmoid(gate.double().cpu()).view(T, Hh, D)
        assert float((one_more - want).abs().max()) > 0.05          # one key more would show
    no_sink = P.sink_attention(z(q), z(k), z(v), torch.full((Hh,), -1e9, dtype=F64), 0.6, window, P.distance_slopes(Hh))[pos0:]
    assert float((no_sink * torch.sigmoid(gate.double().cpu()).view(T, Hh, D) - want).abs().max()) > 0.05


def test_sink_share_temperature_mixing_and_gate():
    from lgml_b200 import ops

    torch.manual_seed(2)
    T, Hh, G, D, Dv = 70, 4, 4, 16, 12
    q, k, v = torch.randn(T, Hh, D, dtype=F64) * 0.5, torch.randn(T, G, D, dtype=F64) * 0.5, torch.randn(T, G, Dv, dtype=F64)
    sink = torch.tensor([3.0, 0.0, -2.0, 6.0], dtype=F64)         # head 3's sink takes most of the mass
    # temperature: position p multiplies q by 1 + c ln(floor((p + 1) / e) + 1); start the portion at position 37
    pos0, temp = 37, (0.6, 5)
    kfull = torch.cat([torch.zeros(pos0, G, D, dtype=F64), k])
    # (keys before the portion are zero cells in the pages: score 0 minus the distance bias, as in the plain run below)
    qt = q * P.query_temperature(torch.arange(pos0, pos0 + T), *temp)[:, None, None]
    qfull = torch.cat([torch.zeros(pos0, Hh, D, dtype=F64), qt])
    vfull = torch.cat([torch.zeros(pos0, G, Dv, dtype=F64), v])
    want = P.sink_attention(qfull, kfull, vfull, sink, 0.4, 50, P.distance_slopes(Hh))[pos0:]
    got = run_sink_attention(q, k, v, sink, 0.4, 50, torch.float32, temp=temp, pos0=pos0)
    assert float((got - want).abs().max()) < 2e-5
    no_sink = P.sink_attention(qfull, kfull, vfull, torch.full((Hh,), -1e9, dtype=F64), 0.4, 50, P.distance_slopes(Hh))[pos0:]
    assert float((no_sink - want).abs().max()) > 0.1          # leaving the sink out would show
    # value mixing: mode 1 keeps v, mode 2 stores (1 - lambda) v + lambda kept
    kept = torch.empty(T, G * Dv, dtype=torch.float32, device=DEV)
    first = run_sink_attention(q, k, v, sink, 0.4, None, torch.float32, keep_mode=1, kept=kept)
    assert torch.equal(kept.cpu().view(T, G, Dv), v.float())
    v2 = torch.randn(T, G, Dv, dtype=F64)
    lam = torch.tensor([0.35], dtype=torch.float32, device=DEV)
    mixed = run_sink_attention(q, k, v2, sink, 0.4, None, torch.float32, keep_mode=2, kept=kept, lam=lam)
    want_mixed = P.sink_attention(q, k, (1 - 0.35) * v2 + 0.35 * v.float().double(), sink, 0.4, None, P.distance_slopes(Hh))
    assert float((mixed - want_mixed).abs().max()) < 2e-5
    assert float((first - P.sink_attention(q, k, v, sink, 0.4, None, P.distance_slopes(Hh))).abs().max()) < 2e-5
    # the tensor-core form with a start in the middle of a page, the temperature and head sizes that are no multiple of 8
    got16 = run_sink_attention(q, k, v, sink, 0.4, 50, torch.bfloat16, temp=temp, pos0=pos0, mma=True)
    assert float((got16 - want).abs().max()) < 3e-2
    # the gate, from a column slice of a wider buffer
    wide = torch.randn(T, Hh * Dv + 7, dtype=torch.float32, device=DEV)
    gated = run_sink_attention(q, k, v, sink, 0.4, None, torch.float32, gate=wide[:, 3:3 + Hh * Dv])
    want_gated = first * torch.sigmoid(wide[:, 3:3 + Hh * Dv].double().cpu()).view(T, Hh, Dv)
    assert float((gated - want_gated).abs().max()) < 2e-5
    gated16 = run_sink_attention(q, k, v, sink, 0.4, None, torch.bfloat16, gate=wide[:, 3:3 + Hh * Dv], mma=True)
    assert float((gated16 - want_gated).abs().max()) < 3e-2
    split16 = run_sink_attention(q, k, v, sink, 0.4, None, torch.bfloat16, gate=wide[:, 3:3 + Hh * Dv], mma="split")
    assert float((split16 - want_gated).abs().max()) < 3e-2
    got_split = run_sink_attention(q, k, v, sink, 0.4, 50, torch.bfloat16, temp=temp, pos0=pos0, mma="split")
    assert float((got_split - want).abs().max()) < 3e-2


@pytest.mark.parametrize("D,Dv,Hh,G", [(12, 20, 3, 1), (40, 12, 2, 2), (128, 64, 2, 1), (200, 130, 1, 1)])
def test_delta_scan_in_pieces_matches_the_plain_recurrence(D, Dv, Hh, G):
    """Two requests of unequal length in one launch, then the same tokens in pieces of 1, 2, 9, ...
    with the state carried in the slots: equal bit for bit, and equal to the plain recurrence."""
    from lgml_b200 import ops

    torch.manual_seed(3)
    lens = [37, 5]
    C = 2 * G * D + Hh * Dv
    data = []
    for n in lens:
        q = torch.nn.functional.normalize(torch.randn(n, G, D, dtype=F64), dim=-1) * D ** -0.5
        k = torch.nn.functional.normalize(torch.randn(n, G, D, dtype=F64), dim=-1)
        v = torch.randn(n, Hh, Dv, dtype=F64)
        beta = torch.rand(n, Hh, dtype=F64)
        decay = torch.rand(n, Hh, D, dtype=F64) ** 0.2
        data.append((q, k, v, beta, decay))
    floats = Hh * D * Dv + 5

    def run(pieces):
        state = torch.zeros(4, floats, dtype=torch.float32, device=DEV)
        state[:, Hh * D * Dv:] = 7.0            # what follows S in a slot is not the scan's to touch
        slots = torch.tensor([2, 0], dtype=torch.int32, device=DEV)
        outs = [[], []]
        fed = [0, 0]
        for piece in pieces:
            rows, starts, act = [], [0], []
            for s, n in enumerate(piece):
                if n == 0:
                    continue
                q, k, v, beta, decay = (t[fed[s]:fed[s] + n] for t in data[s])
                rows.append((torch.cat([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1)], 1), beta, decay.reshape(n, -1)))
                starts.append(starts[-1] + n)
                act.append(s)
                fed[s] += n
            qkv = torch.cat([r[0] for r in rows]).float().to(DEV).contiguous()
            b = torch.cat([r[1] for r in rows]).float()
            dc = torch.cat([r[2] for r in rows]).float().view(-1, Hh, D)
            gb = torch.cat([dc, b[:, :, None], torch.zeros(b.shape[0], Hh, 3)], 2).to(DEV).contiguous()     # per head: decays, beta, zeros
            o = ops.delta_scan(qkv, gb, state, torch.tensor(starts, dtype=torch.int32, device=DEV), slots[act].contiguous(), Hh, G, D, Dv)
            for i, s in enumerate(act):
                outs[s].append(o[starts[i]:starts[i + 1]].cpu())
        assert bool((state[:, Hh * D * Dv:] == 7.0).all()) and bool((state[[1, 3]][:, :Hh * D * Dv] == 0).all())
        return [torch.cat(o) for o in outs]

    whole = run([lens])
    pieces = run([[1, 1], [2, 0], [9, 2], [1, 2], [24, 0]])
    for s in range(2):
        assert torch.equal(whole[s], pieces[s])
        q, k, v, beta, decay = data[s]
        for h in range(Hh):
            g = h // (Hh // G)
            want = P.gated_delta_rule(q[:, g], k[:, g], v[:, h], beta[:, h], decay[:, h])
            got = whole[s].view(lens[s], Hh, Dv)[:, h].double()
            assert float((got - want).abs().max()) < 1e-5


def test_delta_scan_of_many_requests_at_once():
    """48 requests of three tokens in one launch (the kernel then gives a thread two columns of the
    state; 96 value columns leave the last block's second columns empty), a second launch on the
    states the first left, against the plain recurrence over all six tokens."""
    from lgml_b200 import ops

    torch.manual_seed(6)
    n_req, Hh, G, D, Dv = 48, 4, 2, 64, 96
    q = torch.nn.functional.normalize(torch.randn(n_req, 6, G, D, dtype=F64), dim=-1) * D ** -0.5
    k = torch.nn.functional.normalize(torch.randn(n_req, 6, G, D, dtype=F64), dim=-1)
    v = torch.randn(n_req, 6, Hh, Dv, dtype=F64)
    beta = torch.rand(n_req, 6, Hh, dtype=F64)
    decay = torch.rand(n_req, 6, Hh, D, dtype=F64) ** 0.3
    state = torch.zeros(n_req + 2, Hh * D * Dv, dtype=torch.float32, device=DEV)
    slots = torch.randperm(n_req + 2)[:n_req].to(torch.int32).to(DEV)
    starts = torch.arange(0, 3 * n_req + 1, 3, dtype=torch.int32, device=DEV)
    outs = []
    for lo in (0, 3):
        sl = slice(lo, lo + 3)
        qkv = torch.cat([q[:, sl].reshape(n_req * 3, -1), k[:, sl].reshape(n_req * 3, -1), v[:, sl].reshape(n_req * 3, -1)], 1).float().to(DEV).contiguous()
        gb = torch.cat([decay[:, sl], beta[:, sl, :, None], torch.zeros(n_req, 3, Hh, 3, dtype=F64)], 3).reshape(n_req * 3, Hh, D + 4).float().to(DEV).contiguous()
        outs.append(ops.delta_scan(qkv, gb, state, starts, slots, Hh, G, D, Dv).cpu().view(n_req, 3, Hh, Dv))
    got = torch.cat(outs, 1).double()
    for s in (0, 17, 47):
        for h in range(Hh):
            want = P.gated_delta_rule(q[s, :, h // 2], k[s, :, h // 2], v[s, :, h], beta[s, :, h], decay[s, :, h])
            assert float((got[s, :, h] - want).abs().max()) < 1e-5


@pytest.mark.parametrize("taps", [1, 2, 5])
def test_delta_prepare_carries_the_filter_inputs_across_portions(taps):
    from lgml_b200 import ops

    torch.manual_seed(4)
    Hh, G, D, Dv, n = 3, 1, 10, 6, 23
    C = 2 * G * D + Hh * Dv
    x = torch.randn(n, C + Hh, dtype=F64)
    a_pre = torch.randn(n, Hh * D, dtype=F64)
    conv_w = torch.randn(C, taps, dtype=F64) * 0.5
    a_log, dt_bias = torch.randn(Hh, dtype=F64) * 0.5, torch.randn(Hh * D, dtype=F64)
    y = P.causal_conv_silu(x[:, :C], conv_w)
    qn = y[:, :G * D].view(n, G, D)
    qn = qn / torch.sqrt((qn * qn).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    kn = y[:, G * D:2 * G * D].view(n, G, D)
    kn = kn / torch.sqrt((kn * kn).sum(-1, keepdim=True) + 1e-6)
    want_c = torch.cat([qn.reshape(n, -1), kn.reshape(n, -1), y[:, 2 * G * D:]], 1)
    want_beta = torch.sigmoid(x[:, C:])
    want_decay = torch.exp(-torch.exp(a_log).repeat_interleave(D) * torch.nn.functional.softplus(a_pre + dt_bias))
    S_floats = Hh * D * Dv
    state = torch.zeros(3, S_floats + (taps - 1) * C, dtype=torch.float32, device=DEV)
    slot = torch.tensor([1], dtype=torch.int32, device=DEV)
    got_c, got_b, got_d = [], [], []
    tail = []
    fed = 0
    for m in (1, 1, 2, 1, 7, 3, 8):             # portions shorter than the filter among them
        xs = x[fed:fed + m].float().to(DEV).contiguous()
        c, gb = ops.delta_prepare(xs, a_pre[fed:fed + m].float().to(DEV).contiguous(), conv_w.float().to(DEV), state, S_floats,
                                  torch.zeros(m, dtype=torch.int32, device=DEV), torch.tensor([0, m], dtype=torch.int32, device=DEV),
                                  slot, a_log.float().to(DEV), dt_bias.float().to(DEV), Hh, G, D, Dv)
        gb = gb.cpu()
        got_c.append(c.cpu()), got_b.append(gb[:, :, D]), got_d.append(gb[:, :, :D].reshape(m, Hh * D)), tail.append(gb[:, :, D + 1:])
        fed += m
    assert fed == n
    for got, want in ((got_c, want_c), (got_b, want_beta), (got_d, want_decay)):
        assert float((torch.cat(got).double() - want).abs().max()) < 1e-5
    assert bool((torch.cat(tail) == 0).all())
    assert bool((state[[0, 2]] == 0).all()) and bool((state[1, :S_floats] == 0).all())


def test_delta_output_norm_and_relu_squared():
    from lgml_b200 import ops

    torch.manual_seed(5)
    n, Hh, Dv = 5, 3, 20
    o = torch.randn(n, Hh * Dv, dtype=torch.float32, device=DEV) * 3
    wt = torch.randn(Dv, dtype=torch.float32, device=DEV)
    gate = torch.randn(n, Hh * Dv + 4, dtype=torch.float32, device=DEV)[:, 4:]
    got = ops.delta_output(o, wt, gate, 1e-3, torch.float32, Hh).double().cpu().view(n, Hh, Dv)
    od = o.double().cpu().view(n, Hh, Dv)
    want = od / torch.sqrt((od * od).mean(-1, keepdim=True) + 1e-3) * wt.double().cpu() * torch.sigmoid(gate.double().cpu()).view(n, Hh, Dv)
    assert float((got - want).abs().max()) < 1e-5
    x = torch.randn(7, 33, dtype=torch.float32, device=DEV)
    assert torch.equal(ops.relu_sq(x.clone()), torch.relu(x) ** 2)
    xb = x.to(torch.bfloat16)
    assert torch.equal(ops.relu_sq(xb.clone()), (torch.relu(xb.float()) ** 2).to(torch.bfloat16))


# ---------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------

@pytest.fixture(scope="module", params=sorted(L.CONFIGS))
def model(request, tmp_path_factory):
    cfg, ranks = L.CONFIGS[request.param]
    made = {}
    # float32 runs see attention sharpened (a wrong key moves the logits far past the tolerance);
    # bfloat16's own rounding of q and k would be amplified alike, so its models are left as drawn
    for dtype, sharpen in (("float32", 2.0), ("bfloat16", 1.0)):
        weights = L.random_weights(cfg, ranks, seed=11, sharpen=sharpen)
        made[dtype] = (weights, L.write_folder(tmp_path_factory.mktemp(f"{request.param}_{dtype}"), cfg, weights))
    return request.param, cfg, made


def make_runner(folder, dtype, n_pages, slots=4, **kw):
    from lgml_b200.engine.engine import parse_dtype
    from lgml_b200.engine.runner import ModelRunner

    return ModelRunner.from_folder(folder, parse_dtype(dtype), DEV, n_pages=n_pages, max_slots=slots, max_step_tokens=n_pages * 64, **kw)


def sequences(cfg, lens, seed=50):
    return {f"r{i}": H.random_ids(n, cfg["vocab"], seed + i) for i, n in enumerate(lens)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_all_cuttings_match_the_plain_model(model, dtype):
    """Whole; the last 32 tokens one by one; portions down to two tokens; and up to three live
    requests in two... four slots with so few pages that pages and slots are used again."""
    name, cfg, made = model
    weights, folder = made[dtype]
    seqs = sequences(cfg, [1, 5, 23, 64, 65, 97, 150, 201])
    pages_one = 4
    results = {}
    for kind, trace in (("whole", H.trace_whole(seqs)), ("tail", H.trace_tail(seqs)), ("portions", H.trace_portions(seqs))):
        runner = make_runner(folder, dtype, n_pages=pages_one)
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
    """Three tokens of prompt, then 180 tokens one by one (through captured steps): every window of
    the models (1, 3, 20, 40, 65, 70, 100) passes over decoded tokens, and the state is carried 180 times."""
    name, cfg, made = model
    weights, folder = made[dtype]
    seqs = sequences(cfg, [183], seed=70)
    runner = make_runner(folder, dtype, n_pages=3)
    got = H.run_trace(runner, H.trace_tail(seqs, tail=180))
    assert runner.graph_replays > 100
    L.compare(got, cfg, weights, seqs, **TOL[dtype])


def test_slots_are_zeroed_when_used_again(model):
    """One slot, six requests one after the other, each decoded in a different cutting: a state or
    a filter input left behind by the request before would show."""
    name, cfg, made = model
    weights, folder = made["float32"]
    seqs = sequences(cfg, [30, 7, 66, 2, 41, 12], seed=90)
    runner = make_runner(folder, "float32", n_pages=2, slots=1)
    got = H.run_trace(runner, H.trace_portions(seqs, sizes=(3, 2, 11, 1, 40)))
    L.compare(got, cfg, weights, seqs, **TOL["float32"])


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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(model, dtype):
    """Engine.generate (scheduler, portions of 16 prompt tokens, sampling on the device, steps run
    ahead) and Engine.greedy against greedy decoding with the plain model."""
    import lgml_b200

    name, cfg, made = model
    weights, folder = made[dtype]
    prompts = [H.random_ids(n, cfg["vocab"], 200 + n) for n in (37, 5, 70)]
    eng = lgml_b200.Engine(str(folder), dtype=dtype, n_ctx=256, slots=2, ubatch=16)
    outs = eng.generate(prompts, max_tokens=10, temperature=0.0, stop=[])
    solo, _ = eng.greedy(prompts[0], 10)
    for prompt, got in zip(prompts, outs):
        assert len(got) == 10
        for i, tok in enumerate(got):
            row = L.oracle_logits(cfg, weights, prompt + got[:i])[-1]
            gap = float(row.max() - row[tok])
            bound = 0.0 if dtype == "float32" and gap > 1e-4 else (1e-4 if dtype == "float32" else 5e-2 * float(row.abs().max()))
            assert gap <= bound, f"{dtype}: token {i} is {tok}, the plain model prefers {int(row.argmax())} by {gap:.3g}"
    if dtype == "float32":
        assert solo == outs[0]


def test_trace_run_as_a_process(model, tmp_path):
    name, cfg, made = model
    weights, folder = made["float32"]
    seqs = sequences(cfg, [70, 20, 131], seed=300)
    trace = H.trace_mixed(seqs, max_tokens=64 * 4, seed=2, max_live=2)
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out),
                           "--max-tokens", str(64 * 4)], input="\n".join(json.dumps(s) for s in trace) + "\n", text=True,
                          capture_output=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    done = [ln for ln in proc.stdout.splitlines() if ln.startswith("done ")]
    assert done == [f"done {s['step']}" for s in trace]
    import numpy as np

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
    L.compare(got, cfg, weights, seqs, **TOL["float32"])


def test_command_line_generates_with_the_folders_architecture(model):
    """python -m lgml_b200 on a Lefulorn folder (no context given: the design names no limit): greedy ids as the plain model's."""
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
