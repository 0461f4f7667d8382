"""Test material for the Lefulorn design: small configurations that differ from each other in
every size and option, random weights made so that the mechanisms show, and the oracle."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List, Tuple

import torch

from tests.plain import lefulorn_plain as P


def attention(heads, kv, dim, vdim, scale, window=None, q_temp=None, v_mix=False, ff=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix}
    if window is not None:
        m["mask"] = {"size": window}
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return {"type": "attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def delta(heads, kv, dim, vdim, conv, ff=None):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(vocab, width, layers, eps=1e-5, logit_scale=1.0):
    return {"architecture": "Lefulorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_scale": logit_scale, "layers": layers}


# Starts with a delta layer; grouped heads in both mixers; windows below and above a page and
# none at all; a value-mixing chain that starts in the middle and skips a layer; feed-forwards
# on some layers of either kind.
MIXED = config(97, 64, [
    delta(4, 2, 16, 24, conv=3, ff=80),
    attention(4, 2, 32, 16, scale=0.2, window=20, q_temp=(0.3, 8)),
    attention(6, 3, 16, 8, scale=0.3, window=70, v_mix=True, ff=48),
    delta(2, 2, 40, 12, conv=2),
    attention(3, 3, 24, 8, scale=0.25, v_mix=True, q_temp=(0.7, 5), ff=32),
    attention(6, 3, 8, 8, scale=0.5, window=3, v_mix=True),
], eps=1e-5, logit_scale=0.5)
MIXED_RANKS = {0: (12, 8), 3: (4, 20)}       # layer -> (rank of the decay's projection, of the gate's)

# One head everywhere, sizes that are no multiple of 8 or 32, a window of 1, long filters.
ODD = config(61, 36, [
    attention(1, 1, 20, 12, scale=0.4, window=1, ff=20),
    delta(1, 1, 12, 20, conv=5, ff=28),
    attention(5, 1, 12, 4, scale=0.35, window=65, q_temp=(1.0, 1)),
    delta(3, 1, 36, 4, conv=1),
], eps=3e-6)
ODD_RANKS = {1: (6, 6), 3: (10, 2)}

ONLY_DELTA = config(50, 32, [delta(2, 1, 16, 16, conv=4, ff=40), delta(2, 2, 8, 16, conv=4)], eps=1e-6, logit_scale=2.0)
ONLY_DELTA_RANKS = {0: (8, 8), 1: (8, 8)}

# Attention only, no window anywhere and no state: the engine then replays short portions from
# captured steps (padded to a page's edge) and pads decode batches with repeated rows.
ONLY_ATTENTION = config(83, 48, [
    attention(4, 2, 16, 8, scale=0.3, v_mix=True, q_temp=(0.4, 3), ff=64),
    attention(2, 2, 32, 16, scale=0.2),
    attention(4, 2, 16, 8, scale=0.3, v_mix=True, ff=24),
], eps=1e-5, logit_scale=1.0)

# Keys and values of one head size, 64 or 128: prompts and portions of these layers run on the
# two-tile tcgen05 attention kernel (groups of 2, 1 and 3 heads; windows across pages and none).
WIDE_HEADS = config(101, 96, [
    attention(4, 2, 64, 64, scale=0.15, window=100, q_temp=(0.3, 16), v_mix=True, ff=72),
    delta(2, 1, 32, 64, conv=3),
    attention(2, 2, 128, 128, scale=0.1),
    attention(6, 2, 64, 64, scale=0.15, window=40, v_mix=True),
], eps=1e-5, logit_scale=0.7)
WIDE_HEADS_RANKS = {1: (8, 16)}

CONFIGS = {"mixed": (MIXED, MIXED_RANKS), "odd": (ODD, ODD_RANKS), "only_delta": (ONLY_DELTA, ONLY_DELTA_RANKS),
           "only_attention": (ONLY_ATTENTION, {}), "wide_heads": (WIDE_HEADS, WIDE_HEADS_RANKS)}


def random_weights(cfg: dict, ranks: Dict[int, Tuple[int, int]], seed: int, sharpen: float = 1.0) -> Dict[str, torch.Tensor]:
    """Weights as bfloat16-representable float32 tensors (integer-free), scaled so that no
    mechanism is lost in the noise: attention far from uniform, sinks that take a visible share,
    decays between almost none and almost all, a mixing weight well inside (0, 1)."""
    g = torch.Generator().manual_seed(seed)
    E = cfg["width"]

    def mat(o, i, gain=1.0):
        return torch.randn(o, i, generator=g) * gain / i ** 0.5

    def vec(n, sd, mean=0.0):
        return torch.randn(n, generator=g) * sd + mean

    w = {"embed": torch.randn(cfg["vocab"], E, generator=g), "final.norm": vec(E, 0.1, 1.0), "head": mat(cfg["vocab"], E)}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        w[p + "norm1"] = vec(E, 0.1, 1.0)
        if layer["type"] == "attention":
            w[p + "mix.q"], w[p + "mix.q.b"] = mat(H * D, E, sharpen), vec(H * D, 0.2)
            w[p + "mix.k"], w[p + "mix.k.b"] = mat(G * D, E, sharpen), vec(G * D, 0.2)
            w[p + "mix.v"], w[p + "mix.v.b"] = mat(G * Dv, E), vec(G * Dv, 0.2)
            w[p + "mix.vmix"] = torch.tensor(0.3 + 0.1 * i)
            w[p + "mix.sink"] = vec(H, 1.0, 0.5)
            w[p + "mix.g"], w[p + "mix.o"] = mat(H * Dv, E, 2.0), mat(E, H * Dv)
        else:
            ra, rg = ranks[i]
            taps = m["conv"]
            for n, rows in (("q", G * D), ("k", G * D), ("v", H * Dv)):
                w[p + f"mix.{n}"] = mat(rows, E, 2.0)
                w[p + f"mix.{n}.conv"] = torch.randn(rows, taps, generator=g) * 0.6
            w[p + "mix.b"] = mat(H, E, 2.0)
            w[p + "mix.A_log"] = vec(H, 0.7, -0.5)
            w[p + "mix.norm"] = vec(Dv, 0.1, 1.0)
            w[p + "mix.a1"], w[p + "mix.a2"] = mat(ra, E), mat(H * D, ra, 2.0)
            w[p + "mix.dt_bias"] = vec(H * D, 1.0, -1.0)
            w[p + "mix.g1"], w[p + "mix.g2"] = mat(rg, E), mat(H * Dv, rg, 2.0)
            w[p + "mix.o"] = mat(E, H * Dv)
        if layer.get("mlp"):
            F = layer["mlp"]["ff"]
            w[p + "norm2"] = vec(E, 0.1, 1.0)
            w[p + "mlp.up"], w[p + "mlp.up.b"] = mat(F, E), vec(F, 0.2)
            w[p + "mlp.down"], w[p + "mlp.down.b"] = mat(E, F), vec(E, 0.1)
    return {n: t.to(torch.bfloat16).float() for n, t in w.items()}


def write_folder(folder: Path, cfg: dict, weights: Dict[str, torch.Tensor]) -> Path:
    """config.json and model.safetensors (bfloat16) of a model."""
    from lgml_b200.weights import write_safetensors

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    write_safetensors(folder / "model.safetensors", {n: t.to(torch.bfloat16) for n, t in weights.items()})
    return folder


_oracle: Dict[Tuple[int, Tuple[int, ...]], torch.Tensor] = {}


def oracle_logits(cfg: dict, weights: Dict[str, torch.Tensor], ids: List[int]) -> torch.Tensor:
    key = (id(weights), tuple(ids))
    if key not in _oracle:
        _oracle[key] = P.forward(cfg, weights, ids)
    return _oracle[key]


def compare(got: Dict[Tuple[str, int], torch.Tensor], cfg, weights, seqs: Dict[str, List[int]], atol: float, rtol: float) -> float:
    """Largest error over all rows that ``got`` holds; raises naming the first wrong (request, position)."""
    worst = 0.0
    for rid, ids in seqs.items():
        ref = oracle_logits(cfg, weights, ids)
        for p in range(len(ids)):
            if (rid, p) not in got:
                continue
            row = got[(rid, p)].double()
            err = (row - ref[p]).abs()
            bound = atol + rtol * ref[p].abs().max()
            if bool((err > bound).any()):
                j = int(err.argmax())
                raise AssertionError(f"request {rid} position {p} (page {p // 64}, cell {p % 64}): logit {j} is {row[j]:.6g}, "
                                     f"oracle {ref[p, j]:.6g}, |diff| {err[j]:.3g} > {bound:.3g}")
            worst = max(worst, float(err.max()))
    return worst
