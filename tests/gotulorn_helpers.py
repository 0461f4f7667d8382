"""Test material for the Gotulorn design: small configurations that differ from each other in every
size and option, random weights made so that the mechanisms show, and the oracle."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List, Tuple

import numpy as np
import torch

from tests.plain import gotulorn_plain as P


def dense(ff, limit=2.0):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def attention(heads, kv, dim, vdim, scale, diff, window=None, keep_first=0, kv_from=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if window is not None:
        m["mask"] = {"size": window, "keep_first": keep_first}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, rank, scale, base=10000.0, dims=None, mlp=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
                      "rot": {"base": base, "dims": rot_dim if dims is None else dims}}}


def config(vocab, width, layers, eps=1e-5, embed_scale=1.0):
    return {"architecture": "Gotulorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embed_scale},
            "layers": layers}


# Grouped heads; windows below a page, across pages; a reader with a wider window and more kept
# tokens than the layer whose keys it reads, and one with a narrower mask; kept tokens that fill
# more than a page; experts with top 1, 2 and all; layers without a feed-forward.
MIXED = config(97, 64, [
    attention(4, 2, 16, 24, scale=0.25, diff=0.2, window=20, keep_first=3, mlp=dense(80, 1.5)),
    latent(3, 16, 8, 12, 24, scale=0.2, base=5000.0, mlp=moe(24, 5, 2)),
    attention(4, 2, 16, 24, scale=0.3, diff=0.4, window=70, keep_first=5, kv_from=0, mlp=moe(16, 3, 1)),
    attention(6, 3, 8, 8, scale=0.35, diff=0.1, window=3, keep_first=0),
    latent(2, 24, 12, 20, 40, scale=0.15, base=300.0, dims=8, mlp=dense(48, 3.0)),
    attention(6, 3, 8, 8, scale=0.3, diff=0.25, window=2, keep_first=70, kv_from=3, mlp=moe(12, 4, 4)),
], eps=1e-5, embed_scale=6.0)

# One head everywhere, sizes that are no multiple of 8, a window of 1 with one kept token, one
# expert, no embedding scale, no difference constant.
ODD = config(61, 36, [
    latent(1, 12, 2, 20, 10, scale=0.3, base=77.0, mlp=moe(20, 1, 1)),
    attention(1, 1, 20, 12, scale=0.4, diff=0.0, window=1, keep_first=1, mlp=dense(20, 0.5)),
    attention(5, 1, 12, 4, scale=0.35, diff=0.5, window=65, keep_first=2),
    attention(5, 1, 12, 4, scale=0.2, diff=0.3, window=64, keep_first=64, kv_from=2, mlp=dense(28, 10.0)),
], eps=3e-6, embed_scale=1.0)

# No window anywhere: every layer keeps all keys (the engine then replays short portions from
# captured steps and pads decode batches with repeated rows).
NO_WINDOW = config(83, 48, [
    attention(4, 2, 16, 8, scale=0.3, diff=0.3, mlp=dense(64, 2.0)),
    latent(4, 8, 8, 8, 16, scale=0.25, base=1000.0, mlp=moe(16, 6, 3)),
    attention(4, 2, 16, 8, scale=0.3, diff=0.3, kv_from=0),
], eps=1e-5, embed_scale=3.0)

# Head sizes the tensor-core attention kernels take (multiples of 32): prompts and decoding of these
# layers run on them.
WIDE_HEADS = config(101, 96, [
    attention(4, 2, 64, 64, scale=0.12, diff=0.3, window=100, keep_first=6, mlp=dense(72, 2.0)),
    latent(4, 32, 32, 32, 96, scale=0.1, base=30000.0, mlp=moe(40, 8, 2)),
    attention(4, 2, 64, 64, scale=0.12, diff=0.2, window=40, keep_first=2, kv_from=0, mlp=moe(40, 8, 2)),
    attention(2, 1, 32, 96, scale=0.2, diff=0.35, window=130, keep_first=65),
    latent(2, 64, 32, 64, 32, scale=0.1, base=500.0, dims=16),
], eps=1e-5, embed_scale=8.0)

CONFIGS = {"mixed": MIXED, "odd": ODD, "no_window": NO_WINDOW, "wide_heads": WIDE_HEADS}


def random_weights(cfg: dict, seed: int, sharpen: float = 1.0) -> Dict[str, torch.Tensor]:
    """Weights as bfloat16-representable float32 tensors, scaled so that no mechanism is lost in the
    noise: attention far from uniform, a lambda well away from 0, router logits apart, gate and up
    values on both sides of the clamp."""
    g = torch.Generator().manual_seed(seed)
    E = cfg["width"]

    def mat(o, i, gain=1.0):
        return torch.randn(o, i, generator=g) * gain / i ** 0.5

    def vec(n, sd, mean=0.0):
        return torch.randn(n, generator=g) * sd + mean

    def norm(name, w):
        w[name], w[name + ".b"], w[name + ".alpha"] = vec(E, 0.1, 1.0), vec(E, 0.1), torch.tensor(0.4) + 0.2 * torch.rand((), generator=g)

    w = {"embed": torch.randn(cfg["vocab"], E, generator=g) * 0.5, "head": mat(cfg["vocab"], E)}
    norm("embed.norm", w)
    norm("final.norm", w)
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        norm(p + "norm1", w)
        if layer["type"] == "attention":
            H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[p + "mix.q"] = mat(H * 2 * D, E, 1.5 * sharpen)
            if m.get("kv_from") is None:
                w[p + "mix.k"], w[p + "mix.v"] = mat(G * 2 * D, E, 1.5 * sharpen), mat(G * Dv, E, 2.0)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                w[p + "mix." + n] = vec(D, 0.12)        # lambda stays near diff: 1 - lambda is no small number
            w[p + "mix.o"] = mat(E, H * Dv)
        else:
            H, D, Dr, Dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            w[p + "mix.q"] = mat(H * (D + Dr), E, 1.5 * sharpen)
            w[p + "mix.dkv"] = mat(R + Dr, E, 1.5 * sharpen)
            w[p + "mix.dkv.norm"] = vec(R, 0.2, 1.0)
            w[p + "mix.uk"], w[p + "mix.uv"] = mat(H * D, R, 1.5), mat(H * Dv, R, 1.5)
            w[p + "mix.o"] = mat(E, H * Dv)
        f = layer.get("mlp")
        if f:
            norm(p + "norm2", w)
            if f["kind"] == "dense":
                F = f["ff"]
                w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = mat(F, E, 3.0), mat(F, E, 3.0), mat(E, F)
            else:
                F, X = f["expert"]["ff"], f["router"]["experts"]
                w[p + "mlp.router"], w[p + "mlp.router.b"] = mat(X, E, 4.0), vec(X, 0.5)
                for e in range(X):
                    w[f"{p}mlp.e{e}.gate"], w[f"{p}mlp.e{e}.up"], w[f"{p}mlp.e{e}.down"] = mat(F, E, 2.0), mat(F, E, 2.0), mat(E, F, 1.0 + 0.3 * e)
    return {n: t.to(torch.bfloat16).float() for n, t in w.items()}


def write_folder(folder: Path, cfg: dict, weights: Dict[str, torch.Tensor]) -> Path:
    """config.json and model.safetensors (bfloat16) of a model."""
    from lgml_b200.weights import write_safetensors

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    write_safetensors(folder / "model.safetensors", {n: t.to(torch.bfloat16) for n, t in weights.items()})
    return folder


def as_numpy(weights: Dict[str, torch.Tensor]) -> Dict[str, np.ndarray]:
    return {n: t.double().numpy() for n, t in weights.items()}


_oracle: Dict[Tuple[int, Tuple[int, ...]], torch.Tensor] = {}
_numpy: Dict[int, Dict[str, np.ndarray]] = {}


def oracle_logits(cfg: dict, weights: Dict[str, torch.Tensor], ids: List[int]) -> torch.Tensor:
    key = (id(weights), tuple(ids))
    if key not in _oracle:
        if id(weights) not in _numpy:
            _numpy[id(weights)] = as_numpy(weights)
        _oracle[key] = torch.from_numpy(P.forward(cfg, _numpy[id(weights)], list(ids)))
    return _oracle[key]


def clear_ids(cfg: dict, weights: Dict[str, torch.Tensor], n: int, seed: int, gap: float = 0.3) -> List[int]:
    """n random token ids for which no router of the plain model decides by less than ``gap``: a bfloat16
    run may not rest on a close call between two experts (one flipped choice moves every later logit).
    The model is causal, so the first close call is redrawn and the sequence checked again."""
    import random

    rng = random.Random(seed)
    ids = [rng.randrange(cfg["vocab"]) for _ in range(n)]
    if id(weights) not in _numpy:
        _numpy[id(weights)] = as_numpy(weights)
    for _ in range(40 * n):
        gaps: list = []
        P.forward(cfg, _numpy[id(weights)], ids, router_gaps=gaps)
        if not gaps:
            return ids
        close = np.nonzero(np.min(np.stack(gaps), axis=0) < gap)[0]
        if close.size == 0:
            return ids
        ids[int(close[0])] = rng.randrange(cfg["vocab"])
    raise AssertionError("no sequence without a close call was found")


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
