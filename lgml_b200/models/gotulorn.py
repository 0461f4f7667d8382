"""The Gotulorn decoder: which parts a ``GotulornConfig`` asks for, layer by layer.

The embedding's rows are scaled and go through the model's norm; that is the residual stream.
Every layer is pre-norm: x += mixer(norm1(x)), then, unless its ``mlp`` is null, x += ff(norm2(x)).
Every norm is a dynamic tanh.  The mixer is chosen per layer by ``type``: ``attention``
(differential attention under a window that keeps a request's first tokens;
``parts/diff_attention.py``) or ``latent_attention`` (``parts/latent_attention.py``).  An attention
layer with ``kv_from`` reads the keys and values of an earlier layer: its schedule entry names that
layer's cache, which then keeps what the widest mask among its readers needs.  The feed-forward is
the clamped gated one (``dense``) or a mixture of experts (``moe``).  After the last layer come the
model's norm and the head.

Tensor names: ``embed``, ``embed.norm``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config import GotulornConfig, register_architecture
from ..parts import LMHead, TokenEmbedding, make_part
from .decoder import DecoderModel, LayerCall

NAMES = {"mixer_norm": "norm1", "mixer": "mix", "ffn_norm": "norm2", "ffn": "mlp"}


def cache_needs(cfg: GotulornConfig):
    """Per attention layer with keys and values of its own: (window, keep_first) that its cache has to
    serve, the widest among the layer itself and the layers that read it (window None: everything)."""
    needs = {}
    for i, layer in enumerate(cfg.layers):
        if layer["type"] != "attention":
            continue
        m = layer["mixer"]
        owner = m.get("kv_from", i) if m.get("kv_from") is not None else i
        mask = m.get("mask")
        window, keep = (mask["size"], mask.get("keep_first", 0)) if mask else (None, 0)
        if owner not in needs:
            needs[owner] = (window, keep)
        else:
            w0, k0 = needs[owner]
            needs[owner] = (None if window is None or w0 is None else max(w0, window), max(k0, keep))
    return needs


def mixer_of(cfg: GotulornConfig, i: int, needs):
    layer = cfg.layers[i]
    m = layer["mixer"]
    if layer["type"] == "attention":
        mask = m.get("mask")
        own = m.get("kv_from") is None
        window, keep = needs.get(i, (None, 0))
        return make_part("mixer", "differential_attention", width=cfg.width, n_heads=m["heads"], n_kv_heads=m["kv_heads"], head_dim=m["dim"],
                         v_head_dim=m["vdim"], scale=m["scale"], diff=m["diff"], eps=cfg.norm_eps, window=mask["size"] if mask else None,
                         keep_first=mask.get("keep_first", 0) if mask else 0, own_kv=own, cache_window=window, cache_keep_first=keep)
    return make_part("mixer", "latent_attention", width=cfg.width, n_heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"],
                     v_head_dim=m["vdim"], rank=m["kv_rank"], scale=m["scale"], eps=cfg.norm_eps, rope_base=m["rot"]["base"],
                     rope_dims=m["rot"]["dims"])


def feed_forward_of(cfg: GotulornConfig, mlp):
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return make_part("feed_forward", "clamped_glu", width=cfg.width, inner=mlp["ff"], limit=mlp["limit"])
    return make_part("feed_forward", "routed_experts", width=cfg.width, inner=mlp["expert"]["ff"], n_experts=mlp["router"]["experts"],
                     top=mlp["router"]["top"])


def build_gotulorn(cfg: GotulornConfig) -> DecoderModel:
    norm = lambda **kw: make_part("norm", "dynamic_tanh", width=cfg.width, **kw)
    needs = cache_needs(cfg)
    blocks, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        ffn = feed_forward_of(cfg, layer.get("mlp"))
        blocks.append(make_part("block", "pre_norm", mixer_norm=norm(), mixer=mixer_of(cfg, i, needs), ffn_norm=norm() if ffn else None,
                                ffn=ffn, names=NAMES))
        src = layer["mixer"].get("kv_from") if layer["type"] == "attention" else None
        schedule.append(LayerCall(i, cache=src))
    embedding = TokenEmbedding(cfg.vocab, cfg.width, name="embed")
    head = LMHead(cfg.vocab, cfg.width, name="head")
    return DecoderModel(cfg, embedding, blocks, norm(), head, schedule=schedule, block_prefix="l{}", final_norm_prefix="final.norm",
                        embed_norm=norm(pre_scale=cfg.embedding_scale), embed_norm_prefix="embed.norm")


register_architecture("Gotulorn", GotulornConfig, build_gotulorn)
