"""The Lefulorn decoder: which parts a ``LefulornConfig`` asks for, layer by layer.

Every layer is pre-norm: x += mixer(norm1(x)), then, unless its ``mlp`` is null,
x += ff(norm2(x)).  The mixer is chosen per layer by ``type``: ``attention`` (a window, a
distance bias, a sink, a temperature on the queries, values mixed with those of the first
value-mixing layer, an output gate; ``parts/sink_attention.py``) or ``channel_delta`` (the
gated delta rule with a decay per key channel; ``parts/delta.py``).  The feed-forward is dense
with a squared relu.  After the last layer come the model's norm and the head, whose logits
are multiplied by ``logit_scale``.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config import LefulornConfig, register_architecture
from ..parts import LMHead, TokenEmbedding, make_part
from .decoder import DecoderModel

NAMES = {"mixer_norm": "norm1", "mixer": "mix", "ffn_norm": "norm2", "ffn": "mlp"}


def mixer_of(cfg: LefulornConfig, layer: dict, first_mixing: bool):
    m = layer["mixer"]
    common = dict(width=cfg.width, n_heads=m["heads"], n_kv_heads=m["kv_heads"], head_dim=m["dim"], v_head_dim=m["vdim"])
    if layer["type"] == "attention":
        qt = m.get("q_temp")
        mask = m.get("mask")
        return make_part("mixer", "sink_attention", scale=m["scale"], window=mask["size"] if mask else None,
                         temperature=(qt["coef"], qt["every"]) if qt else None,
                         v_mix=("keep" if first_mixing else "mix") if m.get("v_mix") else None, **common)
    return make_part("mixer", "channel_delta", taps=m["conv"], rank_a=m.get("rank_a", cfg.default_rank),
                     rank_g=m.get("rank_g", cfg.default_rank), eps=cfg.norm_eps, **common)


def build_lefulorn(cfg: LefulornConfig) -> DecoderModel:
    norm = lambda: make_part("norm", "rmsnorm", width=cfg.width, eps=cfg.norm_eps, suffix="")
    blocks = []
    seen_mixing = False
    for layer in cfg.layers:
        mixes = layer["type"] == "attention" and bool(layer["mixer"].get("v_mix"))
        mixer = mixer_of(cfg, layer, first_mixing=mixes and not seen_mixing)
        seen_mixing = seen_mixing or mixes
        mlp = layer.get("mlp")
        ffn = make_part("feed_forward", "dense_mlp", width=cfg.width, inner=mlp["ff"]) if mlp else None
        blocks.append(make_part("block", "pre_norm", mixer_norm=norm(), mixer=mixer, ffn_norm=norm() if mlp else None, ffn=ffn,
                                names=NAMES))
    embedding = TokenEmbedding(cfg.vocab, cfg.width, name="embed")
    head = LMHead(cfg.vocab, cfg.width, name="head")
    return DecoderModel(cfg, embedding, blocks, norm(), head, block_prefix="l{}", final_norm_prefix="final.norm",
                        logit_scale=cfg.logit_scale if cfg.logit_scale != 1.0 else None)


register_architecture("Lefulorn", LefulornConfig, build_lefulorn)
