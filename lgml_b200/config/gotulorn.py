"""Configuration of the Gotulorn decoder, from its own ``config.json`` keys.

``architecture`` names it; ``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` are the model's
own numbers; ``layers`` lists the layers one by one: ``type`` (the mixer: ``attention`` or
``latent_attention``), ``mixer`` (its sizes and constants) and ``mlp`` (the feed-forward, or null for
a layer without one).

attention ``mixer`` (differential attention under a window that keeps the first tokens): ``heads``,
``kv_heads``, ``dim`` (per map), ``vdim``, ``scale``, ``diff``, ``mask.size`` / ``mask.keep_first``
(absent: every earlier token), ``kv_from`` (the layer whose keys and values it reads instead of
projecting its own).

latent_attention ``mixer``: ``heads``, ``dim`` (unrotated per head), ``rot_dim`` (rotated, shared by
the heads on the key side), ``vdim``, ``kv_rank``, ``scale``, ``rot.base`` / ``rot.dims``.

``mlp``: ``kind`` ``dense`` with ``ff`` and ``limit``, or ``moe`` with ``expert.ff``,
``router.experts`` and ``router.top``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List

from .base import ConfigError, ModelConfig

MIXERS = ("attention", "latent_attention")
MLP_KINDS = ("dense", "moe")


def _positive_int(where: str, d: Dict[str, Any], key: str) -> int:
    v = d.get(key) if isinstance(d, dict) else None
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, not {v!r}")
    return v


def _number(where: str, d: Dict[str, Any], key: str) -> float:
    v = d.get(key) if isinstance(d, dict) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, not {v!r}")
    return float(v)


@dataclass
class GotulornConfig(ModelConfig):
    architecture: str = "Gotulorn"
    vocab: int = 0
    width: int = 0
    norm_eps: float = 0.0
    embedding_scale: float = 1.0
    layers: List[Dict[str, Any]] = field(default_factory=list)
    torch_dtype: str = "bfloat16"

    # the names other parts of the engine ask a configuration for
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "GotulornConfig":
        for key in ("vocab", "width", "layers", "norm"):
            if key not in d or d[key] is None:
                raise ConfigError(f"config.json: '{key}' is missing")
        norm = d["norm"]
        if not isinstance(norm, dict) or "eps" not in norm:
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        if not isinstance(d["layers"], list):
            raise ConfigError("config.json: 'layers' must be a list")
        emb = d.get("embedding") or {}
        if not isinstance(emb, dict):
            raise ConfigError("config.json: 'embedding' must be an object")
        layers = copy.deepcopy(d["layers"])
        for layer in layers:        # sizes a mixer may leave out: KV heads default to the heads, values to the keys' size
            m = layer.get("mixer") if isinstance(layer, dict) else None
            if isinstance(m, dict) and layer.get("type") == "attention":
                if "heads" in m:
                    m.setdefault("kv_heads", m["heads"])
                if "dim" in m:
                    m.setdefault("vdim", m["dim"])
        return cls(vocab=int(d["vocab"]), width=int(d["width"]), norm_eps=float(norm["eps"]), embedding_scale=float(emb.get("scale", 1.0)),
                   layers=layers, torch_dtype=str(d.get("torch_dtype", "bfloat16")))

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        if not self.norm_eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        if not self.layers:
            raise ConfigError("config.json: 'layers' is empty")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in MIXERS:
                raise ConfigError(f"config.json: {where}.type must be one of {MIXERS}, not {layer.get('type') if isinstance(layer, dict) else layer!r}")
            m = layer.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: {where}.mixer must be an object")
            mw = where + ".mixer"
            heads = _positive_int(mw, m, "heads")
            _positive_int(mw, m, "dim")
            _positive_int(mw, m, "vdim")
            _number(mw, m, "scale")
            if layer["type"] == "attention":
                kv = _positive_int(mw, m, "kv_heads")
                if heads % kv:
                    raise ConfigError(f"config.json: {mw}.heads {heads} is no multiple of kv_heads {kv}")
                _number(mw, m, "diff")
                if m.get("mask") is not None:
                    _positive_int(mw + ".mask", m["mask"], "size")
                    kf = m["mask"].get("keep_first", 0)
                    if isinstance(kf, bool) or not isinstance(kf, int) or kf < 0:
                        raise ConfigError(f"config.json: {mw}.mask.keep_first must be a non-negative integer, not {kf!r}")
                src = m.get("kv_from")
                if src is not None:
                    if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i:
                        raise ConfigError(f"config.json: {mw}.kv_from must name an earlier layer, not {src!r}")
                    other = self.layers[src]
                    om = other.get("mixer", {})
                    if other.get("type") != "attention" or om.get("kv_from") is not None:
                        raise ConfigError(f"config.json: {mw}.kv_from {src} is no attention layer with keys and values of its own")
                    for key in ("kv_heads", "dim", "vdim"):
                        if om.get(key) != m.get(key):
                            raise ConfigError(f"config.json: {mw}.{key} {m.get(key)!r} differs from layer {src}'s {om.get(key)!r}, whose keys and values it reads")
            else:
                _positive_int(mw, m, "rot_dim")
                _positive_int(mw, m, "kv_rank")
                rot = m.get("rot")
                if not isinstance(rot, dict):
                    raise ConfigError(f"config.json: {mw}.rot must be an object with 'base' and 'dims'")
                _number(mw + ".rot", rot, "base")
                dims = _positive_int(mw + ".rot", rot, "dims")
                if dims % 2 or dims > m["rot_dim"]:
                    raise ConfigError(f"config.json: {mw}.rot.dims {dims} must be even and at most rot_dim {m['rot_dim']}")
            mlp = layer.get("mlp")
            if mlp is not None:
                fw = where + ".mlp"
                if not isinstance(mlp, dict) or mlp.get("kind") not in MLP_KINDS:
                    raise ConfigError(f"config.json: {fw}.kind must be one of {MLP_KINDS}")
                if mlp["kind"] == "dense":
                    _positive_int(fw, mlp, "ff")
                    _number(fw, mlp, "limit")
                else:
                    _positive_int(fw + ".expert", mlp.get("expert"), "ff")
                    n = _positive_int(fw + ".router", mlp.get("router"), "experts")
                    top = _positive_int(fw + ".router", mlp.get("router"), "top")
                    if top > n:
                        raise ConfigError(f"config.json: {fw}.router.top {top} is more than its {n} experts")

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "embedding": {"scale": self.embedding_scale}, "layers": copy.deepcopy(self.layers)}
