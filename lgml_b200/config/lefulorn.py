"""Configuration of the Lefulorn decoder, from its own ``config.json`` keys.

The file names the architecture under ``architecture`` and lists its layers one by one under
``layers``: each entry has ``type`` (the mixer: ``attention`` or ``channel_delta``), ``mixer``
(that mixer's sizes and constants) and ``mlp`` (the feed-forward, or null for a layer without
one).  Everything that can differ between two models of the design is read here; what the
design fixes (the distance slopes, the unit norms' epsilon) lives with the parts.

attention ``mixer``: ``heads``, ``kv_heads``, ``dim`` (q and k per head), ``vdim`` (v per
head), ``scale`` (of the scores), ``mask.size`` (the window; absent: every earlier token),
``q_temp.coef`` / ``q_temp.every`` (the queries' temperature by position; absent: none),
``v_mix`` (values mixed with those of the first such layer).

channel_delta ``mixer``: ``heads``, ``kv_heads``, ``dim`` (keys per head), ``vdim`` (values per
head), ``conv`` (taps of the short convolutions).  The rank of its two low-rank projections is
not in the file: it is the shape of their tensors, and the loader reads it from the folder.

``mlp``: ``kind`` (``dense``) and ``ff`` (the inner width).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError, ModelConfig

MIXERS = ("attention", "channel_delta")
MLP_KINDS = ("dense",)


def _positive_int(where: str, d: Dict[str, Any], key: str) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, not {v!r}")
    return v


@dataclass
class LefulornConfig(ModelConfig):
    architecture: str = "Lefulorn"
    vocab: int = 0
    width: int = 0
    norm_eps: float = 0.0
    logit_scale: float = 1.0
    layers: List[Dict[str, Any]] = field(default_factory=list)
    # the rank of a channel_delta layer's low-rank projections, when the layer's entry does not
    # give one ("rank"): random-weights mode needs a number, a folder's tensors carry their own
    default_rank: int = 16
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
    def from_dict(cls, d: Dict[str, Any]) -> "LefulornConfig":
        for key in ("vocab", "width", "layers", "norm"):
            if key not in d or d[key] is None:
                raise ConfigError(f"config.json: '{key}' is missing")
        norm = d["norm"]
        if not isinstance(norm, dict) or "eps" not in norm:
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        if not isinstance(d["layers"], list):
            raise ConfigError("config.json: 'layers' must be a list")
        layers = copy.deepcopy(d["layers"])
        for layer in layers:        # sizes a mixer may leave out: KV heads default to the heads, values to the keys' size
            m = layer.get("mixer") if isinstance(layer, dict) else None
            if isinstance(m, dict):
                if "heads" in m:
                    m.setdefault("kv_heads", m["heads"])
                if "dim" in m:
                    m.setdefault("vdim", m["dim"])
        return cls(vocab=int(d["vocab"]), width=int(d["width"]), norm_eps=float(norm["eps"]),
                   logit_scale=float(d.get("logit_scale", 1.0)), layers=layers,
                   torch_dtype=str(d.get("torch_dtype", "bfloat16")))

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        if not self.norm_eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        if not self.layers:
            raise ConfigError("config.json: 'layers' is empty")
        mixed = None        # (kv_heads, vdim) of the first value-mixing layer
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in MIXERS:
                raise ConfigError(f"config.json: {where}.type must be one of {MIXERS}, not {layer.get('type') if isinstance(layer, dict) else layer!r}")
            m = layer.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: {where}.mixer must be an object")
            mw = where + ".mixer"
            heads, kv = _positive_int(mw, m, "heads"), _positive_int(mw, m, "kv_heads")
            _positive_int(mw, m, "dim")
            _positive_int(mw, m, "vdim")
            if heads % kv:
                raise ConfigError(f"config.json: {mw}.heads {heads} is no multiple of kv_heads {kv}")
            if layer["type"] == "attention":
                if "scale" not in m:
                    raise ConfigError(f"config.json: {mw}.scale is missing")
                if m.get("mask") is not None:
                    _positive_int(mw + ".mask", m["mask"], "size")
                if m.get("q_temp") is not None:
                    _positive_int(mw + ".q_temp", m["q_temp"], "every")
                    if "coef" not in m["q_temp"]:
                        raise ConfigError(f"config.json: {mw}.q_temp.coef is missing")
                if m.get("v_mix"):
                    if mixed is None:
                        mixed = (kv, m["vdim"])
                    elif mixed != (kv, m["vdim"]):
                        raise ConfigError(f"config.json: {mw}: a value-mixing layer needs the first one's kv_heads and vdim {mixed}")
            else:
                _positive_int(mw, m, "conv")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") not in MLP_KINDS:
                    raise ConfigError(f"config.json: {where}.mlp.kind must be one of {MLP_KINDS}")
                _positive_int(where + ".mlp", mlp, "ff")

    def complete_from_folder(self, folder) -> None:
        """Sizes that only the folder's tensors give: the ranks of the low-rank projections of
        every channel_delta layer (rows of ``a1`` and ``g1``)."""
        from ..weights.safetensors import SafetensorsError, index_folder

        try:
            index = index_folder(folder)
        except (SafetensorsError, OSError):
            return          # a folder without weights: the loader will say so
        for i, layer in enumerate(self.layers):
            if layer.get("type") != "channel_delta":
                continue
            for key, name in (("rank_a", "a1"), ("rank_g", "g1")):
                ent = index.get(f"l{i}.mix.{name}")
                if ent is not None and len(ent.shape) == 2:
                    layer["mixer"][key] = int(ent.shape[0])

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "logit_scale": self.logit_scale, "layers": copy.deepcopy(self.layers)}
