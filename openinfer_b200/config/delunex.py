"""Delunex configuration.

config.json of this design is nested: the model's sizes and constants at the top (``vocab``, ``width``,
``embedding.scale``, ``norm.eps``, ``canon.taps``, ``logit_scale``) and one entry per layer under ``layers``
(``type``, the mixer's sizes under ``mixer``, the feed-forward under ``mlp`` or null). The architecture is named
by the singular key ``architecture``. Every size comes from here or from a tensor's shape; nothing is assumed
equal between layers.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig

MIXER_TYPES = ("latent_attention",)
MLP_KINDS = ("dense",)


def _positive_int(where: str, d: Dict[str, Any], key: str) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or v != int(v) or int(v) <= 0:
        raise ConfigError(f"{where}: {key!r} must be a positive integer, got {v!r}")
    return int(v)


def _number(where: str, d: Dict[str, Any], key: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"{where}: {key!r} must be a number, got {v!r}")
    return float(v)


@dataclasses.dataclass(frozen=True)
class DelunexConfig(ModelConfig):
    architecture = "Delunex"
    model_type = ""

    vocab: int
    width: int
    layers: Tuple[dict, ...]
    embedding: dict
    norm: dict
    logit_scale: float = 1.0
    canon: Optional[dict] = None
    max_position_embeddings: int = 0          # 0: no limit (the design has no position tables)
    stop_token_ids: Tuple[int, ...] = ()

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError(f"vocab and width must be positive, got {self.vocab} and {self.width}")
        if not isinstance(self.embedding, dict) or not isinstance(self.norm, dict):
            raise ConfigError("'embedding' and 'norm' must be objects")
        _number("embedding", self.embedding, "scale")
        if not _number("norm", self.norm, "eps") > 0.0:
            raise ConfigError("norm.eps must be > 0")
        if self.canon is not None:
            if not isinstance(self.canon, dict):
                raise ConfigError("'canon' must be an object")
            _positive_int("canon", self.canon, "taps")
        if not self.layers:
            raise ConfigError("'layers' must list at least one layer")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or not isinstance(layer.get("mixer"), dict):
                raise ConfigError(f"{where}: an object with a 'mixer' object is expected")
            if layer.get("type") not in MIXER_TYPES:
                raise ConfigError(f"{where}: type {layer.get('type')!r} is not known (known: {', '.join(MIXER_TYPES)})")
            m = layer["mixer"]
            for key in ("heads", "dim", "vdim", "kv_rank"):
                _positive_int(where + ".mixer", m, key)
            _number(where + ".mixer", m, "scale")
            if m.get("mask") is not None:
                if not isinstance(m["mask"], dict):
                    raise ConfigError(f"{where}.mixer: 'mask' must be an object")
                _positive_int(where + ".mixer.mask", m["mask"], "size")
            src = m.get("kv_from")
            if src is not None:
                if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i:
                    raise ConfigError(f"{where}.mixer: kv_from {src!r} must name an earlier layer")
                other = self.layers[src]["mixer"]
                if other.get("kv_from") is not None:
                    raise ConfigError(f"{where}.mixer: kv_from names layer {src}, which has no latent of its own")
                if int(other["kv_rank"]) != int(m["kv_rank"]):
                    raise ConfigError(f"{where}.mixer: kv_rank {m['kv_rank']} differs from layer {src}'s {other['kv_rank']}")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") not in MLP_KINDS:
                    raise ConfigError(f"{where}.mlp: kind must be one of {', '.join(MLP_KINDS)}, or the mlp null")
                _positive_int(where + ".mlp", mlp, "ff")

    def with_stop_token_ids(self, ids) -> "DelunexConfig":
        return dataclasses.replace(self, stop_token_ids=tuple(int(i) for i in ids))

    @property
    def taps(self) -> int:
        return int(self.canon["taps"]) if self.canon else 0

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "embedding": dict(self.embedding), "norm": dict(self.norm), "logit_scale": self.logit_scale,
            "layers": [dict(layer) for layer in self.layers],
        }
        if self.canon is not None:
            d["canon"] = dict(self.canon)
        if self.max_position_embeddings:
            d["max_position_embeddings"] = self.max_position_embeddings
        return d
