"""Pilonex configuration.

config.json of this design is nested: ``vocab``, ``width``, ``norm.eps``, optionally ``streams`` (residual streams with
hyper-connection coefficients per sublayer) and ``loop`` (``start``, ``stop``, ``times``: layers start .. stop - 1 run
``times`` times in a row with the same weights), and one entry per layer under ``layers``: ``type`` ("mlstm" or
"parallel"), the mixer's sizes under ``mixer`` and the feed-forward under ``mlp`` (``kind`` "dense" or "moe", or null).
A "parallel" mixer has a ``left`` (windowed attention: heads, kv_heads, dim, vdim, scale, optional mask.size, optional
rot with dims, base and optional scaling) and a ``right`` (gated delta rule: heads, kv_heads, dim, vdim, conv) with
``left_scale`` and ``right_scale``. Every size comes from here or from a tensor's shape; nothing is assumed equal between
layers.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig
from .delunex import _number, _positive_int

MIXER_TYPES = ("mlstm", "parallel")
MLP_KINDS = ("dense", "moe")


def _object(where: str, d: Dict[str, Any], key: str) -> Dict[str, Any]:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: {key!r} must be an object, got {v!r}")
    return v


@dataclasses.dataclass(frozen=True)
class PilonexConfig(ModelConfig):
    architecture = "Pilonex"
    model_type = ""

    vocab: int
    width: int
    layers: Tuple[dict, ...]
    norm: dict
    streams: Optional[int] = None
    loop: Optional[dict] = None
    max_position_embeddings: int = 65536      # positions the rotation tables are made for
    stop_token_ids: Tuple[int, ...] = ()

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError(f"vocab and width must be positive, got {self.vocab} and {self.width}")
        if not isinstance(self.norm, dict) or not _number("norm", self.norm, "eps") > 0.0:
            raise ConfigError("norm.eps must be a number > 0")
        if self.streams is not None and not 1 <= self.streams <= 16:
            raise ConfigError(f"streams must be 1 to 16, got {self.streams}")
        if not self.layers:
            raise ConfigError("'layers' must list at least one layer")
        if self.loop is not None:
            if not isinstance(self.loop, dict):
                raise ConfigError("'loop' must be an object")
            times = _positive_int("loop", self.loop, "times")
            start, stop = self.loop.get("start"), self.loop.get("stop")
            if not all(isinstance(v, int) and not isinstance(v, bool) for v in (start, stop)) or not 0 <= start <= stop <= len(self.layers):
                raise ConfigError(f"loop: start {start!r} and stop {stop!r} must bound a run of the {len(self.layers)} layers")
            del times
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or not isinstance(layer.get("mixer"), dict):
                raise ConfigError(f"{where}: an object with a 'mixer' object is expected")
            if layer.get("type") not in MIXER_TYPES:
                raise ConfigError(f"{where}: type {layer.get('type')!r} is not known (known: {', '.join(MIXER_TYPES)})")
            m = layer["mixer"]
            if layer["type"] == "mlstm":
                for key in ("heads", "dim", "vdim"):
                    _positive_int(where + ".mixer", m, key)
                if not _number(where + ".mixer", m, "gate_cap") > 0.0:
                    raise ConfigError(f"{where}.mixer: gate_cap must be > 0")
            else:
                left, right = _object(where + ".mixer", m, "left"), _object(where + ".mixer", m, "right")
                _number(where + ".mixer", m, "left_scale")
                _number(where + ".mixer", m, "right_scale")
                for side, d, keys in (("left", left, ("heads", "kv_heads", "dim", "vdim")),
                                      ("right", right, ("heads", "kv_heads", "dim", "vdim", "conv"))):
                    for key in keys:
                        _positive_int(f"{where}.mixer.{side}", d, key)
                    if d["heads"] % d["kv_heads"]:
                        raise ConfigError(f"{where}.mixer.{side}: heads {d['heads']} must be a multiple of kv_heads {d['kv_heads']}")
                _number(where + ".mixer.left", left, "scale")
                if left.get("mask") is not None:
                    _positive_int(where + ".mixer.left.mask", _object(where + ".mixer.left", left, "mask"), "size")
                rot = left.get("rot")
                if rot is not None:
                    rot = _object(where + ".mixer.left", left, "rot")
                    dims = _positive_int(where + ".mixer.left.rot", rot, "dims")
                    if dims % 2 or dims > left["dim"]:
                        raise ConfigError(f"{where}.mixer.left.rot: dims {dims} must be even and at most dim {left['dim']}")
                    if not _number(where + ".mixer.left.rot", rot, "base") > 0.0:
                        raise ConfigError(f"{where}.mixer.left.rot: base must be > 0")
                    if rot.get("scaling") is not None:
                        sc = _object(where + ".mixer.left.rot", rot, "scaling")
                        for key in ("factor", "low", "high", "original"):
                            _number(where + ".mixer.left.rot.scaling", sc, key)
                        if sc["factor"] == 0:
                            raise ConfigError(f"{where}.mixer.left.rot.scaling: factor must differ from 0")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") not in MLP_KINDS:
                    raise ConfigError(f"{where}.mlp: kind must be one of {', '.join(MLP_KINDS)}, or the mlp null")
                if mlp["kind"] == "dense":
                    _positive_int(where + ".mlp", mlp, "ff")
                    _number(where + ".mlp", mlp, "limit")
                else:
                    expert, router = _object(where + ".mlp", mlp, "expert"), _object(where + ".mlp", mlp, "router")
                    _positive_int(where + ".mlp.expert", expert, "ff")
                    _number(where + ".mlp.expert", expert, "limit")
                    n, top = _positive_int(where + ".mlp.router", router, "experts"), _positive_int(where + ".mlp.router", router, "top")
                    if top > n or top > 32:
                        raise ConfigError(f"{where}.mlp.router: top {top} of {n} experts (at most 32 a token)")

    def with_stop_token_ids(self, ids) -> "PilonexConfig":
        return dataclasses.replace(self, stop_token_ids=tuple(int(i) for i in ids))

    def run_order(self) -> Tuple[int, ...]:
        """Layer indices in the order they run: the looped run repeated ``times`` times in a row."""
        n = len(self.layers)
        if not self.loop:
            return tuple(range(n))
        a, b, k = int(self.loop["start"]), int(self.loop["stop"]), int(self.loop["times"])
        return tuple(range(a)) + tuple(range(a, b)) * k + tuple(range(b, n))

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": dict(self.norm),
                             "layers": [dict(layer) for layer in self.layers]}
        if self.streams is not None:
            d["streams"] = self.streams
        if self.loop is not None:
            d["loop"] = dict(self.loop)
        if self.max_position_embeddings != 65536:
            d["max_position_embeddings"] = self.max_position_embeddings
        return d
