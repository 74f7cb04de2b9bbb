"""Two mixers side by side: both read the same rows, the result is left_scale * left + right_scale * right.

The two are whatever mixers their specs name (an attention beside a recurrence, for instance); each keeps its own tensors
under its own prefix, the cache entry is the one that asks for pages, and the state slots are the left's followed by the
right's. Both hand their results back in float32; the weighted sum is formed by the kernel that carries a block's result into
its streams when the block asks for the pair (``as_pair``), else by a kernel of its own.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional

import torch

from ..cache.manager import KvNeed, StateNeed
from ..kernels import ops
from .base import CacheBinding, Mixer
from .registry import build_mixer, register_mixer
from .spec import ParallelMixerSpec, ParamInfo


@register_mixer("parallel")
class ParallelMixer(Mixer):
    takes_out_dtype = True
    returns_pair = True      # forward(as_pair=True) hands back both sides and their scales instead of the sum

    def __init__(self, spec: ParallelMixerSpec) -> None:
        super().__init__(spec)
        self.left = build_mixer(spec.left)
        self.right = build_mixer(spec.right)
        if self.left.kv_need() is not None and self.right.kv_need() is not None:
            raise ValueError("a parallel mixer takes at most one side with paged keys and values")
        for side in (self.left, self.right):
            if not getattr(side, "takes_out_dtype", False):
                raise ValueError(f"a parallel mixer needs sides that can return float32, {type(side).__name__} cannot")

    @property
    def graph_safe(self) -> bool:
        return bool(self.left.graph_safe and self.right.graph_safe)

    def _sides(self):
        return ((self.spec.left_name, self.left), (self.spec.right_name, self.right))

    def parameters(self) -> Dict[str, ParamInfo]:
        return {prefix + name: info for prefix, side in self._sides() for name, info in side.parameters().items()}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        for prefix, side in self._sides():
            side.load({name: tensors[prefix + name] for name in side.parameters()})

    def prepare(self, device: torch.device, dtype: torch.dtype) -> None:
        self.left.prepare(device, dtype)
        self.right.prepare(device, dtype)

    def kv_need(self) -> Optional[KvNeed]:
        return self.left.kv_need() or self.right.kv_need()

    def state_needs(self) -> List[StateNeed]:
        return self.left.state_needs() + self.right.state_needs()

    def forward(self, x: torch.Tensor, ctx, binding: CacheBinding, out_dtype: Optional[torch.dtype] = None, as_pair: bool = False):
        n_left = len(self.left.state_needs())
        kv_left = self.left.kv_need() is not None
        lb = dataclasses.replace(binding, kv=binding.kv if kv_left else None, states=binding.states[:n_left])
        rb = dataclasses.replace(binding, kv=None if kv_left else binding.kv, states=binding.states[n_left:])
        a = self.left.forward(x, ctx, lb, out_dtype=torch.float32)
        b = self.right.forward(x, ctx, rb, out_dtype=torch.float32)
        if as_pair:
            return a, b, float(self.spec.left_scale), float(self.spec.right_scale)
        out = ops.scaled_sum(torch.empty_like(a), a, b, self.spec.left_scale, self.spec.right_scale)
        return out if out_dtype in (None, torch.float32) else out.to(out_dtype)
