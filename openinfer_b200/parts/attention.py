"""Attention mixer over the paged cache: grouped-query, causal, optional window,
optional per-head q/k norm, optional rotation.

One fused projection q|k|v (the reference also stores the three matrices as one,
pegainfer-qwen3/src/weights/load.rs:98-134), then the fused norm + rotation + cache
write, attention over the request's pages, and the output projection
(pegainfer-qwen3/src/unified_forward.rs:414-536). When the call reads another call's
cache only the query projection exists and nothing is written.

Queries / keys of ``qk_dim`` and values of ``v_dim`` numbers per head (``AttentionSpec.qk_dim``, ``v_dim``) run on the same
kernels: the cached row is ``head_dim`` (a multiple of 8 that holds both), the projections get zero rows up to it when
they are loaded (zeros change neither a score nor a value), and a per-head norm over qk_dim numbers is the norm over
head_dim with eps * qk_dim / head_dim whose result is long by sqrt(head_dim / qk_dim) in q and in k alike, which the
softmax scale takes back.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache.manager import KvNeed
from ..kernels import attention as attn_kernels
from ..kernels.linear import linear
from .base import CacheBinding, Mixer
from .registry import build_position_encoding, register_mixer
from .spec import AttentionSpec, ParamInfo


@register_mixer("attention")
class Attention(Mixer):
    graph_safe = True

    def __init__(self, spec: AttentionSpec) -> None:
        super().__init__(spec)
        s = spec
        if s.num_heads % s.num_kv_heads:
            raise ValueError(f"num_heads ({s.num_heads}) must be a multiple of num_kv_heads ({s.num_kv_heads})")
        if s.head_dim % 8 or s.head_dim > 512:
            raise ValueError(f"head_dim {s.head_dim} unsupported: multiples of 8 up to 512")
        self.qk = s.qk_dim or s.head_dim
        self.vd = s.v_dim or s.head_dim
        if self.qk > s.head_dim or self.vd > s.head_dim:
            raise ValueError(f"head_dim {s.head_dim} must hold queries of {self.qk} and values of {self.vd} numbers")
        self.q_dim = s.num_heads * s.head_dim
        self.kv_dim = s.num_kv_heads * s.head_dim
        # a norm over qk of head_dim numbers (see the file's head)
        self.norm_eps_factor = self.qk / s.head_dim
        self.scale = s.softmax_scale * (self.qk / s.head_dim if (s.qk_norm is not None and self.qk != s.head_dim) else 1.0)
        self.position = build_position_encoding(s.position)
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.q_norm_w: Optional[torch.Tensor] = None
        self.k_norm_w: Optional[torch.Tensor] = None
        self.tables = None

    def kv_need(self) -> Optional[KvNeed]:
        s = self.spec
        return KvNeed(s.num_kv_heads, s.head_dim, s.window)

    def parameters(self) -> Dict[str, ParamInfo]:
        s = self.spec
        p = {
            s.q_name: ParamInfo((s.num_heads * self.qk, s.hidden_size)),
            s.k_name: ParamInfo((s.num_kv_heads * self.qk, s.hidden_size)),
            s.v_name: ParamInfo((s.num_kv_heads * self.vd, s.hidden_size)),
            s.o_name: ParamInfo((s.hidden_size, s.num_heads * self.vd)),
        }
        if s.qk_norm is not None:
            p[s.q_norm_name] = ParamInfo((self.qk,), ("one_plus_normal", 0.02))
            p[s.k_norm_name] = ParamInfo((self.qk,), ("one_plus_normal", 0.02))
        return p

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        q, k, v = tensors[s.q_name], tensors[s.k_name], tensors[s.v_name]
        if not (q.dtype == k.dtype == v.dtype):
            raise ValueError("the q, k and v projections must be stored in one dtype to be fused")
        hd = s.head_dim

        def rows_padded(w, heads, size):       # [heads * size, in] -> [heads * head_dim, in], zero rows behind each head's
            if size == hd:
                return w
            out = torch.zeros((heads, hd, w.shape[1]), dtype=w.dtype, device=w.device)
            out[:, :size] = w.view(heads, size, -1)
            return out.view(heads * hd, -1)

        self.w_qkv = torch.cat([rows_padded(q, s.num_heads, self.qk), rows_padded(k, s.num_kv_heads, self.qk),
                                rows_padded(v, s.num_kv_heads, self.vd)], dim=0).contiguous()
        o = tensors[s.o_name]
        if self.vd != hd:
            wide = torch.zeros((o.shape[0], s.num_heads, hd), dtype=o.dtype, device=o.device)
            wide[:, :, : self.vd] = o.view(o.shape[0], s.num_heads, self.vd)
            o = wide.view(o.shape[0], s.num_heads * hd)
        self.w_o = o.contiguous()
        if self.spec.qk_norm is not None:
            def norm_padded(w):
                if self.qk == hd:
                    return w.contiguous()
                out = torch.zeros(hd, dtype=w.dtype, device=w.device)
                out[: self.qk] = w
                return out

            self.q_norm_w = norm_padded(tensors[s.q_norm_name])
            self.k_norm_w = norm_padded(tensors[s.k_norm_name])
            if self.q_norm_w.dtype != self.k_norm_w.dtype:
                self.k_norm_w = self.k_norm_w.to(self.q_norm_w.dtype)

    def prepare(self, device: torch.device, dtype: torch.dtype) -> None:
        self.tables = self.position.rotation_tables(device)

    takes_out_dtype = True

    def forward(self, x: torch.Tensor, ctx, binding: CacheBinding, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        s = self.spec
        if binding.kv is None:
            raise RuntimeError("attention needs a cache binding")
        group = ctx.groups[binding.kv.group]
        k_cache, v_cache, page_stride = ctx.cache.kv_views(binding.kv)
        w = self.w_qkv if binding.owns_kv else self.w_qkv[: self.q_dim]
        qkv = linear(x, w)
        cos, sin = self.tables if self.tables is not None else (None, None)
        qn = s.qk_norm
        out = torch.empty((x.shape[0], self.q_dim), dtype=x.dtype, device=x.device)
        # One native call: the norm + rotation + cache write (in a kernel of its own, or inside the decode kernel when
        # the step is single tokens in one wave), then the attention kernel(s) that take the step's shape.
        step = attn_kernels.attention_step(ctx, group, qkv, out, k_cache, page_stride, s.num_heads, s.num_kv_heads,
                                           s.head_dim, s.window, cos=cos, q_norm_w=self.q_norm_w)
        layer = attn_kernels.attention_layer(
            qkv, out, k_cache, v_cache, s.num_heads, s.num_kv_heads, s.head_dim, self.scale, s.window,
            q_norm_w=self.q_norm_w, k_norm_w=self.k_norm_w, eps=qn.eps * self.norm_eps_factor if qn else 0.0,
            weight_offset=qn.weight_offset if qn else 0.0, cos=cos, sin=sin, write_kv=binding.owns_kv, rope_mode=1,
            interleaved=bool(getattr(s.position, "interleaved", False)))
        attn_kernels.run_attention(step, layer)
        return linear(out, self.w_o, out_dtype=out_dtype)
