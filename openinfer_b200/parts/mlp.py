"""Gated feed-forward: down( act(gate x) * (up x) ), act chosen by the spec ("silu": SwiGLU, the
reference's; "gelu_tanh": the tanh form of GELU).

gate and up are one fused [2*intermediate, hidden] matrix, as in the reference
(pegainfer-qwen3/src/weights/load.rs:136-154), so one product feeds the activation kernel
(pegainfer-qwen3/src/unified_forward.rs:557-595).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import gemm_tcgen05, native, ops
from ..kernels import lib as _lib
from ..kernels.linear import ensure_library, linear
from .base import FeedForward
from .registry import register_feed_forward
from .spec import GatedMlpSpec, ParamInfo



@register_feed_forward("gated_mlp")
class GatedMlp(FeedForward):
    def __init__(self, spec: GatedMlpSpec) -> None:
        super().__init__(spec)
        self.act_code = ops.glu_code(spec.activation)   # refuses a name no kernel knows; the kernels take the code
        # activations with a limit are formed by the stand-alone kernel behind the plain gate|up product
        self.fused = spec.activation in ops.ACTIVATIONS
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamInfo]:
        s = self.spec
        return {
            s.gate_name: ParamInfo((s.intermediate_size, s.hidden_size)),
            s.up_name: ParamInfo((s.intermediate_size, s.hidden_size)),
            s.down_name: ParamInfo((s.hidden_size, s.intermediate_size)),
        }

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        g, u = tensors[self.spec.gate_name], tensors[self.spec.up_name]
        if g.dtype != u.dtype:
            raise ValueError("gate_proj and up_proj must be stored in one dtype to be fused")
        inter = self.spec.intermediate_size
        # Rows of the fused matrix: blocks of `block` gate rows followed by the up rows of the same
        # indices. With block = 64 a 128-row tile of the tensor-core products holds a gate block and
        # its up block side by side, and the activation is formed in those kernels' epilogues.
        self.block = gemm_tcgen05.ACT_BLOCK if (g.dtype == torch.bfloat16 and inter % gemm_tcgen05.ACT_BLOCK == 0) else inter
        nb = inter // self.block
        self.w_gate_up = torch.stack([g.view(nb, self.block, -1), u.view(nb, self.block, -1)], dim=1).reshape(2 * inter, -1).contiguous()
        self.w_down = tensors[self.spec.down_name].contiguous()

    takes_out_dtype = True

    def _gate_up_with_activation(self, act: torch.Tensor, x: torch.Tensor, L) -> bool:
        """act = activation(gate, up) by ONE product kernel, when one takes the operands."""
        from ..kernels import policy
        s = self.spec
        M, N, K = x.shape[0], self.w_gate_up.shape[0], x.shape[1]
        if (x.dtype != torch.bfloat16 or self.w_gate_up.dtype != torch.bfloat16 or self.block != gemm_tcgen05.ACT_BLOCK or K % 8
                or x.data_ptr() % 16 or policy.batch_invariant()):
            return False
        if M <= 32 and N % 128 == 0:
            _lib.check(L.oi_gemm_stream_glu(act.data_ptr(), 1, act.stride(0), x.data_ptr(), x.stride(0), self.w_gate_up.data_ptr(),
                                            self.w_gate_up.stride(0), M, N, K, L.oi_stream_slices(N, K), self.act_code, float(s.limit),
                                            _lib.current_stream()), "gemm_stream_glu")
            return True
        if M >= 128 and N % 256 == 0:
            _lib.check(L.oi_gemm_tcgen05_glu(act.data_ptr(), act.stride(0), x.data_ptr(), x.stride(0), self.w_gate_up.data_ptr(),
                                             self.w_gate_up.stride(0), M, N, K, 1 if M >= 2048 else 0, self.act_code, float(s.limit),
                                             _lib.current_stream()), "gemm_tcgen05_glu")
            return True
        return False

    def forward(self, x: torch.Tensor, ctx, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """One native call (``oi_gated_mlp``): it picks, by the step's rows, the product that forms the activation in
        its epilogue (tcgen05 tiles from 128 rows, the weight stream up to 32) or the plain product and the
        stand-alone activation kernel, then the down projection."""
        s = self.spec
        M, inter = x.shape[0], s.intermediate_size
        L = _lib.load()
        codes = native.DTYPE_CODE
        if not x.is_contiguous():
            x = x.contiguous()
        if M > 32:
            ensure_library(x.device)
        if not self.fused or out_dtype not in (None, x.dtype):
            # an activation with a limit, or a float32 result: the gate/up product with the activation in its epilogue where
            # a hand-written product takes the shape (the weight stream up to 32 rows, tcgen05 tiles from 128), else the
            # plain product and the activation kernel; then the down projection
            act = torch.empty((M, inter), dtype=x.dtype, device=x.device)
            if not self._gate_up_with_activation(act, x, L):
                gate_up = linear(x, self.w_gate_up)
                ops.glu_act(act, gate_up, self.block, s.activation, s.limit)
            return linear(act, self.w_down, out_dtype=out_dtype)
        out = torch.empty((M, s.hidden_size), dtype=x.dtype, device=x.device)
        act = torch.empty((M, inter), dtype=x.dtype, device=x.device)
        gate_up = None
        if L.oi_gated_mlp_needs_gate_up(codes[x.dtype], codes[self.w_gate_up.dtype], M, s.hidden_size, inter, self.block):
            gate_up = torch.empty((M, 2 * inter), dtype=x.dtype, device=x.device)
        _lib.check(L.oi_gated_mlp(out.data_ptr(), x.data_ptr(), codes[x.dtype], M, s.hidden_size, inter,
                                  self.w_gate_up.data_ptr(), codes[self.w_gate_up.dtype], self.w_down.data_ptr(),
                                  codes[self.w_down.dtype], self.act_code, self.block, act.data_ptr(), 0 if gate_up is None else gate_up.data_ptr(),
                                  _lib.current_stream()), "gated_mlp")
        return out


@register_feed_forward("dense_mlp")
class DenseMlp(FeedForward):
    """down( act(up x) ) with one up-projection; "xielu" is a quadratic above zero and an exponential below it,
    a_p z^2 + z / 2 and a_n (e^z - 1 - z) + z / 2, whose a_p = softplus(p) and a_n = 1/2 + softplus(q) come from a tensor
    of two numbers and are formed on the device in float32."""

    takes_out_dtype = True

    def __init__(self, spec) -> None:
        super().__init__(spec)
        if spec.activation != "xielu":
            raise ops.KernelError(f"activation {spec.activation!r} has no kernel for a dense feed-forward (known: xielu)")
        self.w_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None
        self.act: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamInfo]:
        s = self.spec
        return {
            s.up_name: ParamInfo((s.intermediate_size, s.hidden_size), ("normal", s.hidden_size ** -0.5)),
            s.down_name: ParamInfo((s.hidden_size, s.intermediate_size), ("normal", s.intermediate_size ** -0.5)),
            s.act_name: ParamInfo((2,), ("normal", 0.5)),
        }

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.w_up = tensors[s.up_name].contiguous()
        self.w_down = tensors[s.down_name].contiguous()
        self.act = tensors[s.act_name].contiguous()
        # the numbers the formula uses, for the products that apply the activation in their epilogue (float32, as the
        # stand-alone kernel forms them on the device)
        pq = self.act.detach().to(torch.float32).cpu()
        soft = torch.nn.functional.softplus(pq)
        self.a_p, self.a_n = float(soft[0]), float(0.5 + soft[1])

    def forward(self, x: torch.Tensor, ctx, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """One native call (``oi_dense_mlp``): the up-projection with the activation in its epilogue where a hand-written
        product takes the shape (else the plain product and the activation kernel), then the down-projection, float32."""
        s = self.spec
        M = x.shape[0]
        if not x.is_contiguous():
            x = x.contiguous()
        if M > 32:
            ensure_library(x.device)
        codes = native.DTYPE_CODE
        out = torch.empty((M, s.hidden_size), dtype=torch.float32, device=x.device)
        z = torch.empty((M, s.intermediate_size), dtype=x.dtype, device=x.device)
        _lib.check(_lib.load().oi_dense_mlp(out.data_ptr(), x.data_ptr(), codes[x.dtype], M, s.hidden_size, s.intermediate_size,
                                            self.w_up.data_ptr(), codes[self.w_up.dtype], self.w_down.data_ptr(),
                                            codes[self.w_down.dtype], self.act.data_ptr(), codes[self.act.dtype], self.a_p,
                                            self.a_n, z.data_ptr(), _lib.current_stream()), "dense_mlp")
        return out if out_dtype in (None, torch.float32) else out.to(out_dtype)
