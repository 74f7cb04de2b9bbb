"""Pilonex: how a ``PilonexConfig`` becomes a ``ModelSpec``.

Every layer is a "hyper" block: pre-norm sublayers (norm weights stored around zero, used as 1 + w) over ``streams``
float32 residual streams that every sublayer reads and writes through three small coefficient tensors; without
``streams`` the plain residual. Layer types: "mlstm", a matrix-memory recurrence with capped exponential gating, and
"parallel", windowed grouped-query attention (per-head q/k norm, partial rotary positions with long waves stretched, keys
and values of different sizes) beside a gated delta rule behind short causal filters, summed with two scales. The
feed-forward is a gated layer with a clamped activation, dense or as routed experts. ``loop`` repeats a run of layers;
every pass is an entry of the run order with a cache and a state of its own. Tensor names: ``embed``, ``head``,
``final.norm``, and per layer ``l<i>.`` + ``norm1``, ``norm2``, ``hc1.{in,mix,out}``, ``hc2.*``, ``mix.*``, ``mlp.*``.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.pilonex import PilonexConfig
from ..parts.spec import (AttentionSpec, BlockSpec, GatedDeltaSpec, GatedMlpSpec, MatrixMemorySpec, ModelSpec, NormSpec,
                          ParallelMixerSpec, PositionSpec, RoutedExpertsSpec)


def _pad8(n: int) -> int:
    return (n + 7) & ~7


def _mixer(cfg: PilonexConfig, layer: dict, eps: float):
    W, m = cfg.width, layer["mixer"]
    if layer["type"] == "mlstm":
        return MatrixMemorySpec(hidden_size=W, num_heads=int(m["heads"]), qk_dim=int(m["dim"]), v_dim=int(m["vdim"]),
                                gate_cap=float(m["gate_cap"]), eps=eps)
    left, right = m["left"], m["right"]
    dim, vdim = int(left["dim"]), int(left["vdim"])
    rot = left.get("rot")
    position = PositionSpec(kind="none")
    if rot:
        sc = rot.get("scaling")
        position = PositionSpec(kind="rope", rotary_dim=int(rot["dims"]), theta=float(rot["base"]),
                                max_positions=cfg.max_position_embeddings, precise=True,
                                scaling=(float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])) if sc else None)
    attention = AttentionSpec(
        hidden_size=W, num_heads=int(left["heads"]), num_kv_heads=int(left["kv_heads"]), head_dim=_pad8(max(dim, vdim)),
        softmax_scale=float(left["scale"]), position=position, qk_norm=NormSpec(kind="rms", size=dim, eps=eps),
        window=int(left["mask"]["size"]) if left.get("mask") else None, qk_dim=dim, v_dim=vdim,
        q_name="q", k_name="k", v_name="v", o_name="o", q_norm_name="q.norm", k_norm_name="k.norm")
    delta = GatedDeltaSpec(hidden_size=W, num_heads=int(right["heads"]), num_kv_heads=int(right["kv_heads"]), qk_dim=int(right["dim"]),
                           v_dim=int(right["vdim"]), conv_taps=int(right["conv"]), eps=eps,
                           decay_rank=int(right.get("decay_rank", 0)), gate_rank=int(right.get("gate_rank", 0)))
    return ParallelMixerSpec(left=attention, right=delta, left_scale=float(m["left_scale"]), right_scale=float(m["right_scale"]))


def _feed_forward(cfg: PilonexConfig, mlp):
    if not mlp:
        return None
    if mlp["kind"] == "dense":
        return GatedMlpSpec(hidden_size=cfg.width, intermediate_size=int(mlp["ff"]), activation="swiglu_clamp",
                            limit=float(mlp["limit"]), gate_name="gate", up_name="up", down_name="down")
    return RoutedExpertsSpec(hidden_size=cfg.width, intermediate_size=int(mlp["expert"]["ff"]), experts=int(mlp["router"]["experts"]),
                             top=int(mlp["router"]["top"]), activation="swiglu_clamp", limit=float(mlp["expert"]["limit"]))


def build_spec(cfg: PilonexConfig) -> ModelSpec:
    eps = float(cfg.norm["eps"])
    W = cfg.width
    norm = NormSpec(kind="rms", size=W, eps=eps, weight_offset=1.0, param_name="")
    blocks = []
    for i, layer in enumerate(cfg.layers):
        ff = _feed_forward(cfg, layer.get("mlp"))
        blocks.append(BlockSpec(
            kind="hyper", name=f"l{i}.", mixer=_mixer(cfg, layer, eps), feed_forward=ff, input_norm=norm,
            post_norm=norm if ff is not None else None, mixer_name="mix.", feed_forward_name="mlp.",
            input_norm_name="norm1", post_norm_name="norm2", streams=cfg.streams or 1, stream_coefficients=cfg.streams is not None))
    return ModelSpec(
        vocab_size=cfg.vocab, hidden_size=W, blocks=tuple(blocks), order=cfg.run_order(), final_norm=norm,
        embedding_name="embed", final_norm_name="final.norm", head_name="head", max_positions=cfg.max_position_embeddings,
        stop_token_ids=tuple(cfg.stop_token_ids), residual_dtype="float32", streams=cfg.streams or 1)


register_architecture(PilonexConfig.architecture, PilonexConfig, build_spec)
