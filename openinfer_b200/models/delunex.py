"""Delunex: how a ``DelunexConfig`` becomes a ``ModelSpec``.

Every layer is a "branchnorm" block over a float32 stream: the mixer reads x + conv(x) (a causal convolution over
``canon.taps`` positions per channel), its output is normed and added, then the same for a dense feed-forward with the
xIELU activation where the layer has one; after the layer the stream becomes a weighted sum of all layers' results so
far and of the embedding output. The mixer is windowed attention over a cached low-rank latent with a sigmoid gate per
head and no position encoding; a layer with ``kv_from`` reads the latent of an earlier layer's pages. The embedding is
scaled going in, and going out the logits are the final norm's rows times the (unscaled) embedding table times
``logit_scale``. Tensor names: ``embed``, ``final.norm``, and per layer ``l<i>.`` + ``norm1``, ``norm2``, ``canon1``,
``dwa``, ``mix.{q,dkv,dkv.norm,uk,uv,g,o}``, ``mlp.{up,down,act}``.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.delunex import DelunexConfig
from ..parts.spec import (BlockSpec, DenseMlpSpec, DepthAverageSpec, LatentAttentionSpec, LayerCall, ModelSpec, NormSpec,
                          ShortConvSpec)


def build_spec(cfg: DelunexConfig) -> ModelSpec:
    eps = float(cfg.norm["eps"])
    W = cfg.width
    stream_norm = NormSpec(kind="rms", size=W, eps=eps, param_name="")
    blocks, order = [], []
    for i, layer in enumerate(cfg.layers):
        m = layer["mixer"]
        src = m.get("kv_from")
        rank = int(m["kv_rank"])
        mixer = LatentAttentionSpec(
            hidden_size=W, num_heads=int(m["heads"]), qk_dim=int(m["dim"]), v_dim=int(m["vdim"]), latent_rank=rank,
            softmax_scale=float(m["scale"]), latent_norm=NormSpec(kind="rms", size=rank, eps=eps),
            window=int(m["mask"]["size"]) if m.get("mask") else None, output_gate=True, has_latent=src is None)
        mlp = layer.get("mlp")
        ff = DenseMlpSpec(hidden_size=W, intermediate_size=int(mlp["ff"]), activation="xielu") if mlp else None
        blocks.append(BlockSpec(
            kind="branchnorm", name=f"l{i}.", mixer=mixer, feed_forward=ff, input_norm=stream_norm,
            post_norm=stream_norm if ff is not None else None, mixer_name="mix.", feed_forward_name="mlp.",
            input_norm_name="norm1", post_norm_name="norm2",
            input_conv=ShortConvSpec(channels=W, taps=cfg.taps) if cfg.taps else None, input_conv_name="canon1",
            depth_average=DepthAverageSpec(terms=i + 2), depth_average_name="dwa"))
        order.append(LayerCall(i, read_cache_of=None if src is None else int(src)))
    return ModelSpec(
        vocab_size=cfg.vocab, hidden_size=W, blocks=tuple(blocks), order=tuple(order), final_norm=stream_norm,
        embedding_name="embed", final_norm_name="final.norm", head_name=None,
        max_positions=cfg.max_position_embeddings, stop_token_ids=tuple(cfg.stop_token_ids),
        embedding_scale=float(cfg.embedding["scale"]), logit_scale=float(cfg.logit_scale), residual_dtype="float32")


register_architecture(DelunexConfig.architecture, DelunexConfig, build_spec)
