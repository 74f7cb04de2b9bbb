"""Plain-data descriptions of a model's parts.

An architecture turns its config into a ``ModelSpec``: a list of ``BlockSpec``
(each naming its mixer, feed-forward and norms with all their sizes and
constants), the order in which the blocks run, and the embedding / final norm /
head. Parts are built from these specs through the registries in
``parts.registry``; a spec's ``kind`` is the registry key. Nothing here knows
which architecture produced it.
"""
from __future__ import annotations

import dataclasses
from typing import Any, List, Optional, Tuple, Union


@dataclasses.dataclass(frozen=True)
class ParamInfo:
    """One tensor a part wants from the checkpoint.

    ``init`` is how the random-weights mode draws it: ("normal", std),
    ("one_plus_normal", std) or ("normal_around", std, mean). ``integer`` tensors are kept as int32.
    """

    shape: Tuple[int, ...]
    init: Tuple = ("normal", 0.02)
    integer: bool = False


@dataclasses.dataclass(frozen=True)
class NormSpec:
    kind: str = "rms"
    size: int = 0
    eps: float = 1e-6
    weight_offset: float = 0.0  # scale is (weight_offset + w)
    param_name: str = "weight"  # local tensor name (appended to the prefix the enclosing part gives the norm)


@dataclasses.dataclass(frozen=True)
class PositionSpec:
    """Position encoding applied to queries and keys inside a mixer."""

    kind: str = "rope"          # "rope" or "none"
    rotary_dim: int = 0         # leading dims of each head that rotate (<= head_dim, even)
    theta: float = 10000.0
    max_positions: int = 0
    interleaved: bool = False   # angle d turns the neighbours (2 d, 2 d + 1) instead of (d, d + rotary_dim / 2)


@dataclasses.dataclass(frozen=True)
class AttentionSpec:
    kind: str = "attention"
    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    softmax_scale: float = 0.0
    position: PositionSpec = PositionSpec(kind="none")
    qk_norm: Optional[NormSpec] = None      # per-head norm over head_dim, before the rotation
    window: Optional[int] = None            # keys visible to a query, itself included; None = all


@dataclasses.dataclass(frozen=True)
class LatentAttentionSpec:
    """Attention over a low-rank latent: one vector c of ``latent_rank`` numbers per position is cached, and every head
    forms its keys and values from it (k = Wuk_h c, v = Wuv_h c). No position encoding."""

    kind: str = "latent_attention"
    hidden_size: int = 0
    num_heads: int = 0
    qk_dim: int = 0                         # per head: size of queries and keys
    v_dim: int = 0                          # per head: size of values
    latent_rank: int = 0
    softmax_scale: float = 0.0
    latent_norm: Optional[NormSpec] = None  # norm of the latent before it is cached and used
    window: Optional[int] = None            # keys visible to a query, itself included; None = all
    output_gate: bool = False               # head h's output is multiplied by sigmoid(Wg x)_h
    has_latent: bool = True                 # False: the layer reads the latent of an earlier layer and has no down-projection
    # how the per-head up-projections are applied: "weights" multiplies them into the query and output projections
    # once at load time; "runtime" applies them to the queries and to the attention's output in every step
    absorb: str = "weights"
    q_name: str = "q"
    down_name: str = "dkv"
    latent_norm_name: str = "dkv.norm"
    up_k_name: str = "uk"
    up_v_name: str = "uv"
    gate_name: str = "g"
    out_name: str = "o"


@dataclasses.dataclass(frozen=True)
class DenseMlpSpec:
    """down( act(up x) ) with one up-projection. ``activation`` "xielu": the two shape numbers are a tensor."""

    kind: str = "dense_mlp"
    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "xielu"
    up_name: str = "up"
    down_name: str = "down"
    act_name: str = "act"


@dataclasses.dataclass(frozen=True)
class ShortConvSpec:
    """Causal convolution over time on each channel; the last ``taps - 1`` inputs are per-request state."""

    kind: str = "short_conv"
    channels: int = 0
    taps: int = 0
    add_input: bool = True                  # out = x + conv(x) rather than conv(x)
    param_name: str = ""


@dataclasses.dataclass(frozen=True)
class DepthAverageSpec:
    """After a layer, the stream becomes a weighted sum of the outputs of all layers so far (and of the embedding
    output): ``terms`` weights, one tensor."""

    kind: str = "depth_average"
    terms: int = 0
    param_name: str = ""


@dataclasses.dataclass(frozen=True)
class GatedMlpSpec:
    kind: str = "gated_mlp"
    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "silu"


@dataclasses.dataclass(frozen=True)
class BlockSpec:
    """One layer: its parts and the tensor-name prefixes under which they live."""

    kind: str = "prenorm"
    name: str = ""                               # e.g. "model.layers.3."
    mixer: Any = None
    feed_forward: Any = None
    input_norm: Optional[NormSpec] = None
    post_norm: Optional[NormSpec] = None
    mixer_name: str = "self_attn."
    feed_forward_name: str = "mlp."
    input_norm_name: str = "input_layernorm."
    post_norm_name: str = "post_attention_layernorm."
    input_conv: Any = None                       # blocks that filter the mixer's input over time (ShortConvSpec)
    input_conv_name: str = "conv."
    depth_average: Any = None                    # blocks whose result is averaged with earlier layers' (DepthAverageSpec)
    depth_average_name: str = "depth."


@dataclasses.dataclass(frozen=True)
class LayerCall:
    """One entry of the run order: which block runs, and whose cache it reads.

    ``read_cache_of`` is the index (in the order list) of an EARLIER call whose
    keys and values this call's mixer reads instead of writing its own.
    """

    layer: int
    read_cache_of: Optional[int] = None


@dataclasses.dataclass(frozen=True)
class ModelSpec:
    vocab_size: int
    hidden_size: int
    blocks: Tuple[BlockSpec, ...]
    order: Tuple[Union[int, LayerCall], ...]
    final_norm: NormSpec
    embedding_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm."
    head_name: Optional[str] = "lm_head.weight"   # None: the head is the embedding table (tied)
    max_positions: int = 0
    stop_token_ids: Tuple[int, ...] = ()
    embedding_scale: float = 1.0     # the embedded rows are multiplied by this (1: as stored, the reference's Qwen3)
    logit_soft_cap: float = 0.0      # > 0: logits = cap * tanh(logits / cap)
    logit_scale: float = 1.0         # the logits are multiplied by this
    residual_dtype: str = "model"    # "model": the stream between layers has the model's type; "float32": always 32-bit

    def calls(self) -> List[LayerCall]:
        return [c if isinstance(c, LayerCall) else LayerCall(int(c)) for c in self.order]
