"""Bisudra as a list of blocks: the only place that knows this architecture.

Every layer is a block whose norms act on what its sublayers return (`parts.block.SublayerNormBlock`): a differential attention
with a sliding window that reads the stream plus a short causal convolution of it, then a dense feed-forward (squared ReLU, biases)
or a mixture of experts (softmax over the chosen logits), each result gated by a sigmoid of the stream; then a per-layer input by
token id; and what a layer hands on is a learned mix of the embedding output and every layer's result so far.  The norms are layer
norms with bias; the residual stream is 32-bit.  Tensor names: `embed`, `side.embed`, `l<i>.*`, `final.norm`, `final.norm.b`; the
head is the embedding table.
"""
from __future__ import annotations

from ..config.bisudra import ARCHITECTURE, MODEL_TYPE, BisudraConfig
from ..config.registry import register_architecture
from ..config.specs import (DenseFeedForwardSpec, DifferentialAttentionSpec, ModelSpec, NormSpec, PairRotationSpec, RoutedExpertsSpec,
                            ScheduleEntry, SublayerNormBlockSpec, TokenSideSpec)

# The design numbers no positions and keeps no table over them; the limit is that of a 32-bit position.
MAX_POSITIONS = (1 << 31) - 1
SIDE_TABLE = "side.embed"


def _mixer_spec(mixer, width: int, eps: float) -> DifferentialAttentionSpec:
    position = PairRotationSpec(rotary_dim=mixer.rot_dims, theta=mixer.rot_base) if mixer.rot_dims else None
    return DifferentialAttentionSpec(hidden=width, n_heads=mixer.heads, n_kv_heads=mixer.kv_heads, dim=mixer.dim, value_dim=mixer.vdim,
                                     softmax_scale=mixer.scale, diff=mixer.diff, eps=eps, position=position, window=mixer.window, gate=True)


def _feed_forward_spec(mlp, width: int):
    if mlp is None:
        return None
    if mlp.kind == "dense":
        return DenseFeedForwardSpec(hidden=width, intermediate=mlp.ff, activation="relu_squared", bias=True)
    return RoutedExpertsSpec(hidden=width, intermediate=mlp.expert_ff, experts=mlp.experts, top=mlp.top, score="softmax", correction=False,
                             renormalize=True, shared=None, shared_gate=False, router_bias=True)


def build_bisudra_spec(config: BisudraConfig) -> ModelSpec:
    norm = NormSpec(width=config.width, eps=config.eps, kind="layer_norm", bias_suffix=".b")
    table_width = len(config.layers) * config.side_dim
    blocks = tuple(
        SublayerNormBlockSpec(
            prefix=f"l{index}", mixer=_mixer_spec(layer.mixer, config.width, config.eps), feed_forward=_feed_forward_spec(layer.mlp, config.width),
            mixer_norm=norm, feed_forward_norm=norm if layer.mlp is not None else None, input_taps=config.taps, residual_gate=True,
            token_side=TokenSideSpec(table=SIDE_TABLE, table_width=table_width, offset=index * config.side_dim, dim=config.side_dim, eps=config.eps),
            depth_mix=index + 2)
        for index, layer in enumerate(config.layers)
    )
    # Layers whose mixers keep the same thing share a cache group; each has a cache layer of its own there.  The convolutions'
    # tails are one more group, a cache layer per layer.
    schedule, kinds, layers_of = [], [], {}
    for index, block in enumerate(blocks):
        if block.mixer not in kinds:
            kinds.append(block.mixer)
        group = f"{block.mixer.kind}.{kinds.index(block.mixer)}"
        extra = (("taps", "taps", index),) if config.taps > 1 else ()
        schedule.append(ScheduleEntry(layer=index, cache_group=group, cache_layer=layers_of.get(group, 0), writes_cache=True, extra_cache=extra))
        layers_of[group] = layers_of.get(group, 0) + 1
    return ModelSpec(
        architecture=ARCHITECTURE, vocab_size=config.vocab, hidden=config.width, max_positions=MAX_POSITIONS, embedding_name="embed",
        blocks=blocks, schedule=tuple(schedule), final_norm=norm, final_norm_name="final.norm", head_name="head", tie_head=True,
        declared_dtype=config.declared_dtype, residual_dtype="float32", keeps_results=True,
        shared_tensors=((SIDE_TABLE, (config.vocab, table_width), "matrix"),),
    )


register_architecture(ARCHITECTURE, MODEL_TYPE, BisudraConfig.from_json, build_bisudra_spec, storage_dtype="bfloat16")
