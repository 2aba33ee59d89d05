"""Fasesun as a list of blocks: the only place that knows this architecture.

Every layer is a parallel block (one norm; the mixer and the feed-forward both read its output and their sum joins the
residual stream, which is kept in 32-bit).  A layer's mixer is latent attention, a matrix memory with exponential gates
(mLSTM) or linear attention with a constant decay per head (lightning attention); its feed-forward is a mixture of
experts with a shared expert, or nothing.  A run of layers may repeat with the same weights; every run keeps a cache or
state of its own.  Tensor names: `embed`, `l<i>.norm1`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`; the head is the
embedding table.
"""
from __future__ import annotations

from ..config.fasesun import ARCHITECTURE, MODEL_TYPE, FasesunConfig
from ..config.registry import register_architecture
from ..config.specs import (BlockSpec, LatentAttentionSpec, LinearRecurrenceSpec, ModelSpec, NormSpec, PairRotationSpec,
                            RoutedExpertsSpec, ScheduleEntry, SwiGLUSpec)

# The design numbers no positions and keeps no table over them; the limit is that of a 32-bit position.
MAX_POSITIONS = (1 << 31) - 1


def _mixer_spec(mixer, width: int, eps: float):
    if mixer.type == "latent_attention":
        return LatentAttentionSpec(
            hidden=width, n_heads=mixer.heads, head_dim=mixer.dim, rot_dim=mixer.rot_dim, value_dim=mixer.vdim, q_rank=mixer.q_rank,
            kv_rank=mixer.kv_rank, softmax_scale=mixer.scale, eps=eps,
            position=PairRotationSpec(rotary_dim=mixer.rot_dims, theta=mixer.rot_base), sink=True, gate=True)
    if mixer.type == "mlstm":
        return LinearRecurrenceSpec(hidden=width, n_heads=mixer.heads, key_dim=mixer.dim, value_dim=mixer.vdim, gating="exponential",
                                    eps=eps, norm_groups="head", gate_cap=mixer.gate_cap, query_scale=mixer.dim ** -0.5)
    return LinearRecurrenceSpec(hidden=width, n_heads=mixer.heads, key_dim=mixer.dim, value_dim=mixer.vdim, gating="decay", eps=eps,
                                norm_groups="all", decays=mixer.decay, activation="silu")


def _feed_forward_spec(mlp, width: int):
    if mlp is None:
        return None
    names = dict(gate_name="gate", up_name="up", down_name="down", weight_suffix="")
    shared = None if mlp.shared_ff is None else SwiGLUSpec(hidden=width, intermediate=mlp.shared_ff, **names)
    return RoutedExpertsSpec(hidden=width, intermediate=mlp.expert_ff, experts=mlp.experts, top=mlp.top, score="sigmoid",
                             correction=True, renormalize=False, shared=shared, shared_gate=shared is not None)


def build_fasesun_spec(config: FasesunConfig) -> ModelSpec:
    norm = NormSpec(width=config.width, eps=config.eps)
    blocks = tuple(
        BlockSpec(prefix=f"l{index}", mixer=_mixer_spec(layer.mixer, config.width, config.eps),
                  feed_forward=_feed_forward_spec(layer.mlp, config.width), mixer_norm=norm, feed_forward_norm=None, kind="parallel")
        for index, layer in enumerate(config.layers)
    )
    # Runs whose mixers keep the same thing share a cache group; each run has a cache layer of its own there.
    schedule, kinds, layers_of = [], [], {}
    for index in config.layer_runs():
        mixer = blocks[index].mixer
        if mixer not in kinds:
            kinds.append(mixer)
        group = f"{mixer.kind}.{kinds.index(mixer)}"
        schedule.append(ScheduleEntry(layer=index, cache_group=group, cache_layer=layers_of.get(group, 0), writes_cache=True))
        layers_of[group] = layers_of.get(group, 0) + 1
    return ModelSpec(
        architecture=ARCHITECTURE, vocab_size=config.vocab, hidden=config.width, max_positions=MAX_POSITIONS, embedding_name="embed",
        blocks=blocks, schedule=tuple(schedule), final_norm=norm, final_norm_name="final.norm", head_name="head", tie_head=True,
        declared_dtype=config.declared_dtype, residual_dtype="float32",
    )


register_architecture(ARCHITECTURE, MODEL_TYPE, FasesunConfig.from_json, build_fasesun_spec, storage_dtype="bfloat16")
