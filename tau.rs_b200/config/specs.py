"""Descriptions of parts: what a layer is made of, as data.

A model is a list of block descriptions and a schedule.  Each description names the
kind of part (looked up in `tau_rs_b200.parts.registry`) and carries every size and
constant that the part needs, so no part reads a model-wide configuration and none
knows which architecture it serves.  tau.rs expresses the same idea with one enum per
layer (crates/models/src/qwen3_5_common/decoder.rs:22-25,59-78: each layer owns either
kind of token mixer and its own state).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    width: int
    eps: float
    kind: str = "rms_norm"


@dataclass(frozen=True)
class PositionSpec:
    """Rotary position encoding of the first `rotary_dim` elements of each head."""

    rotary_dim: int
    theta: float
    max_positions: int
    kind: str = "rope_half"


@dataclass(frozen=True)
class AttentionSpec:
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    bias: bool
    softmax_scale: float
    qk_norm: Optional[NormSpec] = None
    position: Optional[PositionSpec] = None
    window: Optional[int] = None
    kind: str = "attention"


@dataclass(frozen=True)
class SwiGLUSpec:
    """`down(silu(gate(x)) * up(x))`.  The three tensors are `<prefix>.<name><weight_suffix>`."""

    hidden: int
    intermediate: int
    kind: str = "swiglu"
    gate_name: str = "gate_proj"
    up_name: str = "up_proj"
    down_name: str = "down_proj"
    weight_suffix: str = ".weight"


@dataclass(frozen=True)
class PairRotationSpec:
    """Rotary position encoding of the first `rotary_dim` elements of a vector in which element `2i` is paired with
    `2i + 1` (the interleaved layout); the angle of pair `i` at position `p` is `p * theta^(-2i / rotary_dim)`."""

    rotary_dim: int
    theta: float
    kind: str = "rope_pairs"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Softmax attention whose keys and values are expanded from a cached latent of `kv_rank` elements per position, with
    `rot_dim` rotated key elements per position that all heads share, queries through a latent of `q_rank` elements, an
    optional learned sink per head in the softmax denominator and an optional sigmoid output gate."""

    hidden: int
    n_heads: int
    head_dim: int          # unrotated query/key elements per head
    rot_dim: int           # rotated query/key elements per head (the key's are shared by the heads)
    value_dim: int
    q_rank: int
    kv_rank: int
    softmax_scale: float
    eps: float             # of the two latent norms
    position: Optional[PairRotationSpec] = None
    sink: bool = True
    gate: bool = True
    window: Optional[int] = None
    kind: str = "latent_attention"


@dataclass(frozen=True)
class LinearRecurrenceSpec:
    """A matrix state per head, `S_t = a_t S_(t-1) + b_t k_t v_t^T`, read as `S_t^T q_t`.

    `gating == "decay"`: `a_t` is the head's constant of `decays`, `b_t = 1`, and q, k, v pass through `activation`.
    `gating == "exponential"`: a log input gate and a log forget gate per head and token (both soft-capped at `gate_cap`),
    a running maximum that keeps the exponentials in range, a normaliser state, and queries scaled by `query_scale`.
    `norm_groups` says over what the output is divided by its root mean square before the weight and the sigmoid gate:
    `"head"` (each head alone) or `"all"` (the concatenated heads)."""

    hidden: int
    n_heads: int
    key_dim: int
    value_dim: int
    gating: str
    eps: float
    norm_groups: str
    decays: Tuple[float, ...] = ()
    gate_cap: float = 0.0
    query_scale: float = 1.0
    activation: Optional[str] = None
    kind: str = "linear_recurrence"


@dataclass(frozen=True)
class RoutedExpertsSpec:
    """`top` of `experts` gated feed-forwards per token.  The router's logits pass through `score` ("sigmoid" or
    "softmax"); experts are chosen by score plus a correction per expert (if `correction`), weighted by the score itself,
    renormalised over the chosen ones only if `renormalize`.  `shared` is a feed-forward that every token passes; with
    `shared_gate` its output is scaled by the sigmoid of one more projection of the token."""

    hidden: int
    intermediate: int
    experts: int
    top: int
    score: str = "sigmoid"
    correction: bool = True
    renormalize: bool = False
    shared: Optional[SwiGLUSpec] = None
    shared_gate: bool = False
    kind: str = "routed_experts"


@dataclass(frozen=True)
class BlockSpec:
    """One layer: its weight-name prefix, its two parts and the norm before each."""

    prefix: str
    mixer: object
    feed_forward: object
    mixer_norm: NormSpec
    feed_forward_norm: Optional[NormSpec]
    kind: str = "pre_norm"


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.

    `layer` indexes the model's blocks (a block may be named by several entries and
    then runs several times with the same weights).  `cache_group` and `cache_layer`
    say where the mixer keeps what it remembers; two entries with the same pair share
    that storage, and an entry with `writes_cache=False` only reads what another entry
    wrote earlier in the same step.
    """

    layer: int
    cache_group: Optional[str] = None
    cache_layer: int = 0
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden: int
    max_positions: int
    embedding_name: str
    blocks: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: NormSpec
    final_norm_name: str
    head_name: str
    tie_head: bool
    declared_dtype: Optional[str] = None
    extra: dict = field(default_factory=dict, compare=False)
    # A position encoding that acts on the embedded tokens before the first block (learned or absolute positions): a spec of
    # the "position" family whose part offers `add_to(hidden, step)`.  None for encodings that act inside the mixers.
    input_position: Optional[object] = None
    # "float32": the residual stream is kept in 32-bit whatever the run's dtype (None: in the run's dtype).
    residual_dtype: Optional[str] = None
