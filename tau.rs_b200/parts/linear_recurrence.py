"""Mixers with a matrix state per head that is carried from token to token: `S_t = a_t S_(t-1) + b_t k_t v_t^T`, read `S_t^T q_t`.

Two gatings (`LinearRecurrenceSpec.gating`):

* `"decay"` (lightning attention): `a_t` is a constant per head, `b_t = 1`; q, k and v pass through SiLU; the concatenated
  heads are divided by their common root mean square.
* `"exponential"` (the matrix memory of xLSTM, mLSTM): a log input gate `i = cap tanh((W_i h + b_i) / cap)` and a log forget
  gate `f = logsigmoid(cap tanh((W_f h + b_f) / cap))` per head; a running maximum `m_t = max(f + m_(t-1), i)` starting at 0;
  `a_t = exp(f + m_(t-1) - m_t)`, `b_t = exp(i - m_t)`; a normaliser `n_t` with the same recurrence over `k` alone; the
  read-out is divided by `max(|n_t . q_t|, exp(-m_t)) + 1e-6`; queries are scaled by `key_dim^-1/2`; each head is divided
  by its own root mean square.

Both end the same way: times the weight `norm` (all heads' width), times `sigmoid(W_g h)`, then `W_o`.  The state is
32-bit, zero when a sequence starts, and lives in the cache's state group; gates, decays, exponentials, the state and the
norms are computed in 32-bit, the projections in the run's dtype.  One kernel walks a run of new tokens of any length, so
prompts, parts of prompts and single tokens are the same code.  Tensor names under the prefix: `q`, `k`, `v`, `g`, `o`,
`norm`, and for the gates `i`, `i.b`, `f`, `f.b`.
"""
from __future__ import annotations

import torch

from ..csrc import kernels
from ..weights.tensor_spec import TensorSpec
from .base import CacheNeed, Mixer
from .linear import StackedLinear
from .registry import register_mixer


@register_mixer("linear_recurrence")
class LinearRecurrence(Mixer):
    def __init__(self, spec, prefix: str, dtype, device):
        if spec.gating not in ("decay", "exponential"):
            raise ValueError(f"unknown gating {spec.gating!r}")
        if spec.norm_groups not in ("head", "all"):
            raise ValueError(f"unknown norm_groups {spec.norm_groups!r}")
        if spec.gating == "decay" and len(spec.decays) != spec.n_heads:
            raise ValueError("one decay per head is needed")
        if spec.activation not in (None, "silu"):
            raise ValueError(f"unknown activation {spec.activation!r}")
        if not 1 <= spec.key_dim <= kernels.RECURRENCE_MAX_KEY_DIM:
            raise ValueError(f"key_dim must lie between 1 and {kernels.RECURRENCE_MAX_KEY_DIM}")
        self.spec, self.prefix, self.device = spec, prefix, device
        self.exponential = spec.gating == "exponential"
        self.k_width, self.v_width = spec.n_heads * spec.key_dim, spec.n_heads * spec.value_dim
        plain = dict(weight_suffix="", bias_suffix=".b")
        self.inputs = StackedLinear([(f"{prefix}.q", self.k_width), (f"{prefix}.k", self.k_width), (f"{prefix}.v", self.v_width),
                                     (f"{prefix}.g", self.v_width)], spec.hidden, False, dtype, device, **plain)
        self.gates = None
        if self.exponential:
            self.gates = StackedLinear([(f"{prefix}.i", spec.n_heads), (f"{prefix}.f", spec.n_heads)], spec.hidden, True, dtype, device, **plain)
        self.out = StackedLinear([(f"{prefix}.o", spec.hidden)], self.v_width, False, dtype, device, **plain)
        self._linears = tuple(part for part in (self.inputs, self.gates, self.out) if part is not None)
        self.norm_name = f"{prefix}.norm"
        self.norm_weight = None
        self.decays = None

    def state_floats(self) -> int:
        spec = self.spec
        per_head = (spec.value_dim + 1) * spec.key_dim + 1 if self.exponential else spec.value_dim * spec.key_dim
        return spec.n_heads * per_head

    def cache_need(self):
        return CacheNeed("state", state_shape=(self.state_floats(),), state_dtype=torch.float32)

    def tensor_specs(self):
        specs = {self.norm_name: TensorSpec((self.v_width,), role="vector", init="ones")}
        for part in self._linears:
            specs.update(part.tensor_specs())
        return specs

    def assign(self, name, tensor):
        if name == self.norm_name:
            self.norm_weight = tensor
            return
        for part in self._linears:
            if name in part.tensor_specs():
                return part.assign(name, tensor)
        raise KeyError(name)

    def finalize_weights(self):
        for part in self._linears:
            part.finalize_weights()
        if not self.exponential:
            self.decays = torch.tensor(self.spec.decays, dtype=torch.float64).to(torch.float32).to(self.device)

    def forward(self, hidden, step, cache, writes_cache: bool):
        spec = self.spec
        tokens = hidden.shape[0]
        projected = self.inputs.forward(hidden)
        gates = self.gates.forward(hidden, out_dtype=torch.float32) if self.exponential else None
        read = torch.empty((tokens, self.v_width), dtype=torch.float32, device=hidden.device)
        k_end, v_end = 2 * self.k_width, 2 * self.k_width + self.v_width
        kernels.linear_recurrence(projected[:, : self.k_width], projected[:, self.k_width : k_end], projected[:, k_end:v_end], gates, self.decays,
                                  cache.state, step.cu_seqlens, step.seq_slot, read, spec.n_heads, spec.key_dim, spec.value_dim,
                                  self.exponential, spec.gate_cap, spec.query_scale, spec.activation == "silu")
        gated = torch.empty((tokens, self.v_width), dtype=hidden.dtype, device=hidden.device)
        kernels.gated_group_norm(read, self.norm_weight, projected[:, v_end:], gated, spec.n_heads if spec.norm_groups == "head" else 1, spec.eps, True)
        return self.out.forward(gated)
