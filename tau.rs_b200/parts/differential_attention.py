"""Differential attention: two softmax maps per head over the same values, the second subtracted from the first.

Per token, with `h` the mixer's input, `H` heads, `G` key/value heads, `dim` elements per query and key and `vdim` per value:
    q = W_q h as [H, 2, dim];  k = W_k h as [G, 2, dim];  v = W_v h as [G, vdim];  gate = sigmoid(W_g h) as [H, vdim]
    every q and k map: divided by its root mean square over dim, times a weight (`q.norm`, `k.norm`) that heads and maps share,
    then rotated at the token's position
    a_m(head) = softmax over the visible positions j of (q_m . k_m,j) * scale, applied to v_j   (m = 1, 2; group = head // (H / G))
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff
    o = a_1 - lambda * a_2;  o <- o / sqrt(mean(o^2) + eps) * (1 - diff);  out = W_o (o * gate)

A position sees itself and the `window - 1` positions before it.  The four projections of `h` are one product.  Two layouts of
the cache, chosen from the sizes alone:

* `wide = max(dim, vdim)` a multiple of 16 up to 256: every map is an ordinary head of `wide` elements (zeros behind what it
  holds) in a cache of keys and values (`CacheNeed("kv")`, 2 G heads; the group's values stand under both of its maps), so the
  attention kernels of ordinary heads serve it with 2 H query heads: the tensor-core kernels for runs of new tokens, the split
  decode kernel for single tokens, the 32-bit ones in float32.  One kernel then forms `a_1 - lambda * a_2`, the unit RMS and the
  gate.  Against the smallest possible cache this one is `4 wide / (2 dim + vdim)` times as large (2 for vdim = 2 dim).
* any other sizes: one row per position, `[G x (key of map 1 | key of map 2) | G x value]` (`CacheNeed("rows")`), and a kernel
  of its own on the 32-bit pipes that computes both maps, the difference, the norm and the gate per (token, head).

Either way keys are cached normalised and rotated, and the window lets the cache give back pages that fell out of it.  Tensor names under the prefix: `q`, `k`, `v`, `g`,
`o`, `q.norm`, `k.norm`, `lq1`, `lk1`, `lq2`, `lk2`.
"""
from __future__ import annotations

import math

import torch

from ..csrc import kernels
from ..weights.tensor_spec import TensorSpec
from .base import CacheNeed, Mixer
from .linear import StackedLinear
from .registry import build, register_mixer


@register_mixer("differential_attention")
class DifferentialAttention(Mixer):
    def __init__(self, spec, prefix: str, dtype, device):
        if spec.n_heads % spec.n_kv_heads != 0:
            raise ValueError(f"n_heads ({spec.n_heads}) must be a multiple of n_kv_heads ({spec.n_kv_heads})")
        if spec.value_dim > kernels.DIFF_MAX_VALUE_DIM:
            raise ValueError(f"values may have at most {kernels.DIFF_MAX_VALUE_DIM} elements per head, found {spec.value_dim}")
        if spec.position is not None and spec.position.rotary_dim > spec.dim:
            raise ValueError("the rotation is wider than a query")
        self.spec, self.prefix, self.dtype, self.device = spec, prefix, dtype, device
        self.q_width = spec.n_heads * 2 * spec.dim
        self.row_width = spec.n_kv_heads * (2 * spec.dim + spec.value_dim)
        wide = max(spec.dim, spec.value_dim)
        self.wide = wide if wide % 16 == 0 and 16 <= wide <= 256 else 0      # 0: the layout of one row per position
        self.out_width = spec.n_heads * spec.value_dim
        plain = dict(weight_suffix="")
        pieces = [(f"{prefix}.q", self.q_width), (f"{prefix}.k", spec.n_kv_heads * 2 * spec.dim), (f"{prefix}.v", spec.n_kv_heads * spec.value_dim)]
        if spec.gate:
            pieces.append((f"{prefix}.g", self.out_width))
        self.projection = StackedLinear(pieces, spec.hidden, False, dtype, device, **plain)
        self.out = StackedLinear([(f"{prefix}.o", spec.hidden)], self.out_width, False, dtype, device, **plain)
        self.position = None if spec.position is None or spec.position.rotary_dim == 0 else build("position", spec.position, device=device)
        self._own = {f"{prefix}.{name}": TensorSpec((spec.dim,), role="vector", init="ones" if name.endswith("norm") else "normal", std=0.1)
                     for name in ("q.norm", "k.norm", "lq1", "lk1", "lq2", "lk2")}
        self._held = {}
        self.q_norm = self.k_norm = None
        self.lam = 0.0

    def cache_need(self):
        if self.wide:
            return CacheNeed("kv", n_kv_heads=2 * self.spec.n_kv_heads, head_dim=self.wide, window=self.spec.window)
        return CacheNeed("rows", row_width=self.row_width, window=self.spec.window)

    def decode_blocks(self):
        """Blocks that the decode kernel of ordinary heads launches per sequence and context split (the other layout's kernel does
        not split contexts)."""
        if not self.wide:
            return None
        group = self.spec.n_heads // self.spec.n_kv_heads
        heads_per_pass = 8 if group >= 8 else 4 if group > 2 else group
        return 2 * self.spec.n_kv_heads * -(-group // heads_per_pass)

    def tensor_specs(self):
        return {**self._own, **self.projection.tensor_specs(), **self.out.tensor_specs()}

    def assign(self, name, tensor):
        if name in self._own:
            self._held[name] = tensor
        elif name in self.projection.tensor_specs():
            self.projection.assign(name, tensor)
        elif name in self.out.tensor_specs():
            self.out.assign(name, tensor)
        else:
            raise KeyError(name)

    def finalize_weights(self):
        prefix, held = self.prefix, self._held
        self.projection.finalize_weights()
        self.out.finalize_weights()
        if self.position is not None:
            self.position.finalize_weights()
        self.q_norm, self.k_norm = held.pop(f"{prefix}.q.norm"), held.pop(f"{prefix}.k.norm")
        first = float((held.pop(f"{prefix}.lq1").double() * held.pop(f"{prefix}.lk1").double()).sum())
        second = float((held.pop(f"{prefix}.lq2").double() * held.pop(f"{prefix}.lk2").double()).sum())
        self.lam = math.exp(first) - math.exp(second) + self.spec.diff      # one number for the layer, fixed with the weights

    def forward(self, hidden, step, cache, writes_cache: bool):
        spec = self.spec
        tokens = hidden.shape[0]
        # A run that only reads another run's rows needs its queries (and its gate, which lies behind keys and values in the stack).
        projected = self.projection.forward(hidden)
        pages = step.page_rows[cache.group]
        mixed = torch.empty((tokens, self.out_width), dtype=hidden.dtype, device=hidden.device)
        gate = projected[:, self.q_width + self.row_width :] if spec.gate else None
        inv_freq, rotary = (None, 0) if self.position is None else (self.position.inv_freq, spec.position.rotary_dim)
        if self.wide:
            wide, maps = self.wide, 2 * spec.n_heads
            queries = torch.empty((tokens, maps, wide), dtype=hidden.dtype, device=hidden.device)
            kernels.diff_prepare_wide(projected, self.q_norm, self.k_norm, spec.eps, inv_freq, rotary, queries, cache.keys, cache.values, step.positions,
                                      step.token_seq, pages, spec.n_heads, spec.n_kv_heads, spec.dim, spec.value_dim, writes_cache)
            attended = torch.empty((tokens, maps * wide), dtype=hidden.dtype, device=hidden.device)
            kernels.attention(queries.view(tokens, maps * wide), cache.keys, cache.values, attended, step, pages, maps, 2 * spec.n_kv_heads, wide,
                              spec.softmax_scale, spec.window or 0)
            kernels.diff_combine(attended.view(tokens, maps, wide), gate, mixed, spec.n_heads, spec.n_kv_heads, spec.value_dim, self.lam, spec.eps,
                                 1.0 - spec.diff)
            return self.out.forward(mixed, out_dtype=torch.float32)
        queries = torch.empty((tokens, spec.n_heads, 2, spec.dim), dtype=hidden.dtype, device=hidden.device)
        kernels.diff_prepare(projected, self.q_norm, self.k_norm, spec.eps, None if self.position is None else self.position.inv_freq,
                             0 if self.position is None else spec.position.rotary_dim, queries, cache.rows, step.positions, step.token_seq, pages,
                             spec.n_heads, spec.n_kv_heads, spec.dim, spec.value_dim, writes_cache)
        kernels.diff_attention(queries, cache.rows, gate, mixed, step, pages, spec.n_kv_heads, spec.value_dim, spec.softmax_scale, spec.window or 0,
                               self.lam, spec.eps, 1.0 - spec.diff)
        return self.out.forward(mixed, out_dtype=torch.float32)
