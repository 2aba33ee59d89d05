"""Latent attention: keys and values of all heads are expanded from one cached latent per position.

Per token, with `h` the block's normalised input:
    c_q = RMSnorm(W_dq h) * w_dq;   q = W_uq c_q, per head [head_dim unrotated | rot_dim rotated]
    [c' | r] = W_dkv h;   c = RMSnorm(c') * w_dkv  (kv_rank elements);   r (rot_dim elements) is one key part for all heads
    key of head a at position j: [W_uk,a c_j | rotate(r_j, j)];   value: W_uv,a c_j
    score(i, j) = (q_a,i . key_a,j) * scale for j <= i;   softmax whose denominator also holds exp(sink_a)
    out = W_o (concatenated heads * sigmoid(W_g h))

Only `[c | rotate(r)]` is cached, one row per position (`CacheNeed("rows")`).  Steps over cached positions never expand it: since
`q . (W_uk,a c) = (W_uk,a^T q) . c`, each head's unrotated query is carried into the latent's space by one small product per
head, the attention kernel scores `[W_uk,a^T q | rotated q]` against the cached rows as they lie and sums the rows' latent
parts, and one more product per head (`W_uv,a`) turns that sum into the head's values.  Single tokens, portions of prompts
and everything in float32 take this form.  A bfloat16 step whose sequences all start at position 0 (whole prompts, `EXPAND_FROM`
tokens or more) takes the other: there the cache holds nothing yet, so keys and values of the step's own tokens are expanded
once by one tensor-core product, laid into pages of their own, and the attention kernel of ordinary heads (with the sink in its
denominator) serves them; the latent rows are cached all the same for the steps that follow.  Tensor names under the prefix: `dq`, `dq.norm`, `uq`, `dkv`, `dkv.norm`, `uk`, `uv`, `sink`, `g`, `o`.
"""
from __future__ import annotations

import torch

from ..csrc import kernels
from ..weights.tensor_spec import TensorSpec
from .base import CacheNeed, Mixer
from .linear import StackedLinear
from .registry import build, register_mixer


EXPAND_FROM = 128            # tokens of a step from which whole prompts take the expanded form
EXPAND_LIMIT = 4 << 30       # bytes of expanded keys and values that a step may ask for


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    def __init__(self, spec, prefix: str, dtype, device):
        if spec.kv_rank > kernels.LATENT_MAX_RANK:
            raise ValueError(f"kv_rank may be at most {kernels.LATENT_MAX_RANK}, found {spec.kv_rank}")
        self.spec, self.prefix, self.dtype, self.device = spec, prefix, dtype, device
        self.q_width = spec.n_heads * (spec.head_dim + spec.rot_dim)
        self.v_width = spec.n_heads * spec.value_dim
        self.row_width = spec.kv_rank + spec.rot_dim
        plain = dict(weight_suffix="")
        # The key/value down-projection and the gate are one product; the query's latent is its own, so that its norm reads whole rows.
        pieces = [(f"{prefix}.dkv", self.row_width)] + ([(f"{prefix}.g", self.v_width)] if spec.gate else [])
        self.down = StackedLinear(pieces, spec.hidden, False, dtype, device, **plain)
        self.down_q = StackedLinear([(f"{prefix}.dq", spec.q_rank)], spec.hidden, False, dtype, device, **plain)
        self.up_q = StackedLinear([(f"{prefix}.uq", self.q_width)], spec.q_rank, False, dtype, device, **plain)
        self.out = StackedLinear([(f"{prefix}.o", spec.hidden)], self.v_width, False, dtype, device, **plain)
        self.position = None if spec.position is None else build("position", spec.position, device=device)
        if spec.position is not None and spec.position.rotary_dim > spec.rot_dim:
            raise ValueError("the rotation is wider than the rotated part")
        self._own = {
            f"{prefix}.dq.norm": TensorSpec((spec.q_rank,), role="vector", init="ones"),
            f"{prefix}.dkv.norm": TensorSpec((spec.kv_rank,), role="vector", init="ones"),
            f"{prefix}.uk": TensorSpec((spec.n_heads * spec.head_dim, spec.kv_rank), role="matrix"),
            f"{prefix}.uv": TensorSpec((spec.n_heads * spec.value_dim, spec.kv_rank), role="matrix"),
        }
        if spec.sink:
            self._own[f"{prefix}.sink"] = TensorSpec((spec.n_heads,), role="vector", std=1.0)
        self._held = {}
        self._linears = (self.down, self.down_q, self.up_q, self.out)
        self.key_up_transposed = self.value_up = self.q_norm = self.kv_norm = self.sink = None

    def cache_need(self):
        return CacheNeed("rows", row_width=self.row_width, window=self.spec.window)

    def decode_blocks(self) -> int:
        """Blocks per sequence and context range of a decode step: one for every eight heads."""
        return -(-self.spec.n_heads // 8)

    def tensor_specs(self):
        specs = dict(self._own)
        for part in self._linears:
            specs.update(part.tensor_specs())
        return specs

    def assign(self, name, tensor):
        if name in self._own:
            self._held[name] = tensor
            return
        for part in self._linears:
            if name in part.tensor_specs():
                return part.assign(name, tensor)
        raise KeyError(name)

    def finalize_weights(self):
        spec, prefix = self.spec, self.prefix
        for part in self._linears:
            part.finalize_weights()
        if self.position is not None:
            self.position.finalize_weights()
        self.q_norm, self.kv_norm = self._held.pop(f"{prefix}.dq.norm"), self._held.pop(f"{prefix}.dkv.norm")
        self.sink = self._held.pop(f"{prefix}.sink") if spec.sink else None
        # [heads, kv_rank, head_dim]: the product `W_uk,a^T q` reads its weight as [out, in] like every other.
        self.key_up_transposed = self._held.pop(f"{prefix}.uk").view(spec.n_heads, spec.head_dim, spec.kv_rank).transpose(1, 2).contiguous()
        self.value_up = self._held.pop(f"{prefix}.uv").view(spec.n_heads, spec.value_dim, spec.kv_rank)
        # For the expanded form: all heads' key rows, then all heads' value rows, as one weight.
        width = spec.head_dim + spec.rot_dim
        self.expands = (self.dtype == torch.bfloat16 and width % 16 == 0 and 16 <= width <= 256 and spec.value_dim <= width and spec.kv_rank % 8 == 0)
        self.expand_weight = None
        if self.expands:
            self.expand_weight = torch.cat([self.key_up_transposed.transpose(1, 2).reshape(-1, spec.kv_rank), self.value_up.reshape(-1, spec.kv_rank)]).contiguous()
        self._page_tables = {}

    def _expanded(self, hidden, projected, q, step, cache):
        """Whole prompts: keys and values of the step's tokens expanded once, attention by the kernel of ordinary heads."""
        spec = self.spec
        tokens, device, width = hidden.shape[0], hidden.device, spec.head_dim + spec.rot_dim
        latents = torch.empty((tokens, spec.kv_rank), dtype=hidden.dtype, device=device)
        position = self.position
        frequencies, rotary = (None, 0) if position is None else (position.inv_freq, spec.position.rotary_dim)
        kernels.latent_prepare(projected[:, : self.row_width], self.kv_norm, spec.eps, q, None, cache.rows, frequencies, rotary, step.positions,
                               step.token_seq, step.page_rows[cache.group], spec.n_heads, spec.head_dim, spec.rot_dim, spec.kv_rank, True, latents)
        expanded = torch.empty((tokens, self.expand_weight.shape[0]), dtype=hidden.dtype, device=device)
        kernels.linear(latents, self.expand_weight, None, expanded)
        pages = -(-step.max_new // kernels.PAGE_TOKENS)
        key = (step.n_seqs, pages)
        table = self._page_tables.get(key)
        if table is None:
            table = self._page_tables[key] = torch.arange(step.n_seqs * pages, dtype=torch.int32, device=device).view(step.n_seqs, pages)
        shape = (step.n_seqs * pages, spec.n_heads, kernels.PAGE_TOKENS, width)
        keys, values = torch.empty(shape, dtype=hidden.dtype, device=device), torch.empty(shape, dtype=hidden.dtype, device=device)
        queries = torch.empty((tokens, spec.n_heads, width), dtype=hidden.dtype, device=device)
        kernels.latent_expand(q, projected[:, : self.row_width], expanded, queries, keys, values, frequencies, rotary, step.positions, step.token_seq,
                              pages, spec.n_heads, spec.head_dim, spec.rot_dim, spec.kv_rank, spec.value_dim)
        attended = torch.empty((tokens, spec.n_heads * width), dtype=hidden.dtype, device=device)
        kernels.attention_prefill(queries.view(tokens, -1), keys, values, attended, step.cu_seqlens, step.seq_start, table, spec.n_heads, spec.n_heads,
                                  width, spec.softmax_scale, spec.window or 0, self.sink)
        gated = torch.empty((tokens, self.v_width), dtype=hidden.dtype, device=device)
        kernels.head_gate(attended, projected[:, self.row_width :] if spec.gate else None, gated, spec.n_heads, width, spec.value_dim)
        return self.out.forward(gated)

    def forward(self, hidden, step, cache, writes_cache: bool):
        spec = self.spec
        tokens = hidden.shape[0]
        projected = self.down.forward(hidden)
        q_latent = torch.empty((tokens, spec.q_rank), dtype=hidden.dtype, device=hidden.device)
        kernels.rms_norm(self.down_q.forward(hidden), self.q_norm, spec.eps, q_latent)
        q = self.up_q.forward(q_latent)
        if (self.expands and writes_cache and getattr(step, "all_fresh", False) and not step.all_single and tokens >= EXPAND_FROM
                and kernels.optimized_preferred()):
            pages = step.n_seqs * -(-step.max_new // kernels.PAGE_TOKENS)
            if 4 * pages * spec.n_heads * kernels.PAGE_TOKENS * (spec.head_dim + spec.rot_dim) <= EXPAND_LIMIT:
                return self._expanded(hidden, projected, q, step, cache)
        queries = torch.empty((tokens, spec.n_heads, self.row_width), dtype=hidden.dtype, device=hidden.device)
        pages = step.page_rows[cache.group]
        kernels.latent_prepare(projected[:, : self.row_width], self.kv_norm, spec.eps, q, queries, cache.rows,
                               None if self.position is None else self.position.inv_freq, 0 if self.position is None else spec.position.rotary_dim,
                               step.positions, step.token_seq, pages, spec.n_heads, spec.head_dim, spec.rot_dim, spec.kv_rank, writes_cache)
        kernels.gemm_simt_batched(q.view(tokens, spec.n_heads, spec.head_dim + spec.rot_dim)[:, :, : spec.head_dim], self.key_up_transposed,
                                  queries[:, :, : spec.kv_rank])
        summed = torch.empty((tokens, spec.n_heads, spec.kv_rank), dtype=hidden.dtype, device=hidden.device)
        # A step of single tokens cuts each context into ranges so that the machine has blocks enough; the number is the engine's
        # (part of a captured graph's key) or chosen here from the longest context.
        splits = 1
        if step.all_single:
            splits = min(step.decode_splits or kernels.decode_splits(step.n_seqs, step.max_len, self.decode_blocks()), 64)
        kernels.latent_attention(queries, cache.rows, summed, self.sink, step.positions, step.token_seq, pages, spec.n_heads, spec.kv_rank,
                                 spec.rot_dim, spec.softmax_scale, spec.window or 0, splits)
        if not spec.gate:
            mixed = torch.empty((tokens, self.v_width), dtype=hidden.dtype, device=hidden.device)
            kernels.gemm_simt_batched(summed, self.value_up, mixed.view(tokens, spec.n_heads, spec.value_dim))
            return self.out.forward(mixed)
        values = torch.empty((tokens, self.v_width), dtype=torch.float32, device=hidden.device)
        kernels.gemm_simt_batched(summed, self.value_up, values.view(tokens, spec.n_heads, spec.value_dim))
        gated = torch.empty((tokens, self.v_width), dtype=hidden.dtype, device=hidden.device)
        kernels.gated_group_norm(values, None, projected[:, self.row_width :], gated, 1, 0.0, False)
        return self.out.forward(gated)
