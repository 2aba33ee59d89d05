"""Plain, slow statement of the Fasesun decoder: whole sequences, no cache, one function per mechanism.

Nothing here is imported from the library and the library imports nothing from here.  Everything runs on the CPU in
float64 (or float32).  Notation: `h` is a layer's normalised input `[T, width]`, `W` maps tensor names to tensors stored
`[out, in]`, `p` is a token's position counted from 0.

`round_to` emulates a storage dtype at the outputs of matrix products; statistics, scores, states and the residual
stream stay in full precision.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, Optional, Sequence

import torch

Rounding = Callable[[torch.Tensor], torch.Tensor]


def no_rounding(values: torch.Tensor) -> torch.Tensor:
    return values


def bfloat16_rounding(values: torch.Tensor) -> torch.Tensor:
    return values.to(torch.bfloat16).to(values.dtype)


def linear(x: torch.Tensor, weight: torch.Tensor, round_to: Rounding = no_rounding) -> torch.Tensor:
    return round_to(x @ weight.to(x.dtype).T)


# --------------------------------------------------------------------------- small pieces
def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """`x / sqrt(mean(x^2) + eps) * w`, eps inside the root."""
    out = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return out if weight is None else out * weight.to(x.dtype)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """Rotates the first `dims` elements of the last axis: element 2i is paired with 2i + 1, angle `p * base^(-2i/dims)`.

    `x` is `[T, ..., d]` and `positions` `[T]`; elements from `dims` on pass unchanged."""
    out = x.clone()
    index = torch.arange(dims // 2, dtype=x.dtype)
    frequency = base ** (-2.0 * index / dims)
    angle = positions.to(x.dtype)[:, None] * frequency[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = torch.cos(angle).reshape(shape), torch.sin(angle).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


# --------------------------------------------------------------------------- mixers
def latent_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], prefix: str, mixer: dict, eps: float,
                     round_to: Rounding = no_rounding) -> torch.Tensor:
    """Attention whose keys and values are expanded from a cached latent, with one rotated key part shared by all heads,
    a sink in the softmax denominator and a sigmoid output gate."""
    T = h.shape[0]
    heads, dim, rot_dim, vdim, rank = mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["vdim"], mixer["kv_rank"]
    base, rot = mixer["rot"]["base"], mixer["rot"]["dims"]
    positions = torch.arange(T)
    c_q = round_to(rms_norm(linear(h, W[prefix + ".dq"], round_to), W[prefix + ".dq.norm"], eps))
    q = linear(c_q, W[prefix + ".uq"], round_to).view(T, heads, dim + rot_dim)
    q_plain, q_rot = q[..., :dim], rotate_pairs(q[..., dim:], positions, base, rot)
    down = linear(h, W[prefix + ".dkv"], round_to)
    c = round_to(rms_norm(down[:, :rank], W[prefix + ".dkv.norm"], eps))
    k_rot = rotate_pairs(down[:, rank:], positions, base, rot)                       # [T, rot_dim], every head's
    k_plain = linear(c, W[prefix + ".uk"], round_to).view(T, heads, dim)
    v = linear(c, W[prefix + ".uv"], round_to).view(T, heads, vdim)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * mixer["scale"]
    causal = positions[None, :] <= positions[:, None]
    if mixer.get("window"):          # not a part of Fasesun: a window that other designs may put on this mixer
        causal = causal & (positions[None, :] > positions[:, None] - mixer["window"])
    scores = scores.masked_fill(~causal[None], float("-inf"))
    sink = W[prefix + ".sink"].to(h.dtype)                                           # [heads]; one more term of the denominator
    top = torch.maximum(scores.max(dim=-1).values, sink[:, None])
    weights = torch.exp(scores - top[..., None])
    weights = weights / (weights.sum(dim=-1) + torch.exp(sink[:, None] - top))[..., None]
    mixed = torch.einsum("hij,jhd->ihd", weights, v).reshape(T, heads * vdim)
    gate = torch.sigmoid(linear(h, W[prefix + ".g"], round_to))
    return linear(round_to(mixed * gate), W[prefix + ".o"], round_to)


def lightning(h: torch.Tensor, W: Dict[str, torch.Tensor], prefix: str, mixer: dict, eps: float,
              round_to: Rounding = no_rounding) -> torch.Tensor:
    """Linear attention with a fixed decay per head: `S_t = decay_h S_(t-1) + k_t v_t^T`, `o_t = S_t^T q_t`."""
    T = h.shape[0]
    heads, dim, vdim = mixer["heads"], mixer["dim"], mixer["vdim"]
    q = silu(linear(h, W[prefix + ".q"], round_to)).view(T, heads, dim)
    k = silu(linear(h, W[prefix + ".k"], round_to)).view(T, heads, dim)
    v = silu(linear(h, W[prefix + ".v"], round_to)).view(T, heads, vdim)
    decay = torch.tensor(mixer["decay"], dtype=h.dtype)
    state = torch.zeros(heads, dim, vdim, dtype=h.dtype)
    out = torch.zeros(T, heads, vdim, dtype=h.dtype)
    for t in range(T):
        state = decay[:, None, None] * state + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", state, q[t])
    normed = rms_norm(out.reshape(T, heads * vdim), W[prefix + ".norm"], eps)
    gate = torch.sigmoid(linear(h, W[prefix + ".g"], round_to))
    return linear(round_to(normed * gate), W[prefix + ".o"], round_to)


def mlstm(h: torch.Tensor, W: Dict[str, torch.Tensor], prefix: str, mixer: dict, eps: float,
          round_to: Rounding = no_rounding) -> torch.Tensor:
    """Matrix memory with exponential input gate and a running maximum that starts at 0."""
    T = h.shape[0]
    heads, dim, vdim, cap = mixer["heads"], mixer["dim"], mixer["vdim"], mixer["gate_cap"]
    q = linear(h, W[prefix + ".q"], round_to).view(T, heads, dim) * dim ** -0.5
    k = linear(h, W[prefix + ".k"], round_to).view(T, heads, dim)
    v = linear(h, W[prefix + ".v"], round_to).view(T, heads, vdim)
    log_in = cap * torch.tanh((linear(h, W[prefix + ".i"]) + W[prefix + ".i.b"].to(h.dtype)) / cap)              # [T, heads]
    log_forget = torch.nn.functional.logsigmoid(cap * torch.tanh((linear(h, W[prefix + ".f"]) + W[prefix + ".f.b"].to(h.dtype)) / cap))
    S = torch.zeros(heads, dim, vdim, dtype=h.dtype)
    n = torch.zeros(heads, dim, dtype=h.dtype)
    m = torch.zeros(heads, dtype=h.dtype)
    out = torch.zeros(T, heads, vdim, dtype=h.dtype)
    for t in range(T):
        m_new = torch.maximum(log_forget[t] + m, log_in[t])
        keep, take = torch.exp(log_forget[t] + m - m_new), torch.exp(log_in[t] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        m = m_new
        denominator = torch.maximum((n * q[t]).sum(dim=-1).abs(), torch.exp(-m)) + 1e-6
        out[t] = torch.einsum("hdv,hd->hv", S, q[t]) / denominator[:, None]
    normed = rms_norm(out, None, eps).reshape(T, heads * vdim) * W[prefix + ".norm"].to(h.dtype)     # each head over its own vdim
    gate = torch.sigmoid(linear(h, W[prefix + ".g"], round_to))
    return linear(round_to(normed * gate), W[prefix + ".o"], round_to)


MIXERS = {"latent_attention": latent_attention, "lightning": lightning, "mlstm": mlstm}


# --------------------------------------------------------------------------- feed-forward
def gated_expert(h: torch.Tensor, W: Dict[str, torch.Tensor], prefix: str, round_to: Rounding = no_rounding) -> torch.Tensor:
    inner = round_to(silu(linear(h, W[prefix + ".gate"], round_to)) * linear(h, W[prefix + ".up"], round_to))
    return linear(inner, W[prefix + ".down"], round_to)


def route(h: torch.Tensor, W: Dict[str, torch.Tensor], prefix: str, experts: int, top: int):
    """Sigmoid scores; the choice adds a correction per expert, the weights do not; no renormalisation."""
    scores = torch.sigmoid(linear(h, W[prefix + ".router"]))
    choice = scores + W[prefix + ".correction"].to(h.dtype)
    chosen = torch.topk(choice, top, dim=-1).indices
    return chosen, torch.gather(scores, 1, chosen)


def mixture_of_experts(h: torch.Tensor, W: Dict[str, torch.Tensor], prefix: str, mlp: dict,
                       round_to: Rounding = no_rounding) -> torch.Tensor:
    experts, top = mlp["router"]["experts"], mlp["router"]["top"]
    chosen, weights = route(h, W, prefix, experts, top)
    out = torch.zeros_like(h)
    for token in range(h.shape[0]):
        for place in range(top):
            expert = int(chosen[token, place])
            out[token] += weights[token, place] * gated_expert(h[token : token + 1], W, f"{prefix}.e{expert}", round_to)[0]
    if mlp.get("shared") is not None:
        shared_gate = torch.sigmoid(linear(h, W[prefix + ".shared.sg"]))            # [T, 1]
        out = out + shared_gate * gated_expert(h, W, prefix + ".shared", round_to)
    return out


# --------------------------------------------------------------------------- model
def layer_runs(config: dict) -> Sequence[int]:
    """The order in which layers run: those before `start` once, `start .. stop-1` `times` times in a row, then the rest."""
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(count))
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    return list(range(start)) + list(range(start, stop)) * times + list(range(stop, count))


def forward(config: dict, W: Dict[str, torch.Tensor], tokens: Sequence[int], round_to: Rounding = no_rounding,
            dtype=torch.float64, keep_layers: Optional[list] = None) -> torch.Tensor:
    """Logits `[T, vocab]` of one sequence.  `keep_layers` (a list) receives the residual stream after every layer run."""
    W = {name: value.to(dtype) if value.is_floating_point() else value for name, value in W.items()}
    eps = config["norm"]["eps"]
    x = W["embed"][torch.tensor(list(tokens), dtype=torch.long)]
    for index in layer_runs(config):
        layer = config["layers"][index]
        h = round_to(rms_norm(x, W[f"l{index}.norm1"], eps))
        branch = MIXERS[layer["type"]](h, W, f"l{index}.mix", layer["mixer"], eps, round_to)
        if layer.get("mlp") is not None:
            branch = branch + mixture_of_experts(h, W, f"l{index}.mlp", layer["mlp"], round_to)
        x = x + branch
        if keep_layers is not None:
            keep_layers.append(x.clone())
    return linear(round_to(rms_norm(x, W["final.norm"], eps)), W["embed"])
