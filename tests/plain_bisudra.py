"""Bisudra stated plainly: one function per mechanism, float64, whole sequences, masks instead of caches.

Shares nothing with the library.  `weights` maps tensor names to float64 tensors, `config` is the dictionary that a
folder's config.json holds.  Every function takes one sequence `[tokens, ...]` whose first row is position 0.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def layer_norm(x, weight, bias, eps):
    mean = x.mean(-1, keepdim=True)
    deviation = x - mean
    return deviation / torch.sqrt((deviation * deviation).mean(-1, keepdim=True) + eps) * weight + bias


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def causal_taps(h, taps_weight):
    """`out[t] = sum_j w[:, j] * h[t - taps + 1 + j]`, rows before the sequence's start being zero."""
    tokens, _ = h.shape
    taps = taps_weight.shape[1]
    out = torch.zeros_like(h)
    for j in range(taps):
        back = taps - 1 - j                      # tap j reads the row `back` positions earlier
        if back < tokens:
            out[back:] += taps_weight[:, j] * h[: tokens - back]
    return out


def rotate_pairs(x, rotary_dim, base, first_position=0):
    """`x` [tokens, ..., dim]: elements (2i, 2i+1) of the first `rotary_dim` turn by `position * base^(-2i / rotary_dim)`."""
    out = x.clone()
    positions = torch.arange(first_position, first_position + x.shape[0], dtype=F).view(-1, *([1] * (x.dim() - 2)))
    for i in range(rotary_dim // 2):
        angle = positions * base ** (-2.0 * i / rotary_dim)
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * torch.cos(angle) - v * torch.sin(angle)
        out[..., 2 * i + 1] = v * torch.cos(angle) + u * torch.sin(angle)
    return out


def windowed_softmax_attention(q, k, v, scale, window):
    """One head: `q`, `k` [tokens, dim], `v` [tokens, vdim]; token i sees j with 0 <= i - j < window."""
    tokens = q.shape[0]
    distance = torch.arange(tokens).view(-1, 1) - torch.arange(tokens).view(1, -1)          # i - j
    scores = (q @ k.T) * scale
    scores = scores.masked_fill((distance < 0) | (distance >= window), float("-inf"))
    return torch.softmax(scores, dim=-1) @ v


def differential_attention(h, weights, prefix, mixer, eps):
    """Two softmax maps per head over the same values, the second subtracted `lambda` times; unit RMS per head; sigmoid gate."""
    heads, kv_heads, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    diff, scale, window = mixer["diff"], mixer["scale"], mixer["mask"]["size"]
    tokens = h.shape[0]
    q = (h @ weights[f"{prefix}.q"].T).view(tokens, heads, 2, dim)
    k = (h @ weights[f"{prefix}.k"].T).view(tokens, kv_heads, 2, dim)
    v = (h @ weights[f"{prefix}.v"].T).view(tokens, kv_heads, vdim)
    q = unit_rms(q, eps) * weights[f"{prefix}.q.norm"]
    k = unit_rms(k, eps) * weights[f"{prefix}.k.norm"]
    q = rotate_pairs(q, mixer["rot"]["dims"], mixer["rot"]["base"])
    k = rotate_pairs(k, mixer["rot"]["dims"], mixer["rot"]["base"])
    lam = (math.exp(float((weights[f"{prefix}.lq1"] * weights[f"{prefix}.lk1"]).sum()))
           - math.exp(float((weights[f"{prefix}.lq2"] * weights[f"{prefix}.lk2"]).sum())) + diff)
    out = torch.zeros((tokens, heads, vdim), dtype=F)
    for head in range(heads):
        group = head // (heads // kv_heads)
        first = windowed_softmax_attention(q[:, head, 0], k[:, group, 0], v[:, group], scale, window)
        second = windowed_softmax_attention(q[:, head, 1], k[:, group, 1], v[:, group], scale, window)
        out[:, head] = unit_rms(first - lam * second, eps) * (1.0 - diff)
    gate = torch.sigmoid(h @ weights[f"{prefix}.g"].T)
    return (out.reshape(tokens, heads * vdim) * gate) @ weights[f"{prefix}.o"].T


def dense_feed_forward(h, weights, prefix):
    inner = torch.relu(h @ weights[f"{prefix}.up"].T + weights[f"{prefix}.up.b"]) ** 2
    return inner @ weights[f"{prefix}.down"].T + weights[f"{prefix}.down.b"]


def routed_feed_forward(h, weights, prefix, mlp):
    experts, top = mlp["router"]["experts"], mlp["router"]["top"]
    logits = h @ weights[f"{prefix}.router"].T + weights[f"{prefix}.router.b"]
    chosen = torch.topk(logits, top, dim=-1).indices                  # the largest logits
    share = torch.zeros_like(logits).scatter(1, chosen, torch.softmax(torch.gather(logits, 1, chosen), dim=-1))
    out = torch.zeros_like(h)
    for expert in range(experts):                                      # every expert on every token, weighted by zero where not chosen
        name = f"{prefix}.e{expert}"
        gate = h @ weights[f"{name}.gate"].T
        inner = gate * torch.sigmoid(gate) * (h @ weights[f"{name}.up"].T)
        out += share[:, expert : expert + 1] * (inner @ weights[f"{name}.down"].T)
    return out


def token_side_input(x, tokens, weights, prefix, layer, side_dim, eps):
    table = weights["side.embed"][tokens][:, layer * side_dim : (layer + 1) * side_dim]
    y = (gelu_tanh(x @ weights[f"{prefix}.side.gate"].T) * table) @ weights[f"{prefix}.side.proj"].T
    return unit_rms(y, eps) * weights[f"{prefix}.side.norm"]


def forward(tokens, weights, config, return_layers=False):
    """Logits `[tokens, vocab]` of one sequence from its first token on (and the results of the layers, if asked)."""
    eps = config["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = weights["embed"][tokens]
    results = [x]
    for index, layer in enumerate(config["layers"]):
        p = f"l{index}"
        if layer["type"] != "attention":
            raise ValueError(layer["type"])
        read = x + causal_taps(x, weights[f"{p}.canon1"])
        mixed = differential_attention(read, weights, f"{p}.mix", layer["mixer"], eps)
        mixed = mixed * torch.sigmoid(x @ weights[f"{p}.rg1"].T + weights[f"{p}.rg1.b"])
        x = x + layer_norm(mixed, weights[f"{p}.norm1"], weights[f"{p}.norm1.b"], eps)
        mlp = layer["mlp"]
        if mlp is not None:
            fed = dense_feed_forward(x, weights, f"{p}.mlp") if mlp["kind"] == "dense" else routed_feed_forward(x, weights, f"{p}.mlp", mlp)
            fed = fed * torch.sigmoid(x @ weights[f"{p}.rg2"].T + weights[f"{p}.rg2.b"])
            x = x + layer_norm(fed, weights[f"{p}.norm2"], weights[f"{p}.norm2.b"], eps)
        x = x + token_side_input(x, tokens, weights, p, index, config["token_side"]["dim"], eps)
        results.append(x)
        x = sum(weights[f"{p}.dwa"][j] * results[j] for j in range(index + 2))
    logits = layer_norm(x, weights["final.norm"], weights["final.norm.b"], eps) @ weights["embed"].T
    return (logits, results[1:]) if return_layers else logits
