"""Small Bisudra configurations and weights for the tests, made here from the config alone (names, shapes and scales are written
out by hand; nothing is taken from the library's own list of tensors)."""
from __future__ import annotations

import json
import os
from typing import Dict

import torch

from tau_rs_b200.weights.safetensors_io import write_safetensors


def dense(ff=72):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=40):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def attention(heads=4, kv_heads=2, dim=16, vdim=24, window=37, rot_dims=8, base=5000.0, scale=None, diff=0.3, mlp="default"):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff, "scale": dim ** -0.5 if scale is None else scale,
                      "mask": {"size": window}, "rot": {"base": base, "dims": rot_dims}},
            "mlp": dense() if mlp == "default" else mlp}


def config(layers, width=96, vocab=211, eps=1e-5, taps=3, side_dim=10) -> dict:
    return {"architecture": "Bisudra", "canon": {"taps": taps}, "layers": layers, "norm": {"eps": eps}, "token_side": {"dim": side_dim},
            "vocab": vocab, "width": width}


# Both feed-forwards and none, windows shorter and longer than a page, rotations narrower than, as wide as and absent from a head.
MIXED = config([attention(), attention(heads=6, kv_heads=3, dim=8, vdim=40, window=70, rot_dims=8, diff=0.6, mlp=moe()),
                attention(heads=2, kv_heads=2, dim=24, vdim=16, window=130, rot_dims=0, diff=0.1, mlp=None),
                attention(heads=3, kv_heads=1, dim=32, vdim=32, window=64, rot_dims=16, mlp=moe(experts=5, top=3, ff=24))])
# Sizes that happen to be 1 or equal elsewhere, and nothing a multiple of 8: one head, a window of one position, two taps, one
# expert of one, all experts chosen, values wider than a warp's pass, a side input of one element.
ODD = config([attention(heads=1, kv_heads=1, dim=12, vdim=150, window=1, rot_dims=6, mlp=moe(experts=1, top=1, ff=20)),
              attention(heads=9, kv_heads=3, dim=10, vdim=6, window=5, rot_dims=10, diff=0.8, mlp=moe(experts=4, top=4, ff=12)),
              attention(heads=2, kv_heads=1, dim=20, vdim=34, window=1000, rot_dims=2, mlp=dense(ff=30))], width=100, vocab=77, eps=1e-6, taps=2, side_dim=1)
# One tap: the convolution reads the token alone and keeps no state.
ONE_TAP = config([attention(heads=2, kv_heads=1, dim=16, vdim=8, window=20, mlp=dense(ff=40)), attention(mlp=moe(experts=3, top=1, ff=16))],
                 width=64, vocab=50, taps=1, side_dim=4)
# Attention with a sharp softmax, so that single keys carry a query's weight: a key lost far back, at a page border or at the
# window's edge, or one seen beyond it, moves the logits by much more than rounding does.
PEAKY = config([attention(heads=3, kv_heads=1, dim=16, vdim=24, window=300, rot_dims=16, scale=3.0, mlp=None)], width=64, vocab=97, taps=5, side_dim=6)
EDGY = config([attention(heads=4, kv_heads=2, dim=16, vdim=16, window=33, rot_dims=4, scale=4.0, mlp=None),
               attention(heads=2, kv_heads=1, dim=16, vdim=32, window=64, rot_dims=16, scale=4.0, mlp=None)], width=64, vocab=97, taps=4, side_dim=6)


def weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """Random weights of the scales that keep every branch alive, every value one that bfloat16 holds."""
    generator = torch.Generator().manual_seed(seed)
    width, side, taps = cfg["width"], cfg["token_side"]["dim"], cfg["canon"]["taps"]
    out: Dict[str, torch.Tensor] = {}

    def matrix(name, rows, columns, gain=1.0):
        out[name] = torch.randn(rows, columns, generator=generator) * gain / columns ** 0.5

    def vector(name, count, mean, spread):
        out[name] = mean + spread * torch.randn(count, generator=generator)

    out["embed"] = torch.randn(cfg["vocab"], width, generator=generator)
    out["side.embed"] = torch.randn(cfg["vocab"], side * len(cfg["layers"]), generator=generator)
    vector("final.norm", width, 0.2, 0.05)
    vector("final.norm.b", width, 0.0, 0.1)
    for index, layer in enumerate(cfg["layers"]):
        p, mixer = f"l{index}", layer["mixer"]
        heads, kv_heads, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
        for norm in ("norm1", "norm2")[: 2 if layer["mlp"] is not None else 1]:
            vector(f"{p}.{norm}", width, 0.7, 0.2)
            vector(f"{p}.{norm}.b", width, 0.0, 0.1)
        matrix(f"{p}.mix.q", heads * 2 * dim, width)
        matrix(f"{p}.mix.k", kv_heads * 2 * dim, width)
        matrix(f"{p}.mix.v", kv_heads * vdim, width)
        matrix(f"{p}.mix.g", heads * vdim, width)
        matrix(f"{p}.mix.o", width, heads * vdim)
        vector(f"{p}.mix.q.norm", dim, 1.0, 0.2)
        vector(f"{p}.mix.k.norm", dim, 1.0, 0.2)
        for name in ("lq1", "lk1", "lq2", "lk2"):
            vector(f"{p}.mix.{name}", dim, 0.0, 0.25)
        out[f"{p}.canon1"] = 0.4 * torch.randn(width, taps, generator=generator)
        matrix(f"{p}.rg1", width, width, 2.0)
        vector(f"{p}.rg1.b", width, 0.3, 0.5)
        mlp = layer["mlp"]
        if mlp is not None:
            matrix(f"{p}.rg2", width, width, 2.0)
            vector(f"{p}.rg2.b", width, -0.2, 0.5)
            if mlp["kind"] == "dense":
                matrix(f"{p}.mlp.up", mlp["ff"], width)
                vector(f"{p}.mlp.up.b", mlp["ff"], 0.1, 0.3)
                matrix(f"{p}.mlp.down", width, mlp["ff"])
                vector(f"{p}.mlp.down.b", width, 0.0, 0.2)
            else:
                experts, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
                matrix(f"{p}.mlp.router", experts, width, 2.0)
                vector(f"{p}.mlp.router.b", experts, 0.0, 0.7)
                for expert in range(experts):
                    matrix(f"{p}.mlp.e{expert}.gate", ff, width)
                    matrix(f"{p}.mlp.e{expert}.up", ff, width)
                    matrix(f"{p}.mlp.e{expert}.down", width, ff)
        vector(f"{p}.dwa", index + 2, 0.5, 0.3)
        matrix(f"{p}.side.gate", side, width, 2.0)
        matrix(f"{p}.side.proj", width, side)
        vector(f"{p}.side.norm", width, 0.5, 0.15)
    return {name: value.to(torch.bfloat16).float() for name, value in out.items()}


def write_model(folder: str, cfg: dict, seed: int, storage=torch.bfloat16, values=None) -> Dict[str, torch.Tensor]:
    os.makedirs(folder, exist_ok=True)
    values = weights(cfg, seed) if values is None else values
    write_safetensors(os.path.join(folder, "model.safetensors"), ((name, value.to(storage)) for name, value in values.items()))
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(cfg, handle)
    return values
