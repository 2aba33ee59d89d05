"""Small Fasesun configurations and weights for the tests, made here from the config alone (names, shapes and scales are
written out by hand; nothing is taken from the library's own list of tensors)."""
from __future__ import annotations

import json
import os
from typing import Dict

import torch

from tau_rs_b200.weights.safetensors_io import write_safetensors


def moe(experts=6, top=3, ff=40, shared_ff=56):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}, "shared": {"ff": shared_ff}}


def latent(heads=5, dim=24, rot_dim=16, rot_dims=None, vdim=40, q_rank=48, kv_rank=72, scale=None, base=5000.0, mlp="default"):
    rot_dims = rot_dim if rot_dims is None else rot_dims
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                                                   "scale": (dim + rot_dim) ** -0.5 if scale is None else scale, "rot": {"base": base, "dims": rot_dims}},
            "mlp": moe() if mlp == "default" else mlp}


def mlstm(heads=2, dim=40, vdim=24, gate_cap=12.0, mlp="default"):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": gate_cap}, "mlp": moe() if mlp == "default" else mlp}


def lightning(heads=3, dim=24, vdim=40, decay=None, mlp="default"):
    decay = decay or [0.5 + 0.499 * (index + 1) / heads for index in range(heads)]
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}, "mlp": moe() if mlp == "default" else mlp}


def config(layers, width=96, vocab=211, eps=1e-5, loop=None) -> dict:
    out = {"architecture": "Fasesun", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if loop is not None:
        out["loop"] = dict(zip(("start", "stop", "times"), loop))
    return out


# Every mixer, a loop over the middle two layers, a layer without a feed-forward, a rotation narrower than the rotated part.
MIXED = config([lightning(), latent(rot_dims=8), mlstm(), latent(heads=2, dim=16, rot_dim=8, vdim=16, q_rank=24, kv_rank=40, mlp=None)], loop=(1, 3, 3))
# Sizes that happen to be 1 or equal elsewhere: one head, one expert of one, all experts chosen, more heads than a block serves at once,
# a value width beyond one tile of the state kernel, key widths that several threads share.
ODD = config([mlstm(heads=1, dim=16, vdim=150, gate_cap=4.0, mlp=moe(experts=1, top=1, ff=24, shared_ff=16)),
              latent(heads=9, dim=16, rot_dim=8, vdim=16, q_rank=24, kv_rank=40, mlp=moe(experts=4, top=4, ff=24, shared_ff=24)),
              lightning(heads=1, dim=72, vdim=8, decay=[0.97], mlp=moe(experts=5, top=1, ff=16, shared_ff=8)),
              mlstm(heads=3, dim=136, vdim=8, mlp=None)], width=64, vocab=130, eps=1e-6)
# Attention alone with a sharp softmax, so that single keys carry a query's weight and a lost key shows.
PEAKY = config([latent(heads=3, dim=16, rot_dim=16, vdim=24, q_rank=32, kv_rank=48, scale=2.5, mlp=None)], width=64, vocab=97)


# Nothing a multiple of 8: rows that no 16-byte load can take, products that no tensor-core tile fits.
RAGGED = config([latent(heads=3, dim=12, rot_dim=6, vdim=10, q_rank=20, kv_rank=30, mlp=moe(experts=5, top=2, ff=20, shared_ff=12)),
                 mlstm(heads=2, dim=12, vdim=10, mlp=moe(experts=5, top=2, ff=20, shared_ff=12)),
                 lightning(heads=2, dim=10, vdim=6, mlp=None)], width=100, vocab=77, loop=(0, 2, 2))


def weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """Random weights of the scales that keep every branch alive, every value one that bfloat16 holds."""
    generator = torch.Generator().manual_seed(seed)
    width = cfg["width"]
    out: Dict[str, torch.Tensor] = {}

    def matrix(name, rows, columns, gain=1.0):
        out[name] = torch.randn(rows, columns, generator=generator) * gain / columns ** 0.5

    def vector(name, count, mean, spread):
        out[name] = mean + spread * torch.randn(count, generator=generator)

    out["embed"] = torch.randn(cfg["vocab"], width, generator=generator)
    vector("final.norm", width, 0.1, 0.03)
    for index, layer in enumerate(cfg["layers"]):
        mixer, prefix = layer["mixer"], f"l{index}.mix"
        vector(f"l{index}.norm1", width, 1.0, 0.2)
        heads, dim, vdim = mixer["heads"], mixer["dim"], mixer["vdim"]
        if layer["type"] == "latent_attention":
            rot, q_rank, kv_rank = mixer["rot_dim"], mixer["q_rank"], mixer["kv_rank"]
            matrix(prefix + ".dq", q_rank, width)
            vector(prefix + ".dq.norm", q_rank, 1.0, 0.2)
            matrix(prefix + ".uq", heads * (dim + rot), q_rank, 1.5)
            matrix(prefix + ".dkv", kv_rank + rot, width)
            vector(prefix + ".dkv.norm", kv_rank, 1.0, 0.2)
            matrix(prefix + ".uk", heads * dim, kv_rank, 1.5)
            matrix(prefix + ".uv", heads * vdim, kv_rank)
            vector(prefix + ".sink", heads, 1.0, 1.5)
            matrix(prefix + ".g", heads * vdim, width)
            matrix(prefix + ".o", width, heads * vdim)
        else:
            matrix(prefix + ".q", heads * dim, width)
            matrix(prefix + ".k", heads * dim, width)
            matrix(prefix + ".v", heads * vdim, width)
            matrix(prefix + ".g", heads * vdim, width)
            matrix(prefix + ".o", width, heads * vdim)
            vector(prefix + ".norm", heads * vdim, 1.0, 0.2)
            if layer["type"] == "mlstm":
                matrix(prefix + ".i", heads, width, 2.0)
                vector(prefix + ".i.b", heads, 0.3, 0.6)
                matrix(prefix + ".f", heads, width, 2.0)
                vector(prefix + ".f.b", heads, 3.0, 2.0)
        mlp = layer["mlp"]
        if mlp is not None:
            prefix = f"l{index}.mlp"
            experts, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            matrix(prefix + ".router", experts, width, 2.0)
            vector(prefix + ".correction", experts, 0.0, 0.5)
            for expert in range(experts):
                matrix(f"{prefix}.e{expert}.gate", ff, width)
                matrix(f"{prefix}.e{expert}.up", ff, width)
                matrix(f"{prefix}.e{expert}.down", width, ff)
            shared = mlp["shared"]["ff"]
            matrix(prefix + ".shared.gate", shared, width)
            matrix(prefix + ".shared.up", shared, width)
            matrix(prefix + ".shared.down", width, shared)
            matrix(prefix + ".shared.sg", 1, width, 2.0)
    return {name: value.to(torch.bfloat16).float() for name, value in out.items()}


def write_model(folder: str, cfg: dict, seed: int, storage=torch.bfloat16) -> Dict[str, torch.Tensor]:
    os.makedirs(folder, exist_ok=True)
    values = weights(cfg, seed)
    write_safetensors(os.path.join(folder, "model.safetensors"), ((name, value.to(storage)) for name, value in values.items()))
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(cfg, handle)
    return values
