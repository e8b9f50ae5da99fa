"""Tiny Bepuzen configurations and weights for the tests.

The configurations differ from one another in every size, in the order of the layer types and in what a layer has:
a layer without feed-forward, a model without the per-layer token input, fewer rotated coordinates than the rotated
part is wide, query/key size different from the value size, one head, latent sizes that the tensor-core kernel takes
(multiples of 64) and one it does not, head counts on both sides of the kernel's row-tile shapes (16, 32).

Weights are drawn so that activations stay of order one through the layers (matrices with variance 1 / inputs), which
makes attention far from uniform: a key that is skipped or read from a wrong place changes the logits visibly.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, Optional

import torch

from llmengine_b200.weights import write_safetensors


def mixer1(heads, dim, rot_dim, vdim, kv_rank, scale, base=10000.0, dims=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
            "rot": {"base": base, "dims": rot_dim if dims is None else dims}}


def mixer2(heads, dim, vdim, kv_rank, scale):
    return {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale}


def layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


L1, L2 = "latent_attention", "latent_attention_2"

TINY_P = {
    "architecture": "Bepuzen", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "token_side": {"dim": 8},
    "layers": [
        layer(L1, mixer1(4, 16, 16, 24, 64, 0.21, base=500.0, dims=8), 96),
        layer(L2, mixer2(2, 32, 16, 64, 0.17), 0),
        layer(L1, mixer1(1, 8, 8, 8, 128, 0.4), 40),
    ],
}
TINY_Q = {
    "architecture": "Bepuzen", "vocab": 211, "width": 96, "norm": {"eps": 3e-4},
    "layers": [
        layer(L2, mixer2(3, 16, 32, 48, 0.25), 72),
        layer(L2, mixer2(40, 8, 8, 64, 0.35), 64),
        layer(L1, mixer1(20, 8, 16, 8, 64, 0.2, base=77.0), 0),
    ],
}
# odd sizes everywhere: no 16-byte rows, products that only the library takes, a latent size no tensor-core kernel is built for
TINY_S = {
    "architecture": "Bepuzen", "vocab": 131, "width": 100, "norm": {"eps": 2e-5}, "token_side": {"dim": 5},
    "layers": [
        layer(L1, mixer1(3, 20, 12, 12, 72, 0.27, base=333.0, dims=6), 70),
        layer(L1, mixer1(5, 6, 10, 14, 40, 0.31, base=9.0), 0),
        layer(L2, mixer2(7, 10, 6, 56, 0.4), 33),
    ],
}
# one layer of each mixer and nothing else, and single sublayers added to it: each mechanism by itself
ONLY_L2 = {"architecture": "Bepuzen", "vocab": 61, "width": 48, "norm": {"eps": 1e-6},
           "layers": [layer(L2, mixer2(4, 16, 8, 64, 0.3), 0)]}
ONLY_L1 = {"architecture": "Bepuzen", "vocab": 61, "width": 48, "norm": {"eps": 1e-6},
           "layers": [layer(L1, mixer1(4, 8, 24, 16, 64, 0.3, base=100.0, dims=16), 0)]}
WITH_FF = {"architecture": "Bepuzen", "vocab": 61, "width": 48, "norm": {"eps": 1e-6},
           "layers": [layer(L2, mixer2(2, 8, 8, 64, 0.3), 80)]}
WITH_SIDE = {"architecture": "Bepuzen", "vocab": 61, "width": 48, "norm": {"eps": 1e-6}, "token_side": {"dim": 24},
             "layers": [layer(L2, mixer2(2, 8, 8, 64, 0.3), 0), layer(L2, mixer2(2, 8, 8, 64, 0.3), 0)]}
# wide enough for sharp attention over long contexts; pages of 16 put many page edges into a sequence
TINY_R = {
    "architecture": "Bepuzen", "vocab": 300, "width": 128, "norm": {"eps": 1e-5}, "token_side": {"dim": 12},
    "layers": [
        layer(L2, mixer2(6, 32, 32, 128, 0.5), 192),
        layer(L1, mixer1(6, 32, 16, 24, 128, 0.4), 176),
    ],
}


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    """Names and shapes of a model's tensors, from its config.json keys."""
    D, V = cfg["width"], cfg["vocab"]
    n = len(cfg["layers"])
    side = cfg.get("token_side")
    shapes: Dict[str, tuple] = {"embed": (V, D), "final.norm": (), "head": (V, D)}
    if side:
        shapes["side.embed"] = (V, n * side["dim"])
    for i, L in enumerate(cfg["layers"]):
        m, p = L["mixer"], f"l{i}."
        rot = m.get("rot_dim", 0) if L["type"] == L1 else 0
        shapes[p + "norm1"] = ()
        shapes[p + "mix.q"] = (m["heads"] * (m["dim"] + rot), D)
        shapes[p + "mix.dkv"] = (m["kv_rank"] + rot, D)
        shapes[p + "mix.dkv.norm"] = (m["kv_rank"],)
        shapes[p + "mix.uk"] = (m["heads"] * m["dim"], m["kv_rank"])
        shapes[p + "mix.uv"] = (m["heads"] * m["vdim"], m["kv_rank"])
        shapes[p + "mix.o"] = (D, m["heads"] * m["vdim"])
        if L["type"] == L1:
            shapes[p + "mix.sink"] = (m["heads"],)
            shapes[p + "mix.g"] = (m["heads"] * m["vdim"], D)
        if L["mlp"]:
            shapes[p + "mlp.up"] = (L["mlp"]["ff"], D)
            shapes[p + "mlp.down"] = (D, L["mlp"]["ff"])
            shapes[p + "mlp.act"] = (2,)
        if side:
            shapes[p + "side.gate"] = (side["dim"], D)
            shapes[p + "side.proj"] = (D, side["dim"])
            shapes[p + "side.norm"] = (D,)
    return shapes


def random_tensors(cfg: dict, seed: int, sharpen: float = 1.0) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1",) or name == "final.norm":
            t = 1.0 + 0.2 * torch.randn((), generator=g)
        elif leaf == "norm":
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif leaf in ("sink", "act"):
            t = torch.randn(shape, generator=g)
        elif name == "side.embed":
            t = torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
            if leaf == "q":
                t = t * sharpen
        out[name] = t.to(torch.bfloat16)
    return out


def make_bepuzen_dir(path: str, cfg: dict, seed: int, sharpen: float = 1.0,
                     edit=None) -> str:
    """A model folder with random weights; `edit(tensors)` may change single tensors before they are written."""
    os.makedirs(path, exist_ok=True)
    tensors = random_tensors(cfg, seed, sharpen)
    if edit is not None:
        edit(tensors)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(path, "model.safetensors"), tensors, {"format": "pt"})
    return path
