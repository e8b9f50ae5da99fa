"""Tiny Torisun configurations and weights for the tests.

The configurations differ from one another in every size, in the order of the layers and in what a layer has: grouped
heads and one head per key/value head, value size below and above the query/key size, fewer rotated coordinates than a
head is wide, rotation with and without the stretching, windows shorter and longer than the sequences, no kept first
positions, a layer that reads an EARLIER layer's keys with a mask of its own (wider and narrower than the owner's), a
layer without feed-forward, one, two and three chosen experts out of counts that are no powers of two, with and without
the shared expert, sizes that are no multiples of 8 or 16.

Weights are drawn so that activations stay of order one through the layers (matrices with variance 1 / inputs), which
makes attention far from uniform: a key that is skipped or read from a wrong place changes the logits visibly.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict

import torch

from llmengine_b200.weights import write_safetensors


def mixer(heads, kv_heads, dim, vdim, scale, size, keep_first, base=10000.0, dims=None, scaling=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
         "mask": {"size": size, "keep_first": keep_first}, "rot": {"base": base, "dims": dim if dims is None else dims}}
    if scaling is not None:
        m["rot"]["scaling"] = scaling
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff, scale, shared=0):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(m, mlp):
    return {"type": "attention", "mixer": m, "mlp": mlp}


YARN = {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}

# sizes the tensor-core kernels take (multiples of 16), grouped heads, a reader with a narrower mask than its owner
TINY_A = {
    "architecture": "Torisun", "vocab": 97, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        layer(mixer(4, 2, 32, 16, 0.2, 24, 3, base=500.0, dims=16, scaling=YARN), moe(6, 2, 40, 1.5, shared=24)),
        layer(mixer(4, 2, 32, 16, 0.3, 9, 1, base=500.0, dims=16, scaling=YARN, kv_from=0), dense(72, 2.0)),
        layer(mixer(2, 1, 16, 48, 0.25, 40, 0, base=90.0), None),
    ],
}
# odd sizes everywhere (no 16-byte rows: the plain kernels and the library product), one chosen expert, no shared expert,
# a reader whose window is wider than its owner's, a window longer than any sequence of the tests
TINY_B = {
    "architecture": "Torisun", "vocab": 131, "width": 100, "norm": {"eps": 3e-4},
    "layers": [
        layer(mixer(3, 3, 20, 12, 0.27, 17, 5, base=333.0, dims=6), dense(70, 0.8)),
        layer(mixer(6, 3, 20, 12, 0.31, 30, 2, base=333.0, dims=6, kv_from=0), moe(5, 1, 33, 2.5)),
        layer(mixer(5, 1, 10, 14, 0.4, 100000, 4, base=9.0, dims=10, scaling={"factor": 1.5, "original": 32, "fast": 8.0, "slow": 1.0}),
              moe(7, 3, 24, 0.7, shared=10)),
    ],
}
# wide enough for sharp attention over long contexts; pages of 64 and 16 put page edges inside and outside the windows
TINY_C = {
    "architecture": "Torisun", "vocab": 300, "width": 128, "norm": {"eps": 2e-6},
    "layers": [
        layer(mixer(8, 2, 64, 64, 0.14, 130, 70, base=5e5, dims=32, scaling={"factor": 3.0, "original": 256, "fast": 24.0, "slow": 1.5}),
              dense(192, 1.2)),
        layer(mixer(8, 2, 64, 64, 0.11, 64, 17, base=5e5, dims=32, scaling={"factor": 3.0, "original": 256, "fast": 24.0, "slow": 1.5},
                    kv_from=0), moe(12, 3, 48, 1.8, shared=64)),
        layer(mixer(4, 4, 32, 32, 0.18, 31, 0, base=1e4), moe(12, 3, 48, 1.8)),
    ],
}
# one layer with one mechanism each
ONLY_ATTENTION = {"architecture": "Torisun", "vocab": 61, "width": 48, "norm": {"eps": 1e-6},
                  "layers": [layer(mixer(4, 2, 16, 32, 0.3, 11, 2, base=100.0, dims=8), None)]}
WITH_DENSE = {"architecture": "Torisun", "vocab": 61, "width": 48, "norm": {"eps": 1e-6},
              "layers": [layer(mixer(2, 2, 16, 16, 0.3, 50, 0, base=100.0), dense(80, 1.0))]}
WITH_MOE = {"architecture": "Torisun", "vocab": 61, "width": 48, "norm": {"eps": 1e-6},
            "layers": [layer(mixer(2, 2, 16, 16, 0.3, 50, 0, base=100.0), moe(9, 2, 32, 1.0, shared=16))]}
WITH_READER = {"architecture": "Torisun", "vocab": 61, "width": 48, "norm": {"eps": 1e-6},
               "layers": [layer(mixer(2, 1, 16, 32, 0.3, 7, 1, base=100.0, dims=8), None),
                          layer(mixer(2, 1, 16, 32, 0.5, 13, 3, base=100.0, dims=8, kv_from=0), None)]}


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    """Names and shapes of a model's tensors, from its config.json keys."""
    D, V = cfg["width"], cfg["vocab"]
    shapes: Dict[str, tuple] = {"embed": (V, D), "embed.norm": (D,), "final.norm": (D,)}
    for i, L in enumerate(cfg["layers"]):
        m, p = L["mixer"], f"l{i}."
        H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        shapes[p + "norm1"] = (D,)
        shapes[p + "mix.q"] = (H * dk, D)
        shapes[p + "mix.q.norm"] = (H * dk,)
        shapes[p + "mix.sink"] = (H,)
        shapes[p + "mix.o"] = (D, H * dv)
        if m.get("kv_from") is None:
            shapes[p + "mix.k"] = (G * dk, D)
            shapes[p + "mix.v"] = (G * dv, D)
            shapes[p + "mix.k.norm"] = (G * dk,)
        mlp = L["mlp"]
        if mlp is None:
            continue
        shapes[p + "norm2"] = (D,)
        subs = []
        if mlp["kind"] == "dense":
            subs.append(("mlp.", mlp["ff"]))
        else:
            shapes[p + "mlp.router"] = (mlp["router"]["experts"], D)
            subs += [(f"mlp.e{e}.", mlp["expert"]["ff"]) for e in range(mlp["router"]["experts"])]
            if mlp.get("shared"):
                subs.append(("mlp.shared.", mlp["shared"]["ff"]))
        for s, ff in subs:
            shapes[p + s + "gate"] = (ff, D)
            shapes[p + s + "up"] = (ff, D)
            shapes[p + s + "down"] = (D, ff)
    return shapes


def random_tensors(cfg: dict, seed: int, sharpen: float = 1.0) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm", "norm1", "norm2"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
            if name.endswith("q.norm"):
                t = t * sharpen
        elif leaf == "sink":
            t = torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        elif leaf == "router":
            t = 2.0 * torch.randn(shape, generator=g) / math.sqrt(shape[1])
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
        out[name] = t.to(torch.bfloat16)
    return out


def make_torisun_dir(path: str, cfg: dict, seed: int, sharpen: float = 1.0, edit=None) -> str:
    """A model folder with random weights; `edit(tensors)` may change single tensors before they are written."""
    os.makedirs(path, exist_ok=True)
    tensors = random_tensors(cfg, seed, sharpen)
    if edit is not None:
        edit(tensors)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(path, "model.safetensors"), tensors, {"format": "pt"})
    return path
