"""The plain implementation of the Torisun design: whole sequences, no cache, one function per
mechanism, elementary tensor arithmetic on the CPU.

It shares no code with the engine: it reads config.json and model.safetensors itself.  `round_to`
rounds to bfloat16 where the engine's bfloat16 path stores bfloat16 (weights, the inputs of the matrix
products, cached keys and values); the arithmetic itself is always 32-bit.

Notation: D width, H query heads, G key/value heads, dk query/key size and dv value size per head,
T tokens, E experts.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch

from plain_bepuzen import read_safetensors

F32 = torch.float32


def _r(x: torch.Tensor, round_to: Optional[torch.dtype]) -> torch.Tensor:
    return x if round_to is None else x.to(round_to).to(F32)


# --------------------------------------------------------------------- mechanisms
def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * w over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w.to(F32)


def yarn_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """(f [dims/2], amplitude).  f_i = base^(-2i/dims); with scaling the slow turning coordinates are slowed by
    `factor`, the fast ones kept, a linear ramp between them, and cos and sin are stretched by 0.1 ln(factor) + 1."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    if not scaling:
        return f.to(F32), 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def turn(t):          # the coordinate that makes t turns over the original length
        return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(turn(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((torch.arange(half, dtype=torch.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    f = f / factor * ramp + f * (1.0 - ramp)
    return f.to(F32), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, f: torch.Tensor, amplitude: float) -> torch.Tensor:
    """x [T, heads, d]: the first 2 len(f) coordinates of every head in rotate-half pairs (i, i + len(f)), the rest pass."""
    half = f.numel()
    ang = positions.to(F32)[:, None] * f[None, :]                     # 32-bit angle
    c, s = (torch.cos(ang) * amplitude)[:, None, :], (torch.sin(ang) * amplitude)[:, None, :]
    u, v = x[..., :half], x[..., half:2 * half]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., 2 * half:]], -1)


def visible(T: int, size: int, keep_first: int) -> torch.Tensor:
    """[T, T] bool: query i sees key j if j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def sink_softmax(scores: torch.Tensor, sink: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """scores [H, T, T], sink [H]: softmax over the visible keys whose denominator also holds exp(sink_h)."""
    s = scores.masked_fill(~mask[None], float("-inf"))
    m = torch.maximum(s.max(-1, keepdim=True).values, sink.to(F32)[:, None, None])
    e = torch.exp(s - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink.to(F32)[:, None, None] - m))


def keys_and_values(h, w, pre, m, eps, positions, round_to):
    """A layer's own keys (normed over the whole projection, rotated) [T, G, dk] and values [T, G, dv]."""
    G, dk, dv = m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    k = rms_norm(_r(h @ w[pre + "k"].t(), round_to), w[pre + "k.norm"], eps).view(T, G, dk)
    f, amp = yarn_frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    k = _r(rotate(k, positions, f, amp), round_to)
    v = _r(h @ w[pre + "v"].t(), round_to).view(T, G, dv)
    return k, v


def attention(h, w, pre, m, eps, positions, kv, round_to):
    """The mixer: h [T, D] (already rounded for the products), `kv` = (keys, values) of the layer whose cache it reads."""
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = rms_norm(_r(h @ w[pre + "q"].t(), round_to), w[pre + "q.norm"], eps).view(T, H, dk)
    f, amp = yarn_frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    q = _r(rotate(q, positions, f, amp), round_to)
    k, v = kv
    rep = H // G
    kh = k.repeat_interleave(rep, 1)                                   # query head h reads key/value head h // rep
    vh = v.repeat_interleave(rep, 1)
    scores = torch.einsum("ihd,jhd->hij", q, kh) * m["scale"]
    p = sink_softmax(scores, w[pre + "sink"], visible(T, m["mask"]["size"], m["mask"]["keep_first"]))
    o = _r(torch.einsum("hij,jhd->ihd", p, vh).reshape(T, H * dv), round_to)
    return o @ w[pre + "o"].t()


def dense_ff(h, w, pre, limit, round_to):
    g = torch.clamp(_r(h @ w[pre + "gate"].t(), round_to), max=limit)
    u = torch.clamp(_r(h @ w[pre + "up"].t(), round_to), -limit, limit)
    y = g * torch.sigmoid(1.702 * g) * (u + 1.0)
    return _r(y, round_to) @ w[pre + "down"].t()


def silu_ff(h, w, pre, round_to):
    g = _r(h @ w[pre + "gate"].t(), round_to)
    u = _r(h @ w[pre + "up"].t(), round_to)
    return _r(g * torch.sigmoid(g) * u, round_to) @ w[pre + "down"].t()


def route(h, w_router, top: int, scale: float):
    """(experts [T, top], weights [T, top]): the `top` largest sigmoid scores, divided by their sum, times `scale`."""
    s = torch.sigmoid(h @ w_router.t())
    val, idx = torch.topk(s, top, dim=-1)
    return idx, val / (val.sum(-1, keepdim=True) + 1e-20) * scale


def routing_gaps(h, w_router, top: int) -> torch.Tensor:
    """[T]: how far the last chosen expert's router logit lies above the first one not chosen (inf: all are chosen)."""
    z = torch.sort(h @ w_router.t(), dim=-1, descending=True).values
    return z[:, top - 1] - z[:, top] if top < z.shape[1] else torch.full((h.shape[0],), float("inf"))


def moe_ff(h, w, pre, mlp, round_to, gaps=None):
    r = mlp["router"]
    idx, wt = route(h, w[pre + "router"], r["top"], r["scale"])
    if gaps is not None:
        gaps.append(routing_gaps(h, w[pre + "router"], r["top"]))
    out = torch.zeros(h.shape[0], w[pre + "e0.down"].shape[0])
    for e in range(r["experts"]):
        rows, slot = torch.nonzero(idx == e, as_tuple=True)
        if rows.numel():
            out[rows] += wt[rows, slot][:, None] * silu_ff(h[rows], w, f"{pre}e{e}.", round_to)
    if mlp.get("shared"):
        out = out + silu_ff(h, w, pre + "shared.", round_to)
    return out


# --------------------------------------------------------------------- the model
class PlainTorisun:
    def __init__(self, model_dir: str, round_to: Optional[torch.dtype] = None):
        with open(os.path.join(model_dir, "config.json")) as f:
            self.cfg = json.load(f)
        self.w = {n: t.to(F32) for n, t in read_safetensors(os.path.join(model_dir, "model.safetensors")).items()}
        self.round_to = round_to

    def forward(self, ids: Sequence[int], layers_out: Optional[list] = None) -> torch.Tensor:
        cfg, w, rt = self.cfg, self.w, self.round_to
        eps = cfg["norm"]["eps"]
        T = len(ids)
        pos = torch.arange(T)
        x = rms_norm(w["embed"][torch.tensor(list(ids), dtype=torch.long)], w["embed.norm"], eps)
        kv: Dict[int, tuple] = {}
        gaps: list = []
        for i, L in enumerate(cfg["layers"]):
            m, pre = L["mixer"], f"l{i}.mix."
            h = _r(x, rt)
            src = m.get("kv_from")
            if src is None:
                kv[i] = keys_and_values(h, w, pre, m, eps, pos, rt)
                src = i
            x = x + rms_norm(attention(h, w, pre, m, eps, pos, kv[src], rt), w[f"l{i}.norm1"], eps)
            mlp = L.get("mlp")
            if mlp is not None:
                h = _r(x, rt)
                if mlp["kind"] == "dense":
                    y = dense_ff(h, w, f"l{i}.mlp.", mlp["limit"], rt)
                else:
                    y = moe_ff(h, w, f"l{i}.mlp.", mlp, rt, gaps)
                x = x + rms_norm(y, w[f"l{i}.norm2"], eps)
            if layers_out is not None:
                layers_out.append(x.clone())
        # per position, the closest call any router of the model made (a test may want to keep away from those)
        self.gaps = torch.stack(gaps).min(0).values if gaps else torch.full((T,), float("inf"))
        return _r(rms_norm(x, w["final.norm"], eps), rt) @ w["embed"].t()

    def logits(self, ids: Sequence[int]) -> torch.Tensor:
        return self.forward(ids)
