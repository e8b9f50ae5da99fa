"""The plain implementation of the Bepuzen design: whole sequences, no cache, one function per
mechanism, elementary tensor arithmetic on the CPU.

It shares no code with the engine: it reads config.json and model.safetensors itself and keeps
keys and values per head, as the design is defined (the engine caches the latent and never forms
them).  `round_to` rounds to bfloat16 where the engine's bfloat16 path stores bfloat16 (weights, the
inputs of the matrix products, the cached latent); the arithmetic itself is always 32-bit.

Notation: D width, H heads, dn unrotated and dr rotated query/key size per head, dv value size, r latent
size, T tokens.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

F32 = torch.float32


def _r(x: torch.Tensor, round_to: Optional[torch.dtype]) -> torch.Tensor:
    return x if round_to is None else x.to(round_to).to(F32)


def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """8-byte little-endian header length, a JSON header (name -> dtype, shape, data_offsets), the data."""
    with open(path, "rb") as f:
        raw = f.read()
    n = struct.unpack("<Q", raw[:8])[0]
    head = json.loads(raw[8:8 + n])
    data = raw[8 + n:]
    out = {}
    for name, e in head.items():
        if name == "__metadata__":
            continue
        a, b = e["data_offsets"]
        buf = data[a:b]
        if e["dtype"] == "BF16":
            u = np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(u.view(np.float32).copy())
        elif e["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(buf, dtype="<f4").copy())
        elif e["dtype"] == "I32":
            t = torch.from_numpy(np.frombuffer(buf, dtype="<i4").copy())
        else:
            raise ValueError(f"{name}: dtype {e['dtype']}")
        out[name] = t.reshape(e["shape"])
    return out


# --------------------------------------------------------------------- mechanisms
def scalar_rms_norm(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * g with a single number g for all coordinates."""
    ms = (x * x).mean(-1, keepdim=True)
    return x / torch.sqrt(ms + eps) * g.to(F32).reshape(())


def weighted_rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * w with one weight per coordinate."""
    ms = (x * x).mean(-1, keepdim=True)
    return x / torch.sqrt(ms + eps) * w.to(F32)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0)


def xielu(z: torch.Tensor, pq: torch.Tensor) -> torch.Tensor:
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2."""
    p, q = pq.to(F32)[0], pq.to(F32)[1]
    pos = softplus(p) * z * z + 0.5 * z
    neg = (0.5 + softplus(q)) * (torch.expm1(torch.clamp(z, max=0)) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def rotate_half(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """The first `dims` coordinates of the last axis: coordinate i pairs with i + dims/2; the pair (u, v) at
    position p becomes (u cos a - v sin a, v cos a + u sin a), a = p * base^(-2i/dims), the angle in 32-bit.
    The coordinates from `dims` on pass unchanged.  x is [T, ..., d]."""
    half = dims // 2
    i = torch.arange(half, dtype=F32)
    f = torch.pow(torch.tensor(base, dtype=F32), -2.0 * i / dims)
    a = positions.to(F32)[:, None] * f[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    co, si = torch.cos(a.double()).to(F32).reshape(shape), torch.sin(a.double()).to(F32).reshape(shape)
    u, v, rest = x[..., :half], x[..., half:dims], x[..., dims:]
    return torch.cat([u * co - v * si, v * co + u * si, rest], dim=-1)


def causal_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                             sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q, k [T, H, d], v [T, H, dv]; position i sees every j <= i; with `sink` [H] the softmax denominator also
    holds exp(sink_h), which has no value, is not scaled and counts once."""
    T, H, _ = q.shape
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, float("-inf"))
    if sink is not None:
        s = torch.cat([s, sink.to(F32)[:, None, None].expand(H, T, 1)], dim=-1)
    w = torch.softmax(s, dim=-1)[..., :T]
    return torch.einsum("hij,jhd->ihd", w, v)


def latent_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], m: dict, eps: float, positions: torch.Tensor,
                     rotary: bool, round_to=None) -> torch.Tensor:
    """Both latent mixers.  `rotary` True: rotated query/key part shared by all heads, sink, output gate."""
    H, dn, dv, r = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
    dr = m["rot_dim"] if rotary else 0
    T = h.shape[0]
    hb = _r(h, round_to)
    q = _r(hb @ W["q"].t(), round_to).reshape(T, H, dn + dr)
    dkv = hb @ W["dkv"].t()
    c = _r(weighted_rms_norm(dkv[:, :r], W["dkv.norm"], eps), round_to)
    k = _r(c @ W["uk"].t(), round_to).reshape(T, H, dn)
    v = _r(c @ W["uv"].t(), round_to).reshape(T, H, dv)
    if rotary:
        rot = m["rot"]
        kr = _r(rotate_half(_r(dkv[:, r:], round_to), positions, rot["base"], rot["dims"]), round_to)
        qr = _r(rotate_half(q[..., dn:], positions, rot["base"], rot["dims"]), round_to)
        q = torch.cat([q[..., :dn], qr], dim=-1)
        k = torch.cat([k, kr[:, None, :].expand(T, H, dr)], dim=-1)
    o = causal_softmax_attention(q, k, v, m["scale"], W["sink"] if rotary else None)
    o = _r(o.reshape(T, H * dv), round_to)
    if rotary:
        o = _r(o * torch.sigmoid(_r(hb @ W["g"].t(), round_to)), round_to)
    return o @ W["o"].t()


def dense_xielu(h: torch.Tensor, W: Dict[str, torch.Tensor], round_to=None) -> torch.Tensor:
    up = _r(_r(h, round_to) @ W["up"].t(), round_to)
    return _r(xielu(up, W["act"]), round_to) @ W["down"].t()


def token_side_input(x: torch.Tensor, ids: torch.Tensor, table: torch.Tensor, layer: int, dim: int,
                     W: Dict[str, torch.Tensor], eps: float, round_to=None) -> torch.Tensor:
    """e = table[token][layer*dim : (layer+1)*dim]; g = gelu_tanh(gate x) * e; y = proj g;
    x + y / rms(y) * norm."""
    e = table[ids][:, layer * dim:(layer + 1) * dim].to(F32)
    g = _r(gelu_tanh(_r(_r(x, round_to) @ W["gate"].t(), round_to)) * e, round_to)
    y = g @ W["proj"].t()
    return x + weighted_rms_norm(y, W["norm"], eps)


class PlainBepuzen:
    def __init__(self, model_dir: str, round_to: Optional[torch.dtype] = None):
        with open(os.path.join(model_dir, "config.json")) as f:
            self.cfg = json.load(f)
        self.w = {n: (t if t.dtype == torch.int32 else _r(t.to(F32), round_to))
                  for n, t in read_safetensors(os.path.join(model_dir, "model.safetensors")).items()}
        self.round_to = round_to

    def _sub(self, prefix: str) -> Dict[str, torch.Tensor]:
        return {n[len(prefix):]: t for n, t in self.w.items() if n.startswith(prefix)}

    def layer_outputs(self, ids: Sequence[int]) -> List[torch.Tensor]:
        """The residual stream after every layer, [T, D] each; the last entry's logits come from `logits`."""
        cfg, rt = self.cfg, self.round_to
        eps = cfg["norm"]["eps"]
        ids_t = torch.as_tensor(list(ids), dtype=torch.long)
        pos = torch.arange(len(ids))
        x = self.w["embed"][ids_t].to(F32)
        outs = []
        for i, L in enumerate(cfg["layers"]):
            p = f"l{i}."
            h = scalar_rms_norm(x, self.w[p + "norm1"], eps)
            y = latent_attention(h, self._sub(p + "mix."), L["mixer"], eps, pos, L["type"] == "latent_attention", rt)
            if L.get("mlp") is not None:
                y = y + dense_xielu(h, self._sub(p + "mlp."), rt)
            x = x + y
            side = cfg.get("token_side")
            if side is not None:
                x = token_side_input(x, ids_t, self.w["side.embed"], i, side["dim"], self._sub(p + "side."), eps, rt)
            outs.append(x)
        return outs

    def logits(self, ids: Sequence[int]) -> torch.Tensor:
        x = self.layer_outputs(ids)[-1]
        h = scalar_rms_norm(x, self.w["final.norm"], self.cfg["norm"]["eps"])
        return _r(h, self.round_to) @ self.w["head"].t()
