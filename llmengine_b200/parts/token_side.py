"""A per-layer input that depends on the token alone, gated by the residual stream."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..engine.plan import Plan
from .base import Part, Runtime, WeightSpec, register_part, register_category


register_category("token_side")


@register_part("token_side", "token_side_input")
class TokenSideInput(Part):
    """With e = table[token][offset : offset + dim] (a slice of a per-token table that the model stores once for
    all layers): g = gelu_tanh(W_gate x) * e, y = W_proj g, x += y / sqrt(mean(y^2) + eps) * norm.  It reads the
    residual stream itself, not a normed copy, so the contributions of the layer's sublayers are added first; the
    part takes them (`a`, `b`) and does that addition too."""

    def __init__(self, rt: Runtime, prefix: str, hidden_size: int, dim: int, offset: int, table_width: int,
                 vocab_size: int, eps: float, table: str):
        super().__init__(rt, prefix)
        self.hidden, self.dim, self.offset, self.eps = int(hidden_size), int(dim), int(offset), float(eps)
        self.table_width, self.vocab, self.table_name = int(table_width), int(vocab_size), table
        if self.offset + self.dim > self.table_width:
            raise ValueError(f"{prefix}: columns {self.offset}..{self.offset + self.dim} lie outside a table of {self.table_width}")
        self.w_gate = self.w_proj = self.gain = self.table = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {
            self.name("gate"): WeightSpec((self.dim, self.hidden)),
            self.name("proj"): WeightSpec((self.hidden, self.dim)),
            self.name("norm"): WeightSpec((self.hidden,), role="vector", init="gain"),
        }

    def load_weights(self, t: Dict[str, torch.Tensor]) -> None:
        self.w_gate = t[self.name("gate")].contiguous()
        self.w_proj = t[self.name("proj")].contiguous()
        self.gain = t[self.name("norm")].contiguous()

    def tied_tensors(self) -> Dict[str, str]:
        return {self.name("table"): self.table_name}

    def receive_tied(self, tensors: Dict[str, torch.Tensor]) -> None:
        table = tensors[self.name("table")]
        if tuple(table.shape) != (self.vocab, self.table_width):
            raise ValueError(f"{self.prefix}: the table {self.table_name!r} is {tuple(table.shape)}, expected "
                             f"{(self.vocab, self.table_width)}")
        self.table = table

    def emit(self, plan: Plan, x: torch.Tensor, a: torch.Tensor, b: Optional[torch.Tensor]) -> None:
        rt = self.rt
        plan.token_side(x=x, a=a, b=b, table=self.table, offset=self.offset, dim=self.dim, w_gate=self.w_gate,
                        w_proj=self.w_proj, gain=self.gain, eps=self.eps,
                        xb=rt.workspace("side_x", self.hidden, rt.dtype), g=rt.workspace("side_g", self.dim, rt.dtype),
                        y=rt.workspace("side_y", self.hidden, torch.float32))
