"""Feed-forward parts."""
from __future__ import annotations

from typing import Dict

import torch

from ..engine.plan import Plan
from .base import Part, Runtime, WeightSpec, register_part, run_alone


@register_part("feed_forward", "swiglu")
class SwiGLU(Part):
    """down( silu(gate(h)) * up(h) ), no biases; silu(g) = g / (1 + exp(-g))
    (src/model/transformer_graph_builder.cpp:261-274; src/runtime/kernels/cpu_kernels.cpp:848-859).
    The gate and up matrices are stored as one [gate | up] matrix so that one product serves both; where a
    kernel carries the activation in its epilogue the [T, 2 * intermediate] product never exists in memory."""

    def __init__(self, rt: Runtime, prefix: str, hidden_size: int, intermediate_size: int):
        super().__init__(rt, prefix)
        self.hidden, self.inter = int(hidden_size), int(intermediate_size)
        self.w_gate_up = self.w_down = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {
            self.name("gate_proj.weight"): WeightSpec((self.inter, self.hidden)),
            self.name("up_proj.weight"): WeightSpec((self.inter, self.hidden)),
            self.name("down_proj.weight"): WeightSpec((self.hidden, self.inter)),
        }

    def load_weights(self, t: Dict[str, torch.Tensor]) -> None:
        self.w_gate_up = torch.cat([t[self.name("gate_proj.weight")], t[self.name("up_proj.weight")]], 0).contiguous()
        self.w_down = t[self.name("down_proj.weight")].contiguous()

    def emit(self, plan: Plan, h: torch.Tensor) -> torch.Tensor:
        rt = self.rt
        act = rt.workspace("act", self.inter, rt.dtype)
        gate_up = rt.workspace("gate_up", 2 * self.inter, rt.dtype)
        plan.linear_swiglu(h, self.w_gate_up, gate_up, act)
        delta = rt.workspace("ffn_out", self.hidden, torch.float32)
        plan.linear(act, self.w_down, delta)
        return delta

    def forward(self, h: torch.Tensor, batch=None) -> torch.Tensor:
        from ..engine.batch import StepBatch
        plan = Plan()
        delta = self.emit(plan, h)
        run_alone(self.rt, plan, batch if batch is not None else StepBatch.bare(h.shape[0], h.device))
        return delta[: h.shape[0]]


def _softplus32(v: torch.Tensor) -> float:
    v = v.detach().to("cpu", torch.float32)
    return float(torch.log1p(torch.exp(-v.abs())) + torch.clamp(v, min=0))


@register_part("feed_forward", "dense_xielu")
class DenseXIELU(Part):
    """down( act(up(h)) ), no biases, with the activation xIELU and its two learned numbers (p, q):
    z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2.
    The two coefficients are formed once in 32-bit when the weights are loaded and travel as constants."""

    def __init__(self, rt: Runtime, prefix: str, hidden_size: int, intermediate_size: int):
        super().__init__(rt, prefix)
        self.hidden, self.inter = int(hidden_size), int(intermediate_size)
        self.w_up = self.w_down = None
        self.a_pos = self.a_neg = 0.0

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {
            self.name("up"): WeightSpec((self.inter, self.hidden)),
            self.name("down"): WeightSpec((self.hidden, self.inter)),
            self.name("act"): WeightSpec((2,), role="vector", init="unit"),
        }

    def load_weights(self, t: Dict[str, torch.Tensor]) -> None:
        self.w_up = t[self.name("up")].contiguous()
        self.w_down = t[self.name("down")].contiguous()
        pq = t[self.name("act")]
        self.a_pos = _softplus32(pq[0])
        self.a_neg = float(torch.tensor(0.5, dtype=torch.float32) + torch.tensor(_softplus32(pq[1]), dtype=torch.float32))

    def emit(self, plan: Plan, h: torch.Tensor) -> torch.Tensor:
        rt = self.rt
        up = rt.workspace("ffn_up", self.inter, rt.dtype)
        act = rt.workspace("act", self.inter, rt.dtype)
        plan.linear_act(h, self.w_up, up, act, "xielu", (self.a_pos, self.a_neg))
        delta = rt.workspace("ffn_out", self.hidden, torch.float32)
        plan.linear(act, self.w_down, delta)
        return delta

    def forward(self, h: torch.Tensor, batch=None) -> torch.Tensor:
        from ..engine.batch import StepBatch
        plan = Plan()
        delta = self.emit(plan, h)
        run_alone(self.rt, plan, batch if batch is not None else StepBatch.bare(h.shape[0], h.device))
        return delta[: h.shape[0]]
