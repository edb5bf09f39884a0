"""Routed experts as a feed-forward: x += m sum_e w_e Wdown_e (silu(Wgate_e h) * (Wup_e h)) over a row's chosen experts.

The router (`ops.route_experts`, float32) gives every row a weight per expert, zero for the experts it does not use.
The experts then run as two products for all of them together: gate and up rows of all experts stacked into one
[2 x experts x ff, dim] matrix (with the SwiGLU epilogue of the tensor-core products in bfloat16), and the down matrices
laid side by side along k as one [dim, experts x ff] matrix, whose product adds into the residual stream. Between the
two, a row's hidden values of expert e are multiplied by its weight (and by the residual scale m): an expert the row
does not use contributes exact zeros, and the sum over experts is the product's own float32 accumulation. Every weight
streams once per step however the rows choose; what this costs against running only the chosen experts is experts / top
times the multiply-adds.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.loader import TensorWant
from .base import FeedForward, register_feed_forward
from .linear import Linear


class RoutedExperts(FeedForward):
    takes_residual_scale = True

    def __init__(self, spec, dim: int, tensors: dict, prefix: str, runtime):
        self.spec, self.dim, self.rt = spec, dim, runtime
        self.residual_scale = 1.0
        E, ff = spec.experts, spec.hidden
        self.hidden = E * ff
        gate = torch.cat([tensors.pop(f"{prefix}e{e}.gate") for e in range(E)], dim=0)
        up = torch.cat([tensors.pop(f"{prefix}e{e}.up") for e in range(E)], dim=0)
        self.fused = gate.dtype == torch.bfloat16 and dim % 8 == 0 and self.hidden % 8 == 0
        if self.fused:      # blocks of 8 gate rows followed by their 8 up rows: the product's epilogue applies SwiGLU
            stacked = torch.stack([gate.view(self.hidden // 8, 8, dim), up.view(self.hidden // 8, 8, dim)], dim=1)
            self.gate_up = Linear(stacked.reshape(2 * self.hidden, dim).contiguous())
            del stacked
        else:
            self.gate_up = Linear(torch.cat([gate, up], dim=0).contiguous())
        del gate, up
        self.down = Linear(torch.cat([tensors.pop(f"{prefix}e{e}.down") for e in range(E)], dim=1).contiguous())
        self.router = tensors.pop(prefix + "router")
        self.correction = tensors.pop(prefix + "correction") if spec.correction else None

    @classmethod
    def wants(cls, spec, dim: int, prefix: str) -> dict:
        out = {prefix + "router": TensorWant((spec.experts, dim), "matrix_fp32")}
        if spec.correction:
            out[prefix + "correction"] = TensorWant((spec.experts,), "vector")
        for e in range(spec.experts):
            out[f"{prefix}e{e}.gate"] = TensorWant((spec.hidden, dim))
            out[f"{prefix}e{e}.up"] = TensorWant((spec.hidden, dim))
            out[f"{prefix}e{e}.down"] = TensorWant((dim, spec.hidden))
        return out

    def forward(self, xb, x, batch) -> None:
        s, rows = self.spec, xb.shape[0]
        weights = self.rt.buffer("expert_weights", s.experts, torch.float32)[:rows]
        ops.route_experts(xb, self.router, self.correction, s.top, s.scale * self.residual_scale, s.normalize, weights)
        h = self.rt.buffer("experts_hidden", self.hidden)[:rows]
        if self.fused:
            self.gate_up.forward(xb, h, swiglu=True)
        else:
            gate_up = self.rt.buffer("experts_gate_up", 2 * self.hidden)[:rows]
            self.gate_up.forward(xb, gate_up)
            ops.swiglu(gate_up, h)
        ops.scale_expert_hidden(h, weights, s.hidden)
        self.down.forward(h, x, accumulate=True)


register_feed_forward("routed_experts", RoutedExperts, replace=True)
