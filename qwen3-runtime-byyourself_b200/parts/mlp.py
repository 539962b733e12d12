"""Gated feed-forward as a part: down( act(gate(x)) * up(x) ), act = SiLU (SwiGLU, Qwen3) or the tanh form of GELU.

Reference: src/model/mlp.cpp:101-115 (three products and one elementwise kernel) and
src/ops/elementwise.cu:47-65.  Here gate and up run as one product over one matrix made
at bind time, their rows interleaved in blocks of eight; for the few rows of a decode
step the product's kernel applies SiLU and the gating itself.  The activation and the
checkpoint names of the three matrices are parameters.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from ..weights.loader import WeightSpec
from ..weights.upload import fuse_interleaved, fuse_rows
from .base import Part, register_part
from . import linear as linear_module
from .linear import linear


TENSOR_NAMES = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}


class SwiGLU(Part):
    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str = "", activation: str = "silu",
                 names: Optional[dict] = None, limit: float = float("inf"), alpha: float = 1.702):
        """`activation="clamped"`: down( g sigmoid(alpha g) (u + 1) ) with g = min(gate, limit), u = clamp(up, -limit, limit),
        the form of the routed experts (parts/moe.py) as a dense feed-forward."""
        if activation not in ops.ACTIVATIONS and activation != "clamped":
            raise ValueError(f"activation {activation!r}: 'clamped' or one of {sorted(ops.ACTIVATIONS)}")
        self.hidden_size, self.intermediate_size, self.prefix = int(hidden_size), int(intermediate_size), prefix
        self.activation, self.limit, self.alpha = activation, float(limit), float(alpha)
        self.names = dict(TENSOR_NAMES, **(names or {}))
        self.w_gate_up = self.w_down = None

    def weight_specs(self, prefix: str) -> dict:
        p, H, I, n = prefix + self.prefix, self.hidden_size, self.intermediate_size, self.names
        return {p + n["gate"]: WeightSpec((I, H)), p + n["up"]: WeightSpec((I, H)), p + n["down"]: WeightSpec((H, I))}

    def bind(self, weights: dict, prefix: str, dtype, device) -> None:
        p = prefix + self.prefix
        gate, up = p + self.names["gate"], p + self.names["up"]
        # gate and up rows interleaved in blocks of eight: one product gives both, and a kernel that owns
        # 16 consecutive output rows can finish silu(g) * u itself
        self.interleaved = self.intermediate_size % 8 == 0
        self.w_gate_up = fuse_interleaved(weights, gate, up, 8) if self.interleaved else fuse_rows(weights, [gate, up])
        self.w_down = weights.pop(p + self.names["down"]).contiguous()

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        N, I = ctx.n_tokens, self.intermediate_size
        act = ctx.scratch.get("ff.act", (N, I), ctx.dtype)
        fused = self.interleaved and ctx.dtype == torch.bfloat16 and self.hidden_size % 8 == 0 and self.activation != "clamped"
        if fused and N <= linear_module.skinny_rows:
            ops.gemm_skinny_gated(x, self.w_gate_up, act, self.activation)   # product, activation and gating in one kernel
        elif fused and linear_module.tcgen05_form(N, 2 * I, self.hidden_size, gated=True) == "weights_first":
            ops.gemm_tcgen05_mid_gated(x, self.w_gate_up, act, activation=self.activation)   # gating where the cluster's partial tiles meet
        elif fused:
            ops.gemm_tcgen05_pair(x, self.w_gate_up, act, gated=True,  # the gating runs in the product's epilogue
                                  splits=linear_module.pair_plan(N, 2 * I, self.hidden_size)[1], activation=self.activation)
        else:
            gate_up = ctx.scratch.get("ff.gate_up", (N, 2 * I), ctx.dtype)
            linear(x, self.w_gate_up, gate_up)
            if self.activation == "clamped":
                ops.clamped_mul(gate_up, act, self.limit, self.alpha, self.interleaved)
            else:
                ops.silu_mul(gate_up, act, self.interleaved, self.activation)
        out = ctx.scratch.get("ff.out", (N, self.hidden_size), ctx.dtype)
        return linear(act, self.w_down, out)


class DenseMLP(Part):
    """A feed-forward without a gate: down( act(up(x)) ); act one of `ops.PLAIN_ACTIVATIONS` (GELU with the error
    function by default).  The checkpoint names of the two matrices are parameters."""

    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str = "", activation: str = "gelu",
                 names: Optional[dict] = None):
        if activation not in ops.PLAIN_ACTIVATIONS:
            raise ValueError(f"activation {activation!r}: one of {sorted(ops.PLAIN_ACTIVATIONS)}")
        self.hidden_size, self.intermediate_size, self.prefix = int(hidden_size), int(intermediate_size), prefix
        self.activation = activation
        self.names = dict({"up": "up_proj.weight", "down": "down_proj.weight"}, **(names or {}))
        self.w_up = self.w_down = None

    def weight_specs(self, prefix: str) -> dict:
        p, H, I, n = prefix + self.prefix, self.hidden_size, self.intermediate_size, self.names
        return {p + n["up"]: WeightSpec((I, H)), p + n["down"]: WeightSpec((H, I))}

    def bind(self, weights: dict, prefix: str, dtype, device) -> None:
        p = prefix + self.prefix
        self.w_up = weights.pop(p + self.names["up"]).contiguous()
        self.w_down = weights.pop(p + self.names["down"]).contiguous()

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        N = ctx.n_tokens
        act = ctx.scratch.get("ff.act", (N, self.intermediate_size), ctx.dtype)
        linear(x, self.w_up, act)
        ops.activation(act, act, self.activation)
        out = ctx.scratch.get("ff.out", (N, self.hidden_size), ctx.dtype)
        return linear(act, self.w_down, out)


register_part("feed_forward", "dense_mlp", DenseMLP)
register_part("feed_forward", "swiglu", SwiGLU)
register_part("feed_forward", "gated_mlp", SwiGLU)
