"""A matrix memory with exponential gates (the mLSTM cell of xLSTM) as a mixer part.

q = W_q x * dim^(-1/2) and k = W_k x (heads x dim), v = W_v x (heads x vdim); per head a log input gate
i = cap tanh((w_i . x + b_i) / cap) and a log forget gate f = logsigmoid(cap tanh((w_f . x + b_f) / cap)).  With a running
maximum m that starts at 0, a matrix S [dim, vdim] and a normaliser n [dim] that start at zero:

    m_t = max(f_t + m_(t-1), i_t)
    S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T,      n_t likewise with k_t alone
    o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + floor)

Every head's o is brought to unit rms over its vdim values; the heads side by side are multiplied by a weight vector
and by sigmoid(W_g x) and projected by W_o.  q, k, v and the output gate run as one product; the two gates' logits
leave their product in 32-bit, and gates, maximum, state and norm are 32-bit whatever the compute type.  The state
lives in the cache's state rows: per sequence heads x dim x (vdim + 1) values (the normaliser is a last column of S
whose value is 1 for every token), then one m per head.  No keys in the cache.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..cache.book import CacheNeed
from ..csrc import ops
from ..weights.loader import WeightSpec
from ..weights.upload import fuse_rows
from .base import Part, register_part
from .linear import linear

TENSOR_NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "i": "i", "f": "f", "i_bias": "i.b", "f_bias": "f.b"}


class MatrixMemory(Part):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, gate_cap: float, eps: float,
                 floor: float = 1e-6, prefix: str = "", names: Optional[dict] = None):
        if not 0 < head_dim <= 256 or not 0 < value_dim < 256 or num_heads <= 0 or not gate_cap > 0:
            raise ValueError("matrix memory: key size up to 256, value size up to 255, a positive gate cap")
        self.hidden_size, self.num_heads, self.head_dim, self.value_dim = int(hidden_size), int(num_heads), int(head_dim), int(value_dim)
        self.gate_cap, self.eps, self.floor, self.prefix = float(gate_cap), float(eps), float(floor), prefix
        self.names = dict(TENSOR_NAMES, **(names or {}))
        self.out_name = "mixer.out"
        self.w_in = self.w_gates = self.w_o = self.norm_weight = self.bias_i = self.bias_f = None

    def weight_specs(self, prefix: str) -> dict:
        p, n, H, h = prefix + self.prefix, self.names, self.hidden_size, self.num_heads
        qk, vg = h * self.head_dim, h * self.value_dim
        return {p + n["q"]: WeightSpec((qk, H)), p + n["k"]: WeightSpec((qk, H)), p + n["v"]: WeightSpec((vg, H)),
                p + n["g"]: WeightSpec((vg, H)), p + n["o"]: WeightSpec((H, vg)), p + n["norm"]: WeightSpec((vg,), "norm"),
                p + n["i"]: WeightSpec((h, H)), p + n["f"]: WeightSpec((h, H)),
                p + n["i_bias"]: WeightSpec((h,), "bias"), p + n["f_bias"]: WeightSpec((h,), "bias")}

    def bind(self, weights: dict, prefix: str, dtype, device) -> None:
        p, n = prefix + self.prefix, self.names
        self.w_in = fuse_rows(weights, [p + n[k] for k in ("q", "k", "v", "g")])
        self.w_gates = fuse_rows(weights, [p + n["i"], p + n["f"]])
        self.w_o = weights.pop(p + n["o"]).contiguous()
        f32 = dict(device=device, dtype=torch.float32)
        self.norm_weight = weights[p + n["norm"]].to(**f32).contiguous()
        self.bias_i = weights[p + n["i_bias"]].to(**f32).contiguous()
        self.bias_f = weights[p + n["f_bias"]].to(**f32).contiguous()

    def state_size(self) -> int:
        return self.num_heads * self.head_dim * (self.value_dim + 1) + self.num_heads

    def cache_need(self) -> CacheNeed:
        return CacheNeed("none", state_shape=(self.state_size(),))

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        N, h, d, vd = ctx.n_tokens, self.num_heads, self.head_dim, self.value_dim
        proj = ctx.scratch.get("memory.proj", (N, 2 * h * (d + vd)), ctx.dtype)
        linear(x, self.w_in, proj)
        z = ctx.scratch.get("memory.z", (N, 2 * h), torch.float32)
        linear(x, self.w_gates, z)
        state = cache.state.view(cache.state.shape[0], -1)
        cells = h * d * (vd + 1)
        keep, write, low = (ctx.scratch.get("memory." + name, (N, h), torch.float32) for name in ("keep", "write", "low"))
        ops.memory_gates(z, self.bias_i, self.bias_f, self.gate_cap, state[:, cells:cells + h], ctx.seq_start, ctx.seq_slots, keep,
                         write, low, ctx.n_seqs, h)
        o = ctx.scratch.get("memory.o", (N, h * (vd + 1)), torch.float32)
        ops.decay_scan(proj[:, :h * d], proj[:, h * d:2 * h * d], proj[:, 2 * h * d:2 * h * d + h * vd], state[:, :cells], ctx.seq_start,
                       ctx.seq_slots, o, ctx.n_seqs, h, d, vd, q_scale=d ** -0.5, keep=keep, write=write, ones=True)
        gated = ctx.scratch.get("memory.gated", (N, h * vd), ctx.dtype)
        ops.head_gated_norm(o, self.norm_weight, proj[:, 2 * h * d + h * vd:], self.eps, gated, h, vd, act="sigmoid", low=low,
                            floor=self.floor)
        out = ctx.scratch.get(self.out_name, (N, self.hidden_size), ctx.dtype)
        return linear(gated, self.w_o, out)


register_part("mixer", "matrix_memory", MatrixMemory)
