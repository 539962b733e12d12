"""Linear attention whose forget gate also decides what is written (HGRN2), as a mixer part.

q = SiLU(W_q x) (heads x dim), v = W_v x (heads x vdim); the forget gate per head and channel is bounded from below,
f = low + (1 - low) * sigmoid(W_f x + b) with `low` a stored vector; per head a state S [dim, vdim] that lives in
float32 in the cache's state rows (zero for a new sequence, carried from step to step):

    S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T,     o_t = S_t^T q_t      (no key, no other scale)

Every head's o is brought to unit rms over its vdim values and multiplied by one weight vector that the heads share;
the heads side by side are projected by W_o.  The three input projections run as one product; gate, recurrence
and norm are 32-bit whatever the compute type.  The part needs no keys in the cache:
`CacheNeed("none", state_shape=(heads, dim, vdim))`.
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

TENSOR_NAMES = {"q": "q", "f": "f", "f_bias": "f.b", "lower": "lower", "v": "v", "norm": "norm", "o": "o"}


class GatedRecurrence(Part):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, eps: float, prefix: str = "",
                 names: Optional[dict] = None):
        if not 0 < head_dim <= 256 or not 0 < value_dim <= 256 or num_heads <= 0:
            raise ValueError("gated recurrence: head sizes up to 256")
        self.hidden_size, self.num_heads, self.head_dim, self.value_dim = int(hidden_size), int(num_heads), int(head_dim), int(value_dim)
        self.eps, self.prefix = float(eps), prefix
        self.names = dict(TENSOR_NAMES, **(names or {}))
        self.w_in = self.w_o = self.norm_weight = self.low = self.bias = None

    def weight_specs(self, prefix: str) -> dict:
        p, n, H = prefix + self.prefix, self.names, self.hidden_size
        qf, vv = self.num_heads * self.head_dim, self.num_heads * self.value_dim
        return {p + n["q"]: WeightSpec((qf, H)), p + n["f"]: WeightSpec((qf, H)), p + n["v"]: WeightSpec((vv, H)),
                p + n["f_bias"]: WeightSpec((qf,), "bias"), p + n["lower"]: WeightSpec((qf,), "bias"),
                p + n["norm"]: WeightSpec((self.value_dim,), "norm"), p + n["o"]: WeightSpec((H, vv))}

    def bind(self, weights: dict, prefix: str, dtype, device) -> None:
        p, n = prefix + self.prefix, self.names
        self.w_in = fuse_rows(weights, [p + n[k] for k in ("q", "f", "v")])
        self.w_o = weights.pop(p + n["o"]).contiguous()
        f32 = dict(device=device, dtype=torch.float32)
        self.norm_weight = weights[p + n["norm"]].to(**f32).contiguous()
        self.low = weights[p + n["lower"]].to(**f32).contiguous()
        self.bias = weights[p + n["f_bias"]].to(**f32).contiguous()

    def cache_need(self) -> CacheNeed:
        return CacheNeed("none", state_shape=(self.num_heads, self.head_dim, self.value_dim))

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        N, h, d, vd = ctx.n_tokens, self.num_heads, self.head_dim, self.value_dim
        proj = ctx.scratch.get("recurrence.proj", (N, h * (2 * d + vd)), ctx.dtype)
        linear(x, self.w_in, proj)
        o = ctx.scratch.get("recurrence.o", (N, h * vd), torch.float32)
        ops.gated_scan(proj, cache.state, self.low, self.bias, ctx.seq_start, ctx.seq_slots, o, ctx.n_seqs, h, d, vd)
        normed = ctx.scratch.get("recurrence.normed", (N, h * vd), ctx.dtype)
        ops.head_rms_norm(o, self.norm_weight, self.eps, normed, vd)
        out = ctx.scratch.get("mixer.out", (N, self.hidden_size), ctx.dtype)
        return linear(normed, self.w_o, out)


register_part("mixer", "gated_recurrence", GatedRecurrence)
