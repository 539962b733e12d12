"""Gated linear attention as a mixer part: linear attention with keys and a decay per key channel.

q = W_q x * dim^(-1/2) and k = W_k x (heads x dim), v = W_v x (heads x vdim); the decay comes through a narrow
projection, z = W_a2 (W_a1 x) + b (heads x dim), alpha = sigmoid(z)^(1/tau); per head a state S [dim, vdim] that lives
in float32 in the cache's state rows (zero for a new sequence, carried from step to step):

    S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,     o_t = S_t^T q_t

Every head's o is brought to unit rms over its vdim values, multiplied by one weight vector that the heads share and
by SiLU(W_g x); the heads side by side are projected by W_o.  q, k, v and the output gate run as one product; the decay
logits leave their product in 32-bit, and decay, recurrence and norm are 32-bit whatever the compute type.  The part
needs no keys in the cache: `CacheNeed("none", state_shape=(heads * dim * vdim,))`.
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

TENSOR_NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "a1": "a1", "a2": "a2", "a2_bias": "a2.b"}


class GatedLinearAttention(Part):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, tau: float, eps: float, prefix: str = "",
                 names: Optional[dict] = None, decay_rank: Optional[int] = None):
        """`decay_rank`: the width of the narrow projection; None: read from the tensor's shape when the weights arrive."""
        if not 0 < head_dim <= 256 or not 0 < value_dim <= 256 or num_heads <= 0 or not tau > 0:
            raise ValueError("gated linear attention: head sizes up to 256, a positive tau")
        self.hidden_size, self.num_heads, self.head_dim, self.value_dim = int(hidden_size), int(num_heads), int(head_dim), int(value_dim)
        self.tau, self.eps, self.prefix, self.decay_rank = float(tau), float(eps), prefix, decay_rank
        self.names = dict(TENSOR_NAMES, **(names or {}))
        self.out_name = "mixer.out"
        self.w_in = self.w_a1 = self.w_a2 = self.w_o = self.norm_weight = self.decay_bias = None

    def weight_specs(self, prefix: str) -> dict:
        p, n, H = prefix + self.prefix, self.names, self.hidden_size
        qk, vg = self.num_heads * self.head_dim, self.num_heads * self.value_dim
        rank = self.decay_rank if self.decay_rank else -1          # -1: any size (the two tensors have to agree)
        return {p + n["q"]: WeightSpec((qk, H)), p + n["k"]: WeightSpec((qk, H)), p + n["v"]: WeightSpec((vg, H)),
                p + n["g"]: WeightSpec((vg, H)), p + n["o"]: WeightSpec((H, vg)), p + n["norm"]: WeightSpec((self.value_dim,), "norm"),
                p + n["a1"]: WeightSpec((rank, H)), p + n["a2"]: WeightSpec((qk, rank)), p + n["a2_bias"]: WeightSpec((qk,), "bias")}

    def bind(self, weights: dict, prefix: str, dtype, device) -> None:
        p, n = prefix + self.prefix, self.names
        self.w_in = fuse_rows(weights, [p + n[k] for k in ("q", "k", "v", "g")])
        self.w_a1 = weights.pop(p + n["a1"]).contiguous()
        self.w_a2 = weights.pop(p + n["a2"]).contiguous()
        if self.w_a1.shape[0] != self.w_a2.shape[1]:
            raise ValueError(f"{p}: the two decay projections do not fit each other")
        self.w_o = weights.pop(p + n["o"]).contiguous()
        f32 = dict(device=device, dtype=torch.float32)
        self.norm_weight = weights[p + n["norm"]].to(**f32).contiguous()
        self.decay_bias = weights[p + n["a2_bias"]].to(**f32).contiguous()

    def cache_need(self) -> CacheNeed:
        return CacheNeed("none", state_shape=(self.num_heads * self.head_dim * self.value_dim,))

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        N, h, d, vd = ctx.n_tokens, self.num_heads, self.head_dim, self.value_dim
        proj = ctx.scratch.get("gla.proj", (N, 2 * h * (d + vd)), ctx.dtype)
        linear(x, self.w_in, proj)
        narrow = ctx.scratch.get("gla.narrow", (N, self.w_a1.shape[0]), ctx.dtype)
        linear(x, self.w_a1, narrow)
        z = ctx.scratch.get("gla.z", (N, h * d), torch.float32)
        linear(narrow, self.w_a2, z)
        ops.channel_decay(z, self.decay_bias, self.tau)          # once per token and channel: every block of the scan reads it
        o = ctx.scratch.get("gla.o", (N, h * vd), torch.float32)
        state = cache.state.view(cache.state.shape[0], -1)
        ops.decay_scan(proj[:, :h * d], proj[:, h * d:2 * h * d], proj[:, 2 * h * d:2 * h * d + h * vd], state, ctx.seq_start,
                       ctx.seq_slots, o, ctx.n_seqs, h, d, vd, q_scale=d ** -0.5, decay=z)
        gated = ctx.scratch.get("gla.gated", (N, h * vd), ctx.dtype)
        ops.head_gated_norm(o, self.norm_weight, proj[:, 2 * h * d + h * vd:], self.eps, gated, h, vd, act="silu")
        out = ctx.scratch.get(self.out_name, (N, self.hidden_size), ctx.dtype)
        return linear(gated, self.w_o, out)


register_part("mixer", "gated_linear_attention", GatedLinearAttention)
