"""Attention whose keys and values are expanded from a small latent per token, as a mixer part.

Per token the input is projected down to `rank + rot_dim` values: the first `rank`, brought to unit rms and multiplied
by a weight, are the latent c; the last `rot_dim` are one key part that is rotated by the token's position and that
all heads share.  A head's key is [W_uk c | rotated part] (`head_dim` + `rot_dim` values), its value W_uv c
(`value_dim` values), its query [plain | rotated]; the score is their dot product times `scale`.  Only c and the
rotated part are cached: one cache row of rank + rot_dim values per token and layer, as keys, and c once more as values.

The expansion never runs.  W_uk is absorbed into the query (q~ = W_uk^T q_plain, `rank` values per head) and W_uv is
applied to the attention's output, so that the attention itself is multi-query attention of `num_heads` query heads of
size rank + rot_dim over one key head (the cache rows) with values of size rank; it runs on the kernels of
`GQAAttention` (general, and the tiled tensor-core ones where the sizes fit).

Options: `q_rank` (the queries go through a latent of their own: a down projection, unit rms times a weight, an up
projection; else one projection), `window` (position i sees j with 0 <= i - j < window), `sink` (one learned score per
head in the softmax's denominator, without key or value, not scaled), `gate` (the heads' outputs are multiplied by the
sigmoid of one more projection of the input), `rot_dims` <= rot_dim (how much of the rotated part really turns),
`interleaved` (pairs (2i, 2i + 1), else (i, i + rot_dims / 2)), `theta`.  All projections of the input run as one
product; norms, rotation, scores, softmax and the products per head accumulate in 32-bit whatever the compute type.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..cache.book import CacheNeed
from ..config.plan import PartSpec
from ..csrc import ops
from ..weights.loader import WeightSpec
from ..weights.upload import fuse_rows
from .attention import GQAAttention
from .base import build_part, register_part
from .linear import linear

TENSOR_NAMES = {"q": "q", "q_down": "dq", "q_norm": "dq.norm", "q_up": "uq", "kv_down": "dkv", "kv_norm": "dkv.norm",
                "k_up": "uk", "v_up": "uv", "sink": "sink", "gate": "g", "o": "o"}
MAX_KEY_ROW, MAX_VALUE_ROW = 1024, 512       # what the general attention kernel takes as one cache row


class LatentAttention(GQAAttention):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, value_dim: int, kv_rank: int,
                 scale: float, eps: float, theta: float, max_positions: int, rot_dims: Optional[int] = None,
                 interleaved: bool = False, q_rank: Optional[int] = None, window: Optional[int] = None, sink: bool = False,
                 gate: bool = False, prefix: str = "", names: Optional[dict] = None):
        rot_dims = int(rot_dim if rot_dims is None else rot_dims)
        if min(num_heads, head_dim, value_dim, kv_rank) <= 0 or rot_dim < 0 or rot_dims % 2 or not 0 <= rot_dims <= rot_dim:
            raise ValueError("latent attention: positive sizes, an even number of rotated values within rot_dim")
        if kv_rank + rot_dim > MAX_KEY_ROW or kv_rank > MAX_VALUE_ROW:
            raise ValueError(f"latent attention: a cache row of up to {MAX_KEY_ROW} values with a latent of up to {MAX_VALUE_ROW}")
        self.hidden_size, self.heads, self.plain_dim, self.rot_dim = int(hidden_size), int(num_heads), int(head_dim), int(rot_dim)
        self.out_dim, self.rank, self.rot_dims = int(value_dim), int(kv_rank), rot_dims
        self.q_rank = int(q_rank) if q_rank else None
        self.eps, self.prefix, self.interleaved, self.gated = float(eps), prefix, bool(interleaved), bool(gate)
        self.names = dict(TENSOR_NAMES, **(names or {}))
        # what the attention kernels see: multi-query attention over the cache rows
        self.num_heads, self.num_kv_heads, self.value_heads = self.heads, 1, 1
        self.head_dim, self.value_dim = self.rank + self.rot_dim, self.rank
        self.scale, self.window, self.sink = float(scale), (int(window) if window else None), bool(sink)
        self.softcap, self.chunk, self.has_bias, self.bias = 0.0, None, False, None
        self.out_float32 = self.shared_values = self.plain = False
        self.sink_values = None
        self.q_norm = self.k_norm = None
        self.position = build_part("position", PartSpec("rope", {
            "head_dim": max(self.rot_dim, 2), "theta": float(theta), "max_positions": int(max_positions),
            "rotary_dim": max(rot_dims, 2), "interleaved": self.interleaved, "theta_float32": False})) if rot_dims else None
        self.w_in = self.w_q_up = self.w_k_up = self.w_v_up = self.w_o = self.c_norm = self.cq_norm = None
        self.q_off = self.kv_off = self.gate_off = 0

    # -- weights
    def _input_rows(self):
        """(name, rows) of the projections of the input, in the order in which they are fused."""
        n, H = self.names, self.heads
        first = (n["q_down"], self.q_rank) if self.q_rank else (n["q"], H * (self.plain_dim + self.rot_dim))
        rows = [first, (n["kv_down"], self.rank + self.rot_dim)]
        if self.gated:
            rows.append((n["gate"], H * self.out_dim))
        return rows

    def weight_specs(self, prefix: str) -> dict:
        p, n, H, W = prefix + self.prefix, self.names, self.heads, self.hidden_size
        specs = {p + name: WeightSpec((rows, W)) for name, rows in self._input_rows()}
        if self.q_rank:
            specs[p + n["q_norm"]] = WeightSpec((self.q_rank,), "norm")
            specs[p + n["q_up"]] = WeightSpec((H * (self.plain_dim + self.rot_dim), self.q_rank))
        specs[p + n["kv_norm"]] = WeightSpec((self.rank,), "norm")
        specs[p + n["k_up"]] = WeightSpec((H * self.plain_dim, self.rank))
        specs[p + n["v_up"]] = WeightSpec((H * self.out_dim, self.rank))
        if self.sink:
            specs[p + n["sink"]] = WeightSpec((H,), "bias")
        specs[p + n["o"]] = WeightSpec((W, H * self.out_dim))
        return specs

    def bind(self, weights: dict, prefix: str, dtype, device) -> None:
        p, n, H = prefix + self.prefix, self.names, self.heads
        rows = self._input_rows()
        self.w_in = fuse_rows(weights, [p + name for name, _ in rows])
        self.q_off, self.kv_off = 0, rows[0][1]
        self.gate_off = rows[0][1] + rows[1][1]
        f32 = dict(device=device, dtype=torch.float32)
        if self.q_rank:
            self.w_q_up = weights.pop(p + n["q_up"]).contiguous()
            self.cq_norm = weights[p + n["q_norm"]].to(**f32).contiguous()
        self.c_norm = weights[p + n["kv_norm"]].to(**f32).contiguous()
        k_up, v_up = weights.pop(p + n["k_up"]), weights.pop(p + n["v_up"])
        getattr(weights, "wait", lambda: None)()              # a streamed checkpoint: the tensors are in place now
        # per head [inner, outer] for `head_product`: W_uk as stored ([plain_dim, rank]: the absorption contracts the
        # head's plain values), W_uv transposed ([rank, value_dim]: the expansion contracts the latent)
        self.w_k_up = k_up.reshape(H, self.plain_dim, self.rank).contiguous()
        self.w_v_up = v_up.reshape(H, self.out_dim, self.rank).transpose(1, 2).contiguous()
        if self.sink:
            self.sink_values = weights[p + n["sink"]].to(**f32).contiguous()
        self.w_o = weights.pop(p + n["o"]).contiguous()

    def output_width(self) -> int:
        return self.heads * self.out_dim

    # -- cache
    def cache_need(self) -> CacheNeed:
        return CacheNeed("window" if self.window else "full", 1, self.rank + self.rot_dim, self.window, value_dim=self.rank)

    # -- step
    def mix(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        N, H, d, r, rank, vd = ctx.n_tokens, self.heads, self.plain_dim, self.rot_dim, self.rank, self.out_dim
        table = ctx.page_tables[cache.group]
        cos = sin = None
        if self.position is not None:
            self.position.prepare(ctx.max_positions, ctx.device)
            cos, sin = self.position.cos, self.position.sin
        proj = ctx.scratch.get("latent.proj", (N, self.w_in.shape[0]), ctx.dtype)
        linear(x, self.w_in, proj)
        cq = ctx.scratch.get("latent.cq", (N, self.q_rank), ctx.dtype) if self.q_rank else None
        ops.latent_prepare(proj, self.kv_off, self.q_off, self.c_norm, self.cq_norm, cq, cache.keys, cache.values, cos, sin,
                           ctx.token_seq, ctx.token_pos, table, N, rank, r, self.rot_dims, self.interleaved, self.eps,
                           write_kv=not cache.shared)
        if self.q_rank:
            q = ctx.scratch.get("latent.q", (N, H * (d + r)), ctx.dtype)
            linear(cq, self.w_q_up, q)
        else:
            q = proj[:, :H * (d + r)]
        q_full = ctx.scratch.get("attn.q", (N, H * (rank + r)), ctx.dtype)
        ops.head_product(q, d + r, 0, self.w_k_up, q_full, rank + r, 0, N)
        ops.latent_queries(q, q_full, cos, sin, ctx.token_pos, N, H, d, rank, r, self.rot_dims, self.interleaved)
        mixed = ctx.scratch.get("attn.ctx", (N, H * rank), ctx.dtype)
        self.attend(q_full, cache, mixed, ctx, table)
        heads_out = ctx.scratch.get("latent.heads", (N, H * vd), ctx.dtype)
        gate = proj[:, self.gate_off:self.gate_off + H * vd] if self.gated else None
        return ops.head_product(mixed, rank, 0, self.w_v_up, heads_out, vd, 0, N, gate=gate)


register_part("mixer", "latent_attention", LatentAttention)
