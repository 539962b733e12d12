"""Grouped-query attention over the paged cache, as a mixer part.

Order of operations as in the reference (src/model/self_attention.cpp:122-169):
q/k/v projections -> per-head RMSNorm of q and k -> rotation -> cache write ->
causal attention over the cache (scale d^-0.5 after the dot, 32-bit softmax) ->
output projection.  The three projections run as one product over the row-wise
concatenation [Wq; Wk; Wv] made at bind time; norm, rotation and the cache write are
one kernel.  Head counts, head size, scale, window, norm and position encoding are
parameters; the part does not know its model.

Further parameters, none of which Qwen3 uses: biases on the q/k/v projections, values of
another size than keys (`value_dim`), scores capped smoothly (`softcap`: s <- c tanh(s / c)),
chunked attention (`chunk`: a query reads the keys of its own chunk of that many positions,
chunks counted from position 0 of the sequence), a sink (`sink`: the softmax's denominator has
one more term exp(0), which carries no value), an interleaved rotary encoding (the rows of the
q and k projections are reordered at load time so that the kernels' half-split rotation
applies), and the checkpoint names of the tensors (`names`).

Further still, for other designs: `keep_first` (with `window`): every query also sees the first so many keys of its
sequence, at their true positions; `out_bias`: a bias on the output projection; `conv_taps`: a short causal convolution
over time on every channel of q, k and v right after the projection, before the rotation (tensors `<q|k|v>` +
`conv_suffix`, [channels, taps]; the last taps - 1 projected rows of a sequence are part of its state);
`head_gate`: every head's output is multiplied by sigmoid(w_h . x), one number per token and head (tensor `head_gate`
[heads, hidden]); `value_mix`: values blended across layers: the layer that says "first" keeps the step's values
(after the bias) for the others, a layer that says "blend" goes on with v <- (1 - lambda) v + lambda v_first, lambda
its scalar tensor `value_mix`, and caches the blend (a "first" layer may store the scalar too; it is not read).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..cache.book import CacheNeed
from ..config.plan import PartSpec
from ..csrc import ops
from ..weights.loader import WeightSpec
from ..weights.upload import fuse_rows
from .base import Part, build_part, register_part
from .linear import linear

# Hand-written bfloat16 kernels register themselves here: fn(part, q, cache, out, ctx, table) -> bool
PREFILL_KERNELS = []
DECODE_KERNELS = []
# Kernels that take the projection output as it is and do norm, rotation, cache write and attention of a decode
# step in one launch: fn(part, qkv, cache, out, ctx, table, q_norm_w, k_norm_w, eps, cos, sin) -> bool
FUSED_DECODE_KERNELS = []
# Kernels that do the q/k/v product of a prompt step themselves, with norm, rotation and cache write in its
# epilogue: fn(part, x, cache, q, ctx, table, q_norm_w, k_norm_w, eps, cos, sin) -> bool (q is filled, the pages written)
FUSED_PROJECTION_KERNELS = []


TENSOR_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
                "q_bias": "q_proj.bias", "k_bias": "k_proj.bias", "v_bias": "v_proj.bias",
                "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", "o_bias": "o_proj.bias", "value_mix": "value_mix",
                "head_gate": "gate.weight", "conv_suffix": ".conv"}


class GQAAttention(Part):
    # what a part that builds on this one without its constructor still finds (the options beyond plain attention are off)
    out_name = "mixer.out"
    keep_first, out_bias, value_mix, conv_taps, head_gate = 0, False, None, 0, False
    o_bias = bias_v = conv_weight = w_gate = None
    mix_lambda = 0.0

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                 qk_norm: Optional[PartSpec] = None, position: Optional[PartSpec] = None,
                 window: Optional[int] = None, prefix: str = "", value_dim: Optional[int] = None, bias: bool = False,
                 softcap: Optional[float] = None, chunk: Optional[int] = None, sink: bool = False,
                 names: Optional[dict] = None, value_heads: Optional[int] = None, out_float32: bool = False,
                 keep_first: int = 0, out_bias: bool = False, value_mix: Optional[str] = None, conv_taps: int = 0,
                 head_gate: bool = False):
        self.sink_values = None      # float32 [num_heads]: the sink's score per head, for a part that has learned ones (else 0)
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        value_dim = int(value_dim or head_dim)
        if not 0 < head_dim <= 256 or not 0 < value_dim <= 256:
            raise ValueError(f"head_dim {head_dim} (values {value_dim}): the attention kernels take sizes up to 256 "
                             f"(the tensor-core kernels: multiples of 16)")
        if window and chunk:
            raise ValueError("attention takes a window or chunks, not both")
        if value_mix not in (None, "first", "blend") or keep_first < 0 or conv_taps < 0 or (keep_first and not window):
            raise ValueError("attention: value_mix is 'first' or 'blend'; keep_first goes with a window")
        self.keep_first, self.out_bias, self.value_mix = int(keep_first), bool(out_bias), value_mix
        self.conv_taps, self.head_gate = int(conv_taps), bool(head_gate)
        self.out_name = "mixer.out"  # the scratch buffer of the result; a part that runs several mixers side by side renames it
        self.o_bias = self.bias_v = self.conv_weight = self.w_gate = None
        self.mix_lambda = 0.0
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        self.scale, self.window, self.prefix = float(scale), window, prefix
        self.value_dim, self.has_bias, self.sink = value_dim, bool(bias), bool(sink)
        # values that several key heads share (`value_heads` < num_kv_heads), and an output that stays in 32-bit for
        # a part that goes on with it (`out_float32`): the general kernel and the `capped` tensor-core kernels take both
        self.value_heads = int(value_heads or num_kv_heads)
        if num_kv_heads % self.value_heads:
            raise ValueError("num_kv_heads must be a multiple of value_heads")
        self.out_float32 = bool(out_float32)
        self.shared_values = self.value_heads != num_kv_heads or self.out_float32
        self.softcap = float(softcap) if softcap else 0.0
        self.chunk = int(chunk) if chunk else None
        self.names = dict(TENSOR_NAMES, **(names or {}))
        self.q_norm = build_part("norm", qk_norm) if qk_norm else None
        self.k_norm = build_part("norm", qk_norm) if qk_norm else None
        self.position = build_part("position", position) if position else None
        self.w_qkv = self.w_o = self.bias = None
        self.reordered = False       # the rows of the q and k projections follow the position encoding's kernel order
        # what the kernels written for Qwen3's attention take
        self.plain = not (self.has_bias or self.softcap or self.chunk or self.sink or value_dim != head_dim or head_dim % 16
                          or self.shared_values or self.keep_first or self.value_mix)

    # -- weights
    def weight_specs(self, prefix: str) -> dict:
        p, n = prefix + self.prefix, self.names
        nq, nkv, d, vd, H, nv = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim, self.hidden_size, self.value_heads
        specs = {p + n["q"]: WeightSpec((nq * d, H)), p + n["k"]: WeightSpec((nkv * d, H)),
                 p + n["v"]: WeightSpec((nv * vd, H)), p + n["o"]: WeightSpec((H, self.output_width()))}
        if self.has_bias:
            specs.update({p + n["q_bias"]: WeightSpec((nq * d,), "bias"), p + n["k_bias"]: WeightSpec((nkv * d,), "bias"),
                          p + n["v_bias"]: WeightSpec((nv * vd,), "bias")})
        if self.q_norm is not None:
            specs.update(self.q_norm.weight_specs(p + n["q_norm"]))
            specs.update(self.k_norm.weight_specs(p + n["k_norm"]))
        if self.out_bias:
            specs[p + n["o_bias"]] = WeightSpec((H,), "bias")
        if self.value_mix:
            specs[p + n["value_mix"]] = WeightSpec((), "bias")
        if self.head_gate:
            specs[p + n["head_gate"]] = WeightSpec((nq, H))
        if self.conv_taps:
            for which, rows in (("q", nq * d), ("k", nkv * d), ("v", nv * vd)):
                specs[p + n[which] + n["conv_suffix"]] = WeightSpec((rows, self.conv_taps), "bias")
        return specs

    def output_width(self) -> int:
        """Columns of the output projection: what the attention hands to it per token."""
        return self.num_heads * self.value_dim

    def bind(self, weights: dict, prefix: str, dtype, device) -> None:
        p, n = prefix + self.prefix, self.names
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        self.w_qkv = fuse_rows(weights, [p + n["q"], p + n["k"], p + n["v"]])
        self.w_o = weights.pop(p + n["o"]).contiguous()
        if self.has_bias:
            tensors = [weights[p + n[k]] for k in ("q_bias", "k_bias", "v_bias")]
            getattr(weights, "wait", lambda: None)()          # a streamed checkpoint: the tensors are in place now
            self.bias = torch.cat([t.to(device=device, dtype=torch.float32).reshape(-1) for t in tensors]).contiguous()
        f32 = dict(device=device, dtype=torch.float32)
        if self.out_bias:
            self.o_bias = weights[p + n["o_bias"]].to(**f32).contiguous()
        if self.head_gate:
            self.w_gate = weights.pop(p + n["head_gate"]).contiguous()
        if self.conv_taps:
            taps = [weights[p + n[which] + n["conv_suffix"]] for which in ("q", "k", "v")]
            getattr(weights, "wait", lambda: None)()
            self.conv_weight = torch.cat([t.to(**f32) for t in taps], dim=0).contiguous()
        if self.value_mix:
            lam = weights[p + n["value_mix"]]
            getattr(weights, "wait", lambda: None)()
            self.mix_lambda = float(lam.to(torch.float32).reshape(-1)[0].item()) if self.value_mix == "blend" else 0.0
            if self.bias is not None:          # the values' bias is added where they are blended, before the cache write
                v0 = (nq + nkv) * d
                self.bias_v = self.bias[v0:].clone()
                self.bias[v0:] = 0.0
        order = self.position.kernel_order() if self.position is not None and hasattr(self.position, "kernel_order") else None
        if order is not None:
            # q.k does not change when the values of every query and key head are reordered alike: put the pairs
            # of the rotation where the kernels expect them, once
            if self.q_norm is not None:
                raise ValueError("an interleaved rotation with per-head norm weights is not supported")
            getattr(weights, "wait", lambda: None)()
            rows = (torch.arange(nq + nkv, device=self.w_qkv.device)[:, None] * d
                    + torch.tensor(order, device=self.w_qkv.device)[None, :]).reshape(-1)
            self.w_qkv[:rows.numel()] = self.w_qkv[:rows.numel()][rows]
            if self.bias is not None:
                self.bias[:rows.numel()] = self.bias[:rows.numel()][rows]
            if self.conv_weight is not None:
                self.conv_weight[:rows.numel()] = self.conv_weight[:rows.numel()][rows]
            self.reordered = True
        if self.conv_weight is not None:
            self.conv_weight = self.conv_weight.t().contiguous()        # [taps, channels], as the kernel reads it
        if self.q_norm is not None:
            self.q_norm.bind(weights, p + n["q_norm"], dtype, device)
            self.k_norm.bind(weights, p + n["k_norm"], dtype, device)

    # -- cache
    def cache_need(self) -> CacheNeed:
        kind = "window" if self.window else ("chunk" if self.chunk else "full")
        state = ((self.conv_taps - 1) * self.projection_width(),) if self.conv_taps > 1 else ()
        return CacheNeed(kind, self.num_kv_heads, self.head_dim, self.window or self.chunk,
                         value_dim=self.value_dim if self.value_dim != self.head_dim else None,
                         value_heads=self.value_heads if self.value_heads != self.num_kv_heads else None,
                         keep_first=self.keep_first if self.window else 0, state_shape=state)

    def projection_width(self) -> int:
        """Columns of the q/k/v projection."""
        return (self.num_heads + self.num_kv_heads) * self.head_dim + self.value_heads * self.value_dim

    # -- step
    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        out = ctx.scratch.get(self.out_name, (ctx.n_tokens, self.hidden_size), ctx.dtype)
        attn = self.mix(x, ctx, cache)
        if self.head_gate:
            gate = ctx.scratch.get("attn.head_gate", (ctx.n_tokens, self.num_heads), ctx.dtype)
            ops.head_gate(attn, linear(x, self.w_gate, gate), self.num_heads, self.value_dim)
        linear(attn, self.w_o, out)
        return ops.add_bias(out, self.o_bias) if self.out_bias else out

    def mix(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        """Everything before the output projection: [N, num_heads * value_dim] in the compute type (float32 with
        `out_float32`)."""
        nq, nkv, d, vd = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim
        N = ctx.n_tokens
        table = ctx.page_tables[cache.group]
        attn = ctx.scratch.get("attn.ctx", (N, nq * vd), torch.float32 if self.out_float32 else ctx.dtype)
        norm_eps = self.q_norm.eps if self.q_norm is not None else 0.0
        qw = self.q_norm.weight if self.q_norm is not None else None
        kw = self.k_norm.weight if self.k_norm is not None else None
        tables = self.position is None or getattr(self.position, "fused_tables", False)
        cos = sin = None
        if tables and self.position is not None:
            self.position.prepare(ctx.max_positions, ctx.device)
            cos, sin = self.position.cos, self.position.sin
        special = ctx.dtype == torch.bfloat16
        if tables and not ctx.is_decode and special and not self.conv_taps and not self.value_mix:
            q = ctx.scratch.get("attn.q", (N, nq * d), ctx.dtype)
            for kernel in FUSED_PROJECTION_KERNELS:
                if kernel(self, x, cache, q, ctx, table, qw, kw, norm_eps, cos, sin):
                    self.attend(q, cache, attn, ctx, table)
                    return attn
        qkv = ctx.scratch.get("attn.qkv", (N, self.projection_width()), ctx.dtype)
        if self.conv_taps:
            raw = ctx.scratch.get("attn.qkv_raw", (N, self.projection_width()), ctx.dtype)
            linear(x, self.w_qkv, raw)
            if self.conv_taps > 1 and cache.state is None:
                raise ops.KernelError("the short convolution keeps rows per sequence: the cache was built without its state")
            # one tap carries no rows from step to step: the kernel then gets rows of no values
            state = cache.state.view(cache.state.shape[0], -1) if cache.state is not None else ctx.scratch.get("attn.no_state", (1, 0), torch.float32)
            ops.short_conv(raw, self.conv_weight, state, ctx.token_seq, ctx.seq_start, ctx.seq_slots, qkv, ctx.n_seqs)
        else:
            linear(x, self.w_qkv, qkv)
        if self.value_mix:
            width = self.value_heads * vd
            first = ctx.scratch.get("attn.v_first", (N, width), ctx.dtype)      # one buffer for the step: layers run in order
            ops.value_mix(qkv, (nq + nkv) * d, width, self.bias_v, first, self.value_mix == "first", self.mix_lambda)
        if tables and ctx.is_decode and special:
            for kernel in FUSED_DECODE_KERNELS:
                if kernel(self, qkv, cache, attn, ctx, table, qw, kw, norm_eps, cos, sin):
                    return attn
        q = ctx.scratch.get("attn.q", (N, nq * d), ctx.dtype)
        if tables:
            ops.qkv_prepare(qkv, q, cache.keys, cache.values, qw, kw, cos, sin, ctx.token_seq, ctx.token_pos, table,
                            N, nq, nkv, d, norm_eps, write_kv=not cache.shared, bias=self.bias, value_dim=vd,
                            value_heads=self.value_heads)
        else:
            self._prepare_unfused(qkv, q, cache, ctx, table, qw, kw, norm_eps)
        self.attend(q, cache, attn, ctx, table)
        return attn

    def attend(self, q, cache, out, ctx, table) -> None:
        if ctx.dtype == torch.bfloat16:
            for kernel in (DECODE_KERNELS if ctx.is_decode else PREFILL_KERNELS):
                if kernel(self, q, cache, out, ctx, table):
                    return
        ops.attention_generic(q, cache.keys, cache.values, out, ctx.token_seq, ctx.token_pos, table, ctx.n_tokens,
                              self.num_heads, self.num_kv_heads, self.head_dim, self.scale, self.window,
                              value_dim=self.value_dim, softcap=self.softcap, chunk=self.chunk, sink=self.sink,
                              value_heads=self.value_heads, sink_values=self.sink_values, keep_first=self.keep_first)

    def _prepare_unfused(self, qkv, q, cache, ctx, table, qw, kw, eps) -> None:
        """A position encoding without kernel tables: norm, then `apply_`, then the cache write."""
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        N = ctx.n_tokens
        if self.bias is not None:
            qkv = (qkv.float() + self.bias).to(qkv.dtype)
        qs = qkv[:, :nq * d].contiguous().view(N, nq, d)
        ks = qkv[:, nq * d:(nq + nkv) * d].contiguous().view(N, nkv, d)
        if qw is not None:                                  # into buffers of their own: the norm kernel's input and
            qn, kn = torch.empty_like(qs), torch.empty_like(ks)   # output may not be the same memory
            ops.rms_norm(qs, qw, eps, qn)
            ops.rms_norm(ks, kw, eps, kn)
            qs, ks = qn, kn
        self.position.prepare(ctx.max_positions, ctx.device)
        if self.reordered:
            self.position.apply_(qs, ks, ctx.token_pos[:N], kernel_order=True)
        else:
            self.position.apply_(qs, ks, ctx.token_pos[:N])
        packed = torch.cat([qs.view(N, -1), ks.view(N, -1), qkv[:, (nq + nkv) * d:]], dim=1).contiguous()
        ops.qkv_prepare(packed, q, cache.keys, cache.values, None, None, None, None, ctx.token_seq, ctx.token_pos,
                        table, N, nq, nkv, d, 0.0, write_kv=not cache.shared, value_dim=self.value_dim)


def _decode_split_kernel(part, q, cache, out, ctx, table) -> bool:
    """The split-key tensor-core decode kernel: bfloat16, groups of up to 16 query heads."""
    if not part.plain:
        return False
    nq, nkv, d = part.num_heads, part.num_kv_heads, part.head_dim
    if nq // nkv > 16:
        return False
    splits = ops.attention_decode_splits(ctx.n_tokens, nkv, _sm_count(ctx.device))
    scratch = ctx.scratch.get("attn.decode_scratch", (ctx.n_tokens * nq * splits * (d + 2),), torch.float32)
    ops.attention_decode(q, cache.keys, cache.values, out, scratch, ctx.token_seq, ctx.token_pos, table, ctx.n_tokens,
                         nq, nkv, d, part.scale, part.window, splits)
    return True


def _decode_fused_kernel(part, qkv, cache, out, ctx, table, q_norm_w, k_norm_w, eps, cos, sin) -> bool:
    """Norm, rotation, cache write, split-key attention and the merge of the splits (inside a thread-block
    cluster) in one launch: bfloat16, groups of up to 16 query heads, up to 16 splits."""
    if not part.plain:
        return False
    nq, nkv, d = part.num_heads, part.num_kv_heads, part.head_dim
    if nq // nkv > 16:
        return False
    splits = ops.attention_decode_splits(ctx.n_tokens, nkv, _sm_count(ctx.device))
    if splits > 8:
        # more than eight blocks per (sequence, kv head) - a cluster beyond the portable size - pay for one or two
        # sequences with long contexts only (one sequence of 32,768 keys: 39.6 us with 16 splits against 53.8 with 8;
        # two: 54.7 with 12 against 64.8; at 2,048 keys 11.8 against 11.1)
        wide = min(splits, max(8, wide_cluster_blocks // (ctx.n_tokens * nkv)), ops.attention_decode_fused_max_splits(d, ctx.device))
        splits = wide if ctx.max_context > long_context_keys else 8
    ops.attention_decode_fused(qkv, cache.keys, cache.values, out, q_norm_w, k_norm_w, cos, sin, eps, ctx.token_seq,
                               ctx.token_pos, table, ctx.n_tokens, nq, nkv, d, part.scale, part.window, splits,
                               write_kv=not cache.shared)
    return True


def _projection_pair_kernel(part, x, cache, q, ctx, table, q_norm_w, k_norm_w, eps, cos, sin) -> bool:
    """The q/k/v product on pairs of SMs with norm, rotation and the cache write in its epilogue, where `linear`
    would take the persistent pairs kernel anyway: head sizes 64, 128 and 256, the whole head rotated."""
    if not part.plain:
        return False
    from . import linear as linear_module
    nq, nkv, d = part.num_heads, part.num_kv_heads, part.head_dim
    N, K = ctx.n_tokens, part.hidden_size
    if d not in ops.PAIR_QKV_HEAD_DIMS or K % 8 != 0 or N < fused_projection_rows:
        return False
    if cos is not None and 2 * cos.shape[-1] != d:
        return False
    if linear_module.set_bf16_kernel_active() or linear_module.tcgen05_form(N, (nq + 2 * nkv) * d, K) != "pair" \
            or linear_module.pair_plan(N, (nq + 2 * nkv) * d, K)[1] != 1:
        return False
    ops.gemm_tcgen05_pair_qkv(x, part.w_qkv, q, cache.keys, cache.values, q_norm_w, k_norm_w, cos, sin, eps, ctx.token_seq,
                              ctx.token_pos, table, N, nq, nkv, d, write_kv=not cache.shared)
    return True


_sm_counts = {}


def _sm_count(device) -> int:
    device = torch.device(device)
    count = _sm_counts.get(device)
    if count is None:
        count = _sm_counts[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return count


def _prefill_flash_kernel(part, q, cache, out, ctx, table) -> bool:
    """The tiled tensor-core kernel for steps that bring prompts (or any mix of lengths)."""
    if not part.plain:
        return False
    ops.attention_prefill(q, cache.keys, cache.values, out, ctx.seq_start, ctx.seq_pos0, table, ctx.n_seqs,
                          ctx.max_new, part.num_heads, part.num_kv_heads, part.head_dim, part.scale, part.window)
    return True


def _prefill_tcgen05_kernel(part, q, cache, out, ctx, table) -> bool:
    """Both products of the attention on tcgen05 with TMA-fed tiles: head sizes 64 and 128, no window,
    and enough new tokens for 128-row tiles to be worth it."""
    if not part.plain:
        return False
    if not ops.attention_prefill_tc_fits(part.head_dim, part.window) or ctx.max_new < tc_prefill_rows or part.scale <= 0:
        return False
    ops.attention_prefill_tc(q[:ctx.n_tokens], cache.keys, cache.values, out, ctx.seq_start, ctx.seq_pos0, table,
                             ctx.n_seqs, ctx.max_new, ctx.n_tokens, part.num_heads, part.num_kv_heads, part.head_dim,
                             part.scale)
    return True


def _prefill_capped_kernel(part, q, cache, out, ctx, table) -> bool:
    """Capped scores, chunks, a sink, values of their own size: the tiled tensor-core kernel for those."""
    if part.plain or not ops.attention_capped_fits(part.head_dim, part.value_dim, part.window, 1):
        return False
    ops.attention_capped_prefill(q, cache.keys, cache.values, out, ctx.seq_start, ctx.seq_pos0, table, ctx.n_seqs, ctx.max_new,
                                 part.num_heads, part.num_kv_heads, part.head_dim, part.value_dim, part.scale, part.softcap,
                                 part.chunk, part.sink, window=part.window, value_heads=part.value_heads,
                                 sink_values=part.sink_values, keep_first=part.keep_first)
    return True


def _prefill_capped_tcgen05_kernel(part, q, cache, out, ctx, table) -> bool:
    """The same on tcgen05 with TMA-fed tiles: head sizes 64 and 128, values as wide as keys, and enough new tokens
    for 128-row tiles to be worth it."""
    if part.plain or part.keep_first or part.shared_values or not ops.attention_capped_prefill_tc_fits(part.head_dim, part.value_dim, part.window) \
            or ctx.max_new < tc_prefill_rows or part.scale <= 0 or part.sink_values is not None:
        return False
    ops.attention_capped_prefill_tc(q[:ctx.n_tokens], cache.keys, cache.values, out, ctx.seq_start, ctx.seq_pos0, table,
                                    ctx.n_seqs, ctx.max_new, ctx.n_tokens, part.num_heads, part.num_kv_heads, part.head_dim,
                                    part.scale, part.softcap, part.chunk, part.sink)
    return True


def _decode_capped_kernel(part, q, cache, out, ctx, table) -> bool:
    """The same for decode steps: split over the keys of the chunk (or of the whole context), merged with the sink."""
    nq, nkv = part.num_heads, part.num_kv_heads
    if part.plain or not ops.attention_capped_fits(part.head_dim, part.value_dim, part.window, nq // nkv):
        return False
    splits = ops.attention_capped_splits(ctx.n_tokens, nkv, _sm_count(ctx.device),
                                         min(part.chunk or (part.window or 0) + part.keep_first or ctx.max_context, ctx.max_context))
    scratch = ctx.scratch.get("attn.capped_scratch", (ctx.n_tokens * nq * splits * (part.value_dim + 2),), torch.float32)
    ops.attention_capped_decode(q, cache.keys, cache.values, out, scratch, ctx.token_seq, ctx.token_pos, table, ctx.n_tokens,
                                nq, nkv, part.head_dim, part.value_dim, part.scale, part.softcap, part.chunk, part.sink, splits,
                                window=part.window, value_heads=part.value_heads, sink_values=part.sink_values,
                                keep_first=part.keep_first)
    return True


def _decode_capped_fused_kernel(part, qkv, cache, out, ctx, table, q_norm_w, k_norm_w, eps, cos, sin) -> bool:
    """Bias, rotation, cache write and the split-key attention of a decode step in one kernel (and the small merge)."""
    nq, nkv = part.num_heads, part.num_kv_heads
    if part.plain or part.shared_values or part.window or q_norm_w is not None or cache.shared or part.sink_values is not None \
            or not ops.attention_capped_fits(part.head_dim, part.value_dim, part.window, nq // nkv):
        return False
    splits = ops.attention_capped_splits(ctx.n_tokens, nkv, _sm_count(ctx.device), part.chunk or ctx.max_context)
    scratch = ctx.scratch.get("attn.capped_scratch", (ctx.n_tokens * nq * splits * (part.value_dim + 2),), torch.float32)
    ops.attention_capped_decode_fused(qkv, cache.keys, cache.values, out, scratch, part.bias, cos, sin, ctx.token_seq,
                                      ctx.token_pos, table, ctx.n_tokens, nq, nkv, part.head_dim, part.value_dim, part.scale,
                                      part.softcap, part.chunk, part.sink, splits)
    return True


long_context_keys = 4096  # a decode step whose sequences may be longer takes wider clusters (if they are few)
wide_cluster_blocks = 200 # blocks of a decode step with clusters beyond the portable size
tc_prefill_rows = 128     # from this many new tokens of the longest sequence on, the tcgen05 kernel runs
# From this many tokens in a step on, the q/k/v product does norm, rotation and cache write in its epilogue: with
# several tiles per pair of SMs the longer epilogue hides under the next tile's K steps (measured: 8,192 tokens
# 321-338 us against 381-412 for product + qkv_prepare, 2,048 tokens 83.5 against 86, 512 tokens 41 against 34).
fused_projection_rows = 2048

DECODE_KERNELS.append(_decode_split_kernel)
FUSED_DECODE_KERNELS.append(_decode_fused_kernel)
FUSED_DECODE_KERNELS.append(_decode_capped_fused_kernel)
FUSED_PROJECTION_KERNELS.append(_projection_pair_kernel)
PREFILL_KERNELS.append(_prefill_tcgen05_kernel)
PREFILL_KERNELS.append(_prefill_flash_kernel)
PREFILL_KERNELS.append(_prefill_capped_tcgen05_kernel)
PREFILL_KERNELS.append(_prefill_capped_kernel)
DECODE_KERNELS.append(_decode_capped_kernel)

register_part("mixer", "gqa_attention", GQAAttention)
