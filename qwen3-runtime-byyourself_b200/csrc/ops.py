"""Python face of the CUDA entry points: tensors in, launches on torch's current stream.

Each function checks what the kernel relies on (device, dtype, contiguity, sizes),
passes raw pointers to the `extern "C"` entry point and raises `KernelError` if the
launch reports an error.  Nothing here computes on the host and nothing falls back
to a library: a CPU tensor or a missing compiler is an error.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_int64, c_uint64, c_void_p
from typing import Optional

import torch

from ..cache.book import PAGE_TOKENS
from .build import load_library

_ERRORS = {10001: "a size the kernel does not take", 10002: "more rows than one launch takes",
           10003: "a pointer or stride that is not 16-byte aligned"}
_SUFFIX = {torch.float32: "f32", torch.bfloat16: "bf16"}
_fn_cache = {}


class KernelError(RuntimeError):
    """A kernel refused its arguments or its launch failed."""


# Programmatic dependent launch: a kernel launched with it may start (set up its barriers and tensor memory, fetch
# weights) while the kernel before it on the stream drains, and waits for that kernel's results only where it
# first needs them.  By default the sources named here launch their kernels that way: measured on whole decode
# steps of an 8B-sized model, the TMA + tcgen05 products gain 2.5-5 % at batches of 16 to 64 (4.92 -> 4.74 ms a
# step at batch 16), while the few-row product loses (batch 8: chains of waiting blocks take the room that a kernel's
# own later waves need) and the decode attention, which asks for its first pages before it waits, gains 0.5 % at batch
# 16 and 32 and loses 0.3 % at batch 64.  QWEN3_B200_PDL=1 / =0 turns it on / off for all.
PDL_SOURCES = ("gemm_tcgen05.cu",)
_pdl_override = {"1": True, "0": False}.get(os.environ.get("QWEN3_B200_PDL", ""))
_libs = {}


def _pdl_for(source: str) -> bool:
    return _pdl_override if _pdl_override is not None else source in PDL_SOURCES


def set_pdl(on) -> None:
    """Programmatic dependent launch for every kernel of the library (True / False), or back to the default
    (None): on for the sources in `PDL_SOURCES` only."""
    global _pdl_override
    _pdl_override = None if on is None else bool(on)
    for (source, _), lib in _libs.items():
        lib.q3_set_pdl(int(_pdl_for(source)))


class KernelTimer:
    """Times every launch of this library with a pair of CUDA events while it is active:

        with ops.KernelTimer() as timer:
            engine.step(...)
        timer.summary()  ->  {entry point: (launches, total microseconds)}

    For steps that are launched afresh (a captured step is one replay and shows nothing).  The events add a
    few microseconds of host work per launch, so the step as a whole runs slower than untimed; the
    durations are those of the kernels."""

    def __init__(self):
        self.records = []

    def __enter__(self):
        global _timer
        self._before, _timer = _timer, self
        return self

    def __exit__(self, *exc):
        global _timer
        _timer = self._before
        return False

    def run(self, name, fn, args):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        stream = torch.cuda.ExternalStream(_stream()) if _stream() else torch.cuda.current_stream()
        start.record(stream)
        code = fn(*args)
        stop.record(stream)
        self.records.append((name, start, stop))
        return code

    def summary(self) -> dict:
        torch.cuda.synchronize()
        out = {}
        for name, start, stop in self.records:
            n, us = out.get(name, (0, 0.0))
            out[name] = (n + 1, us + start.elapsed_time(stop) * 1e3)
        return out


_timer: Optional[KernelTimer] = None


def _fn(source: str, name: str, argtypes, defines=()):
    fn = _fn_untimed(source, name, argtypes, defines)
    if _timer is None:
        return fn
    timer = _timer
    return lambda *args: timer.run(name, fn, args)


def _fn_untimed(source: str, name: str, argtypes, defines=()):
    key = (source, name, tuple(defines))
    fn = _fn_cache.get(key)
    if fn is None:
        lib = load_library(source, defines)
        if (source, tuple(defines)) not in _libs:
            _libs[(source, tuple(defines))] = lib
            lib.q3_set_pdl.argtypes = [c_int]
            lib.q3_set_pdl.restype = None
            lib.q3_set_pdl(int(_pdl_for(source)))
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int
        _fn_cache[key] = fn
    return fn


_launches = 0


def launch_count() -> int:
    """How many kernels of this library have been launched (or captured into a graph) so far."""
    return _launches


def _count_extra(n: int) -> None:
    """Entry points that launch more than one kernel add the rest here."""
    global _launches
    _launches += n


def _check(code: int, name: str):
    global _launches
    _launches += 1
    if code != 0:
        what = _ERRORS.get(code)
        if what is None:
            what = f"CUDA error {code} at launch"
        raise KernelError(f"{name}: {what}")


_pinned_stream: Optional[int] = None


def _stream() -> int:
    return _pinned_stream if _pinned_stream is not None else torch.cuda.current_stream().cuda_stream


class on_current_stream:
    """Within this scope every launch goes to the stream that is current on entry, looked up once
    (asking torch for the current stream costs more than a launch)."""

    def __enter__(self):
        global _pinned_stream
        self._before = _pinned_stream
        _pinned_stream = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _pinned_stream
        _pinned_stream = self._before
        return False


def _dev(t: torch.Tensor, name: str, dtype=None):
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    return t.data_ptr()


def _suffix(t: torch.Tensor) -> str:
    try:
        return _SUFFIX[t.dtype]
    except KeyError:
        raise KernelError(f"element type {t.dtype} is not supported (float32 or bfloat16)") from None


def _ptr(t: Optional[torch.Tensor], name: str, dtype=None):
    return None if t is None else _dev(t, name, dtype)


# ------------------------------------------------------------------ elementwise
def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t] = table[ids[t]]; ids int32 [N], table [V, H], out [N, H]."""
    s = _suffix(table)
    fn = _fn("elementwise.cu", f"q3_embedding_{s}", [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p])
    n = ids.numel()
    if out.shape[0] < n or out.shape[1] != table.shape[1] or out.dtype != table.dtype:
        raise KernelError("embedding: output does not fit")
    _check(fn(_dev(ids, "ids", torch.int32), _dev(table, "table"), _dev(out, "out"), n, table.shape[1],
              table.shape[0], _stream()), "embedding")
    return out


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
             delta: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = RMSNorm(x) * weight over the last dimension; weight is float32.

    With `delta`, first x += delta in place (32-bit sum, stored in x's type) and the
    norm reads the stored sum.  x: [..., size] with contiguous rows."""
    s = _suffix(x)
    size = x.shape[-1]
    rows = x.numel() // size if size else 0
    if weight.numel() != size or out.shape != x.shape or out.dtype != x.dtype:
        raise KernelError("rms_norm: weight or output does not fit")
    if delta is not None and (delta.shape != x.shape or delta.dtype != x.dtype):
        raise KernelError("rms_norm: delta does not fit")
    if out.data_ptr() == x.data_ptr():
        raise KernelError("rms_norm: the output may not be the input's own memory")
    fn = _fn("elementwise.cu", f"q3_rms_norm_{s}",
             [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_float, c_int64, c_int64, c_void_p])
    _check(fn(_dev(x, "x"), _ptr(delta, "delta"), _dev(weight, "weight", torch.float32), _dev(out, "out"),
              rows, size, float(eps), size, size, _stream()), "rms_norm")
    return out


ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False, activation: str = "silu") -> torch.Tensor:
    """out[r, c] = act(gate[r, c]) * up[r, c], act = SiLU or (`activation="gelu_tanh"`) the tanh form of GELU; a row
    of `gate_up` holds the gate in its first half and the up values in its second, or (`interleaved`) blocks of
    eight gate columns each followed by the eight up columns of the same features."""
    s = _suffix(gate_up)
    rows, two_i = gate_up.shape
    if two_i % 2 or out.shape != (rows, two_i // 2) or out.dtype != gate_up.dtype:
        raise KernelError("silu_mul: output does not fit")
    fn = _fn("elementwise.cu", f"q3_act_mul_{s}", [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p])
    _check(fn(_dev(gate_up, "gate_up"), _dev(out, "out"), rows, two_i // 2, int(bool(interleaved)),
              ACTIVATIONS[activation], _stream()), "silu_mul")
    return out


def clamped_mul(gate_up: torch.Tensor, out: torch.Tensor, limit: float, alpha: float, interleaved: bool = False) -> torch.Tensor:
    """out[r, c] = g sigmoid(alpha g) (u + 1) with g = min(gate[r, c], limit), u = clamp(up[r, c], -limit, limit); `gate_up`
    laid out as for `silu_mul`."""
    s = _suffix(gate_up)
    rows, two_i = gate_up.shape
    if two_i % 2 or out.shape != (rows, two_i // 2) or out.dtype != gate_up.dtype:
        raise KernelError("clamped_mul: output does not fit")
    fn = _fn("elementwise.cu", f"q3_clamped_mul_{s}", [c_void_p, c_void_p, c_int64, c_int, c_int, c_float, c_float, c_void_p])
    _check(fn(_dev(gate_up, "gate_up"), _dev(out, "out"), rows, two_i // 2, int(bool(interleaved)), float(limit), float(alpha),
              _stream()), "clamped_mul")
    return out


def scaled_sum(a: torch.Tensor, b: torch.Tensor, scale_a: float, scale_b: float, out: torch.Tensor) -> torch.Tensor:
    """out = scale_a * a + scale_b * b elementwise, in 32-bit, stored in the tensors' type (`out` may be `a` or `b`)."""
    if a.shape != b.shape or out.shape != a.shape or a.dtype != b.dtype or out.dtype != a.dtype:
        raise KernelError("scaled_sum: shapes do not fit")
    fn = _fn("elementwise.cu", f"q3_scaled_sum_{_suffix(a)}", [c_void_p, c_void_p, c_float, c_float, c_void_p, c_int64, c_void_p])
    _check(fn(_dev(a, "a"), _dev(b, "b"), float(scale_a), float(scale_b), _dev(out, "out"), a.numel(), _stream()), "scaled_sum")
    return out


def add_bias(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x[r, c] += bias[c] in place (32-bit sum, stored in x's type); bias float32."""
    if bias.numel() != x.shape[-1]:
        raise KernelError("add_bias: one value per column")
    fn = _fn("elementwise.cu", f"q3_add_bias_{_suffix(x)}", [c_void_p, c_void_p, c_int64, c_int, c_void_p])
    _check(fn(_dev(x, "x"), _dev(bias, "bias", torch.float32), x.numel() // x.shape[-1], x.shape[-1], _stream()), "add_bias")
    return x


def gather_rows(x: torch.Tensor, idx: torch.Tensor, out: torch.Tensor, delta: Optional[torch.Tensor] = None):
    """out[r] = x[idx[r]] (+ delta[idx[r]], summed in 32-bit)."""
    s = _suffix(x)
    rows, size = idx.numel(), x.shape[-1]
    if out.shape[0] < rows or out.shape[-1] != size or out.dtype != x.dtype:
        raise KernelError("gather_rows: output does not fit")
    fn = _fn("elementwise.cu", f"q3_gather_rows_{s}", [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p])
    _check(fn(_dev(x, "x"), _ptr(delta, "delta", x.dtype), _dev(idx, "idx", torch.int32), _dev(out, "out"),
              rows, size, _stream()), "gather_rows")
    return out


def place_rows(src: torch.Tensor, dst: torch.Tensor, block_rows: int = 0, dst_block_stride: int = 0, dst_row0: int = 0):
    """Rows of `src` [rows, cols] into `dst` [*, cols], converted to dst's type on the way: source row r goes to
    row dst_row0 + (r // block_rows) * dst_block_stride + r % block_rows (block_rows 0: one block, consecutive
    rows from dst_row0).  Load time: the q, k and v matrices into one, gate and up rows interleaved."""
    kinds = {torch.float32: 0, torch.bfloat16: 1}
    if src.dtype not in kinds or dst.dtype not in kinds:
        raise KernelError("place_rows: float32 or bfloat16 on either side")
    rows, cols = src.shape
    block = int(block_rows) or rows
    stride = int(dst_block_stride) or block
    if dst.shape[-1] != cols or rows % block != 0:
        raise KernelError("place_rows: shapes do not fit")
    last = dst_row0 + (rows // block - 1) * stride + block if rows else 0
    if last > dst.shape[0]:
        raise KernelError("place_rows: the rows do not fit the destination")
    fn = _fn("elementwise.cu", "q3_place_rows", [c_void_p, c_int, c_void_p, c_int] + [c_int64] * 5 + [c_void_p])
    _check(fn(_dev(src, "src"), kinds[src.dtype], _dev(dst, "dst"), kinds[dst.dtype], rows, cols, block, stride, int(dst_row0),
              _stream()), "place_rows")
    return dst


# ------------------------------------------------------------------ a hidden state kept in 32-bit (stream_f32.cu)
def embedding_scaled(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float) -> torch.Tensor:
    """out[t] = table[ids[t]] * scale as float32, whatever the table's type."""
    s = _suffix(table)
    n = ids.numel()
    if out.shape[0] < n or out.shape[1] != table.shape[1] or out.dtype != torch.float32:
        raise KernelError("embedding_scaled: output does not fit")
    fn = _fn("stream_f32.cu", f"q3_embedding_scaled_{s}", [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_float, c_void_p])
    _check(fn(_dev(ids, "ids", torch.int32), _dev(table, "table"), _dev(out, "out"), n, table.shape[1], table.shape[0],
              float(scale), _stream()), "embedding_scaled")
    return out


def sandwich_norm(stream: torch.Tensor, branch: Optional[torch.Tensor], w_post: Optional[torch.Tensor], eps_post: float,
                  w_pre: Optional[torch.Tensor], eps_pre: float, out: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """In one pass over the rows of the float32 `stream`: with `branch` (compute type), stream += RMSNorm(branch) *
    w_post; with `out` (compute type), out = RMSNorm(stream) * w_pre of the sum.  Statistics and sums are 32-bit."""
    rows, size = stream.shape
    if stream.dtype != torch.float32 or (branch is None) != (w_post is None) or (out is None) != (w_pre is None):
        raise KernelError("sandwich_norm: a float32 stream, a branch with its weights, an output with its weights")
    ref = branch if branch is not None else out
    if ref is None:
        return None
    for t in (branch, out):
        if t is not None and (t.shape != stream.shape or t.dtype != ref.dtype):
            raise KernelError("sandwich_norm: branch or output does not fit the stream")
    for w in (w_post, w_pre):
        if w is not None and w.numel() != size:
            raise KernelError("sandwich_norm: weights do not fit the rows")
    fn = _fn("stream_f32.cu", f"q3_sandwich_norm_{_suffix(ref)}",
             [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_float, c_float, c_void_p])
    _check(fn(_dev(stream, "stream"), _ptr(branch, "branch"), _ptr(w_post, "w_post", torch.float32),
              _ptr(w_pre, "w_pre", torch.float32), _ptr(out, "out"), rows, size, float(eps_post), float(eps_pre), _stream()),
           "sandwich_norm")
    return out


def concat_cast(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t] = [a[t]; b[t]] in out's type, from two float32 matrices of one shape."""
    rows, size = a.shape
    if a.dtype != torch.float32 or b.dtype != torch.float32 or b.shape != a.shape or out.shape != (rows, 2 * size):
        raise KernelError("concat_cast: shapes do not fit")
    fn = _fn("stream_f32.cu", f"q3_concat_cast_{_suffix(out)}", [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p])
    _check(fn(_dev(a, "a"), _dev(b, "b"), _dev(out, "out"), rows, size, _stream()), "concat_cast")
    return out


def gather_rows_norm(stream: torch.Tensor, idx: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> torch.Tensor:
    """out[r] = RMSNorm(stream[idx[r]]) * weight, from a float32 stream into out's type."""
    rows, size = idx.numel(), stream.shape[-1]
    if stream.dtype != torch.float32 or out.shape[0] < rows or out.shape[-1] != size or weight.numel() != size:
        raise KernelError("gather_rows_norm: shapes do not fit")
    fn = _fn("stream_f32.cu", f"q3_gather_rows_norm_{_suffix(out)}",
             [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_float, c_void_p])
    _check(fn(_dev(stream, "stream"), _dev(idx, "idx", torch.int32), _dev(weight, "weight", torch.float32), _dev(out, "out"),
              rows, size, float(eps), _stream()), "gather_rows_norm")
    return out


def scale_softcap(x: torch.Tensor, scale: float, cap: float = 0.0) -> torch.Tensor:
    """In place on float32 `x`: x <- cap * tanh(x * scale / cap), or x * scale when `cap` is 0."""
    fn = _fn("stream_f32.cu", "q3_scale_softcap_f32", [c_void_p, c_int64, c_float, c_float, c_void_p])
    _check(fn(_dev(x, "x", torch.float32), x.numel(), float(scale), float(cap or 0.0), _stream()), "scale_softcap")
    return x


# ------------------------------------------------------------------ matrix products
def gemm_f32(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T in true 32-bit (fmaf, fixed order over K)."""
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm_f32: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    fn = _fn("gemm_f32.cu", "q3_gemm_tn_f32",
             [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_void_p])
    _check(fn(_dev(x, "x", torch.float32), _dev(w, "w", torch.float32), _dev(out, "out", torch.float32),
              M, N, K, K, K, N, _stream()), "gemm_f32")
    return out


def gemm_bf16_any_width(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T for bfloat16 operands of any width K, on the CUDA cores with 32-bit
    accumulation: the product for widths that the tensor-core kernels refuse (K no multiple of 8)."""
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"gemm_bf16_any_width: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    fn = _fn("gemm_f32.cu", "q3_gemm_tn_bf16",
             [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int, c_void_p])
    _check(fn(_dev(x, "x", torch.bfloat16), _dev(w, "w", torch.bfloat16), _dev(out, "out"), M, N, K, K, K, N,
              int(out.dtype == torch.float32), _stream()), "gemm_bf16_any_width")
    return out


# ------------------------------------------------------------------ attention
def _rotary_dim(cos, sin, d: int) -> int:
    """How many leading values of a head the tables rotate: twice their width (the head size without tables)."""
    if cos is None:
        return d
    if sin is None or cos.shape != sin.shape or cos.dim() != 2 or 2 * cos.shape[1] > d:
        raise KernelError("rotation tables are [positions, rotary_dim / 2] with rotary_dim <= head_dim")
    return 2 * cos.shape[1]


def qkv_prepare(qkv, q_out, k_pages, v_pages, q_norm_w, k_norm_w, cos, sin, token_seq, token_pos, page_table,
                n_tokens: int, nq: int, nkv: int, d: int, eps: float, write_kv: bool = True, bias=None,
                value_dim: Optional[int] = None, value_heads: Optional[int] = None):
    """Per-head norm of q and k, rotation, and the write of k and v into the cache pages
    (`write_kv=False`: only q is prepared, for a layer that reads another layer's cache).  `bias` (float32, one
    value per column of the projection) is added first; `value_dim` is the size of a value head if not `d`,
    `value_heads` their number if not `nkv` (values that several key heads share)."""
    s = _suffix(qkv)
    vd, nv = int(value_dim or d), int(value_heads or nkv)
    if not 0 < d <= 256 or not 0 < vd <= 256 or (d % 2 != 0 and cos is not None and 2 * cos.shape[-1] == d):
        raise KernelError(f"head_dim {d} / value_dim {vd} is not supported: sizes up to 256, an even number of rotated values")
    if qkv.shape[-1] != (nq + nkv) * d + nv * vd or k_pages.dtype != qkv.dtype or k_pages.shape[1:] != (nkv, PAGE_TOKENS, d) \
            or v_pages.shape[1:] != (nv, PAGE_TOKENS, vd) or nkv % nv or (bias is not None and bias.numel() != qkv.shape[-1]):
        raise KernelError("qkv_prepare: shapes do not fit")
    rot = _rotary_dim(cos, sin, d)
    fn = _fn("attention.cu", f"q3_qkv_prepare_{s}",
             [c_void_p] * 11 + [c_int, c_int64, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_int, c_int, c_void_p])
    _check(fn(_dev(qkv, "qkv"), _dev(q_out, "q_out", qkv.dtype), _dev(k_pages, "k_pages"), _dev(v_pages, "v_pages"),
              _ptr(q_norm_w, "q_norm_w", torch.float32), _ptr(k_norm_w, "k_norm_w", torch.float32),
              _ptr(cos, "cos", torch.float32), _ptr(sin, "sin", torch.float32),
              _dev(token_seq, "token_seq", torch.int32), _dev(token_pos, "token_pos", torch.int32),
              _dev(page_table, "page_table", torch.int32), page_table.shape[-1], n_tokens, nq, nkv, d, float(eps),
              int(bool(write_kv)), rot, _ptr(bias, "bias", torch.float32), vd, nv, _stream()), "qkv_prepare")
    return q_out


def _sink_ptr(sink, sink_values, nq: int):
    if sink_values is None:
        return None
    if not sink or sink_values.numel() != nq:
        raise KernelError("attention: sink_values goes with sink and holds one float per query head")
    return _dev(sink_values, "sink_values", torch.float32)


def attention_generic(q, k_pages, v_pages, out, token_seq, token_pos, page_table, n_tokens: int, nq: int, nkv: int,
                      d: int, scale: float, window: Optional[int] = None, value_dim: Optional[int] = None,
                      softcap: float = 0.0, chunk: Optional[int] = None, sink: bool = False, value_heads: Optional[int] = None,
                      sink_values: Optional[torch.Tensor] = None, keep_first: int = 0):
    """Causal grouped-query attention of every token of the step over its sequence's pages.  `keep_first` (with `window`):
    the first so many keys of the sequence are seen beside the window's.  `softcap` > 0 caps the
    scores smoothly (s <- softcap * tanh(s / softcap)); `chunk`: a query reads only the keys of its own chunk of that
    many positions; `sink`: one more term exp(0), without a value, in the softmax's denominator (exp(sink_values[head])
    with `sink_values`, float32 [nq]); `value_dim`: the
    size of a value head (and of an output head) if not `d`; `value_heads`: the number of value heads if not `nkv`
    (each serves nkv / value_heads key heads).  `out` has q's type, or is float32 for a caller that goes on in 32-bit."""
    s = _suffix(q)
    vd, nv = int(value_dim or d), int(value_heads or nkv)
    if out.dtype not in (q.dtype, torch.float32) or nkv % nv:
        raise KernelError("attention: the output has the query's type or float32; key heads are a multiple of value heads")
    if not 0 < d <= 256 or not 0 < vd <= 256:
        raise KernelError(f"head_dim {d} / value_dim {vd} is not supported: sizes up to 256")
    if window and chunk:
        raise KernelError("attention: a window or chunks, not both")
    fn = _fn("attention.cu", f"q3_attention_generic_{s}",
             [c_void_p] * 7 + [c_int, c_int64, c_int, c_int, c_int, c_float, c_int, c_int, c_float, c_int, c_int, c_int, c_int,
                               c_void_p, c_int, c_void_p])
    _check(fn(_dev(q, "q"), _dev(k_pages, "k_pages", q.dtype), _dev(v_pages, "v_pages", q.dtype),
              _dev(out, "out"), _dev(token_seq, "token_seq", torch.int32),
              _dev(token_pos, "token_pos", torch.int32), _dev(page_table, "page_table", torch.int32),
              page_table.shape[-1], n_tokens, nq, nkv, d, float(scale), int(window or 0), vd, float(softcap or 0.0),
              int(chunk or 0), int(bool(sink)), nv, int(out.dtype == torch.float32 and q.dtype != torch.float32),
              _sink_ptr(sink, sink_values, nq), int(keep_first or 0) if window else 0, _stream()),
           "attention_generic")
    return out


def value_mix(rows: torch.Tensor, v_off: int, width: int, bias: Optional[torch.Tensor], first: torch.Tensor, save: bool,
              lam: float = 0.0) -> torch.Tensor:
    """On the columns [v_off, v_off + width) of every row, in place: v += bias (float32, may be None); then `save`:
    first = v, a copy for later layers; else v = (1 - lam) v + lam first.  `first` [N, width] in the rows' type."""
    N = rows.shape[0]
    if first.shape != (N, width) or first.dtype != rows.dtype or (bias is not None and bias.numel() != width):
        raise KernelError("value_mix: shapes do not fit")
    fn = _fn("attention.cu", f"q3_value_mix_{_suffix(rows)}",
             [c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p, c_int, c_float, c_int64, c_void_p])
    _check(fn(_dev(rows, "rows"), rows.shape[1], int(v_off), int(width), _ptr(bias, "bias", torch.float32), _dev(first, "first"),
              int(bool(save)), float(lam), N, _stream()), "value_mix")
    return rows


def head_gate(x: torch.Tensor, gate: torch.Tensor, heads: int, vd: int) -> torch.Tensor:
    """x[t, h, :] *= sigmoid(gate[t, h]) in place; x [N, heads * vd], `gate` a view of [N, heads] columns (its row
    stride may be larger)."""
    N = x.shape[0]
    if x.shape[1] != heads * vd or gate.shape != (N, heads) or gate.stride(1) != 1 or gate.dtype != x.dtype or not x.is_contiguous():
        raise KernelError("head_gate: shapes do not fit")
    fn = _fn("attention.cu", f"q3_head_gate_{_suffix(x)}", [c_void_p, c_void_p, c_int64, c_int, c_int, c_int64, c_void_p])
    _check(fn(x.data_ptr(), gate.data_ptr(), gate.stride(0), int(heads), int(vd), N, _stream()), "head_gate")
    return x


def short_conv(u: torch.Tensor, weight: torch.Tensor, state: torch.Tensor, token_seq, seq_start, seq_slots, out: torch.Tensor,
               n_seqs: int) -> torch.Tensor:
    """Causal convolution over time on the first C columns of u [N, >= C]: out[t, c] = sum_j weight[j, c] u[t - taps + 1 + j, c]
    within every sequence, the rows before the step from `state` (a view [slots, (taps - 1) * C] of float32 rows, the
    oldest row first), which is moved on afterwards.  weight float32 [taps, C] (a checkpoint's [C, taps] transposed);
    out [N, C] in u's type."""
    N, (taps, C) = u.shape[0], weight.shape
    if out.shape != (N, C) or out.dtype != u.dtype or u.shape[1] < C or u.stride(1) != 1 or state.shape[1] != (taps - 1) * C \
            or state.dtype != torch.float32 or (taps > 1 and state.stride(1) != 1) or not out.is_contiguous() or out.data_ptr() == u.data_ptr():
        raise KernelError("short_conv: shapes do not fit")
    fn = _fn("short_conv.cu", f"q3_short_conv_{_suffix(u)}",
             [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int, c_void_p])
    _check(fn(u.data_ptr(), u.stride(0), _dev(weight, "weight", torch.float32), state.data_ptr(), state.stride(0),
              _dev(token_seq, "token_seq", torch.int32), _dev(seq_start, "seq_start", torch.int32),
              _dev(seq_slots, "seq_slots", torch.int32), out.data_ptr(), C, taps, N, int(n_seqs), _stream()), "short_conv")
    if taps > 1:
        _count_extra(1)
    return out


# ------------------------------------------------------------------ several streams of hidden state (hyper-connections)
def embedding_streams(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float, copies: int) -> torch.Tensor:
    """out[t] = `copies` times table[ids[t]] * scale side by side, as float32: out [N, copies * hidden]."""
    n = ids.numel()
    if out.shape[0] < n or out.shape[1] != copies * table.shape[1] or out.dtype != torch.float32:
        raise KernelError("embedding_streams: output does not fit")
    fn = _fn("hyper.cu", f"q3_embedding_streams_{_suffix(table)}",
             [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_float, c_int, c_void_p])
    _check(fn(_dev(ids, "ids", torch.int32), _dev(table, "table"), _dev(out, "out"), n, table.shape[1], table.shape[0],
              float(scale), int(copies), _stream()), "embedding_streams")
    return out


def hyper_norm(streams: torch.Tensor, n_streams: int, branch: Optional[torch.Tensor], mix: Optional[torch.Tensor],
               out_coef: Optional[torch.Tensor], in_coef: Optional[torch.Tensor], norm_w: Optional[torch.Tensor], eps: float,
               out: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None,
               normalize: bool = True, compute_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """One pass over the streams [N, n_streams * hidden] (float32) of every token: settle a pending sublayer output
    `branch` [N, hidden] (x_to <- sum_from mix[from, to] x_from + out_coef[to] branch), form u = sum_s in_coef[s] x_s
    (None: ones) and write out = u / sqrt(mean(u^2) + eps) * norm_w (`normalize=False`: u itself).  `branch` and `out`
    may each be None.  With `rows` (int32 token numbers) only those tokens are worked on, `out` has one row for each
    and the streams are left as they are.  `out` has the compute type (the branch's) or float32."""
    N, width = streams.shape
    hidden = width // n_streams
    ref = branch if branch is not None else out
    if ref is None:
        return None
    kind = compute_dtype or (branch.dtype if branch is not None else out.dtype)
    count = int(n_rows if n_rows is not None else (rows.numel() if rows is not None else N))
    if width != hidden * n_streams or (branch is not None and tuple(branch.shape) != (N, hidden)) \
            or (out is not None and (out.shape[0] < count or out.shape[1] != hidden or out.dtype not in (kind, torch.float32))):
        raise KernelError("hyper_norm: shapes do not fit")
    fn = _fn("hyper.cu", f"q3_hyper_norm_{_SUFFIX[kind]}",
             [c_void_p] * 6 + [c_float, c_void_p, c_int, c_void_p, c_int64, c_int, c_int, c_int, c_void_p])
    _check(fn(_dev(streams, "streams", torch.float32), _ptr(branch, "branch", kind), _ptr(mix, "mix", torch.float32),
              _ptr(out_coef, "out_coef", torch.float32), _ptr(in_coef, "in_coef", torch.float32),
              _ptr(norm_w, "norm_w", torch.float32), float(eps), _ptr(out, "out"),
              int(out is not None and out.dtype == torch.float32 and kind != torch.float32), _ptr(rows, "rows", torch.int32),
              count, int(n_streams), hidden, int(bool(normalize)), _stream()), "hyper_norm")
    return out


# ------------------------------------------------------------------ linear attention with a decay and a state per sequence
def lightning_attention(proj: torch.Tensor, state: torch.Tensor, decay: torch.Tensor, seq_start: torch.Tensor,
                        seq_slots: torch.Tensor, out: torch.Tensor, n_seqs: int, heads: int, d: int, vd: int,
                        chunked: bool = False) -> torch.Tensor:
    """S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t over the new tokens of every sequence, from and to the state rows
    [slot, heads, d, vd] (float32).  `proj` [N, 2 heads d + 2 heads vd] holds q, k, v (SiLU is applied here) and a gate
    that is not read; `out` [N, heads * vd] float32.  `chunked`: the form for prompts (32 tokens at a time)."""
    if proj.shape[1] != 2 * heads * (d + vd) or tuple(state.shape[1:]) != (heads, d, vd) or out.shape[1] != heads * vd \
            or out.dtype != torch.float32 or decay.numel() != heads:
        raise KernelError("lightning_attention: shapes do not fit")
    name = "chunks" if chunked else "scan"
    if chunked and proj.dtype == torch.bfloat16 and lightning_tensor_cores and lightning_chunks_tc_fit(d, vd):
        name = "chunks_tc"                                   # the chunks' products on the tensor cores (TF32 hi + lo operands)
    fn = _fn("lightning.cu", f"q3_lightning_{name}_{_suffix(proj)}", [c_void_p] * 6 + [c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_dev(proj, "proj"), _dev(state, "state", torch.float32), _dev(decay, "decay", torch.float32),
              _dev(seq_start, "seq_start", torch.int32), _dev(seq_slots, "seq_slots", torch.int32), _dev(out, "out"),
              int(n_seqs), heads, d, vd, _stream()), f"lightning_{name}")
    return out


lightning_tensor_cores = True      # tests switch it off to run the fmaf form of the chunks in bfloat16


def lightning_chunks_tc_fit(d: int, vd: int) -> bool:
    """Whether the tensor-core form of the chunks takes these head sizes: steps of 8, buffers within an SM's shared memory."""
    dp = (d + 15) // 16 * 16
    return d % 8 == 0 and vd % 8 == 0 and (2 * 32 * (dp + 4) + 32 * (min(vd, 64) + 8) + 32 * 36 + dp * (min(vd, 64) + 8)) * 4 <= 200 * 1024


def lightning_chunks_fit(d: int, vd: int) -> bool:
    """Whether the chunked form's buffers fit in an SM's shared memory for these head sizes."""
    vt = min(vd, 64)
    R = min(d, 512 // vt)
    return (2 * 32 * (d + 1) + 32 * vt + 32 * 33 + R * 32 * vt) * 4 <= 200 * 1024


def gated_norm(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> torch.Tensor:
    """out = o / sqrt(mean(o^2) + eps) * weight * sigmoid(gate), row by row; o float32 [N, size], `gate` a view of
    [N, size] columns (its row stride may be larger), out in the compute type."""
    N, size = o.shape
    if gate.shape != o.shape or gate.stride(1) != 1 or out.shape != o.shape or gate.dtype != out.dtype or not out.is_contiguous():
        raise KernelError("gated_norm: shapes do not fit")
    fn = _fn("lightning.cu", f"q3_gated_norm_{_suffix(out)}", [c_void_p, c_void_p, c_int64, c_void_p, c_float, c_void_p, c_int64, c_int, c_void_p])
    _check(fn(_dev(o, "o", torch.float32), gate.data_ptr(), gate.stride(0), _dev(weight, "weight", torch.float32), float(eps),
              out.data_ptr(), N, size, _stream()), "gated_norm")
    return out


# ------------------------------------------------------------------ linear attention with keys: a decay per channel, or gates per head
def _scan_views(q, k, v, state, out, heads, d, vd, vdx):
    row = q.stride(0)
    if q.dtype != k.dtype or q.dtype != v.dtype or k.stride(0) != row or v.stride(0) != row or q.stride(1) != 1 or k.stride(1) != 1 \
            or v.stride(1) != 1 or q.shape[1] != heads * d or k.shape[1] != heads * d or v.shape[1] != heads * vd \
            or state.dtype != torch.float32 or state.shape[1] != heads * d * vdx or state.stride(1) != 1 \
            or out.dtype != torch.float32 or out.shape[1] != heads * vdx or not out.is_contiguous():
        raise KernelError("decay_scan: shapes do not fit")
    return row


def decay_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, state: torch.Tensor, seq_start: torch.Tensor, seq_slots: torch.Tensor,
               out: torch.Tensor, n_seqs: int, heads: int, d: int, vd: int, q_scale: float = 1.0, decay: Optional[torch.Tensor] = None,
               keep: Optional[torch.Tensor] = None, write: Optional[torch.Tensor] = None, ones: bool = False) -> torch.Tensor:
    """S_t = diag(a_t) S_(t-1) + k_t (b_t v_t)^T, o_t = S_t^T (q_t * q_scale) over the new tokens of every sequence, from and to
    the state rows (`state`: a view [slots, heads * d * vdx] of float32 rows).  q, k, v: column views of one projection
    output (same row stride).  With `decay` [N, heads * d] (float32, see `channel_decay`): a per channel, b = 1.  With
    `keep`, `write` [N, heads] (float32): a and b per head.  `ones`: vdx = vd + 1, the state's last column takes
    the value 1 (a normaliser); else vdx = vd.  out [N, heads * vdx] float32."""
    vdx = vd + (1 if ones else 0)
    row = _scan_views(q, k, v, state, out, heads, d, vd, vdx)
    N = q.shape[0]
    z = decay
    if (z is None) == (keep is None) or (z is not None and (tuple(z.shape) != (N, heads * d) or not z.is_contiguous())) \
            or (keep is not None and (write is None or keep.numel() < N * heads or write.numel() < N * heads)):
        raise KernelError("decay_scan: a decay per channel or gates per head (keep, write)")
    fn = _fn("linear_scan.cu", f"q3_decay_scan_{_suffix(q)}",
             [c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_int64,
              c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), row, _ptr(z, "decay", torch.float32), _ptr(keep, "keep", torch.float32), _ptr(write, "write", torch.float32), float(q_scale), int(bool(ones)),
              state.data_ptr(), state.stride(0), _dev(seq_start, "seq_start", torch.int32), _dev(seq_slots, "seq_slots", torch.int32),
              _dev(out, "out"), int(n_seqs), heads, d, vd, _stream()), "decay_scan")
    return out


def channel_decay(z: torch.Tensor, bias: Optional[torch.Tensor], tau: float) -> torch.Tensor:
    """In place: z <- sigmoid(z + bias)^(1 / tau); z [N, width] float32 logits, bias float32 [width] or None."""
    if z.dtype != torch.float32 or z.dim() != 2 or (bias is not None and bias.numel() != z.shape[1]) or not tau > 0:
        raise KernelError("channel_decay: float32 logits [N, width], one bias per column, a positive tau")
    fn = _fn("linear_scan.cu", "q3_channel_decay", [c_void_p, c_void_p, c_float, c_int64, c_int, c_void_p])
    _check(fn(_dev(z, "z"), _ptr(bias, "bias", torch.float32), 1.0 / float(tau), z.shape[0], z.shape[1], _stream()), "channel_decay")
    return z


def memory_gates(z: torch.Tensor, bias_i: torch.Tensor, bias_f: torch.Tensor, cap: float, m_state: torch.Tensor, seq_start, seq_slots,
                 keep: torch.Tensor, write: torch.Tensor, low: torch.Tensor, n_seqs: int, heads: int) -> None:
    """The gates of a matrix memory from z [N, 2 heads] (float32: input-gate logits, then forget-gate logits):
    i = cap tanh((zi + bias_i) / cap), f = logsigmoid(cap tanh((zf + bias_f) / cap)), the running maximum
    m_t = max(f_t + m_(t-1), i_t) from and to `m_state` (a view [slots, heads]), keep = exp(f + m_(t-1) - m_t),
    write = exp(i - m_t), low = exp(-m_t); all [N, heads] float32."""
    N = z.shape[0]
    if z.shape[1] != 2 * heads or z.dtype != torch.float32 or not z.is_contiguous() or m_state.shape[1] != heads \
            or m_state.stride(1) != 1 or m_state.dtype != torch.float32 or min(keep.numel(), write.numel(), low.numel()) < N * heads:
        raise KernelError("memory_gates: shapes do not fit")
    fn = _fn("linear_scan.cu", "q3_memory_gates",
             [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
              c_int64, c_int, c_void_p])
    _check(fn(z.data_ptr(), z.data_ptr() + 4 * heads, _dev(bias_i, "bias_i", torch.float32), _dev(bias_f, "bias_f", torch.float32),
              float(cap), m_state.data_ptr(), m_state.stride(0), _dev(seq_start, "seq_start", torch.int32),
              _dev(seq_slots, "seq_slots", torch.int32), _dev(keep, "keep", torch.float32), _dev(write, "write", torch.float32),
              _dev(low, "low", torch.float32), heads, 2 * heads, int(n_seqs), _stream()), "memory_gates")


def head_gated_norm(o: torch.Tensor, weight: torch.Tensor, gate: torch.Tensor, eps: float, out: torch.Tensor, heads: int, vd: int,
                    act: str = "sigmoid", low: Optional[torch.Tensor] = None, floor: float = 0.0) -> torch.Tensor:
    """Per (token, head): x = o[t, h, :vd] (with `low` [N, heads]: divided by max(|o[t, h, vd]|, low) + floor, the row then
    holding vd + 1 values), out = x / sqrt(mean(x^2) + eps) * weight * act(gate), act 'sigmoid' or 'silu'; `weight` float32
    [vd] (one for all heads) or [heads * vd]; `gate` a view of [N, heads * vd] columns; out in the gate's type."""
    N = o.shape[0]
    vdx = vd + (1 if low is not None else 0)
    if o.shape[1] != heads * vdx or o.dtype != torch.float32 or not o.is_contiguous() or weight.numel() not in (vd, heads * vd) \
            or gate.shape != (N, heads * vd) or gate.stride(1) != 1 or out.shape != (N, heads * vd) or out.dtype != gate.dtype \
            or not out.is_contiguous() or act not in ("sigmoid", "silu") or (low is not None and low.numel() < N * heads):
        raise KernelError("head_gated_norm: shapes do not fit")
    fn = _fn("linear_scan.cu", f"q3_head_gated_norm_{_suffix(out)}",
             [c_void_p, c_void_p, c_float, c_void_p, c_int, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_float, c_int, c_void_p])
    _check(fn(o.data_ptr(), _ptr(low, "low", torch.float32), float(floor), _dev(weight, "weight", torch.float32),
              int(weight.numel() == heads * vd and heads > 1), gate.data_ptr(), gate.stride(0), out.data_ptr(), N, heads, vd, vdx, float(eps),
              int(act == "silu"), _stream()), "head_gated_norm")
    return out


# ------------------------------------------------------------------ differential attention
def diff_combine(a: torch.Tensor, out: torch.Tensor, n_tokens: int, heads: int, per_group: int, vd: int, lam: float, eps: float,
                 gain: float) -> torch.Tensor:
    """out[t, h] = unit_rms(a1 - lam * a2) * gain over vd values; `a` float32 [N, groups, 2 maps, per_group, vd]."""
    if a.dtype != torch.float32 or a.numel() < n_tokens * 2 * heads * vd or out.numel() < n_tokens * heads * vd:
        raise KernelError("diff_combine: shapes do not fit")
    fn = _fn("differential.cu", f"q3_diff_combine_{_suffix(out)}",
             [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_float, c_float, c_float, c_void_p])
    _check(fn(_dev(a, "a"), _dev(out, "out"), n_tokens, heads, per_group, vd, float(lam), float(eps), float(gain), _stream()),
           "diff_combine")
    return out


# ------------------------------------------------------------------ feed-forwards: a plain activation; routed experts
PLAIN_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "gelu": 2}


def activation(x: torch.Tensor, out: torch.Tensor, kind: str) -> torch.Tensor:
    """out = act(x) elementwise (`out` may be `x`); kinds: silu, gelu_tanh, gelu (with the error function)."""
    if out.shape != x.shape or out.dtype != x.dtype:
        raise KernelError("activation: output does not fit")
    fn = _fn("elementwise.cu", f"q3_activation_{_suffix(x)}", [c_void_p, c_void_p, c_int64, c_int, c_void_p])
    _check(fn(_dev(x, "x"), _dev(out, "out"), x.numel(), PLAIN_ACTIVATIONS[kind], _stream()), "activation")
    return out


def moe_route(h: torch.Tensor, w_router: torch.Tensor, correction: torch.Tensor, top_ids: torch.Tensor, top_w: torch.Tensor,
              id_weight: torch.Tensor, n_real: int, top: int, group_count: int = 1, group_keep: int = 1, by_logit: bool = False,
              gate_out: Optional[torch.Tensor] = None, sigmoid: bool = False, group_pair: bool = False,
              weight_scale: float = 1.0) -> None:
    """Router of a mixture of experts for every token of h [N, hidden]: float32 logits, softmax over all outputs
    (`sigmoid`: each output's sigmoid by itself), choice by score + correction within the kept groups (a group's mark:
    its best choice score, or with `group_pair` the sum of its two best), weights = plain scores times `weight_scale`;
    `by_logit`: the largest logits are chosen and weighted by the softmax over the chosen logits alone (the correction is
    not read).  With `gate_out` [N] the router matrix has one more row, and gate_out = sigmoid of its logit; see csrc/moe.cu."""
    N, hidden = h.shape
    n_out = w_router.shape[0] - (1 if gate_out is not None else 0)
    if w_router.shape[1] != hidden or w_router.dtype != h.dtype or (correction is not None and correction.numel() != n_out) \
            or (correction is None and not by_logit) or top_ids.numel() < N * top or top_w.numel() < N * top or id_weight.numel() < N \
            or (gate_out is not None and gate_out.numel() < N) or (by_logit and sigmoid):
        raise KernelError("moe_route: shapes do not fit")
    fn = _fn("moe.cu", f"q3_moe_route_{_suffix(h)}",
             [c_void_p] * 6 + [c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_float, c_void_p])
    _check(fn(_dev(h, "h"), _dev(w_router, "w_router"), _ptr(correction, "correction", torch.float32),
              _dev(top_ids, "top_ids", torch.int32), _dev(top_w, "top_w", torch.float32), _dev(id_weight, "id_weight", torch.float32),
              N, hidden, n_out, int(n_real), int(top), int(group_count), int(group_keep), 1 if by_logit else (2 if sigmoid else 0),
              _ptr(gate_out, "gate_out", torch.float32), int(bool(group_pair)), float(weight_scale), _stream()), "moe_route")


def moe_sort(top_ids: torch.Tensor, n_pairs: int, n_real: int, offsets: torch.Tensor, slot_of_pair: torch.Tensor,
             pair_of_slot: torch.Tensor) -> None:
    """Lays the (token, choice) pairs out expert by expert: offsets [n_real + 1], a slot for every pair (-1: an
    identity expert) and the pair of every slot."""
    if offsets.numel() < n_real + 1 or slot_of_pair.numel() < n_pairs or pair_of_slot.numel() < n_pairs:
        raise KernelError("moe_sort: shapes do not fit")
    fn = _fn("moe.cu", "q3_moe_sort", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(fn(_dev(top_ids, "top_ids", torch.int32), int(n_pairs), int(n_real), _dev(offsets, "offsets", torch.int32),
              _dev(slot_of_pair, "slot_of_pair", torch.int32), _dev(pair_of_slot, "pair_of_slot", torch.int32), _stream()), "moe_sort")


moe_tensor_cores = True      # tests switch it off to run the fmaf tiles in bfloat16


def moe_experts(h: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, offsets: torch.Tensor, pair_of_slot: torch.Tensor,
                act: torch.Tensor, y: torch.Tensor, n_pairs: int, n_real: int, top: int, ff: int, limit: float, alpha: float,
                up_offset: float = 1.0) -> None:
    """The experts' two products for the sorted pairs: act[slot] = g sigmoid(alpha g) (u + up_offset) with g = min(W_gate x, limit),
    u = clamp(W_up x, -limit, limit) (limit infinity, alpha 1, up_offset 0: SiLU(gate) * up), then y[slot] = W_down act[slot] (float32).  w_gate_up [n_real, 2 ff, hidden] (an
    expert's gate rows, then its up rows), w_down [n_real, hidden, ff]."""
    hidden = h.shape[1]
    if w_gate_up.numel() != n_real * 2 * ff * hidden or w_down.numel() != n_real * hidden * ff or act.numel() < n_pairs * ff \
            or y.numel() < n_pairs * hidden or y.dtype != torch.float32 or act.dtype != h.dtype or w_gate_up.dtype != h.dtype:
        raise KernelError("moe_experts: shapes do not fit")
    tensor_cores = h.dtype == torch.bfloat16 and hidden % 32 == 0 and ff % 32 == 0 and moe_tensor_cores
    name = "q3_moe_experts_tc_bf16" if tensor_cores else f"q3_moe_experts_{_suffix(h)}"
    fn = _fn("moe.cu", name, [c_void_p] * 7 + [c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_void_p])
    _check(fn(_dev(h, "h"), _dev(w_gate_up, "w_gate_up"), _dev(w_down, "w_down"), _dev(offsets, "offsets", torch.int32),
              _dev(pair_of_slot, "pair_of_slot", torch.int32), _dev(act, "act"), _dev(y, "y"), int(n_pairs), int(n_real), int(top),
              hidden, int(ff), float(limit), float(alpha), float(up_offset), _stream()), "moe_experts")
    _count_extra(1)


def moe_combine(y: torch.Tensor, h: torch.Tensor, slot_of_pair: torch.Tensor, top_w: torch.Tensor, id_weight: torch.Tensor,
                out: torch.Tensor, top: int, shared: Optional[torch.Tensor] = None, shared_w: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = sum_k top_w[t, k] y[slot_of_pair[t, k]] + id_weight[t] h[t] (+ shared_w[t] shared[t])."""
    N, hidden = h.shape
    if out.shape != h.shape or out.dtype != h.dtype or (shared is None) != (shared_w is None) \
            or (shared is not None and (shared.shape != h.shape or shared.dtype != h.dtype or shared_w.numel() < N)):
        raise KernelError("moe_combine: shapes do not fit")
    fn = _fn("moe.cu", f"q3_moe_combine_{_suffix(h)}", [c_void_p] * 6 + [c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check(fn(_dev(y, "y", torch.float32), _dev(h, "h"), _dev(slot_of_pair, "slot_of_pair", torch.int32),
              _dev(top_w, "top_w", torch.float32), _dev(id_weight, "id_weight", torch.float32), _dev(out, "out"), N, int(top), hidden,
              _ptr(shared, "shared"), _ptr(shared_w, "shared_w", torch.float32), _stream()), "moe_combine")
    return out


# ------------------------------------------------------------------ capped / chunked / sink attention on the tensor cores
def attention_capped_fits(d: int, vd: int, window: Optional[int], group: int) -> bool:
    """Whether `attention_capped_prefill` / `_decode` take these sizes: keys and values in steps of 16 up to 256, at
    most 16 query heads per key/value head (a sliding window is taken)."""
    return d % 16 == 0 and vd % 16 == 0 and 0 < d <= 256 and 0 < vd <= 256 and group <= 16


def _capped_defines(d: int, vd: int):
    return (f"Q3_HEAD_DIM={d}", f"Q3_VALUE_DIM={vd}")


def attention_capped_prefill(q, k_pages, v_pages, out, seq_start, seq_pos0, page_table, n_seqs: int, max_new: int, nq: int,
                             nkv: int, d: int, vd: int, scale: float, softcap: float = 0.0, chunk: Optional[int] = None,
                             sink: bool = False, window: Optional[int] = None, value_heads: Optional[int] = None,
                             sink_values: Optional[torch.Tensor] = None, keep_first: int = 0):
    """Attention of every new token of every sequence over its pages (bfloat16, tiled, tensor cores) with capped scores,
    chunked visibility or a sliding window (beside which the first `keep_first` keys of the sequence stay visible), and a sink (its score per query head in `sink_values`, else 0); q [tokens, nq * d], out [tokens, nq * vd] in bfloat16 or float32;
    `value_heads`: the number of value heads if not `nkv` (each serves nkv / value_heads key heads)."""
    nv = int(value_heads or nkv)
    if q.dtype != torch.bfloat16 or not attention_capped_fits(d, vd, None, 1) or out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("attention_capped_prefill: bfloat16, head sizes in steps of 16 up to 256")
    if k_pages.shape[1:] != (nkv, PAGE_TOKENS, d) or v_pages.shape[1:] != (nv, PAGE_TOKENS, vd) or out.shape[-1] != nq * vd:
        raise KernelError("attention_capped_prefill: shapes do not fit")
    fn = _fn("attention_capped.cu", "q3_attention_capped_prefill_bf16",
             [c_void_p] * 7 + [c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_int, c_int, c_int, c_int, c_void_p,
                               c_int, c_void_p],
             defines=_capped_defines(d, vd))
    _check(fn(_dev(q, "q"), _dev(k_pages, "k_pages", torch.bfloat16), _dev(v_pages, "v_pages", torch.bfloat16),
              _dev(out, "out"), _dev(seq_start, "seq_start", torch.int32),
              _dev(seq_pos0, "seq_pos0", torch.int32), _dev(page_table, "page_table", torch.int32), page_table.shape[-1],
              n_seqs, max_new, nq, nkv, float(scale), float(softcap or 0.0), int(chunk or 0), int(bool(sink)), int(window or 0), nv,
              int(out.dtype == torch.float32), _sink_ptr(sink, sink_values, nq), int(keep_first or 0) if window else 0, _stream()),
           "attention_capped_prefill")
    return out


def attention_capped_splits(n_tokens: int, nkv: int, sm_count: int, max_keys: int) -> int:
    """Key ranges per (token, kv head) of the decode kernel: enough blocks for two per SM, no more than pages."""
    pages = max(1, -(-int(max_keys) // PAGE_TOKENS) + 1)
    return int(max(1, min(16, pages, (2 * sm_count) // max(1, n_tokens * nkv))))


def attention_capped_decode(q, k_pages, v_pages, out, scratch, token_seq, token_pos, page_table, n_tokens: int, nq: int,
                            nkv: int, d: int, vd: int, scale: float, softcap: float, chunk: Optional[int], sink: bool,
                            n_splits: int, window: Optional[int] = None, value_heads: Optional[int] = None,
                            sink_values: Optional[torch.Tensor] = None, keep_first: int = 0):
    """The same for one new token per sequence, the keys split over `n_splits` blocks per (token, kv head); `scratch`
    holds n_tokens * nq * n_splits * (vd + 2) float32."""
    nv = int(value_heads or nkv)
    if q.dtype != torch.bfloat16 or not attention_capped_fits(d, vd, None, nq // nkv) or out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("attention_capped_decode: bfloat16, head sizes in steps of 16 up to 256, groups of up to 16 heads")
    if k_pages.shape[1:] != (nkv, PAGE_TOKENS, d) or v_pages.shape[1:] != (nv, PAGE_TOKENS, vd) or out.shape[-1] != nq * vd \
            or scratch.numel() < n_tokens * nq * n_splits * (vd + 2):
        raise KernelError("attention_capped_decode: shapes do not fit")
    fn = _fn("attention_capped.cu", "q3_attention_capped_decode_bf16",
             [c_void_p] * 8 + [c_int, c_int64, c_int, c_int, c_float, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                               c_int, c_void_p],
             defines=_capped_defines(d, vd))
    _check(fn(_dev(q, "q"), _dev(k_pages, "k_pages", torch.bfloat16), _dev(v_pages, "v_pages", torch.bfloat16),
              _dev(out, "out"), _dev(scratch, "scratch", torch.float32),
              _dev(token_seq, "token_seq", torch.int32), _dev(token_pos, "token_pos", torch.int32),
              _dev(page_table, "page_table", torch.int32), page_table.shape[-1], n_tokens, nq, nkv, float(scale),
              float(softcap or 0.0), int(chunk or 0), int(bool(sink)), int(n_splits), int(window or 0), nv,
              int(out.dtype == torch.float32), _sink_ptr(sink, sink_values, nq), int(keep_first or 0) if window else 0, _stream()),
           "attention_capped_decode")
    _count_extra(1)                                              # the split kernel and the merge kernel
    return out


def attention_capped_decode_fused(qkv, k_pages, v_pages, out, scratch, bias, cos, sin, token_seq, token_pos, page_table,
                                  n_tokens: int, nq: int, nkv: int, d: int, vd: int, scale: float, softcap: float,
                                  chunk: Optional[int], sink: bool, n_splits: int):
    """`attention_capped_decode` from the output of the q/k/v projection as it is: the bias, the rotation of q and k and
    the write of the new key and value into their pages happen in the attention's own kernel."""
    if qkv.dtype != torch.bfloat16 or not attention_capped_fits(d, vd, None, nq // nkv):
        raise KernelError("attention_capped_decode_fused: bfloat16, head sizes in steps of 16 up to 256, groups of up to 16 heads")
    if qkv.shape[-1] != (nq + nkv) * d + nkv * vd or k_pages.shape[1:] != (nkv, PAGE_TOKENS, d) \
            or v_pages.shape[1:] != (nkv, PAGE_TOKENS, vd) or out.shape[-1] != nq * vd \
            or scratch.numel() < n_tokens * nq * n_splits * (vd + 2) or (bias is not None and bias.numel() != qkv.shape[-1]):
        raise KernelError("attention_capped_decode_fused: shapes do not fit")
    rot = _rotary_dim(cos, sin, d)
    fn = _fn("attention_capped.cu", "q3_attention_capped_decode_fused_bf16",
             [c_void_p] * 8 + [c_int] + [c_void_p] * 3 + [c_int, c_int64, c_int, c_int, c_float, c_float, c_int, c_int, c_int, c_void_p],
             defines=_capped_defines(d, vd))
    _check(fn(_dev(qkv, "qkv"), _dev(k_pages, "k_pages", torch.bfloat16), _dev(v_pages, "v_pages", torch.bfloat16),
              _dev(out, "out", torch.bfloat16), _dev(scratch, "scratch", torch.float32), _ptr(bias, "bias", torch.float32),
              _ptr(cos, "cos", torch.float32), _ptr(sin, "sin", torch.float32), rot, _dev(token_seq, "token_seq", torch.int32),
              _dev(token_pos, "token_pos", torch.int32), _dev(page_table, "page_table", torch.int32), page_table.shape[-1],
              n_tokens, nq, nkv, float(scale), float(softcap or 0.0), int(chunk or 0), int(bool(sink)), int(n_splits), _stream()),
           "attention_capped_decode_fused")
    _count_extra(1)
    return out


def attention_capped_prefill_tc_fits(d: int, vd: int, window: Optional[int]) -> bool:
    return d in (64, 128) and vd == d and not window


def attention_capped_prefill_tc(q, k_pages, v_pages, out, seq_start, seq_pos0, page_table, n_seqs: int, max_new: int,
                                n_tokens: int, nq: int, nkv: int, d: int, scale: float, softcap: float = 0.0,
                                chunk: Optional[int] = None, sink: bool = False):
    """`attention_capped_prefill` with both products on tcgen05 (TMA-fed, scores and output in tensor memory): head
    sizes 64 and 128, values as wide as keys."""
    if q.dtype != torch.bfloat16 or not attention_capped_prefill_tc_fits(d, d, None) or not scale > 0:
        raise KernelError("attention_capped_prefill_tc: bfloat16, head size 64 or 128, a positive scale")
    fn = _fn("attention_prefill_tc.cu", "q3_attention_capped_prefill_tc_bf16",
             [c_void_p] * 7 + [c_int, c_int, c_int, c_int64, c_int64, c_int, c_int, c_float, c_float, c_int, c_int, c_void_p, c_void_p],
             defines=(f"Q3_HEAD_DIM={d}", "Q3_CAPPED=1"))
    _check(fn(_dev(q, "q"), _dev(k_pages, "k_pages", torch.bfloat16), _dev(v_pages, "v_pages", torch.bfloat16),
              _dev(out, "out", torch.bfloat16), _dev(seq_start, "seq_start", torch.int32),
              _dev(seq_pos0, "seq_pos0", torch.int32), _dev(page_table, "page_table", torch.int32),
              page_table.shape[-1], n_seqs, max_new, n_tokens, k_pages.shape[0], nq, nkv, float(scale), float(softcap or 0.0),
              int(chunk or 0), int(bool(sink)), _status_word(q.device).data_ptr(), _stream()), "attention_capped_prefill_tc")
    return out


# ------------------------------------------------------------------ sampling
def argmax(logits: torch.Tensor, out: torch.Tensor, valid: Optional[int] = None) -> torch.Tensor:
    """out[r] = index of the highest logit of row r (lowest id among equals, NaN as -inf)."""
    rows, vocab = logits.shape
    fn = _fn("sampling.cu", "q3_argmax_f32", [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_dev(logits, "logits", torch.float32), vocab, rows, int(valid or vocab),
              _dev(out, "out", torch.int32), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: float, top_k: int, top_p: float, seed: int,
           seq_ids: torch.Tensor, steps, valid: Optional[int] = None) -> torch.Tensor:
    """One draw per row; out[r] = -1 marks a row with a non-finite logit.  `steps` is an int32 tensor with
    the step of every row, or one int for all rows."""
    rows, vocab = logits.shape
    fn = _fn("sampling.cu", "q3_sample_f32",
             [c_void_p, c_int64, c_int, c_int, c_float, c_int, c_float, c_uint64, c_void_p, c_void_p, c_int, c_void_p,
              c_void_p])
    per_row = isinstance(steps, torch.Tensor)
    _check(fn(_dev(logits, "logits", torch.float32), vocab, rows, int(valid or vocab), float(temperature), int(top_k),
              float(top_p), int(seed) & 0xFFFFFFFFFFFFFFFF, _dev(seq_ids, "seq_ids", torch.int64),
              _dev(steps, "steps", torch.int32) if per_row else None, 0 if per_row else int(steps),
              _dev(out, "out", torch.int32), _stream()), "sample")
    return out


# ------------------------------------------------------------------ bfloat16 decode attention
def attention_decode_splits(n_tokens: int, nkv: int, sm_count: int) -> int:
    """Key splits such that the whole grid (splits x kv heads x tokens) is resident at once, two
    blocks per SM, and at most 16: fixed by the batch size alone.  (Measured at batch 8, 4,096
    keys: 4 splits 29 us, 5 splits - a second wave - 39 us.)"""
    return max(1, min(16, (2 * sm_count) // max(1, n_tokens * nkv)))


def attention_decode(q, k_pages, v_pages, out, scratch, token_seq, token_pos, page_table, n_tokens: int, nq: int,
                     nkv: int, d: int, scale: float, window: Optional[int], n_splits: int):
    """One token per sequence against its cached keys; `scratch` is float32 with at least
    n_tokens * nq * n_splits * (d + 2) elements."""
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_decode is a bfloat16 kernel")
    if nq // nkv > 16 or d % 16 != 0 or d > 256:
        raise KernelError(f"attention_decode: group of {nq // nkv} heads or head_dim {d} not supported")
    if scratch.numel() < n_tokens * nq * n_splits * (d + 2):
        raise KernelError("attention_decode: scratch too small")
    fn = _fn("attention_decode.cu", "q3_attention_decode_bf16",
             [c_void_p] * 8 + [c_int, c_int64, c_int, c_int, c_float, c_int, c_int, c_void_p],
             defines=(f"Q3_HEAD_DIM={d}",))
    _check(fn(_dev(q, "q"), _dev(k_pages, "k_pages", torch.bfloat16), _dev(v_pages, "v_pages", torch.bfloat16),
              _dev(out, "out", torch.bfloat16), _dev(scratch, "scratch", torch.float32),
              _dev(token_seq, "token_seq", torch.int32), _dev(token_pos, "token_pos", torch.int32),
              _dev(page_table, "page_table", torch.int32), page_table.shape[-1], n_tokens, nq, nkv, float(scale),
              int(window or 0), int(n_splits), _stream()), "attention_decode")
    _count_extra(1)
    return out


FUSED_DECODE_MAX_SPLITS = 16
_fused_max_splits = {}


def attention_decode_fused_max_splits(d: int, device) -> int:
    """The most key splits `attention_decode_fused` takes on `device` for head size `d`: 16 where the device places
    clusters of 16 blocks (beyond the portable size), else 8."""
    key = (d, torch.device(device))
    got = _fused_max_splits.get(key)
    if got is None:
        fn = _fn_untimed("attention_decode.cu", "q3_attention_decode_fused_max_splits", [], defines=(f"Q3_HEAD_DIM={d}",))
        with torch.cuda.device(key[1]):
            got = _fused_max_splits[key] = int(fn())
    return got


def attention_decode_fused(qkv, k_pages, v_pages, out, q_norm_w, k_norm_w, cos, sin, eps: float, token_seq, token_pos,
                           page_table, n_tokens: int, nq: int, nkv: int, d: int, scale: float, window: Optional[int],
                           n_splits: int, write_kv: bool = True):
    """The attention of a decode step in one launch: per-head norm and rotation of the new query and key, the
    write of key and value into the cache pages, attention over the pages split over the keys, and the merge of
    the splits inside a thread-block cluster.  `qkv` is the projection output [tokens, (nq + 2 nkv) * d]."""
    if qkv.dtype != torch.bfloat16:
        raise KernelError("attention_decode_fused is a bfloat16 kernel")
    if nq // nkv > 16 or d % 16 != 0 or d > 256 or not 0 < n_splits <= FUSED_DECODE_MAX_SPLITS:
        raise KernelError(f"attention_decode_fused: group of {nq // nkv} heads, head_dim {d} or {n_splits} splits not supported")
    if qkv.shape[-1] != (nq + 2 * nkv) * d or k_pages.shape[1:] != (nkv, PAGE_TOKENS, d) or out.shape[-1] != nq * d:
        raise KernelError("attention_decode_fused: shapes do not fit")
    fn = _fn("attention_decode.cu", "q3_attention_decode_fused_bf16",
             [c_void_p] * 8 + [c_float] + [c_void_p] * 3 + [c_int, c_int64, c_int, c_int, c_float, c_int, c_int, c_int, c_int,
                                                            c_void_p],
             defines=(f"Q3_HEAD_DIM={d}",))
    _check(fn(_dev(qkv, "qkv"), _dev(k_pages, "k_pages", torch.bfloat16), _dev(v_pages, "v_pages", torch.bfloat16),
              _dev(out, "out", torch.bfloat16), _ptr(q_norm_w, "q_norm_w", torch.float32), _ptr(k_norm_w, "k_norm_w", torch.float32),
              _ptr(cos, "cos", torch.float32), _ptr(sin, "sin", torch.float32), float(eps),
              _dev(token_seq, "token_seq", torch.int32), _dev(token_pos, "token_pos", torch.int32),
              _dev(page_table, "page_table", torch.int32), page_table.shape[-1], n_tokens, nq, nkv, float(scale),
              int(window or 0), int(n_splits), int(bool(write_kv)), _rotary_dim(cos, sin, d), _stream()), "attention_decode_fused")
    return out


# ------------------------------------------------------------------ bfloat16 weight-streaming product
SKINNY_MAX_ROWS = 64


def gemm_skinny_fits(M: int, K: int) -> bool:
    return 0 < M <= SKINNY_MAX_ROWS and K % 8 == 0


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T for M <= 64, bfloat16 operands, out bfloat16 or float32."""
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or not gemm_skinny_fits(M, K):
        raise KernelError(f"gemm_skinny: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    name = {torch.bfloat16: "q3_gemm_skinny_bf16", torch.float32: "q3_gemm_skinny_bf16_f32out"}.get(out.dtype)
    if name is None:
        raise KernelError("gemm_skinny: output must be bfloat16 or float32")
    fn = _fn("gemm_skinny_bf16.cu", name, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_dev(x, "x", torch.bfloat16), _dev(w, "w", torch.bfloat16), _dev(out, "out"), M, N, K, _stream()),
           "gemm_skinny")
    return out


# ------------------------------------------------------------------ bfloat16 prompt attention
def attention_prefill(q, k_pages, v_pages, out, seq_start, seq_pos0, page_table, n_seqs: int, max_new: int, nq: int,
                      nkv: int, d: int, scale: float, window: Optional[int] = None):
    """Causal attention of every new token of every sequence over its pages (tiled, tensor cores)."""
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_prefill is a bfloat16 kernel")
    if d % 16 != 0 or d > 256:
        raise KernelError(f"head_dim {d} is not supported: multiples of 16 up to 256")
    fn = _fn("attention_prefill.cu", "q3_attention_prefill_bf16",
             [c_void_p] * 7 + [c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
             defines=(f"Q3_HEAD_DIM={d}",))
    _check(fn(_dev(q, "q"), _dev(k_pages, "k_pages", torch.bfloat16), _dev(v_pages, "v_pages", torch.bfloat16),
              _dev(out, "out", torch.bfloat16), _dev(seq_start, "seq_start", torch.int32),
              _dev(seq_pos0, "seq_pos0", torch.int32), _dev(page_table, "page_table", torch.int32),
              page_table.shape[-1], n_seqs, max_new, nq, nkv, float(scale), int(window or 0), _stream()),
           "attention_prefill")
    return out


# ------------------------------------------------------------------ bfloat16 tcgen05 product
_tc_status = {}


def _status_word(device) -> torch.Tensor:
    word = _tc_status.get(device)
    if word is None:
        word = _tc_status[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return word


def tcgen05_status(device) -> int:
    """0, or where a bounded wait inside the tcgen05 product gave up (1 producer, 2 MMA, 3 epilogue);
    reading it synchronises the device and clears it."""
    word = _status_word(torch.device(device))
    value = int(word.item())
    if value:
        word.zero_()
    return value


def gemm_tcgen05_mid(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, splits: int = 0) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T for a few hundred rows at most on the 5th-generation tensor cores,
    weights first: TMA-fed tiles of 128 rows of w, accumulator in tensor memory, K split over the `splits` blocks
    of a cluster (0 = chosen from N and K) that add their partial tiles through distributed shared
    memory.  bfloat16 operands, out bfloat16 or float32; K a multiple of 8."""
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or K % 8 != 0:
        raise KernelError(f"gemm_tcgen05_mid: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("gemm_tcgen05_mid: output must be bfloat16 or float32")
    fn = _fn("gemm_tcgen05.cu", "q3_gemm_tcgen05_mid_bf16",
             [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_dev(x, "x", torch.bfloat16), _dev(w, "w", torch.bfloat16), _dev(out, "out"), M, N, K,
              int(out.dtype == torch.float32), 0, int(splits), _status_word(x.device).data_ptr(), _stream()),
           "gemm_tcgen05_mid")
    return out


def gemm_tcgen05_mid_splits(M: int, N: int, K: int) -> int:
    """The number of K ranges `gemm_tcgen05_mid` chooses for this shape."""
    lib = load_library("gemm_tcgen05.cu", ())
    lib.q3_gemm_tcgen05_mid_splits.argtypes = [c_int, c_int, c_int]
    lib.q3_gemm_tcgen05_mid_splits.restype = c_int
    return int(lib.q3_gemm_tcgen05_mid_splits(N, K, M))


def gemm_tcgen05_mid_gated(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, splits: int = 0,
                           activation: str = "silu") -> torch.Tensor:
    """out[M, N/2] = round(act(g)) * u (act: SiLU or the tanh form of GELU) for a few hundred rows at most; `w` [N, K] holds the gate and up rows interleaved
    in blocks of eight (`interleave_gate_up`); the gating runs where the cluster's partial tiles are added."""
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N // 2) or K % 8 != 0 or N % 16 != 0 or out.dtype != torch.bfloat16:
        raise KernelError(f"gemm_tcgen05_mid_gated: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    fn = _fn("gemm_tcgen05.cu", "q3_gemm_tcgen05_mid_bf16",
             [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_dev(x, "x", torch.bfloat16), _dev(w, "w", torch.bfloat16), _dev(out, "out"), M, N, K, 0,
              ACTIVATIONS[activation] + 1, int(splits), _status_word(x.device).data_ptr(), _stream()), "gemm_tcgen05_mid_gated")
    return out


def gemm_skinny_gated(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, activation: str = "silu") -> torch.Tensor:
    """out[M, N/2] = round(act(g)) * u where g and u are the products of x with the gate and up rows of
    w [N, K], which holds them interleaved in blocks of eight rows (see `interleave_gate_up`); act is SiLU or
    (`activation="gelu_tanh"`) the tanh form of GELU."""
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N // 2) or N % 16 != 0 or not gemm_skinny_fits(M, K):
        raise KernelError(f"gemm_skinny_gated: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    fn = _fn("gemm_skinny_bf16.cu", "q3_gemm_skinny_act_bf16", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_dev(x, "x", torch.bfloat16), _dev(w, "w", torch.bfloat16), _dev(out, "out", torch.bfloat16), M, N, K,
              ACTIVATIONS[activation] + 1, _stream()), "gemm_skinny_gated")
    return out


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[2I, K]: rows 16t..16t+7 are gate rows 8t..8t+7, rows 16t+8..16t+15 the up rows of the same features."""
    I, K = gate.shape
    if I % 8 != 0 or up.shape != gate.shape:
        raise KernelError("interleave_gate_up: the intermediate size must be a multiple of 8")
    return torch.stack([gate.view(I // 8, 8, K), up.view(I // 8, 8, K)], dim=1).reshape(2 * I, K).contiguous()


def gemm_tcgen05_prompt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tile_n: int = 256) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T for many rows: persistent blocks, tiles of 128 tokens by `tile_n`
    (128 or 256) rows of w, accumulators double-buffered in tensor memory."""
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or K % 8 != 0:
        raise KernelError(f"gemm_tcgen05_prompt: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("gemm_tcgen05_prompt: output must be bfloat16 or float32")
    fn = _fn("gemm_tcgen05.cu", "q3_gemm_tcgen05_prompt_bf16",
             [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_dev(x, "x", torch.bfloat16), _dev(w, "w", torch.bfloat16), _dev(out, "out"), M, N, K,
              int(out.dtype == torch.float32), int(tile_n), _status_word(x.device).data_ptr(), _stream()),
           "gemm_tcgen05_prompt")
    return out


def gemm_tcgen05_pair(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gated: bool = False,
                      splits: int = 1, activation: str = "silu") -> torch.Tensor:
    """The prompt product on pairs of SMs (tcgen05 cta_group::2): tiles of 256 tokens by 256 rows of w, each
    block of a pair loading its own tokens and half of the w tile.  `gated`: w holds gate and up rows
    interleaved in blocks of eight and out is [M, N/2] = round(act(g)) * u, act being SiLU or (`activation`) the tanh
    form of GELU.  `splits` (1..4): K split over
    that many pairs of one cluster, whose partial tiles are summed over distributed shared memory in a fixed
    order (for shapes with too few tiles, or a tile count just above a whole number of waves)."""
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N // 2 if gated else N) or K % 8 != 0 or (gated and N % 16 != 0):
        raise KernelError(f"gemm_tcgen05_pair: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    if out.dtype not in ((torch.bfloat16,) if gated else (torch.bfloat16, torch.float32)):
        raise KernelError("gemm_tcgen05_pair: output must be bfloat16 (or float32 when not gated)")
    if not 1 <= splits <= PAIR_MAX_SPLITS:
        raise KernelError(f"gemm_tcgen05_pair: 1 to {PAIR_MAX_SPLITS} K ranges, not {splits}")
    fn = _fn("gemm_tcgen05.cu", "q3_gemm_tcgen05_pair_bf16",
             [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_dev(x, "x", torch.bfloat16), _dev(w, "w", torch.bfloat16), _dev(out, "out"), M, N, K,
              int(out.dtype == torch.float32), ACTIVATIONS[activation] + 1 if gated else 0, int(splits),
              _status_word(x.device).data_ptr(), _stream()),
           "gemm_tcgen05_pair")
    return out


PAIR_MAX_SPLITS = 4


def gemm_tcgen05_pair_capacity(splits: int) -> int:
    """How many pairs of SMs of the current device run at once when a cluster is `splits` pairs (0: none fit)."""
    fn = _fn_untimed("gemm_tcgen05.cu", "q3_gemm_tcgen05_pair_capacity", [c_int])
    return int(fn(int(splits)))


PAIR_QKV_HEAD_DIMS = (64, 128, 256)


def gemm_tcgen05_pair_qkv(x: torch.Tensor, w: torch.Tensor, q_out, k_pages, v_pages, q_norm_w, k_norm_w, cos, sin, eps,
                          token_seq, token_pos, page_table, n_tokens: int, nq: int, nkv: int, d: int,
                          write_kv: bool = True) -> None:
    """The q/k/v product of a prompt step on pairs of SMs with `qkv_prepare`'s work in its epilogue: per-head
    RMSNorm of q and k (weights may be None), rotation of the whole head (tables [positions, d/2], may be None),
    q into q_out [n_tokens, nq*d], k and v into the pages at the tokens' positions (`write_kv`); the product's
    own output is never stored.  w [(nq + 2 nkv) d, K] holds the q, k and v rows one after the other.  bfloat16,
    head sizes 64, 128 and 256."""
    M, K = x.shape
    if x.dtype != torch.bfloat16 or M != n_tokens or w.shape != ((nq + 2 * nkv) * d, K) or K % 8 != 0 or d not in PAIR_QKV_HEAD_DIMS:
        raise KernelError(f"gemm_tcgen05_pair_qkv: shapes {tuple(x.shape)} x {tuple(w.shape)}^T for {nq}+2*{nkv} heads of {d}")
    if q_out.shape != (n_tokens, nq * d) or (q_norm_w is None) != (k_norm_w is None) or (cos is None) != (sin is None):
        raise KernelError("gemm_tcgen05_pair_qkv: q_out, norm weights or tables do not fit")
    if cos is not None and _rotary_dim(cos, sin, d) != d:
        raise KernelError("gemm_tcgen05_pair_qkv rotates the whole head only")
    fn = _fn("gemm_tcgen05.cu", "q3_gemm_tcgen05_pair_qkv_bf16",
             [c_void_p, c_void_p, c_int, c_int] + [c_void_p] * 7 + [c_float] + [c_void_p] * 3 + [c_int] * 5 + [c_void_p, c_void_p])
    _check(fn(_dev(x, "x", torch.bfloat16), _dev(w, "w", torch.bfloat16), M, K, _dev(q_out, "q_out", torch.bfloat16),
              _dev(k_pages, "k_pages", torch.bfloat16), _dev(v_pages, "v_pages", torch.bfloat16),
              _ptr(q_norm_w, "q_norm_w", torch.float32), _ptr(k_norm_w, "k_norm_w", torch.float32),
              _ptr(cos, "cos", torch.float32), _ptr(sin, "sin", torch.float32), float(eps),
              _dev(token_seq, "token_seq", torch.int32), _dev(token_pos, "token_pos", torch.int32),
              _dev(page_table, "page_table", torch.int32), page_table.shape[-1], nq, nkv, d, int(bool(write_kv)),
              _status_word(x.device).data_ptr(), _stream()), "gemm_tcgen05_pair_qkv")


def gemm_tcgen05_prompt_gated(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N/2] = round(silu(g)) * u for many rows; `w` [N, K] holds the gate and up rows interleaved in
    blocks of eight (`interleave_gate_up`); the gating runs in the product's epilogue."""
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N // 2) or K % 8 != 0 or N % 16 != 0 or out.dtype != torch.bfloat16:
        raise KernelError(f"gemm_tcgen05_prompt_gated: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    fn = _fn("gemm_tcgen05.cu", "q3_gemm_tcgen05_prompt_gated_bf16",
             [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_dev(x, "x", torch.bfloat16), _dev(w, "w", torch.bfloat16), _dev(out, "out"), M, N, K,
              _status_word(x.device).data_ptr(), _stream()), "gemm_tcgen05_prompt_gated")
    return out


# ------------------------------------------------------------------ bfloat16 prompt attention on tcgen05
def attention_prefill_tc_fits(d: int, window: Optional[int]) -> bool:
    return d in (64, 128) and not window


def attention_prefill_tc(q, k_pages, v_pages, out, seq_start, seq_pos0, page_table, n_seqs: int, max_new: int,
                         n_tokens: int, nq: int, nkv: int, d: int, scale: float):
    """Causal attention of every new token over its pages with both products on tcgen05 (TMA-fed,
    scores and output accumulated in tensor memory).  Head sizes 64 and 128."""
    if q.dtype != torch.bfloat16 or not attention_prefill_tc_fits(d, None):
        raise KernelError("attention_prefill_tc: bfloat16, head size 64 or 128")
    fn = _fn("attention_prefill_tc.cu", "q3_attention_prefill_tc_bf16",
             [c_void_p] * 7 + [c_int, c_int, c_int, c_int64, c_int64, c_int, c_int, c_float, c_void_p, c_void_p],
             defines=(f"Q3_HEAD_DIM={d}",))
    _check(fn(_dev(q, "q"), _dev(k_pages, "k_pages", torch.bfloat16), _dev(v_pages, "v_pages", torch.bfloat16),
              _dev(out, "out", torch.bfloat16), _dev(seq_start, "seq_start", torch.int32),
              _dev(seq_pos0, "seq_pos0", torch.int32), _dev(page_table, "page_table", torch.int32),
              page_table.shape[-1], n_seqs, max_new, n_tokens, k_pages.shape[0], nq, nkv, float(scale),
              _status_word(q.device).data_ptr(), _stream()), "attention_prefill_tc")
    return out


# ------------------------------------------------------------------ a float32 stream with norms of several kinds, a token shift, a side input
NORM_KINDS = {"none": 0, "rms": 1, "dynamic_tanh": 2, "round": 3}


def _norm_args(norm, size: int, what: str):
    """(kind, weight, b, alpha, eps) of a norm part for `settle_norm`; None: no norm at this place.  The string
    "round" asks for the rounded sum alone (an output only)."""
    if norm is None:
        return 0, None, None, 0.0, 0.0
    if norm == "round":
        return 3, None, None, 0.0, 0.0
    kind = NORM_KINDS[getattr(norm, "stream_kind", "rms")]
    w, b = norm.weight, getattr(norm, "b", None)
    if w.numel() != size or (b is not None and b.numel() != size):
        raise KernelError(f"settle_norm: the {what} norm's vectors do not fit the rows")
    return kind, _dev(w, "weight", torch.float32), _ptr(b, "b", torch.float32), float(getattr(norm, "alpha", 0.0)), float(norm.eps)


def settle_norm(stream: torch.Tensor, branch: Optional[torch.Tensor], post, pre, out: Optional[torch.Tensor],
                rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None,
                compute_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """One pass over the rows of the float32 `stream`: with `branch` (compute type) and the norm part `post`,
    stream += post(branch); with `out` and `pre` (a norm part, or "round"), out = pre(stream) of the sum.  `out` is of the
    compute type or float32.  The norm parts are RMS norms (unit rms times a weight) or dynamic-tanh norms
    (tanh(alpha x) * weight + b).  With `rows` (int32) only those rows are read, nothing is written to the stream
    and out[r] belongs to rows[r]."""
    total, size = stream.shape
    if stream.dtype != torch.float32 or (branch is None) != (post is None) or (out is None) != (pre is None):
        raise KernelError("settle_norm: a float32 stream, a branch with its norm, an output with its norm")
    if branch is None and out is None:
        return None
    dtype = branch.dtype if branch is not None else (compute_dtype or out.dtype)
    if branch is not None and (branch.shape != stream.shape or not branch.is_contiguous()):
        raise KernelError("settle_norm: the branch does not fit the stream")
    n = total if rows is None else int(n_rows if n_rows is not None else rows.numel())
    if out is not None and (out.shape[0] < n or out.shape[-1] != size or out.dtype not in (dtype, torch.float32)):
        raise KernelError("settle_norm: the output does not fit")
    pk, pw, pb, pa, pe = _norm_args(post, size, "post")
    qk, qw, qb, qa, qe = _norm_args(pre, size, "pre")
    fn = _fn("stream_shift.cu", f"q3_settle_norm_{_SUFFIX[dtype]}",
             [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_float, c_int, c_void_p, c_void_p, c_float, c_float,
              c_void_p, c_int, c_void_p, c_int64, c_int, c_void_p])
    _check(fn(_dev(stream, "stream"), _ptr(branch, "branch"), pk, pw, pb, pa, pe, qk, qw, qb, qa, qe, _ptr(out, "out"),
              int(out is not None and out.dtype == torch.float32 and dtype != torch.float32),
              _ptr(rows, "rows", torch.int32), n, size, _stream()), "settle_norm")
    return out


def token_shift(h: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, out: torch.Tensor, token_seq: torch.Tensor,
                seq_start: torch.Tensor, seq_slots: torch.Tensor, n_tokens: int) -> torch.Tensor:
    """out[t] = h[t] + (h[t-1] - h[t]) * mu within every sequence (h float32, out the compute type).  The row before a
    sequence's first row of the step is state[slot] (zero for a new sequence); the sequence's last row replaces it."""
    size = h.shape[-1]
    if h.dtype != torch.float32 or mu.numel() != size or state.shape[-1] != size or out.shape[-1] != size \
            or h.shape[0] < n_tokens or out.shape[0] < n_tokens:
        raise KernelError("token_shift: shapes do not fit")
    fn = _fn("stream_shift.cu", f"q3_token_shift_{_suffix(out)}", [c_void_p] * 7 + [c_int64, c_int, c_void_p])
    _check(fn(_dev(h, "h"), _dev(mu, "mu", torch.float32), _dev(state, "state", torch.float32), _dev(out, "out"),
              _dev(token_seq, "token_seq", torch.int32), _dev(seq_start, "seq_start", torch.int32),
              _dev(seq_slots, "seq_slots", torch.int32), int(n_tokens), size, _stream()), "token_shift")
    return out


def side_gate(a: torch.Tensor, ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, col0: int) -> torch.Tensor:
    """out[t, j] = gelu_tanh(a[t, j]) * table[ids[t], col0 + j]; a, out [N, dim], table [vocab, columns]."""
    N, dim = a.shape
    if out.shape != a.shape or out.dtype != a.dtype or table.dtype != a.dtype or ids.numel() < N:
        raise KernelError("side_gate: shapes do not fit")
    fn = _fn("stream_shift.cu", f"q3_side_gate_{_suffix(a)}", [c_void_p] * 4 + [c_int64, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_dev(a, "a"), _dev(ids, "ids", torch.int32), _dev(table, "table"), _dev(out, "out"), N, dim, int(col0),
              table.shape[1], table.shape[0], _stream()), "side_gate")
    return out


# ------------------------------------------------------------------ linear attention whose forget gate also writes (HGRN2)
def gated_scan(proj: torch.Tensor, state: torch.Tensor, low: torch.Tensor, bias: torch.Tensor, seq_start: torch.Tensor,
               seq_slots: torch.Tensor, out: torch.Tensor, n_seqs: int, heads: int, d: int, vd: int) -> torch.Tensor:
    """f = low + (1 - low) sigmoid(z + bias), S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T SiLU(q_t) over the new
    tokens of every sequence, from and to the state rows [slot, heads, d, vd] (float32).  `proj` [N, heads (2 d + vd)]
    holds q, z and v head by head; `out` [N, heads * vd] float32."""
    if proj.shape[1] != heads * (2 * d + vd) or tuple(state.shape[1:]) != (heads, d, vd) or out.shape[1] != heads * vd \
            or out.dtype != torch.float32 or low.numel() != heads * d or bias.numel() != heads * d:
        raise KernelError("gated_scan: shapes do not fit")
    fn = _fn("gated_recurrence.cu", f"q3_gated_scan_{_suffix(proj)}", [c_void_p] * 7 + [c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_dev(proj, "proj"), _dev(state, "state", torch.float32), _dev(low, "low", torch.float32),
              _dev(bias, "bias", torch.float32), _dev(seq_start, "seq_start", torch.int32),
              _dev(seq_slots, "seq_slots", torch.int32), _dev(out, "out"), int(n_seqs), heads, d, vd, _stream()), "gated_scan")
    return out


def head_rms_norm(o: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, vd: int) -> torch.Tensor:
    """out = o / sqrt(mean(o^2) + eps) * weight over every run of `vd` values of a row (one weight vector for all
    heads); o float32 [N, heads * vd], out in the compute type."""
    if o.dtype != torch.float32 or out.shape != o.shape or weight.numel() != vd or o.shape[-1] % vd:
        raise KernelError("head_rms_norm: shapes do not fit")
    fn = _fn("gated_recurrence.cu", f"q3_head_rms_norm_{_suffix(out)}", [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_float, c_void_p])
    _check(fn(_dev(o, "o"), _dev(weight, "weight", torch.float32), _dev(out, "out"), o.numel() // vd, vd, float(eps), _stream()),
           "head_rms_norm")
    return out


# ------------------------------------------------------------------ attention over a latent cache
def latent_prepare(proj: torch.Tensor, kv_off: int, q_off: int, w_c: torch.Tensor, w_q: Optional[torch.Tensor],
                   cq: Optional[torch.Tensor], k_pages: torch.Tensor, v_pages: torch.Tensor, cos, sin, token_seq, token_pos,
                   page_table, n_tokens: int, rank: int, rot: int, rot_dims: int, interleaved: bool, eps: float,
                   write_kv: bool = True) -> None:
    """Per token, from the row `proj[t]`: c = unit_rms(proj[t, kv_off : kv_off + rank]) * w_c and the next `rot` values,
    rotated by the token's position, go to the token's key row [c | rotated] in its page, c also to its value row.  With
    `cq` [N, q_rank]: cq[t] = unit_rms(proj[t, q_off : q_off + q_rank]) * w_q, the latent of the queries."""
    q_rank = 0 if cq is None else cq.shape[-1]
    if proj.stride(-1) != 1 or k_pages.shape[1:] != (1, PAGE_TOKENS, rank + rot) or v_pages.shape[1:] != (1, PAGE_TOKENS, rank) \
            or w_c.numel() != rank or (cq is not None and (w_q is None or w_q.numel() != q_rank or cq.dtype != proj.dtype)) \
            or kv_off + rank + rot > proj.shape[1] or q_off + q_rank > proj.shape[1]:
        raise KernelError("latent_prepare: shapes do not fit")
    fn = _fn("latent.cu", f"q3_latent_prepare_{_suffix(proj)}",
             [c_void_p, c_int64, c_int, c_int] + [c_void_p] * 10 + [c_int, c_int64, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                                                   c_void_p])
    _check(fn(_dev(proj, "proj"), proj.stride(0), int(kv_off), int(q_off), _dev(w_c, "w_c", torch.float32),
              _ptr(w_q, "w_q", torch.float32), _ptr(cq, "cq"), _dev(k_pages, "k_pages", proj.dtype),
              _dev(v_pages, "v_pages", proj.dtype), _ptr(cos, "cos", torch.float32), _ptr(sin, "sin", torch.float32),
              _dev(token_seq, "token_seq", torch.int32), _dev(token_pos, "token_pos", torch.int32),
              _dev(page_table, "page_table", torch.int32), page_table.shape[-1], int(n_tokens), int(rank), int(rot), int(rot_dims),
              int(bool(interleaved)), int(q_rank), float(eps), int(bool(write_kv)), _stream()), "latent_prepare")


def latent_queries(q: torch.Tensor, q_full: torch.Tensor, cos, sin, token_pos, n_tokens: int, heads: int, d: int, rank: int,
                   rot: int, rot_dims: int, interleaved: bool) -> None:
    """q_full[t, h, rank:] = rotate(q[t, h, d:]) for q [N, heads * (d + rot)] (a view whose rows may lie apart) and
    q_full [N, heads * (rank + rot)]."""
    if q.shape[1] != heads * (d + rot) or q_full.shape[1] != heads * (rank + rot) or q.dtype != q_full.dtype \
            or q.stride(-1) != 1 or not q_full.is_contiguous() or not q.is_cuda:
        raise KernelError("latent_queries: shapes do not fit")
    fn = _fn("latent.cu", f"q3_latent_queries_{_suffix(q)}",
             [c_void_p, c_int64] + [c_void_p] * 4 + [c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(q.data_ptr(), q.stride(0), _dev(q_full, "q_full"), _ptr(cos, "cos", torch.float32), _ptr(sin, "sin", torch.float32),
              _dev(token_pos, "token_pos", torch.int32), int(n_tokens), heads, d, rank, rot, int(rot_dims), int(bool(interleaved)),
              _stream()), "latent_queries")


def head_product(x: torch.Tensor, x_head: int, x_off: int, w: torch.Tensor, out: torch.Tensor, out_head: int, out_off: int,
                 n_tokens: int, gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t, h * out_head + out_off + j] = sum_i x[t, h * x_head + x_off + i] * w[h, i, j] for w [heads, K, N], a product per
    head (32-bit accumulation); with `gate` (a view [N, heads * N] whose rows may lie apart) the result is multiplied by
    sigmoid(gate[t, h * N + j])."""
    heads, K, N = w.shape
    if x.dtype != w.dtype or out.dtype != w.dtype or x.stride(-1) != 1 or out.stride(-1) != 1 \
            or x_off + K > x_head or out_off + N > out_head or heads * x_head > x.shape[1] or heads * out_head > out.shape[1] \
            or (gate is not None and (gate.dtype != w.dtype or gate.stride(-1) != 1 or gate.shape[1] != heads * N)):
        raise KernelError("head_product: shapes do not fit")
    fn = _fn("latent.cu", f"q3_head_product_{_suffix(w)}",
             [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_int64, c_int64, c_int, c_int, c_int,
              c_void_p])
    if not (x.is_cuda and out.is_cuda and w.is_cuda and w.is_contiguous()):
        raise KernelError("head_product: contiguous CUDA weights, CUDA operands")
    _check(fn(x.data_ptr(), x.stride(0), int(x_head), int(x_off), w.data_ptr(), out.data_ptr(), out.stride(0), int(out_head),
              int(out_off), None if gate is None else gate.data_ptr(), 0 if gate is None else gate.stride(0), int(n_tokens), heads, K, N,
              _stream()), "head_product")
    return out
