"""Rotary position encoding as a part.

Table as in the reference (src/ops/rope.cu:276-295): inv_freq_i = theta^(-2i/d),
angle = position * inv_freq_i computed in float64, cosine and sine stored as
float32.  Rotation is half-split, pairs (i, i + d/2) (src/ops/rope.cu:60-84); the
attention part hands the tables to its fused kernel, `apply_` is the stand-alone form.

Two options beyond Qwen3.  `interleaved`: the pairs are (2i, 2i + 1).  Since a dot product
does not change when queries and keys are reordered alike, a mixer may reorder the rows of
its query and key projections once, at load time, with `kernel_order()` and run the
half-split kernels on the result.  `scaling`: the frequencies are rescaled by wavelength
for contexts beyond the trained one: with l = 2 pi / f, f stays where l < original / high,
becomes f / factor where l > original / low, and in between is the blend
(1 - s) f / factor + s f with s = (original / l - low) / (high - low).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .base import Part, register_part


class RotaryEmbedding(Part):
    fused_tables = True   # exposes cos/sin [positions, rotary_dim/2] float32 for a kernel to read

    def __init__(self, head_dim: int, theta: float, max_positions: int, rotary_dim: int = 0, interleaved: bool = False,
                 scaling: Optional[dict] = None, theta_float32: bool = True):
        """`rotary_dim` (default: the head size, as in Qwen3): only the first `rotary_dim` values of a head are
        rotated, in pairs (i, i + rotary_dim/2) with inv_freq_i = theta^(-2i/rotary_dim); the rest pass through.
        `interleaved`: pairs (2i, 2i + 1) instead.  `scaling`: {factor, low, high, original}, see the top of the file.
        `theta_float32`: theta is rounded to a 32-bit float first, as the reference holds it; False takes it as given."""
        rotary_dim = int(rotary_dim) or int(head_dim)
        if rotary_dim % 2 or not 0 < rotary_dim <= head_dim:
            raise ValueError("rotary encoding needs an even rotary_dim within the head")
        self.head_dim, self.theta, self.max_positions = int(head_dim), float(theta), int(max_positions)
        self.rotary_dim = rotary_dim
        self.interleaved, self.theta_float32 = bool(interleaved), bool(theta_float32)
        self.scaling = None
        if scaling:
            self.scaling = {k: float(scaling[k]) for k in ("factor", "low", "high", "original")}
            if self.scaling["high"] == self.scaling["low"] or min(self.scaling.values()) <= 0:
                raise ValueError("frequency scaling needs positive factor, low, high, original and low != high")
        self.cos = self.sin = None

    def frequencies(self):
        """The rotary_dim / 2 angular frequencies, in float64, after the rescaling by wavelength."""
        half = self.rotary_dim // 2
        # theta is held as a 32-bit float by the reference (include/qwen3/model/config.h:22)
        theta = float(torch.tensor(self.theta, dtype=torch.float32).item()) if self.theta_float32 else self.theta
        freq = [math.pow(theta, -(2.0 * i) / self.rotary_dim) for i in range(half)]
        if self.scaling:
            sc = self.scaling
            for i, f in enumerate(freq):
                wavelength = 2.0 * math.pi / f
                if wavelength < sc["original"] / sc["high"]:
                    continue
                if wavelength > sc["original"] / sc["low"]:
                    freq[i] = f / sc["factor"]
                else:
                    blend = (sc["original"] / wavelength - sc["low"]) / (sc["high"] - sc["low"])
                    freq[i] = (1.0 - blend) * f / sc["factor"] + blend * f
        return freq

    def kernel_order(self):
        """For an interleaved encoding: the order of a head's values in which pair i sits at (i, i + rotary_dim/2),
        as the kernels rotate it (`order[j]` = the value that moves to place j); None for a half-split encoding."""
        if not self.interleaved:
            return None
        r = self.rotary_dim
        return list(range(0, r, 2)) + list(range(1, r, 2)) + list(range(r, self.head_dim))

    def prepare(self, n_positions: int, device) -> None:
        n = min(int(n_positions), self.max_positions)
        if self.cos is not None and self.cos.shape[0] >= n and self.cos.device == torch.device(device):
            return
        inv_freq = torch.tensor(self.frequencies(), dtype=torch.float64)
        angle = torch.arange(n, dtype=torch.float64)[:, None] * inv_freq[None, :]
        self.cos = torch.cos(angle).to(torch.float32).to(device).contiguous()
        self.sin = torch.sin(angle).to(torch.float32).to(device).contiguous()

    def apply_(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor, kernel_order: bool = False) -> None:
        """Rotate q [N, heads, d] and k in place (32-bit arithmetic, result in the tensors' type).  `kernel_order`:
        the heads were reordered with `kernel_order()`, so an interleaved encoding rotates half-split pairs."""
        half = self.rotary_dim // 2
        c = self.cos[positions.long()][:, None, :]
        s = self.sin[positions.long()][:, None, :]
        first_at, second_at = slice(0, half), slice(half, 2 * half)
        if self.interleaved and not kernel_order:
            first_at, second_at = slice(0, 2 * half, 2), slice(1, 2 * half, 2)
        for t in (q, k):
            a, b = t[..., first_at].float(), t[..., second_at].float()
            first, second = a * c - b * s, b * c + a * s     # both from the unrotated values
            t[..., first_at] = first.to(t.dtype)
            t[..., second_at] = second.to(t.dtype)


register_part("position", "rope", RotaryEmbedding)
