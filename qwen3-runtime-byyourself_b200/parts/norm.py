"""RMSNorm as a part: y = round(x * rsqrt(mean(x^2) + eps)) * w, statistics in 32-bit.

Formula and rounding points of the reference: src/ops/rms_norm.cu:87-120 (eps inside
the root, the weight multiplies directly).  The optional `delta` fuses the residual
sum of src/ops/elementwise.cu:30-34 into the same pass.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import Part, register_part


class RMSNorm(Part):
    stream_kind = "rms"          # how the kernels of a float32 stream apply this part (ops.NORM_KINDS)

    def __init__(self, size: int, eps: float, one_plus: bool = False):
        """`one_plus`: the stored weight lies around zero and the norm multiplies by 1 + weight."""
        self.size, self.eps, self.one_plus = int(size), float(eps), bool(one_plus)
        self.weight = None

    def weight_specs(self, name: str) -> dict:
        return {name: WeightSpec((self.size,), "bias" if self.one_plus else "norm")}

    def bind(self, weights: dict, name: str, dtype, device) -> None:
        # a scale vector is used in 32-bit whatever it was stored in (exact for bfloat16)
        self.weight = weights[name].to(device=device, dtype=torch.float32).contiguous()
        if self.one_plus:
            getattr(weights, "wait", lambda: None)()          # a streamed checkpoint: the tensor is in place now
            self.weight = (self.weight + 1.0).contiguous()

    def __call__(self, x: torch.Tensor, out: torch.Tensor, delta=None) -> torch.Tensor:
        return ops.rms_norm(x, self.weight, self.eps, out, delta)


class DynamicTanh(Part):
    """The norm without statistics: y = tanh(alpha * x) * weight + b, element by element, with one scalar `alpha` and
    a vector `b` stored beside the weight as `<name>.alpha` and `<name>.b`.  It is applied by the kernels of a float32
    stream (`ops.settle_norm`), which take it wherever they take an RMS norm; `eps` is accepted and not used."""
    stream_kind = "dynamic_tanh"

    def __init__(self, size: int, eps: float = 0.0, alpha_name: str = ".alpha", b_name: str = ".b"):
        self.size, self.eps = int(size), float(eps)
        self.alpha_name, self.b_name = alpha_name, b_name
        self.weight = self.b = None
        self.alpha = 1.0

    def weight_specs(self, name: str) -> dict:
        return {name: WeightSpec((self.size,), "norm"), name + self.b_name: WeightSpec((self.size,), "bias"),
                name + self.alpha_name: WeightSpec((), "bias")}

    def bind(self, weights: dict, name: str, dtype, device) -> None:
        self.weight = weights[name].to(device=device, dtype=torch.float32).contiguous()
        self.b = weights[name + self.b_name].to(device=device, dtype=torch.float32).contiguous()
        alpha = weights[name + self.alpha_name]
        getattr(weights, "wait", lambda: None)()              # a streamed checkpoint: the tensor is in place now
        self.alpha = float(alpha.float().reshape(-1)[0].item())   # a launch argument: read once, here

    def __call__(self, x: torch.Tensor, out: torch.Tensor, delta=None) -> torch.Tensor:
        if x.dtype != torch.float32 or delta is not None:
            raise ops.KernelError("dynamic_tanh is applied on a float32 stream by settle_norm")
        return ops.settle_norm(x, None, None, self, out)


register_part("norm", "rms_norm", RMSNorm)
register_part("norm", "dynamic_tanh", DynamicTanh)
