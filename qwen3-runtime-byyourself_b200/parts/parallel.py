"""Several mixers side by side as one mixer part: all read the same input, and the layer's result is the weighted sum
of theirs, sum_i scale_i * mixer_i(x).

What the mixers ask of the cache is put together: at most one of them may hold keys and values (the layer's pages are
its pages); their per-sequence states lie one after the other in the layer's state row, and every mixer gets a view of
its own columns.
"""
from __future__ import annotations

import dataclasses
from typing import Sequence

import torch

from ..cache.book import CacheNeed
from ..config.plan import PartSpec
from ..csrc import ops
from .base import Part, build_part, register_part


class ParallelMixers(Part):
    def __init__(self, hidden_size: int, mixers: Sequence[PartSpec], scales: Sequence[float]):
        if len(mixers) < 2 or len(mixers) != len(scales):
            raise ValueError("parallel mixers: at least two, one scale each")
        self.hidden_size = int(hidden_size)
        self.mixers = [build_part("mixer", spec) for spec in mixers]
        self.scales = [float(s) for s in scales]
        for i, mixer in enumerate(self.mixers):
            if not hasattr(mixer, "out_name"):
                raise ValueError(f"a {type(mixer).__name__} cannot run beside other mixers: its result's buffer has no name to change")
            mixer.out_name = f"mixer.out.{i}"
        needs = [m.cache_need() for m in self.mixers]
        if sum(1 for n in needs if n.kind != "none") > 1 or any(n.block_state for n in needs):
            raise ValueError("parallel mixers: only one of them may keep keys and values")
        self.state_sizes = []
        for n in needs:
            size = 1
            for s in n.state_shape:
                size *= int(s)
            self.state_sizes.append(size if n.state_shape else 0)
        paged = [n for n in needs if n.kind != "none"]
        self._need = dataclasses.replace(paged[0] if paged else CacheNeed("none"),
                                         state_shape=(sum(self.state_sizes),) if sum(self.state_sizes) else ())
        self.graph_safe = all(getattr(m, "graph_safe", True) for m in self.mixers)

    def weight_specs(self, prefix: str) -> dict:
        specs = {}
        for mixer in self.mixers:
            specs.update(mixer.weight_specs(prefix))
        return specs

    def bind(self, weights: dict, prefix: str, dtype, device) -> None:
        for mixer in self.mixers:
            mixer.bind(weights, prefix, dtype, device)

    def cache_need(self) -> CacheNeed:
        return self._need

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        whole = cache.state.view(cache.state.shape[0], -1) if cache.state is not None else None
        outs, at = [], 0
        for mixer, size in zip(self.mixers, self.state_sizes):
            view = dataclasses.replace(cache, state=whole[:, at:at + size] if size else None)
            outs.append(mixer.forward(x, ctx, view))
            at += size
        out = ctx.scratch.get("mixer.out", (ctx.n_tokens, self.hidden_size), ctx.dtype)
        ops.scaled_sum(outs[0], outs[1], self.scales[0], self.scales[1], out)
        for o, s in zip(outs[2:], self.scales[2:]):
            ops.scaled_sum(out, o, 1.0, s, out)
        return out


register_part("mixer", "parallel_mixers", ParallelMixers)
