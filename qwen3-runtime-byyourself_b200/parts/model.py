"""A model put together from a `ModelPlan`: embedding, layers in their order, final norm, head.

The forward pass is the reference's (src/model/model.cpp:107-147: embedding ->
layers -> final norm) followed by the output projection (src/model/lm_head.cpp:
188-191), with two differences of arrangement: it runs on packed tokens of several
sequences of unequal length, and the final norm and the head run only on the rows
whose logits are wanted (the reference normalises every row and drops all but the
last).
"""
from __future__ import annotations

import dataclasses
import sys
from typing import Dict, List, Optional

import torch

from ..cache.book import CacheNeed
from ..config.plan import ModelPlan
from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import build_part


class Model:
    def __init__(self, plan: ModelPlan):
        self.plan = plan
        self.embedding = build_part("embedding", plan.embedding)
        self.blocks = []
        for spec in plan.layers:
            mixer = build_part("mixer", spec.mixer)
            feed_forward = build_part("feed_forward", spec.feed_forward) if spec.feed_forward is not None else None
            self.blocks.append(build_part("block", spec.block, mixer, feed_forward))
        self.stream_steps = {}            # run -> (part, tensor name): what rewrites the hidden state before that run
        for step in plan.stream_steps:
            self.stream_steps[step.before_run] = (build_part("stream", step.part), step.name)
        self.residual_dtype = torch.float32 if plan.residual_dtype == "float32" else None
        self.final_norm_name = plan.final_norm_name or plan.final_norm_prefix + "weight"
        self.final_norm = build_part("norm", plan.final_norm)
        self.head = build_part("head", plan.head)
        self.dtype: Optional[torch.dtype] = None
        self.device = None
        self._warned_rounding = False
        self.after_run = None             # a debugging hook: after_run(run, residual, pending, ctx) after every layer run

    # -- weights
    def weight_specs(self) -> Dict[str, WeightSpec]:
        p = self.plan
        specs = dict(self.embedding.weight_specs(p.embedding_prefix))
        for spec, block in zip(p.layers, self.blocks):
            specs.update(block.weight_specs(spec.prefix))
        for part, name in self.stream_steps.values():
            specs.update(part.weight_specs(name))
        specs.update(self.final_norm.weight_specs(self.final_norm_name))
        specs.update(self.head.weight_specs(p.head_prefix))
        return specs

    def ignorable_names(self) -> List[str]:
        names = list(getattr(self.head, "ignorable", lambda prefix: [])(self.plan.head_prefix))
        for spec, block in zip(self.plan.layers, self.blocks):
            names += list(getattr(block, "ignorable", lambda prefix: [])(spec.prefix))
        return names

    def bind(self, weights, dtype: torch.dtype, device) -> None:
        """Take the tensors (by checkpoint name) for computing in `dtype` on `device`.  `weights` is a dict of
        tensors, or a checkpoint that uploads on demand (`weights.loader.open_upload`).

        Matrices are used in the compute type: a bfloat16 checkpoint widens exactly for
        the 32-bit path; a 32-bit matrix is rounded to bfloat16 for a bfloat16 engine, with
        one line on stderr saying so.  Scale vectors are always read as float32."""
        from ..weights.upload import TensorDict
        if isinstance(weights, dict):
            weights = TensorDict(weights, self.weight_specs(), dtype, device, self._warn_rounding)
        p = self.plan
        self.dtype, self.device = dtype, torch.device(device)
        self.embedding.bind(weights, p.embedding_prefix, dtype, device)
        self.final_norm.bind(weights, self.final_norm_name, dtype, device)
        for part, name in self.stream_steps.values():
            part.bind(weights, name, dtype, device)
        self.head.bind(weights, p.head_prefix, dtype, device)
        for spec, block in zip(p.layers, self.blocks):
            block.bind(weights, spec.prefix, dtype, device)

    def _warn_rounding(self, name: str) -> None:
        if not self._warned_rounding:
            self._warned_rounding = True
            print(f"[qwen3_b200] {name} (and other matrices) are stored in 32-bit and are rounded to bfloat16 "
                  f"for the bfloat16 kernels; use dtype float32 to compute with them as stored", file=sys.stderr)

    # -- cache
    def cache_needs(self) -> List[Optional[CacheNeed]]:
        """What every cache of the plan holds, by cache number: a layer's own, and the further ones of layers
        that keep one cache per run."""
        needs = []
        for owner in self.plan.cache_owners():
            if owner is None or self.plan.layers[owner].cache_from is not None:
                needs.append(None)
            else:
                need = self.blocks[owner].mixer.cache_need()
                extra = int(getattr(self.blocks[owner], "state_size", 0) or 0)     # what the block itself keeps per sequence
                needs.append(dataclasses.replace(need, block_state=extra) if extra else need)
        return needs

    def cache_sources(self) -> Dict[int, int]:
        return {i: spec.cache_from for i, spec in enumerate(self.plan.layers) if spec.cache_from is not None}

    # -- one step over packed tokens
    def forward(self, ctx, cache) -> Optional[torch.Tensor]:
        """Runs the step's tokens through every layer (filling the cache); returns float32
        logits [n_want, vocab] for the wanted rows, or None if none is wanted."""
        N, H = ctx.n_tokens, self.plan.hidden_size
        stream_dtype = self.residual_dtype or ctx.dtype
        residual = ctx.scratch.get("model.residual", (N, self.plan.streams * H), stream_dtype)
        self.embedding.forward(ctx.token_ids[:N], residual)
        x0 = None
        if self.stream_steps:                              # the embedding's output is read again later: keep it
            x0 = residual
            if 0 not in self.stream_steps:                 # the first layers work on a copy
                residual = ctx.scratch.get("model.residual_copy", (N, H), stream_dtype)
                residual.copy_(x0)
        delta = None
        for run, index in enumerate(self.plan.order):
            step = self.stream_steps.get(run)
            if step is not None:
                residual, delta = step[0].forward(residual, delta, x0, ctx)
            residual, delta = self.blocks[index].forward(residual, delta, ctx, cache.layer(self.plan.cache_of_run(run)))
            if self.after_run is not None:
                self.after_run(run, residual, delta, ctx)
        if ctx.n_want == 0:
            return None
        R = ctx.n_want
        normed = ctx.scratch.get("model.rows_normed", (R, H), ctx.dtype)
        finish = getattr(self.blocks[self.plan.order[-1]], "finish", None)
        if finish is not None:                             # the block knows how its hidden state travels
            finish(residual, delta, self.final_norm, ctx, normed)
        elif self.residual_dtype is not None:                # a float32 stream: its pending sum and norms have kernels of their own
            from .block import settle
            if ctx.want_all:
                settle(residual, delta, self.final_norm, normed)
            else:
                settle(residual, delta)
                ops.gather_rows_norm(residual, ctx.want_rows[:R], self.final_norm.weight, self.final_norm.eps, normed)
        elif ctx.want_all:                                 # a decode step: the last residual sum rides in the norm
            self.final_norm(residual, normed, delta)
        else:
            rows = ctx.scratch.get("model.rows", (R, H), ctx.dtype)
            ops.gather_rows(residual, ctx.want_rows[:R], rows, delta)
            self.final_norm(rows, normed)
        logits = ctx.scratch.get("model.logits", (R, self.plan.vocab_size), torch.float32)
        return self.head.forward(normed, logits)


def build_model(plan: ModelPlan) -> Model:
    return Model(plan)
