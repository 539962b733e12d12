"""A routed feed-forward (mixture of experts) as a part.

Router: logits z = W_r x in 32-bit, scores s = softmax(z) over all router outputs; the choice is made on
s + correction (a stored vector), among the experts of the `group_keep` best of `group_count` equal groups of
neighbours (a group's score: its best choice score); the `top` best are chosen and weighted by their plain
scores s, not renormalised.  The last `identity` router outputs are experts without tensors whose output is the
input itself.  An expert: g = min(W_gate x, limit), u = clamp(W_up x, -limit, limit), W_down (g sigmoid(alpha g) (u + 1)).

Options beside that form.  `scoring="sigmoid"`: s = sigmoid(z), every output by itself.  `group_mark="top2_sum"`: a group's
score is the sum of its two best choice scores.  `weight_scale`: the weights are multiplied by it.  `scoring="top_logits"`: the `top` largest logits are chosen and weighted by the softmax over
the chosen logits alone (no correction vector).  `expert_activation="silu"`: an expert is W_down (SiLU(W_gate x) * (W_up x)),
without limit.  `shared_size`: one more expert of that inner size (`shared.gate / up / down`) that every token uses; its
output is multiplied by sigmoid(w_sg . x), one number per token (`shared.sg`, computed with the router's logits), and added.

Nothing on the host depends on how many tokens an expert gets: the pairs (token, choice) are laid out expert by
expert on the device and the experts' products walk that layout, so a decode step with this part can be captured.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from ..weights.loader import WeightSpec
from ..weights.upload import fuse_rows
from .base import Part, register_part

SIGMOID_ALPHA = 1.702


class RoutedExperts(Part):
    def __init__(self, hidden_size: int, intermediate_size: int, experts: int, top: int, limit: float = float("inf"), identity: int = 0,
                 group_count: int = 1, group_keep: int = 1, prefix: str = "", alpha: float = SIGMOID_ALPHA,
                 names: Optional[dict] = None, scoring: str = "softmax_all", expert_activation: str = "clamped",
                 shared_size: Optional[int] = None, group_mark: str = "best", weight_scale: float = 1.0):
        outputs = experts + identity
        if not 0 < top <= outputs or outputs % group_count or not 0 < group_keep <= group_count \
                or group_keep * (outputs // group_count) < top:
            raise ValueError("routed experts: 0 < top <= experts + identity, groups divide them, the kept groups hold top experts")
        if scoring not in ("softmax_all", "top_logits", "sigmoid") or expert_activation not in ("clamped", "silu"):
            raise ValueError("routed experts: scoring 'softmax_all', 'sigmoid' or 'top_logits', expert_activation 'clamped' or 'silu'")
        if scoring == "top_logits" and (group_count != 1 or weight_scale != 1.0):
            raise ValueError("routed experts: groups and a weight scale go with scoring 'softmax_all' or 'sigmoid'")
        if group_mark not in ("best", "top2_sum"):
            raise ValueError("routed experts: group_mark 'best' or 'top2_sum'")
        self.group_mark, self.weight_scale = group_mark, float(weight_scale)
        self.scoring, self.expert_activation = scoring, expert_activation
        self.shared_size = int(shared_size) if shared_size else None
        self.hidden_size, self.intermediate_size, self.prefix = int(hidden_size), int(intermediate_size), prefix
        self.experts, self.identity, self.top = int(experts), int(identity), int(top)
        self.limit, self.alpha, self.up_offset = float(limit), float(alpha), 1.0
        if expert_activation == "silu":
            self.limit, self.alpha, self.up_offset = float("inf"), 1.0, 0.0
        self.group_count, self.group_keep = int(group_count), int(group_keep)
        self.names = dict({"router": "router", "correction": "correction", "expert": "e{}.", "gate": "gate", "up": "up",
                           "down": "down", "shared": "shared.", "shared_gate": "shared.sg"}, **(names or {}))
        self.w_router = self.correction = self.w_gate_up = self.w_down = None
        self.shared = None
        if self.shared_size:
            from .mlp import SwiGLU
            self.shared = SwiGLU(hidden_size, self.shared_size, prefix=prefix + self.names["shared"],
                                 names={k: self.names[k] for k in ("gate", "up", "down")})

    def _expert(self, p: str, e: int, which: str) -> str:
        return p + self.names["expert"].format(e) + self.names[which]

    def weight_specs(self, prefix: str) -> dict:
        p, H, I = prefix + self.prefix, self.hidden_size, self.intermediate_size
        specs = {p + self.names["router"]: WeightSpec((self.experts + self.identity, H))}
        if self.scoring != "top_logits":
            specs[p + self.names["correction"]] = WeightSpec((self.experts + self.identity,), "bias")
        if self.shared is not None:
            specs[p + self.names["shared_gate"]] = WeightSpec((1, H))
            specs.update(self.shared.weight_specs(prefix))
        for e in range(self.experts):
            specs.update({self._expert(p, e, "gate"): WeightSpec((I, H)), self._expert(p, e, "up"): WeightSpec((I, H)),
                          self._expert(p, e, "down"): WeightSpec((H, I))})
        return specs

    def bind(self, weights: dict, prefix: str, dtype, device) -> None:
        p = prefix + self.prefix
        if self.shared is not None:        # the shared expert's gate is one more row of the router's matrix
            self.w_router = fuse_rows(weights, [p + self.names["router"], p + self.names["shared_gate"]])
            self.shared.bind(weights, prefix, dtype, device)
        else:
            self.w_router = weights.pop(p + self.names["router"]).contiguous()
        if self.scoring != "top_logits":
            self.correction = weights[p + self.names["correction"]].to(device=device, dtype=torch.float32).contiguous()
        if self.experts:
            # [expert, gate rows then up rows, hidden] and [expert, hidden, ff], each one matrix
            self.w_gate_up = fuse_rows(weights, [self._expert(p, e, w) for e in range(self.experts) for w in ("gate", "up")])
            self.w_down = fuse_rows(weights, [self._expert(p, e, "down") for e in range(self.experts)])

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        N, H, I, top = ctx.n_tokens, self.hidden_size, self.intermediate_size, self.top
        P = N * top
        s = ctx.scratch
        top_ids, top_w = s.get("moe.top_ids", (P,), torch.int32), s.get("moe.top_w", (P,), torch.float32)
        id_weight = s.get("moe.id_weight", (N,), torch.float32)
        shared_w = s.get("moe.shared_w", (N,), torch.float32) if self.shared is not None else None
        ops.moe_route(x, self.w_router, self.correction, top_ids, top_w, id_weight, self.experts, top, self.group_count,
                      self.group_keep, by_logit=self.scoring == "top_logits", gate_out=shared_w,
                      sigmoid=self.scoring == "sigmoid", group_pair=self.group_mark == "top2_sum", weight_scale=self.weight_scale)
        offsets = s.get("moe.offsets", (self.experts + 1,), torch.int32)
        slot_of_pair, pair_of_slot = s.get("moe.slot_of_pair", (P,), torch.int32), s.get("moe.pair_of_slot", (P,), torch.int32)
        ops.moe_sort(top_ids, P, self.experts, offsets, slot_of_pair, pair_of_slot)
        y = s.get("moe.y", (P, H), torch.float32)
        if self.experts:
            act = s.get("moe.act", (P, I), ctx.dtype)
            ops.moe_experts(x, self.w_gate_up, self.w_down, offsets, pair_of_slot, act, y, P, self.experts, top, I, self.limit,
                            self.alpha, self.up_offset)
        shared = None
        if self.shared is not None:        # its output lands in "ff.out"; the sum gets a buffer of its own
            shared = self.shared.forward(x, ctx)
        out = s.get("moe.out" if shared is not None else "ff.out", (N, H), ctx.dtype)
        return ops.moe_combine(y, x, slot_of_pair, top_w, id_weight, out, top, shared, shared_w)


register_part("feed_forward", "routed_experts", RoutedExperts)
