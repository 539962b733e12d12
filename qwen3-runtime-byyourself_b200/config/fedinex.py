"""Typed configuration of the Fedinex decoder, read from its config.json.

A Fedinex model is a list of pre-norm layers on a float32 hidden state, x += mixer(norm1(x)) and then
x += ff(norm2(x)) with RMS norms; each layer has one of three mixers and a dense or a routed feed-forward (or none).
What the file gives, key by key:

  architecture        "Fedinex"
  vocab, width        sizes of the embedding table and of the hidden state
  norm.eps            eps of every RMS norm (inside the root)
  layers[i].type      "gla": mixer {heads, dim, vdim, tau}: gated linear attention, a decay per key channel
                      sigmoid(z)^(1/tau) from a low-rank projection, a float32 state per sequence (the projection's rank
                      is the checkpoint's; an optional key `rank` states it for a model with random weights)
                      "attention": mixer {heads, kv_heads, dim, vdim, scale, rot {base, dims}, mask {size, keep_first},
                      v_mix}: grouped-query attention with biases, rotation of pairs (i, i + dims/2), a sliding window
                      that keeps the first tokens, and values blended with those of the first layer that says v_mix
                      "parallel": mixer {left {...}, right {...}, left_scale, right_scale}: two mixers that read the same
                      input; left {heads, kv_heads, dim, vdim, scale, rot {base, dims}, conv}: attention over every
                      earlier key with a short causal convolution on q, k and v, rotation of pairs (2i, 2i + 1) and a
                      sigmoid gate per head; right {heads, dim, vdim, gate_cap}: a matrix memory with exponential gates
  layers[i].mlp       {kind "dense", ff, limit} | {kind "moe", expert {ff, limit}, router {experts, top, scale,
                      groups {count, keep}}} | null

Optional keys (`mlp`, `mask`, `mask.keep_first`, `rot`, `conv`, `v_mix`, `router.groups`) may be null or absent: the
mechanism is then not there.  The file has no bound on positions and no stop tokens.  `plan()` states the model as data
for the parts, the cache and the step function.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List

from .dozazen import MAX_POSITIONS, _get, _opt
from .plan import LayerSpec, ModelPlan, PartSpec
from .registry import ConfigError, register_architecture

MAX_ROUTER = 1022              # what the router kernel takes
SIGMOID_ALPHA = 1.702          # the design's gated activation: g sigmoid(1.702 g) (u + 1)
NORMALIZER_FLOOR = 1e-6        # added to the matrix memory's divisor


@dataclass(frozen=True)
class FedinexConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: List[Dict[str, Any]]            # as in the file, checked
    torch_dtype: str = "bfloat16"

    architecture = "Fedinex"

    @classmethod
    def from_dict(cls, root: dict) -> "FedinexConfig":
        if not isinstance(root, dict):
            raise ConfigError("model config root must be a JSON object")
        name = root.get("architecture", (root.get("architectures") or [None])[0])
        if name != cls.architecture:
            raise ConfigError(f"only {cls.architecture} is read by this class, not {name!r}")
        layers = root.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config field 'layers' must be a non-empty array")
        config = cls(
            vocab=_get(root, "vocab", int),
            width=_get(root, "width", int),
            norm_eps=_get(_get(root, "norm", dict), "eps", float, "norm."),
            layers=copy.deepcopy(layers),
            torch_dtype=_opt(root, "torch_dtype", str) or "bfloat16",
        )
        config.validate()
        return config

    # -- checks
    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("vocab and width must be positive")
        if not self.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        if self.torch_dtype not in ("bfloat16", "float32"):
            raise ConfigError("torch_dtype is bfloat16 or float32")
        mixed_width = None
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            if not isinstance(layer, dict):
                raise ConfigError(f"{where[:-1]} must be an object")
            kind = _get(layer, "type", str, where)
            m, w = _get(layer, "mixer", dict, where), where + "mixer."
            if kind == "gla":
                self._check_heads(m, w)
                if not _get(m, "tau", float, w) > 0:
                    raise ConfigError(f"{w}tau must be positive")
                rank = _opt(m, "rank", int, w)
                if rank is not None and rank <= 0:
                    raise ConfigError(f"{w}rank must be positive")
            elif kind == "attention":
                self._check_attention(m, w)
                if _opt(m, "v_mix", bool, w):
                    width = (m["kv_heads"], m["vdim"])
                    if mixed_width not in (None, width):
                        raise ConfigError(f"{w}v_mix: every layer that blends values has (kv_heads, vdim) = {mixed_width}")
                    mixed_width = width
            elif kind == "parallel":
                self._check_attention(_get(m, "left", dict, w), w + "left.")
                conv = _opt(m["left"], "conv", int, w + "left.")
                if conv is not None and not 1 <= conv <= 16:
                    raise ConfigError(f"{w}left.conv: 1 to 16 taps")
                right = _get(m, "right", dict, w)
                self._check_heads(right, w + "right.")
                if not _get(right, "gate_cap", float, w + "right.") > 0:
                    raise ConfigError(f"{w}right.gate_cap must be positive")
                _get(m, "left_scale", float, w)
                _get(m, "right_scale", float, w)
            else:
                raise ConfigError(f"{where}type: 'gla', 'attention' or 'parallel', not {kind!r}")
            mlp = _opt(layer, "mlp", dict, where)
            if mlp is not None:
                self._check_mlp(mlp, where + "mlp.")

    @staticmethod
    def _check_heads(m: dict, w: str) -> None:
        heads, dim, vdim = _get(m, "heads", int, w), _get(m, "dim", int, w), _get(m, "vdim", int, w)
        if heads <= 0 or not 0 < dim <= 256 or not 0 < vdim <= 255:
            raise ConfigError(f"{w}heads must be positive, dim up to 256 and vdim up to 255 (what the recurrence runs)")

    @staticmethod
    def _check_attention(m: dict, w: str) -> None:
        heads, kv = _get(m, "heads", int, w), _get(m, "kv_heads", int, w)
        dim, vdim = _get(m, "dim", int, w), _get(m, "vdim", int, w)
        if heads <= 0 or kv <= 0 or heads % kv or not 0 < dim <= 256 or not 0 < vdim <= 256:
            raise ConfigError(f"{w}heads must be a multiple of kv_heads, dim and vdim up to 256")
        if not _get(m, "scale", float, w) > 0:
            raise ConfigError(f"{w}scale must be positive")
        rot = _opt(m, "rot", dict, w)
        if rot is not None:
            dims = _get(rot, "dims", int, w + "rot.")
            if dims < 0 or dims % 2 or dims > dim:
                raise ConfigError(f"{w}rot.dims must be even and at most dim")
            if _get(rot, "base", float, w + "rot.") <= 0:
                raise ConfigError(f"{w}rot.base must be positive")
        mask = _opt(m, "mask", dict, w)
        if mask is not None:
            if _get(mask, "size", int, w + "mask.") <= 0:
                raise ConfigError(f"{w}mask.size must be positive")
            if (_opt(mask, "keep_first", int, w + "mask.") or 0) < 0:
                raise ConfigError(f"{w}mask.keep_first must not be negative")

    @staticmethod
    def _check_mlp(mlp: dict, where: str) -> None:
        kind = _get(mlp, "kind", str, where)
        if kind == "dense":
            if _get(mlp, "ff", int, where) <= 0 or not _get(mlp, "limit", float, where) > 0:
                raise ConfigError(f"{where}ff and limit must be positive")
            return
        if kind != "moe":
            raise ConfigError(f"{where}kind: 'dense' or 'moe', not {kind!r}")
        expert = _get(mlp, "expert", dict, where)
        if _get(expert, "ff", int, where + "expert.") <= 0 or not _get(expert, "limit", float, where + "expert.") > 0:
            raise ConfigError(f"{where}expert.ff and expert.limit must be positive")
        r, w = _get(mlp, "router", dict, where), where + "router."
        experts, top = _get(r, "experts", int, w), _get(r, "top", int, w)
        if not 0 < top <= experts or experts > MAX_ROUTER:
            raise ConfigError(f"{w}needs 0 < top <= experts <= {MAX_ROUTER}")
        _get(r, "scale", float, w)
        groups = _opt(r, "groups", dict, w)
        if groups is not None:
            count, keep = _get(groups, "count", int, w + "groups."), _get(groups, "keep", int, w + "groups.")
            if count <= 0 or experts % count or not 0 < keep <= count or keep * (experts // count) < top:
                raise ConfigError(f"{w}groups: count divides experts, 0 < keep <= count, and the kept groups hold top experts")

    def to_dict(self) -> dict:
        """The keys of a config.json that `from_dict` reads back to an equal object."""
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "layers": copy.deepcopy(self.layers), "torch_dtype": self.torch_dtype}

    # -- the model as data
    def _attention_spec(self, m: dict, prefix: str, interleaved: bool, bias: bool, share=None) -> PartSpec:
        rot, mask = m.get("rot") or {}, m.get("mask") or {}
        position = None
        if rot.get("dims"):
            position = PartSpec("rope", {"head_dim": m["dim"], "theta": float(rot["base"]), "max_positions": MAX_POSITIONS,
                                         "rotary_dim": rot["dims"], "interleaved": interleaved, "theta_float32": False})
        names = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "o_bias": "o.b",
                 "value_mix": "vmix", "head_gate": "g", "conv_suffix": ".conv"}
        return PartSpec("gqa_attention", {
            "hidden_size": self.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "value_dim": m["vdim"], "scale": float(m["scale"]), "position": position, "window": mask.get("size"),
            "keep_first": mask.get("keep_first") or 0, "bias": bias, "out_bias": bias, "value_mix": share,
            "conv_taps": m.get("conv") or 0, "head_gate": not bias, "prefix": prefix, "names": names})

    def plan(self) -> ModelPlan:
        H, eps = self.width, self.norm_eps
        norm = PartSpec("rms_norm", {"size": H, "eps": eps})
        layers, first_mix = [], None
        for i, layer in enumerate(self.layers):
            m = layer["mixer"]
            if layer["type"] == "gla":
                mixer = PartSpec("gated_linear_attention", {
                    "hidden_size": H, "num_heads": m["heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
                    "tau": float(m["tau"]), "eps": eps, "prefix": "mix.", "decay_rank": m.get("rank")})
            elif layer["type"] == "attention":
                share = None
                if m.get("v_mix"):
                    share = "first" if first_mix is None else "blend"
                    first_mix = i if first_mix is None else first_mix
                mixer = self._attention_spec(m, "mix.", interleaved=False, bias=True, share=share)
            else:
                r = m["right"]
                right = PartSpec("matrix_memory", {
                    "hidden_size": H, "num_heads": r["heads"], "head_dim": r["dim"], "value_dim": r["vdim"],
                    "gate_cap": float(r["gate_cap"]), "eps": eps, "floor": NORMALIZER_FLOOR, "prefix": "mix.right."})
                mixer = PartSpec("parallel_mixers", {
                    "hidden_size": H, "mixers": [self._attention_spec(m["left"], "mix.left.", interleaved=True, bias=False), right],
                    "scales": [float(m["left_scale"]), float(m["right_scale"])]})
            feed_forward, mlp = None, layer.get("mlp")
            if mlp is not None and mlp["kind"] == "dense":
                feed_forward = PartSpec("gated_mlp", {
                    "hidden_size": H, "intermediate_size": mlp["ff"], "prefix": "mlp.", "activation": "clamped",
                    "limit": float(mlp["limit"]), "alpha": SIGMOID_ALPHA, "names": {"gate": "gate", "up": "up", "down": "down"}})
            elif mlp is not None:
                r = mlp["router"]
                groups = r.get("groups") or {}
                feed_forward = PartSpec("routed_experts", {
                    "hidden_size": H, "intermediate_size": mlp["expert"]["ff"], "limit": float(mlp["expert"]["limit"]),
                    "alpha": SIGMOID_ALPHA, "experts": r["experts"], "top": r["top"], "scoring": "sigmoid",
                    "group_count": groups.get("count", 1), "group_keep": groups.get("keep", 1), "group_mark": "top2_sum",
                    "weight_scale": float(r["scale"]), "prefix": "mlp."})
            block = PartSpec("hyper_connections", {"norm": norm, "streams": None, "residual_mult": 1.0, "hidden_size": H})
            layers.append(LayerSpec(block=block, mixer=mixer, feed_forward=feed_forward, prefix=f"l{i}."))
        return ModelPlan(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=H, max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": H, "tensor": "", "copies": 1}),
            embedding_prefix="embed", layers=layers, order=list(range(len(layers))), residual_dtype="float32",
            final_norm=norm, final_norm_prefix="final.", final_norm_name="final.norm",
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": H, "tensor": ""}),
            head_prefix="head", stop_token_ids=[],
        )


register_architecture(FedinexConfig.architecture, FedinexConfig)
