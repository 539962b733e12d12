"""Typed configuration of the Fagunex decoder, read from its config.json.

A Fagunex model is a list of layers; each has one of three mixers and, optionally, a mixture of experts with a shared
expert.  Every sublayer stands between two dynamic-tanh norms, the mixer reads a token-shifted input, and after the
feed-forward every layer adds a gated slice of a second embedding of the token.  A stretch of the layers can run several
times in a row with the same weights.  What the file gives, key by key:

  architecture        "Fagunex"
  vocab, width        sizes of the embedding table and of the hidden state
  norm.eps            eps of every RMS norm (inside the root); the layers' own norms are dynamic tanh and do not use it
  token_side.dim      width of a layer's slice of the second embedding `side.embed` [vocab, layers * dim]
  layers[i].type      "hgrn2": mixer {heads, dim, vdim}: linear attention whose forget gate also writes, with a float32
                      state per sequence
                      "latent_attention": mixer {heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, mask {size},
                      rot {base, dims}}: attention over a cached latent, queries through a latent of their own, rotation
                      of pairs (2i, 2i + 1), a sliding window, a learned sink per head, a sigmoid gate on the output
                      "latent_attention_2": mixer {heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims}}: the same
                      cache, one query projection, rotation of pairs (i, i + dims/2), every earlier key, plain softmax
  layers[i].mlp       {kind "moe", expert {ff}, router {experts, top}, shared {ff}} | null
  loop                {start, stop, times}: layers start .. stop-1 run `times` times, each pass with a cache and state
                      of its own

Optional keys (`loop`, `token_side`, `mlp`, `mlp.shared`, `mask`, `q_rank`) may be null or absent: the mechanism is then
not there.  The file has no bound on positions and no stop tokens.  `plan()` states the model as data for the parts, the
cache and the step function.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

from .dozazen import MAX_POSITIONS, _get, _opt
from .plan import LayerSpec, ModelPlan, PartSpec
from .registry import ConfigError, register_architecture

LATENT_TYPES = {"latent_attention": {"interleaved": True, "sink": True, "gate": True},
                "latent_attention_2": {"interleaved": False, "sink": False, "gate": False}}
MAX_KEY_ROW, MAX_LATENT, MAX_ROUTER = 1024, 512, 1022      # what the attention and router kernels take


@dataclass(frozen=True)
class FagunexConfig:
    vocab: int
    width: int
    norm_eps: float
    side_dim: Optional[int]
    layers: List[Dict[str, Any]]            # as in the file, checked
    loop: Optional[Dict[str, int]]
    torch_dtype: str = "bfloat16"

    architecture = "Fagunex"

    @classmethod
    def from_dict(cls, root: dict) -> "FagunexConfig":
        if not isinstance(root, dict):
            raise ConfigError("model config root must be a JSON object")
        name = root.get("architecture", (root.get("architectures") or [None])[0])
        if name != cls.architecture:
            raise ConfigError(f"only {cls.architecture} is read by this class, not {name!r}")
        layers = root.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config field 'layers' must be a non-empty array")
        loop = _opt(root, "loop", dict)
        if loop is not None:
            loop = {k: _get(loop, k, int, "loop.") for k in ("start", "stop", "times")}
        side = _opt(root, "token_side", dict)
        config = cls(
            vocab=_get(root, "vocab", int),
            width=_get(root, "width", int),
            norm_eps=_get(_get(root, "norm", dict), "eps", float, "norm."),
            side_dim=_get(side, "dim", int, "token_side.") if side is not None else None,
            layers=copy.deepcopy(layers),
            loop=loop,
            torch_dtype=_opt(root, "torch_dtype", str) or "bfloat16",
        )
        config.validate()
        return config

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("vocab and width must be positive")
        if not self.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        if self.torch_dtype not in ("bfloat16", "float32"):
            raise ConfigError("torch_dtype is bfloat16 or float32")
        if self.side_dim is not None and self.side_dim <= 0:
            raise ConfigError("token_side.dim must be positive")
        n = len(self.layers)
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            if not isinstance(layer, dict):
                raise ConfigError(f"{where[:-1]} must be an object")
            kind = _get(layer, "type", str, where)
            m, w = _get(layer, "mixer", dict, where), where + "mixer."
            heads, dim, vdim = _get(m, "heads", int, w), _get(m, "dim", int, w), _get(m, "vdim", int, w)
            if heads <= 0 or dim <= 0 or vdim <= 0:
                raise ConfigError(f"{w}heads, dim and vdim must be positive")
            if kind == "hgrn2":
                if dim > 256 or vdim > 256:
                    raise ConfigError(f"{w}dim {dim}, vdim {vdim}: the recurrence runs head sizes up to 256")
            elif kind in LATENT_TYPES:
                self._check_latent(m, w, kind)
            else:
                raise ConfigError(f"{where}type: 'hgrn2', 'latent_attention' or 'latent_attention_2', not {kind!r}")
            mlp = _opt(layer, "mlp", dict, where)
            if mlp is not None:
                self._check_mlp(mlp, where + "mlp.")
        if self.loop is not None:
            start, stop, times = self.loop["start"], self.loop["stop"], self.loop["times"]
            if not (0 <= start < stop <= n) or times < 1:
                raise ConfigError("loop needs 0 <= start < stop <= number of layers and times >= 1")

    @staticmethod
    def _check_latent(m: dict, w: str, kind: str) -> None:
        rank, rot_dim = _get(m, "kv_rank", int, w), _get(m, "rot_dim", int, w)
        if rank <= 0 or rot_dim < 0 or rank > MAX_LATENT or rank + rot_dim > MAX_KEY_ROW:
            raise ConfigError(f"{w}kv_rank up to {MAX_LATENT}, kv_rank + rot_dim up to {MAX_KEY_ROW}")
        if not _get(m, "scale", float, w) > 0:
            raise ConfigError(f"{w}scale must be positive")
        q_rank = _opt(m, "q_rank", int, w)
        if q_rank is not None and q_rank <= 0:
            raise ConfigError(f"{w}q_rank must be positive")
        mask = _opt(m, "mask", dict, w)
        if mask is not None and _get(mask, "size", int, w + "mask.") <= 0:
            raise ConfigError(f"{w}mask.size must be positive")
        if rot_dim:
            rot = _get(m, "rot", dict, w)
            dims = _get(rot, "dims", int, w + "rot.")
            if dims < 0 or dims % 2 or dims > rot_dim:
                raise ConfigError(f"{w}rot.dims must be even and at most rot_dim")
            if _get(rot, "base", float, w + "rot.") <= 0:
                raise ConfigError(f"{w}rot.base must be positive")

    @staticmethod
    def _check_mlp(mlp: dict, where: str) -> None:
        if _get(mlp, "kind", str, where) != "moe":
            raise ConfigError(f"{where}kind: only 'moe' feed-forwards exist in this architecture")
        if _get(_get(mlp, "expert", dict, where), "ff", int, where + "expert.") <= 0:
            raise ConfigError(f"{where}expert.ff must be positive")
        r, w = _get(mlp, "router", dict, where), where + "router."
        experts, top = _get(r, "experts", int, w), _get(r, "top", int, w)
        if not 0 < top <= experts or experts > MAX_ROUTER:
            raise ConfigError(f"{w}needs 0 < top <= experts <= {MAX_ROUTER}")
        shared = _opt(mlp, "shared", dict, where)
        if shared is not None and _get(shared, "ff", int, where + "shared.") <= 0:
            raise ConfigError(f"{where}shared.ff must be positive")

    def to_dict(self) -> dict:
        """The keys of a config.json that `from_dict` reads back to an equal object."""
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "token_side": {"dim": self.side_dim} if self.side_dim is not None else None,
                "layers": copy.deepcopy(self.layers), "loop": dict(self.loop) if self.loop else None,
                "torch_dtype": self.torch_dtype}

    # -- the model as data
    def runs(self) -> List[int]:
        """The layers in the order in which they run."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        start, stop, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))

    def plan(self) -> ModelPlan:
        H, eps = self.width, self.norm_eps
        norm = PartSpec("dynamic_tanh", {"size": H, "eps": eps})
        n = len(self.layers)
        layers = []
        for i, layer in enumerate(self.layers):
            m = layer["mixer"]
            if layer["type"] == "hgrn2":
                mixer = PartSpec("gated_recurrence", {"hidden_size": H, "num_heads": m["heads"], "head_dim": m["dim"],
                                                      "value_dim": m["vdim"], "eps": eps, "prefix": "mix."})
            else:
                options, rot = LATENT_TYPES[layer["type"]], m.get("rot") or {}
                mixer = PartSpec("latent_attention", {
                    "hidden_size": H, "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"],
                    "value_dim": m["vdim"], "kv_rank": m["kv_rank"], "scale": float(m["scale"]), "eps": eps,
                    "theta": float(rot.get("base", 10000.0)), "rot_dims": rot.get("dims", 0) if m["rot_dim"] else 0,
                    "max_positions": MAX_POSITIONS, "q_rank": m.get("q_rank"),
                    "window": m["mask"]["size"] if m.get("mask") else None, "prefix": "mix.", **options})
            feed_forward, mlp = None, layer.get("mlp")
            if mlp is not None:
                feed_forward = PartSpec("routed_experts", {
                    "hidden_size": H, "intermediate_size": mlp["expert"]["ff"], "experts": mlp["router"]["experts"],
                    "top": mlp["router"]["top"], "scoring": "top_logits", "expert_activation": "silu",
                    "shared_size": mlp["shared"]["ff"] if mlp.get("shared") else None, "prefix": "mlp."})
            side = None
            if self.side_dim is not None:
                side = {"table": "side.embed", "vocab": self.vocab, "columns": n * self.side_dim, "dim": self.side_dim,
                        "index": i, "eps": eps, "gate": "side.gate", "proj": "side.proj", "norm": "side.norm"}
            block = PartSpec("shift_sandwich", {"norm": norm, "hidden_size": H, "side": side})
            layers.append(LayerSpec(block=block, mixer=mixer, feed_forward=feed_forward, prefix=f"l{i}."))
        order, caches = list(range(n)), None
        if self.loop is not None:
            start, stop, times = self.loop["start"], self.loop["stop"], self.loop["times"]
            order, caches, extra = list(range(start)), list(range(start)), n
            for p in range(times):
                for i in range(start, stop):
                    order.append(i)
                    caches.append(i if p == 0 else extra)       # a cache and state of its own for every further pass
                    extra += 0 if p == 0 else 1
            order += list(range(stop, n))
            caches += list(range(stop, n))
        return ModelPlan(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=H, max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": H, "tensor": ""}),
            embedding_prefix="embed", layers=layers, order=order, caches=caches, residual_dtype="float32",
            final_norm=norm, final_norm_prefix="final.", final_norm_name="final.norm",
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": H, "tensor": ""}),
            head_prefix="head", stop_token_ids=[],
        )


register_architecture(FagunexConfig.architecture, FagunexConfig)
