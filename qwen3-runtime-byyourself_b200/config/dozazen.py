"""Typed configuration of the Dozazen decoder, read from its config.json.

A Dozazen model is a list of layers, each with an attention mixer of its own sizes and,
optionally, a gated feed-forward; a stretch of the layers can run several times in a row with
the same weights.  What the file gives, key by key:

  architecture        "Dozazen"
  vocab, width        sizes of the embedding table and of the hidden state
  embedding.scale     the embedding's output is multiplied by it
  norm.eps            eps of every RMS norm (inside the root)
  layers[i]           type "attention"; mixer {heads, kv_heads, dim, vdim, scale, softcap,
                      mask {size}, rot {base, dims, scaling {factor, low, high, original}}};
                      mlp {kind "dense", ff} or null
  loop                {start, stop, times}: layers start .. stop-1 run `times` times, each pass
                      with a cache of its own; before the first layer of every pass the hidden
                      state x becomes W [x; x0] (tensor `loop.in`), x0 the embedding's output
  logit_scale, logit_softcap   logits = cap * tanh(head(x) * scale / cap)

The hidden state is kept in float32; every layer has a norm before and after each sublayer.
Optional keys (`loop`, `mask`, `softcap`, `rot`, `rot.scaling`, `logit_softcap`, `mlp`) may
be null or absent: the mechanism is then not there.  The file has no bound on positions and no
stop tokens.  `plan()` states the model as data for the parts, the cache and the step function.
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

from .plan import LayerSpec, ModelPlan, PartSpec, StreamStep
from .registry import ConfigError, register_architecture

MAX_POSITIONS = 1 << 24        # the file bounds no sequence; the cache's capacity does


def _get(root: dict, key: str, kind, where: str = ""):
    if not isinstance(root, dict) or key not in root or root[key] is None:
        raise ConfigError(f"missing required config field '{where}{key}'")
    return _typed(root[key], kind, where + key)


def _opt(root: dict, key: str, kind, where: str = ""):
    if not isinstance(root, dict) or root.get(key) is None:
        return None
    return _typed(root[key], kind, where + key)


def _typed(v, kind, name: str):
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"config field '{name}' must be an integer")
        return v
    if kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(float(v)):
            raise ConfigError(f"config field '{name}' must be a finite number")
        return float(v)
    if kind is dict:
        if not isinstance(v, dict):
            raise ConfigError(f"config field '{name}' must be an object")
        return v
    if kind is str:
        if not isinstance(v, str):
            raise ConfigError(f"config field '{name}' must be a string")
        return v
    if kind is bool:
        if not isinstance(v, bool):
            raise ConfigError(f"config field '{name}' must be true or false")
        return v
    raise TypeError(kind)


@dataclass(frozen=True)
class DozazenConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: List[Dict[str, Any]]            # as in the file, checked
    loop: Optional[Dict[str, int]]
    logit_scale: float
    logit_softcap: Optional[float]
    torch_dtype: str = "bfloat16"

    architecture = "Dozazen"

    @classmethod
    def from_dict(cls, root: dict) -> "DozazenConfig":
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
        embedding = _opt(root, "embedding", dict) or {}
        config = cls(
            vocab=_get(root, "vocab", int),
            width=_get(root, "width", int),
            embedding_scale=_opt(embedding, "scale", float, "embedding.") or 1.0,
            norm_eps=_get(_get(root, "norm", dict), "eps", float, "norm."),
            layers=copy.deepcopy(layers),
            loop=loop,
            logit_scale=_opt(root, "logit_scale", float) or 1.0,
            logit_softcap=_opt(root, "logit_softcap", float),
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
        n = len(self.layers)
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            if not isinstance(layer, dict) or _get(layer, "type", str, where) != "attention":
                raise ConfigError(f"{where}type: only 'attention' layers exist in this architecture")
            m = _get(layer, "mixer", dict, where)
            w = where + "mixer."
            heads, kv, dim = _get(m, "heads", int, w), _get(m, "kv_heads", int, w), _get(m, "dim", int, w)
            vdim = _opt(m, "vdim", int, w) or dim
            if heads <= 0 or kv <= 0 or heads % kv:
                raise ConfigError(f"{w}heads must be a positive multiple of kv_heads")
            if dim <= 0 or dim > 256 or vdim <= 0 or vdim > 256:
                raise ConfigError(f"{w}dim {dim}, vdim {vdim}: this library runs head sizes up to 256")
            _get(m, "scale", float, w)
            cap = _opt(m, "softcap", float, w)
            if cap is not None and cap <= 0:
                raise ConfigError(f"{w}softcap must be positive")
            mask = _opt(m, "mask", dict, w)
            if mask is not None and _get(mask, "size", int, w + "mask.") <= 0:
                raise ConfigError(f"{w}mask.size must be positive")
            rot = _opt(m, "rot", dict, w)
            if rot is not None:
                dims = _get(rot, "dims", int, w + "rot.")
                if dims <= 0 or dims % 2 or dims > dim:
                    raise ConfigError(f"{w}rot.dims must be even and at most dim")
                if _get(rot, "base", float, w + "rot.") <= 0:
                    raise ConfigError(f"{w}rot.base must be positive")
                sc = _opt(rot, "scaling", dict, w + "rot.")
                if sc is not None:
                    values = [_get(sc, k, float, w + "rot.scaling.") for k in ("factor", "low", "high", "original")]
                    if min(values) <= 0 or values[1] == values[2]:
                        raise ConfigError(f"{w}rot.scaling needs positive values and low != high")
            mlp = _opt(layer, "mlp", dict, where)
            if mlp is not None:
                if _get(mlp, "kind", str, where + "mlp.") != "dense":
                    raise ConfigError(f"{where}mlp.kind: only 'dense' feed-forwards exist in this architecture")
                if _get(mlp, "ff", int, where + "mlp.") <= 0:
                    raise ConfigError(f"{where}mlp.ff must be positive")
        if self.loop is not None:
            start, stop, times = self.loop["start"], self.loop["stop"], self.loop["times"]
            if not (0 <= start < stop <= n) or times < 1:
                raise ConfigError("loop needs 0 <= start < stop <= number of layers and times >= 1")
        if self.logit_softcap is not None and self.logit_softcap <= 0:
            raise ConfigError("logit_softcap must be positive")

    def to_dict(self) -> dict:
        """The keys of a config.json that `from_dict` reads back to an equal object."""
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
                "layers": copy.deepcopy(self.layers), "loop": dict(self.loop) if self.loop else None,
                "logit_scale": self.logit_scale, "logit_softcap": self.logit_softcap, "torch_dtype": self.torch_dtype}

    # -- the model as data
    def plan(self) -> ModelPlan:
        H = self.width
        norm = PartSpec("rms_norm", {"size": H, "eps": self.norm_eps})
        block = PartSpec("sandwich_norm", {"norm": norm, "names": ("norm1", "norm1b", "norm2", "norm2b")})
        layers = []
        for i, layer in enumerate(self.layers):
            m = layer["mixer"]
            rot, position = m.get("rot"), None
            if rot is not None:
                position = PartSpec("rope", {"head_dim": m["dim"], "theta": float(rot["base"]), "max_positions": MAX_POSITIONS,
                                             "rotary_dim": rot["dims"], "interleaved": True,
                                             "scaling": dict(rot["scaling"]) if rot.get("scaling") else None})
            mixer = PartSpec("gqa_attention", {
                "hidden_size": H, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                "value_dim": m.get("vdim") or m["dim"], "scale": float(m["scale"]), "position": position,
                "bias": True, "softcap": m.get("softcap"), "chunk": m["mask"]["size"] if m.get("mask") else None,
                "sink": True, "prefix": "mix.",
                "names": {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b"},
            })
            feed_forward = None
            if layer.get("mlp") is not None:
                feed_forward = PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": layer["mlp"]["ff"], "prefix": "mlp.",
                                                      "activation": "gelu_tanh",
                                                      "names": {"gate": "gate", "up": "up", "down": "down"}})
            layers.append(LayerSpec(block=block, mixer=mixer, feed_forward=feed_forward, prefix=f"l{i}."))
        n = len(layers)
        order, caches, steps = list(range(n)), None, []
        if self.loop is not None:
            start, stop, times = self.loop["start"], self.loop["stop"], self.loop["times"]
            order, caches, extra = list(range(start)), list(range(start)), n
            for p in range(times):
                steps.append(StreamStep(len(order), PartSpec("mix_in", {"hidden_size": H}), "loop.in"))
                for i in range(start, stop):
                    order.append(i)
                    caches.append(i if p == 0 else extra)       # a cache of its own for every further pass
                    extra += 0 if p == 0 else 1
            order += list(range(stop, n))
            caches += list(range(stop, n))
        return ModelPlan(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=H, max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": H, "scale": self.embedding_scale,
                                                   "tensor": ""}),
            embedding_prefix="embed", layers=layers, order=order, caches=caches, stream_steps=steps,
            residual_dtype="float32", final_norm=norm, final_norm_prefix="final.", final_norm_name="final.norm",
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": H, "scale": self.logit_scale,
                                      "softcap": self.logit_softcap, "tensor": ""}),
            head_prefix="head", stop_token_ids=[],
        )


register_architecture(DozazenConfig.architecture, DozazenConfig)
