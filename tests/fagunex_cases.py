"""Shared by the Fagunex tests: small configurations that differ in every size and option, and model folders with
weights lively enough that attention is peaked, forget gates span their range, the dynamic-tanh norms bend and the
routers decide clearly; stored in bfloat16 so that the plain implementation reads the same values."""
import copy
import os

import numpy as np


def latent(heads, dim, rot_dim, vdim, rank, scale, base, q_rank=None, mask=None, dims=None):
    """A 'latent_attention' layer (queries through a latent, pairs (2i, 2i + 1), a window, a sink, an output gate)."""
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim if dims is None else dims}}
    if q_rank is not None:
        m["q_rank"] = q_rank
    if mask is not None:
        m["mask"] = {"size": mask}
    return {"type": "latent_attention", "mixer": m}


def latent2(heads, dim, rot_dim, vdim, rank, scale, base, dims=None):
    """A 'latent_attention_2' layer (one query projection, pairs (i, i + dims/2), every earlier key, plain softmax)."""
    out = latent(heads, dim, rot_dim, vdim, rank, scale, base, dims=dims)
    out["type"] = "latent_attention_2"
    return out


def hgrn2(heads, dim, vdim):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}}


def moe(ff, experts, top, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def layer(mixer, mlp):
    return dict(copy.deepcopy(mixer), mlp=copy.deepcopy(mlp))


# A stretch in the middle runs three times; a window that is no multiple of a page; values wider than the plain key part;
# a recurrence whose values are wider than its keys; a layer without feed-forward; a shared expert of another size than
# the routed ones; a token side input of five values.
F_A = {
    "architecture": "Fagunex", "vocab": 211, "width": 64, "norm": {"eps": 1e-6}, "token_side": {"dim": 5},
    "layers": [layer(latent(3, 8, 6, 12, 20, 0.3, 10000.0, q_rank=10, mask=70), moe(40, 5, 2, shared=24)),
               layer(hgrn2(2, 16, 24), moe(24, 4, 1)),
               layer(latent2(2, 16, 8, 8, 24, 0.25, 500.0), None),
               layer(hgrn2(1, 8, 8), moe(16, 3, 3, shared=16))],
    "loop": {"start": 1, "stop": 3, "times": 3},
}
# No loop and no token side input; a window of exactly one page; only part of the rotated values really turns; one head;
# queries without a latent in the windowed kind; a single expert.
F_B = {
    "architecture": "Fagunex", "vocab": 128, "width": 96, "norm": {"eps": 1e-5},
    "layers": [layer(latent(1, 32, 8, 32, 40, 0.18, 250.0, mask=64, dims=4), moe(48, 1, 1, shared=48)),
               layer(hgrn2(1, 64, 128), moe(32, 6, 2)),
               layer(latent2(4, 8, 4, 16, 16, 0.35, 1e6, dims=2), moe(48, 4, 2, shared=8))],
}
# Sizes the tensor cores like (cache rows of 128 and 96 values, latents of 112 and 64); a window of several pages; all layers
# run twice; a state of 128 x 128.
F_C = {
    "architecture": "Fagunex", "vocab": 320, "width": 128, "norm": {"eps": 1e-5}, "token_side": {"dim": 16},
    "layers": [layer(latent(4, 32, 16, 32, 112, 0.15, 10000.0, q_rank=48, mask=200), moe(64, 8, 4, shared=64)),
               layer(hgrn2(2, 128, 128), moe(64, 8, 2)),
               layer(latent2(8, 16, 32, 16, 64, 0.14, 50000.0), moe(32, 4, 2, shared=96))],
    "loop": {"start": 0, "stop": 3, "times": 2},
}
# Sizes that rule out every vector path: a width that is no multiple of 4, odd head sizes and vocabulary; windows of one
# position (a token sees itself and the sink only) and of seven; two rotated values; every expert chosen; a loop of one
# layer that runs once (no loop at all, said another way); a side input of one value.
F_D = {
    "architecture": "Fagunex", "vocab": 97, "width": 50, "norm": {"eps": 1e-5}, "token_side": {"dim": 1},
    "layers": [layer(latent(2, 5, 2, 7, 13, 0.4, 100.0, q_rank=3, mask=7), moe(30, 3, 3, shared=10)),
               layer(hgrn2(3, 5, 9), moe(21, 2, 1)),
               layer(latent(3, 6, 4, 9, 11, 0.3, 10000.0, mask=1), None),
               layer(latent2(1, 11, 2, 3, 9, 0.3, 30.0), moe(12, 5, 4, shared=7))],
    "loop": {"start": 1, "stop": 2, "times": 1},
}
CASES = {"A": F_A, "B": F_B, "C": F_C, "D": F_D}


def case(name, **changes):
    cfg = copy.deepcopy(CASES[name])
    cfg.update(changes)
    return cfg


def lively_weights(specs, seed):
    """{name: bfloat16 tensor}: matrices N(0, 1/fan_in) (routers four times that, so that choices are clear; query and
    key projections twice, so that attention is peaked), embedding tables N(0, 1), norm weights around 1, the dynamic-tanh
    slopes between 0.5 and 1.5 with offsets around 0, shifts and the gates' lower bounds spread over [0, 0.9], sinks N(0, 1)."""
    import torch
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name in sorted(specs):
        spec = specs[name]
        draw = torch.randn(spec.shape, generator=gen, dtype=torch.float32)
        tail = name.rsplit(".", 1)[-1]
        if tail == "alpha":
            draw = 1.0 + 0.5 * torch.tanh(draw)
        elif tail in ("shift", "lower"):
            draw = 0.9 * torch.rand(spec.shape, generator=gen)
        elif tail == "sink":
            draw = draw
        elif spec.role == "norm":
            draw = 1.0 + 0.2 * draw
        elif spec.role == "bias":
            draw = 0.2 * draw
        elif tail == "router":
            draw = 4.0 * draw / (spec.shape[-1] ** 0.5)
        elif tail in ("q", "uq", "uk", "dkv") and ".mix." in name:
            draw = 2.0 * draw / (spec.shape[-1] ** 0.5)
        elif name not in ("embed", "side.embed"):
            draw = draw / (spec.shape[-1] ** 0.5)
        out[name] = draw.to(torch.bfloat16)
    return out


def decide_routers(tensors, seed):
    """Make the SET of chosen experts the same for every token, so that no rounded input can change it, while their
    weights still follow the token: the first value of the feed-forward's input is made the constant 1 (its norm's weight
    0, its offset 1), the routers' first column puts the experts 2 apart in some order, and the rest of the router is
    made small.  What a comparison in bfloat16 needs, where a close call would otherwise go either way."""
    import torch
    gen = torch.Generator().manual_seed(seed)
    for key in list(tensors):
        if not key.endswith(".mlp.router"):
            continue
        prefix = key[:-len("mlp.router")]
        w = tensors[key].float() * 0.08
        n = w.shape[0]
        w[:, 0] = 2.0 * torch.randperm(n, generator=gen).float() - n
        tensors[key] = w.to(torch.bfloat16)
        tensors[prefix + "norm2"][0] = 0.0
        tensors[prefix + "norm2.b"][0] = 1.0
    return tensors


def make_folder(tmp_path, cfg, seed, name="model", tensors=None, decided=False):
    """Write a model folder; returns (folder, weights as float64 NumPy arrays by name)."""
    import torch
    import qwen3_b200 as q
    config = q.config_from_dict(cfg)
    if tensors is None:
        tensors = lively_weights(q.build_model(config.plan()).weight_specs(), seed)
    if decided:
        tensors = decide_routers(tensors, seed + 1)
    folder = os.path.join(str(tmp_path), name)
    q.write_model_folder(folder, config, tensors)
    return folder, {k: v.to(torch.float64).numpy() for k, v in tensors.items()}


def random_tokens(rng, n, vocab):
    return [int(t) for t in rng.integers(0, vocab, size=n)]
