"""Shared by the Fedinex tests: small configurations that differ in every size and option, and model folders with
weights lively enough that attention is peaked, decays and gates span their range and the routers decide clearly;
stored in bfloat16 so that the plain implementation reads the same values."""
import copy
import os


def gla(heads, dim, vdim, tau, rank):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}}


def attention(heads, kv_heads, dim, vdim, scale, base=None, dims=None, window=None, keep_first=None, v_mix=False):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if dims:
        m["rot"] = {"base": base, "dims": dims}
    if window is not None:
        m["mask"] = {"size": window}
        if keep_first is not None:
            m["mask"]["keep_first"] = keep_first
    if v_mix:
        m["v_mix"] = True
    return {"type": "attention", "mixer": m}


def parallel(left, right, left_scale, right_scale):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}}


def conv_attention(heads, kv_heads, dim, vdim, scale, base=None, dims=None, conv=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if dims:
        m["rot"] = {"base": base, "dims": dims}
    if conv:
        m["conv"] = conv
    return m


def memory(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(ff, limit, experts, top, scale, groups=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}


def layer(mixer, mlp):
    return dict(copy.deepcopy(mixer), mlp=copy.deepcopy(mlp))


# Every mixer once; a window that is no multiple of a page with several kept keys; values blended over three layers, the
# first of which is not the model's first layer; four taps; values wider than keys in every mixer; three groups of which
# two are kept; a layer without feed-forward.
E_A = {
    "architecture": "Fedinex", "vocab": 211, "width": 64, "norm": {"eps": 1e-6},
    "layers": [layer(gla(3, 8, 12, 8.0, 6), dense(96, 1.2)),
               layer(attention(4, 2, 16, 24, 0.3, 10000.0, 8, window=70, keep_first=5, v_mix=True), moe(40, 1.5, 6, 3, 1.7, groups=(3, 2))),
               layer(parallel(conv_attention(4, 1, 16, 24, 0.2, 500.0, 6, conv=4), memory(3, 8, 12, 6.0), 0.7, 1.1), dense(72, 2.0)),
               layer(attention(2, 2, 32, 24, 0.2, 7e5, 32, window=33, keep_first=1, v_mix=True), None),
               layer(attention(6, 2, 8, 24, 0.4, window=9, keep_first=9, v_mix=True), moe(24, 3.0, 4, 1, 0.5))],
}
# The order the other way round; a window of exactly one page without kept keys; attention without rotation, without
# window and without blended values; a convolution of two taps and one without any; one head everywhere; one expert; one
# group; the whole head rotated.
E_B = {
    "architecture": "Fedinex", "vocab": 128, "width": 96, "norm": {"eps": 1e-5},
    "layers": [layer(parallel(conv_attention(1, 1, 32, 32, 0.18, 250.0, 32, conv=2), memory(1, 64, 48, 10.0), 1.0, 1.0), moe(48, 2.25, 1, 1, 1.0)),
               layer(attention(2, 2, 16, 16, 0.25, window=64), dense(160, 7.0)),
               layer(gla(1, 64, 128, 20.0, 8), moe(32, 1.0, 8, 8, 1.25, groups=(1, 1))),
               layer(parallel(conv_attention(2, 1, 16, 8, 0.25), memory(2, 16, 16, 4.0), -0.5, 2.0), dense(64, 0.8)),
               layer(attention(3, 1, 32, 16, 0.2, 50000.0, 16), moe(64, 2.0, 6, 2, 3.0, groups=(2, 1)))],
}
# Sizes the tensor cores like: head sizes 64 and 128, windows of several pages, a kept stretch longer than a page, a
# state of 128 x 128; groups of four experts.
E_C = {
    "architecture": "Fedinex", "vocab": 320, "width": 128, "norm": {"eps": 1e-5},
    "layers": [layer(attention(4, 2, 64, 64, 0.14, 5e5, 32, window=150, keep_first=70, v_mix=True), moe(64, 1.75, 8, 2, 2.0, groups=(2, 1))),
               layer(gla(2, 128, 128, 12.0, 24), dense(256, 1.25)),
               layer(parallel(conv_attention(8, 4, 64, 64, 0.11, 300000.0, 48, conv=3), memory(2, 128, 64, 12.0), 0.8, 0.7), moe(80, 2.5, 8, 4, 3.0, groups=(4, 2))),
               layer(attention(2, 2, 128, 64, 0.09, 10000.0, 128, window=200, keep_first=3, v_mix=True), dense(128, 1.75))],
}
# Sizes that rule out every vector path: a width that is no multiple of 4, odd head sizes and vocabulary; a window of one
# position (a token sees itself and the kept keys only); two rotated values; every expert chosen; pairs of experts as
# groups; five taps.
E_D = {
    "architecture": "Fedinex", "vocab": 97, "width": 50, "norm": {"eps": 1e-5},
    "layers": [layer(gla(3, 5, 9, 3.0, 3), moe(21, 1.0, 4, 4, 1.5, groups=(2, 2))),
               layer(attention(3, 3, 6, 9, 0.3, 100.0, 2, window=1, keep_first=2, v_mix=True), dense(30, 1.4)),
               layer(parallel(conv_attention(2, 1, 5, 7, 0.4, 30.0, 4, conv=5), memory(1, 11, 3, 2.5), 0.3, 1.4), None),
               layer(attention(3, 3, 11, 9, 0.3, 1000.0, 10, window=7, v_mix=True), moe(12, 2.5, 6, 3, 1.0, groups=(3, 2)))],
}
CASES = {"A": E_A, "B": E_B, "C": E_C, "D": E_D}


def case(name, **changes):
    cfg = copy.deepcopy(CASES[name])
    cfg.update(changes)
    return cfg


def lively_weights(specs, seed):
    """{name: bfloat16 tensor}: matrices N(0, 1/fan_in) (routers four times that, so that choices are clear; query and
    key projections twice, so that attention is peaked), the embedding table N(0, 1), norm weights around 1, biases around 0 (the decay's around 2, so that the
    state lives for a while; the matrix memory's forget gate around 3 for the same reason: a memory that one token overwrites
    reads as (k . q) v, whose sign hangs on a rounding where k . q is small), convolution taps around 0.5, blending weights in (0.2, 0.8), corrections N(0, 0.3)."""
    import torch
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name in sorted(specs):
        spec = specs[name]
        draw = torch.randn(spec.shape, generator=gen, dtype=torch.float32)
        tail = name.rsplit(".", 1)[-1]
        if tail == "vmix":
            draw = 0.5 + 0.3 * torch.tanh(draw)
        elif tail == "conv":
            draw = 0.5 * draw
        elif tail == "correction":
            draw = 0.3 * draw
        elif name.endswith(".a2.b"):
            draw = 2.0 + draw
        elif name.endswith(".right.f.b"):
            draw = 3.0 + draw
        elif spec.role == "norm":
            draw = 1.0 + 0.2 * draw
        elif spec.role == "bias":
            draw = 0.2 * draw
        elif tail == "router":
            draw = 4.0 * draw / (spec.shape[-1] ** 0.5)
        elif tail in ("q", "k") and ".mix." in name:
            draw = 2.0 * draw / (spec.shape[-1] ** 0.5)
        elif name != "embed":
            draw = draw / (spec.shape[-1] ** 0.5)
        out[name] = draw
    # a recurrent memory that holds one token (a sequence's first) reads as (k . q) v, and the unit norm that follows keeps
    # its sign only: queries that lean towards their own keys keep k . q away from zero, where a rounding would decide
    for name in out:
        if name.endswith(".q") and name[:-1] + "k" in out and (".right." in name or name[:-1] + "a1" in out):
            out[name] = 0.8 * out[name[:-1] + "k"] + 0.6 * out[name]
    return {name: draw.to(torch.bfloat16) for name, draw in out.items()}


def decide_routers(tensors, seed):
    """Make the SET of chosen experts the same for every token, so that no rounded input can change it, while their
    weights still follow the token: the routers are made small and the corrections put the experts 2 apart in some
    order (a sigmoid's scores lie within 1 of each other).  What a comparison in bfloat16 needs, where a close call would
    otherwise go either way."""
    import torch
    gen = torch.Generator().manual_seed(seed)
    for key in list(tensors):
        if not key.endswith(".mlp.router"):
            continue
        prefix = key[:-len("router")]
        tensors[key] = (tensors[key].float() * 0.25).to(torch.bfloat16)
        n = tensors[key].shape[0]
        tensors[prefix + "correction"] = (2.0 * torch.randperm(n, generator=gen).float() - n).to(torch.bfloat16)
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
