"""Plain float64 restatement of the Fagunex decoder: whole sequences, no cache, no batching, one function
per mechanism, NumPy only.  It shares no code with the package and is the oracle of its tests.

Notation: x [T, width] a sequence's hidden rows; W matrices stored [out, in] and applied as x @ W.T;
`cfg` is the dict of a config.json, `w` a dict name -> float64 array.  `rnd` (default: the identity) is applied
to what a 16-bit implementation may round: the input and the output of every matrix product.  The tests take
the deviation it causes as the scale of their bfloat16 tolerance.
"""
from __future__ import annotations

import math

import numpy as np


def same(x):
    return x


def round_bf16(x):
    """Round to the nearest bfloat16 (ties to even), as float64."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32).astype(np.float64).reshape(np.shape(x))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


# ---------------------------------------------------------------- norms, shift, token side input
def dynamic_tanh(x, w, name):
    """The norm without statistics: tanh(alpha x) * weight + b."""
    return np.tanh(float(w[name + ".alpha"]) * x) * w[name] + w[name + ".b"]


def token_shift(h, mu):
    """Every row moves towards the row before it (zeros before the first): h_t + (h_(t-1) - h_t) * mu."""
    before = np.concatenate([np.zeros_like(h[:1]), h[:-1]], axis=0)
    return h + (before - h) * mu


def token_side(x, ids, w, p, index, dim, eps, rnd=same):
    """The per-layer token input: a slice of a second embedding, gated by the hidden state, projected back and
    added with unit rms and a weight."""
    e = w["side.embed"][np.asarray(ids)][:, index * dim:(index + 1) * dim]
    g = gelu_tanh(rnd(rnd(x) @ w[p + "side.gate"].T)) * e
    y = rnd(rnd(g) @ w[p + "side.proj"].T)
    return x + rms_unit(y, eps) * w[p + "side.norm"]


# ---------------------------------------------------------------- rotation
def rotary(v, positions, base, dims, interleaved):
    """Rotate the first `dims` values of the last axis of v [T, ..., n]: pairs (2i, 2i + 1) if `interleaved`, else
    (i, i + dims/2); angle = position * base^(-2i/dims)."""
    half = dims // 2
    freq = np.array([base ** (-2.0 * i / dims) for i in range(half)])
    a = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    shape = (len(positions),) + (1,) * (v.ndim - 2) + (half,)
    c, s = np.cos(a).reshape(shape), np.sin(a).reshape(shape)
    out = v.copy()
    first = slice(0, dims, 2) if interleaved else slice(0, half)
    second = slice(1, dims, 2) if interleaved else slice(half, dims)
    u, t = v[..., first], v[..., second]
    out[..., first] = u * c - t * s
    out[..., second] = t * c + u * s
    return out


# ---------------------------------------------------------------- mixers
def hgrn2_mixer(h, w, p, m, eps, rnd=same):
    """Linear attention whose forget gate also decides what is written: per head S_t = diag(f_t) S_(t-1) +
    (1 - f_t) v_t^T, o_t = S_t^T q_t; every head's o gets unit rms over its values and a weight."""
    T = h.shape[0]
    H, d, vd = m["heads"], m["dim"], m["vdim"]
    hr = rnd(h)
    q = silu(rnd(hr @ w[p + "q"].T)).reshape(T, H, d)
    v = rnd(hr @ w[p + "v"].T).reshape(T, H, vd)
    low = w[p + "lower"]
    f = (low + (1.0 - low) * sigmoid(rnd(hr @ w[p + "f"].T) + w[p + "f.b"])).reshape(T, H, d)
    S = np.zeros((H, d, vd))
    o = np.zeros((T, H, vd))
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hdv,hd->hv", S, q[t])
    o = rms_unit(o, eps) * w[p + "norm"]
    return rnd(rnd(o.reshape(T, H * vd)) @ w[p + "o"].T)


def masked_softmax_attention(q, k, v, scale, window=None, sink=None):
    """q [T, H, n], k [T, H, n], v [T, H, vd]: position i sees j <= i (and i - j < window); `sink` [H] adds
    exp(sink_h) to the denominator of head h."""
    T, H, _ = q.shape
    out = np.zeros((T, H, v.shape[-1]))
    for i in range(T):
        lo = 0 if window is None else max(0, i - window + 1)
        for hd in range(H):
            s = (k[lo:i + 1, hd] @ q[i, hd]) * scale
            top = max(s.max(), sink[hd]) if sink is not None else s.max()
            e = np.exp(s - top)
            den = e.sum() + (math.exp(sink[hd] - top) if sink is not None else 0.0)
            out[i, hd] = (e / den) @ v[lo:i + 1, hd]
    return out


def latent_mixer(h, w, p, m, eps, interleaved, gated, positions=None, rnd=same):
    """Attention whose keys and values are expanded from a small latent per token, with one rotated key part
    that all heads share.  With `q_rank` in `m` the queries go through a latent of their own; `gated`: a sink in
    the softmax and a sigmoid gate on the heads' outputs (the two come together in this design)."""
    T = h.shape[0]
    H, d, r, vd, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    positions = list(range(T)) if positions is None else positions
    hr = rnd(h)
    if m.get("q_rank"):
        cq = rms_unit(rnd(hr @ w[p + "dq"].T), eps) * w[p + "dq.norm"]
        q = rnd(rnd(cq) @ w[p + "uq"].T)
    else:
        q = rnd(hr @ w[p + "q"].T)
    q = q.reshape(T, H, d + r)
    down = rnd(hr @ w[p + "dkv"].T)
    c = rnd(rms_unit(down[:, :rank], eps) * w[p + "dkv.norm"])
    k_rot = down[:, rank:]
    rot = m["rot"]
    q_rot = rotary(q[:, :, d:], positions, rot["base"], rot["dims"], interleaved)
    k_rot = rotary(k_rot, positions, rot["base"], rot["dims"], interleaved)
    k_plain = rnd(c @ w[p + "uk"].T).reshape(T, H, d)
    v = rnd(c @ w[p + "uv"].T).reshape(T, H, vd)
    qq = rnd(np.concatenate([q[:, :, :d], q_rot], axis=-1))
    kk = rnd(np.concatenate([k_plain, np.broadcast_to(k_rot[:, None, :], (T, H, r))], axis=-1))
    window = m["mask"]["size"] if m.get("mask") else None
    sink = w[p + "sink"] if gated else None
    o = masked_softmax_attention(qq, kk, v, m["scale"], window, sink).reshape(T, H * vd)
    if gated:
        o = o * sigmoid(rnd(hr @ w[p + "g"].T))
    return rnd(rnd(o) @ w[p + "o"].T)


# ---------------------------------------------------------------- feed-forward
def gated_expert(h, w, p, rnd=same):
    return rnd(rnd(silu(rnd(h @ w[p + "gate"].T)) * rnd(h @ w[p + "up"].T)) @ w[p + "down"].T)


def router_choice(h, w_router, top):
    """Per row: the `top` largest logits' indices (largest first) and the softmax over those logits only."""
    z = h @ w_router.T
    ids = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    zs = np.take_along_axis(z, ids, axis=-1)
    e = np.exp(zs - zs.max(axis=-1, keepdims=True))
    return ids, e / e.sum(axis=-1, keepdims=True)


def moe(h, w, p, mlp, rnd=same):
    """A mixture of experts: the chosen experts' outputs weighted, plus a shared expert times a sigmoid gate of
    one number per token."""
    hr = rnd(h)
    ids, weights = router_choice(hr, w[p + "router"], mlp["router"]["top"])
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t], weights[t]):
            out[t] += a * gated_expert(hr[t:t + 1], w, f"{p}e{e}.", rnd)[0]
    if mlp.get("shared"):
        out += sigmoid(hr @ w[p + "shared.sg"].T) * gated_expert(hr, w, p + "shared.", rnd)
    return out


# ---------------------------------------------------------------- the model
def runs_of(cfg):
    """The layers in the order in which they run: a stretch may run several times in a row."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    body = list(range(loop["start"], loop["stop"]))
    return list(range(loop["start"])) + body * loop["times"] + list(range(loop["stop"], n))


def layer(x, ids, w, cfg, i, rnd=same):
    spec, eps, p = cfg["layers"][i], cfg["norm"]["eps"], f"l{i}."
    h = token_shift(dynamic_tanh(x, w, p + "norm1"), w[p + "shift"])
    m = spec["mixer"]
    if spec["type"] == "hgrn2":
        y = hgrn2_mixer(h, w, p + "mix.", m, eps, rnd)
    elif spec["type"] == "latent_attention":
        y = latent_mixer(h, w, p + "mix.", m, eps, True, True, rnd=rnd)
    elif spec["type"] == "latent_attention_2":
        y = latent_mixer(h, w, p + "mix.", m, eps, False, False, rnd=rnd)
    else:
        raise ValueError(spec["type"])
    x = x + dynamic_tanh(y, w, p + "norm1b")
    if spec.get("mlp"):
        x = x + dynamic_tanh(moe(dynamic_tanh(x, w, p + "norm2"), w, p + "mlp.", spec["mlp"], rnd), w, p + "norm2b")
    if cfg.get("token_side"):
        x = token_side(x, ids, w, p, i, cfg["token_side"]["dim"], eps, rnd)
    return x


def forward(cfg, w, ids, rnd=same, after_run=None):
    """Logits [T, vocab] of one sequence; `after_run(run, x)` sees the hidden rows after every layer run."""
    x = w["embed"][np.asarray(ids)]
    for run, i in enumerate(runs_of(cfg)):
        x = layer(x, ids, w, cfg, i, rnd)
        if after_run is not None:
            after_run(run, x)
    return rnd(dynamic_tanh(x, w, "final.norm")) @ w["head"].T


def generate_greedy(cfg, w, prompt, n_new):
    """`n_new` tokens after `prompt`, each the best of the whole sequence run again (lowest id among equals)."""
    ids, out = list(prompt), []
    for _ in range(n_new):
        out.append(int(np.argmax(forward(cfg, w, ids)[-1])))
        ids.append(out[-1])
    return out
