"""Plain float64 restatement of the Fedinex decoder: whole sequences, no cache, no batching, one function
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


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, weight, eps):
    return rms_unit(x, eps) * weight


def product(x, W, rnd=same, bias=None):
    """x @ W.T (+ bias) with the rounding points of a 16-bit product: its input and its output."""
    y = rnd(x) @ W.T
    if bias is not None:
        y = y + bias
    return rnd(y)


# ---------------------------------------------------------------- rotation, short convolution
def rotary(v, positions, base, dims, interleaved):
    """Rotate the first `dims` values of the last axis of v [T, heads, n]: pairs (2i, 2i + 1) if `interleaved`, else
    (i, i + dims/2); the angle of pair i at position p is p * base^(-2i/dims)."""
    half = dims // 2
    freq = np.array([base ** (-2.0 * i / dims) for i in range(half)])
    a = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    c, s = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
    out = v.copy()
    first = slice(0, dims, 2) if interleaved else slice(0, half)
    second = slice(1, dims, 2) if interleaved else slice(half, dims)
    u, t = v[..., first], v[..., second]
    out[..., first] = u * c - t * s
    out[..., second] = t * c + u * s
    return out


def short_conv(u, taps_w):
    """Causal convolution over time on every channel: u [T, C], taps_w [C, taps]; tap j weighs the row taps - 1 - j
    steps back, rows before the sequence are zero."""
    T, C = u.shape
    taps = taps_w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C)), u], axis=0)
    y = np.zeros_like(u)
    for j in range(taps):
        y += padded[j:j + T] * taps_w[:, j][None, :]
    return y


# ---------------------------------------------------------------- softmax attention
def visible(T, window=None, keep_first=0):
    """[T, T] mask: key j is seen from i if j <= i and (no window, or i - j < window, or j < keep_first)."""
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    see = j <= i
    if window is not None:
        see &= (i - j < window) | (j < keep_first)
    return see


def softmax_attention(q, k, v, scale, mask):
    """q [T, H, d], k [T, G, d], v [T, G, vd]; query head h reads key/value head h // (H / G).  Returns [T, H, vd]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = np.where(mask, s, -np.inf)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        p /= p.sum(axis=1, keepdims=True)
        out[:, h] = p @ v[:, g]
    return out


def attention_mixer(h, w, p, m, eps, shared, rnd=same):
    """The 'attention' mixer: biased projections, half-split rotation of the first rot.dims values, a sliding window
    that keeps the first tokens, values blended with those of the first such layer (`shared["v_first"]`)."""
    T = h.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = product(h, w[p + "q"], rnd, w[p + "q.b"]).reshape(T, H, d)
    k = product(h, w[p + "k"], rnd, w[p + "k.b"]).reshape(T, G, d)
    v = product(h, w[p + "v"], rnd, w[p + "v.b"]).reshape(T, G, vd)
    rot = m.get("rot")
    if rot and rot["dims"]:
        q = rotary(q, range(T), rot["base"], rot["dims"], False)
        k = rotary(k, range(T), rot["base"], rot["dims"], False)
    if m.get("v_mix"):
        if "v_first" not in shared:
            shared["v_first"] = v
        else:
            lam = float(w[p + "vmix"])
            v = (1.0 - lam) * v + lam * shared["v_first"]
    mask = m.get("mask")
    see = visible(T, mask["size"], mask.get("keep_first", 0)) if mask else visible(T)
    o = softmax_attention(rnd(q), rnd(k), rnd(v), m["scale"], see)
    return product(o.reshape(T, H * vd), w[p + "o"], rnd, w[p + "o.b"])


def conv_attention(h, w, p, m, rnd=same):
    """The left half of the 'parallel' mixer: projections without biases, a short convolution on every channel of
    q, k and v, interleaved rotation, every earlier key, and one sigmoid gate per head on the output."""
    T = h.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = (product(h, w[p + n], rnd) for n in ("q", "k", "v"))
    if m.get("conv"):
        q, k, v = (rnd(short_conv(t, w[p + n + ".conv"])) for t, n in ((q, "q"), (k, "k"), (v, "v")))
    q, k, v = q.reshape(T, H, d), k.reshape(T, G, d), v.reshape(T, G, vd)
    rot = m.get("rot")
    if rot and rot["dims"]:
        q = rotary(q, range(T), rot["base"], rot["dims"], True)
        k = rotary(k, range(T), rot["base"], rot["dims"], True)
    o = softmax_attention(rnd(q), rnd(k), v, m["scale"], visible(T))
    gate = sigmoid(product(h, w[p + "g"], rnd))                     # [T, H]
    o = o * gate[:, :, None]
    return product(o.reshape(T, H * vd), w[p + "o"], rnd)


# ---------------------------------------------------------------- recurrences
def matrix_memory(h, w, p, m, eps, rnd=same):
    """The right half of the 'parallel' mixer: a matrix memory with exponential gates kept stable by a running
    maximum (which starts at 0), read with a normaliser."""
    T = h.shape[0]
    H, d, vd, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (product(h, w[p + "q"], rnd) * d ** -0.5).reshape(T, H, d)
    k = product(h, w[p + "k"], rnd).reshape(T, H, d)
    v = product(h, w[p + "v"], rnd).reshape(T, H, vd)
    zi = rnd(h) @ w[p + "i"].T + w[p + "i.b"]
    zf = rnd(h) @ w[p + "f"].T + w[p + "f.b"]
    gi = cap * np.tanh(zi / cap)
    gf = log_sigmoid(cap * np.tanh(zf / cap))
    out = np.zeros((T, H, vd))
    for a in range(H):
        S, n, mx = np.zeros((d, vd)), np.zeros(d), 0.0
        for t in range(T):
            m_new = max(gf[t, a] + mx, gi[t, a])
            keep, write = math.exp(gf[t, a] + mx - m_new), math.exp(gi[t, a] - m_new)
            S = keep * S + write * np.outer(k[t, a], v[t, a])
            n = keep * n + write * k[t, a]
            mx = m_new
            out[t, a] = (S.T @ q[t, a]) / (max(abs(n @ q[t, a]), math.exp(-mx)) + 1e-6)
    o = rms_unit(out, eps).reshape(T, H * vd) * w[p + "norm"]
    o = o * sigmoid(product(h, w[p + "g"], rnd))
    return product(o, w[p + "o"], rnd)


def gated_linear_attention(h, w, p, m, eps, rnd=same):
    """The 'gla' mixer: a decay per key channel from a low-rank projection, S_t = diag(alpha_t) S_(t-1) + k_t v_t^T."""
    T = h.shape[0]
    H, d, vd, tau = m["heads"], m["dim"], m["vdim"], m["tau"]
    q = (product(h, w[p + "q"], rnd) * d ** -0.5).reshape(T, H, d)
    k = product(h, w[p + "k"], rnd).reshape(T, H, d)
    v = product(h, w[p + "v"], rnd).reshape(T, H, vd)
    z = rnd(product(h, w[p + "a1"], rnd)) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = np.exp(log_sigmoid(z) / tau).reshape(T, H, d)
    out = np.zeros((T, H, vd))
    for a in range(H):
        S = np.zeros((d, vd))
        for t in range(T):
            S = alpha[t, a][:, None] * S + np.outer(k[t, a], v[t, a])
            out[t, a] = S.T @ q[t, a]
    o = (rms_unit(out, eps) * w[p + "norm"]).reshape(T, H * vd)
    g = product(h, w[p + "g"], rnd)
    o = o * (g * sigmoid(g))
    return product(o, w[p + "o"], rnd)


def parallel_mixer(h, w, p, m, eps, rnd=same):
    left = conv_attention(h, w, p + "left.", m["left"], rnd)
    right = matrix_memory(h, w, p + "right.", m["right"], eps, rnd)
    return m["left_scale"] * left + m["right_scale"] * right


# ---------------------------------------------------------------- feed-forwards
def clamped_glu(h, w, p, limit, rnd=same):
    """down( g sigmoid(1.702 g) (u + 1) ), g = min(gate, limit), u = clamp(up, -limit, limit)."""
    g = np.minimum(product(h, w[p + "gate"], rnd), limit)
    u = np.clip(product(h, w[p + "up"], rnd), -limit, limit)
    return product(g * sigmoid(1.702 * g) * (u + 1.0), w[p + "down"], rnd)


def route(h, w, p, r, rnd=same):
    """For every token the chosen experts and their weights: sigmoid scores; the choice is by score + correction among
    the experts of the best groups (a group's mark: the sum of its two largest choice scores); the weights are the
    plain scores times router.scale."""
    T = h.shape[0]
    E, top = r["experts"], r["top"]
    s = sigmoid(rnd(h) @ w[p + "router"].T)
    choice = s + w[p + "correction"]
    groups = r.get("groups")
    if groups and groups["count"] > 1:
        per = E // groups["count"]
        by_group = choice.reshape(T, groups["count"], per)
        mark = np.sort(by_group, axis=2)[:, :, -2:].sum(axis=2) if per >= 2 else by_group.sum(axis=2)
        kept = np.argsort(-mark, axis=1, kind="stable")[:, :groups["keep"]]
        allowed = np.zeros((T, groups["count"]), dtype=bool)
        np.put_along_axis(allowed, kept, True, axis=1)
        choice = np.where(np.repeat(allowed, per, axis=1), choice, -np.inf)
    ids = np.argsort(-choice, axis=1, kind="stable")[:, :top]
    return ids, np.take_along_axis(s, ids, axis=1) * r["scale"]


def mixture(h, w, p, mlp, rnd=same):
    ids, weights = route(h, w, p, mlp["router"], rnd)
    out = np.zeros_like(h)
    for e in range(mlp["router"]["experts"]):
        rows, which = np.nonzero(ids == e)
        if rows.size:
            out[rows] += weights[rows, which][:, None] * clamped_glu(h[rows], w, f"{p}e{e}.", mlp["expert"]["limit"], rnd)
    return out


def feed_forward(h, w, p, mlp, rnd=same):
    if mlp["kind"] == "dense":
        return clamped_glu(h, w, p, mlp["limit"], rnd)
    return mixture(h, w, p, mlp, rnd)


# ---------------------------------------------------------------- the model
def mixer(h, w, p, layer, eps, shared, rnd=same):
    kind, m = layer["type"], layer["mixer"]
    if kind == "gla":
        return gated_linear_attention(h, w, p, m, eps, rnd)
    if kind == "attention":
        return attention_mixer(h, w, p, m, eps, shared, rnd)
    if kind == "parallel":
        return parallel_mixer(h, w, p, m, eps, rnd)
    raise ValueError(kind)


def hidden_states(cfg, w, tokens, rnd=same):
    """The hidden rows after every layer, [layers, T, width]."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)]
    shared, states = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        x = x + mixer(rms_norm(x, w[p + "norm1"], eps), w, p + "mix.", layer, eps, shared, rnd)
        if layer.get("mlp"):
            x = x + feed_forward(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.", layer["mlp"], rnd)
        states.append(x)
    return np.stack(states)


def forward(cfg, w, tokens, rnd=same):
    """Logits [T, vocab] of one sequence."""
    x = hidden_states(cfg, w, tokens, rnd)[-1]
    return rnd(rms_norm(x, w["final.norm"], cfg["norm"]["eps"])) @ w["head"].T
