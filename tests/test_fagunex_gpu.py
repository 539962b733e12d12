"""Fagunex on the GPU against the plain implementation (tests/plain/fagunex_plain.py): every mechanism alone,
then the engine under every way of cutting requests into steps, in 32-bit and in bfloat16."""
import os

import numpy as np
import pytest

import schedules
from fagunex_cases import CASES, case, hgrn2, latent, latent2, layer, lively_weights, make_folder, random_tokens
from fagunex_cases import moe as moe_spec
from plain import fagunex_plain as plain
from test_engine_gpu import run_steps

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = ["float32", "bfloat16"]
FP32_TOL = 3e-4


def torch_dtype(name):
    import torch
    return {"float32": torch.float32, "bfloat16": torch.bfloat16}[name]


def dev(a, dtype):
    import torch
    return torch.tensor(np.asarray(a), dtype=dtype, device="cuda")


def f64(t):
    return t.double().cpu().numpy()


class Norm:
    """What `ops.settle_norm` reads of a norm part."""

    def __init__(self, kind, size, rng, eps=1e-5):
        import torch
        self.stream_kind, self.eps = kind, eps
        self.weight = dev(1 + 0.3 * rng.standard_normal(size), torch.float32)
        self.b = dev(0.2 * rng.standard_normal(size), torch.float32) if kind == "dynamic_tanh" else None
        self.alpha = float(np.float32(0.5 + rng.random()))

    def plain(self, x):
        if self.stream_kind == "dynamic_tanh":
            return np.tanh(self.alpha * x) * f64(self.weight) + f64(self.b)
        return plain.rms_unit(x, self.eps) * f64(self.weight)


# ============================================================================ mechanisms, one at a time
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("size", [50, 64, 384, 4100])
@pytest.mark.parametrize("post,pre", [("dynamic_tanh", "dynamic_tanh"), ("rms", "dynamic_tanh"), ("dynamic_tanh", "rms")])
def test_stream_settles_a_branch_and_norms_the_sum_in_one_pass(dtype, size, post, pre):
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(size)
    T, N = torch_dtype(dtype), 7
    x = dev(rng.standard_normal((N, size)) * 2, torch.float32)
    y = dev(rng.standard_normal((N, size)) * 1.5, T)
    a, b = Norm(post, size, rng), Norm(pre, size, rng, eps=1e-6)
    xd, yd = f64(x), f64(y)
    settled = xd + a.plain(yd)
    tol = dict(rtol=2e-5, atol=2e-5) if dtype == "float32" else dict(rtol=1e-2, atol=1e-2)
    # a norm of the stream alone: the stream stays as it is; the output may be 32-bit whatever the compute type
    for out_type in (T, torch.float32):
        out = torch.empty((N, size), dtype=out_type, device="cuda")
        ops.settle_norm(x, None, None, b, out, compute_dtype=T)
        assert np.allclose(f64(out), b.plain(xd), **(tol if out_type == T else dict(rtol=2e-5, atol=2e-5)))
    assert np.array_equal(f64(x), xd)
    # the branch, the sum and the next norm in one pass
    s = x.clone()
    out = torch.empty((N, size), dtype=T, device="cuda")
    ops.settle_norm(s, y, a, b, out)
    assert np.allclose(f64(s), settled, rtol=1e-5, atol=1e-5)
    assert np.allclose(f64(out), b.plain(settled), **tol)
    # the sum alone, then its rounding
    s2 = x.clone()
    ops.settle_norm(s2, y, a, None, None)
    assert np.allclose(f64(s2), settled, rtol=1e-5, atol=1e-5)
    s3 = x.clone()
    rounded = torch.empty((N, size), dtype=T, device="cuda")
    ops.settle_norm(s3, y, a, "round", rounded)
    assert np.allclose(f64(rounded), settled, **tol) and np.allclose(f64(s3), settled, rtol=1e-5, atol=1e-5)
    # the tail: chosen rows, nothing written back
    s4 = x.clone()
    rows = torch.tensor([5, 0, 6], dtype=torch.int32, device="cuda")
    tail = torch.empty((3, size), dtype=T, device="cuda")
    ops.settle_norm(s4, y, a, b, tail, rows=rows)
    assert np.allclose(f64(tail), b.plain(settled[[5, 0, 6]]), **tol)
    assert np.array_equal(f64(s4), xd)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("size", [50, 256, 1030])
def test_token_shift_reads_the_row_before_and_keeps_the_last(dtype, size):
    """Unequal sequences in slots in no particular order, three steps: whole prompts, portions, single tokens.  A new
    sequence's first token sees zeros; a step's first token sees the last row of the step before."""
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(size)
    T = torch_dtype(dtype)
    mu = dev(rng.uniform(-0.2, 1.1, size), torch.float32)
    slots, n_slots = [4, 0, 5, 2], 7
    state = torch.zeros((n_slots + 1, size), dtype=torch.float32, device="cuda")
    state[3] = 7.0                                                     # a slot no sequence uses
    history = {s: np.zeros((0, size)) for s in slots}
    for lengths in ([1, 9, 2, 30], [3, 1, 0, 2], [1, 1, 1, 1]):
        live = [(s, n) for s, n in zip(slots, lengths) if n > 0]
        N = sum(n for _, n in live)
        h = dev(rng.standard_normal((N, size)), torch.float32)
        start = np.concatenate([[0], np.cumsum([n for _, n in live])]).astype(np.int32)
        seq = np.concatenate([np.full(n, i) for i, (_, n) in enumerate(live)])
        out = torch.full((N, size), 9.0, dtype=T, device="cuda")
        ops.token_shift(h, mu, state, out, dev(seq, torch.int32), dev(start, torch.int32), dev([s for s, _ in live], torch.int32), N)
        hd = f64(h)
        for i, (slot, n) in enumerate(live):
            before = len(history[slot])
            history[slot] = np.concatenate([history[slot], hd[start[i]:start[i + 1]]])
            want = plain.token_shift(history[slot], f64(mu))[before:]
            assert np.allclose(f64(out)[start[i]:start[i + 1]], want, atol=1e-6 if dtype == "float32" else 3e-2), (slot, lengths)
    final = f64(state)
    for slot in slots:
        assert np.array_equal(final[slot], history[slot][-1])
    assert np.all(final[3] == 7.0) and np.all(final[1] == 0.0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_side_gate_takes_the_layer_s_slice_of_the_second_table(dtype):
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(2)
    T, N, dim, layers, vocab = torch_dtype(dtype), 11, 5, 3, 37
    a = dev(rng.standard_normal((N, dim)) * 2, T)
    table = dev(rng.standard_normal((vocab, layers * dim)), T)
    ids = rng.integers(0, vocab, N)
    for index in range(layers):
        out = torch.empty((N, dim), dtype=T, device="cuda")
        ops.side_gate(a, dev(ids, torch.int32), table, out, index * dim)
        want = plain.gelu_tanh(f64(a)) * f64(table)[ids][:, index * dim:(index + 1) * dim]
        assert np.allclose(f64(out), want, atol=1e-6 if dtype == "float32" else 3e-2)


def plain_scan(q, f, v, state):
    """o [T, vd] and the state after the tokens, from activated q, gates f [T, d], v [T, vd] and a state [d, vd]."""
    out = np.zeros((q.shape[0], v.shape[1]))
    for t in range(q.shape[0]):
        state = f[t][:, None] * state + (1.0 - f[t])[:, None] * v[t][None, :]
        out[t] = state.T @ q[t]
    return out, state


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,d,vd", [(3, 5, 9), (2, 16, 24), (1, 64, 128), (2, 128, 128), (1, 256, 64), (1, 256, 256), (2, 48, 96), (1, 1, 1)])
def test_gated_recurrence_over_unequal_sequences_and_from_its_state(dtype, heads, d, vd):
    """Sequences of unequal length in slots in no particular order, continued in a second and a third step from the state
    the step before left; lengths around the number of tokens that are fetched together; lower bounds of 0 and nearly 1."""
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(d * vd + heads)
    T = torch_dtype(dtype)
    low = rng.uniform(0.0, 0.95, heads * d)
    low[0], low[-1] = 0.0, 0.999
    bias = rng.standard_normal(heads * d)
    slots = [4, 0, 5, 2, 7, 1]
    state = torch.zeros((9, heads, d, vd), dtype=torch.float32, device="cuda")
    state[3] = 7.0
    want_state = {s: np.zeros((heads, d, vd)) for s in slots}
    lowd, biasd = f64(dev(low, torch.float32)), f64(dev(bias, torch.float32))
    for lengths in ([1, 7, 8, 9, 100, 17], [40, 1, 2, 16, 0, 33], [1, 1, 1, 0, 1, 1]):
        live = [(s, n) for s, n in zip(slots, lengths) if n > 0]
        N = sum(n for _, n in live)
        proj = dev(rng.standard_normal((N, heads * (2 * d + vd))) * 1.5, T)
        pd = f64(proj)
        start = np.concatenate([[0], np.cumsum([n for _, n in live])]).astype(np.int32)
        out = torch.full((N, heads * vd), 9.0, dtype=torch.float32, device="cuda")
        ops.gated_scan(proj, state, dev(low, torch.float32), dev(bias, torch.float32), dev(start, torch.int32),
                       dev([s for s, _ in live], torch.int32), out, len(live), heads, d, vd)
        got = f64(out)
        for i, (slot, n) in enumerate(live):
            rows = pd[start[i]:start[i + 1]]
            for h in range(heads):
                ch = slice(h * d, (h + 1) * d)
                q = plain.silu(rows[:, ch])
                f = lowd[ch] + (1 - lowd[ch]) * plain.sigmoid(rows[:, heads * d + h * d:heads * d + (h + 1) * d] + biasd[ch])
                v = rows[:, 2 * heads * d + h * vd:2 * heads * d + (h + 1) * vd]
                o, want_state[slot][h] = plain_scan(q, f, v, want_state[slot][h])
                scale = max(1.0, float(np.abs(o).max()))
                err = float(np.abs(got[start[i]:start[i + 1], h * vd:(h + 1) * vd] - o).max())
                assert err <= 3e-5 * scale, (slot, h, lengths, err, scale)
    final = f64(state)
    for slot in slots:
        assert np.allclose(final[slot], want_state[slot], rtol=1e-5, atol=1e-5)
    assert np.all(final[3] == 7.0) and np.all(final[6] == 0.0) and np.all(final[8] == 0.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vd", [1, 9, 32, 200])
def test_unit_rms_per_head_with_one_weight_for_all_heads(dtype, vd):
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(vd)
    N, heads = 5, 3
    o = dev(rng.standard_normal((N, heads * vd)) * 4, torch.float32)
    w = dev(1 + 0.3 * rng.standard_normal(vd), torch.float32)
    out = torch.empty((N, heads * vd), dtype=torch_dtype(dtype), device="cuda")
    ops.head_rms_norm(o, w, 1e-5, out, vd)
    want = (plain.rms_unit(f64(o).reshape(N, heads, vd), 1e-5) * f64(w)).reshape(N, heads * vd)
    assert np.allclose(f64(out), want, atol=1e-5 if dtype == "float32" else 3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,K,N", [(3, 8, 20), (2, 24, 8), (4, 32, 112), (1, 5, 13), (2, 200, 70)])
def test_product_per_head_with_and_without_the_gate(dtype, heads, K, N):
    """Operands that are views into wider rows, as the mixer hands them over."""
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(K * N)
    T, rows = torch_dtype(dtype), 70
    wide = dev(rng.standard_normal((rows, 7 + heads * (K + 3) + heads * N)), T)
    x = wide[:, 7:7 + heads * (K + 3)]                                  # per head: K values, then 3 that are not read
    gate = wide[:, 7 + heads * (K + 3):]
    w = dev(rng.standard_normal((heads, K, N)) / K ** 0.5, T)
    want = np.einsum("thk,hkn->thn", f64(x).reshape(rows, heads, K + 3)[:, :, :K], f64(w))
    out = torch.full((rows, heads * (N + 2)), 5.0, dtype=T, device="cuda")
    ops.head_product(x, K + 3, 0, w, out, N + 2, 2, rows)
    got = f64(out).reshape(rows, heads, N + 2)
    tol = 2e-5 if dtype == "float32" else 3e-2
    assert np.allclose(got[:, :, 2:], want, atol=tol) and np.all(got[:, :, :2] == 5.0)
    ops.head_product(x, K + 3, 0, w, out, N + 2, 2, rows, gate=gate)
    got = f64(out).reshape(rows, heads, N + 2)
    assert np.allclose(got[:, :, 2:], want * plain.sigmoid(f64(gate).reshape(rows, heads, N)), atol=tol)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,K,N,rows", [(3, 48, 72, 150), (2, 128, 192, 70), (16, 200, 40, 9), (1, 8, 8, 64), (2, 72, 136, 129),
                                            (5, 64, 64, 1)])
def test_product_per_head_on_rows_that_split_into_packets(dtype, heads, K, N, rows):
    """Sizes and views the tensor-core tiles take in bfloat16: every offset a multiple of 8 values, tokens and outputs that
    do not fill the last tile, inner sizes that end inside a chunk and inside a step."""
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(K + N + rows)
    T = torch_dtype(dtype)
    wide = dev(rng.standard_normal((rows, 8 + heads * (K + 16) + heads * N)), T)
    x = wide[:, 8:8 + heads * (K + 16)]                                 # per head: 8 values that are not read, K, 8 more
    gate = wide[:, 8 + heads * (K + 16):]
    w = dev(rng.standard_normal((heads, K, N)) / K ** 0.5, T)
    want = np.einsum("thk,hkn->thn", f64(x).reshape(rows, heads, K + 16)[:, :, 8:8 + K], f64(w))
    out = torch.full((rows, heads * (N + 4)), 5.0, dtype=T, device="cuda")
    tol = 2e-5 if dtype == "float32" else 3e-2
    ops.head_product(x, K + 16, 8, w, out, N + 4, 2, rows)
    got = f64(out).reshape(rows, heads, N + 4)
    assert np.allclose(got[:, :, 2:N + 2], want, atol=tol) and np.all(got[:, :, :2] == 5.0) and np.all(got[:, :, N + 2:] == 5.0)
    ops.head_product(x, K + 16, 8, w, out, N + 4, 2, rows, gate=gate)
    got = f64(out).reshape(rows, heads, N + 4)
    assert np.allclose(got[:, :, 2:N + 2], want * plain.sigmoid(f64(gate).reshape(rows, heads, N)), atol=tol)
    assert np.all(got[:, :, :2] == 5.0) and np.all(got[:, :, N + 2:] == 5.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rank,rot,dims,interleaved,q_rank", [(20, 6, 6, True, 10), (24, 8, 8, False, 0), (40, 8, 4, True, 0),
                                                              (13, 2, 2, False, 3), (112, 16, 16, True, 48), (9, 0, 0, False, 0)])
def test_latent_rows_are_normed_rotated_and_written_to_their_pages(dtype, rank, rot, dims, interleaved, q_rank):
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(rank + rot)
    T = torch_dtype(dtype)
    lengths, base, eps, H, d = [70, 1, 130], 300.0, 1e-5, 3, 4
    N = sum(lengths)
    seq = np.concatenate([np.full(n, s) for s, n in enumerate(lengths)])
    pos = np.concatenate([np.arange(n) for n in lengths])
    per_seq = 3
    table = rng.permutation(11)[:per_seq * len(lengths)].reshape(len(lengths), per_seq)
    proj = dev(rng.standard_normal((N, q_rank + rank + rot + 5)) * 2, T)
    w_c, w_q = dev(1 + 0.3 * rng.standard_normal(rank), torch.float32), dev(1 + 0.3 * rng.standard_normal(max(q_rank, 1)), torch.float32)
    k_pages = torch.full((12, 1, 64, rank + rot), 50.0, dtype=T, device="cuda")
    v_pages = torch.full((12, 1, 64, rank), 50.0, dtype=T, device="cuda")
    half = max(dims // 2, 1)
    freq = np.array([base ** (-2.0 * i / max(dims, 1)) for i in range(half)])
    angle = np.arange(200)[:, None] * freq[None, :]
    cos, sin = dev(np.cos(angle), torch.float32), dev(np.sin(angle), torch.float32)
    cq = torch.empty((N, q_rank), dtype=T, device="cuda") if q_rank else None
    ops.latent_prepare(proj, q_rank, 0, w_c, w_q if q_rank else None, cq, k_pages, v_pages, cos if dims else None,
                       sin if dims else None, dev(seq, torch.int32), dev(pos, torch.int32), dev(table, torch.int32), N, rank, rot,
                       dims, interleaved, eps)
    pd = f64(proj)
    c = plain.rms_unit(pd[:, q_rank:q_rank + rank], eps) * f64(w_c)
    tail = pd[:, q_rank + rank:q_rank + rank + rot]
    k_rot = np.concatenate([plain.rotary(tail[seq == s], list(range(n)), base, dims, interleaved) for s, n in enumerate(lengths)]) \
        if dims else tail
    tol = 2e-5 if dtype == "float32" else 4e-2
    kp, vp = f64(k_pages), f64(v_pages)
    for t in range(N):
        page, at = table[seq[t], pos[t] // 64], pos[t] % 64
        assert np.allclose(kp[page, 0, at], np.concatenate([c[t], k_rot[t]]), atol=tol), t
        assert np.allclose(vp[page, 0, at], c[t], atol=tol)
    written = {(table[seq[t], pos[t] // 64], pos[t] % 64) for t in range(N)}
    assert all(np.all(kp[p, 0, a] == 50.0) for p in range(12) for a in range(64) if (p, a) not in written)
    if q_rank:
        assert np.allclose(f64(cq), plain.rms_unit(pd[:, :q_rank], eps) * f64(w_q), atol=tol)
    if rot:
        q = dev(rng.standard_normal((N, H * (d + rot))), T)
        q_full = torch.full((N, H * (rank + rot)), 5.0, dtype=T, device="cuda")
        ops.latent_queries(q, q_full, cos if dims else None, sin if dims else None, dev(pos, torch.int32), N, H, d, rank, rot, dims, interleaved)
        qd = f64(q).reshape(N, H, d + rot)[:, :, d:]
        want = np.concatenate([plain.rotary(qd[seq == s], list(range(n)), base, dims, interleaved) for s, n in enumerate(lengths)]) \
            if dims else qd
        got = f64(q_full).reshape(N, H, rank + rot)
        assert np.allclose(got[:, :, rank:], want, atol=tol) and np.all(got[:, :, :rank] == 5.0)


# ============================================================================ parts inside an engine, fed with rows of the test's own
class PartProbe:
    """Replaces what a part of a running engine reads by rows of the test's own and keeps what it returns, so that the
    part runs with the engine's own step context, cache pages and state rows, under any way of cutting the steps."""

    def __init__(self, part, rows, dtype):
        self.part, self.rows, self.dtype = part, rows, dtype
        self.take, self.seen = None, []
        self.inner = part.forward
        part.forward = self.forward

    def forward(self, x, ctx, *rest):
        N = ctx.n_tokens
        assert len(self.take) == N
        x[:N].copy_(dev(self.rows[self.take], self.dtype))
        out = self.inner(x, ctx, *rest)
        self.seen.append((self.take, out[:N].double().cpu().numpy().copy()))
        return out

    def step(self, engine, entries):
        """entries: [(slot, first row, one past the last row)]: the rows are the tokens' stand-ins (token ids are 0)."""
        from qwen3_b200 import StepEntry
        self.take = np.concatenate([np.arange(lo, hi) for _, lo, hi in entries])
        engine.step([StepEntry(slot, [0] * (hi - lo), []) for slot, lo, hi in entries])

    def gathered(self, total):
        out = {}
        for take, block in self.seen:
            for r, row in zip(take, block):
                assert r not in out
                out[int(r)] = row
        assert sorted(out) == list(range(total))
        return np.stack([out[r] for r in range(total)])


def planted_latent_inputs(rng, w, p, m, width, lengths, backs, eps, peak):
    """Mixer inputs [sum(lengths), width] in which the query at position i of a sequence points at the key at i - back
    (back taken in turn from `backs`, where i - back >= 0): the first half of the input only feeds the queries, the
    second half only the latent (the weights are changed accordingly), and a query's half is solved so that every head's
    plain query is `peak` times the unit vector of that key."""
    H, d, r, rank = m["heads"], m["dim"], m["rot_dim"], m["kv_rank"]
    half = width // 2
    first = "dq" if m.get("q_rank") else "q"
    w[p + first][:, half:] = 0.0
    w[p + "dkv"][:, :half] = 0.0
    N = sum(lengths)
    h = plain.round_bf16(rng.standard_normal((N, width)) * 0.5)
    down = h @ w[p + "dkv"].T
    c = plain.rms_unit(down[:, :rank], eps) * w[p + "dkv.norm"]
    keys = (c @ w[p + "uk"].T).reshape(N, H, d)
    start = np.concatenate([[0], np.cumsum(lengths)])
    targets = {}
    for s, n in enumerate(lengths):
        for i in range(n):
            back = backs[(i * 7 + s) % len(backs)]
            if back > i:
                continue
            j = start[s] + i - back
            t = np.zeros((H, d + r))
            t[:, :d] = peak * keys[j] / np.linalg.norm(keys[j], axis=-1, keepdims=True)
            t = t.reshape(-1)
            if m.get("q_rank"):
                cq = np.linalg.pinv(w[p + "uq"]) @ t
                cq = cq / np.sqrt(np.mean(cq ** 2)) / w[p + "dq.norm"]              # a unit-rms latent; the scale is W_uq's
                h[start[s] + i, :half] = np.linalg.pinv(w[p + "dq"][:, :half]) @ cq
            else:
                h[start[s] + i, :half] = np.linalg.pinv(w[p + "q"][:, :half]) @ t
            targets[start[s] + i] = j
    return plain.round_bf16(h), targets, np.linalg.norm(keys, axis=-1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind,heads,d,r,vd,rank,q_rank,window,dims", [
    ("latent_attention", 2, 32, 8, 16, 48, None, 70, 8), ("latent_attention", 3, 32, 4, 40, 40, 120, 64, 2),
    ("latent_attention_2", 2, 48, 16, 24, 64, None, None, 16), ("latent_attention", 4, 32, 16, 32, 112, None, 200, 16),
    ("latent_attention", 1, 64, 2, 8, 88, None, 1, 2)])
def test_latent_attention_with_keys_that_stand_out(tmp_path, dtype, kind, heads, d, r, vd, rank, q_rank, window, dims):
    """One layer inside an engine.  Every query points at ONE earlier key whose score then dominates: itself, the key
    before, keys at page borders, just inside and just outside the window, the first tokens, far back.  One head's sink
    is as large as the planted score, so that it takes about half of the weight.  Whole prompts of unequal length in one
    batch; then the same sequences as a prompt, portions of 2 and more tokens, and single tokens."""
    import qwen3_b200 as q
    rng = np.random.default_rng(heads * d + (window or 0))
    width, eps, scale, peak = 416, 1e-5, 0.5, 4.0
    mk = latent if kind == "latent_attention" else latent2
    extra = dict(q_rank=q_rank, mask=window) if kind == "latent_attention" else {}
    cfg = {"architecture": "Fagunex", "vocab": 16, "width": width, "norm": {"eps": eps},
           "layers": [layer(mk(heads, d, r, vd, rank, scale, 1000.0, dims=dims, **extra), None)]}
    config = q.config_from_dict(cfg)
    tensors = lively_weights(q.build_model(config.plan()).weight_specs(), 5)
    w = {k: v.double().numpy().copy() for k, v in tensors.items()}
    p, m = "l0.mix.", cfg["layers"][0]["mixer"]
    lengths = [300, 65, 1, 200]
    backs = [0, 1, 62, 63, 64, 65, 127, 128, 129, 190, 250] + ([window - 2, window - 1, window, window + 1] if window else [299, 198])
    backs = [b for b in backs if b >= 0]
    if q_rank:
        w[p + "uq"] *= 6.0
    h, targets, key_norms = planted_latent_inputs(rng, w, p, m, width, lengths, backs, eps, peak)
    gated = kind == "latent_attention"
    if gated:
        w[p + "sink"][:] = -2.0
        w[p + "sink"][0] = scale * peak * float(np.median(key_norms[:, 0]))
    import torch
    stored = {k: torch.tensor(plain.round_bf16(v)).to(torch.bfloat16) for k, v in w.items()}
    folder, w = make_folder(tmp_path, cfg, 0, tensors=stored)
    h = f64(dev(h, torch_dtype(dtype)))                                        # what the mixer really reads
    start = np.concatenate([[0], np.cumsum(lengths)])
    want = np.concatenate([plain.latent_mixer(h[start[s]:start[s + 1]], w, p, m, eps, gated, gated) for s in range(len(lengths))])
    # the test has teeth: a window that is one off, or a forgotten sink, moves the plain result by far more than the tolerance
    if window and window > 1:
        for other in (window - 1, window + 1):
            off = plain.latent_mixer(h[:300], w, p, dict(m, mask={"size": other}), eps, gated, gated)
            assert float(np.abs(off - want[:300]).max()) > 0.5
    if gated:
        no_sink = dict(w)
        no_sink[p + "sink"] = np.full(heads, -60.0)
        assert float(np.abs(plain.latent_mixer(h[:300], no_sink, p, m, eps, gated, gated) - want[:300]).max()) > 0.5
    tol = 3e-4 if dtype == "float32" else 0.25
    engine = q.Engine.from_folder(folder, dtype=dtype, max_tokens=64 * 12, use_graphs=False)
    probe = PartProbe(engine.model.blocks[0].mixer, h, torch_dtype(dtype))
    slots = [engine.new_sequence() for _ in lengths]
    probe.step(engine, [(slots[s], start[s], start[s + 1]) for s in range(len(lengths))])
    got = probe.gathered(sum(lengths))
    err = np.abs(got - want).max(axis=1)
    assert err.max() <= tol, ("whole", int(err.argmax()), float(err.max()))
    for s in slots:
        engine.release(s)
    # a prompt, portions down to two tokens, then single tokens, for two sequences together (other slots and pages)
    probe.seen.clear()
    pair = [0, 3]
    slots = {s: engine.new_sequence() for s in pair}
    fed = {0: 61, 3: 130}
    probe.step(engine, [(slots[s], start[s], start[s] + fed[s]) for s in pair])
    for portion in ({0: 2, 3: 2}, {0: 5, 3: 63}, {0: 64, 3: 2}, {0: 100, 3: 1}):
        probe.step(engine, [(slots[s], start[s] + fed[s], start[s] + fed[s] + n) for s, n in portion.items()])
        fed = {s: fed[s] + portion[s] for s in pair}
    while any(fed[s] < lengths[s] for s in pair):
        live = [s for s in pair if fed[s] < lengths[s]]
        probe.step(engine, [(slots[s], start[s] + fed[s], start[s] + fed[s] + 1) for s in live])
        fed = {s: fed[s] + (1 if s in live else 0) for s in pair}
    seen = {}
    for take, block in probe.seen:
        seen.update({int(r): row for r, row in zip(take, block)})
    assert sorted(seen) == sorted(list(range(0, 300)) + list(range(start[3], start[4])))
    worst = max((float(np.abs(row - want[r]).max()), r) for r, row in seen.items())
    assert worst[0] <= tol, ("in steps", worst)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,ff,experts,top,shared", [(72, 40, 5, 2, 24), (96, 64, 8, 8, 64), (50, 21, 3, 1, None), (128, 96, 1, 1, 8)])
@pytest.mark.parametrize("N", [1, 7, 300])
def test_experts_chosen_by_logit_with_a_gated_shared_expert(tmp_path, dtype, N, width, ff, experts, top, shared):
    import qwen3_b200 as q
    rng = np.random.default_rng(N + width)
    cfg = {"architecture": "Fagunex", "vocab": 16, "width": width, "norm": {"eps": 1e-5},
           "layers": [layer(hgrn2(1, 4, 4), moe_spec(ff, experts, top, shared))]}
    folder, w = make_folder(tmp_path, cfg, seed=N)
    x = f64(dev(rng.standard_normal((N, width)) * 1.5, torch_dtype(dtype)))
    engine = q.Engine.from_folder(folder, dtype=dtype, max_tokens=64 * 5, use_graphs=False)
    probe = PartProbe(engine.model.blocks[0].feed_forward, x, torch_dtype(dtype))
    probe.step(engine, [(engine.new_sequence(), 0, N)])
    got = probe.gathered(N)
    want = plain.moe(x, w, "l0.mlp.", cfg["layers"][0]["mlp"])
    err = np.abs(got - want).max(axis=1)
    scale = max(1.0, float(np.abs(want).max()))
    if dtype == "float32":
        assert err.max() <= 3e-5 * scale, float(err.max())
    else:                                   # a close call between two experts may go the other way for a few rows
        assert float(np.mean(err > 4e-2 * scale)) <= 0.02, float(err.max())


# ============================================================================ the engine
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("fagunex")
    out = {}
    for i, name in enumerate(sorted(CASES)):
        out[name, "float32"] = make_folder(base, case(name), seed=31 + i, name=name)
        # bfloat16 runs use routers whose set of chosen experts no rounding can change (see make_folder)
        out[name, "bfloat16"] = make_folder(base, case(name), seed=31 + i, name=name + "_decided", decided=True)
    return out


def engine_for(folder, dtype, max_tokens, **kw):
    from qwen3_b200 import Engine
    return Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, **kw)


def make_requests(cfg, lengths, seed):
    rng = np.random.default_rng(seed)
    return {f"r{i}": random_tokens(rng, n, cfg["vocab"]) for i, n in enumerate(lengths)}


_exact = {}


def oracle(name, weights, toks):
    key = (name, id(weights), tuple(toks))
    if key not in _exact:
        cfg = case(name)
        exact = plain.forward(cfg, weights, toks)
        rounded = plain.forward(cfg, weights, toks, rnd=plain.round_bf16)
        _exact[key] = (exact, 4.0 * float(np.max(np.abs(rounded - exact))) + 1e-6, float(np.abs(exact).max()))
    return _exact[key]


def check(got, requests, name, weights, dtype, label):
    for rid, toks in requests.items():
        exact, bf16_tol, scale = oracle(name, weights, toks)
        tol = FP32_TOL * max(1.0, scale) if dtype == "float32" else bf16_tol
        for p in range(len(toks)):
            if (rid, p) not in got:
                continue
            row = got[(rid, p)]
            assert np.all(np.isfinite(row)), f"{label}: request {rid} position {p}: non-finite logits"
            err = float(np.max(np.abs(row - exact[p])))
            assert err <= tol, f"{label} [{dtype}] case {name}: request {rid} position {p} of {len(toks)}: {err:.3e} > {tol:.3e}"


@pytest.mark.parametrize("name", sorted(CASES))
def test_hidden_rows_after_every_layer_run(folders, name):
    """32-bit: the hidden rows after each run of a layer (a layer of a repeated stretch counts every time)."""
    import torch
    from qwen3_b200 import StepEntry
    folder, weights = folders[name, "float32"]
    cfg = case(name)
    toks = random_tokens(np.random.default_rng(0), 150, cfg["vocab"])
    engine = engine_for(folder, "float32", 192)
    seen = []

    def after_run(run, residual, pending, ctx):
        x = residual[:ctx.n_tokens].double()
        if pending is not None:
            y, n = pending.branch[:ctx.n_tokens].double(), pending.norm
            if getattr(n, "stream_kind", "rms") == "dynamic_tanh":
                x = x + torch.tanh(n.alpha * y) * n.weight.double() + n.b.double()
            else:
                x = x + y * torch.rsqrt((y * y).mean(-1, keepdim=True) + n.eps) * n.weight.double()
        seen.append(x.cpu().numpy())
    engine.model.after_run = after_run
    engine.step([StepEntry(engine.new_sequence(), toks, [0])])
    states = []
    plain.forward(cfg, weights, toks, after_run=lambda run, x: states.append(x.copy()))
    assert len(seen) == len(states) == len(plain.runs_of(cfg))
    for run, (got, want) in enumerate(zip(seen, states)):
        err = float(np.max(np.abs(got - want)))
        assert err <= 2e-4 * max(1.0, float(np.max(np.abs(want)))), f"case {name}: after run {run}: {err:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,lengths", [("A", [1, 2, 3, 63, 64, 65, 69, 70, 71, 141, 300]), ("B", [63, 64, 65, 129, 260]),
                                          ("C", [31, 199, 200, 201, 450]), ("D", [1, 6, 7, 8, 70, 150])])
def test_whole_requests(folders, name, lengths, dtype):
    folder, weights = folders[name, dtype]
    requests = make_requests(case(name), lengths, seed=1)
    steps, rows = schedules.whole(requests)
    engine = engine_for(folder, dtype, schedules.peak_tokens(steps))
    got = run_steps(engine, steps, rows)
    assert len(got) == sum(lengths)
    check(got, requests, name, weights, dtype, "whole")
    assert engine.cache.pages_held() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,lengths,tail", [("A", [30, 100, 215], 160), ("B", [70, 200], 140), ("C", [230, 420], 210), ("D", [20, 90], 40)])
def test_prompt_then_token_by_token_across_window_edges(folders, name, lengths, tail, dtype):
    """The last `tail` tokens one a step, more than a window of them: the window passes over decoded tokens, the
    recurrent state and the shift's row are carried through a long decode (a request shorter than the tail goes token
    by token from its first token)."""
    folder, weights = folders[name, dtype]
    requests = make_requests(case(name), lengths, seed=2)
    steps, rows = schedules.tail_one_by_one(requests, tail)
    engine = engine_for(folder, dtype, schedules.peak_tokens(steps))
    got = run_steps(engine, steps, rows)
    check(got, requests, name, weights, dtype, "tail one by one")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,length,cuts", [
    ("A", 260, [2, 4, 31, 33, 69, 71, 80, 82, 120, 190, 258]), ("A", 150, list(range(2, 150, 2))),
    ("B", 200, [63, 65, 128, 130]), ("C", 420, [16, 199, 201, 203, 400]), ("D", 100, [3, 6, 8, 10, 12, 50])])
def test_prompts_fed_in_portions(folders, name, length, cuts, dtype):
    """Portions of many sizes, down to two tokens, that start and end at, before and after window and page edges."""
    folder, weights = folders[name, dtype]
    requests = make_requests(case(name), [length], seed=3)
    steps, rows = schedules.chunked(requests, {"r0": cuts})
    engine = engine_for(folder, dtype, schedules.peak_tokens(steps))
    got = run_steps(engine, steps, rows)
    assert len(got) == length
    check(got, requests, name, weights, dtype, "portions")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,lengths,prompts,batch", [
    ("A", [13, 130, 9, 90, 76, 45, 128, 3], [5, 100, 1, 69, 71, 40, 39, 3], 3),
    ("B", [140, 70, 200, 66], [130, 1, 64, 63], 2),
    ("C", [300, 110, 9, 260, 210], [199, 104, 1, 201, 103], 3),
    ("D", [30, 7, 50], [8, 7, 1], 3),
])
def test_unequal_batches_one_after_another(folders, name, lengths, prompts, batch, dtype):
    """Requests of different lengths start together and are decoded together; the shorter ones end earlier; the next
    batch takes over their slots, pages, state rows and shift rows.  Every row must be what the request gives alone."""
    folder, weights = folders[name, dtype]
    requests = make_requests(case(name), lengths, seed=4)
    steps, rows = schedules.batched(requests, dict(zip(requests, prompts)), batch, want_all_prompt=True)
    engine = engine_for(folder, dtype, schedules.peak_tokens(steps))
    got = run_steps(engine, steps, rows)
    check(got, requests, name, weights, dtype, "batches")
    assert engine.cache.pages_held() == 0 and engine.cache.slots.n_free == engine.cache.n_slots
    again = run_steps(engine, steps, rows)                       # the same once more: other slots and pages, same rows
    worst = max(float(np.max(np.abs(got[k] - again[k]))) for k in got)
    assert worst <= (1e-5 if dtype == "float32" else 0.05) * max(1.0, oracle(name, weights, requests["r0"])[2]), worst


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "D"])
def test_mixed_steps_of_portions_and_single_tokens(folders, name, dtype):
    folder, weights = folders[name, dtype]
    requests = make_requests(case(name), [150, 90, 200], seed=5)
    steps, rows = schedules.mixed(requests, {"r0": 38, "r1": 41, "r2": 1}, {"r0": 1, "r1": 7, "r2": 33})
    engine = engine_for(folder, dtype, schedules.peak_tokens(steps))
    got = run_steps(engine, steps, rows)
    check(got, requests, name=name, weights=weights, dtype=dtype, label="mixed")


def test_windowed_layers_free_pages_while_decoding_and_a_reused_slot_starts_from_nothing(tmp_path):
    """A long decode of one sequence: the windowed layer gives back the pages that fell
    out of the window, and a slot that is used again starts with a zero state and a zero shift row."""
    from qwen3_b200 import StepEntry
    cfg = {"architecture": "Fagunex", "vocab": 90, "width": 48, "norm": {"eps": 1e-5}, "token_side": {"dim": 3},
           "layers": [layer(latent(2, 8, 4, 8, 16, 0.3, 1000.0, mask=64), moe_spec(16, 3, 2, shared=8)),
                      layer(hgrn2(2, 8, 12), None)],
           "loop": {"start": 0, "stop": 2, "times": 2}}
    folder, weights = make_folder(tmp_path, cfg, seed=9)
    toks = random_tokens(np.random.default_rng(6), 330, cfg["vocab"])
    exact = plain.forward(cfg, weights, toks)
    scale = float(np.abs(exact).max())
    engine = engine_for(folder, "float32", 384, n_slots=1)
    for round_ in range(2):
        slot = engine.new_sequence()
        rows = [engine.step([StepEntry(slot, toks[:100], [99])])[0].cpu().numpy()]
        for p in range(100, 330):
            rows.append(engine.step([StepEntry(slot, [toks[p]], [0])])[0].cpu().numpy())
        assert max(len(g.held_pages(slot)) for g in engine.cache.groups) <= 2          # a window of 64 keys: two pages at most
        engine.release(slot)
        err = max(float(np.max(np.abs(r - exact[99 + i]))) for i, r in enumerate(rows))
        assert err <= FP32_TOL * max(1.0, scale), (round_, err)


@pytest.mark.parametrize("name", ["A", "C", "D"])
def test_greedy_generation_through_the_entry_point(folders, name):
    import qwen3_b200 as q
    folder, weights = folders[name, "float32"]
    cfg = case(name)
    rng = np.random.default_rng(7)
    prompts = [random_tokens(rng, n, cfg["vocab"]) for n in (5, 38, 1, 70)]
    engine = engine_for(folder, "float32", 64 * 8)
    got = q.generate_token_ids(engine, prompts, q.SamplingParams.greedy(), q.GenerationOptions(max_new_tokens=12))
    for p, r in zip(prompts, got):
        assert r.token_ids == plain.generate_greedy(cfg, weights, p, 12) and r.stop_reason == q.MAX_NEW_TOKENS
    assert engine.cache.pages_held() == 0
    small = engine_for(folder, "float32", 64 * 4, n_slots=2)      # fewer slots than requests: one batch after another
    again = q.generate_token_ids(small, prompts, q.SamplingParams.greedy(), q.GenerationOptions(max_new_tokens=12))
    assert [r.token_ids for r in again] == [r.token_ids for r in got]


def test_the_command_line_generates_from_token_ids(folders):
    """bin/qwen3_chat on a Fagunex folder: the model class comes from config.json; greedy sampling through the scheduler."""
    import subprocess
    import sys
    folder, weights = folders["A", "float32"]
    cfg = case("A")
    prompts = [[7, 8, 9, 150, 2], [100, 3]]
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "qwen3_chat"), folder, "--greedy", "--dtype", "float32",
                          "--max-new-tokens", "9", "--max-context", "64", "--tokens", "7,8,9,150,2", "--tokens", "100 3"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.strip().splitlines() if l and l[0].isdigit()]
    assert len(lines) == 2
    for p, line in zip(prompts, lines):
        assert [int(t) for t in line.split("#")[0].strip().split(",")] == plain.generate_greedy(cfg, weights, p, 9)


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay_from_the_command_line(tmp_path, folders, dtype, monkeypatch):
    from test_trace_run_gpu import replay
    unpadded = schedules.peak_tokens
    monkeypatch.setattr(schedules, "peak_tokens", lambda steps, page=64: unpadded(steps, 1))
    folder, weights = folders["A", dtype]
    cfg = case("A")
    requests = make_requests(cfg, [75, 1, 130], seed=8)
    w_steps, w_rows = schedules.whole(requests)
    b_steps, b_rows = schedules.batched(requests, {"r0": 40, "r1": 1, "r2": 81}, 3)
    steps, rows = [], []
    for part_steps, part_rows in ((w_steps, w_rows), (b_steps, b_rows)):
        for s, r in zip(part_steps, part_rows):
            steps.append(dict(s, step=len(steps)))
            rows.append([(f"{len(steps)}:{rid}", rid, p) for rid, p in r])
    got = replay(folder, dtype, steps, [[(tag, p) for tag, _, p in r] for r in rows], str(tmp_path / "out"), cfg["vocab"])
    for r in rows:
        for tag, rid, p in r:
            exact, bf16_tol, scale = oracle("A", weights, requests[rid])
            err = float(np.max(np.abs(got[(tag, p)] - exact[p])))
            assert err <= (FP32_TOL * max(1.0, scale) if dtype == "float32" else bf16_tol), (tag, p, err)
