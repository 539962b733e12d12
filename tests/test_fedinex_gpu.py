"""Fedinex on the GPU against the plain implementation (tests/plain/fedinex_plain.py): every mechanism alone,
then the engine under every way of cutting requests into steps, in 32-bit and in bfloat16."""
import math
import os

import numpy as np
import pytest

import schedules
from fedinex_cases import CASES, attention, case, conv_attention, dense, gla, layer, make_folder, memory, parallel, random_tokens
from fedinex_cases import moe as moe_spec
from plain import fedinex_plain as plain
from test_engine_gpu import run_steps

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = ["float32", "bfloat16"]
FP32_TOL = 3e-4
PAGE = 64


def torch_dtype(name):
    import torch
    return {"float32": torch.float32, "bfloat16": torch.bfloat16}[name]


def dev(a, dtype):
    import torch
    return torch.tensor(np.asarray(a), dtype=dtype, device="cuda")


def f64(t):
    return t.double().cpu().numpy()


def packed(lengths):
    """seq_start and token_seq of a step whose sequences bring `lengths` tokens (all positive)."""
    start = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    seq = np.concatenate([np.full(n, i) for i, n in enumerate(lengths)]).astype(np.int32)
    return start, seq


# ============================================================================ mechanisms, one at a time
def plain_decay_scan(q, k, v, a, b, S):
    """S <- diag(a_t) S + k_t (b_t v_t)^T row by row; returns the outputs S^T q."""
    out = np.zeros((q.shape[0], v.shape[1]))
    for t in range(q.shape[0]):
        S *= a[t][:, None]
        S += np.outer(k[t], b[t] * v[t])
        out[t] = S.T @ q[t]
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("per_channel", [True, False])
@pytest.mark.parametrize("heads,d,vd", [(3, 5, 9), (2, 16, 24), (1, 64, 128), (2, 128, 128), (1, 256, 64), (1, 256, 255), (2, 48, 96), (1, 1, 1)])
def test_decay_scan_over_unequal_sequences_and_from_its_state(dtype, per_channel, heads, d, vd):
    """Three steps on slots in no particular order: whole prompts, portions, single tokens; the state is carried in
    columns of a wider row, as a mixer beside another mixer holds it.  Per channel: the decay from logits; per head: keep
    and write scales, with the normaliser as a last column of ones."""
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(heads * 1000 + d + vd)
    T, tau, scale = torch_dtype(dtype), 4.0, 0.7
    vdx = vd + (0 if per_channel else 1)
    slots, n_slots, before, after = [4, 0, 5, 2], 7, 3, 2
    whole = torch.zeros((n_slots + 1, before + heads * d * vdx + after), dtype=torch.float32, device="cuda")
    whole[:, :before], whole[:, before + heads * d * vdx:] = 7.0, -7.0
    state = whole[:, before:before + heads * d * vdx]
    S = {s: np.zeros((heads, d, vdx)) for s in slots}
    bias = rng.standard_normal(heads * d) + 1.5
    tol = dict(rtol=2e-4, atol=2e-4) if dtype == "float32" else dict(rtol=3e-2, atol=3e-2)
    for lengths in ([1, 40, 2, 17], [3, 1, 0, 2], [1, 1, 1, 1]):
        live = [(s, n) for s, n in zip(slots, lengths) if n > 0]
        start, _ = packed([n for _, n in live])
        N = int(start[-1])
        proj = dev(rng.standard_normal((N, heads * (2 * d + vd) + 5)) * 0.7, T)      # q, k, v and five columns nobody reads
        z = dev(rng.standard_normal((N, heads * d)) * 2, torch.float32)
        keep = dev(rng.uniform(0.3, 1.0, (N, heads)), torch.float32)
        write = dev(rng.uniform(0.0, 1.5, (N, heads)), torch.float32)
        out = torch.full((N, heads * vdx), 9.0, dtype=torch.float32, device="cuda")
        qv, kv, vv = proj[:, :heads * d], proj[:, heads * d:2 * heads * d], proj[:, 2 * heads * d:2 * heads * d + heads * vd]
        logits = f64(z)
        kw = dict(decay=ops.channel_decay(z, dev(bias, torch.float32), tau)) if per_channel else dict(keep=keep, write=write, ones=True)
        ops.decay_scan(qv, kv, vv, state, dev(start, torch.int32), dev([s for s, _ in live], torch.int32), out, len(live), heads, d, vd,
                       q_scale=scale, **kw)
        got = f64(out).reshape(N, heads, vdx)
        pd = f64(proj)
        for i, (slot, n) in enumerate(live):
            rows = slice(start[i], start[i + 1])
            for h in range(heads):
                q = pd[rows, h * d:(h + 1) * d] * scale
                k = pd[rows, (heads + h) * d:(heads + h + 1) * d]
                v = pd[rows, 2 * heads * d + h * vd:2 * heads * d + (h + 1) * vd]
                if per_channel:
                    a = plain.sigmoid(logits[rows, h * d:(h + 1) * d] + bias[h * d:(h + 1) * d]) ** (1.0 / tau)
                    b = np.ones(n)
                else:
                    a = np.repeat(f64(keep)[rows, h][:, None], d, axis=1)
                    b = f64(write)[rows, h]
                    v = np.concatenate([v, np.ones((n, 1))], axis=1)
                want = plain_decay_scan(q, k, v, a, b[:, None], S[slot][h])
                assert np.allclose(got[rows, h], want, **tol), (lengths, slot, h)
    final = f64(whole)
    for slot in slots:
        assert np.allclose(final[slot, before:-after].reshape(heads, d, vdx), S[slot], **tol)
    assert np.all(final[:, :before] == 7.0) and np.all(final[:, -after:] == -7.0) and np.all(final[[1, 3, 6, 7], before:-after] == 0.0)


@pytest.mark.parametrize("heads", [1, 3])
def test_memory_gates_walk_the_running_maximum_from_zero_and_across_steps(heads):
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(heads)
    cap, slots, n_slots = 6.0, [2, 0, 3], 4
    whole = torch.zeros((n_slots + 1, heads + 3), dtype=torch.float32, device="cuda")
    m_state = whole[:, 2:2 + heads]
    bi, bf = rng.standard_normal(heads), rng.standard_normal(heads) + 1.0
    m = {s: np.zeros(heads) for s in slots}
    for lengths in ([70, 1, 33], [1, 1, 1], [2, 40, 0]):
        live = [(s, n) for s, n in zip(slots, lengths) if n > 0]
        start, _ = packed([n for _, n in live])
        N = int(start[-1])
        z = dev(rng.standard_normal((N, 2 * heads)) * 8, torch.float32)
        keep, write, low = (torch.full((N, heads), 9.0, dtype=torch.float32, device="cuda") for _ in range(3))
        ops.memory_gates(z, dev(bi, torch.float32), dev(bf, torch.float32), cap, m_state, dev(start, torch.int32),
                         dev([s for s, _ in live], torch.int32), keep, write, low, len(live), heads)
        zd = f64(z)
        gi = cap * np.tanh((zd[:, :heads] + bi) / cap)
        gf = plain.log_sigmoid(cap * np.tanh((zd[:, heads:] + bf) / cap))
        for i, (slot, n) in enumerate(live):
            for t in range(start[i], start[i + 1]):
                m_new = np.maximum(gf[t] + m[slot], gi[t])
                assert np.allclose(f64(keep)[t], np.exp(gf[t] + m[slot] - m_new), rtol=1e-4, atol=1e-7)
                assert np.allclose(f64(write)[t], np.exp(gi[t] - m_new), rtol=1e-4, atol=1e-7)
                assert np.allclose(f64(low)[t], np.exp(-m_new), rtol=1e-4, atol=1e-7)
                m[slot] = m_new
    for slot in slots:
        assert np.allclose(f64(m_state)[slot], m[slot], rtol=1e-5, atol=1e-5)
    assert np.all(f64(whole)[:, :2] == 0.0) and np.all(f64(whole)[1] == 0.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,vd,normaliser,shared_weight,act", [(3, 9, False, True, "silu"), (2, 48, True, False, "sigmoid"),
                                                                  (1, 200, True, False, "sigmoid"), (4, 1, False, True, "silu")])
def test_heads_are_divided_normed_weighted_and_gated(dtype, heads, vd, normaliser, shared_weight, act):
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(vd)
    T, N, eps, floor = torch_dtype(dtype), 13, 1e-5, 1e-6
    vdx = vd + (1 if normaliser else 0)
    o = dev(rng.standard_normal((N, heads * vdx)) * 3, torch.float32)
    low = dev(np.exp(rng.standard_normal((N, heads)) * 2), torch.float32) if normaliser else None
    w = dev(1 + 0.3 * rng.standard_normal(vd if shared_weight else heads * vd), torch.float32)
    proj = dev(rng.standard_normal((N, heads * vd + 7)) * 2, T)
    out = torch.empty((N, heads * vd), dtype=T, device="cuda")
    ops.head_gated_norm(o, w, proj[:, 7:], eps, out, heads, vd, act=act, low=low, floor=floor)
    x = f64(o).reshape(N, heads, vdx)
    if normaliser:
        x = x[:, :, :vd] / (np.maximum(np.abs(x[:, :, vd]), f64(low)) + floor)[:, :, None]
    g = f64(proj)[:, 7:]
    gate = plain.sigmoid(g) * (g if act == "silu" else 1.0)
    weight = np.tile(f64(w), heads) if shared_weight else f64(w)
    want = plain.rms_unit(x, eps).reshape(N, heads * vd) * weight * gate
    assert np.allclose(f64(out), want, **(dict(rtol=2e-5, atol=2e-5) if dtype == "float32" else dict(rtol=2e-2, atol=2e-2)))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("channels,taps,extra", [(7, 4, 3), (64, 3, 3), (200, 2, 3), (5, 1, 3), (9, 8, 3), (64, 3, 8), (200, 2, 0), (16, 4, 16),
                                                 (64, 5, 8), (8, 1, 8)])
def test_short_convolution_carries_its_last_rows_from_step_to_step(dtype, channels, taps, extra):
    """Steps of whole prompts, of portions shorter than the taps, and of single tokens: every output row is what the
    whole sequence gives, and the state ends as the last taps - 1 rows.  `extra` columns that are not convolved follow the
    channels: with rows of whole 16-byte packets the kernels that move packets run (for 2 to 4 taps the one that walks runs
    of tokens, whose runs here start inside, before and after a sequence's start)."""
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(channels)
    T = torch_dtype(dtype)
    w = dev(rng.standard_normal((channels, taps)), torch.float32)
    slots, n_slots, width = [3, 1, 4], 5, (taps - 1) * channels
    whole = torch.zeros((n_slots + 1, width + 4), dtype=torch.float32, device="cuda")
    whole[:, width:] = 5.0
    state = whole[:, :width]
    history = {s: np.zeros((0, channels)) for s in slots}
    for lengths in ([9, 1, 2], [1, 1, 1], [2, 0, 1], [1, 30, 3], [1, 1, 1], [70, 3, 131], [1200, 0, 5]):
        live = [(s, n) for s, n in zip(slots, lengths) if n > 0]
        start, seq = packed([n for _, n in live])
        N = int(start[-1])
        u = dev(rng.standard_normal((N, channels + extra)), T)             # more columns that are not convolved
        out = torch.full((N, channels), 9.0, dtype=T, device="cuda")
        ops.short_conv(u, w.t().contiguous(), state, dev(seq, torch.int32), dev(start, torch.int32), dev([s for s, _ in live], torch.int32), out, len(live))
        for i, (slot, n) in enumerate(live):
            old = len(history[slot])
            history[slot] = np.concatenate([history[slot], f64(u)[start[i]:start[i + 1], :channels]])
            want = plain.short_conv(history[slot], f64(w))[old:]
            assert np.allclose(f64(out)[start[i]:start[i + 1]], want, atol=1e-5 if dtype == "float32" else 5e-2), (lengths, slot)
    final = f64(whole)
    for slot in slots:
        tail = np.concatenate([np.zeros((taps - 1, channels)), history[slot]])[len(history[slot]):]
        assert np.array_equal(final[slot, :width].reshape(taps - 1, channels), tail)
    assert np.all(final[:, width:] == 5.0) and np.all(final[[0, 2, 5], :width] == 0.0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_values_are_kept_by_the_first_layer_and_blended_by_the_others(dtype):
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(3)
    T, N, off, width = torch_dtype(dtype), 19, 11, 14
    tol = 1e-6 if dtype == "float32" else 3e-2
    bias = rng.standard_normal(width)
    rows0 = dev(rng.standard_normal((N, off + width)), T)
    first = torch.zeros((N, width), dtype=T, device="cuda")
    rows = rows0.clone()
    ops.value_mix(rows, off, width, dev(bias, torch.float32), first, True)
    kept = f64(rows0)[:, off:] + bias
    assert np.allclose(f64(first), kept, atol=tol) and np.array_equal(f64(rows)[:, off:], f64(first))
    assert np.array_equal(f64(rows)[:, :off], f64(rows0)[:, :off])
    later0 = dev(rng.standard_normal((N, off + width)), T)
    for b in (bias, None):
        later = later0.clone()
        ops.value_mix(later, off, width, dev(b, torch.float32) if b is not None else None, first, False, 0.3)
        want = 0.7 * (f64(later0)[:, off:] + (b if b is not None else 0.0)) + 0.3 * f64(first)
        assert np.allclose(f64(later)[:, off:], want, atol=tol) and np.array_equal(f64(later)[:, :off], f64(later0)[:, :off])


@pytest.mark.parametrize("dtype", DTYPES)
def test_small_elementwise_steps(dtype):
    """A gate per head, the clamped gated activation in both layouts, a weighted sum, a bias."""
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(4)
    T, N = torch_dtype(dtype), 21
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == "float32" else dict(rtol=2e-2, atol=2e-2)
    heads, vd = 3, 10
    x = dev(rng.standard_normal((N, heads * vd)), T)
    gates = dev(rng.standard_normal((N, heads + 2)) * 3, T)
    want = (f64(x).reshape(N, heads, vd) * plain.sigmoid(f64(gates)[:, 1:1 + heads])[:, :, None]).reshape(N, -1)
    assert np.allclose(f64(ops.head_gate(x, gates[:, 1:1 + heads], heads, vd)), want, **tol)
    for inter, interleaved in ((24, True), (24, False), (7, False)):
        g, u = rng.standard_normal((N, inter)) * 3, rng.standard_normal((N, inter)) * 3
        both = np.concatenate([g, u], axis=1)
        if interleaved:
            both = np.stack([g.reshape(N, -1, 8), u.reshape(N, -1, 8)], axis=2).reshape(N, 2 * inter)
        gate_up = dev(both, T)
        out = torch.empty((N, inter), dtype=T, device="cuda")
        ops.clamped_mul(gate_up, out, 1.3, 1.702, interleaved)
        gd, ud = (f64(dev(a, T)) for a in (g, u))
        gc = np.minimum(gd, 1.3)
        assert np.allclose(f64(out), gc * plain.sigmoid(1.702 * gc) * (np.clip(ud, -1.3, 1.3) + 1.0), **tol)
    a, b = dev(rng.standard_normal((N, 33)), T), dev(rng.standard_normal((N, 33)), T)
    out = torch.empty_like(a)
    assert np.allclose(f64(ops.scaled_sum(a, b, 0.6, -0.9, out)), 0.6 * f64(a) - 0.9 * f64(b), **tol)
    bias = rng.standard_normal(33)
    want = f64(a) + bias
    assert np.allclose(f64(ops.add_bias(a, dev(bias, torch.float32))), want, **tol)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts,top,groups", [(6, 3, (3, 2)), (8, 4, (2, 1)), (8, 8, None), (1, 1, None), (6, 2, (6, 3)), (12, 3, (3, 2))])
def test_router_with_sigmoid_scores_and_groups_marked_by_their_two_best(dtype, experts, top, groups):
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(experts * 10 + top)
    T, N, hidden, scale = torch_dtype(dtype), 200, 40, 1.75
    h = dev(rng.standard_normal((N, hidden)), T)
    w = dev(rng.standard_normal((experts, hidden)) * 0.6, T)
    correction = rng.standard_normal(experts) * 0.4 - 0.3                # some choice scores are negative
    ids = torch.empty(N * top, dtype=torch.int32, device="cuda")
    weights, id_weight = torch.empty(N * top, dtype=torch.float32, device="cuda"), torch.empty(N, dtype=torch.float32, device="cuda")
    count, keep = groups or (1, 1)
    ops.moe_route(h, w, dev(correction, torch.float32), ids, weights, id_weight, experts, top, count, keep, sigmoid=True, group_pair=True,
                  weight_scale=scale)
    r = {"experts": experts, "top": top, "scale": scale}
    if groups:
        r["groups"] = {"count": count, "keep": keep}
    want_ids, want_w = plain.route(f64(h), {"router": f64(w), "correction": f64(dev(correction, torch.float32))}, "", r)
    got_ids, got_w = ids.cpu().numpy().reshape(N, top), f64(weights).reshape(N, top)
    assert np.array_equal(got_ids, want_ids)
    assert np.allclose(got_w, want_w, rtol=1e-5, atol=1e-6)


def plant_attention(rng, lengths, H, G, d, vd, window, keep, back, peak):
    """Queries, keys and values of sequences in which, for every query, one key `back(p)` positions back has a score that
    towers over the others (if it is visible): a unit direction shared by that key and the query, scaled by `peak`."""
    seqs = []
    for n in lengths:
        q, k, v = rng.standard_normal((n, H, d)) * 0.3, rng.standard_normal((n, G, d)) * 0.3, rng.standard_normal((n, G, vd))
        for p in range(n):
            j = p - back(p)
            if 0 <= j <= p:
                mark = rng.standard_normal(d)
                mark /= np.linalg.norm(mark)
                k[j] += peak * mark
                q[p] += peak * mark
        seqs.append((q, k, v))
    return seqs


WHERE = {"edge_in": lambda p, window, keep: window - 1, "edge_out": lambda p, window, keep: window,
         "kept_in": lambda p, window, keep: p - (keep - 1), "kept_out": lambda p, window, keep: p - keep,
         "far": lambda p, window, keep: p - p // 3}
LENGTHS = [230, 70, 1, 131]


def planted_pages(rng, T, H, G, d, vd, window, keep, where):
    """Sequences of LENGTHS tokens with planted keys, written into pages in no particular order."""
    import torch
    seqs = plant_attention(rng, LENGTHS, H, G, d, vd, window, keep, lambda p: WHERE[where](p, window, keep), 6.0)
    n_pages = sum(-(-n // PAGE) for n in LENGTHS)
    order = rng.permutation(n_pages)
    k_pages = torch.zeros((n_pages + 1, G, PAGE, d), dtype=T, device="cuda")
    v_pages = torch.zeros((n_pages + 1, G, PAGE, vd), dtype=T, device="cuda")
    table = np.full((len(LENGTHS), 4), -1, dtype=np.int32)
    at = 0
    for s, (n, (q, k, v)) in enumerate(zip(LENGTHS, seqs)):
        for pg in range(-(-n // PAGE)):
            page, rows = int(order[at]), slice(pg * PAGE, min(n, (pg + 1) * PAGE))
            at += 1
            table[s, pg] = page
            k_pages[page, :, :rows.stop - rows.start] = dev(k[rows], T).transpose(0, 1)
            v_pages[page, :, :rows.stop - rows.start] = dev(v[rows], T).transpose(0, 1)
    return seqs, k_pages, v_pages, table


def without_unseen_pages(table, take, window, keep):
    """The page table as the cache leaves it: pages that hold no key any of the queries `take` can see are given back."""
    gone = table.copy()
    for s, n in enumerate(LENGTHS):
        first_query = min(p for t, ps in take if t == s for p in ps)
        for pg in range(-(-n // PAGE)):
            if pg * PAGE >= keep and (pg + 1) * PAGE <= first_query - window + 1:
                gone[s, pg] = -1
    return gone


def check_planted(got, take, seqs, T, window, keep, where, tol):
    row = 0
    for s, ps in take:
        q, k, v = (f64(dev(a, T)) for a in seqs[s])
        want = plain.softmax_attention(q, k, v, 0.5, plain.visible(LENGTHS[s], window, keep))
        for p in ps:
            assert np.allclose(got[row], want[p], atol=tol), (s, p, where)
            row += 1


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,d,vd,window,keep", [(4, 2, 16, 24, 37, 5), (2, 1, 64, 64, 70, 70), (3, 3, 5, 9, 1, 2), (2, 2, 32, 32, 64, 0),
                                                  (4, 1, 64, 64, 130, 1), (1, 1, 8, 8, 200, 65)])
@pytest.mark.parametrize("where", sorted(WHERE))
def test_attention_sees_the_window_and_the_kept_keys_and_nothing_between(dtype, H, G, d, vd, window, keep, where):
    """The general attention kernel over pages, with one key made to stand out: just inside the window's edge, just
    outside, the last kept key, the first key after the kept ones, and a key far back; over page borders, for prompts, for
    a prompt's second portion and for single tokens."""
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(d * 100 + window)
    T = torch_dtype(dtype)
    seqs, k_pages, v_pages, table = planted_pages(rng, T, H, G, d, vd, window, keep, where)
    # the queries: every position of sequence 0, the last 30 of sequence 1 (a portion), the last position of 2 and 3
    take = [(0, list(range(LENGTHS[0]))), (1, list(range(40, 70))), (2, [0]), (3, [130])]
    qs = np.concatenate([seqs[s][0][p] for s, p in take])
    seq = np.concatenate([np.full(len(p), s) for s, p in take]).astype(np.int32)
    pos = np.concatenate([p for _, p in take]).astype(np.int32)
    N = len(pos)
    gone = without_unseen_pages(table, take, window, keep)
    out = torch.empty((N, H * vd), dtype=T, device="cuda")
    ops.attention_generic(dev(qs.reshape(N, H * d), T), k_pages, v_pages, out, dev(seq, torch.int32), dev(pos, torch.int32),
                          dev(gone, torch.int32), N, H, G, d, 0.5, window=window, value_dim=vd, keep_first=keep)
    check_planted(f64(out).reshape(N, H, vd), take, seqs, T, window, keep, where, 2e-5 if dtype == "float32" else 3e-2)


@pytest.mark.parametrize("H,G,d,vd,window,keep", [(4, 2, 16, 32, 37, 5), (2, 1, 64, 64, 70, 70), (2, 2, 32, 32, 64, 0), (4, 1, 64, 64, 130, 1),
                                                  (2, 1, 128, 64, 200, 65), (16, 1, 16, 16, 1, 2), (2, 2, 64, 64, 63, 129)])
@pytest.mark.parametrize("where", sorted(WHERE))
def test_tiled_attention_kernels_walk_the_kept_pages_before_the_window_s(H, G, d, vd, window, keep, where):
    """The same through the tensor-core kernels of the bfloat16 path: prompts and portions in tiles of 64 rows, single
    tokens with the pages split over several blocks (1, 2 and 5 of them)."""
    import torch
    from qwen3_b200.csrc import ops
    rng = np.random.default_rng(d * 100 + window + 1)
    T = torch.bfloat16
    seqs, k_pages, v_pages, table = planted_pages(rng, T, H, G, d, vd, window, keep, where)
    take = [(0, list(range(LENGTHS[0]))), (1, list(range(40, 70))), (2, [0]), (3, [130])]
    qs = np.concatenate([seqs[s][0][p] for s, p in take])
    N = len(qs)
    start = np.concatenate([[0], np.cumsum([len(p) for _, p in take])]).astype(np.int32)
    pos0 = np.array([p[0] for _, p in take], dtype=np.int32)
    gone = without_unseen_pages(table, take, window, keep)
    out = torch.empty((N, H * vd), dtype=T, device="cuda")
    ops.attention_capped_prefill(dev(qs.reshape(N, H * d), T), k_pages, v_pages, out, dev(start, torch.int32), dev(pos0, torch.int32),
                                 dev(gone, torch.int32), len(take), LENGTHS[0], H, G, d, vd, 0.5, 0.0, None, False, window=window,
                                 keep_first=keep)
    check_planted(f64(out).reshape(N, H, vd), take, seqs, T, window, keep, where, 3e-2)
    last = [(s, [n - 1]) for s, n in enumerate(LENGTHS)]
    ql = np.concatenate([seqs[s][0][p] for s, p in last])
    gone = without_unseen_pages(table, last, window, keep)
    for splits in (1, 2, 5):
        scratch = torch.empty(len(last) * H * splits * (vd + 2), dtype=torch.float32, device="cuda")
        out = torch.empty((len(last), H * vd), dtype=T, device="cuda")
        ops.attention_capped_decode(dev(ql.reshape(len(last), H * d), T), k_pages, v_pages, out, scratch,
                                    dev(np.arange(len(last)), torch.int32), dev([n - 1 for n in LENGTHS], torch.int32),
                                    dev(gone, torch.int32), len(last), H, G, d, vd, 0.5, 0.0, None, False, splits, window=window,
                                    keep_first=keep)
        check_planted(f64(out).reshape(len(last), H, vd), last, seqs, T, window, keep, where, 3e-2)


# ============================================================================ the engine
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("fedinex")
    out = {}
    for i, name in enumerate(sorted(CASES)):
        out[name, "float32"] = make_folder(base, case(name), seed=51 + i, name=name)
        # bfloat16 runs use routers whose set of chosen experts no rounding can change (see make_folder)
        out[name, "bfloat16"] = make_folder(base, case(name), seed=51 + i, name=name + "_decided", decided=True)
    return out


def engine_for(folder, dtype, max_tokens, **kw):
    from qwen3_b200 import Engine
    return Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, **kw)


def make_requests(cfg, lengths, seed):
    rng = np.random.default_rng(seed)
    return {f"r{i}": random_tokens(rng, n, cfg["vocab"]) for i, n in enumerate(lengths)}


_exact = {}


def oracle(name, weights, toks, cfg=None):
    key = (name, id(weights), tuple(toks))
    if key not in _exact:
        cfg = cfg or case(name)
        exact = plain.forward(cfg, weights, toks)
        rounded = plain.forward(cfg, weights, toks, rnd=plain.round_bf16)
        _exact[key] = (exact, 4.0 * float(np.max(np.abs(rounded - exact))) + 1e-6, float(np.abs(exact).max()))
    return _exact[key]


def check(got, requests, name, weights, dtype, label, cfg=None):
    """32-bit: every row within FP32_TOL.  bfloat16: within four times what rounding does to this very request in the plain
    implementation; a recurrent read-out followed by a unit norm is badly conditioned where the state nearly cancels, so one
    row in fifty may be further off (where the rounding falls differs from the plain run's), but none beyond four times that."""
    for rid, toks in requests.items():
        exact, bf16_tol, scale = oracle(name, weights, toks, cfg)
        tol = FP32_TOL * max(1.0, scale) if dtype == "float32" else bf16_tol
        over, rows = [], 0
        for p in range(len(toks)):
            if (rid, p) not in got:
                continue
            row = got[(rid, p)]
            rows += 1
            assert np.all(np.isfinite(row)), f"{label}: request {rid} position {p}: non-finite logits"
            err = float(np.max(np.abs(row - exact[p])))
            if dtype == "bfloat16" and tol < err <= 4.0 * tol:
                over.append(p)
                continue
            assert err <= tol, f"{label} [{dtype}] case {name}: request {rid} position {p} of {len(toks)}: {err:.3e} > {tol:.3e}"
        assert len(over) <= rows // 50, f"{label} [{dtype}] case {name}: request {rid}: {len(over)} of {rows} rows beyond {tol:.3e}: {over}"


@pytest.mark.parametrize("name", sorted(CASES))
def test_hidden_rows_after_every_layer(folders, name):
    from qwen3_b200 import StepEntry
    folder, weights = folders[name, "float32"]
    cfg = case(name)
    toks = random_tokens(np.random.default_rng(0), 150, cfg["vocab"])
    engine = engine_for(folder, "float32", 192)
    seen = []

    def after_run(run, residual, pending, ctx):
        x = residual[:ctx.n_tokens].double()
        seen.append((x + pending.branch[:ctx.n_tokens].double() if pending is not None else x).cpu().numpy())
    engine.model.after_run = after_run
    engine.step([StepEntry(engine.new_sequence(), toks, [0])])
    states = plain.hidden_states(cfg, weights, toks)
    assert len(seen) == len(states)
    for i, (got, want) in enumerate(zip(seen, states)):
        err = float(np.max(np.abs(got - want)))
        assert err <= 2e-4 * max(1.0, float(np.max(np.abs(want)))), f"case {name}: after layer {i} ({cfg['layers'][i]['type']}): {err:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,lengths", [("A", [1, 2, 3, 4, 5, 6, 9, 10, 33, 34, 63, 64, 65, 70, 71, 141, 300]), ("B", [63, 64, 65, 129, 260]),
                                          ("C", [31, 70, 71, 150, 151, 450]), ("D", [1, 2, 3, 4, 5, 8, 70, 150])])
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
    """The last `tail` tokens one a step, more than a window of them: the window passes over decoded tokens while the
    kept keys stay, the recurrent states and the convolution's rows are carried through a long decode (a request shorter
    than the tail goes token by token from its first token)."""
    folder, weights = folders[name, dtype]
    requests = make_requests(case(name), lengths, seed=2)
    steps, rows = schedules.tail_one_by_one(requests, tail)
    engine = engine_for(folder, dtype, schedules.peak_tokens(steps))
    got = run_steps(engine, steps, rows)
    check(got, requests, name, weights, dtype, "tail one by one")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,length,cuts", [
    ("A", 260, [2, 4, 5, 7, 31, 33, 69, 71, 80, 82, 120, 190, 258]), ("A", 150, list(range(2, 150, 2))),
    ("B", 200, [63, 65, 128, 130]), ("C", 420, [16, 69, 71, 149, 151, 203, 400]), ("D", 100, [2, 4, 6, 8, 10, 12, 50])])
def test_prompts_fed_in_portions(folders, name, length, cuts, dtype):
    """Portions of many sizes, down to two tokens (fewer than the convolution's taps), that start and end at, before and
    after the edges of windows, kept stretches and pages."""
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
    batch takes over their slots, pages and state rows.  Every row must be what the request gives alone."""
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


def test_a_long_decode_gives_pages_back_but_for_the_kept_ones_and_a_reused_slot_starts_from_nothing(tmp_path):
    from qwen3_b200 import StepEntry
    cfg = {"architecture": "Fedinex", "vocab": 90, "width": 48, "norm": {"eps": 1e-5},
           "layers": [layer(attention(2, 1, 8, 8, 0.3, 1000.0, 4, window=64, keep_first=3, v_mix=True), moe_spec(16, 2.0, 3, 2, 1.5)),
                      layer(parallel(conv_attention(2, 1, 8, 8, 0.3, 1000.0, 8, conv=3), memory(2, 8, 12, 5.0), 0.8, 0.8), None),
                      layer(gla(2, 8, 12, 6.0, 4), dense(32, 2.0)),
                      layer(attention(2, 1, 8, 8, 0.3, 1000.0, 4, window=30, v_mix=True), None)]}
    folder, weights = make_folder(tmp_path, cfg, seed=9)
    toks = random_tokens(np.random.default_rng(6), 330, cfg["vocab"])
    exact = plain.forward(cfg, weights, toks)
    scale = float(np.abs(exact).max())
    engine = engine_for(folder, "float32", 2 * 384, n_slots=1)
    for round_ in range(2):
        slot = engine.new_sequence()
        rows = [engine.step([StepEntry(slot, toks[:100], [99])])[0].cpu().numpy()]
        for p in range(100, 330):
            rows.append(engine.step([StepEntry(slot, [toks[p]], [0])])[0].cpu().numpy())
        held = {g.need.kind + str(g.need.keep_first): len(g.held_pages(slot)) for g in engine.cache.groups}
        assert held == {"window3": 3, "full0": 6, "window0": 2}, held          # the first page stays where the first keys are kept
        engine.release(slot)
        err = max(float(np.max(np.abs(r - exact[99 + i]))) for i, r in enumerate(rows))
        assert err <= FP32_TOL * max(1.0, scale), (round_, err)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["gla", "parallel", "attention", "one_tap"])
def test_models_of_one_kind_of_layer(tmp_path, kind, dtype):
    """No page group at all (only recurrences), only layers with pages and state, only attention (blended values with and
    without a window, head sizes the tiled kernels take), and a convolution of one tap (no rows to carry): prompt, then token
    by token."""
    mixers = {"gla": [gla(2, 8, 12, 5.0, 4), gla(1, 16, 8, 9.0, 2)],
              "parallel": [parallel(conv_attention(2, 1, 8, 8, 0.3, 1000.0, 4, conv=2), memory(2, 8, 8, 5.0), 0.5, 0.5)] * 2,
              "attention": [attention(2, 2, 16, 16, 0.3, 100.0, 8, v_mix=True), attention(4, 2, 16, 16, 0.3, window=20, keep_first=2, v_mix=True),
                            attention(2, 2, 32, 16, 0.2, 3000.0, 32, v_mix=True)],
              "one_tap": [parallel(conv_attention(2, 2, 8, 8, 0.3, conv=1), memory(1, 8, 8, 3.0), 1.0, -1.0)]}[kind]
    cfg = {"architecture": "Fedinex", "vocab": 80, "width": 40, "norm": {"eps": 1e-5},
           "layers": [layer(m, dense(48, 2.0) if i % 2 else moe_spec(16, 2.0, 4, 2, 1.5, groups=(2, 1))) for i, m in enumerate(mixers)]}
    folder, weights = make_folder(tmp_path, cfg, seed=12, decided=dtype == "bfloat16")
    requests = make_requests(cfg, [90, 3], seed=13)
    steps, rows = schedules.tail_one_by_one(requests, 40)
    engine = engine_for(folder, dtype, schedules.peak_tokens(steps))
    got = run_steps(engine, steps, rows)
    check(got, requests, "one kind: " + kind, weights, dtype, "one kind", cfg=cfg)
    assert engine.cache.pages_held() == 0


@pytest.mark.parametrize("name", ["A", "C", "D"])
def test_greedy_generation_through_the_entry_point(folders, name):
    import qwen3_b200 as q
    folder, weights = folders[name, "float32"]
    cfg = case(name)
    rng = np.random.default_rng(7)
    prompts = [random_tokens(rng, n, cfg["vocab"]) for n in (5, 38, 1, 70)]

    def greedy(prompt, n):
        toks = list(prompt)
        for _ in range(n):
            toks.append(int(np.argmax(plain.forward(cfg, weights, toks)[-1])))
        return toks[len(prompt):]
    engine = engine_for(folder, "float32", 64 * 8)
    got = q.generate_token_ids(engine, prompts, q.SamplingParams.greedy(), q.GenerationOptions(max_new_tokens=10))
    for p, r in zip(prompts, got):
        assert r.token_ids == greedy(p, 10) and r.stop_reason == q.MAX_NEW_TOKENS
    assert engine.cache.pages_held() == 0
    small = engine_for(folder, "float32", 64 * 4, n_slots=2)      # fewer slots than requests: one batch after another
    again = q.generate_token_ids(small, prompts, q.SamplingParams.greedy(), q.GenerationOptions(max_new_tokens=10))
    assert [r.token_ids for r in again] == [r.token_ids for r in got]


def test_the_command_line_generates_from_token_ids(folders):
    """bin/qwen3_chat on a Fedinex folder: the model class comes from config.json; greedy sampling through the scheduler."""
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
        toks = list(p)
        for _ in range(9):
            toks.append(int(np.argmax(plain.forward(cfg, weights, toks)[-1])))
        assert [int(t) for t in line.split("#")[0].strip().split(",")] == toks[len(p):]


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
