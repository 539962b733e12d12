"""Fedinex without a GPU: the configuration, the plan it makes, the cache's bookkeeping for a window that keeps the
first keys, and the plain implementation against closed forms."""
import copy
import math

import numpy as np
import pytest

from fedinex_cases import CASES, case, decide_routers, lively_weights
from plain import fedinex_plain as plain


@pytest.mark.parametrize("name", sorted(CASES))
def test_configuration_round_trip_and_plan(name):
    import qwen3_b200 as q
    cfg = case(name)
    config = q.config_from_dict(cfg)
    assert isinstance(config, q.FedinexConfig)
    assert q.config_from_dict(config.to_dict()) == config
    plan = config.plan()
    assert plan.order == list(range(len(cfg["layers"]))) and plan.residual_dtype == "float32" and plan.streams == 1
    model = q.build_model(plan)
    names = set(model.weight_specs())
    assert {"embed", "final.norm", "head"} <= names
    needs = model.cache_needs()
    blended = [i for i, l in enumerate(cfg["layers"]) if l["type"] == "attention" and l["mixer"].get("v_mix")]
    for i, layer in enumerate(cfg["layers"]):
        p, m, need = f"l{i}.", layer["mixer"], needs[i]
        assert p + "norm1" in names and (p + "norm2" in names) == (layer["mlp"] is not None)
        if layer["type"] == "gla":
            assert {p + "mix.q", p + "mix.a1", p + "mix.a2", p + "mix.a2.b", p + "mix.norm", p + "mix.g", p + "mix.o"} <= names
            assert need.kind == "none" and need.state_shape == (m["heads"] * m["dim"] * m["vdim"],)
        elif layer["type"] == "attention":
            assert {p + "mix.q.b", p + "mix.k.b", p + "mix.v.b", p + "mix.o.b"} <= names and p + "mix.g" not in names
            assert (p + "mix.vmix" in names) == bool(m.get("v_mix"))
            mask = m.get("mask")
            assert need.kind == ("window" if mask else "full") and need.window == (mask or {}).get("size")
            assert need.keep_first == ((mask or {}).get("keep_first") or 0) and need.state_shape == ()
            mixer = model.blocks[i].mixer
            assert mixer.value_mix == (None if i not in blended else ("first" if i == blended[0] else "blend"))
        else:
            left, right = m["left"], m["right"]
            assert {p + "mix.left.g", p + "mix.left.o", p + "mix.right.i", p + "mix.right.f.b", p + "mix.right.norm"} <= names
            assert (p + "mix.left.k.conv" in names) == bool(left.get("conv")) and p + "mix.left.q.b" not in names
            columns = (left["heads"] + left["kv_heads"]) * left["dim"] + left["kv_heads"] * left["vdim"]
            cells = right["heads"] * right["dim"] * (right["vdim"] + 1) + right["heads"]
            assert need.kind == "full" and need.state_shape == (max((left.get("conv") or 1) - 1, 0) * columns + cells,)
        if layer["mlp"] is not None and layer["mlp"]["kind"] == "moe":
            last = layer["mlp"]["router"]["experts"] - 1
            assert {p + "mlp.router", p + "mlp.correction", p + f"mlp.e{last}.down"} <= names and p + f"mlp.e{last + 1}.up" not in names
        elif layer["mlp"] is not None:
            assert {p + "mlp.gate", p + "mlp.up", p + "mlp.down"} <= names


@pytest.mark.parametrize("change,message", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].update(eps=0.0), "eps"),
    (lambda c: c["layers"][0].update(type="hgrn2"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(tau=0.0), "tau"),
    (lambda c: c["layers"][0]["mixer"].update(dim=300), "dim"),
    (lambda c: c["layers"][0]["mixer"].update(rank=0), "rank"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(base=0.0), "rot.base"),
    (lambda c: c["layers"][1]["mixer"]["mask"].update(size=0), "mask.size"),
    (lambda c: c["layers"][1]["mixer"]["mask"].update(keep_first=-1), "keep_first"),
    (lambda c: c["layers"][1]["mixer"].update(v_mix=1), "v_mix"),
    (lambda c: c["layers"][3]["mixer"].update(kv_heads=1, vdim=48), "v_mix"),
    (lambda c: c["layers"][2]["mixer"]["left"].update(conv=40), "conv"),
    (lambda c: c["layers"][2]["mixer"]["right"].update(gate_cap=0.0), "gate_cap"),
    (lambda c: c["layers"][2]["mixer"]["right"].update(vdim=256), "vdim"),
    (lambda c: c["layers"][2]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c["layers"][0]["mlp"].update(kind="gelu"), "kind"),
    (lambda c: c["layers"][0]["mlp"].update(limit=0.0), "limit"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][1]["mlp"]["router"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(keep=1), "groups"),
])
def test_configuration_faults_are_named(change, message):
    import qwen3_b200 as q
    cfg = case("A")
    change(cfg)
    with pytest.raises(q.ConfigError, match=message):
        q.config_from_dict(cfg)


def test_optional_mechanisms_may_be_absent_or_null():
    import qwen3_b200 as q
    bare = case("A")
    for layer in bare["layers"]:
        layer["mlp"] = None
        m = layer["mixer"]
        for key in ("mask", "rot", "v_mix"):
            m.pop(key, None)
        if "left" in m:
            m["left"]["conv"] = None
            m["left"]["rot"] = None
    model = q.build_model(q.config_from_dict(bare).plan())
    names = set(model.weight_specs())
    assert "l1.mix.vmix" not in names and "l2.mix.left.q.conv" not in names and "l1.mlp.router" not in names and "l1.norm2" not in names
    needs = model.cache_needs()
    assert needs[1].kind == "full" and needs[1].keep_first == 0
    right = bare["layers"][2]["mixer"]["right"]
    assert needs[2].state_shape == (right["heads"] * right["dim"] * (right["vdim"] + 1) + right["heads"],)
    assert model.blocks[1].mixer.position is None and model.blocks[2].mixer.mixers[0].position is None


def test_a_size_the_file_does_not_give_comes_from_the_checkpoint(tmp_path):
    """The rank of the decay's narrow projection: stated for random weights, read from the tensors otherwise."""
    import qwen3_b200 as q
    from fedinex_cases import make_folder
    cfg = case("D")
    folder, _ = make_folder(tmp_path, cfg, seed=1)
    del cfg["layers"][0]["mixer"]["rank"]
    model = q.build_model(q.config_from_dict(cfg).plan())
    specs = model.weight_specs()
    assert specs["l0.mix.a1"].shape == (-1, 50) and specs["l0.mix.a2"].shape == (15, -1)
    loaded = q.load_weights(folder, specs)
    assert tuple(loaded["l0.mix.a1"].shape) == (3, 50) and tuple(loaded["l0.mix.a2"].shape) == (15, 3)
    with pytest.raises(ValueError, match="random weights"):
        q.random_weights(specs, 0)


def test_the_book_keeps_the_pages_of_the_first_keys_of_a_window_group():
    from qwen3_b200.cache import CacheBook, CacheNeed
    page = 64
    needs = [CacheNeed("window", 1, 8, window=45, keep_first=70), CacheNeed("window", 1, 8, window=45),
             CacheNeed("window", 1, 8, window=45, keep_first=1), CacheNeed("full", 1, 8)]
    book = CacheBook(needs, max_tokens=10 * page, max_seq_len=10 * page, n_slots=2)
    assert len(book.groups) == 4                                    # the kept stretch is part of what a group is
    slot = book.alloc_slot()
    book.reserve([(slot, 5 * page + 3)])
    book.commit([(slot, 5 * page + 3)])
    held = [sorted(int(i) for i in np.nonzero(g.table[slot] >= 0)[0]) for g in book.groups]
    assert held[0] == [0, 1, 4, 5] and held[1] == [4, 5] and held[2] == [0, 4, 5] and held[3] == [0, 1, 2, 3, 4, 5]
    for _ in range(70):                                             # token by token over a page border
        book.reserve([(slot, 1)])
        book.commit([(slot, 1)])
    held = [sorted(int(i) for i in np.nonzero(g.table[slot] >= 0)[0]) for g in book.groups]
    assert held[0] == [0, 1, 5, 6] and held[1] == [5, 6] and held[2] == [0, 5, 6]
    book.free_slot(slot)
    assert all(g.n_free == g.n_pages for g in book.groups)
    again = book.alloc_slot()
    book.reserve([(again, 3)])
    book.commit([(again, 3)])
    assert [len(g.held_pages(again)) for g in book.groups] == [1, 1, 1, 1]


# ---------------------------------------------------------------- the plain implementation against closed forms
def test_gated_linear_attention_equals_its_sum_form():
    """o_t = sum_(j <= t) sum_c q_tc (prod_(j < s <= t) alpha_sc) k_jc v_j, channel by channel."""
    rng = np.random.default_rng(0)
    T, H, d, vd, width, rank, tau = 25, 2, 5, 4, 12, 3, 4.0
    m = {"heads": H, "dim": d, "vdim": vd, "tau": tau}
    w = {"q": rng.standard_normal((H * d, width)), "k": rng.standard_normal((H * d, width)), "v": rng.standard_normal((H * vd, width)),
         "g": rng.standard_normal((H * vd, width)), "a1": rng.standard_normal((rank, width)), "a2": rng.standard_normal((H * d, rank)),
         "a2.b": rng.standard_normal(H * d) + 1.0, "norm": 1 + 0.1 * rng.standard_normal(vd), "o": np.eye(H * vd)}
    h = rng.standard_normal((T, width)) * 0.5
    got = plain.gated_linear_attention(h, w, "", m, 1e-6)
    q, k, v = (h @ w["q"].T) * d ** -0.5, h @ w["k"].T, h @ w["v"].T
    alpha = plain.sigmoid((h @ w["a1"].T) @ w["a2"].T + w["a2.b"]) ** (1.0 / tau)
    assert 0.0 < alpha.min() and alpha.max() < 1.0
    o = np.zeros((T, H, vd))
    for head in range(H):
        ch, vs = slice(head * d, (head + 1) * d), slice(head * vd, (head + 1) * vd)
        for t in range(T):
            for j in range(t + 1):
                decay = np.prod(alpha[j + 1:t + 1, ch], axis=0)
                o[t, head] += np.sum(q[t, ch] * decay * k[j, ch]) * v[j, vs]
    g = h @ w["g"].T
    want = (plain.rms_unit(o, 1e-6) * w["norm"]).reshape(T, H * vd) * g * plain.sigmoid(g)
    assert np.allclose(got, want, rtol=1e-9, atol=1e-9)


def test_matrix_memory_equals_its_unstabilised_form():
    """Without the running maximum: C_t = sigma(f~) C + exp(i) k v^T, o = C^T q / max(|n . q|, 1): the maximum only rescales
    (with gates small enough for plain exponentials; the floor of 1e-6 is scaled too, hence the tolerance)."""
    rng = np.random.default_rng(1)
    T, H, d, vd, width, cap = 30, 2, 4, 3, 10, 5.0
    m = {"heads": H, "dim": d, "vdim": vd, "gate_cap": cap}
    w = {n: rng.standard_normal((H * s, width)) for n, s in (("q", d), ("k", d), ("v", vd), ("g", vd))}
    w.update({"i": rng.standard_normal((H, width)), "f": rng.standard_normal((H, width)), "i.b": rng.standard_normal(H),
              "f.b": rng.standard_normal(H) + 2.0, "norm": np.ones(H * vd), "o": np.eye(H * vd)})
    h = rng.standard_normal((T, width))
    got = plain.matrix_memory(h, w, "", m, 1e-6)
    q, k, v = (h @ w["q"].T * d ** -0.5).reshape(T, H, d), (h @ w["k"].T).reshape(T, H, d), (h @ w["v"].T).reshape(T, H, vd)
    gi = cap * np.tanh((h @ w["i"].T + w["i.b"]) / cap)
    gf = plain.log_sigmoid(cap * np.tanh((h @ w["f"].T + w["f.b"]) / cap))
    o = np.zeros((T, H, vd))
    for a in range(H):
        C, n = np.zeros((d, vd)), np.zeros(d)
        for t in range(T):
            C = math.exp(gf[t, a]) * C + math.exp(gi[t, a]) * np.outer(k[t, a], v[t, a])
            n = math.exp(gf[t, a]) * n + math.exp(gi[t, a]) * k[t, a]
            o[t, a] = C.T @ q[t, a] / max(abs(n @ q[t, a]), 1.0)
    want = plain.rms_unit(o, 1e-6).reshape(T, H * vd) * plain.sigmoid(h @ w["g"].T)
    assert np.allclose(got, want, rtol=1e-4, atol=1e-4)


def test_short_convolution_is_causal_and_starts_from_zeros():
    rng = np.random.default_rng(2)
    u, taps = rng.standard_normal((9, 3)), rng.standard_normal((3, 4))
    y = plain.short_conv(u, taps)
    for t in range(9):
        want = sum(taps[:, j] * (u[t - 3 + j] if t - 3 + j >= 0 else 0.0) for j in range(4))
        assert np.allclose(y[t], want)
    changed = u.copy()
    changed[5] += 1.0
    assert np.array_equal(plain.short_conv(changed, taps)[:5], y[:5])


def test_window_that_keeps_the_first_keys():
    see = plain.visible(12, window=3, keep_first=2)
    for i in range(12):
        assert [j for j in range(12) if see[i, j]] == sorted(set(range(min(2, i + 1))) | set(range(max(0, i - 2), i + 1)))
    assert np.array_equal(plain.visible(5), np.tril(np.ones((5, 5), dtype=bool)))


def test_rotation_of_a_part_of_the_head_in_both_layouts():
    rng = np.random.default_rng(3)
    v = rng.standard_normal((6, 2, 10))
    for interleaved in (False, True):
        out = plain.rotary(v, range(6), 100.0, 4, interleaved)
        assert np.array_equal(out[..., 4:], v[..., 4:]) and np.array_equal(out[0], v[0])
        pairs = [(0, 1), (2, 3)] if interleaved else [(0, 2), (1, 3)]
        for i, (a, b) in enumerate(pairs):
            angle = 3 * 100.0 ** (-2.0 * i / 4)
            assert np.allclose(out[3, :, a], v[3, :, a] * math.cos(angle) - v[3, :, b] * math.sin(angle))
            assert np.allclose(out[3, :, b], v[3, :, b] * math.cos(angle) + v[3, :, a] * math.sin(angle))


def test_router_takes_groups_by_their_two_best_and_weights_by_plain_scores():
    w = {"router": np.eye(6), "correction": np.array([0.0, 0.0, 0.0, 0.0, 0.0, 0.0])}
    r = {"experts": 6, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 1}}
    h = np.array([[4.0, -9.0, 1.0, 1.5, 0.0, 0.0]])            # group 0 holds the best expert, group 1 the best pair
    ids, weights = plain.route(h, w, "", r)
    assert sorted(ids[0]) == [2, 3] and np.allclose(sorted(weights[0]), [2.0 * plain.sigmoid(1.0), 2.0 * plain.sigmoid(1.5)])
    w["correction"] = np.array([0.0, 0.0, -5.0, -5.0, -1.0, -1.5])   # corrections choose, plain scores weigh; all negative is fine
    ids, weights = plain.route(np.zeros((1, 6)), w, "", dict(r, groups={"count": 3, "keep": 2}))
    assert list(ids[0]) == [0, 1] and np.allclose(weights[0], [1.0, 1.0])
    ids, _ = plain.route(np.zeros((1, 6)), w, "", dict(r, top=3, groups={"count": 3, "keep": 2}))
    assert list(ids[0]) == [0, 1, 4]                                  # the third comes from the second-best group, not from the dropped one


def test_decided_routers_choose_the_same_set_whatever_the_token():
    import qwen3_b200 as q
    cfg = case("A")
    tensors = decide_routers(lively_weights(q.build_model(q.config_from_dict(cfg).plan()).weight_specs(), 5), 6)
    w = {k: v.double().numpy() for k, v in tensors.items()}
    rng = np.random.default_rng(4)
    h = rng.standard_normal((50, cfg["width"])) * 3
    for i, layer in enumerate(cfg["layers"]):
        if layer["mlp"] and layer["mlp"]["kind"] == "moe":
            ids, _ = plain.route(h, w, f"l{i}.mlp.", layer["mlp"]["router"])
            assert len({tuple(sorted(row)) for row in ids}) == 1


def test_greedy_choice_of_the_plain_model_is_causal():
    import qwen3_b200 as q
    cfg = case("D")
    tensors = lively_weights(q.build_model(q.config_from_dict(cfg).plan()).weight_specs(), 7)
    w = {k: v.double().numpy() for k, v in tensors.items()}
    toks = [int(t) for t in np.random.default_rng(5).integers(0, cfg["vocab"], 40)]
    full = plain.forward(cfg, w, toks)
    assert np.allclose(plain.forward(cfg, w, toks[:17]), full[:17], rtol=1e-9, atol=1e-9)
    assert copy.deepcopy(cfg) == case("D")
