"""Fagunex without a GPU: the configuration, the plan it makes, and the plain implementation against closed forms."""
import copy

import numpy as np
import pytest

from fagunex_cases import CASES, case, decide_routers, lively_weights
from plain import fagunex_plain as plain


@pytest.mark.parametrize("name", sorted(CASES))
def test_configuration_round_trip_and_plan(name):
    import qwen3_b200 as q
    cfg = case(name)
    config = q.config_from_dict(cfg)
    assert isinstance(config, q.FagunexConfig)
    assert q.config_from_dict(config.to_dict()) == config
    plan = config.plan()
    n = len(cfg["layers"])
    assert plan.order == plain.runs_of(cfg) == config.runs() and plan.residual_dtype == "float32" and plan.streams == 1
    # the first pass of a repeated stretch uses the layers' own caches, every further pass caches of its own
    caches = plan.caches if plan.caches is not None else plan.order
    assert len(set(caches)) == len(caches)
    seen = set()
    for run, layer in enumerate(plan.order):
        assert (caches[run] == layer) == (layer not in seen) and (caches[run] >= n) == (layer in seen)
        seen.add(layer)
    model = q.build_model(plan)
    names = set(model.weight_specs())
    assert {"embed", "final.norm", "final.norm.alpha", "final.norm.b", "head"} <= names
    assert ("side.embed" in names) == ("token_side" in cfg)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        assert {p + "norm1", p + "norm1.alpha", p + "norm1.b", p + "norm1b", p + "shift", p + "mix.o"} <= names
        assert (p + "side.gate" in names) == ("token_side" in cfg)
        assert (p + "norm2" in names) == (layer["mlp"] is not None) == (p + "norm2" not in model.ignorable_names())
        if layer["type"] == "hgrn2":
            assert {p + "mix.q", p + "mix.f", p + "mix.f.b", p + "mix.lower", p + "mix.v", p + "mix.norm"} <= names
        else:
            first = layer["type"] == "latent_attention"
            assert {p + "mix.dkv", p + "mix.dkv.norm", p + "mix.uk", p + "mix.uv"} <= names
            assert (p + "mix.sink" in names) == (p + "mix.g" in names) == first
            assert (p + "mix.dq" in names) == (p + "mix.uq" in names) == (p + "mix.q" not in names) == bool(m.get("q_rank"))
        if layer["mlp"] is not None:
            assert (p + "mlp.shared.sg" in names) == (p + "mlp.shared.down" in names) == ("shared" in layer["mlp"])
            assert p + "mlp.router" in names and p + f"mlp.e{layer['mlp']['router']['experts'] - 1}.up" in names
            assert p + "mlp.correction" not in names
    needs = model.cache_needs()
    for run, i in enumerate(plan.order):
        need, m = needs[caches[run]], cfg["layers"][i]["mixer"]
        assert need.block_state == cfg["width"]                          # the token shift's row, per run
        if cfg["layers"][i]["type"] == "hgrn2":
            assert need.kind == "none" and need.state_shape == (m["heads"], m["dim"], m["vdim"])
        else:
            assert need.kind == ("window" if m.get("mask") else "full") and need.window == (m.get("mask") or {}).get("size")
            assert (need.num_kv_heads, need.head_dim, need.value_dim) == (1, m["kv_rank"] + m["rot_dim"], m["kv_rank"])


@pytest.mark.parametrize("change,message", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].update(eps=0.0), "eps"),
    (lambda c: c["token_side"].update(dim=0), "token_side"),
    (lambda c: c["layers"][0].update(type="attention"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"].update(kv_rank=600), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"].update(q_rank=0), "q_rank"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "mask.size"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=5), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=8), "rot.dims"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(base=0.0), "rot.base"),
    (lambda c: c["layers"][1]["mixer"].update(dim=300), "dim"),
    (lambda c: c["layers"][1]["mixer"].update(heads=0), "heads"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "kind"),
    (lambda c: c["layers"][0]["mlp"]["shared"].update(ff=0), "shared.ff"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].update(times=0), "loop"),
])
def test_configuration_faults_are_named(change, message):
    import qwen3_b200 as q
    cfg = case("A")
    change(cfg)
    with pytest.raises(q.ConfigError, match=message):
        q.config_from_dict(cfg)


def test_optional_mechanisms_may_be_absent_or_null():
    import qwen3_b200 as q
    cfg = case("A")
    bare = copy.deepcopy(cfg)
    bare["loop"], bare["token_side"] = None, None
    for layer in bare["layers"]:
        layer["mlp"] = None
        layer["mixer"].pop("mask", None)
        layer["mixer"].pop("q_rank", None)
    plan = q.config_from_dict(bare).plan()
    assert plan.order == [0, 1, 2, 3] and plan.caches is None
    names = set(q.build_model(plan).weight_specs())
    assert "side.embed" not in names and "l0.mix.q" in names and "l0.mix.dq" not in names and "l0.mlp.router" not in names
    assert q.build_model(plan).cache_needs()[0].kind == "full"


def test_recurrence_equals_its_sum_form():
    """o_t = sum_(j <= t) q_t . ((1 - f_j) prod_(j < s <= t) f_s) v_j, channel by channel: the recurrence of the plain
    implementation against the sum, with a gate that is bounded from below."""
    rng = np.random.default_rng(0)
    T, H, d, vd, width = 30, 2, 5, 4, 12
    m = {"heads": H, "dim": d, "vdim": vd}
    w = {"q": rng.standard_normal((H * d, width)), "f": rng.standard_normal((H * d, width)), "f.b": rng.standard_normal(H * d),
         "lower": rng.uniform(0, 0.9, H * d), "v": rng.standard_normal((H * vd, width)), "norm": np.ones(vd), "o": np.eye(H * vd)}
    h = rng.standard_normal((T, width)) * 0.5
    got = plain.hgrn2_mixer(h, w, "", m, 1e-6)
    q, v = plain.silu(h @ w["q"].T), h @ w["v"].T
    f = w["lower"] + (1 - w["lower"]) * plain.sigmoid(h @ w["f"].T + w["f.b"])
    assert f.min() >= w["lower"].min() and f.max() < 1.0
    o = np.zeros((T, H, vd))
    for head in range(H):
        ch = slice(head * d, (head + 1) * d)
        for t in range(T):
            for j in range(t + 1):
                keep = np.prod(f[j + 1:t + 1, ch], axis=0)
                o[t, head] += (q[t, ch] * keep * (1 - f[j, ch])).sum() * v[j, head * vd:(head + 1) * vd]
    assert np.allclose(got, plain.rms_unit(o, 1e-6).reshape(T, H * vd), atol=1e-10)


def test_router_takes_the_largest_logits_and_weighs_them_among_themselves():
    z = np.array([[0.1, 2.0, -1.0, 1.0, 2.0]])
    ids, weights = plain.router_choice(z, np.eye(5), 3)
    assert list(ids[0]) == [1, 4, 3]                                       # equal logits: the lower index first
    e = np.exp(np.array([2.0, 2.0, 1.0]))
    assert np.allclose(weights[0], e / e.sum()) and np.isclose(weights.sum(), 1.0)
    ids, weights = plain.router_choice(z, np.eye(5), 1)
    assert list(ids[0]) == [1] and np.allclose(weights, 1.0)


def test_sink_takes_weight_without_giving_a_value():
    """One key, score 0: the output is v / (1 + exp(sink)); a very negative sink is plain softmax."""
    q, k, v = np.zeros((1, 1, 4)), np.ones((1, 1, 4)), np.full((1, 1, 3), 2.0)
    for sink in (-30.0, 0.0, 1.5):
        out = plain.masked_softmax_attention(q, k, v, 1.0, None, np.array([sink]))
        assert np.allclose(out, 2.0 / (1.0 + np.exp(sink)))


def test_rotations_pair_neighbours_or_halves():
    v = np.arange(1.0, 9.0).reshape(1, 8)
    a = plain.rotary(v, [3], 100.0, 4, True)
    b = plain.rotary(v, [3], 100.0, 4, False)
    ang = [3.0, 3.0 * 100.0 ** -0.5]
    assert np.allclose(a[0, :2], [1 * np.cos(ang[0]) - 2 * np.sin(ang[0]), 2 * np.cos(ang[0]) + 1 * np.sin(ang[0])])
    assert np.allclose(b[0, [0, 2]], [1 * np.cos(ang[0]) - 3 * np.sin(ang[0]), 3 * np.cos(ang[0]) + 1 * np.sin(ang[0])])
    assert np.allclose(b[0, [1, 3]], [2 * np.cos(ang[1]) - 4 * np.sin(ang[1]), 4 * np.cos(ang[1]) + 2 * np.sin(ang[1])])
    assert np.array_equal(a[0, 4:], v[0, 4:]) and np.array_equal(b[0, 4:], v[0, 4:])      # the rest passes unchanged


def test_decided_routers_choose_the_same_experts_for_every_token():
    import qwen3_b200 as q
    cfg = case("A")
    specs = q.build_model(q.config_from_dict(cfg).plan()).weight_specs()
    w = {k: v.double().numpy() for k, v in decide_routers(lively_weights(specs, 3), 4).items()}
    rng = np.random.default_rng(1)
    x = rng.standard_normal((200, cfg["width"])) * 3
    n2 = plain.dynamic_tanh(x, w, "l0.norm2")
    ids, weights = plain.router_choice(n2, w["l0.mlp.router"], 2)
    assert len({tuple(sorted(r)) for r in ids}) == 1 and weights.min() > 0.02 and np.ptp(weights[:, 0]) > 0.05
