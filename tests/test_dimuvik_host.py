"""Dimuvik on the host: configuration and plan, tensor names, cache and state needs, the random-weights folder, and
the plain implementation's own mechanisms against independent closed forms."""
import copy
import json
import math

import numpy as np
import pytest

import helpers
import plain_dimuvik as P

RAW = {"architecture": "Dimuvik", "width": 40, "vocab": 70, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.5},
       "layers": [
           {"type": "latent_attention",
            "mixer": {"heads": 3, "dim": 10, "rot_dim": 6, "vdim": 14, "kv_rank": 20, "q_rank": 12, "rot": {"base": 300.0, "dims": 4},
                      "scale": 0.3},
            "mlp": {"kind": "dense", "ff": 56}},
           {"type": "attention",
            "mixer": {"heads": 6, "kv_heads": 2, "dim": 4, "vdim": 10, "conv": 3, "diff": 0.35, "scale": 0.5,
                      "q_temp": {"coef": 0.4, "every": 7}},
            "mlp": {"kind": "moe", "expert": {"ff": 12}, "router": {"experts": 5, "top": 2, "scale": 1.7}, "shared": {"ff": 20}}},
           {"type": "latent_attention",
            "mixer": {"heads": 2, "dim": 5, "rot_dim": 6, "vdim": 7, "kv_rank": 20, "q_rank": 9, "rot": {"base": 300.0, "dims": 4},
                      "scale": 0.2, "kv_from": 0},
            "mlp": None},
           {"type": "attention",
            "mixer": {"heads": 2, "kv_heads": 2, "dim": 4, "vdim": 10, "conv": 3, "diff": 0.8, "scale": 0.25, "kv_from": 1},
            "mlp": {"kind": "moe", "expert": {"ff": 8}, "router": {"experts": 3, "top": 3, "scale": 1.0}}},
       ]}


def plan_of(raw):
    import cajeta_llm_b200  # noqa: F401
    from cajeta_llm_b200.config import parse_config_dict
    from cajeta_llm_b200.config.base import get_architecture
    cfg = parse_config_dict(raw)
    return cfg, get_architecture(cfg.architecture).build_plan(cfg)


def test_the_plan_follows_the_list_of_layers():
    cfg, plan = plan_of(RAW)
    assert [l.block.kind for l in plan.layers] == ["sandwich"] * 4
    assert [l.mixer.kind for l in plan.layers] == ["latent_attention", "differential_attention"] * 2
    assert [None if l.feed_forward is None else l.feed_forward.kind for l in plan.layers] == ["dense_relu2", "sparse_moe", None, "sparse_moe"]
    assert [(e.layer, e.cache_from) for e in plan.schedule] == [(0, None), (1, None), (2, 0), (3, 1)]
    assert plan.final_norm.kind == "dyt" and all(l.mixer_norm.kind == "dyt" for l in plan.layers)
    assert plan.embedding["scale"] == 2.5
    lat = plan.layers[0].mixer
    assert (lat["q_rank"], lat["kv_rank"], lat["rot_dim"], lat["gate"], lat["sink"], lat["owns_cache"]) == (12, 20, 6, False, "sink", True)
    assert lat["position"].kind == "rope" and lat["position"]["rotary_dim"] == 4 and lat["position"]["theta"] == 300.0
    assert not plan.layers[2].mixer["owns_cache"]
    att = plan.layers[1].mixer
    assert (att["num_heads"], att["num_kv_heads"], att["head_dim"], att["value_dim"]) == (6, 2, 4, 10)
    assert att["lambda_init"] == 0.35 and att["scale"] == 0.5 and att["bias"] and att["proj_conv"] == {"taps": 3}
    assert att["q_temp"] == {"coef": 0.4, "every": 7}
    borrowed = plan.layers[3].mixer
    assert not borrowed["owns_cache"] and "q_temp" not in borrowed.params
    ff = plan.layers[1].feed_forward
    assert (ff["top_k"], ff["route_scale"], ff["correction"], ff["shared_intermediate_size"], ff["norm_topk_prob"]) == (2, 1.7, "correction", 20, False)
    assert plan.layers[3].feed_forward["shared_intermediate_size"] == 0
    assert plan.launch_overlap is True
    assert cfg.to_json_dict() == RAW


def test_tensor_names_shapes_and_needs():
    from cajeta_llm_b200.engine.model import build_model
    from cajeta_llm_b200.parts.base import Runtime
    cfg, _ = plan_of(RAW)
    model = build_model(cfg, Runtime("float32", "cpu"))
    p = {n: tuple(s.shape) for n, s in model.params().items()}
    for norm in ("l0.norm1", "l0.norm1b", "l0.norm2", "l0.norm2b", "l2.norm1", "l2.norm1b", "final.norm"):
        assert p[norm] == (40,) and p[norm + ".b"] == (40,) and p[norm + ".alpha"] == ()
    assert "l2.norm2" not in p and "l2.norm2b.alpha" not in p
    assert p["l0.mix.dq"] == (12, 40) and p["l0.mix.dq.norm"] == (12,) and p["l0.mix.uq"] == (3 * 16, 12)
    assert p["l0.mix.dkv"] == (26, 40) and p["l0.mix.dkv.norm"] == (20,) and p["l0.mix.uk"] == (30, 20) and p["l0.mix.uv"] == (42, 20)
    assert p["l0.mix.sink"] == (3,) and p["l0.mix.o"] == (40, 42) and "l0.mix.g" not in p and "l0.mix.q" not in p
    assert "l2.mix.dkv" not in p and "l2.mix.dkv.norm" not in p and p["l2.mix.uk"] == (10, 20)
    assert p["l1.mix.q"] == (48, 40) and p["l1.mix.k"] == (16, 40) and p["l1.mix.v"] == (20, 40)
    assert p["l1.mix.q.b"] == (48,) and p["l1.mix.k.conv"] == (16, 3) and p["l1.mix.v.conv"] == (20, 3)
    assert all(p[f"l1.mix.{n}"] == (4,) for n in ("lq1", "lk1", "lq2", "lk2")) and p["l1.mix.o"] == (40, 60)
    assert p["l3.mix.q"] == (16, 40) and p["l3.mix.q.conv"] == (16, 3) and not any(n.startswith("l3.mix.k") or n.startswith("l3.mix.v") for n in p)
    assert p["l0.mlp.up"] == (56, 40) and p["l0.mlp.down"] == (40, 56) and "l0.mlp.gate" not in p
    assert p["l1.mlp.router"] == (5, 40) and p["l1.mlp.correction"] == (5,) and p["l1.mlp.e4.gate"] == (12, 40)
    assert p["l1.mlp.shared.up"] == (20, 40) and p["l1.mlp.shared.down"] == (40, 20) and "l3.mlp.shared.up" not in p
    assert p["embed"] == (70, 40) and p["head"] == (70, 40)
    kv = model.kv_needs()
    assert (kv[0].kv_heads, kv[0].head_dim, kv[0].values) == (1, 26, False) and kv[2] == kv[0]
    assert (kv[1].kv_heads, kv[1].head_dim, kv[1].value_dim, kv[1].window) == (2, 8, 10, 0) and kv[3] == kv[1]
    # the convolutions' last inputs: q, k and v of the layer that owns its cache, q alone of the one that borrows
    st = model.state_needs()
    assert st[0] is None and st[2] is None and st[1].shape == (2 * (48 + 16 + 20),) and st[3].shape == (2 * 16,)
    assert model.cache_from() == [None, None, 0, 1]


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="mamba"), "type"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=4), "multiple"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"].pop("diff"), "diff"),
    (lambda c: c["layers"][1]["mixer"]["q_temp"].update(every=0), "every"),
    (lambda c: c["layers"][1]["mixer"].update(conv=0), "conv"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=8), "dims"),
    (lambda c: c["layers"][0]["mixer"].pop("q_rank"), "q_rank"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=21), "kv_rank"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=11), "vdim"),
    (lambda c: c["layers"][0]["mlp"].update(kind="gated"), "kind"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=6), "top"),
    (lambda c: c["layers"][1]["mlp"]["shared"].update(ff=0), "ff"),
    (lambda c: c["embedding"].update(scale=0), "embedding.scale"),
    (lambda c: c.pop("norm"), "norm.eps"),
    (lambda c: c.pop("layers"), "layers"),
])
def test_configuration_errors_name_the_key(change, message):
    from cajeta_llm_b200.config.base import ConfigError
    raw = copy.deepcopy(RAW)
    change(raw)
    with pytest.raises(ConfigError) as e:
        plan_of(raw)
    assert message in str(e.value)


def test_random_weights_folder_round_trip(tmp_path):
    helpers.write_model(str(tmp_path), RAW, seed=3)
    cfg, W = P.load_folder(str(tmp_path))
    assert cfg == RAW and W["l1.mix.k.conv"].shape == (16, 3) and W["final.norm.alpha"].shape == ()
    after = []
    logits = P.forward(cfg, W, [1, 2, 3, 4, 5], layer_outputs=after)
    assert logits.shape == (5, 70) and len(after) == 4 and after[0].shape == (5, 40) and bool(np.isfinite(logits).all())
    # a model without an embedding scale reads as scale 1
    bare = {k: v for k, v in RAW.items() if k != "embedding"}
    cfg2, plan = plan_of(bare)
    assert cfg2.embedding_scale == 1.0 and plan.embedding["scale"] == 0.0


def test_the_engine_s_frequency_table_equals_the_plain_one():
    from cajeta_llm_b200.parts.base import Runtime, make_part
    from cajeta_llm_b200.parts.plan import PartSpec
    for base, dims in ((300.0, 4), (500000.0, 32), (10000.0, 16)):
        part = make_part("position", PartSpec("rope", {"head_dim": dims, "rotary_dim": dims, "theta": base}), "", Runtime("float32", "cpu"))
        want = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])
        assert np.allclose(part.inv_freq.double().numpy(), want, rtol=1e-6)


def test_rotation_pairs_neighbours_and_keeps_relative_angles():
    rng = np.random.default_rng(0)
    a, b = rng.normal(size=10), rng.normal(size=10)
    # the product of two rotated vectors depends on the distance alone; entries past `dims` pass unchanged
    d1 = P.rotate_pairs(a, 17, 100.0, 6) @ P.rotate_pairs(b, 12, 100.0, 6)
    d2 = P.rotate_pairs(a, 105, 100.0, 6) @ P.rotate_pairs(b, 100, 100.0, 6)
    assert abs(d1 - d2) < 1e-9
    assert np.array_equal(P.rotate_pairs(a, 9, 100.0, 6)[6:], a[6:])
    one = P.rotate_pairs(np.array([1.0, 0.0, 0.0, 0.0]), 3, 100.0, 4)
    assert np.allclose(one, [math.cos(3.0), math.sin(3.0), 0.0, 0.0])


def test_convolution_is_causal_and_ends_on_the_newest_input():
    u = np.arange(12.0).reshape(6, 2)
    w = np.array([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]])
    y = P.causal_conv(u, w)
    assert np.array_equal(y[:, 0], u[:, 0])                                       # the last tap is the row itself
    assert np.array_equal(y[:, 1], np.concatenate([[0.0, 0.0], u[:-2, 1]]))       # the first tap lies taps - 1 rows back


def test_the_sink_counts_once_and_has_no_value():
    s = np.array([0.3, -1.0, 2.0])
    w = P.softmax_rows(s, sink=1.5)
    e = np.exp(s)
    assert np.allclose(w, e / (e.sum() + math.exp(1.5))) and w.sum() < 1.0
    assert np.allclose(P.softmax_rows(s).sum(), 1.0)


def test_the_query_temperature_steps_with_the_position():
    assert P.query_temperature(0, 0.5, 4) == 1.0 and P.query_temperature(2, 0.5, 4) == 1.0
    assert math.isclose(P.query_temperature(3, 0.5, 4), 1.0 + 0.5 * math.log(2.0))
    assert math.isclose(P.query_temperature(6, 0.5, 4), 1.0 + 0.5 * math.log(2.0))
    assert math.isclose(P.query_temperature(7, 0.5, 4), 1.0 + 0.5 * math.log(3.0))


def test_differential_attention_by_hand():
    """One head, one key head, two tokens, no convolution to speak of, identity projections: the second row's two maps
    by hand, their difference, the norm."""
    m = {"heads": 1, "kv_heads": 1, "dim": 1, "vdim": 2, "diff": 0.25, "scale": 1.0}
    W = {".q": np.eye(2), ".q.b": np.zeros(2), ".q.conv": np.array([[0.0, 1.0]] * 2), ".o": np.eye(2),
         ".lq1": np.array([0.5]), ".lk1": np.array([2.0]), ".lq2": np.array([1.0]), ".lk2": np.array([0.0])}
    h = np.array([[1.0, 2.0], [0.5, -1.0]])
    k = np.array([[1.0, 0.0], [2.0, 1.0]])
    v = np.array([[1.0, 0.0], [0.0, 3.0]])
    got = P.differential_attention(h, W, "", m, 1e-6, k, v)
    lam = math.exp(1.0) - math.exp(0.0) + 0.25
    q1, q2 = 0.5, -1.0
    w1 = np.exp([q1 * 1.0, q1 * 2.0]); w1 /= w1.sum()
    w2 = np.exp([q2 * 0.0, q2 * 1.0]); w2 /= w2.sum()
    o = w1 @ v - lam * (w2 @ v)
    want = o / math.sqrt(np.mean(o * o) + 1e-6) * 0.75
    assert np.allclose(got[1], want)
    assert np.allclose(got[0], np.array([1.0 - lam, 0.0]) / math.sqrt((1.0 - lam) ** 2 / 2 + 1e-6) * 0.75)


def test_the_router_chooses_with_the_correction_and_weighs_without_it():
    W = {".router": np.array([[2.0, 0.0], [1.0, 0.0], [0.0, 0.0]]), ".correction": np.array([-0.6, 0.0, 0.4])}
    ff = {"router": {"experts": 3, "top": 2, "scale": 3.0}}
    picks, weights = P.route(np.array([[1.0, 5.0]]), W, "", ff)
    s = np.exp([2.0, 1.0, 0.0]); s /= s.sum()
    assert picks.tolist() == [[2, 1]]                       # 0.09 + 0.4, 0.245, 0.665 - 0.6
    assert np.allclose(weights, [[3.0 * s[2], 3.0 * s[1]]])


def test_the_norm_without_statistics():
    W = {"n": np.array([2.0, -1.0]), "n.b": np.array([0.5, 0.25]), "n.alpha": np.asarray(0.7)}
    x = np.array([[1.0, -3.0]])
    assert np.allclose(P.dyt(x, W, "n"), [[math.tanh(0.7) * 2.0 + 0.5, -math.tanh(-2.1) + 0.25]])


def test_command_line_writes_a_random_model_folder(tmp_path):
    import subprocess
    import sys
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(RAW))
    out = tmp_path / "model"
    r = subprocess.run([sys.executable, "-m", "cajeta_llm_b200", "random-weights", "--config", str(cfg), "--seed", "4", "--out", str(out)],
                       cwd=helpers.ROOT, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-1000:]
    config, W = P.load_folder(str(out))
    assert config == RAW and W["l1.mix.lq2"].shape == (4,) and W["l1.mlp.e4.down"].shape == (40, 12) and W["l3.norm2b.alpha"].shape == ()
