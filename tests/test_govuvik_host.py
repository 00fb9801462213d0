"""Govuvik on the host: configuration and plan, tensor names and state sizes, the random-weights folder, and the
plain implementation's own mechanisms against independent closed forms."""
import copy
import json
import math

import numpy as np
import pytest

import helpers
import plain_govuvik as P


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


RAW = {"architecture": "Govuvik", "width": 40, "vocab": 70, "norm": {"eps": 1e-5}, "canon": {"taps": 3}, "logit_softcap": 9.0,
       "layers": [
           {"type": "parallel",
            "mixer": {"left": {"conv": 2, "dim": 12, "heads": 6, "kv_heads": 3, "vdim": 10, "scale": 0.3, "mask": {"size": 11},
                               "rot": {"base": 500.0, "dims": 8, "scaling": {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 20}}},
                      "right": {"heads": 2, "dim": 6, "vdim": 14, "tau": 5.0, "decay_rank": 7}},
            "mlp": moe(5, 2, 12)},
           {"type": "mlstm", "mixer": {"heads": 3, "dim": 10, "vdim": 6, "gate_cap": 4.0}, "mlp": None},
           {"type": "parallel",
            "mixer": {"left": {"dim": 8, "heads": 2, "kv_heads": 2, "vdim": 8, "scale": 0.5},
                      "right": {"heads": 1, "dim": 4, "vdim": 4, "tau": 1.0, "decay_rank": 2}},
            "mlp": moe(3, 3, 8)},
       ]}


def plan_of(raw):
    import cajeta_llm_b200  # noqa: F401
    from cajeta_llm_b200.config import parse_config_dict
    from cajeta_llm_b200.config.base import get_architecture
    cfg = parse_config_dict(raw)
    return cfg, get_architecture(cfg.architecture).build_plan(cfg)


def test_the_plan_follows_the_list_of_layers():
    cfg, plan = plan_of(RAW)
    assert [l.block.kind for l in plan.layers] == ["sandwich"] * 3
    assert [l.mixer.kind for l in plan.layers] == ["side_by_side", "mlstm", "side_by_side"]
    assert [None if l.feed_forward is None else l.feed_forward.kind for l in plan.layers] == ["sparse_moe", None, "sparse_moe"]
    assert [e.layer for e in plan.schedule] == [0, 1, 2]
    assert plan.layers[0].block["input_conv"] == {"taps": 3, "name": "canon1"}
    left, right = plan.layers[0].mixer["left"], plan.layers[0].mixer["right"]
    assert left.kind == "attention" and right.kind == "gla" and plan.layers[0].mixer["coef"] == 0.5
    assert left["window"] == 11 and left["scale"] == 0.3 and left["value_dim"] == 10 and left["proj_conv"]["taps"] == 2
    assert left["qk_norm"]["whole"] and left["head_temp"] == "temp" and left["talk"] == "talk" and left["sink"] == "sink"
    assert left["position"].kind == "rope" and left["position"]["rotary_dim"] == 8 and left["position"]["scaling"]["kind"] == "wavelength"
    assert right["tau"] == 5.0 and right["decay_rank"] == 7
    bare = plan.layers[2].mixer["left"]
    assert bare["window"] == 0 and bare["position"].kind == "none" and "proj_conv" not in bare.params
    memory = plan.layers[1].mixer
    assert memory["gate_cap"] == 4.0 and memory["floor"] == 1e-6 and memory["eps"] == 1e-5
    ff = plan.layers[0].feed_forward
    assert ff["activation"] == "relu2" and ff["top_k"] == 2 and ff["norm_topk_prob"] and ff["score"] == "softmax"
    assert plan.head["softcap"] == 9.0 and plan.embedding["norm"]["weight_name"] == "embed.norm"
    assert cfg.to_json_dict() == RAW


def test_a_model_without_the_optional_pieces():
    raw = {k: v for k, v in RAW.items() if k not in ("canon", "logit_softcap")}
    cfg, plan = plan_of(raw)
    assert "input_conv" not in plan.layers[0].block.params and plan.head["softcap"] == 0.0
    assert cfg.to_json_dict() == raw
    from cajeta_llm_b200.engine.model import build_model
    from cajeta_llm_b200.parts.base import Runtime
    assert not any(n.endswith("canon1") for n in build_model(cfg, Runtime("float32", "cpu")).params())


def test_tensor_names_shapes_and_needs():
    from cajeta_llm_b200.csrc import kernels as K
    from cajeta_llm_b200.engine.model import build_model
    from cajeta_llm_b200.parts.base import Runtime
    cfg, _ = plan_of(RAW)
    model = build_model(cfg, Runtime("float32", "cpu"))
    p = {n: tuple(s.shape) for n, s in model.params().items()}
    assert p["embed"] == (70, 40) and p["embed.norm"] == (40,) and p["head"] == (70, 40) and p["final.norm"] == (40,)
    for n in ("norm1", "norm1b", "norm2", "norm2b"):
        assert p[f"l0.{n}"] == (40,)
    assert "l1.norm2" not in p and "l1.norm2b" not in p and p["l1.norm1b"] == (40,)
    assert p["l0.canon1"] == (40, 3) and p["l1.canon1"] == (40, 3)
    assert p["l0.mix.left.q"] == (72, 40) and p["l0.mix.left.k"] == (36, 40) and p["l0.mix.left.v"] == (30, 40)
    assert p["l0.mix.left.o"] == (40, 60) and p["l0.mix.left.q.norm"] == (72,) and p["l0.mix.left.k.norm"] == (36,)
    assert p["l0.mix.left.q.conv"] == (72, 2) and p["l0.mix.left.k.conv"] == (36, 2) and p["l0.mix.left.v.conv"] == (30, 2)
    assert p["l0.mix.left.talk"] == (6, 6) and p["l0.mix.left.temp"] == (6,) and p["l0.mix.left.sink"] == (6,)
    assert p["l0.mix.left.out"] == (40,) and p["l0.mix.right.out"] == (40,)
    assert p["l0.mix.right.q"] == (12, 40) and p["l0.mix.right.v"] == (28, 40) and p["l0.mix.right.g"] == (28, 40)
    assert p["l0.mix.right.a1"] == (7, 40) and p["l0.mix.right.a2"] == (12, 7) and p["l0.mix.right.a2.b"] == (12,)
    assert p["l0.mix.right.norm"] == (14,) and p["l0.mix.right.o"] == (40, 28)
    assert "l2.mix.left.q.conv" not in p and p["l2.mix.left.q.norm"] == (16,)
    assert p["l1.mix.q"] == (30, 40) and p["l1.mix.v"] == (18, 40) and p["l1.mix.g"] == (18, 40) and p["l1.mix.o"] == (40, 18)
    assert p["l1.mix.i"] == (3, 40) and p["l1.mix.f.b"] == (3,) and p["l1.mix.norm"] == (18,)
    assert p["l0.mlp.router"] == (5, 40) and p["l0.mlp.e4.up"] == (12, 40) and p["l0.mlp.e0.down"] == (40, 12)
    assert not any("gate" in n for n in p) and not any(n.startswith("l1.mlp") for n in p)
    kv = model.kv_needs()
    assert (kv[0].kv_heads, kv[0].head_dim, kv[0].value_dim, kv[0].window) == (3, 12, 10, 11) and kv[1] is None and kv[2].window == 0
    # a request's state, layer by layer: the input convolution's rows, the projections' rows, the matrices
    st = model.state_needs()
    assert st[0].shape == (2 * 40 + 1 * (72 + 36 + 30) + K.state_scan_floats(2, 6, 14, K.SCAN_GLA),)
    assert st[1].shape == (2 * 40 + K.state_scan_floats(3, 10, 6, K.SCAN_MLSTM),)
    assert st[2].shape == (2 * 40 + K.state_scan_floats(1, 4, 4, K.SCAN_GLA),)


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="attention"), "type"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=4), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "dims"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"]["scaling"].pop("high"), "high"),
    (lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(size=0), "size"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(tau=0), "tau"),
    (lambda c: c["layers"][1]["mixer"].pop("gate_cap"), "gate_cap"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=0), "vdim"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "kind"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "top"),
    (lambda c: c["canon"].update(taps=0), "taps"),
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


def test_random_weights_folder_round_trip_and_the_rank_from_the_tensor(tmp_path):
    helpers.write_model(str(tmp_path), RAW, seed=3)
    cfg, W = P.read_model(str(tmp_path))
    assert cfg == RAW and W["l0.mix.left.talk"].shape == (6, 6) and W["l0.mix.right.a1"].shape == (7, 40)
    logits, after = P.forward(cfg, W, [1, 2, 3, 4, 5], keep_layers=True)
    assert logits.shape == (5, 70) and after.shape == (3, 5, 40) and bool(np.isfinite(logits).all())
    assert float(np.abs(logits).max()) < 9.0
    # a folder whose configuration does not give the decay's inner size: the tensor's shape does
    bare = copy.deepcopy(RAW)
    for layer in bare["layers"]:
        if layer["type"] == "parallel":
            layer["mixer"]["right"].pop("decay_rank")
    with open(tmp_path / "config.json", "w") as f:
        json.dump(bare, f)
    from cajeta_llm_b200.config import load_config
    from cajeta_llm_b200.config.base import get_architecture
    parsed = load_config(str(tmp_path))
    plan = get_architecture(parsed.architecture).build_plan(parsed)
    assert plan.layers[0].mixer["right"]["decay_rank"] == 7 and plan.layers[2].mixer["right"]["decay_rank"] == 2


def test_the_engine_s_frequency_table_equals_the_plain_one():
    from cajeta_llm_b200.parts.base import Runtime, make_part
    from cajeta_llm_b200.parts.plan import PartSpec
    for rot in ({"base": 500.0, "dims": 8, "scaling": {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 20}},
                {"base": 250000.0, "dims": 48, "scaling": {"factor": 16.0, "low": 0.5, "high": 8.0, "original": 300}},
                {"base": 100.0, "dims": 12, "scaling": {"factor": 2.0, "low": 2.0, "high": 2.5, "original": 9}},
                {"base": 10000.0, "dims": 16}):
        sc = rot.get("scaling")
        part = make_part("position", PartSpec("rope", {"head_dim": 64, "rotary_dim": rot["dims"], "theta": rot["base"],
                                                       "scaling": dict(sc, kind="wavelength") if sc else None}), "", Runtime("float32", "cpu"))
        want = P.rope_frequencies(rot)
        assert part.magnitude == 1.0 and np.allclose(part.inv_freq.double().numpy(), want, rtol=1e-6, atol=0.0)
        if sc:      # the three regimes are all there in the first two tables: some kept, some divided
            plain = np.array([rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)])
            assert want[0] == plain[0] and abs(want[-1] - plain[-1] / sc["factor"]) < 1e-15 or rot["dims"] == 12


# -- the plain implementation's mechanisms against closed forms of their own --------------
def test_rotation_pairs_entry_i_with_i_plus_half_and_keeps_relative_angles():
    g = np.random.default_rng(1)
    f = P.rope_frequencies({"base": 100.0, "dims": 4})
    e = P.rotate_half(np.array([[1.0, 0.0, 0.0, 0.0, 5.0, 6.0]]), 2, f, 4)
    assert np.allclose(e[0], [math.cos(2.0), 0.0, math.sin(2.0), 0.0, 5.0, 6.0])
    q, k = g.standard_normal((1, 6)), g.standard_normal((1, 6))
    a = (P.rotate_half(q, 7, f, 4)[0, :4] * P.rotate_half(k, 3, f, 4)[0, :4]).sum()
    b = (P.rotate_half(q, 14, f, 4)[0, :4] * P.rotate_half(k, 10, f, 4)[0, :4]).sum()
    assert abs(a - b) < 1e-12


def test_convolution_is_causal_and_ends_on_the_newest_input():
    u = np.arange(1.0, 6.0)[:, None] * np.ones((1, 2))
    w = np.array([[100.0, 10.0, 1.0], [0.0, 0.0, 2.0]])
    y = P.causal_conv(u, w)
    assert y[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0, 345.0] and y[:, 1].tolist() == [2.0, 4.0, 6.0, 8.0, 10.0]


def test_router_weights_are_the_softmax_over_the_picked_logits_alone():
    z = np.array([0.5, 3.0, -1.0, 2.0, 2.0])
    order, w, gap = P.route(z, 3)
    assert order == [1, 3, 4] and abs(gap - 1.5) < 1e-12
    e = np.exp([3.0, 2.0, 2.0])
    assert np.allclose(w, e / e.sum())
    assert P.route(z, 1)[0] == [1] and np.allclose(P.route(z, 1)[1], [1.0]) and P.route(z, 5)[2] == float("inf")


def test_attention_sink_window_and_mixed_heads_by_hand():
    # two heads, one key head, width 2; identity projections; queries and keys are the (normed) inputs
    m = {"heads": 2, "kv_heads": 1, "dim": 2, "vdim": 2, "scale": 1.0, "mask": {"size": 2}}
    eye = np.eye(2)
    W = {"q": np.vstack([eye, eye]), "k": eye, "v": eye, "o": np.hstack([eye, eye]), "q.norm": np.ones(4), "k.norm": np.ones(2),
         "temp": np.array([1.0, 2.0]), "talk": np.array([[1.0, 0.0], [0.5, 0.5]]), "sink": np.array([0.0, -np.inf])}
    h = np.array([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]])
    out = P.windowed_attention(m, W, "", h, 0.0)
    # row 2 sees rows 1 and 2 only; q = h / rms(q over both heads) = h / 1, k = h / rms(h) = h
    k = h / np.sqrt((h * h).mean(-1, keepdims=True))
    q2 = np.array([1.0, 1.0])
    raw0 = np.array([k[1] @ q2, k[2] @ q2])
    s0, s1 = raw0, 0.5 * raw0 + 0.5 * 2.0 * raw0
    w0 = np.exp(s0) / (np.exp(s0).sum() + 1.0)                       # the divisor's extra term: e^sink with sink = 0
    w1 = np.exp(s1) / np.exp(s1).sum()                               # no sink for head 1
    want = w0 @ h[1:3] + w1 @ h[1:3]
    assert np.allclose(out[2], want)


def test_matrix_memory_first_steps_by_hand():
    m = {"heads": 1, "dim": 1, "vdim": 1, "gate_cap": 100.0}
    W = {"q": np.array([[1.0]]), "k": np.array([[1.0]]), "v": np.array([[1.0]]), "g": np.array([[0.0]]), "o": np.array([[1.0]]),
         "norm": np.ones(1), "i": np.array([[1.0]]), "i.b": np.zeros(1), "f": np.array([[0.0]]), "f.b": np.zeros(1)}
    # one channel: the read-out is +-1 after the unit norm; the sign and the finite values are what is checked,
    # then the state itself through a second head size
    out = P.mlstm_mixer(m, W, "", np.array([[2.0], [-3.0]]), 0.0)
    assert out.shape == (2, 1) and np.allclose(np.abs(out), 0.5) and out[0, 0] > 0


def test_decay_acts_on_the_rows_of_key_channels():
    m = {"heads": 1, "dim": 2, "vdim": 1, "tau": 2.0}
    big = 50.0
    W = {"q": np.array([[1.0], [1.0]]) * math.sqrt(2.0), "k": np.array([[1.0], [1.0]]), "v": np.array([[1.0]]), "g": np.array([[1.0]]),
         "o": np.array([[1.0]]), "norm": np.ones(1), "a1": np.array([[0.0]]), "a2": np.zeros((2, 1)), "a2.b": np.array([big, 0.0])}
    # channel 0 keeps (sigmoid(50)^(1/2) = 1), channel 1 decays by sigmoid(0)^(1/2) = sqrt(1/2) a step
    h = np.array([[1.0], [1.0], [1.0]])
    T = 3
    S = np.zeros(2)
    o = []
    for t in range(T):
        S = np.array([1.0, math.sqrt(0.5)]) * S + 1.0
        o.append(S.sum())
    got = P.gated_linear_attention(m, W, "", h, 0.0)
    gate = 1.0 / (1.0 + math.exp(-1.0))
    assert np.allclose(got[:, 0], np.sign(o) * gate)                # a head of one value: its norm leaves the sign
    m2 = dict(m, vdim=2)
    W2 = dict(W, v=np.array([[1.0], [3.0]]), g=np.array([[1.0], [1.0]]), o=np.eye(2), norm=np.ones(2))
    got = P.gated_linear_attention(m2, W2, "", h, 0.0)
    want = np.array([1.0, 3.0]) / math.sqrt(5.0) * gate
    assert np.allclose(got, np.tile(want, (3, 1)))


def test_command_line_writes_a_random_model_folder(tmp_path):
    import subprocess
    import sys
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(RAW))
    out = tmp_path / "model"
    r = subprocess.run([sys.executable, "-m", "cajeta_llm_b200", "random-weights", "--config", str(cfg), "--seed", "4", "--out", str(out)],
                       cwd=helpers.ROOT, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-1000:]
    config, W = P.read_model(str(out))
    assert config == RAW and W["l1.mix.i.b"].shape == (3,) and W["l0.mlp.e4.down"].shape == (40, 12)
