"""Govuvik through the engine against the plain implementation (``plain_govuvik.py``).

Small configurations of their own whose sizes differ in every field (head groups, picked experts, taps and
ranks that are neither 1 nor equal to one another; values of another size than keys; windows that are no
multiple of a page; a rotation over a part of a head with and without stretched frequencies; layers without
a feed-forward).  Each mechanism alone as a one-layer model; whole prompts against token-by-token decoding
and portions down to two tokens; unequal requests in one batch against each alone; slots and pages used
again; attention made sharp so that single keys - far ones, those at page borders, those just inside and
just outside the window - decide a row, in prompts and in decoding; first tokens; long decoding; greedy
generation through the entry point and its scheduler.
"""
import copy
import json
import math
import os
import random

import numpy as np
import pytest
import torch

import helpers
import plain_govuvik as P

pytestmark = pytest.mark.gpu


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


MEMORY = {"type": "mlstm", "mixer": {"heads": 3, "dim": 10, "vdim": 14, "gate_cap": 2.5}, "mlp": None}
MEMORY_B = {"type": "mlstm", "mixer": {"heads": 2, "dim": 24, "vdim": 8, "gate_cap": 6.0}, "mlp": moe(6, 3, 20)}
PAIR = {"type": "parallel",
        "mixer": {"left": {"conv": 3, "dim": 12, "heads": 6, "kv_heads": 2, "vdim": 20, "scale": 0.4, "mask": {"size": 21},
                           "rot": {"base": 900.0, "dims": 8, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 24}}},
                  "right": {"heads": 3, "dim": 6, "vdim": 10, "tau": 4.0, "decay_rank": 5}},
        "mlp": None}
PAIR_B = {"type": "parallel",
          "mixer": {"left": {"conv": 2, "dim": 16, "heads": 2, "kv_heads": 1, "vdim": 16, "scale": 0.25, "mask": {"size": 37},
                             "rot": {"base": 10000.0, "dims": 16}},
                    "right": {"heads": 1, "dim": 20, "vdim": 12, "tau": 16.0, "decay_rank": 3}},
          "mlp": moe(5, 2, 12)}
PAIR_C = {"type": "parallel",
          "mixer": {"left": {"conv": 4, "dim": 8, "heads": 3, "kv_heads": 3, "vdim": 4, "scale": 0.5, "mask": {"size": 5}},
                    "right": {"heads": 4, "dim": 4, "vdim": 4, "tau": 1.0, "decay_rank": 7}},
          "mlp": moe(9, 1, 16)}


def config_of(layers, width=64, vocab=200, eps=1e-5, taps=4, softcap=12.0):
    return {"architecture": "Govuvik", "width": width, "vocab": vocab, "norm": {"eps": eps}, "canon": {"taps": taps},
            "logit_softcap": softcap, "layers": copy.deepcopy(layers)}


WIDE = [
    {"type": "mlstm", "mixer": {"heads": 4, "dim": 32, "vdim": 64, "gate_cap": 10.0}, "mlp": moe(8, 2, 128)},
    {"type": "parallel",
     "mixer": {"left": {"conv": 3, "dim": 64, "heads": 4, "kv_heads": 2, "vdim": 64, "scale": 0.125, "mask": {"size": 48},
                        "rot": {"base": 50000.0, "dims": 32, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}},
               "right": {"heads": 2, "dim": 32, "vdim": 64, "tau": 8.0, "decay_rank": 12}},
     "mlp": moe(4, 3, 136)},
    {"type": "parallel",
     "mixer": {"left": {"conv": 2, "dim": 128, "heads": 2, "kv_heads": 1, "vdim": 96, "scale": 0.09, "mask": {"size": 70}},
               "right": {"heads": 4, "dim": 16, "vdim": 32, "tau": 2.0, "decay_rank": 16}},
     "mlp": None},
]
CONFIGS = {
    "mixed": config_of([MEMORY, PAIR, PAIR_B, MEMORY_B, PAIR_C]),
    "other": config_of([PAIR_C, MEMORY_B, PAIR], width=72, vocab=150, eps=1e-6, taps=2, softcap=40.0),
    "bare": config_of([PAIR_B, MEMORY], width=40, vocab=90, taps=1, softcap=5.0),
    # wide enough for the tensor-core products of the bfloat16 path
    "wide": config_of(WIDE, width=256, vocab=500, taps=3),
}
ALONE = {"memory": [MEMORY], "memory_b": [MEMORY_B], "pair": [PAIR], "pair_b": [PAIR_B], "pair_c": [PAIR_C]}


def louder(model_dir, sharp=1.0):
    """The random-weights mode draws small values (standard deviation 0.02): every gate would sit at one half,
    every softmax would be flat and the router near a tie everywhere.  What feeds gates, scores and routers is
    multiplied up so that the mechanisms bite; ``sharp`` multiplies the scores' per-head numbers further."""
    from cajeta_llm_b200.weights.safetensors_io import Checkpoint, write_safetensors
    ck = Checkpoint(model_dir)
    tensors = {n: ck.load(n).float() for n in ck.names()}
    ck.close()
    for n, t in tensors.items():
        leaf = n.split(".")[-1]
        g = torch.Generator().manual_seed(len(n) + 7 * t.numel())
        if leaf in ("router", "g", "i", "f", "a1"):
            t *= 15.0
        elif leaf in ("up", "down", "v", "o", "q", "k"):
            t *= 4.0
        elif leaf == "temp":
            t.copy_((1.0 + 2.0 * torch.rand(t.shape, generator=g)) * sharp)
        elif leaf in ("norm", "out", "norm1", "norm2", "norm1b", "norm2b"):
            t += 0.3 * torch.randn(t.shape, generator=g)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), {n: t.to(torch.bfloat16) for n, t in tensors.items()})


def sharp(model_dir):
    louder(model_dir, sharp=6.0)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name, raw, seed=5, touch=louder):
        if name not in made:
            d = str(tmp_path_factory.mktemp(f"govuvik_{name}"))
            helpers.write_model(d, raw, seed=seed)
            if touch is not None:
                touch(d)
            made[name] = (d, P.read_model(d))
        return made[name]
    return get


def runner_for(model_dir, dtype, max_seqs=4, max_tokens=512, num_pages=None, cuda_graphs=True, page=16):
    import cajeta_llm_b200  # noqa: F401
    from cajeta_llm_b200.engine.model import load_model
    from cajeta_llm_b200.engine.step import ModelRunner
    from cajeta_llm_b200.parts.base import Runtime
    model, _ = load_model(model_dir, Runtime(dtype, "cuda:0"))
    return ModelRunner(model, page_tokens=page, max_seqs=max_seqs, max_tokens_per_seq=max_tokens,
                       num_pages=num_pages if num_pages is not None else -(-max_tokens // page) * max_seqs, cuda_graphs=cuda_graphs)


def oracle(cfg, W, tokens):
    """The plain implementation's logits and its picks by the engine's routing keys."""
    picks = {}
    want = torch.from_numpy(P.forward(cfg, W, tokens, picks=picks))
    return want, {k: torch.tensor(v, dtype=torch.int32) for k, v in picks.items()}


def pin_rows(spans):
    """A step's routing pin from [(request's picks, first position, count)] in the step's order."""
    if not spans or not spans[0][0]:
        return None
    return {key: torch.cat([p[key][lo:lo + n] for p, lo, n in spans]).cuda().contiguous() for key in spans[0][0]}


def feed(runner, slot, tokens, cuts, picks=None):
    from cajeta_llm_b200.engine.step import StepEntry
    out, at = [], 0
    for n in cuts:
        pin = pin_rows([(picks, at, n)]) if picks else None
        out.append(runner.step([StepEntry(slot, tokens[at:at + n], list(range(n)))], routing_pin=pin).cpu())
        at += n
    assert at == len(tokens)
    return torch.cat(out)


def rel_err(got, want):
    """Per row: RMS of the difference (mean taken off) over the RMS of the wanted logits."""
    d = got.double() - want.double()
    d = d - d.mean(dim=-1, keepdim=True)
    w = want.double() - want.double().mean(dim=-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt().clamp_min(1e-9)


def check(got, want, dtype, what, free_routing=False):
    """float32: every row to rounding.  bfloat16 with the routing pinned: the median row within 5 % of the logits'
    spread, at most a tenth of the rows (or three) beyond 12 %, none beyond 60 % (the weights are loud, and a row whose
    read-out divides by a sum near zero, or whose gate sits on a steep flank, carries many times the usual rounding
    of the stored activations; a lost key or a lost state moves most rows by the logits' whole spread, and the
    float32 runs hold every row).  With the routing free a row near a tie may swap an expert, and the recurrent
    layers carry that on to later rows: only the bulk is held."""
    e = rel_err(got, want)
    if dtype == "float32":
        assert float(e.max()) < 1e-4, f"{what}: worst row {int(e.argmax())} differs by {float(e.max()):.2e}"
        return
    over = int((e > 0.12).sum())
    allowed = max(3, int((0.2 if free_routing else 0.1) * e.numel()))
    assert float(e.median()) < 5e-2 and over <= allowed and (free_routing or float(e.max()) < 0.6), \
        f"{what}: median {float(e.median()):.3f}, worst {float(e.max()):.3f} (row {int(e.argmax())}), over 0.12: {over} of {e.numel()}"


@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mechanism_alone_as_a_one_layer_model(folders, name):
    d, (cfg, W) = folders(name, config_of(ALONE[name], width=48, vocab=90, taps=3), seed=3)
    toks = helpers.random_tokens(90, 83, seed=1)
    want, picks = oracle(cfg, W, toks)
    for dtype in ("float32", "bfloat16"):
        pins = picks if dtype == "bfloat16" else None
        r = runner_for(d, dtype, max_tokens=96)
        s = r.admit()
        check(feed(r, s, toks, [83], pins), want, dtype, f"{name} whole {dtype}")
        r.release(s)
        s = r.admit()                                  # the same slot and pages again
        check(feed(r, s, toks, [5, 2, 17, 2, 3, 30] + [1] * 24, pins), want, dtype, f"{name} portions {dtype}")


def test_the_mechanisms_bite(folders):
    """The tests' weights make every mechanism count: an oracle without one of them differs."""
    d, (cfg, W) = folders("mixed", CONFIGS["mixed"], seed=7)
    toks = helpers.random_tokens(cfg["vocab"], 90, seed=2)
    want = torch.from_numpy(P.forward(cfg, W, toks))

    def without(change, weights=None):
        c = copy.deepcopy(cfg)
        w = dict(W)
        change(c, w)
        return float(rel_err(torch.from_numpy(P.forward(c, w, toks)), want)[30:].max())

    left = lambda c, i: c["layers"][i]["mixer"]["left"]
    assert without(lambda c, w: left(c, 1)["mask"].update(size=22)) > 1e-3
    assert without(lambda c, w: left(c, 2)["mask"].update(size=36)) > 1e-3
    assert without(lambda c, w: left(c, 1).update(_no_sink=True)) > 1e-3
    assert without(lambda c, w: left(c, 1)["rot"].pop("scaling")) > 1e-3
    assert without(lambda c, w: left(c, 2).pop("rot")) > 1e-3
    assert without(lambda c, w: w.update({"l1.mix.left.talk": np.eye(6)})) > 1e-3
    assert without(lambda c, w: w.update({"l1.mix.left.temp": np.ones(6)})) > 1e-3
    assert without(lambda c, w: w.update({"l1.mix.left.k.conv": np.eye(3)[2][None, :].repeat(24, 0)})) > 1e-3
    assert without(lambda c, w: w.update({"l1.canon1": 0.0 * w["l1.canon1"]})) > 1e-3
    assert without(lambda c, w: c["layers"][0]["mixer"].update(gate_cap=50.0)) > 1e-3
    assert without(lambda c, w: c["layers"][1]["mixer"]["right"].update(tau=8.0)) > 1e-3
    assert without(lambda c, w: c.update(logit_softcap=1.0)) > 1e-3
    assert without(lambda c, w: c["layers"][3]["mlp"]["router"].update(top=2)) > 1e-3


@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_decoded_and_in_portions(folders, name, dtype):
    d, (cfg, W) = folders(name, CONFIGS[name], seed=7)
    toks = helpers.random_tokens(cfg["vocab"], 150, seed=2)
    want, picks = oracle(cfg, W, toks)
    r = runner_for(d, dtype, max_tokens=160)
    results = []
    for cuts in ([150], [86] + [1] * 64, [2] * 75, [7, 2, 16, 3, 2, 9, 5, 2, 15, 14, 33, 2, 40]):
        s = r.admit()
        results.append(feed(r, s, toks, cuts))                       # routing free: steps replay from graphs in bfloat16
        check(results[-1], want, dtype, f"{name} {dtype} cuts {cuts[:4]}", free_routing=True)
        r.release(s)
        if dtype == "bfloat16":
            s = r.admit()
            check(feed(r, s, toks, cuts, picks), want, dtype, f"{name} {dtype} cuts {cuts[:4]}, routing pinned")
            r.release(s)
    if dtype == "float32":
        for other in results[1:]:                                    # the cut changes nothing but the rounding of sums
            assert float(rel_err(other, results[0]).max()) < 2e-5


def test_unequal_requests_in_one_batch_slots_and_pages_used_again(folders):
    """Up to four live requests, portions of some beside single tokens of others, requests that sit a step
    out, in a pool so small that pages and slots come back into use: every position equals the plain
    implementation's."""
    from cajeta_llm_b200.engine.step import StepEntry
    d, (cfg, W) = folders("mixed", CONFIGS["mixed"], seed=7)
    rng = random.Random(4)
    lens = [23, 48, 17, 64, 35, 29, 52, 2, 41, 1]
    toks = {i: helpers.random_tokens(cfg["vocab"], n, seed=50 + i) for i, n in enumerate(lens)}
    both = {i: oracle(cfg, W, t) for i, t in toks.items()}
    for dtype in ("float32", "bfloat16"):
        r = runner_for(d, dtype, max_seqs=4, max_tokens=64, num_pages=14)
        waiting, live, got = list(toks), {}, {i: [] for i in toks}
        while waiting or live:
            while waiting and len(live) < 4:
                i = waiting[0]
                if sum(-(-(len(toks[j]) + 15) // 16) for j in live) + -(-(len(toks[i]) + 15) // 16) > 14:
                    break
                waiting.pop(0)
                live[i] = [r.admit(), 0, max(1, len(toks[i]) - rng.randint(3, 12))]
            entries, who, spans = [], [], []
            for i, st in list(live.items()):
                if len(live) > 1 and rng.random() < 0.2:
                    continue
                n = 1 if st[1] >= st[2] else min(rng.randint(2, 11), st[2] - st[1])
                entries.append(StepEntry(st[0], toks[i][st[1]:st[1] + n], list(range(n))))
                who.append((i, n))
                spans.append((both[i][1], st[1], n))
                st[1] += n
            if not entries:
                continue
            out = r.step(entries, routing_pin=pin_rows(spans) if dtype == "bfloat16" else None).cpu()
            at = 0
            for i, n in who:
                got[i].append(out[at:at + n])
                at += n
                if live[i][1] == len(toks[i]):
                    r.release(live.pop(i)[0])
        for i in toks:
            check(torch.cat(got[i]), both[i][0], dtype, f"request {i} in the mixed batch ({dtype})")
        r.cache.books.check()


EDGE_LAYERS = {
    # windows that are no multiple of a page, one shorter than a page, one longer than two chunks of keys
    "w37": {"conv": 3, "dim": 16, "heads": 4, "kv_heads": 2, "vdim": 12, "scale": 0.6, "mask": {"size": 37}, "rot": {"base": 100.0, "dims": 8}},
    "w5": {"conv": 2, "dim": 8, "heads": 2, "kv_heads": 1, "vdim": 8, "scale": 0.9, "mask": {"size": 5}},
    "w70": {"conv": 3, "dim": 64, "heads": 2, "kv_heads": 2, "vdim": 32, "scale": 0.3, "mask": {"size": 70},
            "rot": {"base": 5000.0, "dims": 64, "scaling": {"factor": 2.0, "low": 1.0, "high": 4.0, "original": 32}}},
}


@pytest.mark.parametrize("name", sorted(EDGE_LAYERS))
def test_keys_at_the_window_edge_and_at_page_borders(folders, name):
    """Attention made sharp (large numbers per head on the scores): a row's output is then close to the value of
    its best key, which for many rows is the oldest key of the window or the one just outside it.  Every row
    of prompts of several lengths - so that the edge falls on either side of page borders - equals the plain
    implementation's, whole, cut anywhere and decoded one by one, and an oracle whose window is one token off
    is told apart by a wide margin."""
    left = EDGE_LAYERS[name]
    w = left["mask"]["size"]
    layer = {"type": "parallel", "mixer": {"left": left, "right": {"heads": 1, "dim": 4, "vdim": 4, "tau": 2.0, "decay_rank": 2}}, "mlp": None}
    d, (cfg, W) = folders("edge_" + name, config_of([layer], width=32, vocab=60, taps=2, softcap=30.0), seed=9, touch=sharp)
    runners = {dtype: runner_for(d, dtype, max_tokens=256) for dtype in ("float32", "bfloat16")}
    shown = 0
    for n in (w + 3, w + 16, 2 * w + 21, 3 * w + 30):
        toks = helpers.random_tokens(60, n, seed=n)
        want = torch.from_numpy(P.forward(cfg, W, toks))
        for delta in (-1, 1):
            off = copy.deepcopy(cfg)
            off["layers"][0]["mixer"]["left"]["mask"]["size"] = w + delta
            wrong = torch.from_numpy(P.forward(off, W, toks))
            shown += int((rel_err(wrong, want) > 0.1).sum())
        for dtype, r in runners.items():
            for cuts in ([n], [n - 5] + [1] * 5, [w - 1, 2, 2], [3, w - 2, 2], [2, 2, w]):
                cuts = [c for c in cuts if c > 0]
                rest = n - sum(cuts)
                cuts = cuts + ([rest - min(rest, 6)] if rest > 6 else []) + [1] * min(rest, 6) if rest >= 0 else [n]
                s = r.admit()
                got = feed(r, s, toks, cuts)
                r.release(s)
                e = rel_err(got, want)
                if dtype == "float32":
                    assert float(e.max()) < 1e-4, f"{dtype} {n} tokens, cuts {cuts[:4]}: row {int(e.argmax())} differs by {float(e.max()):.2e}"
                else:
                    assert float(e.median()) < 5e-2 and float(e.max()) < 0.6, f"{dtype} {n} tokens, cuts {cuts[:4]}: row {int(e.argmax())} differs by {float(e.max()):.2e}"
    assert shown >= 5, "the test's weights do not show the window's edge"


def test_far_keys_in_a_long_window(folders):
    """A window longer than the prompts: every earlier key is seen, over many pages and chunks; sharp scores."""
    left = {"conv": 3, "dim": 32, "heads": 4, "kv_heads": 1, "vdim": 16, "scale": 0.4, "mask": {"size": 1000}, "rot": {"base": 10000.0, "dims": 16}}
    layer = {"type": "parallel", "mixer": {"left": left, "right": {"heads": 2, "dim": 8, "vdim": 8, "tau": 30.0, "decay_rank": 4}}, "mlp": None}
    d, (cfg, W) = folders("far", config_of([layer, MEMORY], width=32, vocab=60), seed=9, touch=sharp)
    toks = helpers.random_tokens(60, 307, seed=5)
    want = torch.from_numpy(P.forward(cfg, W, toks))
    near = copy.deepcopy(cfg)
    near["layers"][0]["mixer"]["left"]["mask"]["size"] = 150
    assert float(rel_err(torch.from_numpy(P.forward(near, W, toks))[200:], want[200:]).max()) > 0.1
    for dtype in ("float32", "bfloat16"):
        r = runner_for(d, dtype, max_tokens=320)
        for cuts in ([307], [300, 4] + [1] * 3, [17] * 18 + [1]):
            s = r.admit()
            check(feed(r, s, toks, cuts), want, dtype, f"far keys {dtype} cuts {cuts[:3]}")
            r.release(s)


def test_first_tokens_and_long_decoding(folders):
    d, (cfg, W) = folders("other", CONFIGS["other"], seed=7)
    for dtype in ("float32", "bfloat16"):
        r = runner_for(d, dtype, max_tokens=192)
        for n in (1, 2, 3, 4, 6):
            toks = helpers.random_tokens(cfg["vocab"], n, seed=20 + n)
            s = r.admit()
            check(feed(r, s, toks, [1] * n), oracle(cfg, W, toks)[0], dtype, f"{n} first tokens one by one ({dtype})", free_routing=True)
            r.release(s)
            s = r.admit()
            check(feed(r, s, toks, [n]), oracle(cfg, W, toks)[0], dtype, f"{n} first tokens at once ({dtype})", free_routing=True)
            r.release(s)
        toks = helpers.random_tokens(cfg["vocab"], 183, seed=33)
        s = r.admit()
        check(feed(r, s, toks, [3] + [1] * 180), oracle(cfg, W, toks)[0], dtype, f"long decoding ({dtype})", free_routing=True)
        r.release(s)


def test_captured_steps_equal_uncaptured_ones(folders):
    from cajeta_llm_b200.engine.step import StepEntry
    d, (cfg, W) = folders("wide", CONFIGS["wide"], seed=7)
    toks = [helpers.random_tokens(cfg["vocab"], 100, seed=70 + i) for i in range(3)]
    outs = []
    for graphs in (True, False):
        r = runner_for(d, "bfloat16", max_tokens=128, cuda_graphs=graphs)
        slots = [r.admit() for _ in toks]
        got = []
        for lo, hi in ((0, 12), (12, 24), (24, 36), (36, 48)):       # the same shape again and again: captured, then replayed
            got.append(r.step([StepEntry(s, t[lo:hi], [hi - lo - 1]) for s, t in zip(slots, toks)]).cpu())
        for i in range(48, 100):
            got.append(r.step([StepEntry(s, [t[i]], [0]) for s, t in zip(slots, toks)]).cpu())
        outs.append(torch.cat(got))
        if graphs:
            assert r.graph_replays > 0
    assert torch.equal(outs[0], outs[1])


def test_two_streams_equal_one(folders):
    """The halves of a parallel layer on two streams give the bits they give one after the other, in steps launched
    kernel by kernel and in captured ones."""
    from cajeta_llm_b200.engine.step import StepEntry
    d, (cfg, W) = folders("wide", CONFIGS["wide"], seed=7)
    toks = [helpers.random_tokens(cfg["vocab"], 80, seed=90 + i) for i in range(2)]
    outs = []
    for overlap in (True, False):
        r = runner_for(d, "bfloat16", max_tokens=128, cuda_graphs=True)
        pairs = [b.mixer for b in r.model.blocks if hasattr(b.mixer, "overlap")]
        assert pairs and all(m.overlap for m in pairs)
        for m in pairs:
            m.overlap = overlap
        slots = [r.admit() for _ in toks]
        got = [r.step([StepEntry(s, t[:37], [36]) for s, t in zip(slots, toks)]).cpu()]
        for i in range(37, 80):
            got.append(r.step([StepEntry(s, [t[i]], [0]) for s, t in zip(slots, toks)]).cpu())
        outs.append(torch.cat(got))
        assert r.graph_replays > 0
    assert torch.equal(outs[0], outs[1])


def test_a_folder_whose_configuration_leaves_the_decay_rank_to_the_tensor(folders, tmp_path):
    """The decay's inner size is the shape of a tensor: a folder's config.json need not give it."""
    import shutil
    d, (cfg, W) = folders("other", CONFIGS["other"], seed=7)
    dst = str(tmp_path / "model")
    shutil.copytree(d, dst)
    with open(os.path.join(dst, "config.json")) as f:
        raw = json.load(f)
    for layer in raw["layers"]:
        if layer["type"] == "parallel":
            layer["mixer"]["right"].pop("decay_rank")
    with open(os.path.join(dst, "config.json"), "w") as f:
        json.dump(raw, f)
    toks = helpers.random_tokens(cfg["vocab"], 40, seed=3)
    r = runner_for(dst, "float32", max_tokens=64)
    s = r.admit()
    check(feed(r, s, toks, [40]), oracle(cfg, W, toks)[0], "float32", "decay rank from the tensor's shape")


def test_greedy_generation_through_the_entry_point_and_its_scheduler(folders):
    from cajeta_llm_b200.engine.llm_engine import LlmEngine
    from cajeta_llm_b200.engine.options import EngineOptions
    from cajeta_llm_b200.sampling.params import SamplingParams
    d, (cfg, W) = folders("mixed", CONFIGS["mixed"], seed=7)
    prompts = [helpers.random_tokens(cfg["vocab"], n, seed=90 + n) for n in (5, 9, 17, 30, 3, 12)]
    want = [P.greedy(cfg, W, p, 6) for p in prompts]
    # more requests than slots, portions of at most 8 tokens under a budget of 24 a step
    eng = LlmEngine.load(EngineOptions(model=d, dtype="float32", ctx=64, max_seqs=3, chunk=8, max_batch_tokens=24))
    got = eng.generate(prompts, SamplingParams(max_new_tokens=6, stop_token_ids=()))
    assert got == want
    eng.close()
    eng = LlmEngine.load(EngineOptions(model=d, dtype="bfloat16", ctx=64, max_seqs=4))
    got = eng.generate(prompts, SamplingParams(max_new_tokens=6, stop_token_ids=()))
    same = sum(g == w for g, w in zip(got, want))
    assert same >= len(prompts) - 2, f"bfloat16 greedy tokens differ for {len(prompts) - same} prompts"
    eng.close()


def test_replay_tool_on_a_model_folder(folders, tmp_path):
    d, (cfg, W) = folders("other", CONFIGS["other"], seed=7)
    a, b = helpers.random_tokens(cfg["vocab"], 20, seed=1), helpers.random_tokens(cfg["vocab"], 9, seed=2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:11], "want": [10]}, {"id": "b", "tokens": b[:8], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": b[8:], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[11:], "want": [0, 8]}], "end": ["a"]}]
    import subprocess
    import sys
    cmd = [sys.executable, os.path.join(helpers.ROOT, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", str(tmp_path),
           "--max-tokens", "128"]
    proc = subprocess.run(cmd, input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    wa, wb = oracle(cfg, W, a)[0], oracle(cfg, W, b)[0]
    got = {n: torch.from_numpy(np.fromfile(os.path.join(str(tmp_path), f"{n}.f32"), dtype="<f4").reshape(-1, cfg["vocab"])) for n in range(3)}
    check(got[0], wa[10:11], "float32", "step 0")
    check(got[1], wb[8:9], "float32", "step 1")
    check(got[2], wa[[11, 19]], "float32", "step 2")


def random_config(seed):
    """A configuration drawn at random: layer order, every size and constant."""
    rng = random.Random(seed)
    width = rng.choice([40, 72, 136, 256])
    big = width >= 128

    def pick(lo, hi):
        return rng.randint(lo, hi)

    layers = []
    for _ in range(rng.randint(1, 5)):
        if rng.random() < 0.4:
            m = {"heads": pick(1, 5), "dim": rng.choice([64, 48]) if big and rng.random() < 0.4 else pick(2, 40),
                 "vdim": rng.choice([64, 128]) if big and rng.random() < 0.4 else pick(2, 40), "gate_cap": rng.choice([1.5, 6.0, 15.0])}
            kind = "mlstm"
        else:
            kv = pick(1, 3)
            dim = rng.choice([64, 96, 128]) if big and rng.random() < 0.5 else 2 * pick(2, 24)
            left = {"conv": pick(1, 4), "heads": kv * pick(1, 3), "kv_heads": kv, "dim": dim,
                    "vdim": dim if rng.random() < 0.5 else pick(3, 40), "scale": rng.choice([0.1, 0.3, 1.0]),
                    "mask": {"size": rng.choice([1, 2, 7, 16, 17, 33, 64, 100, 400])}}
            if rng.random() < 0.8:
                left["rot"] = {"base": rng.choice([100.0, 10000.0, 500000.0]), "dims": 2 * pick(1, dim // 2)}
                if rng.random() < 0.6:
                    left["rot"]["scaling"] = {"factor": rng.choice([2.0, 8.0]), "original": rng.choice([8, 32, 4096]),
                                              "low": rng.choice([0.5, 1.0]), "high": rng.choice([2.0, 4.0])}
            right = {"heads": pick(1, 4), "dim": pick(2, 40), "vdim": pick(2, 40), "tau": rng.choice([1.0, 4.0, 16.0, 64.0]),
                     "decay_rank": pick(1, 20)}
            m = {"left": left, "right": right}
            kind = "parallel"
        mlp = None
        if rng.random() < 0.7:
            experts = pick(1, 12)
            mlp = moe(experts, pick(1, experts), rng.choice([pick(8, 60), 128, 136]) if big else pick(8, 60))
        layers.append({"type": kind, "mixer": m, "mlp": mlp})
    return config_of(layers, width=width, vocab=rng.choice([70, 131, 300]), eps=rng.choice([1e-5, 1e-6]), taps=pick(1, 5),
                     softcap=rng.choice([5.0, 30.0]))


@pytest.mark.parametrize("seed", range(10))
def test_configurations_drawn_at_random(folders, seed):
    raw = random_config(3000 + seed)
    d, (cfg, W) = folders(f"random{seed}", raw, seed=100 + seed)
    toks = helpers.random_tokens(cfg["vocab"], 120, seed=seed)
    want, picks = oracle(cfg, W, toks)
    for dtype in ("float32", "bfloat16"):
        r = runner_for(d, dtype, max_tokens=128)
        for cuts in ([120], [17, 2, 9, 60] + [1] * 32):
            s = r.admit()
            check(feed(r, s, toks, cuts, picks if dtype == "bfloat16" else None), want, dtype,
                  f"{json.dumps(raw)} {dtype} cuts {cuts[:3]}")
            r.release(s)


def _mixed_attention_formula(q, keys, values, positions, row_req, window, scale, temp, talk, sink):
    """The formula, row by row in float64: raw scores of all heads, times scale and temp, mixed by talk, keys of the
    window, a softmax whose divisor also holds exp(sink).  keys / values: per request [tokens, kv heads, size]."""
    T, H, _ = q.shape
    out = torch.zeros((T, H, values[0].shape[-1]), dtype=torch.float64)
    for t in range(T):
        p, kk, vv = int(positions[t]), keys[int(row_req[t])].double(), values[int(row_req[t])].double()
        lo = max(0, p + 1 - window) if window > 0 else 0
        G = kk.shape[1]
        raw = torch.stack([(kk[lo:p + 1, h // (H // G)] @ q[t, h].double()) * scale * float(temp[h]) for h in range(H)])    # [H, keys]
        s = talk.double() @ raw
        for h in range(H):
            m = max(float(s[h].max()), float(sink[h]))
            e = torch.exp(s[h] - m)
            out[t, h] = (e[:, None] * vv[lo:p + 1, h // (H // G)]).sum(0) / (e.sum() + math.exp(float(sink[h]) - m))
    return out


@pytest.mark.parametrize("H,G,hd,vd,window,requests", [
    (4, 2, 16, 8, 7, [(0, 40)]),
    (8, 2, 64, 64, 33, [(0, 100), (50, 1), (7, 3), (0, 17)]),
    (32, 8, 128, 128, 100, [(0, 150), (255, 1), (3, 2)]),
    (6, 3, 24, 40, 20, [(0, 70), (19, 1), (20, 1), (21, 1)]),
    (64, 8, 32, 16, 0, [(0, 64), (49, 1)]),
    (2, 1, 8, 8, 3, [(0, 9), (2, 1), (3, 1)]),
    (10, 5, 16, 24, 9, [(0, 21), (8, 1), (9, 1), (4, 30)]),      # a block's heads end in the middle of a key head's group
    (4, 4, 40, 8, 1, [(0, 18), (5, 1)]),                        # a window of the row itself
])
def test_tiled_mixed_heads_attention_against_the_formula(H, G, hd, vd, window, requests):
    """The cluster form alone, on pages in a shuffled order: requests of (cached tokens, new rows), single rows just
    inside and just outside the window, tiles that end in the middle of a chunk of keys.  One key of every window's
    far end is made loud, so that a window one key short or long shows."""
    from cajeta_llm_b200.csrc import kernels as K
    assert K.mixed_heads_tile_shape(H, G, hd, vd)
    g = torch.Generator().manual_seed(H * 1000 + hd)
    page, dev = 16, "cuda"
    totals = [p + r for p, r in requests]
    pages_per = [(t + page - 1) // page for t in totals]
    n_pages = sum(pages_per) + 3
    order = torch.randperm(n_pages, generator=g)[:sum(pages_per)].int()
    table = torch.full((len(requests), max(pages_per)), -1, dtype=torch.int32)
    keys = [torch.randn((t, G, hd), generator=g).bfloat16() for t in totals]
    values = [torch.randn((t, G, vd), generator=g).bfloat16() for t in totals]
    for kk in keys:
        kk[::5] *= 3.0
    kp, vp = torch.zeros((n_pages, G, page, hd), dtype=torch.bfloat16), torch.zeros((n_pages, G, page, vd), dtype=torch.bfloat16)
    at = 0
    for r, n in enumerate(pages_per):
        table[r, :n] = order[at:at + n]
        for t in range(totals[r]):
            kp[int(table[r, t // page]), :, t % page] = keys[r][t]
            vp[int(table[r, t // page]), :, t % page] = values[r][t]
        at += n
    q = torch.randn((sum(r for _, r in requests), H, hd), generator=g).bfloat16()
    positions = torch.cat([torch.arange(p, p + r) for p, r in requests]).int()
    row_req = torch.cat([torch.full((r,), i) for i, (_, r) in enumerate(requests)]).int()
    starts = [0]
    for _, r in requests:
        starts.append(starts[-1] + r)
    temp = torch.rand(H, generator=g) + 0.5
    talk = torch.eye(H) + 0.3 * torch.randn((H, H), generator=g)
    sink = torch.randn(H, generator=g)
    scale = hd ** -0.5
    want = _mixed_attention_formula(q, keys, values, positions, row_req, window, scale, temp, talk, sink)
    # the cluster's size and the number of clusters a tile's keys are dealt to, chosen by the library and given
    largest = max(c for c in (1, 2, 4, 8) if H % c == 0 and H // c <= 8)
    smallest = min(c for c in (1, 2, 4, 8) if H % c == 0 and H // c <= 8)
    for blocks, splits in ((0, None), (smallest, 1), (largest, 3), (0, 8)):
        got = torch.full((q.shape[0], H, vd), float("nan"), dtype=torch.bfloat16, device=dev)
        K.mixed_heads_attention(q.to(dev), got, kp.to(dev), vp.to(dev), positions.to(dev), row_req.to(dev), table.to(dev), page, H, G, hd,
                                vd, window, scale, temp=temp.to(dev), talk=talk.to(dev), sink=sink.to(dev),
                                req_start=torch.tensor(starts, dtype=torch.int32, device=dev), n_requests=len(requests),
                                cluster_blocks=blocks, splits=splits)
        assert "attention_mixed" in K.loaded_libraries()
        err = (got.cpu().double() - want).abs()
        assert float(err.max()) < 0.01 * max(1.0, float(want.abs().max())), \
            f"cluster of {blocks}, {splits} shares: row {int(err.amax(dim=(1, 2)).argmax())} differs by {float(err.max()):.3g}"
    if window > 0:
        # the same rows with the window one key longer and one key shorter differ by far more than that
        for other in {window + 1, max(1, window - 1)} - {window}:
            moved = _mixed_attention_formula(q, keys, values, positions, row_req, other, scale, temp, talk, sink)
            assert float((moved - want).abs().max()) > 0.05
