"""Throughput of a Balalorn, a Saropel, a Govuvik or a Dimuvik model at layer sizes that resemble real models', beside the
engine's Qwen2-MoE model at equal width, depth, experts and feed-forward sizes (Govuvik: beside Balalorn, the
engine's other model with recurrent state, at equal width, depth and experts; Dimuvik: beside Balalorn, the engine's
other model with attention over a latent and a borrowed cache, at equal width, depth, heads, latent and experts).

``python bench.py --design balalorn|saropel|govuvik|dimuvik [--sizes small,medium,large]`` prints one JSON line per
(size, model): prefill tokens a second (one prompt of 2,048 tokens), decode tokens a second
(8 requests of 512 tokens each, steps replayed from CUDA graphs), and where the time of both
steps goes by class of work (launches serialised, an event behind each), with the bytes or
flops the attention-like classes must move and their fraction of the measured peaks.
Weights are random; a timed step reads far more than L2 holds.
"""
from __future__ import annotations

import json
import time

SIZES = {
    # width, layers, heads (of 128), kv_rank, experts, top, expert ff, dense ff, state
    "small": dict(width=1024, layers=4, heads=8, rank=256, experts=16, top=2, eff=512, ff=2816, state=64),
    "medium": dict(width=2048, layers=4, heads=16, rank=512, experts=60, top=4, eff=1408, ff=5632, state=128),
    "large": dict(width=4096, layers=4, heads=32, rank=512, experts=32, top=4, eff=2048, ff=11008, state=128),
}
VOCAB, PROMPT, BATCH, PREFILL = 32000, 512, 8, 2048


def balalorn_config(s):
    h, H = s["width"], s["heads"]
    latent = {"heads": H, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": s["rank"], "scale": (128 + 64) ** -0.5,
              "rot": {"base": 10000.0, "dims": 64}}
    moe = {"kind": "moe", "expert": {"ff": s["eff"]}, "router": {"experts": s["experts"], "top": s["top"]}}
    dense = {"kind": "dense", "ff": s["ff"]}
    kinds = [
        lambda i: {"type": "latent_attention", "mixer": dict(latent), "mlp": moe},
        lambda i: {"type": "mamba2", "mixer": {"heads": 2 * h // 64, "vdim": 64, "state": s["state"], "groups": 8, "norm_groups": 8, "conv": 4},
                   "mlp": dense},
        lambda i: {"type": "delta", "mixer": {"heads": H, "kv_heads": H // 2, "dim": 128, "vdim": 128, "conv": 4}, "mlp": moe},
        lambda i: {"type": "latent_attention", "mixer": dict(latent, kv_from=i - 3), "mlp": dense},
    ]
    return {"architecture": "Balalorn", "width": h, "vocab": VOCAB, "norm": {"eps": 1e-6},
            "layers": [kinds[i % 4](i) for i in range(s["layers"])]}


SAROPEL_WINDOWS = (1024, 4096)      # of the capped layers and of the rotated, gated ones


def saropel_config(s):
    """Three layers of weights, four layer runs (the middle layer runs twice, as a looped stretch): capped
    windowed attention + dense, rotated gated attention (values = keys) + routed with a shared expert, capped + dense."""
    h, H = s["width"], s["heads"]
    capped = {"heads": H, "kv_heads": H, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "softcap": 50.0, "mask": {"size": SAROPEL_WINDOWS[0]}}
    rotated = {"heads": H, "kv_heads": H, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "mask": {"size": SAROPEL_WINDOWS[1]},
               "rot": {"base": 1000000.0, "dims": 64, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    moe = {"kind": "moe", "expert": {"ff": s["eff"], "limit": 7.0},
           "router": {"experts": s["experts"], "top": s["top"], "groups": {"count": 4, "keep": 2}},
           "shared": {"ff": s["eff"], "limit": 7.0}}
    dense = {"kind": "dense", "ff": s["ff"]}
    return {"architecture": "Saropel", "width": h, "vocab": VOCAB, "norm": {"eps": 1e-6},
            "embedding": {"bigram": {"buckets": 100003, "mul_prev": 37, "mul_cur": 11}}, "token_side": {"dim": 256},
            "loop": {"start": 1, "stop": 2, "times": 2},
            "layers": [{"type": "attention", "mixer": capped, "mlp": dense}, {"type": "attention_2", "mixer": rotated, "mlp": moe},
                       {"type": "attention", "mixer": capped, "mlp": dense}]}


GOVUVIK_WINDOW = 1024


def govuvik_config(s):
    """Four layers: windowed attention with mixed heads beside gated linear attention, matrix memory, and the two once more;
    every layer with a routed feed-forward of ungated experts."""
    h, H = s["width"], s["heads"]
    memory = {"heads": H // 2, "dim": 128, "vdim": 256, "gate_cap": 10.0}
    left = {"conv": 4, "dim": 128, "heads": H, "kv_heads": H // 4, "vdim": 128, "scale": 128 ** -0.5, "mask": {"size": GOVUVIK_WINDOW},
            "rot": {"base": 500000.0, "dims": 64, "scaling": {"factor": 4.0, "low": 1.0, "high": 8.0, "original": 8192}}}
    right = {"heads": H // 4, "dim": 128, "vdim": 256, "tau": 8.0, "decay_rank": 16}
    moe = {"kind": "moe", "expert": {"ff": s["eff"]}, "router": {"experts": s["experts"], "top": s["top"]}}
    kinds = [lambda: {"type": "parallel", "mixer": {"left": dict(left), "right": dict(right)}, "mlp": moe},
             lambda: {"type": "mlstm", "mixer": dict(memory), "mlp": moe},
             lambda: {"type": "parallel", "mixer": {"left": dict(left), "right": dict(right)}, "mlp": moe},
             lambda: {"type": "mlstm", "mixer": dict(memory), "mlp": moe}]
    return {"architecture": "Govuvik", "width": h, "vocab": VOCAB, "norm": {"eps": 1e-6}, "canon": {"taps": 3}, "logit_softcap": 50.0,
            "layers": [kinds[i % 4]() for i in range(s["layers"])]}


def dimuvik_config(s):
    """Four layers: latent attention (queries through a latent of three times the keys' rank, a sink) + routed with a shared
    expert, differential attention (H heads of two maps of 64 over H/2 key heads, values of 128, 4 taps, a query
    temperature) + dense, latent attention + routed, differential attention on the second layer's keys and values + dense."""
    h, H = s["width"], s["heads"]
    latent = {"heads": H, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": s["rank"], "q_rank": 3 * s["rank"], "scale": (128 + 64) ** -0.5,
              "rot": {"base": 10000.0, "dims": 64}}
    diff = {"heads": H, "kv_heads": H // 2, "dim": 64, "vdim": 128, "conv": 4, "diff": 0.5, "scale": 64 ** -0.5,
            "q_temp": {"coef": 0.1, "every": 1024}}
    moe = {"kind": "moe", "expert": {"ff": s["eff"]}, "router": {"experts": s["experts"], "top": s["top"], "scale": 2.0}, "shared": {"ff": s["eff"]}}
    dense = {"kind": "dense", "ff": s["ff"]}
    kinds = [lambda i: {"type": "latent_attention", "mixer": dict(latent), "mlp": moe},
             lambda i: {"type": "attention", "mixer": dict(diff), "mlp": dense},
             lambda i: {"type": "latent_attention", "mixer": dict(latent), "mlp": moe},
             lambda i: {"type": "attention", "mixer": dict(diff, kv_from=i - 2), "mlp": dense}]
    return {"architecture": "Dimuvik", "width": h, "vocab": VOCAB, "norm": {"eps": 1e-6}, "embedding": {"scale": 2.0},
            "layers": [kinds[i % 4](i) for i in range(s["layers"])]}


def qwen_config(s, shared=0):
    return {"architectures": ["Qwen2MoeForCausalLM"], "hidden_size": s["width"], "intermediate_size": s["ff"],
            "num_hidden_layers": s["layers"], "num_attention_heads": s["heads"], "num_key_value_heads": s["heads"], "head_dim": 128,
            "vocab_size": VOCAB, "max_position_embeddings": 8192, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
            "num_experts": s["experts"], "num_experts_per_tok": s["top"], "moe_intermediate_size": s["eff"],
            "shared_expert_intermediate_size": shared, "norm_topk_prob": False, "decoder_sparse_step": 2, "mlp_only_layers": [],
            "tie_word_embeddings": False, "use_sliding_window": False}


def needs(design, s, rows, ctx, prefill):
    """(bytes, flops) the attention-like classes of one step must move, over all layers."""
    L, H, out = s["layers"], s["heads"], {}
    if design == "qwen2_moe":
        kv = ctx * 2 * H * 128 * 2
        out["attention"] = (rows * kv * L if not prefill else 0, 4 * H * 128 * rows * (rows + 1) // 2 * L if prefill else 0)
        return out
    if design == "saropel":
        by = fl = 0
        for w in (SAROPEL_WINDOWS[0], SAROPEL_WINDOWS[1], SAROPEL_WINDOWS[1], SAROPEL_WINDOWS[0]):      # the four layer runs
            if prefill:
                fl += 4 * H * 128 * sum(min(i + 1, w) for i in range(rows))
            else:
                by += rows * min(ctx, w) * 2 * H * 128 * 2
        out["attention"] = (by, fl)
        return out
    if design == "govuvik":
        n_par, n_mem = (L + 3) // 4 + (L + 1) // 4, (L + 2) // 4 + L // 4
        w = GOVUVIK_WINDOW
        out["attention"] = (rows * min(ctx, w) * 2 * (H // 4) * 128 * 2 * n_par if not prefill else 0,
                            4 * H * 128 * sum(min(i + 1, w) for i in range(rows)) * n_par if prefill else 0)
        reqs = 1 if prefill else rows
        mem, gla = (H // 2) * (128 * 256 + 128 + 1) * 4, (H // 4) * 128 * 256 * 4
        # a state is read and written once a request; every row brings q, k, v (and the decays) in float32
        out["scan"] = (reqs * 2 * (n_mem * mem + n_par * gla)
                       + rows * 4 * (n_mem * (H // 2) * (2 * 128 + 256 + 2) + n_par * (H // 4) * (3 * 128 + 256)),
                       rows * (n_mem * (H // 2) * 128 * 256 * 6 + n_par * (H // 4) * 128 * 256 * 5))
        return out
    if design == "dimuvik":
        n_lat, n_diff = (L + 3) // 4 + (L + 1) // 4, (L + 2) // 4 + L // 4
        width = s["rank"] + 64
        # the latent layers as for Balalorn; a differential layer reads a key head's [k1 | k2] and its value once a row
        # (H/2 key heads of 128 + 128) and multiplies two maps of 64 and two value products of 128
        out["attention"] = (rows * ctx * width * 2 * n_lat if not prefill else 0,
                            2 * H * (128 + 64 + 128) * n_lat * rows * (rows + 1) // 2 if prefill else 0)
        out["differential attention"] = (rows * ctx * (H // 2) * (128 + 128) * 2 * n_diff if not prefill else 0,
                                         2 * H * (2 * 64 + 2 * 128) * n_diff * rows * (rows + 1) // 2 if prefill else 0)
        return out
    n_lat, n_ssd, n_delta = (L + 3) // 4 + L // 4, (L + 2) // 4, (L + 1) // 4
    width = s["rank"] + 64
    # decode: the absorbed form reads each cache entry once; prompt portions: the plain form's flops
    out["attention"] = (rows * ctx * width * 2 * n_lat if not prefill else 0,
                        2 * H * (128 + 64 + 128) * rows * (rows + 1) // 2 * n_lat if prefill else 0)
    reqs = 1 if prefill else rows
    ssd_heads = 2 * s["width"] // 64
    state = n_ssd * ssd_heads * s["state"] * 64 * 4 + n_delta * H * 128 * 128 * 4
    out["scan"] = (reqs * state * 2 + rows * 4 * (n_ssd * (2 * ssd_heads * 64 + 16 * s["state"]) + n_delta * 3 * H * 128),
                   rows * (n_ssd * ssd_heads * s["state"] * 64 * 4 + n_delta * H * 128 * 128 * 8))
    return out


def run(args, peaks) -> int:
    import numpy as np
    import torch

    import cajeta_llm_b200  # noqa: F401
    from cajeta_llm_b200.csrc import kernels as K
    from cajeta_llm_b200.engine.llm_engine import LlmEngine
    from cajeta_llm_b200.engine.options import EngineOptions
    from cajeta_llm_b200.engine.step import StepEntry

    pk = peaks()
    rng = np.random.default_rng(3)
    for size in [x for x in args.sizes.split(",") if x]:
        s = SIZES[size]
        if args.design == "saropel":
            pair = (("saropel", saropel_config(s)), ("qwen2_moe", qwen_config(s, shared=s["eff"])))
        elif args.design == "govuvik":
            pair = (("govuvik", govuvik_config(s)), ("balalorn", balalorn_config(s)))
        elif args.design == "dimuvik":
            pair = (("dimuvik", dimuvik_config(s)), ("balalorn", balalorn_config(s)))
        else:
            pair = (("balalorn", balalorn_config(s)), ("qwen2_moe", qwen_config(s)))
        for design, cfg in pair:
            tokens = BATCH * (PROMPT + 128) + PREFILL + 64
            eng = LlmEngine.load(EngineOptions(config=cfg, random_weights=True, seed=11, dtype="bfloat16", ctx=PREFILL + 64, max_seqs=BATCH,
                                               block_tokens=16, num_blocks=-(-tokens // 16) + BATCH, max_batch_tokens=8192, warmup=False))
            r = eng.runner

            def toks(n):
                return rng.integers(0, VOCAB, size=n).tolist()

            def timed(fn, reps):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                a.record()
                for _ in range(reps):
                    fn()
                b.record()
                torch.cuda.synchronize()
                return a.elapsed_time(b) / reps

            def prefill_once():
                slot = r.admit()
                r.step([StepEntry(slot, toks(PREFILL), [PREFILL - 1])])
                r.release(slot)

            for _ in range(3):
                prefill_once()
            prefill_ms = min(timed(prefill_once, 1) for _ in range(5))

            slots = [r.admit() for _ in range(BATCH)]
            r.step([StepEntry(sl, toks(PROMPT), []) for sl in slots])

            def decode_once():
                r.step([StepEntry(sl, toks(1), [0]) for sl in slots])

            for _ in range(max(3, args.warmup)):
                decode_once()
            decode_ms = timed(decode_once, max(1, args.steps))
            for sl in slots:
                r.release(sl)

            def classes(entries_of, rows, ctx, prefill):
                # one launch after the other on one stream: a mixer that runs its halves on two streams is told not to,
                # so that the time between two events belongs to the launch between them
                for blk in r.model.blocks:
                    if hasattr(getattr(blk, "mixer", None), "overlap"):
                        blk.mixer.overlap = False
                spent = {}
                for keep in (False, False, True):
                    held, entries = entries_of()
                    torch.cuda.synchronize()
                    torch.cuda._sleep(60_000_000)
                    first = torch.cuda.Event(enable_timing=True)
                    first.record()
                    K.start_trace()
                    r.step(entries, routing_dump={})
                    trace = K.stop_trace()
                    torch.cuda.synchronize()
                    for sl in held:
                        r.release(sl)
                    if keep:
                        prev = first
                        for label, ev in trace:
                            spent[label] = spent.get(label, 0.0) + prev.elapsed_time(ev) * 1e3
                            prev = ev
                need = needs(design, s, rows, ctx, prefill)
                out = {}
                for label, us in sorted(spent.items(), key=lambda kv: -kv[1]):
                    e = {"us": round(us, 1)}
                    by, fl = need.get(label, (0, 0))
                    if by:
                        e["bytes"], e["hbm_frac"] = int(by), round(by / (us * 1e-6) / (pk["hbm_gbs"] * 1e9), 4)
                    if fl:
                        e["flops"], e["bf16_frac"] = int(fl), round(fl / (us * 1e-6) / (pk["bf16_tflops"] * 1e12), 4)
                    out[label] = e
                out["_sum_us"] = round(sum(spent.values()), 1)
                return out

            def prefill_entries():
                sl = r.admit()
                return [sl], [StepEntry(sl, toks(PREFILL), [PREFILL - 1])]

            def decode_entries():
                held = [r.admit() for _ in range(BATCH)]
                r.step([StepEntry(sl, toks(PROMPT), []) for sl in held])
                return held, [StepEntry(sl, toks(1), [0]) for sl in held]

            line = {"design": design, "size": size, "sizes": s, "weights_gb": round(eng.model().weight_bytes() / 1e9, 2),
                    "prefill_tokens": PREFILL, "prefill_ms": round(prefill_ms, 3), "prefill_tokens_per_s": round(PREFILL / prefill_ms * 1e3),
                    "decode_batch": BATCH, "decode_context": PROMPT, "decode_ms_per_step": round(decode_ms, 3),
                    "decode_tokens_per_s": round(BATCH / decode_ms * 1e3), "peaks": pk,
                    "prefill_kernels": classes(prefill_entries, PREFILL, PREFILL, True),
                    "decode_kernels": classes(decode_entries, BATCH, PROMPT + 1, False),
                    "gpu_launches": K.launches, "data": "synthetic (random weights, random token ids)", "dtype": "bf16"}
            print(json.dumps(line), flush=True)
            eng.close()
            del eng, r
            torch.cuda.empty_cache()
    return 0
