"""Govuvik restated plainly: one function per mechanism, float64, loops over tokens.

Nothing here is shared with the engine: weights arrive as a dict of numpy arrays by tensor
name, the configuration as the parsed ``config.json``.  Slow on purpose; the tests use small
sizes.  Notation: ``x`` a row of the residual stream, ``h`` what a mixer reads, ``p`` a position.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

import numpy as np

MLSTM_FLOOR = 1e-6       # added to the read-out's divisor


def rms(x: np.ndarray, eps: float) -> np.ndarray:
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def silu(z):
    return z * sigmoid(z)


def causal_conv(u: np.ndarray, w: np.ndarray) -> np.ndarray:
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, taps = u.shape[0], w.shape[1]
    y = np.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def rope_frequencies(rot: dict) -> np.ndarray:
    """dims/2 frequencies; the slow ones divided by ``factor``, a ramp between the two wavelengths."""
    dims, base = rot["dims"], float(rot["base"])
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=np.float64)
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
        out = f.copy()
        for i, fi in enumerate(f):
            wavelength = 2.0 * math.pi / fi
            if wavelength < orig / high:
                out[i] = fi
            elif wavelength > orig / low:
                out[i] = fi / factor
            else:
                s = (orig / wavelength - low) / (high - low)
                out[i] = (1.0 - s) * fi / factor + s * fi
        f = out
    return f


def rotate_half(v: np.ndarray, p: int, f: np.ndarray, dims: int) -> np.ndarray:
    """v [heads, dim] at position p; entry i turns with entry i + dims/2."""
    half = dims // 2
    a, b = v[:, :half].copy(), v[:, half:dims].copy()
    c, s = np.cos(p * f), np.sin(p * f)
    out = v.copy()
    out[:, :half] = a * c - b * s
    out[:, half:dims] = b * c + a * s
    return out


def mlstm_mixer(m: dict, W, pre: str, h: np.ndarray, eps: float) -> np.ndarray:
    """The matrix memory with exponential input gate and a running maximum that starts at 0."""
    T = h.shape[0]
    H, dim, vdim, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ W[pre + "q"].T).reshape(T, H, dim) * dim ** -0.5
    k = (h @ W[pre + "k"].T).reshape(T, H, dim)
    v = (h @ W[pre + "v"].T).reshape(T, H, vdim)
    gi = cap * np.tanh((h @ W[pre + "i"].T + W[pre + "i.b"]) / cap)
    gf = log_sigmoid(cap * np.tanh((h @ W[pre + "f"].T + W[pre + "f.b"]) / cap))
    out = np.zeros((T, H, vdim))
    for hd in range(H):
        S, n, mx = np.zeros((dim, vdim)), np.zeros(dim), 0.0
        for t in range(T):
            new = max(gf[t, hd] + mx, gi[t, hd])
            a, b = math.exp(gf[t, hd] + mx - new), math.exp(gi[t, hd] - new)
            S = a * S + b * np.outer(k[t, hd], v[t, hd])
            n = a * n + b * k[t, hd]
            mx = new
            out[t, hd] = (S.T @ q[t, hd]) / (max(abs(n @ q[t, hd]), math.exp(-mx)) + MLSTM_FLOOR)
    o = rms(out, eps).reshape(T, H * vdim) * W[pre + "norm"]
    return (o * sigmoid(h @ W[pre + "g"].T)) @ W[pre + "o"].T


def windowed_attention(m: dict, W, pre: str, h: np.ndarray, eps: float) -> np.ndarray:
    """Grouped-query attention: convolved projections, one norm over all of q and of k, a partial
    rotation, scores times a number per head and mixed among the heads, a window, a sink."""
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ W[pre + "q"].T, h @ W[pre + "k"].T, h @ W[pre + "v"].T
    if m.get("conv"):
        q, k, v = causal_conv(q, W[pre + "q.conv"]), causal_conv(k, W[pre + "k.conv"]), causal_conv(v, W[pre + "v.conv"])
    q = (rms(q, eps) * W[pre + "q.norm"]).reshape(T, H, dim)
    k = (rms(k, eps) * W[pre + "k.norm"]).reshape(T, G, dim)
    v = v.reshape(T, G, vdim)
    rot = m.get("rot")
    if rot:
        f = rope_frequencies(rot)
        q = np.stack([rotate_half(q[t], t, f, rot["dims"]) for t in range(T)])
        k = np.stack([rotate_half(k[t], t, f, rot["dims"]) for t in range(T)])
    window, scale = (m.get("mask") or {}).get("size") or T, float(m["scale"])
    temp, talk, sink = W[pre + "temp"], W[pre + "talk"], W[pre + "sink"]
    if m.get("_no_sink"):
        sink = np.full_like(sink, -np.inf)
    out = np.zeros((T, H, vdim))
    for t in range(T):
        lo = max(0, t - window + 1)
        s = np.zeros((H, t + 1 - lo))
        for hd in range(H):
            s[hd] = (k[lo:t + 1, hd // (H // G)] @ q[t, hd]) * scale * temp[hd]
        s = talk @ s
        for hd in range(H):
            top = max(s[hd].max(), sink[hd])
            e = np.exp(s[hd] - top)
            out[t, hd] = (e @ v[lo:t + 1, hd // (H // G)]) / (e.sum() + np.exp(sink[hd] - top))
    return out.reshape(T, H * vdim) @ W[pre + "o"].T


def gated_linear_attention(m: dict, W, pre: str, h: np.ndarray, eps: float) -> np.ndarray:
    """A matrix state per head whose rows decay by a factor per key channel."""
    T = h.shape[0]
    H, dim, vdim, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    q = (h @ W[pre + "q"].T).reshape(T, H, dim) * dim ** -0.5
    k = (h @ W[pre + "k"].T).reshape(T, H, dim)
    v = (h @ W[pre + "v"].T).reshape(T, H, vdim)
    z = (h @ W[pre + "a1"].T) @ W[pre + "a2"].T + W[pre + "a2.b"]
    alpha = (sigmoid(z) ** (1.0 / tau)).reshape(T, H, dim)
    out = np.zeros((T, H, vdim))
    for hd in range(H):
        S = np.zeros((dim, vdim))
        for t in range(T):
            S = alpha[t, hd][:, None] * S + np.outer(k[t, hd], v[t, hd])
            out[t, hd] = S.T @ q[t, hd]
    o = (rms(out, eps) * W[pre + "norm"]).reshape(T, H * vdim)
    return (o * silu(h @ W[pre + "g"].T)) @ W[pre + "o"].T


def parallel_mixer(m: dict, W, pre: str, h: np.ndarray, eps: float) -> np.ndarray:
    left = windowed_attention(m["left"], W, pre + "left.", h, eps)
    right = gated_linear_attention(m["right"], W, pre + "right.", h, eps)
    return 0.5 * (rms(left, eps) * W[pre + "left.out"] + rms(right, eps) * W[pre + "right.out"])


def route(z: np.ndarray, top: int):
    """The ``top`` largest logits (ties to the lower index) and the softmax over them alone."""
    order = sorted(range(len(z)), key=lambda e: (-z[e], e))[:top]
    e = np.exp(z[order] - z[order].max())
    rest = sorted(range(len(z)), key=lambda e: (-z[e], e))
    gap = float(z[rest[top - 1]] - z[rest[top]]) if top < len(z) else float("inf")
    return order, e / e.sum(), gap


def moe_ff(ff: dict, W, pre: str, h: np.ndarray, picked=None, gaps=None) -> np.ndarray:
    """Experts ``W_down relu(W_up h)^2`` behind a router whose weights are the softmax over the picked logits."""
    top = ff["router"]["top"]
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        z = W[pre + "router"] @ h[t]
        order, wts, gap = route(z, top)
        if picked is not None:
            picked.append(order)
        if gaps is not None:
            gaps.append(gap)
        for e, w in zip(order, wts):
            a = np.maximum(W[f"{pre}e{e}.up"] @ h[t], 0.0) ** 2
            out[t] += w * (W[f"{pre}e{e}.down"] @ a)
    return out


def layer(cfg, W, i: int, x: np.ndarray, picked=None, gaps=None) -> np.ndarray:
    spec, eps, pre = cfg["layers"][i], float(cfg["norm"]["eps"]), f"l{i}."
    h = rms(x, eps) * W[pre + "norm1"]
    if cfg.get("canon"):
        h = h + causal_conv(h, W[pre + "canon1"])
    if spec["type"] == "mlstm":
        y = mlstm_mixer(spec["mixer"], W, pre + "mix.", h, eps)
    elif spec["type"] == "parallel":
        y = parallel_mixer(spec["mixer"], W, pre + "mix.", h, eps)
    else:
        raise ValueError(spec["type"])
    x = x + rms(y, eps) * W[pre + "norm1b"]
    if spec.get("mlp") is not None:
        y = moe_ff(spec["mlp"], W, pre + "mlp.", rms(x, eps) * W[pre + "norm2"], picked, gaps)
        x = x + rms(y, eps) * W[pre + "norm2b"]
    return x


def forward(cfg, W, tokens: List[int], keep_layers: bool = False, picks: Optional[dict] = None, gaps: Optional[dict] = None):
    """Logits [T, vocab] of a whole sequence; with ``keep_layers`` also the stream after every layer.  ``picks`` /
    ``gaps`` (dicts) receive, by a routed feed-forward's tensor-name prefix, every token's experts and the gap
    between the last picked logit and the next."""
    eps = float(cfg["norm"]["eps"])
    x = rms(W["embed"][np.asarray(tokens)].astype(np.float64), eps) * W["embed.norm"]
    kept = []
    for i in range(len(cfg["layers"])):
        routed = cfg["layers"][i].get("mlp") is not None
        x = layer(cfg, W, i, x, picks.setdefault(f"l{i}.mlp", []) if picks is not None and routed else None,
                  gaps.setdefault(f"l{i}.mlp", []) if gaps is not None and routed else None)
        if keep_layers:
            kept.append(x.copy())
    z = (rms(x, eps) * W["final.norm"]) @ W["head"].T
    cap = float(cfg.get("logit_softcap") or 0.0)
    logits = cap * np.tanh(z / cap) if cap else z
    return (logits, np.stack(kept)) if keep_layers else logits


def greedy(cfg, W, prompt: List[int], new_tokens: int) -> List[int]:
    toks = list(prompt)
    for _ in range(new_tokens):
        toks.append(int(np.argmax(forward(cfg, W, toks)[-1])))
    return toks[len(prompt):]


def read_model(model_dir: str):
    """config.json and every tensor of model.safetensors as float64 (integer tables as they are)."""
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as f:
        cfg = json.load(f)
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    W: Dict[str, np.ndarray] = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw = data[lo:hi]
        if info["dtype"] == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif info["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif info["dtype"] == "I32":
            a = np.frombuffer(raw, dtype="<i4").copy()
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
        W[name] = a.reshape(info["shape"])
    return cfg, W
