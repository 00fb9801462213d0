"""Dimuvik restated plainly: one function per mechanism, float64, loops over tokens.

Nothing here is shared with the engine: weights arrive as a dict of numpy arrays by tensor
name, the configuration as the parsed ``config.json``.  Slow on purpose; the tests use small
sizes.  Notation: ``x`` a row of the residual stream, ``h`` what a sublayer reads, ``p`` a position.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

import numpy as np


def rms(x: np.ndarray, eps: float) -> np.ndarray:
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def dyt(x: np.ndarray, w: Dict[str, np.ndarray], name: str) -> np.ndarray:
    """The norm without statistics: tanh(alpha x) w + b."""
    return np.tanh(float(w[name + ".alpha"]) * x) * w[name] + w[name + ".b"]


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


def rotate_pairs(v: np.ndarray, p: int, base: float, dims: int) -> np.ndarray:
    """Entries (2i, 2i+1) of the first ``dims`` turn by p * base^(-2i/dims); the rest pass."""
    out = v.copy()
    for i in range(dims // 2):
        a = p * base ** (-2.0 * i / dims)
        c, s = math.cos(a), math.sin(a)
        u, w = v[..., 2 * i], v[..., 2 * i + 1]
        out[..., 2 * i] = u * c - w * s
        out[..., 2 * i + 1] = w * c + u * s
    return out


def softmax_rows(s: np.ndarray, sink: Optional[float] = None):
    """Weights of one row of scores; with a sink the divisor also holds exp(sink)."""
    m = s.max() if sink is None else max(s.max(), sink)
    e = np.exp(s - m)
    d = e.sum() + (0.0 if sink is None else math.exp(sink - m))
    return e / d


def query_temperature(p: int, coef: float, every: int) -> float:
    return 1.0 + coef * math.log((p + 1) // every + 1)


def projected(h: np.ndarray, w: Dict[str, np.ndarray], name: str) -> np.ndarray:
    """W h + b, then the convolution over time when the tensor has one."""
    u = h @ w[name].T + w[name + ".b"]
    return causal_conv(u, w[name + ".conv"]) if name + ".conv" in w else u


def differential_keys_values(h: np.ndarray, w: Dict[str, np.ndarray], pre: str):
    """Keys [T, G * 2 * dim] and values [T, G * vdim] after projection, bias and convolution."""
    return projected(h, w, pre + ".k"), projected(h, w, pre + ".v")


def differential_attention(h: np.ndarray, w: Dict[str, np.ndarray], pre: str, m: dict, eps: float, k: np.ndarray, v: np.ndarray) -> np.ndarray:
    """Two softmax maps per head over the same values, o = a1 - lambda a2, normed per head, times (1 - diff)."""
    T = h.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    diff, scale = float(m["diff"]), float(m["scale"])
    q = projected(h, w, pre + ".q")
    qt = m.get("q_temp")
    lam = (math.exp(float(np.sum(w[pre + ".lq1"] * w[pre + ".lk1"]))) - math.exp(float(np.sum(w[pre + ".lq2"] * w[pre + ".lk2"]))) + diff)
    out = np.zeros((T, H * vd))
    for t in range(T):
        qrow = q[t] * (query_temperature(t, float(qt["coef"]), int(qt["every"])) if qt else 1.0)
        for hd in range(H):
            g = hd // (H // G)
            maps = []
            for mp in range(2):
                qv = qrow[(hd * 2 + mp) * d:(hd * 2 + mp + 1) * d]
                keys = k[:t + 1, (g * 2 + mp) * d:(g * 2 + mp + 1) * d]
                wts = softmax_rows((keys @ qv) * scale)
                maps.append(wts @ v[:t + 1, g * vd:(g + 1) * vd])
            o = maps[0] - lam * maps[1]
            out[t, hd * vd:(hd + 1) * vd] = rms(o, eps) * (1.0 - diff)
    return out @ w[pre + ".o"].T


def latent_cache(h: np.ndarray, w: Dict[str, np.ndarray], pre: str, m: dict, eps: float):
    """The latent c [T, kv_rank] (normed, weighted) and the shared rotated key part r [T, rot_dim]."""
    rank = m["kv_rank"]
    d = h @ w[pre + ".dkv"].T
    c = rms(d[:, :rank], eps) * w[pre + ".dkv.norm"]
    r = np.stack([rotate_pairs(d[t, rank:], t, float(m["rot"]["base"]), int(m["rot"]["dims"])) for t in range(h.shape[0])])
    return c, r


def latent_attention(h: np.ndarray, w: Dict[str, np.ndarray], pre: str, m: dict, eps: float, c: np.ndarray, r: np.ndarray) -> np.ndarray:
    """Queries through their own latent, keys and values brought up per head from the cached latents ``c`` and the shared
    rotated key parts ``r`` (this layer's own, or those of the layer whose cache it reads)."""
    T = h.shape[0]
    H, d, rd, vd, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    scale = float(m["scale"])
    cq = rms(h @ w[pre + ".dq"].T, eps) * w[pre + ".dq.norm"]
    q = cq @ w[pre + ".uq"].T
    ku = c @ w[pre + ".uk"].T          # [T, H * dim]
    vu = c @ w[pre + ".uv"].T          # [T, H * vdim]
    out = np.zeros((T, H * vd))
    for t in range(T):
        for hd in range(H):
            qh = q[t, hd * (d + rd):(hd + 1) * (d + rd)]
            q_plain = qh[:d]
            q_rot = rotate_pairs(qh[d:], t, float(m["rot"]["base"]), int(m["rot"]["dims"]))
            s = (ku[:t + 1, hd * d:(hd + 1) * d] @ q_plain + r[:t + 1] @ q_rot) * scale
            wts = softmax_rows(s, float(w[pre + ".sink"][hd]))
            out[t, hd * vd:(hd + 1) * vd] = wts @ vu[:t + 1, hd * vd:(hd + 1) * vd]
    return out @ w[pre + ".o"].T


def dense_feed_forward(h: np.ndarray, w: Dict[str, np.ndarray], pre: str) -> np.ndarray:
    z = np.maximum(h @ w[pre + ".up"].T, 0.0)
    return (z * z) @ w[pre + ".down"].T


def gated_expert(h: np.ndarray, w: Dict[str, np.ndarray], pre: str) -> np.ndarray:
    return (silu(h @ w[pre + ".gate"].T) * (h @ w[pre + ".up"].T)) @ w[pre + ".down"].T


def route(h: np.ndarray, w: Dict[str, np.ndarray], pre: str, ff: dict):
    """Per row: the chosen experts (by score + correction) and their weights (score * router.scale)."""
    z = h @ w[pre + ".router"].T
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z)
    s /= s.sum(axis=-1, keepdims=True)
    choice = s + w[pre + ".correction"]
    top = int(ff["router"]["top"])
    picks = np.argsort(-choice, axis=-1, kind="stable")[:, :top]
    weights = np.take_along_axis(s, picks, axis=-1) * float(ff["router"]["scale"])
    return picks, weights


def routed_feed_forward(h: np.ndarray, w: Dict[str, np.ndarray], pre: str, ff: dict, picks_out: Optional[dict] = None) -> np.ndarray:
    picks, weights = route(h, w, pre, ff)
    if picks_out is not None:
        picks_out[pre] = picks.tolist()
    out = np.zeros((h.shape[0], w[pre + ".e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, wt in zip(picks[t], weights[t]):
            out[t] += wt * gated_expert(h[t:t + 1], w, f"{pre}.e{e}")[0]
    if ff.get("shared"):
        out += gated_expert(h, w, pre + ".shared")
    return out


def forward(cfg: dict, w: Dict[str, np.ndarray], tokens: List[int], layer_outputs: Optional[list] = None,
            picks: Optional[dict] = None) -> np.ndarray:
    """Logits [T, vocab] of one sequence from position 0; ``layer_outputs`` collects the stream after every layer,
    ``picks`` the chosen experts of every routed feed-forward by its tensor-name prefix."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][np.asarray(tokens)] * float(cfg.get("embedding", {}).get("scale", 1.0))
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        pre, m = f"l{i}", layer["mixer"]
        h = dyt(x, w, pre + ".norm1")
        if layer["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = differential_keys_values(h, w, pre + ".mix")
            k, v = kept[i if src is None else src]
            y = differential_attention(h, w, pre + ".mix", m, eps, k, v)
        elif layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = latent_cache(h, w, pre + ".mix", m, eps)
            c, r = kept[i if src is None else src]
            y = latent_attention(h, w, pre + ".mix", m, eps, c, r)
        else:
            raise ValueError(f"unknown layer type {layer['type']}")
        x = x + dyt(y, w, pre + ".norm1b")
        ff = layer.get("mlp")
        if ff is not None:
            h = dyt(x, w, pre + ".norm2")
            y = dense_feed_forward(h, w, pre + ".mlp") if ff["kind"] == "dense" else routed_feed_forward(h, w, pre + ".mlp", ff, picks)
            x = x + dyt(y, w, pre + ".norm2b")
        if layer_outputs is not None:
            layer_outputs.append(x.copy())
    return dyt(x, w, "final.norm") @ w["head"].T


def read_safetensors(path: str) -> Dict[str, np.ndarray]:
    """A reader of its own: 8 bytes of length, a JSON header, raw little-endian data; everything widened to float64
    (integer tables stay integers)."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        raw = data[a:b]
        if info["dtype"] == "BF16":
            arr = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif info["dtype"] == "F32":
            arr = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif info["dtype"] == "I32":
            arr = np.frombuffer(raw, dtype="<i4").copy()
        else:
            raise ValueError(f"{name}: dtype {info['dtype']} is not read here")
        out[name] = arr.reshape(info["shape"])
    return out


def greedy(cfg: dict, w: Dict[str, np.ndarray], prompt: List[int], n: int) -> List[int]:
    """n tokens after the prompt, each the first largest logit."""
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(np.argmax(forward(cfg, w, toks)[-1])))
    return toks[len(prompt):]


def load_folder(model_dir: str):
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))
