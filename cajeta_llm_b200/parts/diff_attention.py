"""Differential attention over the paged cache: two softmax maps per head over the same values.

Per row at position ``p`` with ``H`` query heads over ``G`` key/value heads (head ``h`` reads key head
``h // (H / G)``), a map's query / key size ``dim`` and the values' size ``vdim``::

    q = W_q x (+ b_q)      H * 2 * dim rows, head by head [map 1 | map 2]
    k = W_k x (+ b_k)      G * 2 * dim rows, head by head [map 1 | map 2]
    v = W_v x (+ b_v)      G * vdim rows
    q, k, v <- conv(q), conv(k), conv(v)        a causal convolution over time per channel (optional)
    q <- q * (1 + coef * ln(floor((p + 1) / every) + 1))      the query's temperature (optional)
    a_m = sum_j softmax_j((q_m . k_m,j) scale) v_j ,  j in [from, p]           m = 1, 2
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + lambda_init                     one number for the layer
    o = a_1 - lambda a_2 ;  o <- o / sqrt(mean(o^2) + eps) * (1 - lambda_init)    per head, over vdim, no weight
    then W_o on the heads

The cache holds a key head's ``[k1 | k2]`` as one entry of ``2 * dim`` and its value of ``vdim`` (after the
convolution); the last ``taps - 1`` projected rows of a request are per-request state.  No rotation: positions enter
through the mask and the temperature alone.  Scores, both softmaxes, the difference, ``lambda`` and the head's norm are
float32 on either path.  An entry that reads another entry's cache (``owns_cache`` false in the spec, the plan's
``cache_from``) has no key / value tensors, projects and convolves its queries only, and attends over that entry's
keys and values with its own queries, ``lambda`` and output projection.

Parameters: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim`` (one map's), ``value_dim``, ``scale``,
``lambda_init``, ``eps``, ``window`` (0: none), ``bias`` (q, k and v carry biases named ``<tensor>.b``), ``proj_conv``
(``{"taps": n}``; weights ``<tensor>.conv`` of ``[channels, taps]``), ``q_temp`` (``{"coef": c, "every": n}``),
``owns_cache``, ``names`` (``q k v o lq1 lk1 lq2 lk2`` under the part's prefix).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import kernels as K
from .base import KvNeed, Part, StateNeed, register_part
from .linear import project
from .plan import ParamSpec


@register_part("mixer", "differential_attention")
class DifferentialAttention(Part):
    graph_safe = True             # rows, requests and slots come from the step's device metadata only

    def __init__(self, spec, prefix, runtime):
        super().__init__(spec, prefix, runtime)
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["num_heads"])
        self.kv_heads = int(spec["num_kv_heads"])
        self.dim = int(spec["head_dim"])
        self.vdim = int(spec["value_dim"])
        self.scale = float(spec["scale"])
        self.lambda_init = float(spec["lambda_init"])
        self.eps = float(spec["eps"])
        self.window = int(spec.get("window", 0) or 0)
        self.bias = bool(spec.get("bias", False))
        self.owns_cache = bool(spec.get("owns_cache", True))
        conv = dict(spec.get("proj_conv") or {})
        self.has_conv = bool(conv)
        self.taps = int(conv.get("taps", 1)) if conv else 1
        temp = dict(spec.get("q_temp") or {})
        self.temp_coef = float(temp.get("coef", 0.0)) if temp else 0.0
        self.temp_every = int(temp.get("every", 1)) if temp else 1
        if self.heads % self.kv_heads != 0:
            raise ValueError(f"num_heads {self.heads} is not a multiple of num_kv_heads {self.kv_heads}")
        if self.dim > 256 or self.vdim > 256:
            raise ValueError(f"head_dim {self.dim} / value_dim {self.vdim}: the attention kernels take up to 256")
        if self.taps < 1 or self.temp_every < 1:
            raise ValueError("proj_conv.taps and q_temp.every must be >= 1")
        names = dict(spec.get("names") or {})
        self.n = {k: self.name(names.get(k, k)) for k in ("q", "k", "v", "o", "lq1", "lk1", "lq2", "lk2")}
        self.q_dim = self.heads * 2 * self.dim
        self.k_dim = self.kv_heads * 2 * self.dim if self.owns_cache else 0
        self.v_dim = self.kv_heads * self.vdim if self.owns_cache else 0
        self.o_dim = self.heads * self.vdim
        self.channels = self.q_dim + self.k_dim + self.v_dim
        self.w_in = self.b_in = self.w_conv = self.w_o = None
        self.lam = 0.0

    def _projected(self):
        """(letter, rows) of what this part projects: q alone when it reads another entry's cache."""
        return (("q", self.q_dim), ("k", self.k_dim), ("v", self.v_dim)) if self.owns_cache else (("q", self.q_dim),)

    def cache_need(self) -> Optional[KvNeed]:
        return KvNeed(self.kv_heads, 2 * self.dim, self.window, value_dim=0 if self.vdim == 2 * self.dim else self.vdim)

    def state_need(self) -> Optional[StateNeed]:
        if self.taps > 1:
            return StateNeed(((self.taps - 1) * self.channels,), torch.float32)
        return None

    def params(self) -> Dict[str, ParamSpec]:
        p = {self.n["o"]: ParamSpec((self.hidden, self.o_dim))}
        for letter, rows in self._projected():
            p[self.n[letter]] = ParamSpec((rows, self.hidden))
            if self.bias:
                p[self.n[letter] + ".b"] = ParamSpec((rows,), role="vector")
            if self.has_conv:
                p[self.n[letter] + ".conv"] = ParamSpec((rows, self.taps), role="vector", std=0.3)
        for k in ("lq1", "lk1", "lq2", "lk2"):
            p[self.n[k]] = ParamSpec((self.dim,), role="vector", std=0.1)
        return p

    def libraries(self) -> set:
        libs = {"attention_diff", "attention_paged", "gemm_simt"}
        if self.has_conv:
            libs.add("recurrent")
        if self.runtime.fast_kernels and self.hidden >= 128:
            libs |= {"gemm_tc", "gemm_tc2"}
        return libs

    def _tiled(self) -> bool:
        """Whether attention runs in its tiled form (tensor cores): bfloat16 storage and sizes the form takes; float32
        runs, and other sizes, take the row-at-a-time form."""
        rt = self.runtime
        return bool(rt.fast_kernels and rt.act_dtype == torch.bfloat16 and rt.cache_dtype == torch.bfloat16
                    and K.diff_tile_shape(self.dim, self.vdim))

    def load(self, source) -> None:
        parts = self._projected()
        self.w_in = torch.cat([self.fetch(source, self.n[letter]) for letter, _ in parts], dim=0).contiguous()      # one product
        if self.bias:
            self.b_in = torch.cat([self.fetch(source, self.n[letter] + ".b") for letter, _ in parts], dim=0).contiguous()
        if self.has_conv:
            self.w_conv = torch.cat([self.fetch(source, self.n[letter] + ".conv") for letter, _ in parts], dim=0).contiguous()
        self.w_o = self.fetch(source, self.n["o"])
        # one number for the layer, float32: exp(lq1 . lk1) - exp(lq2 . lk2) + lambda_init
        lq1, lk1, lq2, lk2 = (self.fetch(source, self.n[k]) for k in ("lq1", "lk1", "lq2", "lk2"))
        lam = torch.exp(torch.sum(lq1 * lk1)) - torch.exp(torch.sum(lq2 * lk2)) + self.lambda_init
        self.lam = float(lam.item())

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, entry) -> None:
        rt = self.runtime
        dev = x.device
        T = x.shape[0]
        write = entry.writes_cache
        if write != self.owns_cache:
            raise ValueError(f"{self.prefix}: the plan and the part disagree on who owns the cache")
        C = self.channels
        qkv = torch.empty((T, C), dtype=torch.float32, device=dev)
        K.tag = "qkv"
        project(rt, x, self.w_in, qkv, bias=self.b_in)
        if self.w_conv is not None:
            at = getattr(entry, "state_offset", 0)
            conv = torch.empty((T, C), dtype=torch.float32, device=dev)
            K.tag = "short conv"
            # one tap keeps no state: the kernel then reads none, and is given a word to point at
            state = entry.state if self.taps > 1 else torch.zeros((1, 1), dtype=torch.float32, device=dev)
            K.short_conv(qkv, 0, C, self.taps, self.w_conv, None, state, ctx.row_req, ctx.req_start, ctx.req_slot, conv,
                         activate=False, state_offset=at)
            if self.taps > 1:
                K.short_conv_commit(qkv, 0, C, self.taps, entry.state, ctx.req_start, ctx.req_slot, ctx.n_requests, state_offset=at)
            qkv = conv
        kd = 2 * self.dim
        q = torch.empty((T, self.heads, kd), dtype=rt.act_dtype, device=dev)
        K.tag = "heads + cache write"
        K.head_prepare(qkv, 0, self.q_dim, self.q_dim + self.k_dim, q, entry.k_plane if write else None,
                       entry.v_plane if write else None, ctx.positions, ctx.row_req, entry.block_table, entry.page_tokens,
                       self.heads, self.kv_heads, kd, self.vdim, 0, None, 1.0, None, None, 0.0, write,
                       q_temp_coef=self.temp_coef, q_temp_every=self.temp_every)
        out = torch.empty((T, self.heads, self.vdim), dtype=rt.act_dtype, device=dev)
        K.tag = "differential attention"
        tiled = self._tiled() and hasattr(ctx, "req_start") and hasattr(ctx, "req_prior")
        # how far a row's keys can reach, as a number that a captured step may keep: a decode step's context (its graph is
        # keyed by the context's bucket), otherwise what the block table spans; it only decides into how many stretches a
        # row block's keys are cut when the step has few rows
        reach = 0
        if tiled:
            reach = ctx.max_context if getattr(ctx, "all_single", False) else entry.block_table.shape[1] * entry.page_tokens
        K.diff_attention(q, out, entry.k_plane, entry.v_plane, ctx.positions, ctx.row_req, entry.block_table, entry.page_tokens,
                         self.heads, self.kv_heads, self.dim, self.vdim, self.window, self.scale, self.lam, self.eps,
                         1.0 - self.lambda_init, req_start=ctx.req_start if tiled else None,
                         req_prior=ctx.req_prior if tiled else None, n_requests=ctx.n_requests if tiled else 0, reach=reach,
                         tile_rows=16 if getattr(ctx, "all_single", False) else 64)
        K.tag = "o"
        project(rt, out.view(T, self.o_dim), self.w_o, residual, accumulate=True)
        K.tag = None
        return None
