"""Grouped-query attention over the paged cache.

Per row at absolute position ``p``: ``q = x Wq^T + bq``, ``k = x Wk^T + bk``,
``v = x Wv^T + bv`` (bias after the product, none on the output projection:
model/Attention.cajeta:48-56,102-111, model/Linear.cajeta:1883-1898); the position
encoding rotates q and k; rotated k and raw v are appended to the cache at ``p``
(model/CausalLM.cajeta:1454-1485); head ``h`` attends with kv head
``h / (heads / kv_heads)`` over keys ``[from, p]``, ``from = p + 1 - window`` when a
window is set and exceeded, else 0, scale ``1 / sqrt(head_dim)`` unless given
(model/PagedKvCache.cajeta:374-470, model/Attention.cajeta:67-71); the output
projection is added into the residual stream (model/CausalLM.cajeta:1498,1506).

Parameters: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``window``,
``qkv_bias``, ``out_bias``, ``scale``, ``position`` (a position PartSpec).

Optional, each off by default (a mixer that sets any of them runs the general kernels:
``head_prepare`` and the general paged attention):
``value_dim``: the values' head size when it is not the keys';
``softcap`` c > 0: a score becomes ``c tanh(s / c)`` after the scale;
``qk_norm``: ``{"q": name, "k": name, "eps": e}``, an RMS norm over each head of q and of k with a
weight of ``head_dim`` shared by the heads, before the rotation;
``values_from_keys``: there is no value projection, a key as projected (before norm and rotation)
is also the value;
``head_gate``: a tensor name; ``W_g`` of ``[num_heads, hidden]`` reads the mixer's input and head
``h``'s output is multiplied by ``sigmoid(W_g x)_h`` before the output projection;
``names``: the tensor names of ``q``, ``k``, ``v``, ``o`` under the part's prefix.
A position part's ``magnitude`` (a stretched rotation's) multiplies cos and sin.

Further optional parameters; a mixer that sets any of them runs ``head_prepare`` and the attention kernel that
sees all heads of a row at once (``mixed_heads_attention``):
``proj_conv``: ``{"taps": n, "q": name, "k": name, "v": name}``, a causal convolution over time on every channel
of q, k and v right after the projection (``y_t = sum_j w[:, j] u_(t - taps + 1 + j)``, weights ``[channels, taps]``,
no bias, no activation); the last ``taps - 1`` projected rows of a request are per-request state
(``state_need()``), found at ``entry.state_offset`` of the entry's state;
``qk_norm`` with ``"whole": true``: ONE statistic over all heads of q (of k), weights of ``heads * head_dim``
(``kv_heads * head_dim``) entries;
``head_temp``: a tensor name, ``[heads]``: head h's score is multiplied by its entry (after the scale);
``talk``: a tensor name, ``[heads, heads]``: the heads' scores of a (query, key) pair are mixed before the
softmax, ``s_h <- sum_g talk[h, g] s_g``;
``sink``: a tensor name, ``[heads]``: the softmax's divisor also holds ``exp(sink[h])``, a key without value
that is neither scaled nor mixed.

An entry that reads another entry's cache (``entry.writes_cache`` false) projects and
rotates only q.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..csrc import kernels as K
from .base import KvNeed, Part, make_part, register_part
from .linear import project, project_split
from .plan import ParamSpec


@register_part("mixer", "attention")
class PagedAttention(Part):
    def __init__(self, spec, prefix, runtime):
        super().__init__(spec, prefix, runtime)
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["num_heads"])
        self.kv_heads = int(spec["num_kv_heads"])
        self.head_dim = int(spec["head_dim"])
        self.window = int(spec.get("window", 0) or 0)
        self.qkv_bias = bool(spec.get("qkv_bias", False))
        self.out_bias = bool(spec.get("out_bias", False))
        scale = spec.get("scale")
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.value_dim = int(spec.get("value_dim", 0) or self.head_dim)
        self.softcap = float(spec.get("softcap", 0.0) or 0.0)
        self.qk_norm = dict(spec.get("qk_norm") or {}) or None
        self.values_from_keys = bool(spec.get("values_from_keys", False))
        self.head_gate = spec.get("head_gate") or None
        self.proj_conv = dict(spec.get("proj_conv") or {}) or None
        self.head_temp = spec.get("head_temp") or None
        self.talk = spec.get("talk") or None
        self.sink = spec.get("sink") or None
        names = dict(spec.get("names") or {})
        self.n_proj = {n: self.name(names.get(n, f"{n}_proj.weight")) for n in ("q", "k", "v", "o")}
        self.allow_pending = True          # a block that has no norm after the mixer sets this False
        if self.values_from_keys and self.value_dim != self.head_dim:
            raise ValueError("values_from_keys needs value_dim == head_dim")
        if self.softcap < 0.0:
            raise ValueError(f"softcap must be positive (or 0 for none), found {self.softcap}")
        if self.heads % self.kv_heads != 0:
            raise ValueError(f"num_heads {self.heads} is not a multiple of num_kv_heads {self.kv_heads}")
        if self.head_dim > 256:
            raise ValueError(f"head_dim {self.head_dim} is larger than the attention kernels take (256)")
        self.position = make_part("position", spec["position"], prefix, runtime)
        self.q_dim = self.heads * self.head_dim
        self.kv_dim = self.kv_heads * self.head_dim
        self.v_dim = 0 if self.values_from_keys else self.kv_heads * self.value_dim
        self.o_dim = self.heads * self.value_dim
        self.general = bool(self.softcap > 0.0 or self.qk_norm or self.values_from_keys or self.head_gate
                            or self.value_dim != self.head_dim or getattr(self.position, "magnitude", 1.0) != 1.0)
        self.norm_whole = bool(self.qk_norm and self.qk_norm.get("whole"))
        self.mixed = bool(self.proj_conv or self.head_temp or self.talk or self.sink or self.norm_whole)
        self.general = self.general or self.mixed
        if self.general and (self.qkv_bias or self.out_bias):
            raise ValueError("the general attention path is built without biases")
        if self.mixed and (self.softcap > 0.0 or self.head_gate or self.values_from_keys):
            raise ValueError("mixed heads, a sink or a convolved projection are built without softcap, head_gate and values_from_keys")
        self.taps = int(self.proj_conv["taps"]) if self.proj_conv else 1
        if self.taps < 1:
            raise ValueError(f"proj_conv.taps must be >= 1, found {self.taps}")
        self.graph_safe = True             # rows, requests and slots come from the step's device metadata only
        self.w_conv = self.temp_w = self.talk_w = self.sink_w = None
        self.q_norm_w = self.k_norm_w = None
        self.w_qkv: Optional[torch.Tensor] = None
        self.b_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.b_o: Optional[torch.Tensor] = None

    # -- what the cache manager must provide ----------------------------------------
    def cache_need(self) -> Optional[KvNeed]:
        return KvNeed(self.kv_heads, self.head_dim, self.window, value_dim=0 if self.value_dim == self.head_dim else self.value_dim)

    def state_need(self):
        if self.proj_conv and self.taps > 1:
            from .base import StateNeed
            return StateNeed(((self.taps - 1) * (self.q_dim + self.kv_dim + self.v_dim),), torch.float32)
        return None

    # -- tensors ---------------------------------------------------------------------
    def params(self) -> Dict[str, ParamSpec]:
        p = {
            self.n_proj["q"]: ParamSpec((self.q_dim, self.hidden)),
            self.n_proj["k"]: ParamSpec((self.kv_dim, self.hidden)),
            self.n_proj["o"]: ParamSpec((self.hidden, self.o_dim)),
        }
        if not self.values_from_keys:
            p[self.n_proj["v"]] = ParamSpec((self.v_dim, self.hidden))
        if self.qk_norm:
            p[self.name(self.qk_norm["q"])] = ParamSpec((self.q_dim if self.norm_whole else self.head_dim,), role="vector", init="ones")
            p[self.name(self.qk_norm["k"])] = ParamSpec((self.kv_dim if self.norm_whole else self.head_dim,), role="vector", init="ones")
        if self.proj_conv:
            for n, rows in (("q", self.q_dim), ("k", self.kv_dim), ("v", self.v_dim)):
                p[self.name(self.proj_conv[n])] = ParamSpec((rows, self.taps), role="vector", std=0.2)
        if self.head_temp:
            p[self.name(self.head_temp)] = ParamSpec((self.heads,), role="vector", init="ones")
        if self.talk:
            p[self.name(self.talk)] = ParamSpec((self.heads, self.heads), role="vector", std=0.3)
        if self.sink:
            p[self.name(self.sink)] = ParamSpec((self.heads,), role="vector", std=1.0)
        if self.head_gate:
            p[self.name(self.head_gate)] = ParamSpec((self.heads, self.hidden))
        if self.qkv_bias:
            p[self.name("q_proj.bias")] = ParamSpec((self.q_dim,), role="vector")
            p[self.name("k_proj.bias")] = ParamSpec((self.kv_dim,), role="vector")
            p[self.name("v_proj.bias")] = ParamSpec((self.kv_dim,), role="vector")
        if self.out_bias:
            p[self.name("o_proj.bias")] = ParamSpec((self.hidden,), role="vector")
        return p

    def libraries(self) -> set:
        libs = {"rowwise", "gemm_simt"}
        if self.mixed:
            libs |= {"attention_paged"} | ({"recurrent"} if self.proj_conv else set())
            if self._tiled():
                libs.add("attention_mixed")
        elif self.general:
            libs.add("attention_paged")
            if self.runtime.fast_kernels and self.value_dim == self.head_dim:
                if self.head_dim in (64, 128):
                    libs.add("attention_decode")
                if self.head_dim in (32, 64, 96, 128):
                    libs.add("attention_prefill_tc" if self.head_dim == 128 else "attention_prefill")
        elif self.runtime.fast_kernels and self.head_dim in (64, 128):
            libs |= {"attention_decode", "attention_prefill_tc" if self.head_dim == 128 else "attention_prefill"}
        else:
            libs.add("attention_paged")
        if self.runtime.fast_kernels and self.hidden >= 128:
            libs |= {"gemm_tc", "gemm_tc2"}
        return libs

    def load(self, source) -> None:
        # q, k and v rows are stacked so that one product yields all three
        rows = [self.fetch(source, self.n_proj[n]) for n in (("q", "k") if self.values_from_keys else ("q", "k", "v"))]
        if self.head_gate:
            rows.append(self.fetch(source, self.name(self.head_gate)))      # the gate's rows ride along: one product
        self.w_qkv = torch.cat(rows, dim=0).contiguous()
        if self.qk_norm:
            self.q_norm_w = self.fetch(source, self.name(self.qk_norm["q"]))
            self.k_norm_w = self.fetch(source, self.name(self.qk_norm["k"]))
        if self.proj_conv:
            self.w_conv = torch.cat([self.fetch(source, self.name(self.proj_conv[n])) for n in ("q", "k", "v")], dim=0).contiguous()
        for attr, n in (("temp_w", self.head_temp), ("talk_w", self.talk), ("sink_w", self.sink)):
            if n:
                setattr(self, attr, self.fetch(source, self.name(n)))
        if self.qkv_bias:
            self.b_qkv = torch.cat([self.fetch(source, self.name(f"{n}_proj.bias")) for n in ("q", "k", "v")], dim=0).contiguous()
        self.w_o = self.fetch(source, self.n_proj["o"])
        if self.out_bias:
            self.b_o = self.fetch(source, self.name("o_proj.bias"))

    # -- one step --------------------------------------------------------------------
    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, entry) -> Optional[torch.Tensor]:
        if self.mixed:
            return self._forward_mixed(x, residual, ctx, entry)
        if self.general:
            return self._forward_general(x, residual, ctx, entry)
        rt = self.runtime
        T = x.shape[0]
        pos = self.position
        write = entry.writes_cache
        n_out = self.q_dim + (2 * self.kv_dim if write else 0)
        qkv = torch.empty((T, n_out), dtype=torch.float32, device=x.device)
        K.tag = "qkv"
        project(rt, x, self.w_qkv[:n_out], qkv, bias=None if self.b_qkv is None else self.b_qkv[:n_out])
        q = torch.empty((T, self.heads, self.head_dim), dtype=rt.act_dtype, device=x.device)
        K.tag = "rope + cache write"
        K.rope_kv_write(qkv, 0, self.q_dim, self.q_dim + self.kv_dim, q, entry.k_plane, entry.v_plane,
                        ctx.positions, ctx.row_req, entry.block_table, entry.page_tokens, self.heads, self.kv_heads,
                        self.head_dim, pos.rotary_dim, pos.inv_freq, write)
        out = torch.empty_like(q)
        K.tag = "attention"
        if rt.fast_kernels and getattr(ctx, "all_single", False) and self.head_dim in (64, 128):
            # every request brings one token: the split-KV decode kernel
            K.decode_attention(q, out, entry.k_plane, entry.v_plane, ctx.positions, ctx.row_req, entry.block_table,
                               entry.page_tokens, self.heads, self.kv_heads, self.head_dim, self.window, self.scale,
                               ctx.max_context, getattr(ctx, "decode_scratch", None) or rt.decode_scratch)
        elif rt.fast_kernels and self.head_dim == 128 and entry.page_tokens == 16 and hasattr(ctx, "req_start"):
            # portions of prompts (and whatever single tokens ride along): both products on tcgen05,
            # scores and output in tensor memory
            K.prefill_attention_tc(q, out, entry.k_plane, entry.v_plane, ctx.req_start, ctx.req_prior, entry.block_table,
                                   entry.page_tokens, self.heads, self.kv_heads, self.head_dim, self.window, self.scale)
        elif rt.fast_kernels and self.head_dim in (64, 128) and hasattr(ctx, "req_start"):
            # other page sizes, head size 64: query tiles on mma.sync
            K.prefill_attention(q, out, entry.k_plane, entry.v_plane, ctx.req_start, ctx.req_prior, entry.block_table,
                                entry.page_tokens, self.heads, self.kv_heads, self.head_dim, self.window, self.scale)
        else:
            K.paged_attention(q, out, entry.k_plane, entry.v_plane, ctx.positions, ctx.row_req, entry.block_table,
                              entry.page_tokens, self.heads, self.kv_heads, self.head_dim, self.window, self.scale)
        K.tag = "o"
        parts = project_split(rt, out.view(T, self.q_dim), self.w_o, bias=self.b_o) if self.allow_pending else None
        if parts is None:
            project(rt, out.view(T, self.q_dim), self.w_o, residual, bias=self.b_o, accumulate=True)
        K.tag = None
        return parts                         # partial sums owed to the residual stream (the next norm adds them), or None

    def _forward_general(self, x: torch.Tensor, residual: torch.Tensor, ctx, entry) -> Optional[torch.Tensor]:
        """The path of a mixer with any of the optional parameters: one product for q | k | (v) | (gate), heads made
        ready (norm, rotation, cache write), attention with capped scores and gated heads, output projection."""
        rt = self.runtime
        T = x.shape[0]
        pos = self.position
        write = entry.writes_cache
        gate_cols = self.heads if self.head_gate else 0
        if write:
            w, k_off, v_off, g_off = self.w_qkv, self.q_dim, self.q_dim + self.kv_dim, self.q_dim + self.kv_dim + self.v_dim
        else:
            # an entry that reads another entry's cache projects q (and the gate) only
            w = self.w_qkv[:self.q_dim] if not gate_cols else torch.cat([self.w_qkv[:self.q_dim], self.w_qkv[-gate_cols:]], dim=0)
            k_off, v_off, g_off = 0, 0, self.q_dim
        qkv = torch.empty((T, w.shape[0]), dtype=torch.float32, device=x.device)
        K.tag = "qkv"
        project(rt, x, w, qkv)
        q = torch.empty((T, self.heads, self.head_dim), dtype=rt.act_dtype, device=x.device)
        K.tag = "heads + cache write"
        K.head_prepare(qkv, 0, k_off, -1 if self.values_from_keys else v_off, q, entry.k_plane, entry.v_plane, ctx.positions,
                       ctx.row_req, entry.block_table, entry.page_tokens, self.heads, self.kv_heads, self.head_dim, self.value_dim,
                       pos.rotary_dim, pos.inv_freq, getattr(pos, "magnitude", 1.0), self.q_norm_w, self.k_norm_w,
                       float(self.qk_norm["eps"]) if self.qk_norm else 0.0, write)
        out = torch.empty((T, self.heads, self.value_dim), dtype=rt.act_dtype, device=x.device)
        K.tag = "attention"
        gate = qkv if gate_cols else None
        fast = rt.fast_kernels and self.value_dim == self.head_dim
        if fast and getattr(ctx, "all_single", False) and self.head_dim in (64, 128):
            # every request brings one token: the split-KV decode kernel
            K.decode_attention(q, out, entry.k_plane, entry.v_plane, ctx.positions, ctx.row_req, entry.block_table,
                               entry.page_tokens, self.heads, self.kv_heads, self.head_dim, self.window, self.scale,
                               ctx.max_context, getattr(ctx, "decode_scratch", None) or rt.decode_scratch,
                               softcap=self.softcap, head_gate=gate, gate_offset=g_off)
        elif fast and self.head_dim == 128 and entry.page_tokens == 16 and hasattr(ctx, "req_start"):
            # portions of prompts (and whatever single tokens ride along): both products on tcgen05
            K.prefill_attention_tc(q, out, entry.k_plane, entry.v_plane, ctx.req_start, ctx.req_prior, entry.block_table,
                                   entry.page_tokens, self.heads, self.kv_heads, self.head_dim, self.window, self.scale,
                                   softcap=self.softcap, head_gate=gate, gate_offset=g_off)
        elif fast and self.head_dim in (32, 64, 96, 128) and hasattr(ctx, "req_start"):
            # portions of prompts (and whatever single tokens ride along): query tiles on the tensor cores
            K.prefill_attention(q, out, entry.k_plane, entry.v_plane, ctx.req_start, ctx.req_prior, entry.block_table,
                                entry.page_tokens, self.heads, self.kv_heads, self.head_dim, self.window, self.scale,
                                softcap=self.softcap, head_gate=gate, gate_offset=g_off)
        else:
            K.paged_attention(q, out, entry.k_plane, entry.v_plane, ctx.positions, ctx.row_req, entry.block_table, entry.page_tokens,
                              self.heads, self.kv_heads, self.head_dim, self.window, self.scale, value_dim=self.value_dim,
                              softcap=self.softcap, head_gate=gate, gate_offset=g_off)
        K.tag = "o"
        parts = project_split(rt, out.view(T, self.o_dim), self.w_o) if self.allow_pending else None
        if parts is None:
            project(rt, out.view(T, self.o_dim), self.w_o, residual, accumulate=True)
        K.tag = None
        return parts

    def _tiled(self) -> bool:
        """Whether the mixed-heads attention runs in its tiled form (tensor cores, a cluster over the heads): bfloat16
        storage and sizes the form takes; float32 runs, and other sizes, take the row-at-a-time form."""
        rt = self.runtime
        return bool(rt.fast_kernels and rt.act_dtype == torch.bfloat16 and rt.cache_dtype == torch.bfloat16
                    and K.mixed_heads_tile_shape(self.heads, self.kv_heads, self.head_dim, self.value_dim))

    def _forward_mixed(self, x: torch.Tensor, residual: torch.Tensor, ctx, entry) -> None:
        """The path of a mixer whose projections are convolved over time, whose norm spans all heads, or whose heads'
        scores are scaled, mixed or joined by a sink: one product for q | k | v, the convolution with its state, heads made
        ready (norm, rotation, cache write), attention over all heads of a row at once, output projection."""
        rt = self.runtime
        T = x.shape[0]
        pos = self.position
        if not entry.writes_cache:
            raise ValueError("an attention mixer with mixed heads owns its cache (cache_from is not built for it)")
        k_off, v_off = self.q_dim, self.q_dim + self.kv_dim
        C = v_off + self.v_dim
        qkv = torch.empty((T, C), dtype=torch.float32, device=x.device)
        K.tag = "qkv"
        project(rt, x, self.w_qkv, qkv)
        if self.proj_conv:
            at = getattr(entry, "state_offset", 0)
            conv = torch.empty((T, C), dtype=torch.float32, device=x.device)
            K.tag = "short conv"
            K.short_conv(qkv, 0, C, self.taps, self.w_conv, None, entry.state, ctx.row_req, ctx.req_start, ctx.req_slot, conv,
                         activate=False, state_offset=at)
            K.short_conv_commit(qkv, 0, C, self.taps, entry.state, ctx.req_start, ctx.req_slot, ctx.n_requests, state_offset=at)
            qkv = conv
        q = torch.empty((T, self.heads, self.head_dim), dtype=rt.act_dtype, device=x.device)
        K.tag = "heads + cache write"
        K.head_prepare(qkv, 0, k_off, v_off, q, entry.k_plane, entry.v_plane, ctx.positions, ctx.row_req, entry.block_table,
                       entry.page_tokens, self.heads, self.kv_heads, self.head_dim, self.value_dim, pos.rotary_dim, pos.inv_freq,
                       getattr(pos, "magnitude", 1.0), self.q_norm_w, self.k_norm_w,
                       float(self.qk_norm["eps"]) if self.qk_norm else 0.0, True, norm_whole=self.norm_whole)
        out = torch.empty((T, self.heads, self.value_dim), dtype=rt.act_dtype, device=x.device)
        K.tag = "attention"
        K.mixed_heads_attention(q, out, entry.k_plane, entry.v_plane, ctx.positions, ctx.row_req, entry.block_table,
                                entry.page_tokens, self.heads, self.kv_heads, self.head_dim, self.value_dim, self.window,
                                self.scale, temp=self.temp_w, talk=self.talk_w, sink=self.sink_w,
                                req_start=ctx.req_start if self._tiled() else None, n_requests=ctx.n_requests)
        K.tag = "o"
        project(rt, out.view(T, self.o_dim), self.w_o, residual, accumulate=True)
        K.tag = None
        return None
