"""Attention over a compressed latent (one cache entry per token, shared by all heads).

Per row at position p, H heads with ``dim`` unrotated and ``rot_dim`` rotated query/key
entries, values of ``vdim``, latent of ``kv_rank``::

    q = W_q x                       each head: [dim plain entries | rot_dim entries to rotate]
    d = W_dkv x                     kv_rank + rot_dim rows
    c = rms(d[:kv_rank]) * w        the latent           } one cache entry
    r = rotate(d[kv_rank:], p)      the shared key part  } of kv_rank + rot_dim
    k_h = [W_uk[h] c | r] ,  v_h = W_uv[h] c
    score_h,j = (q_h[:dim] . W_uk[h] c_j + rotate(q_h[dim:], p) . r_j) * scale ,  j <= p
    out_h = sigmoid(W_g x)_h * sum_j softmax(score_h)_j v_h,j ;  then W_o on the heads
    (the gate is optional, and so are a latent of the queries' own and a sink in the softmax: see the parameters)

The rotation pairs entries (2i, 2i+1) of the first ``rotary_dim`` entries of the rotated
part (the position part's ``rotary_dim`` and ``inv_freq``).  Nothing per head is built from
the cache: ``W_uk[h]^T q`` is taken on the query's side and ``W_uv[h]`` applied to the
weighted sum of latents, so the attention kernel reads each cache entry once for all
heads.  Steps that carry long prompt portions on the bfloat16 path take the plain form
instead (``EXPAND_MIN_ROWS`` rows or more): keys ``[W_uk[h] c | r]`` and values ``W_uv[h] c`` of
the requests' tokens are built with two products over the gathered latents and a flash
kernel on the tensor cores runs over them - a (query, key, head) pair then costs
``2 (dim + rot_dim + vdim)`` flops instead of ``2 (2 kv_rank + rot_dim)``.  Such a step reads
the requests' lengths on the host, so it is not captured into a CUDA graph
(``capture_max_rows``).  An entry that reads another entry's cache (``entry.writes_cache`` false) has no
``W_dkv`` of its own: it attends over that entry's latents and key parts with its own
queries, ``W_uk`` and ``W_uv``.

Parameters: ``hidden_size``, ``heads``, ``dim``, ``rot_dim``, ``vdim``, ``kv_rank``,
``scale``, ``eps``, ``position`` (a position PartSpec), ``owns_cache`` (false: no ``dkv``
tensors).  Tensors: ``q``, ``g``, ``dkv``, ``dkv.norm``, ``uk``, ``uv``, ``o``.

Optional, each off by default:
``q_rank`` n > 0: the queries pass a latent of their own, ``c_q = rms(W_dq x) * w`` (``dq``, ``dq.norm``; the layer's
eps), ``q = W_uq c_q`` (``uq``), instead of one projection ``q``; ``W_dq`` rides in the mixer's one input product,
a kernel norms its columns, a second product brings the heads up;
``gate`` false: no sigmoid gate on the heads' outputs (no tensor ``g``);
``sink``: a tensor name, ``[heads]``: the softmax's divisor also holds ``exp(sink[h])``, a term without key or value
that is neither scaled nor rotated and counts once.
"""
from __future__ import annotations

from typing import Dict, Optional

import numpy as np
import torch

from ..csrc import kernels as K
from .base import KvNeed, Part, make_part, register_part
from .linear import project
from .plan import ParamSpec


@register_part("mixer", "latent_attention")
class LatentAttention(Part):
    EXPAND_MIN_ROWS = 256       # steps with at least this many rows (and prompt portions) take the plain form

    def __init__(self, spec, prefix, runtime):
        super().__init__(spec, prefix, runtime)
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["heads"])
        self.dim = int(spec["dim"])
        self.rot = int(spec["rot_dim"])
        self.vdim = int(spec["vdim"])
        self.rank = int(spec["kv_rank"])
        self.scale = float(spec["scale"])
        self.eps = float(spec["eps"])
        self.owns_cache = bool(spec.get("owns_cache", True))
        self.q_rank = int(spec.get("q_rank", 0) or 0)
        self.gate = bool(spec.get("gate", True))
        self.n_sink = self.name(str(spec["sink"])) if spec.get("sink") else None
        self.sink = self.w_qnorm = self.w_uq = None
        self.position = make_part("position", spec["position"], prefix, runtime)
        self.rotary = int(self.position.rotary_dim)
        if self.rotary > self.rot:
            raise ValueError(f"the position part rotates {self.rotary} entries; the rotated part has {self.rot}")
        if self.rank > 1024:
            raise ValueError(f"kv_rank {self.rank} is larger than the attention kernel takes (1024)")
        self.nq = self.heads * (self.dim + self.rot)
        self.w_in = self.w_norm = self.w_uk_t = self.w_uv = self.w_o = self.w_uk = None
        # the plain form's head sizes, padded to what its kernel is built for
        self.dk_pad = -(-(self.dim + self.rot) // 64) * 64
        self.dv_pad = -(-self.vdim // 64) * 64
        self.can_expand = runtime.fast_kernels and self.dk_pad <= 256 and self.dv_pad <= 128

    @property
    def capture_max_rows(self) -> int:
        """Steps with more rows than this are launched kernel by kernel: the plain form lays out the
        requests' tokens from their lengths on the host."""
        return self.EXPAND_MIN_ROWS - 1 if self.can_expand else 1 << 30

    def cache_need(self) -> Optional[KvNeed]:
        return KvNeed(1, self.rank + self.rot, 0, values=False)

    def state_need(self):
        return None

    def params(self) -> Dict[str, ParamSpec]:
        p = {
            self.name("uk"): ParamSpec((self.heads * self.dim, self.rank)),
            self.name("uv"): ParamSpec((self.heads * self.vdim, self.rank)),
            self.name("o"): ParamSpec((self.hidden, self.heads * self.vdim)),
        }
        if self.q_rank:
            p[self.name("dq")] = ParamSpec((self.q_rank, self.hidden))
            p[self.name("dq.norm")] = ParamSpec((self.q_rank,), role="vector", init="ones")
            p[self.name("uq")] = ParamSpec((self.nq, self.q_rank))
        else:
            p[self.name("q")] = ParamSpec((self.nq, self.hidden))
        if self.gate:
            p[self.name("g")] = ParamSpec((self.heads, self.hidden))
        if self.n_sink:
            p[self.n_sink] = ParamSpec((self.heads,), role="vector", std=1.0)
        if self.owns_cache:
            p[self.name("dkv")] = ParamSpec((self.rank + self.rot, self.hidden))
            p[self.name("dkv.norm")] = ParamSpec((self.rank,), role="vector", init="ones")
        return p

    def libraries(self) -> set:
        libs = {"latent_attention", "gemm_simt"} | ({"latent_prefill"} if self.can_expand else set())
        if self.runtime.fast_kernels and self.hidden >= 128:
            libs |= {"gemm_tc", "gemm_tc2"}
        return libs

    def load(self, source) -> None:
        # the mixer's input product: (q, or the queries' latent) | (g) | (dkv), in this order
        rows = [self.fetch(source, self.name("dq" if self.q_rank else "q"))]
        if self.q_rank:
            self.w_qnorm = self.fetch(source, self.name("dq.norm"))
            self.w_uq = self.fetch(source, self.name("uq"))
        if self.gate:
            rows.append(self.fetch(source, self.name("g")))
        if self.n_sink:
            self.sink = self.fetch(source, self.n_sink)
        if self.owns_cache:
            rows.append(self.fetch(source, self.name("dkv")))
            self.w_norm = self.fetch(source, self.name("dkv.norm"))
        self.w_in = torch.cat(rows, dim=0).contiguous()              # one product
        uk = self.fetch(source, self.name("uk"))
        # head h's W_uk^T as the weight of a product over dim: [heads, kv_rank, dim]
        self.w_uk_t = uk.view(self.heads, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_uk = uk if self.can_expand else None               # as stored: the plain form's product over kv_rank
        self.w_uv = self.fetch(source, self.name("uv")).view(self.heads, self.vdim, self.rank).contiguous()
        self.w_o = self.fetch(source, self.name("o"))

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, entry) -> None:
        rt = self.runtime
        dev = x.device
        T, H = x.shape[0], self.heads
        write = entry.writes_cache
        if write and not self.owns_cache:
            raise ValueError(f"{self.prefix}: the plan lets this entry write a cache, but the part has no W_dkv")
        n_q = self.q_rank or self.nq
        gate_off = n_q
        d_off = n_q + (H if self.gate else 0)
        n_out = d_off + ((self.rank + self.rot) if write else 0)
        proj = torch.empty((T, n_out), dtype=torch.float32, device=dev)
        K.tag = "mixer in"
        project(rt, x, self.w_in[:n_out], proj)
        q = proj                               # the heads' queries start at column 0 of this matrix
        if self.q_rank:
            cq = torch.empty((T, self.q_rank), dtype=rt.act_dtype, device=dev)
            K.tag = "q latent norm"
            K.latent_q_norm(proj, 0, self.q_rank, self.w_qnorm, self.eps, cq)
            q = torch.empty((T, self.nq), dtype=torch.float32, device=dev)
            K.tag = "q up"
            project(rt, cq, self.w_uq, q)
        gate = (proj, gate_off) if self.gate else (None, 0)
        inv_freq = self.position.inv_freq
        if write:
            K.tag = "latent norm + rope + cache write"
            K.latent_kv_write(proj, d_off, self.rank, self.rot, self.rotary, self.w_norm, self.eps, inv_freq,
                              ctx.positions, ctx.row_req, entry.block_table, entry.page_tokens, entry.k_plane)
        if self.can_expand and T >= self.EXPAND_MIN_ROWS and not ctx.all_single and len(ctx.h_req_prior) > 0:
            gated = self._plain_form(q, gate, ctx, entry)
        else:
            gated = self._absorbed_form(q, gate, ctx, entry)
        K.tag = "o"
        project(rt, gated, self.w_o, residual, accumulate=True)
        K.tag = None
        return None

    def _absorbed_form(self, proj: torch.Tensor, gate, ctx, entry) -> torch.Tensor:
        """``proj``: float32 rows whose first ``heads * (dim + rot_dim)`` columns are the queries; ``gate``: (matrix, column)
        of the heads' gate values, or (None, 0)."""
        rt = self.runtime
        dev = proj.device
        T, H = proj.shape[0], self.heads
        inv_freq = self.position.inv_freq
        q_plain = torch.empty((H * T, self.dim), dtype=rt.act_dtype, device=dev)
        q_rot = torch.empty((T, H, self.rot), dtype=torch.float32, device=dev)
        K.tag = "q split + rope"
        K.latent_q_split(proj, H, self.dim, self.rot, self.rotary, inv_freq, ctx.positions, q_plain, q_rot)
        # rows are head-major: group h of the grouped products is head h's T rows
        offsets = torch.arange(0, (H + 1) * T, T, dtype=torch.int32, device=dev)
        q_abs = torch.empty((H * T, self.rank), dtype=torch.float32, device=dev)
        K.tag = "q absorb"
        project(rt, q_plain, self.w_uk_t, q_abs, group_offsets=offsets, max_group_rows=T)
        lat = torch.empty((H * T, self.rank), dtype=rt.cache_dtype, device=dev)
        K.tag = "attention"
        # How far a row's keys can reach, as a number that a captured step may keep: a decode step's
        # context (its graph is keyed by the context's bucket), otherwise what the block table spans
        # (laid out at its full width in steps that are captured).  It only decides into how many
        # stretches a row's keys are cut when the step has few rows.
        reach = ctx.max_context if ctx.all_single else entry.block_table.shape[1] * entry.page_tokens
        K.latent_attention(q_abs, q_rot, entry.k_plane, self.rank, self.rot, H, ctx.positions, ctx.row_req, entry.block_table,
                           entry.page_tokens, self.scale, lat, max_context=reach, sink=self.sink)
        o = torch.empty((H * T, self.vdim), dtype=torch.float32, device=dev)
        K.tag = "value up"
        project(rt, lat, self.w_uv, o, group_offsets=offsets, max_group_rows=T, offsets_settled=True)
        gated = torch.empty((T, H * self.vdim), dtype=rt.act_dtype, device=dev)
        K.tag = "head gate" if gate[0] is not None else "heads out"
        K.latent_gate_out(o, gate[0], gate[1], H, self.vdim, gated)
        return gated

    def _plain_form(self, proj: torch.Tensor, gate, ctx, entry) -> torch.Tensor:
        rt = self.runtime
        dev = proj.device
        T, H = proj.shape[0], self.heads
        layout = getattr(ctx, "_latent_tokens", None)
        if layout is None:
            # every token of the step's requests, cached and new, request after request (shared by the step's layers)
            totals = [p + (ctx.h_req_start[i + 1] - ctx.h_req_start[i]) for i, p in enumerate(ctx.h_req_prior)]
            base = np.zeros(ctx.n_requests, dtype=np.int32)
            base[:len(totals)] = np.concatenate([[0], np.cumsum(totals)[:-1]])
            tok_req = np.repeat(np.arange(len(totals), dtype=np.int32), totals)
            tok_pos = np.concatenate([np.arange(t, dtype=np.int32) for t in totals])
            host = torch.from_numpy(np.concatenate([base, tok_req, tok_pos]).astype(np.int32))
            d = host.to(dev, non_blocking=False)
            R, N = ctx.n_requests, int(tok_req.size)
            layout = ctx._latent_tokens = (d[:R], d[R:R + N], d[R + N:], N)
        req_base, tok_req, tok_pos, N = layout
        plane = entry.k_plane
        c_all = torch.empty((N, self.rank), dtype=torch.bfloat16, device=dev)
        K.tag = "latent gather"
        K.latent_gather(plane, self.rank, tok_req, tok_pos, entry.block_table, entry.page_tokens, c_all)
        kp = torch.empty((N, H * self.dim), dtype=torch.bfloat16, device=dev)
        vp = torch.empty((N, H * self.vdim), dtype=torch.bfloat16, device=dev)
        K.tag = "key/value up"
        project(rt, c_all, self.w_uk, kp)
        project(rt, c_all, self.w_uv.view(H * self.vdim, self.rank), vp)
        kx = torch.empty((N, H, self.dk_pad), dtype=torch.bfloat16, device=dev)
        vx = torch.empty((N, H, self.dv_pad), dtype=torch.bfloat16, device=dev)
        K.tag = "key/value pack"
        K.latent_kv_pack(kp, vp, plane, self.rank, self.rot, tok_req, tok_pos, entry.block_table, entry.page_tokens, H, self.dim,
                         self.vdim, kx, vx)
        qx = torch.empty((T, H, self.dk_pad), dtype=torch.bfloat16, device=dev)
        K.tag = "q split + rope"
        K.latent_q_pack(proj, H, self.dim, self.rot, self.rotary, self.position.inv_freq, ctx.positions, qx)
        ox = torch.empty((T, H, self.dv_pad), dtype=torch.bfloat16, device=dev)
        K.tag = "attention"
        K.latent_flash(qx, ox, kx, vx, ctx.req_start, ctx.req_prior, req_base, ctx.n_requests, H, self.scale, sink=self.sink)
        gated = torch.empty((T, H * self.vdim), dtype=torch.bfloat16, device=dev)
        K.tag = "head gate" if gate[0] is not None else "heads out"
        K.latent_gate_rows(ox, gate[0], gate[1], H, self.vdim, gated)
        return gated
