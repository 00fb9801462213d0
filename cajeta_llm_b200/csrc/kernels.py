"""Python face of the CUDA kernels: checks tensors, passes raw pointers through ctypes.

Every function launches on torch's current CUDA stream and raises
:class:`KernelError` when a kernel refuses its arguments or the launch fails.  There is
no fallback: without a CUDA device and the built libraries these functions raise.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional

import torch

from . import build as _build

CJ_F32, CJ_BF16 = 0, 1
_REFUSALS = {-2: "dtype combination not built into this kernel", -3: "a size this kernel does not take",
             -4: "pointer or stride alignment this kernel needs", -5: "null pointer or bad count"}


class KernelError(RuntimeError):
    pass


_libs: Dict[str, ctypes.CDLL] = {}


_launch_overlap = True     # whether kernels may be set up beside the one before them in the stream (see set_launch_overlap)


def library(name: str) -> ctypes.CDLL:
    """The loaded kernel library ``name`` (built first when it has to be)."""
    lib = _libs.get(name)
    if lib is None:
        path = _build.build(name)
        lib = ctypes.CDLL(path)
        _libs[name] = lib
        if not _launch_overlap and hasattr(lib, "cj_set_launch_overlap"):
            lib.cj_set_launch_overlap(_i(0))
    return lib


def set_launch_overlap(on: bool) -> None:
    """Whether a kernel may be set up on the SMs while the one before it in the stream is still draining (programmatic
    dependent launch, the default) or every kernel starts when the one before has ended (plain stream order).  For all
    libraries, those loaded later too; steps captured into CUDA graphs keep what held when they were captured."""
    global _launch_overlap
    _launch_overlap = bool(on)
    for lib in _libs.values():
        if hasattr(lib, "cj_set_launch_overlap"):
            lib.cj_set_launch_overlap(_i(1 if on else 0))


def loaded_libraries() -> Dict[str, str]:
    return {n: l._name for n, l in _libs.items()}


def _code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return CJ_F32
    if t.dtype == torch.bfloat16:
        return CJ_BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, found {t.dtype}")


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    if t is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(t.data_ptr())


# torch's current stream as a raw handle.  torch.cuda.current_stream() builds a Stream object
# through several layers of Python on every call - a third of the host's time in a step of a few
# hundred launches; the raw getter beneath it costs a fraction of a microsecond.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> ctypes.c_void_p:
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


launches = 0      # kernels launched through this module since import (each wrapper launches one)
# Measurement: parts name the class of work their next launches belong to (``tag``: "qkv", "expert
# gate/up", ...; costs an assignment); while a trace is open every launch is followed by an event
# on the stream, so that the time between two events is one launch's device time with the launches
# serialised (an event between two kernels keeps them from overlapping).
tag: Optional[str] = None
_trace: Optional[list] = None


def start_trace() -> None:
    global _trace
    _trace = []


def stop_trace() -> list:
    """[(class of work, event recorded after the launch)] since ``start_trace``."""
    global _trace
    out, _trace = _trace or [], None
    return out


_router_tickets: Dict[torch.device, torch.Tensor] = {}      # arrival tickets of the small-batch router (kept zero by the kernel)


def _check(status: int, what: str) -> None:
    global launches
    if status == 0:
        launches += 1
        if _trace is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            _trace.append((tag or what, ev))
        return
    if status in _REFUSALS:
        raise KernelError(f"{what}: refused: {_REFUSALS[status]}")
    raise KernelError(f"{what}: CUDA error {status} at launch")


def _need(t: torch.Tensor, name: str, dtype: Optional[torch.dtype] = None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor; this engine has no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, found {t.dtype}")


_i = ctypes.c_int
_ll = ctypes.c_longlong
_f = ctypes.c_float


def embed_gather(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, scale: float = 0.0) -> None:
    """out[t, :] = table[ids[t], :] widened to float32 (times ``scale`` unless that is 0).  out: [T, H] float32."""
    _need(out, "out", torch.float32), _need(table, "table"), _need(ids, "ids", torch.int32)
    T, H = out.shape
    V = table.shape[0]
    st = library("rowwise").cj_embed_gather(_ptr(out), _ptr(table), _i(_code(table)), _ptr(ids), _i(T), _i(H), _i(V), _f(scale),
                                            _stream())
    _check(st, "embed_gather")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            out_f32: Optional[torch.Tensor] = None, row_index: Optional[torch.Tensor] = None,
            partials: Optional[torch.Tensor] = None, out_split: Optional[torch.Tensor] = None) -> None:
    """out[r] = rmsnorm(x[row_index[r] or r]) * weight; x, weight float32; out float32 or
    bfloat16; out_f32 an optional float32 copy of the result.  ``partials`` ([S, rows, H]
    float32): x[r] += sum_s partials[s, r] first, and x keeps the sum.  ``out_split``
    (bfloat16 [rows, 3H]): the float32 result as three bfloat16 terms hi | mid | lo."""
    _need(x, "x", torch.float32), _need(weight, "weight", torch.float32), _need(out, "out")
    rows, H = out.shape
    if x.shape[-1] != H or weight.numel() != H:
        raise KernelError(f"rmsnorm: width mismatch x {tuple(x.shape)} weight {tuple(weight.shape)} out {tuple(out.shape)}")
    if out_f32 is not None:
        _need(out_f32, "out_f32", torch.float32)
    if row_index is not None:
        _need(row_index, "row_index", torch.int32)
    if out_split is not None:
        _need(out_split, "out_split", torch.bfloat16)
        if tuple(out_split.shape) != (rows, 3 * H):
            raise KernelError(f"rmsnorm: out_split {tuple(out_split.shape)} is not [{rows}, {3 * H}]")
    n_part, part_stride = 0, 0
    if partials is not None:
        _need(partials, "partials", torch.float32)
        if partials.dim() != 3 or partials.shape[1] != rows or partials.shape[2] != H or row_index is not None:
            raise KernelError(f"rmsnorm: partials {tuple(partials.shape)} do not fit {rows} rows of {H}")
        n_part, part_stride = partials.shape[0], partials.stride(0)
    st = library("rowwise").cj_rmsnorm(_ptr(x), _ptr(weight), _f(eps), _i(rows), _i(H), _ptr(out), _i(_code(out)),
                                       _ptr(out_f32), _ptr(out_split), _ptr(row_index), _ptr(partials), _i(n_part),
                                       _ll(part_stride), _stream())
    _check(st, "rmsnorm")


def dyt(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, alpha: float, out: torch.Tensor,
        out_f32: Optional[torch.Tensor] = None, row_index: Optional[torch.Tensor] = None,
        partials: Optional[torch.Tensor] = None, out_split: Optional[torch.Tensor] = None) -> None:
    """out[r] = tanh(alpha x[row_index[r] or r]) * weight + bias: the norm without statistics.  x, weight, bias float32;
    out float32 or bfloat16; ``out_f32``, ``partials`` and ``out_split`` as for :func:`rmsnorm`."""
    _need(x, "x", torch.float32), _need(weight, "weight", torch.float32), _need(bias, "bias", torch.float32), _need(out, "out")
    rows, H = out.shape
    if x.shape[-1] != H or weight.numel() != H or bias.numel() != H:
        raise KernelError(f"dyt: width mismatch x {tuple(x.shape)} weight {tuple(weight.shape)} bias {tuple(bias.shape)} out {tuple(out.shape)}")
    if out_f32 is not None:
        _need(out_f32, "out_f32", torch.float32)
    if row_index is not None:
        _need(row_index, "row_index", torch.int32)
    if out_split is not None:
        _need(out_split, "out_split", torch.bfloat16)
        if tuple(out_split.shape) != (rows, 3 * H):
            raise KernelError(f"dyt: out_split {tuple(out_split.shape)} is not [{rows}, {3 * H}]")
    n_part, part_stride = 0, 0
    if partials is not None:
        _need(partials, "partials", torch.float32)
        if partials.dim() != 3 or partials.shape[1] != rows or partials.shape[2] != H or row_index is not None:
            raise KernelError(f"dyt: partials {tuple(partials.shape)} do not fit {rows} rows of {H}")
        n_part, part_stride = partials.shape[0], partials.stride(0)
    st = library("rowwise").cj_dyt(_ptr(x), _ptr(weight), _ptr(bias), _f(alpha), _i(rows), _i(H), _ptr(out), _i(_code(out)),
                                   _ptr(out_f32), _ptr(out_split), _ptr(row_index), _ptr(partials), _i(n_part), _ll(part_stride),
                                   _stream())
    _check(st, "dyt")


def dyt_add(hs: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, alpha: float) -> None:
    """hs[r] += tanh(alpha y[r]) * weight + bias; everything float32."""
    _need(hs, "hs", torch.float32), _need(y, "y", torch.float32), _need(weight, "weight", torch.float32), _need(bias, "bias", torch.float32)
    rows, H = hs.shape
    if y.shape != hs.shape or weight.numel() != H or bias.numel() != H:
        raise KernelError(f"dyt_add: shapes hs {tuple(hs.shape)} y {tuple(y.shape)} weight {tuple(weight.shape)} do not agree")
    _check(library("rowwise").cj_dyt_add(_ptr(hs), _ptr(y), _ptr(weight), _ptr(bias), _f(alpha), _i(rows), _i(H), _stream()), "dyt_add")


def gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
         accumulate: bool = False, w_up: Optional[torch.Tensor] = None, group_offsets: Optional[torch.Tensor] = None,
         a_row_index: Optional[torch.Tensor] = None, rows: Optional[int] = None, act_limit: float = 0.0,
         act_alpha: float = 1.0) -> None:
    """out[M, N] (+)= a[M, K] . w[N, K]^T (+ bias) on the float32 FMA pipe.

    ``w_up`` selects the gated form: silu(a.w^T) * (a.w_up^T), or with ``act_limit`` > 0 the capped one,
    g = min(a.w^T, limit), u = clamp(a.w_up^T, +-limit), g * sigmoid(act_alpha g) * (u + 1).  With ``group_offsets``
    ([G + 1] int32) ``w`` is [G, N, K], output row s belongs to the group whose range
    holds s, and ``a_row_index[s]`` names the row of ``a`` that feeds it.
    """
    _need(w, "w"), _need(out, "out")
    if not a.is_cuda or a.dim() != 2 or a.stride(1) != 1:
        raise KernelError("gemm: a must be a CUDA matrix whose rows are contiguous (a column slice of a wider one is fine)")
    grouped = group_offsets is not None
    N, K = w.shape[-2], w.shape[-1]
    M = rows if rows is not None else out.shape[0]
    if a.shape[-1] != K or out.shape[-1] != N:
        raise KernelError(f"gemm: shapes a {tuple(a.shape)} w {tuple(w.shape)} out {tuple(out.shape)} do not agree")
    if w_up is not None:
        _need(w_up, "w_up")
        if w_up.shape != w.shape or w_up.dtype != w.dtype:
            raise KernelError("gemm: w_up must match w")
    if bias is not None:
        _need(bias, "bias", torch.float32)
    G = 0
    if grouped:
        _need(group_offsets, "group_offsets", torch.int32)
        G = w.shape[0]
        if group_offsets.numel() != G + 1:
            raise KernelError("gemm: group_offsets must hold one more entry than w has groups")
    if a_row_index is not None:
        _need(a_row_index, "a_row_index", torch.int32)
    st = library("gemm_simt").cj_gemm_simt(
        _ptr(a), _ll(a.stride(0)), _i(_code(a)), _ptr(w), _ptr(w_up), _ll(K), _i(_code(w)), _ptr(bias),
        _ptr(out), _ll(out.stride(0)), _i(_code(out)), _i(M), _i(N), _i(K), _i(1 if accumulate else 0),
        _ptr(group_offsets), _i(G), _ll(N * K), _ptr(a_row_index), _f(act_limit), _f(act_alpha), _stream())
    _check(st, "gemm")


def rope_kv_write(qkv: torch.Tensor, q_off: int, k_off: int, v_off: int, q_out: torch.Tensor,
                  k_plane: Optional[torch.Tensor], v_plane: Optional[torch.Tensor], positions: torch.Tensor,
                  row_req: Optional[torch.Tensor], table: Optional[torch.Tensor], page_tokens: int, n_heads: int,
                  n_kv: int, head_dim: int, rotary_dim: int, inv_freq: Optional[torch.Tensor], write_kv: bool) -> None:
    """Rotate q and k at each row's position; write q to q_out, rotated k and raw v into
    the cache pages of the row's request.  qkv: float32 [T, ld]."""
    _need(qkv, "qkv", torch.float32), _need(q_out, "q_out"), _need(positions, "positions", torch.int32)
    T = qkv.shape[0]
    cache_dtype = _code(q_out)
    if write_kv:
        _need(k_plane, "k_plane"), _need(v_plane, "v_plane"), _need(row_req, "row_req", torch.int32), _need(table, "table", torch.int32)
        cache_dtype = _code(k_plane)
    st = library("rowwise").cj_rope_kv_write(
        _ptr(qkv), _i(qkv.stride(0)), _i(q_off), _i(k_off), _i(v_off), _ptr(q_out), _i(_code(q_out)),
        _ptr(k_plane), _ptr(v_plane), _i(cache_dtype), _ptr(positions), _ptr(row_req), _ptr(table),
        _i(table.stride(0) if table is not None else 0), _i(page_tokens), _i(T), _i(n_heads), _i(n_kv), _i(head_dim),
        _i(rotary_dim), _ptr(inv_freq), _i(1 if write_kv else 0), _stream())
    _check(st, "rope_kv_write")


def head_prepare(x: torch.Tensor, q_off: int, k_off: int, v_off: int, q_out: torch.Tensor, k_plane: Optional[torch.Tensor],
                 v_plane: Optional[torch.Tensor], positions: torch.Tensor, row_req: Optional[torch.Tensor],
                 table: Optional[torch.Tensor], page_tokens: int, n_heads: int, n_kv: int, head_dim: int, value_dim: int,
                 rotary_dim: int, inv_freq: Optional[torch.Tensor], magnitude: float, q_norm: Optional[torch.Tensor],
                 k_norm: Optional[torch.Tensor], eps: float, write_kv: bool, norm_whole: bool = False,
                 q_temp_coef: float = 0.0, q_temp_every: int = 1) -> None:
    """Queries, keys and values of a step's rows (x float32 [T, ld], columns from q_off, k_off, v_off) made ready
    for attention: an RMS norm over each head of q and k (when ``q_norm`` / ``k_norm``, float32 [head_dim], are
    given), the rotation of their first ``rotary_dim`` entries (entry i with i + rotary_dim / 2; cos and sin times
    ``magnitude``), q to ``q_out``, k and v into the cache pages of the row's request.  ``v_off`` < 0: the
    values are the keys as projected, before norm and rotation.  ``norm_whole``: one statistic over all heads of q
    (of k) at once, and weights of ``n_heads * head_dim`` (``n_kv * head_dim``) entries.  ``q_temp_coef`` != 0: the
    queries are multiplied by ``1 + q_temp_coef * ln(floor((p + 1) / q_temp_every) + 1)`` at position p."""
    _need(x, "x", torch.float32), _need(q_out, "q_out"), _need(positions, "positions", torch.int32)
    cache_dtype = _code(q_out)
    if write_kv:
        _need(k_plane, "k_plane"), _need(v_plane, "v_plane"), _need(row_req, "row_req", torch.int32), _need(table, "table", torch.int32)
        cache_dtype = _code(k_plane)
        if k_plane.shape[-1] != head_dim or v_plane.shape[-1] != value_dim:
            raise KernelError("head_prepare: the cache planes do not have the heads' sizes")
    for n, t in (("q_norm", q_norm), ("k_norm", k_norm), ("inv_freq", inv_freq)):
        if t is not None:
            _need(t, n, torch.float32)
    if norm_whole and ((q_norm is not None and q_norm.numel() != n_heads * head_dim) or (k_norm is not None and k_norm.numel() != n_kv * head_dim)):
        raise KernelError("head_prepare: a norm over the whole projection takes weights of heads * head_dim entries")
    st = library("attention_paged").cj_head_prepare(
        _ptr(x), _i(x.stride(0)), _i(q_off), _i(k_off), _i(v_off), _ptr(q_out), _i(_code(q_out)), _ptr(k_plane), _ptr(v_plane),
        _i(cache_dtype), _ptr(positions), _ptr(row_req), _ptr(table), _i(table.stride(0) if table is not None else 0),
        _i(page_tokens), _i(x.shape[0]), _i(n_heads), _i(n_kv), _i(head_dim), _i(value_dim), _i(rotary_dim), _ptr(inv_freq),
        _f(magnitude), _ptr(q_norm), _ptr(k_norm), _f(eps), _i(1 if write_kv else 0), _i(1 if norm_whole else 0),
        _f(q_temp_coef), _i(q_temp_every), _stream())
    _check(st, "head_prepare")


def _gate(head_gate: Optional[torch.Tensor], gate_offset: int):
    """Pointer to column ``gate_offset`` of a float32 [T, ld] tensor of per-head gate values, and ld."""
    if head_gate is None:
        return ctypes.c_void_p(0), 0
    _need(head_gate, "head_gate", torch.float32)
    return ctypes.c_void_p(head_gate.data_ptr() + 4 * gate_offset), head_gate.stride(0)


def paged_attention(q: torch.Tensor, out: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor,
                    positions: torch.Tensor, row_req: torch.Tensor, table: torch.Tensor, page_tokens: int,
                    n_heads: int, n_kv: int, head_dim: int, window: int, scale: float, value_dim: int = 0,
                    softcap: float = 0.0, head_gate: Optional[torch.Tensor] = None, gate_offset: int = 0) -> None:
    """Attention of every row over its request's cached keys [from, position].  ``value_dim``: the values'
    size when it is not the keys'; ``softcap`` > 0: s <- cap tanh(s / cap); ``head_gate`` (float32 [T, ld]):
    head h of row t is multiplied by sigmoid(head_gate[t, gate_offset + h])."""
    _need(q, "q"), _need(out, "out"), _need(k_plane, "k_plane"), _need(v_plane, "v_plane")
    _need(positions, "positions", torch.int32), _need(row_req, "row_req", torch.int32), _need(table, "table", torch.int32)
    T = q.shape[0]
    if head_dim > 256:
        raise KernelError(f"paged_attention: head_dim {head_dim} is larger than 256")
    gate_ptr, gate_ld = _gate(head_gate, gate_offset)
    st = library("attention_paged").cj_paged_attention(
        _ptr(q), _ptr(out), _i(_code(q)), _ptr(k_plane), _ptr(v_plane), _i(_code(k_plane)), _ptr(positions),
        _ptr(row_req), _ptr(table), _i(table.stride(0)), _i(page_tokens), _i(T), _i(n_heads), _i(n_kv), _i(head_dim),
        _i(value_dim or head_dim), _i(window), _f(scale), _f(softcap), gate_ptr, _i(gate_ld), _stream())
    _check(st, "paged_attention")


def diff_tile_shape(head_dim: int, value_dim: int) -> bool:
    """Whether the tiled form of differential attention takes these sizes (one map's query / key size, the values')."""
    return head_dim in (32, 64, 128) and value_dim in (64, 128)


def diff_attention(q: torch.Tensor, out: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor, positions: torch.Tensor,
                   row_req: torch.Tensor, table: torch.Tensor, page_tokens: int, n_heads: int, n_kv: int, head_dim: int,
                   value_dim: int, window: int, scale: float, lam: float, eps: float, out_scale: float,
                   req_start: Optional[torch.Tensor] = None, req_prior: Optional[torch.Tensor] = None, n_requests: int = 0,
                   reach: int = 0, splits: Optional[int] = None, tile_rows: int = 64) -> None:
    """Differential attention of every row over its request's cached keys [from, position]: a query head is
    [q1 | q2] (``head_dim`` entries each), a cached key [k1 | k2]; each map is a softmax attention of its own over the
    same values, ``o = a1 - lam a2``, then ``o / sqrt(mean(o^2) + eps) * out_scale`` over the head's ``value_dim`` entries.
    q [T, n_heads, 2 head_dim], out [T, n_heads, value_dim].
    With ``req_start`` / ``req_prior`` (int32; request i owns rows [req_start[i], req_start[i + 1]) at positions
    req_prior[i] + j), bfloat16 storage and sizes that :func:`diff_tile_shape` takes, the rows run in the tiled form: 64
    rows of a request and a head a block, the products on tensor cores.  ``reach``: a bound on the longest row's keys that
    the step's shape fixes; with few row blocks their keys are dealt to several blocks in stretches cut from it
    (``splits``: how many, instead of as many as fill the machine).  ``tile_rows``: 64, or 16 when no request of the step brings
    more than 16 rows (single decoded tokens): blocks of two warps, three of them a SM."""
    _need(q, "q"), _need(out, "out", q.dtype), _need(k_plane, "k_plane"), _need(v_plane, "v_plane", k_plane.dtype)
    _need(positions, "positions", torch.int32), _need(row_req, "row_req", torch.int32), _need(table, "table", torch.int32)
    T = q.shape[0]
    if q.numel() != T * n_heads * 2 * head_dim or out.numel() != T * n_heads * value_dim:
        raise KernelError("diff_attention: q or out does not have the heads' sizes")
    if k_plane.shape[-1] != 2 * head_dim or v_plane.shape[-1] != value_dim:
        raise KernelError("diff_attention: the cache planes do not have the heads' sizes")
    if (req_start is not None and req_prior is not None and n_requests > 0 and q.dtype == torch.bfloat16
            and k_plane.dtype == torch.bfloat16 and diff_tile_shape(head_dim, value_dim)):
        _need(req_start, "req_start", torch.int32), _need(req_prior, "req_prior", torch.int32)
        if tile_rows not in (16, 64):
            raise KernelError(f"diff_attention: tile_rows must be 16 or 64, found {tile_rows}")
        blocks = (-(-T // tile_rows) + n_requests) * n_heads
        fill = _sm_count() * (3 if tile_rows == 16 else 1)            # blocks that fill the machine
        if splits is None:
            splits = min(32, -(-fill // blocks)) if blocks < fill else 1
        split_keys, partial = 0, None
        if splits > 1 and reach > 128:
            split_keys = max(128, -(-(-(-reach // splits)) // 64) * 64)
            splits = -(-reach // split_keys)
        if splits > 1 and split_keys > 0:
            partial = torch.empty((splits, T, n_heads, 2, value_dim + 2), dtype=torch.float32, device=q.device)
        else:
            split_keys, splits = 0, 1
        st = library("attention_diff").cj_diff_attention_tile(
            _ptr(q), _ptr(out), _ptr(k_plane), _ptr(v_plane), _ptr(positions), _ptr(req_start), _ptr(req_prior), _i(n_requests), _i(T),
            _ptr(table), _i(table.stride(0)), _i(page_tokens), _i(n_heads), _i(n_kv), _i(head_dim), _i(value_dim), _i(window),
            _f(scale), _f(lam), _f(eps), _f(out_scale), _i(split_keys), _i(splits), _ptr(partial), _i(tile_rows), _stream())
        _check(st, "diff_attention (tiled)")
        if split_keys:
            global launches
            launches += 1                  # the merge is a kernel of its own
        return
    st = library("attention_diff").cj_diff_attention(
        _ptr(q), _ptr(out), _i(_code(q)), _ptr(k_plane), _ptr(v_plane), _i(_code(k_plane)), _ptr(positions), _ptr(row_req),
        _ptr(table), _i(table.stride(0)), _i(page_tokens), _i(T), _i(n_heads), _i(n_kv), _i(head_dim), _i(value_dim), _i(window),
        _f(scale), _f(lam), _f(eps), _f(out_scale), _stream())
    _check(st, "diff_attention")


_sms: Dict[int, int] = {}


def _sm_count() -> int:
    d = torch.cuda.current_device()
    if d not in _sms:
        _sms[d] = int(torch.cuda.get_device_properties(d).multi_processor_count)
    return _sms[d]


def mixed_heads_tile_shape(n_heads: int, n_kv: int, head_dim: int, value_dim: int) -> bool:
    """Whether the tiled form of the mixed-heads attention takes these sizes: head and value sizes multiples of 8 up
    to 128, and heads that 1, 2, 4 or 8 blocks share out evenly, at most 8 a block.  A matter of arithmetic: the
    library is not asked."""
    if n_heads <= 0 or n_kv <= 0 or n_heads % n_kv or head_dim <= 0 or value_dim <= 0:
        return False
    if head_dim % 8 or value_dim % 8 or head_dim > 128 or value_dim > 128:
        return False
    for c in (1, 2, 4, 8):
        if n_heads % c == 0 and n_heads // c <= 8:
            hl, per = n_heads // c, n_heads // n_kv
            kv = max((r * hl + hl - 1) // per - (r * hl) // per + 1 for r in range(c))
            hdp = (head_dim + 15) // 16 * 16
            return (2 * hl * 16 * 40 * 4 + n_heads * 32 + (hl * 16 + kv * 32) * (hdp + 8) * 2 + kv * 32 * (value_dim + 8) * 2) <= 200 * 1024
    return False


def mixed_heads_attention(q: torch.Tensor, out: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor,
                          positions: torch.Tensor, row_req: torch.Tensor, table: torch.Tensor, page_tokens: int,
                          n_heads: int, n_kv: int, head_dim: int, value_dim: int, window: int, scale: float,
                          temp: Optional[torch.Tensor] = None, talk: Optional[torch.Tensor] = None,
                          sink: Optional[torch.Tensor] = None, req_start: Optional[torch.Tensor] = None,
                          n_requests: int = 0, cluster_blocks: int = 0, splits: Optional[int] = None) -> None:
    """Attention of every row over its request's cached keys [from, position] in which the heads' scores are mixed
    before the softmax: raw_g = (q_g . k) scale temp[g]; s_h = sum_g talk[h, g] raw_g; the softmax's divisor also
    holds exp(sink[h]).  ``temp`` [heads], ``talk`` [heads, heads], ``sink`` [heads]: float32, each optional.
    With ``req_start`` (int32 ``[n_requests + 1]``, the first row of each request; a request's rows at consecutive
    positions) and sizes that ``mixed_heads_tile_shape`` takes, bfloat16 rows run in the tiled form: 16 rows of a
    request and all heads on a cluster of blocks, the products on tensor cores."""
    _need(q, "q"), _need(out, "out"), _need(k_plane, "k_plane"), _need(v_plane, "v_plane")
    _need(positions, "positions", torch.int32), _need(row_req, "row_req", torch.int32), _need(table, "table", torch.int32)
    for n, t, size in (("temp", temp, n_heads), ("talk", talk, n_heads * n_heads), ("sink", sink, n_heads)):
        if t is not None:
            _need(t, n, torch.float32)
            if t.numel() != size:
                raise KernelError(f"mixed_heads_attention: {n} must hold {size} entries, found {t.numel()}")
    if (req_start is not None and n_requests > 0 and q.dtype == torch.bfloat16 and k_plane.dtype == torch.bfloat16
            and mixed_heads_tile_shape(n_heads, n_kv, head_dim, value_dim or head_dim)):
        _need(req_start, "req_start", torch.int32)
        vd = value_dim or head_dim
        T = q.shape[0]
        # few tiles (single decoded tokens, a short portion): a tile's chunks of keys are dealt to several clusters, as many
        # as still find room on the SMs at once (two blocks a SM), and put together by a second kernel
        tiles = (T + 15) // 16 + n_requests
        c = next(c for c in (1, 2, 4, 8) if n_heads % c == 0 and n_heads // c <= 8)
        if splits is None:
            splits = max(1, min(8, (2 * _sm_count()) // (tiles * max(c, cluster_blocks))))
            if window > 0:
                splits = min(splits, max(1, (window + 46) // 64))      # at least two chunks of 32 keys a share
        partial = torch.empty((splits, T, n_heads, vd + 2), dtype=torch.float32, device=q.device) if splits > 1 else None
        st = library("attention_mixed").cj_mixed_heads_attention_tile(
            _ptr(q), _ptr(out), _ptr(k_plane), _ptr(v_plane), _ptr(positions), _ptr(req_start), _i(n_requests), _i(T),
            _ptr(table), _i(table.stride(0)), _i(page_tokens), _i(n_heads), _i(n_kv), _i(head_dim), _i(vd),
            _i(window), _f(scale), _ptr(temp), _ptr(talk), _ptr(sink), _i(cluster_blocks), _ptr(partial), _i(splits), _stream())
        _check(st, "mixed_heads_attention (tiled)")
        return
    st = library("attention_paged").cj_mixed_heads_attention(
        _ptr(q), _ptr(out), _i(_code(q)), _ptr(k_plane), _ptr(v_plane), _i(_code(k_plane)), _ptr(positions),
        _ptr(row_req), _ptr(table), _i(table.stride(0)), _i(page_tokens), _i(q.shape[0]), _i(n_heads), _i(n_kv), _i(head_dim),
        _i(value_dim or head_dim), _i(window), _f(scale), _ptr(temp), _ptr(talk), _ptr(sink), _stream())
    _check(st, "mixed_heads_attention")


def _route_mode(norm_topk: bool, sigmoid_scores: bool, groups) -> int:
    """The selection's mode word: bit 0 renormalise the picked scores, bit 1 sigmoid scores, bits 4-15 the
    number of expert groups and bits 16-27 how many of them stay eligible (``groups`` = (count, keep))."""
    mode = (1 if norm_topk else 0) | (2 if sigmoid_scores else 0)
    if groups is not None and int(groups[0]) > 1:
        count, keep = int(groups[0]), int(groups[1])
        if not (1 <= keep <= count <= 0xfff):
            raise KernelError(f"router: {keep} of {count} expert groups cannot be kept")
        mode |= (count << 4) | (keep << 16)
    return mode


def _pin_and_gap(pin: Optional[torch.Tensor], gap: Optional[torch.Tensor], T: int, top_k: int) -> None:
    if pin is not None:
        _need(pin, "pin", torch.int32)
        if pin.numel() != T * top_k or gap is not None:
            raise KernelError(f"router: pin must hold {T} x {top_k} experts and excludes gap")
    if gap is not None:
        _need(gap, "gap", torch.float32)
        if gap.numel() != T:
            raise KernelError(f"router: gap must hold {T} margins")


def _correction(correction: Optional[torch.Tensor], num_experts: int, groups) -> None:
    if correction is not None:
        _need(correction, "correction", torch.float32)
        if correction.numel() != num_experts:
            raise KernelError(f"router: correction must hold {num_experts} entries, found {correction.numel()}")
        if groups is not None and int(groups[0]) > 1:
            raise KernelError("router: a choice correction together with expert groups is not built")


def router_topk(x: torch.Tensor, router_w: torch.Tensor, shared_gate: Optional[torch.Tensor], top_k: int,
                norm_topk: bool, sel: torch.Tensor, weights: torch.Tensor, shared_scale: Optional[torch.Tensor],
                pin: Optional[torch.Tensor] = None, gap: Optional[torch.Tensor] = None, sigmoid_scores: bool = False,
                groups=None, correction: Optional[torch.Tensor] = None, weight_scale: float = 1.0) -> None:
    """Router logits, softmax over all experts (or, with ``sigmoid_scores``, each expert's own
    sigmoid), top-k and the shared expert's sigmoid gate.
    ``pin`` (int32 [T, k]): the experts are given, not chosen; the weights are still the row's own
    probabilities of them.  ``gap`` (float32 [T], not with ``pin``): each row's routing margin
    (p_k - p_{k+1}) / p_k out.  ``groups`` = (count, keep): the experts form ``count`` equal groups of
    neighbours and only those of the ``keep`` groups with the largest best score can be picked.
    ``correction`` (float32 [E]): added to the scores for the choice alone, a pick's weight stays its score;
    ``weight_scale`` multiplies the picks' weights."""
    _need(x, "x", torch.float32), _need(router_w, "router_w", torch.float32)
    _correction(correction, router_w.shape[0], groups)
    _need(sel, "sel", torch.int32), _need(weights, "weights", torch.float32)
    T, H = x.shape
    E = router_w.shape[0]
    _pin_and_gap(pin, gap, T, top_k)
    if E > 1024:
        raise KernelError(f"router_topk: {E} experts; this kernel takes at most 1024")
    if groups is not None and int(groups[0]) > 1 and E % int(groups[0]) != 0:
        raise KernelError(f"router_topk: {E} experts do not form {groups[0]} equal groups")
    if shared_gate is not None:
        _need(shared_gate, "shared_gate", torch.float32), _need(shared_scale, "shared_scale", torch.float32)
    logits = torch.empty((T, E + 1), dtype=torch.float32, device=x.device)
    tickets = _router_tickets.get(x.device)
    if tickets is None:
        tickets = _router_tickets[x.device] = torch.zeros((4,), dtype=torch.int32, device=x.device)
    st = library("moe_route").cj_router_topk(_ptr(x), _ptr(router_w), _ptr(shared_gate), _i(T), _i(H), _i(E), _i(top_k),
                                             _i(_route_mode(norm_topk, sigmoid_scores, groups)), _ptr(sel), _ptr(weights),
                                             _ptr(shared_scale), _ptr(logits), _ptr(tickets), _ptr(pin), _ptr(gap),
                                             _ptr(correction), _f(weight_scale), _stream())
    _check(st, "router_topk")
    if T > 32:
        global launches
        launches += 1                  # many rows take two kernels: logits, then selection


def router_select(partials: torch.Tensor, num_experts: int, top_k: int, norm_topk: bool, sel: torch.Tensor,
                  weights: torch.Tensor, shared_scale: Optional[torch.Tensor], pin: Optional[torch.Tensor] = None,
                  gap: Optional[torch.Tensor] = None, sigmoid_scores: bool = False, groups=None,
                  correction: Optional[torch.Tensor] = None, weight_scale: float = 1.0) -> None:
    """Softmax over all experts, top-k and the shared gate's sigmoid from router logits given
    as partial sums ``[S, T, ld]`` (float32; column ``num_experts`` holds the gate's dot when
    ``shared_scale`` is given); the partials of a row are added in order first."""
    _need(partials, "partials", torch.float32), _need(sel, "sel", torch.int32), _need(weights, "weights", torch.float32)
    if partials.dim() != 3:
        raise KernelError(f"router_select: partials {tuple(partials.shape)} are not [S, T, ld]")
    if num_experts > 1024:
        raise KernelError(f"router_select: {num_experts} experts; this kernel takes at most 1024")
    S, T, ld = partials.shape
    _pin_and_gap(pin, gap, T, top_k)
    _correction(correction, num_experts, groups)
    if shared_scale is not None:
        _need(shared_scale, "shared_scale", torch.float32)
    st = library("moe_route").cj_router_select(_ptr(partials), _i(S), _ll(partials.stride(0)), _i(ld), _i(T), _i(num_experts),
                                               _i(top_k), _i(_route_mode(norm_topk, sigmoid_scores, groups)), _ptr(sel),
                                               _ptr(weights), _ptr(shared_scale), _ptr(pin), _ptr(gap), _ptr(correction),
                                               _f(weight_scale), _stream())
    _check(st, "router_select")


def moe_group(sel: torch.Tensor, top_k: int, num_experts: int, offsets: torch.Tensor, slot_token: torch.Tensor,
              slot_of_pick: torch.Tensor, extra_groups: int = 0) -> None:
    """Counting sort of the picks by expert: offsets [E + extra + 1], slot_token, slot_of_pick.
    ``extra_groups`` groups that hold every token follow the routed ones."""
    for n, t in (("sel", sel), ("offsets", offsets), ("slot_token", slot_token), ("slot_of_pick", slot_of_pick)):
        _need(t, n, torch.int32)
    n = sel.numel()
    if offsets.numel() < num_experts + extra_groups + 1 or slot_token.numel() < n + extra_groups * (n // top_k):
        raise KernelError("moe_group: offsets or slot_token too small for the extra groups")
    st = library("moe_route").cj_moe_group(_ptr(sel), _i(n), _i(top_k), _i(num_experts), _i(extra_groups), _ptr(offsets),
                                           _ptr(slot_token), _ptr(slot_of_pick), _stream())
    _check(st, "moe_group")


def moe_combine(hs: torch.Tensor, y: Optional[torch.Tensor], slot_of_pick: Optional[torch.Tensor],
                weights: Optional[torch.Tensor], top_k: int, shared: Optional[torch.Tensor],
                shared_scale: Optional[torch.Tensor]) -> None:
    """hs[t] += sum_j weights[t, j] * y[slot_of_pick[t, j]] (+ shared_scale[t] * sum_c shared[c, t]).
    ``shared`` is [T, H] or, computed in chunks, [chunks, T, H]."""
    _need(hs, "hs", torch.float32)
    T, H = hs.shape
    for n, t in (("y", y), ("weights", weights), ("shared", shared), ("shared_scale", shared_scale)):
        if t is not None:
            _need(t, n, torch.float32)
    if slot_of_pick is not None:
        _need(slot_of_pick, "slot_of_pick", torch.int32)
    chunks, stride = 1, 0
    if shared is not None and shared.dim() == 3:
        chunks, stride = shared.shape[0], shared.stride(0)
    st = library("rowwise").cj_moe_combine(_ptr(hs), _ptr(y), _ptr(slot_of_pick), _ptr(weights), _i(top_k), _ptr(shared),
                                           _i(chunks), _ll(stride), _ptr(shared_scale), _i(T), _i(H), _stream())
    _check(st, "moe_combine")


# -- steps on the residual stream between layers ---------------------------------------------------------
def pair_embed(out: torch.Tensor, table: torch.Tensor, pair: torch.Tensor, ids: torch.Tensor, positions: torch.Tensor,
               row_req: torch.Tensor, req_start: torch.Tensor, req_slot: torch.Tensor, state: torch.Tensor, buckets: int,
               mul_prev: int, mul_cur: int) -> None:
    """out[t] = table[ids[t]] + pair[(prev * mul_prev + ids[t] * mul_cur) mod buckets], or pair[buckets] at position 0;
    prev is the row before within the request, or ``state[slot]`` (int32, the request's last token of the step
    before) for its first row of the step.  out float32 [T, H]."""
    _need(out, "out", torch.float32), _need(table, "table"), _need(pair, "pair", table.dtype), _need(state, "state", torch.int32)
    for n, t in (("ids", ids), ("positions", positions), ("row_req", row_req), ("req_start", req_start), ("req_slot", req_slot)):
        _need(t, n, torch.int32)
    T, H = out.shape
    if pair.shape != (buckets + 1, H) or table.shape[1] != H:
        raise KernelError(f"pair_embed: tables {tuple(table.shape)} and {tuple(pair.shape)} do not fit {buckets} buckets of {H}")
    st = library("stream_ops").cj_pair_embed(_ptr(out), _ptr(table), _ptr(pair), _i(_code(table)), _ptr(ids), _ptr(positions),
                                             _ptr(row_req), _ptr(req_start), _ptr(req_slot), _ptr(state), _i(T), _i(H),
                                             _i(table.shape[0]), _i(buckets), _ll(mul_prev), _ll(mul_cur), _stream())
    _check(st, "pair_embed")


def pair_commit(ids: torch.Tensor, req_start: torch.Tensor, req_slot: torch.Tensor, state: torch.Tensor, requests: int) -> None:
    """After ``pair_embed``: every request's last token of the step becomes its ``state`` entry."""
    _need(ids, "ids", torch.int32), _need(req_start, "req_start", torch.int32), _need(req_slot, "req_slot", torch.int32)
    _need(state, "state", torch.int32)
    _check(library("stream_ops").cj_pair_commit(_ptr(ids), _ptr(req_start), _ptr(req_slot), _ptr(state), _i(requests), _stream()),
           "pair_commit")


def add_rows(hs: torch.Tensor, other: Optional[torch.Tensor], vec: Optional[torch.Tensor]) -> None:
    """hs[t] += other[t] + vec; everything float32; either may be None."""
    _need(hs, "hs", torch.float32)
    T, H = hs.shape
    if other is not None:
        _need(other, "other", torch.float32)
        if other.shape != hs.shape:
            raise KernelError("add_rows: shapes differ")
    if vec is not None:
        _need(vec, "vec", torch.float32)
        if vec.numel() != H:
            raise KernelError("add_rows: the vector does not have the rows' width")
    _check(library("stream_ops").cj_add_rows(_ptr(hs), _ptr(other), _ptr(vec), _i(T), _i(H), _stream()), "add_rows")


def add_partials(hs: torch.Tensor, parts: torch.Tensor) -> None:
    """hs += parts[0] + parts[1] + ... in that order; hs float32 [T, H], parts float32 [S, T, H] (the partial sums a
    product cut along K leaves behind, when no norm follows that could add them while it reads the row)."""
    _need(hs, "hs", torch.float32), _need(parts, "parts", torch.float32)
    if parts.dim() != 3 or tuple(parts.shape[1:]) != tuple(hs.shape):
        raise KernelError(f"add_partials: parts {tuple(parts.shape)} do not fit hs {tuple(hs.shape)}")
    st = library("stream_ops").cj_add_partials(_ptr(hs), _ptr(parts), _i(parts.shape[0]), _ll(parts.stride(0)), _ll(hs.numel()), _stream())
    _check(st, "add_partials")


def gelu_gate(a: torch.Tensor, table: torch.Tensor, offset: int, ids: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, j] = gelu_tanh(a[t, j]) * table[ids[t], offset + j]; a float32 [T, >= n], out [T, n] in the table's dtype."""
    _need(a, "a", torch.float32), _need(table, "table"), _need(ids, "ids", torch.int32), _need(out, "out", table.dtype)
    T, n = out.shape
    if a.shape[1] < n or table.shape[1] < offset + n:
        raise KernelError("gelu_gate: sizes do not agree")
    st = library("stream_ops").cj_gelu_gate(_ptr(a), _i(a.stride(0)), _ptr(table), _i(_code(table)), _i(table.stride(0)), _i(offset),
                                            _ptr(ids), _i(table.shape[0]), _ptr(out), _i(_code(out)), _i(T), _i(n), _stream())
    _check(st, "gelu_gate")


def stream_cast(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = x (float32) in out's dtype."""
    _need(x, "x", torch.float32), _need(out, "out")
    if out.numel() != x.numel():
        raise KernelError("stream_cast: sizes differ")
    _check(library("stream_ops").cj_stream_cast(_ptr(x), _ptr(out), _i(_code(out)), _ll(x.numel()), _stream()), "stream_cast")


def stream_norm_add(hs: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float) -> None:
    """hs[t] += y[t] / sqrt(mean(y[t]^2) + eps) * weight; everything float32."""
    _need(hs, "hs", torch.float32), _need(y, "y", torch.float32), _need(weight, "weight", torch.float32)
    T, H = hs.shape
    if y.shape != hs.shape or weight.numel() != H:
        raise KernelError("stream_norm_add: shapes do not agree")
    _check(library("stream_ops").cj_stream_norm_add(_ptr(hs), _ptr(y), _ptr(weight), _f(eps), _i(T), _i(H), _stream()), "stream_norm_add")


# -- a block that norms a sublayer's output; mixers with a state per request -----------------------------
def cast_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = x in out's dtype; x float32."""
    _need(x, "x", torch.float32), _need(out, "out")
    if out.numel() != x.numel():
        raise KernelError("cast_rows: sizes differ")
    _check(library("recurrent").cj_cast_rows(_ptr(x), _ptr(out), _i(_code(out)), _ll(x.numel()), _stream()), "cast_rows")


def rmsnorm_add(hs: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float) -> None:
    """hs[r] += y[r] / sqrt(mean(y[r]^2) + eps) * weight; everything float32."""
    _need(hs, "hs", torch.float32), _need(y, "y", torch.float32), _need(weight, "weight", torch.float32)
    rows, H = hs.shape
    if y.shape != hs.shape or weight.numel() != H:
        raise KernelError(f"rmsnorm_add: shapes hs {tuple(hs.shape)} y {tuple(y.shape)} weight {tuple(weight.shape)} do not agree")
    _check(library("recurrent").cj_rmsnorm_add(_ptr(hs), _ptr(y), _ptr(weight), _f(eps), _i(rows), _i(H), _stream()), "rmsnorm_add")


def scale_rows_gather(x: torch.Tensor, slot_of_pick: torch.Tensor, weights: torch.Tensor, top_k: int, out: torch.Tensor) -> None:
    """out[slot_of_pick[t, j]] = weights[t, j] * x[t]: the rows of a mixture's grouped product when
    a pick's score multiplies the expert's input.  x float32 [T, H]; out [T * k, H]."""
    _need(x, "x", torch.float32), _need(slot_of_pick, "slot_of_pick", torch.int32), _need(weights, "weights", torch.float32)
    _need(out, "out")
    T, H = x.shape
    if slot_of_pick.numel() != T * top_k or weights.numel() != T * top_k or out.shape != (T * top_k, H):
        raise KernelError("scale_rows_gather: sizes do not agree")
    st = library("recurrent").cj_scale_rows_gather(_ptr(x), _ptr(slot_of_pick), _ptr(weights), _i(T * top_k), _i(top_k), _i(H),
                                                   _ptr(out), _i(_code(out)), _stream())
    _check(st, "scale_rows_gather")


def short_conv(x: torch.Tensor, x_offset: int, channels: int, taps: int, weight: torch.Tensor, bias: Optional[torch.Tensor],
               state: torch.Tensor, row_req: torch.Tensor, req_start: torch.Tensor, req_slot: torch.Tensor,
               out: torch.Tensor, activate: bool = True, state_offset: int = 0) -> None:
    """Causal convolution per channel over columns [x_offset, x_offset + channels) of x (float32 [T, ld]):
    out[r, c] = act(bias[c] + sum_j weight[c, taps-1-j] * x[r - j, c]), where rows before the
    request's first row of this step come from ``state`` ([slots, n] float32, whose
    (taps-1) * channels entries per slot from ``state_offset`` on are the request's last inputs, oldest first)."""
    _need(x, "x", torch.float32), _need(weight, "weight", torch.float32), _need(state, "state", torch.float32), _need(out, "out")
    for n, t in (("row_req", row_req), ("req_start", req_start), ("req_slot", req_slot)):
        _need(t, n, torch.int32)
    if bias is not None:
        _need(bias, "bias", torch.float32)
    if weight.shape != (channels, taps) or x.shape[1] < x_offset + channels or out.shape[1] < channels or state[0].numel() < state_offset + (taps - 1) * channels:
        raise KernelError("short_conv: sizes do not agree")
    st = library("recurrent").cj_short_conv(ctypes.c_void_p(x.data_ptr() + 4 * x_offset), _i(x.stride(0)), _i(channels), _i(taps), _ptr(weight), _ptr(bias),
                                            ctypes.c_void_p(state.data_ptr() + 4 * state_offset),
                                            _ll(state.stride(0)), _ptr(row_req), _ptr(req_start), _ptr(req_slot), _ptr(out),
                                            _i(out.stride(0)), _i(_code(out)), _i(1 if activate else 0), _i(x.shape[0]), _stream())
    _check(st, "short_conv")


def short_conv_commit(x: torch.Tensor, x_offset: int, channels: int, taps: int, state: torch.Tensor, req_start: torch.Tensor,
                      req_slot: torch.Tensor, requests: int, state_offset: int = 0) -> None:
    """After ``short_conv``: every request's last taps-1 inputs (of this step, and of the state
    where the step brought fewer) become its state."""
    _need(x, "x", torch.float32), _need(state, "state", torch.float32)
    _need(req_start, "req_start", torch.int32), _need(req_slot, "req_slot", torch.int32)
    if taps <= 1:
        return
    st = library("recurrent").cj_short_conv_commit(ctypes.c_void_p(x.data_ptr() + 4 * x_offset), _i(x.stride(0)), _i(channels), _i(taps),
                                                   ctypes.c_void_p(state.data_ptr() + 4 * state_offset),
                                                   _ll(state.stride(0)), _ptr(req_start), _ptr(req_slot), _i(requests), _stream())
    _check(st, "short_conv_commit")


SCAN_SSD, SCAN_DELTA, SCAN_GLA, SCAN_MLSTM = 0, 1, 2, 3


def state_scan_floats(heads: int, rows: int, cols: int, mode: int = SCAN_SSD) -> int:
    """float32 entries of per-request state that ``state_scan`` needs for ``heads`` matrices of
    rows x cols: the scan keeps them in the order its threads hold them (padded to whole tiles;
    ``SCAN_MLSTM`` keeps a vector over the rows and a scalar beside every tile).
    The same arithmetic as the kernel library's ``cj_state_scan_floats_mode`` (tested equal)."""
    dp = 4
    while dp < 32 and dp < rows and (dp < 8 or heads * cols * dp // 32 < 592):
        dp <<= 1
    while dp < 32 and -(-rows // dp) > 64:
        dp <<= 1
    per = -(-rows // dp)
    nper = 1
    while nper < per:
        nper <<= 1
    cols_per_block = 4 * (32 // dp)
    tile = (2 * nper + 1) * 128 if mode == SCAN_MLSTM else nper * 128
    return heads * -(-cols // cols_per_block) * tile


def state_scan(mode: int, x: torch.Tensor, off_a: int, off_b: int, off_v: int, raw: torch.Tensor, off_dt: int, off_beta: int,
               A_log: Optional[torch.Tensor], dt_bias: Optional[torch.Tensor], skip: Optional[torch.Tensor], state: torch.Tensor,
               state_offset: int, req_start: torch.Tensor, req_slot: torch.Tensor, out: torch.Tensor, requests: int, heads: int,
               groups: int, rows: int, cols: int, q_scale: float = 1.0, c0: float = 0.0, c1: float = 0.0) -> None:
    """Walks every request's rows of the step in order through its recurrent state
    (``state[slot, state_offset:]``, ``state_scan_floats(heads, rows, cols)`` float32 entries in the
    scan's own layout; zero = the empty state) and writes a row's
    read-out to ``out`` [T, heads * cols].

    ``SCAN_SSD``: x columns off_a = B [groups, rows], off_b = C, off_v = x [heads, cols]; raw column
    off_dt + h = the step size before softplus.  S = exp(-exp(A_log) dt) S + dt B x^T; y = S^T C + skip x.
    ``SCAN_DELTA``: off_a = q [groups, rows], off_b = k, off_v = v; raw columns off_dt + h (decay input)
    and off_beta + h.  q and k become unit vectors (q times ``q_scale``); S = g S; u = beta (v - S^T k);
    S += k u^T; o = S^T q.
    ``SCAN_GLA``: off_a = q [heads, rows] (times ``q_scale``), off_b = k, off_v = v; raw columns off_dt + h * rows + d = z,
    the decays' inputs; alpha = sigmoid(z)^c0 (c0 = 1 / tau); S = diag(alpha) S + k v^T; o = S^T q.
    ``SCAN_MLSTM``: off_a = q (times ``q_scale``), off_b = k, off_v = v; raw columns off_dt + h and off_beta + h = the
    input and forget gates before their bias (``dt_bias`` = the input gate's, ``A_log`` = the forget gate's);
    i = c0 tanh((. + b) / c0), f = log sigmoid(c0 tanh((. + b) / c0)); m_t = max(f + m, i), m_0 = 0;
    S = e^(f + m - m_t) S + e^(i - m_t) k v^T, n likewise with k alone; o = S^T q / (max(|n . q|, e^(-m_t)) + c1)."""
    _need(x, "x", torch.float32), _need(raw, "raw", torch.float32), _need(state, "state", torch.float32), _need(out, "out", torch.float32)
    if mode != SCAN_GLA:
        _need(A_log, "A_log", torch.float32), _need(dt_bias, "dt_bias", torch.float32)
    _need(req_start, "req_start", torch.int32), _need(req_slot, "req_slot", torch.int32)
    if skip is not None:
        _need(skip, "skip", torch.float32)
    if state[0].numel() < state_offset + state_scan_floats(heads, rows, cols, mode) or out.shape[1] != heads * cols:
        raise KernelError("state_scan: state or out too small")
    st = library("recurrent").cj_state_scan(
        _i(mode), _ptr(x), _i(x.stride(0)), _i(off_a), _i(off_b), _i(off_v), _ptr(raw), _i(raw.stride(0)), _i(off_dt), _i(off_beta),
        _ptr(A_log), _ptr(dt_bias), _ptr(skip), ctypes.c_void_p(state.data_ptr() + 4 * state_offset), _ll(state.stride(0)),
        _ll(state[0].numel() - state_offset), _ptr(req_start), _ptr(req_slot), _ptr(out), _i(requests), _i(heads), _i(groups), _i(rows), _i(cols), _f(q_scale), _f(c0), _f(c1), _stream())
    _check(st, "state_scan")


def gated_group_norm(y: torch.Tensor, part_len: int, z: torch.Tensor, z_offset: int, weight: torch.Tensor, eps: float,
                     gate_first: bool, out: torch.Tensor, sigmoid_gate: bool = False) -> None:
    """Rows of y (float32 [T, n]) in parts of ``part_len``: RMS norm of each part times weight
    (indexed by column modulo its length) and times silu(z[:, z_offset + column]); the gate is
    applied before the norm's statistics when ``gate_first``, after the norm otherwise.  ``sigmoid_gate``: the
    gate is sigmoid(z) instead of silu(z)."""
    _need(y, "y", torch.float32), _need(z, "z", torch.float32), _need(weight, "weight", torch.float32), _need(out, "out")
    T, n = y.shape
    if out.shape != y.shape or z.shape[1] < z_offset + n:
        raise KernelError("gated_group_norm: sizes do not agree")
    st = library("recurrent").cj_gated_group_norm(_ptr(y), _i(n), _i(part_len), ctypes.c_void_p(z.data_ptr() + 4 * z_offset),
                                                  _i(z.stride(0)), _ptr(weight), _i(weight.numel()), _f(eps),
                                                  _i((1 if gate_first else 0) | (2 if sigmoid_gate else 0)), _ptr(out), _i(_code(out)), _i(T), _stream())
    _check(st, "gated_group_norm")


def rmsnorm_mix2(a: torch.Tensor, wa: torch.Tensor, b: torch.Tensor, wb: torch.Tensor, eps: float, coef: float, out: torch.Tensor,
                 accumulate: bool = False) -> None:
    """out (+)= coef (a / rms(a) * wa + b / rms(b) * wb), row by row; everything float32."""
    for n, t in (("a", a), ("wa", wa), ("b", b), ("wb", wb), ("out", out)):
        _need(t, n, torch.float32)
    rows, H = a.shape
    if b.shape != a.shape or out.shape != a.shape or wa.numel() != H or wb.numel() != H:
        raise KernelError("rmsnorm_mix2: shapes do not agree")
    st = library("recurrent").cj_rmsnorm_mix2(_ptr(a), _ptr(wa), _ptr(b), _ptr(wb), _f(eps), _f(coef), _i(1 if accumulate else 0),
                                              _ptr(out), _i(rows), _i(H), _stream())
    _check(st, "rmsnorm_mix2")


def relu2_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = max(x, 0)^2 in out's dtype; x float32."""
    _need(x, "x", torch.float32), _need(out, "out")
    if out.numel() != x.numel():
        raise KernelError("relu2_rows: sizes differ")
    _check(library("recurrent").cj_relu2_rows(_ptr(x), _ptr(out), _i(_code(out)), _ll(x.numel()), _stream()), "relu2_rows")


def softcap_rows(x: torch.Tensor, cap: float) -> None:
    """x <- cap tanh(x / cap) in place; x float32."""
    _need(x, "x", torch.float32)
    _check(library("recurrent").cj_softcap_rows(_ptr(x), _f(cap), _ll(x.numel()), _stream()), "softcap_rows")


# -- attention over a compressed latent ---------------------------------------------------------------
def latent_kv_write(d: torch.Tensor, d_offset: int, rank: int, rot: int, rotary: int, weight: torch.Tensor, eps: float, inv_freq: Optional[torch.Tensor],
                    positions: torch.Tensor, row_req: torch.Tensor, table: torch.Tensor, page_tokens: int,
                    plane: torch.Tensor) -> None:
    """Columns [d_offset, d_offset + rank + rot) of d (float32): the RMS-normed latent (times weight) and
    the key part, its first ``rotary`` entries rotated in pairs (2i, 2i+1), go to the row's place in
    the paged cache (entries of rank + rot)."""
    _need(d, "d", torch.float32), _need(weight, "weight", torch.float32), _need(plane, "plane")
    _need(positions, "positions", torch.int32), _need(row_req, "row_req", torch.int32), _need(table, "table", torch.int32)
    if d.shape[1] < d_offset + rank + rot or plane.shape[-1] != rank + rot:
        raise KernelError("latent_kv_write: sizes do not agree")
    st = library("latent_attention").cj_latent_kv_write(ctypes.c_void_p(d.data_ptr() + 4 * d_offset), _i(d.stride(0)), _i(rank), _i(rot), _i(rotary), _ptr(weight), _f(eps),
                                                        _ptr(inv_freq), _ptr(positions), _ptr(row_req), _ptr(table),
                                                        _i(table.stride(0)), _i(page_tokens), _ptr(plane), _i(_code(plane)),
                                                        _i(d.shape[0]), _stream())
    _check(st, "latent_kv_write")


def latent_q_split(q: torch.Tensor, heads: int, dim: int, rot: int, rotary: int, inv_freq: Optional[torch.Tensor], positions: torch.Tensor,
                   q_plain: torch.Tensor, q_rot: torch.Tensor) -> None:
    """q float32 [T, >= heads * (dim + rot)] -> q_plain [heads, T, dim] and the rotated parts q_rot float32 [T, heads, rot]."""
    _need(q, "q", torch.float32), _need(q_plain, "q_plain"), _need(q_rot, "q_rot", torch.float32), _need(positions, "positions", torch.int32)
    T = q.shape[0]
    if q_plain.numel() != heads * T * dim or q_rot.numel() != T * heads * rot:
        raise KernelError("latent_q_split: sizes do not agree")
    st = library("latent_attention").cj_latent_q_split(_ptr(q), _i(q.stride(0)), _i(heads), _i(dim), _i(rot), _i(rotary), _ptr(inv_freq),
                                                       _ptr(positions), _i(T), _ptr(q_plain), _i(_code(q_plain)), _ptr(q_rot), _stream())
    _check(st, "latent_q_split")


LATENT_SPLIT_MIN_KEYS = 64       # a stretch of a row's keys is at least this long
LATENT_FILL_BLOCKS = 592         # blocks that fill the machine (four an SM); fewer: the rows' keys are cut into stretches


def latent_attention(q_abs: torch.Tensor, q_rot: torch.Tensor, plane: torch.Tensor, rank: int, rot: int, heads: int,
                     positions: torch.Tensor, row_req: torch.Tensor, table: torch.Tensor, page_tokens: int, scale: float,
                     out: torch.Tensor, max_context: int = 0, sink: Optional[torch.Tensor] = None) -> None:
    """Every (row, head): softmax over the row's keys [0, position] of (q_abs . c + q_rot . r) * scale,
    and the weighted sum of the latents.  q_abs float32 [heads, T, rank]; q_rot float32 [T, heads, rot];
    out [heads, T, rank] in the cache's dtype.  ``max_context`` (the longest row's keys, when the
    caller knows it): with few rows the keys of a row are cut into stretches that run side by side.
    ``sink`` (float32 [heads]): the softmax's divisor also holds exp(sink[h])."""
    if sink is not None:
        _need(sink, "sink", torch.float32)
        if sink.numel() != heads:
            raise KernelError(f"latent_attention: sink must hold {heads} entries")
    _need(q_abs, "q_abs", torch.float32), _need(q_rot, "q_rot", torch.float32), _need(plane, "plane"), _need(out, "out", plane.dtype)
    _need(positions, "positions", torch.int32), _need(row_req, "row_req", torch.int32), _need(table, "table", torch.int32)
    T = positions.numel()
    if q_abs.numel() != heads * T * rank or out.numel() != heads * T * rank or plane.shape[-1] != rank + rot:
        raise KernelError("latent_attention: sizes do not agree")
    blocks = T * -(-heads // 8)
    split_keys, splits, part_acc, part_ml = 0, 1, None, None
    if max_context > LATENT_SPLIT_MIN_KEYS and blocks < LATENT_FILL_BLOCKS:
        want = min(64, -(-LATENT_FILL_BLOCKS // blocks))
        split_keys = max(LATENT_SPLIT_MIN_KEYS, -(-(-(-max_context // want)) // 32) * 32)
        splits = -(-max_context // split_keys)
        if splits > 1:
            part_acc = torch.empty((T, heads, splits, rank), dtype=torch.float32, device=out.device)
            part_ml = torch.empty((T, heads, splits, 2), dtype=torch.float32, device=out.device)
        else:
            split_keys = 0
    st = library("latent_attention").cj_latent_attention(_ptr(q_abs), _ptr(q_rot), _ptr(plane), _i(_code(plane)), _i(rank), _i(rot),
                                                         _i(heads), _i(T), _ptr(positions), _ptr(row_req), _ptr(table),
                                                         _i(table.stride(0)), _i(page_tokens), _f(scale), _ptr(out),
                                                         _i(split_keys), _i(splits), _ptr(part_acc), _ptr(part_ml), _ptr(sink), _stream())
    _check(st, "latent_attention")
    if split_keys:
        global launches
        launches += 1                  # the merge is a kernel of its own


# -- the plain form for long prompt portions: keys and values built per head, a flash kernel over them --
def latent_gather(plane: torch.Tensor, rank: int, tok_req: torch.Tensor, tok_pos: torch.Tensor, table: torch.Tensor,
                  page_tokens: int, c_all: torch.Tensor) -> None:
    """c_all[n] = the latent of (request tok_req[n], position tok_pos[n]) from the paged cache; bfloat16."""
    _need(plane, "plane", torch.bfloat16), _need(c_all, "c_all", torch.bfloat16), _need(table, "table", torch.int32)
    _need(tok_req, "tok_req", torch.int32), _need(tok_pos, "tok_pos", torch.int32)
    st = library("latent_prefill").cj_latent_gather(_ptr(plane), _i(plane.shape[-1]), _i(rank), _ptr(tok_req), _ptr(tok_pos), _ptr(table),
                                                    _i(table.stride(0)), _i(page_tokens), _ptr(c_all), _i(tok_req.numel()), _stream())
    _check(st, "latent_gather")


def latent_kv_pack(kp: torch.Tensor, vp: torch.Tensor, plane: torch.Tensor, rank: int, rot: int, tok_req: torch.Tensor,
                   tok_pos: torch.Tensor, table: torch.Tensor, page_tokens: int, heads: int, dim: int, vdim: int,
                   kx: torch.Tensor, vx: torch.Tensor) -> None:
    """kx[n, h] = [kp[n, h] | the cached rotated key part of token n | 0], vx[n, h] = [vp[n, h] | 0]; bfloat16."""
    for n, t in (("kp", kp), ("vp", vp), ("plane", plane), ("kx", kx), ("vx", vx)):
        _need(t, n, torch.bfloat16)
    _need(tok_req, "tok_req", torch.int32), _need(tok_pos, "tok_pos", torch.int32), _need(table, "table", torch.int32)
    N = tok_req.numel()
    if kp.numel() != N * heads * dim or vp.numel() != N * heads * vdim or kx.shape[:2] != (N, heads) or vx.shape[:2] != (N, heads):
        raise KernelError("latent_kv_pack: sizes do not agree")
    st = library("latent_prefill").cj_latent_kv_pack(_ptr(kp), _ptr(vp), _ptr(plane), _i(plane.shape[-1]), _i(rank), _i(rot), _ptr(tok_req),
                                                     _ptr(tok_pos), _ptr(table), _i(table.stride(0)), _i(page_tokens), _i(heads), _i(dim),
                                                     _i(vdim), _i(kx.shape[2]), _i(vx.shape[2]), _ptr(kx), _ptr(vx), _i(N), _stream())
    _check(st, "latent_kv_pack")


def latent_q_pack(q: torch.Tensor, heads: int, dim: int, rot: int, rotary: int, inv_freq: Optional[torch.Tensor],
                  positions: torch.Tensor, qx: torch.Tensor) -> None:
    """qx[t, h] = [q[t, h, :dim] | rotate(q[t, h, dim:]) | 0] in bfloat16; q float32 [T, >= heads (dim + rot)]."""
    _need(q, "q", torch.float32), _need(qx, "qx", torch.bfloat16), _need(positions, "positions", torch.int32)
    st = library("latent_prefill").cj_latent_q_pack(_ptr(q), _i(q.stride(0)), _i(heads), _i(dim), _i(rot), _i(rotary), _ptr(inv_freq),
                                                    _ptr(positions), _i(qx.shape[2]), _ptr(qx), _i(q.shape[0]), _stream())
    _check(st, "latent_q_pack")


def latent_flash(qx: torch.Tensor, out: torch.Tensor, kx: torch.Tensor, vx: torch.Tensor, req_start: torch.Tensor,
                 req_prior: torch.Tensor, req_base: torch.Tensor, requests: int, heads: int, scale: float,
                 sink: Optional[torch.Tensor] = None) -> None:
    """Causal attention of the step's rows (request i: rows [req_start[i], req_start[i+1]) at positions
    req_prior[i] + j) over the dense keys and values of their requests (request i's token p at
    req_base[i] + p).  qx [T, heads, DK], kx [N, heads, DK], vx [N, heads, DV], out [T, heads, DV], bfloat16.
    ``sink`` (float32 [heads]): the softmax's divisor also holds exp(sink[h])."""
    if sink is not None:
        _need(sink, "sink", torch.float32)
    for n, t in (("qx", qx), ("out", out), ("kx", kx), ("vx", vx)):
        _need(t, n, torch.bfloat16)
    for n, t in (("req_start", req_start), ("req_prior", req_prior), ("req_base", req_base)):
        _need(t, n, torch.int32)
    st = library("latent_prefill").cj_latent_flash(_ptr(qx), _ptr(out), _ptr(kx), _ptr(vx), _ptr(req_start), _ptr(req_prior), _ptr(req_base),
                                                   _i(requests), _i(qx.shape[0]), _i(heads), _i(qx.shape[2]), _i(vx.shape[2]), _f(scale),
                                                   _ptr(sink), _stream())
    _check(st, "latent_flash")


def latent_gate_rows(o: torch.Tensor, gate: Optional[torch.Tensor], gate_offset: int, heads: int, vdim: int, out: torch.Tensor) -> None:
    """out[t, h * vdim + e] = o[t, h, e] * sigmoid(gate[t, gate_offset + h]); o bfloat16 [T, heads, DV], gate float32
    (None: no gate, the heads' entries are only moved out of their padding)."""
    _need(o, "o", torch.bfloat16), _need(out, "out", torch.bfloat16)
    gate_ptr, gate_ld = _gate(gate, gate_offset)
    st = library("latent_prefill").cj_latent_gate_rows(_ptr(o), _i(o.shape[2]), gate_ptr,
                                                       _i(gate_ld), _i(heads), _i(vdim), _ptr(out), _i(o.shape[0]), _stream())
    _check(st, "latent_gate_rows")


def latent_q_norm(x: torch.Tensor, offset: int, n: int, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """out[t] = rms(x[t, offset : offset + n]) * weight: the norm of a stretch of columns of a float32 matrix, into
    ``out`` [T, n] in its own dtype."""
    _need(x, "x", torch.float32), _need(weight, "weight", torch.float32), _need(out, "out")
    if weight.numel() != n or tuple(out.shape) != (x.shape[0], n) or offset + n > x.shape[1]:
        raise KernelError("latent_q_norm: sizes do not agree")
    st = library("latent_attention").cj_latent_q_norm(_ptr(x), _i(x.stride(0)), _i(offset), _i(n), _ptr(weight), _f(eps), _ptr(out),
                                                      _i(_code(out)), _i(x.shape[0]), _stream())
    _check(st, "latent_q_norm")


def latent_gate_out(o: torch.Tensor, gate: Optional[torch.Tensor], gate_offset: int, heads: int, vdim: int, out: torch.Tensor) -> None:
    """out[t, h, :] = o[h, t, :] * sigmoid(gate[t, gate_offset + h]); o float32 [heads, T, vdim], gate float32 (None: no gate)."""
    _need(o, "o", torch.float32), _need(out, "out")
    T = out.shape[0]
    if o.numel() != heads * T * vdim or out.shape[1] != heads * vdim:
        raise KernelError("latent_gate_out: sizes do not agree")
    gate_ptr, gate_ld = _gate(gate, gate_offset)
    st = library("latent_attention").cj_latent_gate_out(_ptr(o), gate_ptr, _i(gate_ld),
                                                        _i(heads), _i(vdim), _i(T), _ptr(out), _i(_code(out)), _stream())
    _check(st, "latent_gate_out")


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """First-occurrence argmax of each row of float32 logits into int32 out."""
    _need(logits, "logits", torch.float32), _need(out, "out", torch.int32)
    rows, V = logits.shape
    st = library("sampling").cj_argmax(_ptr(logits), _i(rows), _i(V), _ptr(out), _stream())
    _check(st, "argmax")


def sample(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor, scratch: torch.Tensor,
           out: torch.Tensor, top_k: Optional[torch.Tensor] = None, top_p: Optional[torch.Tensor] = None,
           repeat_penalty: Optional[torch.Tensor] = None, history: Optional[torch.Tensor] = None,
           history_offsets: Optional[torch.Tensor] = None) -> None:
    """One token per row by the reference's sampler order; scratch is [rows, V] float32."""
    _need(logits, "logits", torch.float32), _need(temperature, "temperature", torch.float32)
    _need(uniform, "uniform", torch.float32), _need(scratch, "scratch", torch.float32), _need(out, "out", torch.int32)
    rows, V = logits.shape
    if scratch.numel() < rows * V:
        raise KernelError("sample: scratch is smaller than the logits")
    for n, t, d in (("top_k", top_k, torch.int32), ("top_p", top_p, torch.float32),
                    ("repeat_penalty", repeat_penalty, torch.float32), ("history", history, torch.int32),
                    ("history_offsets", history_offsets, torch.int32)):
        if t is not None:
            _need(t, n, d)
    st = library("sampling").cj_sample(_ptr(logits), _i(rows), _i(V), _ptr(temperature), _ptr(top_k), _ptr(top_p),
                                       _ptr(repeat_penalty), _ptr(uniform), _ptr(history), _ptr(history_offsets),
                                       _ptr(scratch), _ptr(out), _stream())
    _check(st, "sample")


def random_fill(out: torch.Tensor, key: int, scale: float) -> None:
    """out.flat[i] = float32(n(key, i)) * scale, n a centred sum of eight 16-bit integers hashed
    from (key, i); float32 or bfloat16 (see weights/random_fill.py for the same on the host)."""
    _need(out, "out")
    st = library("random_fill").cj_random_fill(_ptr(out), _i(_code(out)), _ll(out.numel()), ctypes.c_ulonglong(key & (2 ** 64 - 1)),
                                               _f(scale), _stream())
    _check(st, "random_fill")


EPI_STORE_F32, EPI_ACC_F32, EPI_SWIGLU_BF16, EPI_STORE_BF16, EPI_RELU2_BF16 = 0, 1, 2, 3, 4


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int, swap: bool, n_mma: int,
            bias: Optional[torch.Tensor] = None, w_up: Optional[torch.Tensor] = None,
            group_offsets: Optional[torch.Tensor] = None, tokens: Optional[int] = None, k_splits: int = 1,
            offsets_settled: bool = False, act_limit: float = 0.0, act_alpha: float = 1.0) -> None:
    """Tensor-core product out[token, feature] (+)= x[token, :] . w[feature, :] (+ bias) in
    bfloat16 with float32 accumulation (tcgen05, TMA).

    ``swap`` False: tiles of 128 tokens x ``n_mma`` (128 or 256) features; True: tiles of 128
    features x ``n_mma`` (16, 32, 64, 96, 128, 160, 192, 256) tokens.  ``epilogue``: EPI_STORE_F32, EPI_ACC_F32,
    EPI_SWIGLU_BF16 (``w_up`` given), EPI_STORE_BF16, EPI_RELU2_BF16 (``max(sum, 0)^2`` rounded to bfloat16).  With ``group_offsets`` the rows of
    ``x`` are sorted by group and ``w`` is [groups, features, K].  ``k_splits`` > 1 (store
    only): ``out`` is [k_splits, tokens, features] of partial sums.  ``offsets_settled``: the
    kernel that wrote ``group_offsets`` is not the one launched just before this product but an
    earlier one; the product then reads them before it waits for the kernel before it.
    """
    _need(x, "x", torch.bfloat16), _need(w, "w", torch.bfloat16), _need(out, "out")
    features, K = w.shape[-2], w.shape[-1]
    T = tokens if tokens is not None else x.shape[0]
    if x.shape[-1] != K or out.shape[-1] != features:
        raise KernelError(f"gemm_tc: shapes x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)} do not agree")
    want = torch.bfloat16 if epilogue in (EPI_SWIGLU_BF16, EPI_STORE_BF16, EPI_RELU2_BF16) else torch.float32
    if out.dtype != want:
        raise KernelError(f"gemm_tc: epilogue {epilogue} writes {want}, out is {out.dtype}")
    if w_up is not None:
        _need(w_up, "w_up", torch.bfloat16)
    if bias is not None:
        _need(bias, "bias", torch.float32)
    G = 0
    if group_offsets is not None:
        _need(group_offsets, "group_offsets", torch.int32)
        G = w.shape[0]
    split_stride = out.stride(0) if k_splits > 1 else 0
    ldo = out.stride(-2)
    st = library("gemm_tc").cj_gemm_tc(
        _ptr(x), _ll(x.stride(0)), _ptr(w), _ptr(w_up), _ptr(bias), _ptr(out), _ll(ldo), _i(T), _i(features), _i(K),
        _i(epilogue), _i(1 if swap else 0), _i(n_mma), _ptr(group_offsets), _i(G), _i(k_splits), _ll(split_stride),
        _i(1 if offsets_settled and group_offsets is not None else 0), _f(act_limit), _f(act_alpha), _stream())
    _check(st, "gemm_tc")


def gemm_tc2(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int, n_tok: int,
             bias: Optional[torch.Tensor] = None, w_up: Optional[torch.Tensor] = None,
             group_offsets: Optional[torch.Tensor] = None, tokens: Optional[int] = None, act_limit: float = 0.0,
             act_alpha: float = 1.0) -> None:
    """The same product as ``gemm_tc`` on pairs of SMs (tcgen05 cta_group::2): tiles of 256
    features x ``n_tok`` (128 or 256) tokens, each SM of a pair loading its own 128 weight rows
    and half of the token rows.  For steps with many rows."""
    _need(x, "x", torch.bfloat16), _need(w, "w", torch.bfloat16), _need(out, "out")
    features, K = w.shape[-2], w.shape[-1]
    T = tokens if tokens is not None else x.shape[0]
    if x.shape[-1] != K or out.shape[-1] != features:
        raise KernelError(f"gemm_tc2: shapes x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)} do not agree")
    want = torch.bfloat16 if epilogue in (EPI_SWIGLU_BF16, EPI_STORE_BF16, EPI_RELU2_BF16) else torch.float32
    if out.dtype != want:
        raise KernelError(f"gemm_tc2: epilogue {epilogue} writes {want}, out is {out.dtype}")
    if w_up is not None:
        _need(w_up, "w_up", torch.bfloat16)
    if bias is not None:
        _need(bias, "bias", torch.float32)
    G = 0
    if group_offsets is not None:
        _need(group_offsets, "group_offsets", torch.int32)
        G = w.shape[0]
    st = library("gemm_tc2").cj_gemm_tc2(
        _ptr(x), _ll(x.stride(0)), _ptr(w), _ptr(w_up), _ptr(bias), _ptr(out), _ll(out.stride(-2)), _i(T), _i(features), _i(K),
        _i(epilogue), _i(n_tok), _ptr(group_offsets), _i(G), _f(act_limit), _f(act_alpha), _stream())
    _check(st, "gemm_tc2")


def gemm_tc_error() -> int:
    """0, or the code of a bounded wait inside a tensor-core kernel that ran out of time."""
    return int(library("gemm_tc").cj_gemm_tc_error())


def gather_rows(x: torch.Tensor, index: torch.Tensor, out: torch.Tensor) -> None:
    """out[s, :] = x[index[s], :]."""
    _need(x, "x"), _need(index, "index", torch.int32), _need(out, "out", x.dtype)
    st = library("rowwise").cj_gather_rows(_ptr(out), _ptr(x), _i(_code(x)), _ptr(index), _i(out.shape[0]), _i(x.shape[-1]), _stream())
    _check(st, "gather_rows")


# CAJETA_B200_DECODE_FMA=1: decode attention on the FMA pipe instead of the tensor cores (for comparison)
DECODE_TENSOR_CORES = os.environ.get("CAJETA_B200_DECODE_FMA", "0") != "1"
# (row, head) pairs from which on the merge of a row's chunks is a kernel of its own: the attention
# blocks then end without a fence and a ticket, and their shared memory is free that much sooner.
# Measured: 64 rows x 16 heads +9 % (576 keys) and +10 % (2,048 keys: 5.1 TB/s); 32 rows the same
# either way; 8 rows of 4,096 keys 7 % slower (few merges, each a long chain, no longer hidden).
# (Rows of many chunks with few rows in the step - 1 or 4 rows of 16,384 keys - were measured too: the merge
# as a kernel of its own is a tail that nothing overlaps, 2.78 -> 3.32 ms and 5.28 -> 6.03 ms a step.)
MERGE_LATER_MIN_ROW_HEADS = 1024


def decode_chunk(span: int) -> int:
    """Keys a block of the split-KV decode kernel takes.  The kernel also takes 64; measured on
    a B200 it gains nothing for a handful of rows and loses 10 % for many, so 128 it is."""
    return 128


def decode_attention(q: torch.Tensor, out: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor,
                     positions: torch.Tensor, row_req: torch.Tensor, table: torch.Tensor, page_tokens: int,
                     n_heads: int, n_kv: int, head_dim: int, window: int, scale: float, max_context: int,
                     scratch: "DecodeScratch", chunk: int = 0, tensor_cores: Optional[bool] = None,
                     merge_later: Optional[bool] = None, softcap: float = 0.0, head_gate: Optional[torch.Tensor] = None,
                     gate_offset: int = 0) -> None:
    """Split-KV attention of few bfloat16 query rows over their cached keys (head_dim 64 or 128).
    ``tensor_cores``: scores and weighted values of a chunk by mma.sync (the default) or on the
    FMA pipe (``chunk`` 64 or 128 applies to that form only).  ``merge_later``: the chunks of a
    row are merged by a kernel of its own instead of the row's last block (the default for steps
    with many rows; same results to the bit).  ``softcap`` and ``head_gate`` as in ``paged_attention``
    (tensor-core form only)."""
    for n, t in (("q", q), ("out", out), ("k_plane", k_plane), ("v_plane", v_plane)):
        _need(t, n, torch.bfloat16)
    _need(positions, "positions", torch.int32), _need(row_req, "row_req", torch.int32), _need(table, "table", torch.int32)
    T = q.shape[0]
    span = min(window, max_context) if window > 0 else max_context
    gate_ptr, gate_ld = _gate(head_gate, gate_offset)
    if tensor_cores is None:
        tensor_cores = (DECODE_TENSOR_CORES and chunk == 0) or softcap > 0.0 or head_gate is not None
    if tensor_cores:
        splits = max(1, -(-span // 128))
        scratch.ensure(T, n_heads, n_kv, head_dim, splits, q.device)
        if merge_later is None:
            merge_later = T * n_heads >= MERGE_LATER_MIN_ROW_HEADS
        st = library("attention_decode").cj_decode_attention_tc(
            _ptr(q), _ptr(out), _ptr(k_plane), _ptr(v_plane), _ptr(positions), _ptr(row_req), _ptr(table),
            _i(table.stride(0)), _i(page_tokens), _i(T), _i(n_heads), _i(n_kv), _i(head_dim), _i(window), _f(scale),
            _i(max_context), _ptr(scratch.acc), _ptr(scratch.ml), _ptr(scratch.counters), _i(scratch.splits),
            _i(1 if merge_later else 0), _f(softcap), gate_ptr, _i(gate_ld), _stream())
        _check(st, "decode_attention")
        if merge_later and splits > 1:
            global launches
            launches += 1                  # the merge kernel
        return
    if softcap > 0.0 or head_gate is not None:
        raise KernelError("decode_attention: capped scores and gated heads are built into the tensor-core form only")
    chunk = chunk or decode_chunk(span)
    splits = max(1, -(-span // chunk))
    scratch.ensure(T, n_heads, n_kv, head_dim, splits, q.device)
    st = library("attention_decode").cj_decode_attention(
        _ptr(q), _ptr(out), _ptr(k_plane), _ptr(v_plane), _ptr(positions), _ptr(row_req), _ptr(table), _i(table.stride(0)),
        _i(page_tokens), _i(T), _i(n_heads), _i(n_kv), _i(head_dim), _i(window), _f(scale), _i(max_context),
        _ptr(scratch.acc), _ptr(scratch.ml), _ptr(scratch.counters), _i(scratch.splits), _i(chunk), _stream())
    _check(st, "decode_attention")


class DecodeScratch:
    """Partial results of the split-KV decode kernel and its arrival counters (kept zero
    between launches by the kernel itself)."""

    def __init__(self):
        self.acc = self.ml = self.counters = None
        self.rows = self.heads = self.kv = self.hd = self.splits = 0

    def ensure(self, rows: int, heads: int, kv: int, hd: int, splits: int, device) -> None:
        if (self.acc is None or rows > self.rows or heads != self.heads or kv != self.kv or hd != self.hd
                or splits > self.splits):
            self.rows, self.heads, self.kv, self.hd = max(rows, self.rows), heads, kv, hd
            self.splits = max(splits, self.splits)
            self.acc = torch.empty((self.rows, heads, self.splits, hd), dtype=torch.float32, device=device)
            self.ml = torch.empty((self.rows, heads, self.splits, 2), dtype=torch.float32, device=device)
            self.counters = torch.zeros((self.rows * heads,), dtype=torch.int32, device=device)


def prefill_attention(q: torch.Tensor, out: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor,
                      req_start: torch.Tensor, req_prior: torch.Tensor, table: torch.Tensor, page_tokens: int,
                      n_heads: int, n_kv: int, head_dim: int, window: int, scale: float, block_rows: int = 0,
                      softcap: float = 0.0, head_gate: Optional[torch.Tensor] = None, gate_offset: int = 0) -> None:
    """Tensor-core attention of a step's rows (request r owns rows req_start[r]..req_start[r+1]
    at positions req_prior[r] + i) over the paged cache; bfloat16, head_dim 32, 64, 96 or 128.
    ``softcap`` and ``head_gate`` as in ``paged_attention``."""
    for n, t in (("q", q), ("out", out), ("k_plane", k_plane), ("v_plane", v_plane)):
        _need(t, n, torch.bfloat16)
    _need(req_start, "req_start", torch.int32), _need(req_prior, "req_prior", torch.int32), _need(table, "table", torch.int32)
    gate_ptr, gate_ld = _gate(head_gate, gate_offset)
    st = library("attention_prefill").cj_prefill_attention(
        _ptr(q), _ptr(out), _ptr(k_plane), _ptr(v_plane), _ptr(req_start), _ptr(req_prior), _i(req_prior.numel()),
        _i(q.shape[0]), _ptr(table), _i(table.stride(0)), _i(page_tokens), _i(n_heads), _i(n_kv), _i(head_dim), _i(window),
        _f(scale), _i(block_rows), _f(softcap), gate_ptr, _i(gate_ld), _stream())
    _check(st, "prefill_attention")


def prefill_attention_tc(q: torch.Tensor, out: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor,
                         req_start: torch.Tensor, req_prior: torch.Tensor, table: torch.Tensor, page_tokens: int,
                         n_heads: int, n_kv: int, head_dim: int, window: int, scale: float, block_rows: int = 0,
                         softcap: float = 0.0, head_gate: Optional[torch.Tensor] = None, gate_offset: int = 0) -> None:
    """The same arguments and meaning as ``prefill_attention``, on the tcgen05 tensor cores: both products
    from shared memory into tensor memory.  ``block_rows``: 256 query rows a block (two tiles
    taking turns), 128, or 0 = by the size of the launch.  Head size 128 and pages of 16 tokens
    only; anything else is refused."""
    for n, t in (("q", q), ("out", out), ("k_plane", k_plane), ("v_plane", v_plane)):
        _need(t, n, torch.bfloat16)
    _need(req_start, "req_start", torch.int32), _need(req_prior, "req_prior", torch.int32), _need(table, "table", torch.int32)
    if head_dim != 128 or page_tokens != 16:
        raise KernelError(f"prefill_attention_tc takes head size 128 and 16-token pages, not {head_dim} and {page_tokens}")
    gate_ptr, gate_ld = _gate(head_gate, gate_offset)
    st = library("attention_prefill_tc").cj_prefill_attention_tc(
        _ptr(q), _ptr(out), _ptr(k_plane), _ptr(v_plane), _i(k_plane.shape[0]), _ptr(req_start), _ptr(req_prior),
        _i(req_prior.numel()), _i(q.shape[0]), _ptr(table), _i(table.stride(0)), _i(page_tokens), _i(n_heads), _i(n_kv),
        _i(head_dim), _i(window), _f(scale), _i(block_rows), _f(softcap), gate_ptr, _i(gate_ld), _stream())
    _check(st, "prefill_attention_tc")


def prefill_attention_tc_error() -> int:
    """0, or the code of a bounded wait inside the tensor-core attention that ran out of time."""
    return int(library("attention_prefill_tc").cj_prefill_attention_tc_error())


def wait_errors() -> Dict[str, int]:
    """Codes of bounded waits that ran out inside the tensor-core kernels, by library; empty
    when all is well.  Only libraries that are already loaded are asked."""
    found = {}
    for name, symbol in (("gemm_tc", "cj_gemm_tc_error"), ("gemm_tc2", "cj_gemm_tc2_error"),
                         ("attention_prefill_tc", "cj_prefill_attention_tc_error")):
        lib = _libs.get(name)
        if lib is not None:
            code = int(getattr(lib, symbol)())
            if code != 0:
                found[name] = code
    return found
