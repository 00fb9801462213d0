"""Mixers that keep a state of fixed size per request: the state-space mixer of Mamba-2 and
the gated delta rule.

Both project the row, pass part of the projection through a short causal convolution over
time (per channel, ``conv`` taps, then SiLU) and walk the request's tokens in order through a
float32 state ``S`` per head.  The state of a request lives in its slot of the cache
manager's state tensor (one flat float32 vector per schedule entry: the convolution's last
``conv - 1`` inputs, then the heads' ``S`` in the order the scan's threads hold them); it is
zeroed when the slot is admitted.  Both
find their rows, requests and slots in the step's device metadata only, so their steps can
be captured into CUDA graphs (``graph_safe``).

``ssd`` (Mamba-2, state-space duality).  ``inner = heads * vdim``; ``W_in x`` is laid out
``[z: inner | x: inner | B: groups * state | C: groups * state | dt: heads]``; x, B and C pass
the convolution (with bias) and SiLU.  ``dt = softplus(dt + dt_bias)`` (no clamp).  Head h,
group ``h // (heads / groups)``::

    S_t = exp(-exp(A_log_h) dt) S_(t-1) + dt B_t x_t^T        (S: state x vdim)
    y_t = S_t^T C_t + D_h x_t

``y * silu(z)`` is RMS-normed in ``norm_groups`` equal parts, times ``norm``, then ``W_o``.
Parameters: ``hidden_size``, ``heads``, ``vdim``, ``state``, ``groups``, ``norm_groups``,
``conv``, ``eps``.  Tensors: ``in``, ``conv``, ``conv.b``, ``dt_bias``, ``A_log``, ``D``,
``norm``, ``o``.

``gated_delta``.  ``q, k`` (``kv_heads x dim``) and ``v`` (``heads x vdim``) each pass a
convolution (no bias) and SiLU; q and k become unit vectors per head
(``x / sqrt(sum x^2 + 1e-6)``), q also times ``dim^(-1/2)``; ``beta = sigmoid(W_b x)``,
``g = exp(-exp(A_log_h) softplus(W_a x + dt_bias))``.  Head h, key head
``h // (heads / kv_heads)``::

    S <- g S ;  u = beta (v - S^T k) ;  S <- S + k u^T ;  o = S^T q      (S: dim x vdim)

Each head's ``o`` is RMS-normed over vdim, times ``norm`` (vdim entries, shared by the
heads), times ``silu(W_g x)``, then ``W_o``.  Parameters: ``hidden_size``, ``heads``,
``kv_heads``, ``dim``, ``vdim``, ``conv``, ``eps``.  Tensors: ``q``, ``q.conv``, ``k``,
``k.conv``, ``v``, ``v.conv``, ``b``, ``a``, ``A_log``, ``dt_bias``, ``g``, ``norm``, ``o``.

``gla`` (gated linear attention).  ``q = W_q x dim^(-1/2)``, ``k = W_k x`` (``heads x dim``), ``v = W_v x``
(``heads x vdim``), no convolution.  A decay per key channel, ``alpha = sigmoid(z)^(1 / tau)`` with
``z = W_a2 (W_a1 x) + b_a2`` (a product through ``decay_rank`` entries), laid out ``heads x dim``::

    S_t = diag(alpha_t) S_(t-1) + k_t v_t^T ;  o_t = S_t^T q_t                    (S: dim x vdim)

Each head's ``o`` is RMS-normed over vdim, times ``norm`` (vdim entries, shared by the heads), times
``silu(W_g x)``, then ``W_o``.  The second product of the decay and the decay itself are float32.
Parameters: ``hidden_size``, ``heads``, ``dim``, ``vdim``, ``decay_rank``, ``tau``, ``eps``.  Tensors: ``q``,
``k``, ``v``, ``g``, ``a1``, ``a2``, ``a2.b``, ``norm``, ``o``.

``mlstm`` (the matrix memory of xLSTM).  ``q = W_q x dim^(-1/2)``, ``k``, ``v`` as above; per head the
logarithms of an input and a forget gate, ``i = cap tanh((W_i x + b_i) / cap)``,
``f = log sigmoid(cap tanh((W_f x + b_f) / cap))``, and a running maximum ``m`` that starts at 0::

    m_t = max(f + m_(t-1), i) ;  S_t = e^(f + m_(t-1) - m_t) S_(t-1) + e^(i - m_t) k v^T ;  n_t likewise with k alone
    o_t = S_t^T q / (max(|n_t . q|, e^(-m_t)) + floor)

Each head's ``o`` is divided by its root mean square, the heads side by side times ``norm`` (``heads * vdim``
entries), times ``sigmoid(W_g x)``, then ``W_o``.  Parameters: ``hidden_size``, ``heads``, ``dim``, ``vdim``,
``gate_cap``, ``floor`` (default 1e-6), ``eps``.  Tensors: ``q``, ``k``, ``v``, ``g``, ``i``, ``i.b``, ``f``,
``f.b``, ``norm``, ``o``.

A mixer inside another part (a block that keeps state of its own before the mixer's, a mixer that runs two
side by side) finds its share of the request's state vector at ``entry.state_offset``.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import kernels as K
from .base import Part, StateNeed, register_part
from .linear import project
from .plan import ParamSpec


class _StateMixer(Part):
    graph_safe = True          # rows, requests and slots come from the step's device metadata only

    def cache_need(self):
        return None

    def libraries(self) -> set:
        libs = {"recurrent", "gemm_simt"}
        if self.runtime.fast_kernels and self.hidden >= 128:
            libs |= {"gemm_tc", "gemm_tc2"}
        return libs

    def _convolve(self, proj: torch.Tensor, offset: int, ctx, entry) -> torch.Tensor:
        """The convolved, activated columns of this step's rows (float32); the state moves on."""
        conv = torch.empty((proj.shape[0], self.conv_channels), dtype=torch.float32, device=proj.device)
        K.tag = "short conv"
        at = getattr(entry, "state_offset", 0)
        K.short_conv(proj, offset, self.conv_channels, self.taps, self.w_conv, self.b_conv, entry.state, ctx.row_req,
                     ctx.req_start, ctx.req_slot, conv, state_offset=at)
        K.short_conv_commit(proj, offset, self.conv_channels, self.taps, entry.state, ctx.req_start, ctx.req_slot, ctx.n_requests,
                            state_offset=at)
        return conv


@register_part("mixer", "ssd")
class StateSpaceMixer(_StateMixer):
    def __init__(self, spec, prefix, runtime):
        super().__init__(spec, prefix, runtime)
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["heads"])
        self.vdim = int(spec["vdim"])
        self.n_state = int(spec["state"])
        self.groups = int(spec["groups"])
        self.norm_groups = int(spec.get("norm_groups", 1))
        self.taps = int(spec["conv"])
        self.eps = float(spec["eps"])
        self.inner = self.heads * self.vdim
        if self.heads % self.groups != 0:
            raise ValueError(f"heads {self.heads} is not a multiple of groups {self.groups}")
        if self.inner % self.norm_groups != 0:
            raise ValueError(f"heads * vdim = {self.inner} is not a multiple of norm_groups {self.norm_groups}")
        if self.taps < 1:
            raise ValueError(f"conv must be >= 1, found {self.taps}")
        self.conv_channels = self.inner + 2 * self.groups * self.n_state
        self.n_in = 2 * self.inner + 2 * self.groups * self.n_state + self.heads
        self.conv_state = (self.taps - 1) * self.conv_channels
        self.w_in = self.w_conv = self.b_conv = self.dt_bias = self.A_log = self.D = self.w_norm = self.w_o = None

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.conv_state + K.state_scan_floats(self.heads, self.n_state, self.vdim),), torch.float32)

    def params(self) -> Dict[str, ParamSpec]:
        return {
            self.name("in"): ParamSpec((self.n_in, self.hidden)),
            self.name("conv"): ParamSpec((self.conv_channels, self.taps), role="vector", std=0.2),
            self.name("conv.b"): ParamSpec((self.conv_channels,), role="vector"),
            self.name("dt_bias"): ParamSpec((self.heads,), role="vector"),
            self.name("A_log"): ParamSpec((self.heads,), role="vector"),
            self.name("D"): ParamSpec((self.heads,), role="vector", init="ones"),
            self.name("norm"): ParamSpec((self.inner,), role="vector", init="ones"),
            self.name("o"): ParamSpec((self.hidden, self.inner)),
        }

    def load(self, source) -> None:
        for attr, n in (("w_in", "in"), ("w_conv", "conv"), ("b_conv", "conv.b"), ("dt_bias", "dt_bias"), ("A_log", "A_log"),
                        ("D", "D"), ("w_norm", "norm"), ("w_o", "o")):
            setattr(self, attr, self.fetch(source, self.name(n)))

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, entry) -> None:
        rt = self.runtime
        T = x.shape[0]
        gn = self.groups * self.n_state
        proj = torch.empty((T, self.n_in), dtype=torch.float32, device=x.device)
        K.tag = "mixer in"
        project(rt, x, self.w_in, proj)
        conv = self._convolve(proj, self.inner, ctx, entry)
        y = torch.empty((T, self.inner), dtype=torch.float32, device=x.device)
        K.tag = "scan"
        K.state_scan(K.SCAN_SSD, conv, self.inner, self.inner + gn, 0, proj, 2 * self.inner + 2 * gn, 0, self.A_log, self.dt_bias,
                     self.D, entry.state, getattr(entry, "state_offset", 0) + self.conv_state, ctx.req_start, ctx.req_slot, y, ctx.n_requests, self.heads,
                     self.groups, self.n_state, self.vdim)
        gated = torch.empty((T, self.inner), dtype=rt.act_dtype, device=x.device)
        K.tag = "gate + norm"
        K.gated_group_norm(y, self.inner // self.norm_groups, proj, 0, self.w_norm, self.eps, True, gated)
        K.tag = "o"
        project(rt, gated, self.w_o, residual, accumulate=True)
        K.tag = None
        return None


@register_part("mixer", "gated_delta")
class GatedDeltaMixer(_StateMixer):
    def __init__(self, spec, prefix, runtime):
        super().__init__(spec, prefix, runtime)
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["heads"])
        self.kv_heads = int(spec["kv_heads"])
        self.dim = int(spec["dim"])
        self.vdim = int(spec["vdim"])
        self.taps = int(spec["conv"])
        self.eps = float(spec["eps"])
        if self.heads % self.kv_heads != 0:
            raise ValueError(f"heads {self.heads} is not a multiple of kv_heads {self.kv_heads}")
        if self.taps < 1:
            raise ValueError(f"conv must be >= 1, found {self.taps}")
        self.qk = self.kv_heads * self.dim
        self.v = self.heads * self.vdim
        self.conv_channels = 2 * self.qk + self.v
        # one product: q | k | v | a | b | g
        self.n_in = self.conv_channels + 2 * self.heads + self.v
        self.conv_state = (self.taps - 1) * self.conv_channels
        self.b_conv = None
        self.w_in = self.w_conv = self.dt_bias = self.A_log = self.w_norm = self.w_o = None

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.conv_state + K.state_scan_floats(self.heads, self.dim, self.vdim),), torch.float32)

    def params(self) -> Dict[str, ParamSpec]:
        p = {}
        for n, rows in (("q", self.qk), ("k", self.qk), ("v", self.v)):
            p[self.name(n)] = ParamSpec((rows, self.hidden))
            p[self.name(f"{n}.conv")] = ParamSpec((rows, self.taps), role="vector", std=0.2)
        p[self.name("b")] = ParamSpec((self.heads, self.hidden))
        p[self.name("a")] = ParamSpec((self.heads, self.hidden))
        p[self.name("A_log")] = ParamSpec((self.heads,), role="vector")
        p[self.name("dt_bias")] = ParamSpec((self.heads,), role="vector")
        p[self.name("g")] = ParamSpec((self.v, self.hidden))
        p[self.name("norm")] = ParamSpec((self.vdim,), role="vector", init="ones")
        p[self.name("o")] = ParamSpec((self.hidden, self.v))
        return p

    def load(self, source) -> None:
        self.w_in = torch.cat([self.fetch(source, self.name(n)) for n in ("q", "k", "v", "a", "b", "g")], dim=0).contiguous()
        self.w_conv = torch.cat([self.fetch(source, self.name(f"{n}.conv")) for n in ("q", "k", "v")], dim=0).contiguous()
        for attr, n in (("dt_bias", "dt_bias"), ("A_log", "A_log"), ("w_norm", "norm"), ("w_o", "o")):
            setattr(self, attr, self.fetch(source, self.name(n)))

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, entry) -> None:
        rt = self.runtime
        T = x.shape[0]
        C = self.conv_channels
        proj = torch.empty((T, self.n_in), dtype=torch.float32, device=x.device)
        K.tag = "mixer in"
        project(rt, x, self.w_in, proj)
        conv = self._convolve(proj, 0, ctx, entry)
        o = torch.empty((T, self.v), dtype=torch.float32, device=x.device)
        K.tag = "scan"
        K.state_scan(K.SCAN_DELTA, conv, 0, self.qk, 2 * self.qk, proj, C, C + self.heads, self.A_log, self.dt_bias, None,
                     entry.state, getattr(entry, "state_offset", 0) + self.conv_state, ctx.req_start, ctx.req_slot, o, ctx.n_requests, self.heads, self.kv_heads,
                     self.dim, self.vdim, q_scale=float(self.dim) ** -0.5)
        gated = torch.empty((T, self.v), dtype=rt.act_dtype, device=x.device)
        K.tag = "gate + norm"
        K.gated_group_norm(o, self.vdim, proj, C + 2 * self.heads, self.w_norm, self.eps, False, gated)
        K.tag = "o"
        project(rt, gated, self.w_o, residual, accumulate=True)
        K.tag = None
        return None


@register_part("mixer", "gla")
class GatedLinearAttention(_StateMixer):
    def __init__(self, spec, prefix, runtime):
        super().__init__(spec, prefix, runtime)
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["heads"])
        self.dim = int(spec["dim"])
        self.vdim = int(spec["vdim"])
        self.rank = int(spec["decay_rank"])
        self.tau = float(spec["tau"])
        self.eps = float(spec["eps"])
        if self.tau <= 0.0:
            raise ValueError(f"tau must be positive, found {self.tau}")
        self.qk = self.heads * self.dim
        self.v = self.heads * self.vdim
        # one product: q | k | v | g | a1
        self.n_in = 2 * self.qk + 2 * self.v + self.rank
        self.w_in = self.w_a2 = self.b_a2 = self.w_norm = self.w_o = None

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((K.state_scan_floats(self.heads, self.dim, self.vdim, K.SCAN_GLA),), torch.float32)

    def params(self) -> Dict[str, ParamSpec]:
        return {
            self.name("q"): ParamSpec((self.qk, self.hidden)),
            self.name("k"): ParamSpec((self.qk, self.hidden)),
            self.name("v"): ParamSpec((self.v, self.hidden)),
            self.name("g"): ParamSpec((self.v, self.hidden)),
            self.name("a1"): ParamSpec((self.rank, self.hidden)),
            # the decay's second product runs in float32 whatever the engine's dtype: held like a vector
            self.name("a2"): ParamSpec((self.qk, self.rank), role="vector", init="normal", std=0.2),
            self.name("a2.b"): ParamSpec((self.qk,), role="vector", init="normal", std=1.0),
            self.name("norm"): ParamSpec((self.vdim,), role="vector", init="ones"),
            self.name("o"): ParamSpec((self.hidden, self.v)),
        }

    def load(self, source) -> None:
        self.w_in = torch.cat([self.fetch(source, self.name(n)) for n in ("q", "k", "v", "g", "a1")], dim=0).contiguous()
        for attr, n in (("w_a2", "a2"), ("b_a2", "a2.b"), ("w_norm", "norm"), ("w_o", "o")):
            setattr(self, attr, self.fetch(source, self.name(n)))

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, entry) -> None:
        rt = self.runtime
        T = x.shape[0]
        off_g, off_a1 = 2 * self.qk + self.v, 2 * self.qk + 2 * self.v
        proj = torch.empty((T, self.n_in), dtype=torch.float32, device=x.device)
        K.tag = "mixer in"
        project(rt, x, self.w_in, proj)
        z = torch.empty((T, self.qk), dtype=torch.float32, device=x.device)
        K.tag = "decay"
        K.gemm(proj[:, off_a1:], self.w_a2, z, bias=self.b_a2)
        o = torch.empty((T, self.v), dtype=torch.float32, device=x.device)
        K.tag = "scan"
        K.state_scan(K.SCAN_GLA, proj, 0, self.qk, 2 * self.qk, z, 0, 0, None, None, None, entry.state,
                     getattr(entry, "state_offset", 0), ctx.req_start, ctx.req_slot, o, ctx.n_requests, self.heads, self.heads,
                     self.dim, self.vdim, q_scale=float(self.dim) ** -0.5, c0=1.0 / self.tau)
        gated = torch.empty((T, self.v), dtype=rt.act_dtype, device=x.device)
        K.tag = "gate + norm"
        K.gated_group_norm(o, self.vdim, proj, off_g, self.w_norm, self.eps, False, gated)
        K.tag = "o"
        project(rt, gated, self.w_o, residual, accumulate=True)
        K.tag = None
        return None


@register_part("mixer", "mlstm")
class MatrixMemoryMixer(_StateMixer):
    def __init__(self, spec, prefix, runtime):
        super().__init__(spec, prefix, runtime)
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["heads"])
        self.dim = int(spec["dim"])
        self.vdim = int(spec["vdim"])
        self.cap = float(spec["gate_cap"])
        self.floor = float(spec.get("floor", 1e-6))
        self.eps = float(spec["eps"])
        if self.cap <= 0.0:
            raise ValueError(f"gate_cap must be positive, found {self.cap}")
        self.qk = self.heads * self.dim
        self.v = self.heads * self.vdim
        # one product: q | k | v | g | i | f
        self.n_in = 2 * self.qk + 2 * self.v + 2 * self.heads
        self.w_in = self.b_i = self.b_f = self.w_norm = self.w_o = None

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((K.state_scan_floats(self.heads, self.dim, self.vdim, K.SCAN_MLSTM),), torch.float32)

    def params(self) -> Dict[str, ParamSpec]:
        return {
            self.name("q"): ParamSpec((self.qk, self.hidden)),
            self.name("k"): ParamSpec((self.qk, self.hidden)),
            self.name("v"): ParamSpec((self.v, self.hidden)),
            self.name("g"): ParamSpec((self.v, self.hidden)),
            self.name("i"): ParamSpec((self.heads, self.hidden)),
            self.name("i.b"): ParamSpec((self.heads,), role="vector", init="normal", std=1.0),
            self.name("f"): ParamSpec((self.heads, self.hidden)),
            self.name("f.b"): ParamSpec((self.heads,), role="vector", init="normal", std=1.0),
            self.name("norm"): ParamSpec((self.v,), role="vector", init="ones"),
            self.name("o"): ParamSpec((self.hidden, self.v)),
        }

    def load(self, source) -> None:
        self.w_in = torch.cat([self.fetch(source, self.name(n)) for n in ("q", "k", "v", "g", "i", "f")], dim=0).contiguous()
        for attr, n in (("b_i", "i.b"), ("b_f", "f.b"), ("w_norm", "norm"), ("w_o", "o")):
            setattr(self, attr, self.fetch(source, self.name(n)))

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, entry) -> None:
        rt = self.runtime
        T = x.shape[0]
        off_g, off_i = 2 * self.qk + self.v, 2 * self.qk + 2 * self.v
        proj = torch.empty((T, self.n_in), dtype=torch.float32, device=x.device)
        K.tag = "mixer in"
        project(rt, x, self.w_in, proj)
        o = torch.empty((T, self.v), dtype=torch.float32, device=x.device)
        K.tag = "scan"
        K.state_scan(K.SCAN_MLSTM, proj, 0, self.qk, 2 * self.qk, proj, off_i, off_i + self.heads, self.b_f, self.b_i, None,
                     entry.state, getattr(entry, "state_offset", 0), ctx.req_start, ctx.req_slot, o, ctx.n_requests, self.heads,
                     self.heads, self.dim, self.vdim, q_scale=float(self.dim) ** -0.5, c0=self.cap, c1=self.floor)
        gated = torch.empty((T, self.v), dtype=rt.act_dtype, device=x.device)
        K.tag = "gate + norm"
        K.gated_group_norm(o, self.vdim, proj, off_g, self.w_norm, self.eps, False, gated, sigmoid_gate=True)
        K.tag = "o"
        project(rt, gated, self.w_o, residual, accumulate=True)
        K.tag = None
        return None
