"""Block arrangements: how a layer's mixer, feed-forward and norms are wired.

``prenorm``: ``hs += mixer(norm_1(hs)); hs += feed_forward(norm_2(hs))`` with the
residual stream ``hs`` in float32 (model/DecoderLayer.cajeta:38-75,
model/CausalLM.cajeta:1445-1446,1506,1512-1517,1575).  Parameters: the tensor-name
pieces ``mixer_norm_name``, ``feed_forward_norm_name``, ``mixer_name``,
``feed_forward_name`` under the layer's prefix.

``outnorm``: the norm sits on each sublayer's OUTPUT and the sublayers read the stream
itself: ``hs += norm_1(mixer(hs)); hs += norm_2(feed_forward(hs))``.  A layer may have no
feed-forward (``LayerSpec.feed_forward`` is None).  The sublayers see ``hs`` rounded to
the activation dtype (a feed-forward that wants its input exactly gets the float32 stream
itself); each adds its result into a zeroed float32 buffer of the stream's shape, which one
kernel norms and adds.  Same parameters as ``prenorm``.

``parallel``: one norm, both sublayers read its output: ``h = norm(hs); hs += mixer(h) + feed_forward(h)``
(each adds its result into the float32 stream).  A layer may have no feed-forward.  After the
sublayers the layer's ``stream_after`` part, when it has one, runs on the stream.  Parameters:
``mixer_norm_name``, ``mixer_name``, ``feed_forward_name``, ``stream_after_name``.

``sandwich``: a norm before AND after each sublayer: ``hs += norm_1b(mixer(c(norm_1(hs))))``,
``hs += norm_2b(feed_forward(norm_2(hs)))``; a layer may have no feed-forward.  ``c`` is an optional causal
convolution over time on the mixer's input (``input_conv``: ``{"taps": n, "name": tensor}``):
``c(h)_t = h_t + sum_j w[:, j] h_(t - taps + 1 + j)`` per channel, rows before a request's first token read as zeros, weights
``[hidden, taps]``; it runs in float32 on the float32 normed row, and the last ``taps - 1`` normed rows of a
request are per-request state.  The block therefore declares state itself (``state_need()``): the
convolution's share first, then the mixer's, which the mixer finds at ``entry.state_offset``.  Parameters:
``mixer_norm_name``, ``mixer_post_norm_name``, ``feed_forward_norm_name``, ``feed_forward_post_norm_name``,
``mixer_name``, ``feed_forward_name``, ``input_conv``, ``hidden_size``.  The post norms are the layer's norm
specs (``mixer_norm`` / ``feed_forward_norm``) under their own names; any norm kind that offers ``add_normed(hs, y)``
(the RMS norm, Dynamic Tanh) serves.
"""
from __future__ import annotations

from dataclasses import replace
from typing import Dict, Optional

import torch

from ..csrc import kernels as K
from .base import Part, StateNeed, make_part, register_part
from .plan import LayerSpec, ParamSpec


@register_part("block", "prenorm")
class PreNormBlock(Part):
    def __init__(self, spec, prefix, runtime, layer: LayerSpec):
        super().__init__(spec, prefix, runtime)
        self.mixer_norm = make_part("norm", layer.mixer_norm, self.name(spec["mixer_norm_name"]), runtime)
        self.mixer = make_part("mixer", layer.mixer, self.name(spec["mixer_name"]), runtime)
        self.feed_forward_norm = make_part("norm", layer.feed_forward_norm, self.name(spec["feed_forward_norm_name"]), runtime)
        self.feed_forward = make_part("feed_forward", layer.feed_forward, self.name(spec["feed_forward_name"]), runtime)

    def parts(self):
        return (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)

    def params(self) -> Dict[str, ParamSpec]:
        out: Dict[str, ParamSpec] = {}
        for p in self.parts():
            out.update(p.params())
        return out

    def libraries(self) -> set:
        out = set()
        for p in self.parts():
            out |= p.libraries()
        return out

    def load(self, source) -> None:
        for p in self.parts():
            p.load(source)

    def forward(self, hs: torch.Tensor, ctx, entry) -> None:
        x, _ = self.mixer_norm.forward(hs)
        # a mixer may return partial sums it still owes the residual stream ([S, rows, H]
        # float32, from a product split along K); the next norm adds them as it reads hs
        pending = self.mixer.forward(x, hs, ctx, entry)
        # the feed-forward may want its input once more in float32 (a router), or, for many
        # rows, as three bfloat16 terms that a tensor-core product can sum to the same grade
        ff = self.feed_forward
        wants_split = getattr(ff, "wants_split_input", None)
        split = bool(wants_split and wants_split(hs.shape[0]))
        x, x_exact = self.feed_forward_norm.forward(hs, want_f32=getattr(ff, "needs_f32_input", False) and not split,
                                                    pending=pending, want_split=split)
        ff.forward(x, x_exact, hs, ctx)


@register_part("block", "outnorm")
class OutputNormBlock(Part):
    def __init__(self, spec, prefix, runtime, layer: LayerSpec):
        super().__init__(spec, prefix, runtime)
        self.mixer_norm = make_part("norm", layer.mixer_norm, self.name(spec["mixer_norm_name"]), runtime)
        self.mixer = make_part("mixer", layer.mixer, self.name(spec["mixer_name"]), runtime)
        self.feed_forward = self.feed_forward_norm = None
        if layer.feed_forward is not None:
            self.feed_forward_norm = make_part("norm", layer.feed_forward_norm, self.name(spec["feed_forward_norm_name"]), runtime)
            self.feed_forward = make_part("feed_forward", layer.feed_forward, self.name(spec["feed_forward_name"]), runtime)
        for n in (self.mixer_norm, self.feed_forward_norm):
            if n is not None and not (hasattr(n, "weight") and hasattr(n, "eps")):
                raise ValueError("an outnorm block takes norms that are a weight and an eps (rmsnorm)")

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward) if p is not None)

    def params(self) -> Dict[str, ParamSpec]:
        out: Dict[str, ParamSpec] = {}
        for p in self.parts():
            out.update(p.params())
        return out

    def libraries(self) -> set:
        out = {"recurrent"}
        for p in self.parts():
            out |= p.libraries()
        return out

    def load(self, source) -> None:
        for p in self.parts():
            p.load(source)

    def _input(self, hs: torch.Tensor) -> torch.Tensor:
        rt = self.runtime
        if rt.act_dtype == torch.float32:
            return hs
        x = torch.empty(hs.shape, dtype=rt.act_dtype, device=hs.device)
        K.tag = "cast"
        K.cast_rows(hs, x)
        return x

    def _add_normed(self, hs: torch.Tensor, y: torch.Tensor, pending, norm) -> None:
        if pending is not None:
            y += pending.sum(dim=0)
        K.tag = "norm + add"
        K.rmsnorm_add(hs, y, norm.weight, norm.eps)
        K.tag = None

    def forward(self, hs: torch.Tensor, ctx, entry) -> None:
        y = torch.zeros_like(hs)
        pending = self.mixer.forward(self._input(hs), y, ctx, entry)
        self._add_normed(hs, y, pending, self.mixer_norm)
        ff = self.feed_forward
        if ff is None:
            return
        y = torch.zeros_like(hs)
        ff.forward(self._input(hs), hs if getattr(ff, "needs_f32_input", False) else None, y, ctx)
        self._add_normed(hs, y, None, self.feed_forward_norm)


@register_part("block", "parallel")
class ParallelBlock(Part):
    def __init__(self, spec, prefix, runtime, layer: LayerSpec):
        super().__init__(spec, prefix, runtime)
        self.mixer_norm = make_part("norm", layer.mixer_norm, self.name(spec["mixer_norm_name"]), runtime)
        self.mixer = make_part("mixer", layer.mixer, self.name(spec["mixer_name"]), runtime)
        self.feed_forward = None
        if layer.feed_forward is not None:
            self.feed_forward = make_part("feed_forward", layer.feed_forward, self.name(spec["feed_forward_name"]), runtime)
        self.after = None
        if layer.stream_after is not None:
            self.after = make_part("stream", layer.stream_after, self.name(spec.get("stream_after_name", "")), runtime)

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.feed_forward, self.after) if p is not None)

    def params(self) -> Dict[str, ParamSpec]:
        out: Dict[str, ParamSpec] = {}
        for p in self.parts():
            out.update(p.params())
        return out

    def libraries(self) -> set:
        out = {"stream_ops"}
        for p in self.parts():
            out |= p.libraries()
        return out

    def load(self, source) -> None:
        for p in self.parts():
            p.load(source)

    def forward(self, hs: torch.Tensor, ctx, entry) -> None:
        ff = self.feed_forward
        wants_split = getattr(ff, "wants_split_input", None)
        split = bool(wants_split and wants_split(hs.shape[0]))
        x, x_exact = self.mixer_norm.forward(hs, want_f32=getattr(ff, "needs_f32_input", False) and not split, want_split=split)
        # partial sums a mixer still owes the stream (its output product cut along K for few rows): no norm
        # follows inside this block that could add them while it reads the row, so a kernel of its own does
        pending = self.mixer.forward(x, hs, ctx, entry)
        if pending is not None:
            K.tag = "o (partial sums)"
            K.add_partials(hs, pending)
            K.tag = None
        if ff is not None:
            ff.forward(x, x_exact, hs, ctx)
        if self.after is not None:
            self.after.forward(hs, ctx)


@register_part("block", "sandwich")
class SandwichBlock(Part):
    def __init__(self, spec, prefix, runtime, layer: LayerSpec):
        super().__init__(spec, prefix, runtime)
        self.hidden = int(spec["hidden_size"])
        self.mixer_norm = make_part("norm", layer.mixer_norm, self.name(spec["mixer_norm_name"]), runtime)
        self.mixer_post_norm = make_part("norm", layer.mixer_norm, self.name(spec["mixer_post_norm_name"]), runtime)
        self.mixer = make_part("mixer", layer.mixer, self.name(spec["mixer_name"]), runtime)
        if hasattr(self.mixer, "allow_pending"):
            self.mixer.allow_pending = False       # the mixer's result is normed before it is added: no partial sums
        self.feed_forward = self.feed_forward_norm = self.feed_forward_post_norm = None
        if layer.feed_forward is not None:
            self.feed_forward_norm = make_part("norm", layer.feed_forward_norm, self.name(spec["feed_forward_norm_name"]), runtime)
            self.feed_forward_post_norm = make_part("norm", layer.feed_forward_norm, self.name(spec["feed_forward_post_norm_name"]), runtime)
            self.feed_forward = make_part("feed_forward", layer.feed_forward, self.name(spec["feed_forward_name"]), runtime)
        for n in (self.mixer_post_norm, self.feed_forward_post_norm):
            if n is not None and not hasattr(n, "add_normed"):
                raise ValueError("a sandwich block takes post norms that can norm a sublayer's result into the stream (add_normed)")
        conv = dict(spec.get("input_conv") or {})
        self.taps = int(conv.get("taps", 1)) if conv else 1
        self.conv_name = self.name(conv["name"]) if conv else None
        if self.taps < 1:
            raise ValueError(f"input_conv.taps must be >= 1, found {self.taps}")
        self.conv_state = (self.taps - 1) * self.hidden if conv else 0
        self.w_conv = None
        self.graph_safe = getattr(self.mixer, "graph_safe", self.mixer.state_need() is None)

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.mixer_post_norm, self.feed_forward_norm, self.feed_forward,
                                 self.feed_forward_post_norm) if p is not None)

    def state_need(self) -> Optional[StateNeed]:
        need = self.mixer.state_need()
        if need is None:
            return StateNeed((self.conv_state,), torch.float32) if self.conv_state else None
        if not self.conv_state:
            return need
        if need.dtype != torch.float32 or len(need.shape) != 1:
            raise ValueError("sandwich: behind an input convolution the mixer's state must be a flat float32 vector")
        return StateNeed((self.conv_state + int(need.shape[0]),), torch.float32)

    def params(self) -> Dict[str, ParamSpec]:
        out: Dict[str, ParamSpec] = {}
        for p in self.parts():
            out.update(p.params())
        if self.conv_name:
            out[self.conv_name] = ParamSpec((self.hidden, self.taps), role="vector", std=0.2)
        return out

    def libraries(self) -> set:
        out = {"recurrent"}
        for p in self.parts():
            out |= p.libraries()
        return out

    def load(self, source) -> None:
        for p in self.parts():
            p.load(source)
        if self.conv_name:
            # h + conv(h) as ONE convolution: the newest tap's weight plus one (exact in float32 for weights that
            # came from 16-bit storage; else the sum rounds once, as h + w h would)
            w = self.fetch(source, self.conv_name).clone()
            w[:, self.taps - 1] += 1.0
            self.w_conv = w.contiguous()

    def _mixer_input(self, hs: torch.Tensor, ctx, entry) -> torch.Tensor:
        rt = self.runtime
        if not self.conv_name:
            x, _ = self.mixer_norm.forward(hs)
            return x
        h, _ = self.mixer_norm.forward(hs, out_dtype=torch.float32)
        x = torch.empty(h.shape, dtype=rt.act_dtype, device=hs.device)
        K.tag = "input conv"
        K.short_conv(h, 0, self.hidden, self.taps, self.w_conv, None, entry.state, ctx.row_req, ctx.req_start, ctx.req_slot, x,
                     activate=False, state_offset=entry.state_offset)
        K.short_conv_commit(h, 0, self.hidden, self.taps, entry.state, ctx.req_start, ctx.req_slot, ctx.n_requests,
                            state_offset=entry.state_offset)
        K.tag = None
        return x

    def forward(self, hs: torch.Tensor, ctx, entry) -> None:
        x = self._mixer_input(hs, ctx, entry)
        y = torch.zeros_like(hs)
        inner = replace(entry, state_offset=entry.state_offset + self.conv_state) if self.conv_state else entry
        pending = self.mixer.forward(x, y, ctx, inner)
        if pending is not None:
            y += pending.sum(dim=0)
        K.tag = "norm + add"
        self.mixer_post_norm.add_normed(hs, y)
        K.tag = None
        ff = self.feed_forward
        if ff is None:
            return
        wants_split = getattr(ff, "wants_split_input", None)
        split = bool(wants_split and wants_split(hs.shape[0]))
        x, x_exact = self.feed_forward_norm.forward(hs, want_f32=getattr(ff, "needs_f32_input", False) and not split, want_split=split)
        y = torch.zeros_like(hs)
        ff.forward(x, x_exact, y, ctx)
        K.tag = "norm + add"
        self.feed_forward_post_norm.add_normed(hs, y)
        K.tag = None
