"""Mixers made of other mixers.

``side_by_side``: two mixers read the same input; each result is RMS-normed over the model width with a plain
weight of its own and the two are averaged (``coef`` = 1/2) or summed (``coef`` = 1):
``y = coef (left / rms(left) * w_left + right / rms(right) * w_right)``, statistics and sum in float32.
Parameters: ``hidden_size``, ``eps``, ``coef`` (default 0.5), ``left`` / ``right`` (mixer PartSpecs),
``left_name`` / ``right_name`` (their tensor-name prefixes under this part's), ``left_out`` / ``right_out`` (the
tensor names of the two weights).  At most one of the two may cache keys and values (the entry's cache plane is
that one's); both may keep per-request state: the entry's state vector holds the left one's share first, then the
right one's, and each finds its own at ``entry.state_offset``.  ``overlap`` (default true): on a CUDA device the left
mixer runs on a side stream while the right one runs on the step's.
"""
from __future__ import annotations

from dataclasses import replace
from typing import Dict, Optional

import torch

from ..csrc import kernels as K
from .base import Part, StateNeed, make_part, register_part
from .plan import ParamSpec


@register_part("mixer", "side_by_side")
class SideBySide(Part):
    def __init__(self, spec, prefix, runtime):
        super().__init__(spec, prefix, runtime)
        self.hidden = int(spec["hidden_size"])
        self.eps = float(spec["eps"])
        self.coef = float(spec.get("coef", 0.5))
        self.left = make_part("mixer", spec["left"], self.name(spec.get("left_name", "left")), runtime)
        self.right = make_part("mixer", spec["right"], self.name(spec.get("right_name", "right")), runtime)
        self.n_left_out = self.name(spec.get("left_out", "left.out"))
        self.n_right_out = self.name(spec.get("right_out", "right.out"))
        if self.left.cache_need() is not None and self.right.cache_need() is not None:
            raise ValueError("side_by_side: only one of the two mixers may cache keys and values")
        for m in (self.left, self.right):
            if hasattr(m, "allow_pending"):
                m.allow_pending = False        # no norm follows that would add partial sums: each adds its own result
        self.graph_safe = all(getattr(m, "graph_safe", m.state_need() is None) for m in (self.left, self.right))
        self.capture_max_rows = min(int(getattr(m, "capture_max_rows", 1 << 30)) for m in (self.left, self.right))
        need = self.left.state_need()
        self.left_state = int(need.shape[0]) if need is not None else 0
        self.w_left = self.w_right = None
        # ``overlap`` (default true): the two mixers run on two streams
        self.overlap = bool(spec.get("overlap", True))
        self._side = None

    def cache_need(self):
        return self.left.cache_need() or self.right.cache_need()

    def state_need(self) -> Optional[StateNeed]:
        total = 0
        for m in (self.left, self.right):
            need = m.state_need()
            if need is not None:
                if need.dtype != torch.float32 or len(need.shape) != 1:
                    raise ValueError("side_by_side: the mixers' states must be flat float32 vectors")
                total += int(need.shape[0])
        return StateNeed((total,), torch.float32) if total else None

    def params(self) -> Dict[str, ParamSpec]:
        p = {self.n_left_out: ParamSpec((self.hidden,), role="vector", init="ones"),
             self.n_right_out: ParamSpec((self.hidden,), role="vector", init="ones")}
        p.update(self.left.params())
        p.update(self.right.params())
        return p

    def libraries(self) -> set:
        return {"recurrent"} | self.left.libraries() | self.right.libraries()

    def load(self, source) -> None:
        self.left.load(source)
        self.right.load(source)
        self.w_left = self.fetch(source, self.n_left_out)
        self.w_right = self.fetch(source, self.n_right_out)

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, entry) -> None:
        base = getattr(entry, "state_offset", 0)
        a = torch.zeros(residual.shape, dtype=torch.float32, device=residual.device)
        b = torch.zeros(residual.shape, dtype=torch.float32, device=residual.device)
        left_entry = replace(entry, state_offset=base)
        right_entry = replace(entry, state_offset=base + self.left_state)
        if self.overlap and residual.is_cuda:
            # the two halves share nothing but their input: the left one runs on a stream of its own beside the right
            # one (their shares of the state vector and the cache planes are apart), and both are back before the
            # norms read them.  What the left half allocates is its stream's and is freed to it; x, a and b are the
            # step's stream's, which waits for the side stream before anything of them is given back.  A step that
            # is being captured records the fork and the join as the graph's branches.
            main = torch.cuda.current_stream()
            if self._side is None:
                self._side = torch.cuda.Stream(device=residual.device)
            self._side.wait_stream(main)
            with torch.cuda.stream(self._side):
                self.left.forward(x, a, ctx, left_entry)
            self.right.forward(x, b, ctx, right_entry)
            main.wait_stream(self._side)
        else:
            self.left.forward(x, a, ctx, left_entry)
            self.right.forward(x, b, ctx, right_entry)
        K.tag = "norm + mix"
        K.rmsnorm_mix2(a, self.w_left, b, self.w_right, self.eps, self.coef, residual, accumulate=True)
        K.tag = None
        return None
