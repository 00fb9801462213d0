"""Norm parts: the RMS norm and Dynamic Tanh.

``ss = sum x_i^2; scale = 1 / sqrt(ss / dim + eps); y_i = x_i * scale * w_i`` with the
statistics in float32 (model/Prim.cajeta:120-151; weight and eps held per norm,
model/RMSNorm.cajeta:14-53).  Parameters: ``dim``, ``eps``, ``weight_name`` (the weight's
tensor name under the part's prefix, default ``weight``; empty: the prefix itself), ``offset``
(optional: the stored weight lies around zero and ``offset + w`` multiplies, so 1 for a ``1 + w`` norm;
the sum is formed once at load, in float32).

``dyt``: Dynamic Tanh, a norm that takes no statistic of the row: ``y_i = tanh(alpha x_i) w_i + b_i`` with a scalar
``alpha`` and a bias stored beside the weight.  Parameters: ``dim``, ``weight_name`` (as above), ``alpha_name`` and
``bias_name`` (suffixes added to the weight's tensor name, defaults ``.alpha`` and ``.b``).

Both offer ``add_normed(hs, y)``: the norm of a sublayer's result added into the residual stream in one kernel, which
the blocks that norm a sublayer's OUTPUT call.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..csrc import kernels as K
from .base import Part, register_part
from .plan import ParamSpec


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    def __init__(self, spec, prefix, runtime):
        super().__init__(spec, prefix, runtime)
        self.dim = int(spec["dim"])
        self.eps = float(spec["eps"])
        self.weight_name = self.name(spec.get("weight_name", "weight"))
        self.offset = float(spec.get("offset", 0.0) or 0.0)
        self.weight: Optional[torch.Tensor] = None

    def params(self) -> Dict[str, ParamSpec]:
        return {self.weight_name: ParamSpec((self.dim,), role="vector", init="normal" if self.offset else "ones")}

    def libraries(self) -> set:
        return {"rowwise"}

    def load(self, source) -> None:
        self.weight = self.fetch(source, self.weight_name)
        if self.offset:
            self.weight = (self.weight + self.offset).contiguous()

    def forward(self, x: torch.Tensor, want_f32: bool = False, row_index: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None, pending: Optional[torch.Tensor] = None,
                want_split: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """Normalise rows of the float32 residual stream.

        Returns the result in the activation dtype and, when ``want_f32``, also in
        float32 (the same tensor on the 32-bit path).  ``row_index`` (int32) picks the
        rows to normalise.  ``pending`` ([S, rows, dim] float32) are partial sums still
        owed to the residual stream by the part before: they are added to ``x`` (in
        order, ``x`` keeps the sum) in the same pass.  ``want_split`` (instead of
        ``want_f32``): the second result is bfloat16 ``[rows, 3 * dim]``, the float32 value
        as three bfloat16 terms hi | mid | lo whose sum is the value to 2^-24 - the form a
        tensor-core product needs to give float32-grade sums."""
        rt = self.runtime
        rows = x.shape[0] if row_index is None else row_index.numel()
        dtype = out_dtype or rt.act_dtype
        out = torch.empty((rows, self.dim), dtype=dtype, device=x.device)
        out_f32 = None
        if want_split:
            split = torch.empty((rows, 3 * self.dim), dtype=torch.bfloat16, device=x.device)
            K.rmsnorm(x, self.weight, self.eps, out, None, row_index, pending, out_split=split)
            return out, split
        if want_f32:
            out_f32 = out if dtype == torch.float32 else torch.empty((rows, self.dim), dtype=torch.float32, device=x.device)
        K.rmsnorm(x, self.weight, self.eps, out, out_f32 if out_f32 is not out else None, row_index, pending)
        return out, out_f32

    def add_normed(self, hs: torch.Tensor, y: torch.Tensor) -> None:
        """``hs += norm(y)``, float32, one kernel."""
        K.rmsnorm_add(hs, y, self.weight, self.eps)


@register_part("norm", "dyt")
class DynamicTanh(Part):
    def __init__(self, spec, prefix, runtime):
        super().__init__(spec, prefix, runtime)
        self.dim = int(spec["dim"])
        self.weight_name = self.name(spec.get("weight_name", "weight"))
        self.alpha_name = self.weight_name + str(spec.get("alpha_name", ".alpha"))
        self.bias_name = self.weight_name + str(spec.get("bias_name", ".b"))
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None
        self.alpha = 1.0

    def params(self) -> Dict[str, ParamSpec]:
        return {self.weight_name: ParamSpec((self.dim,), role="vector", init="ones"),
                self.bias_name: ParamSpec((self.dim,), role="vector", std=0.05),
                self.alpha_name: ParamSpec((), role="vector", init="ones")}

    def libraries(self) -> set:
        return {"rowwise"}

    def load(self, source) -> None:
        self.weight = self.fetch(source, self.weight_name)
        self.bias = self.fetch(source, self.bias_name)
        # a scalar of the file: read once, handed to the kernels by value
        self.alpha = float(self.fetch(source, self.alpha_name).reshape(-1)[0].item())

    def forward(self, x: torch.Tensor, want_f32: bool = False, row_index: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None, pending: Optional[torch.Tensor] = None,
                want_split: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """The rows of the float32 residual stream through ``tanh(alpha x) w + b``; results as the RMS norm's."""
        rt = self.runtime
        rows = x.shape[0] if row_index is None else row_index.numel()
        dtype = out_dtype or rt.act_dtype
        out = torch.empty((rows, self.dim), dtype=dtype, device=x.device)
        if want_split:
            split = torch.empty((rows, 3 * self.dim), dtype=torch.bfloat16, device=x.device)
            K.dyt(x, self.weight, self.bias, self.alpha, out, None, row_index, pending, out_split=split)
            return out, split
        out_f32 = None
        if want_f32:
            out_f32 = out if dtype == torch.float32 else torch.empty((rows, self.dim), dtype=torch.float32, device=x.device)
        K.dyt(x, self.weight, self.bias, self.alpha, out, out_f32 if out_f32 is not out else None, row_index, pending)
        return out, out_f32

    def add_normed(self, hs: torch.Tensor, y: torch.Tensor) -> None:
        """``hs += tanh(alpha y) w + b``, float32, one kernel."""
        K.dyt_add(hs, y, self.weight, self.bias, self.alpha)
