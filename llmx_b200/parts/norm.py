"""Norms.  RMSNorm: y = x * (rsqrt(mean(x^2) + eps) * w), 32-bit arithmetic.

The weight is the plain `w` (not `1 + w`), as the reference computes this
architecture (src/backends/cpu/cpu_backend.hpp:1437-1459).  `one_plus=True` is the
norm of designs that store the weight around zero: y = x * rsqrt(...) * (1 + w);
the sum 1 + w is made once at load, in 32-bit.  `role` names the weight's tensor
("" names it by the part's prefix alone).
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch

from .. import runtime
from ..weights.spec import TensorSpec
from .base import NativeHandle, Part, Precision
from .linear import bare_step


class RMSNorm(Part):
    def __init__(self, width: int, eps: float, role: str = "weight", one_plus: bool = False):
        self.width, self.eps, self.role, self.one_plus = int(width), float(eps), role, bool(one_plus)
        self.weight: Optional[torch.Tensor] = None
        self._native: Optional[NativeHandle] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        if self.one_plus:
            return {self.role: TensorSpec((self.width,), "vector", init="normal", std=0.05)}
        return {self.role: TensorSpec((self.width,), "vector", init="one_plus_normal", std=0.01)}

    def load(self, tensors, precision: Precision) -> None:
        super().load(tensors, precision)
        self.weight = tensors[self.role].to(torch.float32).contiguous()
        if self.one_plus:
            self.weight = (self.weight + 1.0).contiguous()
        self._native = None

    @property
    def native(self) -> int:
        if self._native is None:
            runtime.need("rowwise")
            self._native = NativeHandle(runtime.lib().llmx_rmsnorm_create(self.weight.data_ptr(), self.width, self.eps,
                                                                         runtime.code(self.precision.act)), keep=(self.weight,))
        return self._native.handle

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                row_index: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
                zero: Optional[torch.Tensor] = None) -> torch.Tensor:
        """`zero`: a float32 buffer the part that follows wants cleared; the norm's launch clears it on the way."""
        rows = x.shape[0] if row_index is None else row_index.numel()
        if out is None:
            out = torch.empty((rows, self.width), dtype=out_dtype or self.precision.act, device=x.device)
        if not (x.is_cuda and x.dtype is torch.float32 and x.is_contiguous() and x.dim() == 2 and x.shape[1] == self.width
                and out.is_contiguous() and tuple(out.shape) == (rows, self.width)
                and (row_index is not None or x.shape[0] >= rows)
                and (row_index is None or (row_index.dtype is torch.int32 and row_index.is_contiguous()))
                and (zero is None or (zero.dtype is torch.float32 and zero.numel() % 4 == 0 and zero.is_contiguous()))):
            raise runtime.KernelError("rmsnorm: float32 rows of the norm's width, an output of as many rows, int32 row_index")
        s = bare_step(x.device)
        runtime.check(runtime.lib().llmx_norm_forward(self.native, ctypes.byref(s), x.data_ptr(), out.data_ptr(), runtime.code(out.dtype),
                                                      runtime.ptr(row_index), rows, runtime.ptr(zero),
                                                      0 if zero is None else zero.numel()), "rmsnorm")
        return out


class GroupedRMSNorm(Part):
    """RMS norm in groups: the row is split into `groups` equal consecutive parts, each divided by its own
    sqrt(mean(part^2) + eps), and the whole is multiplied by the weight; 32-bit arithmetic (csrc/rowwise.cu,
    `llmx_group_norm_conv`).  The same interface as RMSNorm (one group is the plain RMS norm); it has no twin in the native
    runtime.  `forward_filtered` also gives the normed rows plus a short causal filter of them over the request's rows
    (what a block hands to its mixer when the design filters the mixer's input), in the same launch."""

    def __init__(self, width: int, eps: float, groups: int = 1, role: str = "weight"):
        if groups < 1 or width % groups:
            raise ValueError("grouped norm: the groups must divide the width")
        self.width, self.eps, self.groups, self.role = int(width), float(eps), int(groups), role
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.role: TensorSpec((self.width,), "vector", init="one_plus_normal", std=0.01)}

    def load(self, tensors, precision: Precision) -> None:
        super().load(tensors, precision)
        self.weight = tensors[self.role].to(torch.float32).contiguous()

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                row_index: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
                zero: Optional[torch.Tensor] = None) -> torch.Tensor:
        from .. import ops
        rows = x.shape[0] if row_index is None else row_index.numel()
        if out is None:
            out = torch.empty((rows, self.width), dtype=out_dtype or self.precision.act, device=x.device)
        if zero is not None and (zero.numel() % 4 or zero.data_ptr() % 16):
            zero.zero_()
            zero = None
        return ops.group_norm_conv(x, self.weight, self.eps, self.groups, out, row_index=row_index, zero=zero)

    def forward_filtered(self, x: torch.Tensor, taps_w: torch.Tensor, state: torch.Tensor, step, zero: Optional[torch.Tensor] = None,
                         state_off: int = 0):
        """(h, h + filter(h)): `taps_w` float32 [taps, width]; the filter's earlier inputs lie in `state` at `state_off`."""
        from .. import ops
        rows = x.shape[0]
        both = torch.empty((2, rows, self.width), dtype=self.precision.act, device=x.device)
        if zero is not None and (zero.numel() % 4 or zero.data_ptr() % 16):
            zero.zero_()
            zero = None
        ops.group_norm_conv(x, self.weight, self.eps, self.groups, both[0], zero=zero, taps_w=taps_w, filtered=both[1],
                            state=state, step=step, state_off=state_off)
        return both[0], both[1]


class LayerNorm(Part):
    """y = (x - mean(x)) / sqrt(var(x) + eps) * w (+ b), var the mean of squared deviations; 32-bit arithmetic
    (csrc/rowwise.cu, `llmx_layernorm_affine`).  `role`: the weight's tensor role ("" names it by the part's prefix
    alone); `bias`: the role of a bias tensor, or None for a norm without one.  The same interface as RMSNorm; it has no
    twin in the native runtime, so a block that holds it is walked from Python.  `add_into(residual, y, factor)`
    norms y and adds factor times the result into the float32 residual in one kernel (the norm after a sublayer)."""

    def __init__(self, width: int, eps: float, role: str = "weight", bias: Optional[str] = None):
        self.width, self.eps, self.role, self.bias_role = int(width), float(eps), role, bias
        if bias is not None and bias == role:
            raise ValueError("layer norm: weight and bias need different roles")
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = {self.role: TensorSpec((self.width,), "vector", init="one_plus_normal", std=0.01)}
        if self.bias_role is not None:
            specs[self.bias_role] = TensorSpec((self.width,), "vector", init="normal", std=0.02)
        return specs

    def load(self, tensors, precision: Precision) -> None:
        super().load(tensors, precision)
        self.weight = tensors[self.role].to(torch.float32).contiguous()
        self.bias = tensors[self.bias_role].to(torch.float32).contiguous() if self.bias_role is not None else None

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                row_index: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
                zero: Optional[torch.Tensor] = None) -> torch.Tensor:
        from .. import ops
        rows = x.shape[0] if row_index is None else row_index.numel()
        if out is None:
            out = torch.empty((rows, self.width), dtype=out_dtype or self.precision.act, device=x.device)
        if zero is not None and (zero.numel() % 4 or zero.data_ptr() % 16):
            zero.zero_()
            zero = None
        return ops.layernorm(x, self.weight, self.eps, out, row_index, zero, bias=self.bias)

    def add_into(self, residual: torch.Tensor, y: torch.Tensor, factor: float, in_bias: Optional[torch.Tensor] = None) -> None:
        """residual += factor * norm(y + in_bias); float32 rows."""
        from .. import ops
        ops.layernorm_add_(residual, y, self.weight, self.bias, self.eps, factor, in_bias=in_bias)
