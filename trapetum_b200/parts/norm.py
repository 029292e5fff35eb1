"""RMSNorm: ``y = x * rsqrt(mean(x^2) + eps) * (offset + w)``.

``unit_offset`` selects the ``(1 + w)`` form.  The reference adds the 1 to the
stored weights at export (model/export_gemma.py:25-26) and then runs the plain
form (runtime/cuda/codebook_gemv.cu:192-202); here the raw weight is kept and
the sum is made in the kernel in 32-bit.

``scalar`` selects the norm whose weight is ONE number for all coordinates
(stored as a tensor without axes): ``y = x * rsqrt(mean(x^2) + eps) * g``.  The
number is spread over the row once, when the weights are bound, so every kernel
of the vector form serves it.  :meth:`RMSNorm.add_scaled_apply` is the fused form
``h += scale * (a + b); y = norm(h)`` for arrangements whose sublayers read one
normed input and add their outputs together.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from ..weights.loader import TensorSpec
from .base import Norm, register_part


class RMSNorm(Norm):
    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.offset = 1.0 if params.get("unit_offset") else 0.0
        self.scalar = bool(params.get("scalar"))
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        # "norm": drawn around 0 in random mode (the (1 + w) form); "gain": around 1 (a plain weight)
        role = self.params.get("role", "gain" if self.scalar else "norm")
        return {self._name("weight"): TensorSpec(() if self.scalar else (self.size,), role)}

    def bind(self, tensors) -> None:
        self.weight = tensors[self._name("weight")]
        if self.scalar:      # one number for the whole row: spread once, in 32 bits (exact for what a file stores in 16)
            self.weight = self.weight.float().reshape(1).expand(self.size).contiguous()

    def add_scaled_apply(self, h: torch.Tensor, branches, scale: float, out_dtype: torch.dtype) -> torch.Tensor:
        """``h += scale * (sum of the branch outputs)`` in place, returns ``norm(h)``; one kernel."""
        return ops.add_scaled_rmsnorm(h, branches, scale, self.weight, self.eps, self.offset, out_dtype)

    def add_apply(self, h: torch.Tensor, a: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """``h += a`` in place (a branch output that no norm follows), returns ``norm(h)``; one kernel where the branch
        output is 32-bit (a matrix or split-K partial sums)."""
        if a.dtype == torch.float32:
            return ops.add_scaled_rmsnorm(h, [a if a.dim() == 3 else a.contiguous()], 1.0, self.weight, self.eps, self.offset,
                                          out_dtype)
        ops.residual_add(h, a)
        return self.apply(h, out_dtype)

    def kernel_files(self):
        return ("norm",)

    def apply(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps, self.offset, out_dtype)

    def add_to(self, h, a, then, out_dtype):
        if then is None:
            return ops.add_rmsnorm(h, a, self.weight, self.eps, self.offset)
        if isinstance(then, RMSNorm) and then.weight.dtype == self.weight.dtype:
            return ops.add_rmsnorm(h, a, self.weight, self.eps, self.offset,
                                   then.weight, then.eps, then.offset, out_dtype)
        ops.add_rmsnorm(h, a, self.weight, self.eps, self.offset)
        return then.apply(h, out_dtype)


    def fold(self, h, a, alpha, out_dtype):
        return ops.fold_rmsnorm(h, a if a.dim() == 3 else a.contiguous(), self.weight, self.eps, self.offset, alpha, out_dtype)


class LayerNorm(Norm):
    """``y = (x - mean) / sqrt(var + eps) * w + b`` with the variance as the mean of the squared deviations;
    statistics, scale and shift in 32-bit.  Parameters: ``size``, ``eps`` and the tensor names ``weight`` and
    ``bias``.  :meth:`add_apply` is the fused form ``h += a; y = norm(h)`` that an arrangement with unnormed branch
    outputs reads the stream through."""

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self._name("weight"): TensorSpec((self.size,), "gain"), self._name("bias"): TensorSpec((self.size,), "norm")}

    def bind(self, tensors) -> None:
        # two short vectors that enter 32-bit arithmetic: kept in 32 bits (exact for what a file stores in 16)
        self.weight = tensors[self._name("weight")].float().contiguous()
        self.bias = tensors[self._name("bias")].float().contiguous()

    def kernel_files(self):
        return ("layernorm", "norm")

    def apply(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        return ops.add_layernorm(x, None, self.weight, self.bias, self.eps, out_dtype)

    def add_apply(self, h: torch.Tensor, a: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """``h += a`` in place (``a`` a branch output or its split-K partial sums), returns ``norm(h)``."""
        return ops.add_layernorm(h, a, self.weight, self.bias, self.eps, out_dtype)


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "layernorm", LayerNorm)
