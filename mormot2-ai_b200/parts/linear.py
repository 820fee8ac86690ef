"""y = x · Wᵀ for a weight [out, in] without bias (``backend.pas:63-68`` of the reference),
with the epilogue fused: store, add into the float32 residual, or SwiGLU over gate and up.

The kernel is chosen by the operand types and sizes: the tensor-core kernels for bfloat16
operands whose sizes they take, else the float32 multiply-add kernel, which takes every size
and every mix of types (a weight stored in 32 bits stays so and is multiplied in 32 bits).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K


class Pending:
    """Partial sums [splits, M, N] (float32) of a product whose K range was split: whoever
    reads the result next adds them up, in split order (an RMSNorm adds them into the residual
    it norms, the q/k norm kernel adds them as it reads q, k and v). They live in one of two
    buffers of the runtime that are used in turn, so at most two products are pending at a
    time."""

    def __init__(self, partial: torch.Tensor):
        self.partial = partial


class Linear:
    def __init__(self, weight: torch.Tensor, rt, swiglu: bool = False):
        """``swiglu``: the weight is [2 * out, in] with rows that alternate gate and up (row 2i
        the gate, row 2i + 1 the up projection of output i) and the product is followed by
        out = silu(gate) * up in the kernel's epilogue."""
        self.weight = weight.contiguous()
        self.rt = rt
        self.swiglu = swiglu
        self.out_features = weight.shape[0] // (2 if swiglu else 1)
        self.in_features = weight.shape[1]
        self.fast = None
        if rt.fast_kernels and weight.dtype == torch.bfloat16 and rt.dtype == torch.bfloat16:
            from .linear_fast import FastLinear
            self.fast = FastLinear.maybe(self.weight, rt, swiglu)

    def __call__(self, a: torch.Tensor, out: Optional[torch.Tensor] = None,
                 add_into: Optional[torch.Tensor] = None,
                 out_dtype: Optional[torch.dtype] = None, defer: bool = False):
        """``add_into``: the float32 residual [M, out] that the product is added to (returned).
        Otherwise the product (or its SwiGLU) is stored in ``out`` (made if None). ``defer``: if
        the kernel splits K, a ``Pending`` with the partial sums is returned instead and neither
        ``out`` nor ``add_into`` is touched."""
        M = a.shape[0]
        if self.fast is not None and defer and not self.swiglu:
            pending = self.fast.deferred(a)
            if pending is not None:
                return pending
        if add_into is None and out is None:
            out = torch.empty((M, self.out_features), dtype=out_dtype or self.rt.dtype,
                              device=a.device)
        if self.fast is not None and self.fast(a, out, add_into):
            return add_into if add_into is not None else out
        if add_into is not None:
            K.gemm_simt(a, self.weight, add_into, K.EPI_ADD)
            return add_into
        K.gemm_simt(a, self.weight, out, K.EPI_SWIGLU_PAIRS if self.swiglu else K.EPI_STORE)
        return out
