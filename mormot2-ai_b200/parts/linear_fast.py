"""The tensor-core path of ``Linear``: bfloat16 operands through ``csrc/gemm_tc.cu``.

Sizes that the kernel does not take (an inner size that is no multiple of 8, operands that
are not 16-byte aligned) go back to the float32 multiply-add kernel.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K


class FastLinear:
    def __init__(self, weight: torch.Tensor, rt, swiglu: bool):
        self.weight, self.rt, self.swiglu = weight, rt, swiglu

    @classmethod
    def maybe(cls, weight: torch.Tensor, rt, swiglu: bool) -> Optional["FastLinear"]:
        if weight.shape[1] % 8 or weight.data_ptr() % 16:
            return None
        return cls(weight, rt, swiglu)

    def deferred(self, a: torch.Tensor):
        """The product with its split sums left pending, or None if this call does not split
        (few tokens and a weight with few row tiles split; see csrc/gemm_tc.cu)."""
        from .linear import Pending
        rt = self.rt
        M, N = a.shape[0], self.weight.shape[0]
        if (a.dtype != torch.bfloat16 or a.stride(0) % 8 or a.data_ptr() % 16 or M > 64
                or -(-N // 128) > rt.sms or rt.pending_bufs is None):
            return None
        # c is only written when the kernel does not split after all
        c = torch.empty((M, N), dtype=torch.float32, device=a.device)
        buf = rt.pending_buf
        splits = K.gemm_tc(a, self.weight, c, False, buf, rt.error_word, rt.sms, defer=True)
        if splits <= 1:
            return Pending(c.unsqueeze(0))
        return Pending(buf[:splits * M * N].view(splits, M, N))

    def __call__(self, a: torch.Tensor, out: Optional[torch.Tensor],
                 add_into: Optional[torch.Tensor]) -> bool:
        """True if the product was done here."""
        if a.dtype != torch.bfloat16 or a.stride(0) % 8 or a.data_ptr() % 16:
            return False
        rt = self.rt
        if self.swiglu:
            K.gemm_tc(a, self.weight, out, False, rt.workspace, rt.error_word, rt.sms, swiglu=True)
            return True
        if add_into is not None:
            K.gemm_tc(a, self.weight, add_into, True, rt.workspace, rt.error_word, rt.sms)
        else:
            K.gemm_tc(a, self.weight, out, False, rt.workspace, rt.error_word, rt.sms)
        return True
