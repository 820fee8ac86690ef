"""RMSNorm: y = w · x / sqrt(mean(x²) + eps), the weight multiplying as it is (not 1 + w);
sums in float32 (``backend.cpu.pas:1769-1795``, ``ops.cu:116-130`` of the reference)."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels as K
from .base import NORMS, Part, TensorNeed


class RmsNorm(Part):
    capturable = True
    accepts_pending = True      # forward(..., pending=) adds split sums into x before it norms

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.name = prefix + spec.params["name"]
        self.weight: Optional[torch.Tensor] = None

    def tensors(self) -> List[TensorNeed]:
        return [TensorNeed(self.name, (self.size,), "vector")]

    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        self.weight = weights[self.name]
        self.rt = rt

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None,
                n_rows: Optional[int] = None, pending=None) -> torch.Tensor:
        """x: the float32 residual [T, size]. ``rows``: only these rows are normed (gathered).
        ``pending``: the split sums of the product before (``parts/linear.py: Pending``), which
        are first added into x."""
        R = n_rows if n_rows is not None else (rows.numel() if rows is not None else x.shape[0])
        out = torch.empty((R, self.size), dtype=self.rt.dtype, device=x.device)
        K.rmsnorm(x, self.weight, self.eps, out, rows, R,
                  pending.partial if pending is not None else None)
        return out


NORMS.register("rmsnorm", RmsNorm)
