"""RMSNorm, fused with the residual sum that precedes it."""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..kernels import ops
from .base import NORMS, Norm, ParamInfo, ResidualStream


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """y = x / sqrt(mean(x^2) + eps) * weight (src/backend/cpu.rs:96-105).

    params: size, eps.  tensor: <prefix>weight [size]."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.size = int(self._param("size"))
        self.eps = float(self._param("eps"))
        self.weight: Optional[torch.Tensor] = None

    def param_infos(self) -> Dict[str, ParamInfo]:
        return {self.prefix + "weight": ParamInfo((self.size,), "vector")}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.prefix + "weight"]

    def rms_weight(self):
        return self.weight, self.eps

    def forward(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        delta, stream.pending = stream.pending, None
        return ops.add_rmsnorm(
            stream.x, delta, self.weight, self.eps, stream.act_dtype, rows=rows, write_x=rows is None
        )
