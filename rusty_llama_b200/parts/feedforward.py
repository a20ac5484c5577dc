"""Dense feed-forward parts."""

from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..errors import ConfigError
from ..kernels import ops
from ..kernels.linear import linear, linear_swiglu, linear_to_stream
from .base import FEED_FORWARDS, FeedForward, ParamInfo


@FEED_FORWARDS.register("gated_mlp")
class GatedMLP(FeedForward):
    """f = W_down (act(W_gate x) * (W_up x)) with act = silu: Llama's SwiGLU
    (src/model.rs:1336-1345, src/backend/cpu.rs:435-440).

    params: hidden_size, intermediate_size, activation ("silu").
    tensors: <prefix>gate_proj.weight [ff, d], up_proj.weight [ff, d], down_proj.weight [d, ff].
    gate and up are kept as one [2 ff, d] matrix so that one product serves both, the
    counterpart of the reference's `matmul_shared` (src/backend/mod.rs:44-56).  In bfloat16 their
    rows alternate (gate i, up i, gate i+1, ...), which lets the product's kernel apply the
    activation to its 32-bit sums and write h directly; in 32-bit the halves follow each other
    and a separate kernel applies the activation."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.d = int(self._param("hidden_size"))
        self.ff = int(self._param("intermediate_size"))
        if self._param("activation") != "silu":
            raise ConfigError(f"gated_mlp: activation '{self._param('activation')}' is not built (only 'silu')")
        self.w_gate_up = None
        self.w_down = None

    def param_infos(self) -> Dict[str, ParamInfo]:
        p = self.prefix
        return {
            p + "gate_proj.weight": ParamInfo((self.ff, self.d)),
            p + "up_proj.weight": ParamInfo((self.ff, self.d)),
            p + "down_proj.weight": ParamInfo((self.d, self.ff)),
        }

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        p = self.prefix
        gate, up = tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"]
        self.fused = self.rt.dtype == torch.bfloat16
        if self.fused:
            self.w_gate_up = torch.stack([gate, up], dim=1).reshape(2 * self.ff, self.d).contiguous()
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = tensors[p + "down_proj.weight"].contiguous()

    def gated_weights(self):
        return (self.w_gate_up, self.w_down) if self.fused else None

    def forward(self, xn: torch.Tensor, step) -> torch.Tensor:
        if self.fused:
            h = linear_swiglu(xn, self.w_gate_up)
        else:
            h = ops.swiglu(linear(xn, self.w_gate_up))
        return linear_to_stream(h, self.w_down)
