"""Token embedding and the classifier."""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..kernels import ops
from ..kernels.linear import linear
from .base import EMBEDDINGS, HEADS, ParamInfo, Part, ResidualStream


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Part):
    """x = E[token], a row copy without scale (src/model.rs:1237-1242), widened to the 32-bit stream.

    params: vocab_size, hidden_size.  tensor: <prefix>weight [V, d]."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.vocab_size = int(self._param("vocab_size"))
        self.d = int(self._param("hidden_size"))
        self.weight: Optional[torch.Tensor] = None

    def param_infos(self) -> Dict[str, ParamInfo]:
        return {self.prefix + "weight": ParamInfo((self.vocab_size, self.d))}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.prefix + "weight"]

    def forward(self, tokens: torch.Tensor) -> ResidualStream:
        return ResidualStream(ops.embed_gather(tokens, self.weight), self.rt.dtype)


@HEADS.register("linear_head")
class LinearHead(Part):
    """logits = W xn in 32-bit (src/model.rs:1366); `tied_to` names the embedding
    tensor that serves as W when the model has no classifier of its own (src/model.rs:469-473).

    params: vocab_size, hidden_size, tied_to (a tensor name or None)."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.vocab_size = int(self._param("vocab_size"))
        self.d = int(self._param("hidden_size"))
        self.tied_to = self._param("tied_to")
        self.weight: Optional[torch.Tensor] = None

    def weight_name(self) -> str:
        return self.tied_to or (self.prefix + "weight")

    def param_infos(self) -> Dict[str, ParamInfo]:
        return {self.weight_name(): ParamInfo((self.vocab_size, self.d))}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name()]

    def forward(self, xn: torch.Tensor) -> torch.Tensor:
        return linear(xn, self.weight, out_dtype=torch.float32)
