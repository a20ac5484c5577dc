"""Arrangements of a layer's parts."""

from __future__ import annotations

import os

import torch

from ..kernels import ops
from ..kernels.linear import STREAM_MAX_ROWS, linear_to_stream
from .base import BLOCKS, Block, ResidualStream


def _fold_enabled() -> bool:
    return os.environ.get("RL_FOLD_NORM", "1") != "0"


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    """x += mixer(norm_m(x)); x += feed_forward(norm_f(x)) (src/model.rs:1244-1357).

    Each sum is left pending on the stream and performed by the next norm's
    kernel, the following layer's or the model's final one.

    A decode step of up to 8 sequences in bfloat16 folds the second norm into the products around it where
    the parts allow it: if the mixer ends in a projection that it can leave to the caller, the norm is an RMSNorm
    and the feed-forward a gated one with fused weights, then the projection's kernel adds its sums to the stream
    itself, writes x * w beside it and leaves the rows' sums of squares, and the gate/up kernel multiplies its sums
    by the rows' 1 / sqrt(mean(x^2) + eps) before the activation: the norm's own kernel, with its pass over the
    stream, is not launched.  The parts are asked, not named: any mixer, norm or feed-forward that answers
    `forward_unprojected`, `rms_weight` and `gated_weights` takes part.  RL_FOLD_NORM=0 in the environment turns
    this off."""

    def forward(self, stream: ResidualStream, step, cache, shared_cache: bool = False) -> None:
        xn = self.norms["mixer"].forward(stream)
        if self._folded(stream, xn, step, cache, shared_cache):
            return
        stream.add(self.mixer.forward(xn, step, cache, shared_cache))
        xn = self.norms["feed_forward"].forward(stream)
        stream.add(self.feed_forward.forward(xn, step))

    def _folded(self, stream: ResidualStream, xn, step, cache, shared_cache: bool) -> bool:
        if not (step.decode_only and self.rt.dtype == torch.bfloat16 and xn.shape[0] <= STREAM_MAX_ROWS and xn.is_cuda and _fold_enabled()):
            return False
        norm, gated = self.norms["feed_forward"].rms_weight(), self.feed_forward.gated_weights()
        if norm is None or gated is None:
            return False
        (w_norm, eps), (w_gate_up, w_down) = norm, gated
        d = stream.x.shape[1]
        if w_gate_up.dtype != torch.bfloat16 or w_gate_up.shape[1] != d or w_norm.shape[0] != d:
            return False
        unprojected = self.mixer.forward_unprojected(xn, step, cache, shared_cache)
        if unprojected is None:
            return False
        a, w_o = unprojected
        M, k = a.shape
        ok = (a.dtype == torch.bfloat16 and w_o.dtype == torch.bfloat16 and tuple(w_o.shape) == (d, k)
              and ops.gemv_stream_slices(M, k, 1) == 1 and ops.gemv_stream_slices(M, d, 1) == 1
              and not (a.stride(0) % 8 or w_o.stride(0) % 8 or w_gate_up.stride(0) % 8 or a.data_ptr() % 16))
        if not ok:
            # the attention has run; finish the layer the plain way
            stream.add(linear_to_stream(a, w_o))
            xn = self.norms["feed_forward"].forward(stream)
            stream.add(self.feed_forward.forward(xn, step))
            return True
        ws = self.rt.workspace
        xw = ws.get("fold_xw", M * d, torch.bfloat16)[: M * d].view(M, d)
        sumsq = ws.get("fold_sumsq", 8 * 1024, torch.float32)
        xw, sumsq, blocks = ops.gemv_stream_into_stream(a, w_o, stream.x, w_norm, xw=xw, sumsq=sumsq)
        h = ops.gemv_stream(xw, w_gate_up, torch.bfloat16, swiglu=True, row_scale=(sumsq, blocks, d, eps))
        stream.add(linear_to_stream(h, w_down))
        return True
