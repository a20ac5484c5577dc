"""Position encodings that an attention mixer can own."""

from __future__ import annotations

import torch

from ..config.rope_scaling import RopeScaling, inverse_frequencies
from ..kernels import ops
from .base import POSITIONS, PositionEncoding


@POSITIONS.register("rotary")
class Rotary(PositionEncoding):
    """Rotary embedding: pair j of every q and k head is turned by pos * inv_freq[j]
    (src/backend/cpu.rs:306-361), the table computed once at load
    (src/config.rs:243-316).  Fused with the cache write in one kernel.

    params: rotary_dim, theta, scaling (RopeScaling), interleaved."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.rotary_dim = int(self._param("rotary_dim"))
        self.interleaved = bool(self._param("interleaved"))
        scaling = self._param("scaling")
        if not isinstance(scaling, RopeScaling):
            scaling = RopeScaling.from_json(scaling)
        table = inverse_frequencies(self.rotary_dim, float(self._param("theta")), scaling)
        self.inv_freq = torch.from_numpy(table).to(runtime.device)

    def write_qk(self, qkv, step, kv, num_heads, num_kv_heads, head_dim, write_kv):
        ops.rope_kv_write(
            qkv, step.tok_pos, step.tok_seq,
            kv.block_table if write_kv else None, kv.k_pages if write_kv else None, kv.v_pages if write_kv else None,
            self.inv_freq, num_heads, num_kv_heads, head_dim, self.rotary_dim, self.interleaved, write_kv=write_kv,
        )

    def rotate(self, q, k, step):
        raise NotImplementedError("Rotary encodes positions inside write_qk")

    def decode_fusion(self):
        if self.rotary_dim % 8:  # the fused kernel moves a pair's halves between lanes in steps of four values
            return None
        return self.inv_freq, self.rotary_dim, self.interleaved


@POSITIONS.register("none")
class NoPosition(PositionEncoding):
    """No position signal: keys and values are stored as they are."""

    def rotate(self, q, k, step):
        return None

    def decode_fusion(self):
        return None, 0, False
