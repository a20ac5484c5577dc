"""Causal grouped-query attention over the paged cache."""

from __future__ import annotations

import math
from typing import Dict, Mapping

import torch

from ..errors import ConfigError
from ..kernels import ops
from ..kernels.device import sm_count
from ..kernels.linear import linear, linear_to_stream
from ..spec import PartSpec
from .base import MIXERS, POSITIONS, KVNeed, Mixer, ParamInfo

# one-warp blocks of the decode kernel that an SM holds at once (four at head size 128, its shared
# memory's limit): measured best when the splits fill the GPU once and no more
_DECODE_BLOCKS_PER_SM = 4
_DECODE_HEADS_PER_BLOCK = 8


# the four-warp kernel for head sizes 64 and 128: two blocks per SM; a split shorter than four pages costs
# more in the merge than it gains (measured at one sequence of 4096: 16 splits 7.5 us, 37 splits 8.8)
_QKV_PARTIALS_MAX_ROWS = 128
_DECODE_TMA_BLOCKS_PER_SM = 2
_DECODE_TMA_MIN_PAGES = 4


def decode_splits(n_seqs: int, num_heads: int, num_kv_heads: int, kv_len: int, head_dim: int = 0, sms: int = 0) -> int:
    """How many pieces to cut the key range into, from shapes only (head_dim tells which of the two
    decode kernels will run; sms: the GPU's multiprocessors, asked from the current device if 0)."""
    sms = sms or sm_count()
    group = num_heads // num_kv_heads
    per_split = n_seqs * num_kv_heads * ((group + _DECODE_HEADS_PER_BLOCK - 1) // _DECODE_HEADS_PER_BLOCK)
    tiles = max(1, (kv_len + ops.PAGE_SIZE - 1) // ops.PAGE_SIZE)
    if head_dim in ops.ATTN_DECODE_TMA_HEAD_DIMS:
        want = _DECODE_TMA_BLOCKS_PER_SM * sms // per_split
        return max(1, min(want, (tiles + _DECODE_TMA_MIN_PAGES - 1) // _DECODE_TMA_MIN_PAGES, 64))
    want = _DECODE_BLOCKS_PER_SM * sms // per_split
    return max(1, min(want, tiles, 64))


@MIXERS.register("attention")
class Attention(Mixer):
    """q = Wq xn, k = Wk xn, v = Wv xn; positions encoded into q and k; k, v stored in the
    cache; each query attends to its sequence's keys up to its own position (all of
    them, or the last `window`); the heads' results go through Wo
    (src/model.rs:1253-1301, src/backend/cpu.rs:363-433).  Query head h reads kv head
    h // (H / K); the score scale is 1/sqrt(head_dim).

    params: hidden_size, num_heads, num_kv_heads, head_dim, window (0 = all keys),
            position (a PartSpec of the position family).
    tensors: <prefix>q_proj.weight [H hd, d], k_proj.weight [K hd, d], v_proj.weight [K hd, d],
             o_proj.weight [d, H hd].  q, k, v are kept as one matrix so that one product
             serves the three (src/backend/cuda.rs:423-442)."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.d = int(self._param("hidden_size"))
        self.H = int(self._param("num_heads"))
        self.K = int(self._param("num_kv_heads"))
        self.hd = int(self._param("head_dim"))
        self.window = int(self._param("window"))
        if self.H % self.K:
            raise ConfigError(f"attention: {self.H} heads are not a multiple of {self.K} kv heads")
        if self.hd > 256:
            raise ConfigError(f"attention: head_dim {self.hd} is above 256, the most the attention kernels built here take")
        if self.hd % 8 and runtime.dtype != torch.float32:
            raise ConfigError(
                f"attention: the bfloat16 kernels move a head in 16-byte pieces and need head_dim to be a multiple of 8, got {self.hd} "
                f"(a float32 run takes any head size up to 256)")
        pos_spec = self._param("position")
        if not isinstance(pos_spec, PartSpec):
            raise ConfigError("attention: 'position' must be a PartSpec")
        self.position = POSITIONS.build(pos_spec, runtime)
        self.scale = 1.0 / math.sqrt(self.hd)
        self.qd, self.kvd = self.H * self.hd, self.K * self.hd
        self.w_qkv = None
        self.w_o = None

    def cache_need(self):
        return KVNeed(self.K, self.hd, self.window)

    def children(self):
        return (self.position,)

    def param_infos(self) -> Dict[str, ParamInfo]:
        p = self.prefix
        return {
            p + "q_proj.weight": ParamInfo((self.qd, self.d)),
            p + "k_proj.weight": ParamInfo((self.kvd, self.d)),
            p + "v_proj.weight": ParamInfo((self.kvd, self.d)),
            p + "o_proj.weight": ParamInfo((self.d, self.qd)),
        }

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        p = self.prefix
        self.w_qkv = torch.cat(
            [tensors[p + "q_proj.weight"], tensors[p + "k_proj.weight"], tensors[p + "v_proj.weight"]], dim=0
        ).contiguous()
        self.w_o = tensors[p + "o_proj.weight"].contiguous()

    def forward(self, xn: torch.Tensor, step, cache, shared_cache: bool = False) -> torch.Tensor:
        a, w_o = self.forward_unprojected(xn, step, cache, shared_cache)
        return linear_to_stream(a, w_o)

    def forward_unprojected(self, xn: torch.Tensor, step, cache, shared_cache: bool = False):
        # a decode step of a bfloat16 run at head size 64 or 128: the attention kernel turns the queries and the
        # new key and stores key and value itself, if the position encoding is one it knows how to apply
        fusion = None
        if step.decode_only and self.rt.dtype == torch.bfloat16 and self.hd in ops.ATTN_DECODE_TMA_HEAD_DIMS:
            fusion = self.position.decode_fusion()
        # the keys and values may be another run's: then only the queries are projected.  The fused attention
        # kernel also takes the projection as partial sums over slices of k, which lets a product with few
        # output tiles use all SMs (measured at the 8B sizes: 3 % of the step gained at 16, 24 and 64 sequences)
        w = self.w_qkv[: self.qd] if shared_cache else self.w_qkv
        qkv = linear_to_stream(xn, w) if (fusion is not None and xn.shape[0] <= _QKV_PARTIALS_MAX_ROWS) else linear(xn, w)
        if fusion is None:
            self.position.write_qk(qkv, step, cache, self.H, self.K, self.hd, write_kv=not shared_cache)
        if self.rt.dtype == torch.float32:
            a = ops.attn_generic(
                qkv, cache.k_pages, cache.v_pages, cache.block_table, step.tok_seq, step.tok_pos,
                self.H, self.K, self.hd, window=self.window, scale=self.scale,
            )
        elif step.decode_only:
            n_splits = decode_splits(step.n_seqs, self.H, self.K, step.plan_kv_len, self.hd)
            scratch = self.rt.workspace.get(
                "attn_decode", ops.attn_decode_scratch_floats(step.n_seqs, self.H, self.hd, n_splits), torch.float32
            )
            # With one split per sequence the attention kernel writes the result itself.  With more, a
            # second kernel adds the splits up: letting the block that finishes last do that (the kernel
            # can) measured slower at batch 1 and 8 (its serial tail costs more than the small kernel).
            counters = None
            if self.hd in ops.ATTN_DECODE_TMA_HEAD_DIMS and n_splits == 1:
                groups = self.K * ((self.H // self.K + _DECODE_HEADS_PER_BLOCK - 1) // _DECODE_HEADS_PER_BLOCK)
                counters = self.rt.workspace.get("attn_decode_counters", step.n_seqs * groups, torch.int32, zeroed=True)
            a = ops.attn_decode(
                qkv, cache.k_pages, cache.v_pages, cache.block_table, step.seq_len, self.H, self.K, self.hd,
                n_splits, scratch, window=self.window, scale=self.scale, counters=counters,
                **({} if fusion is None else dict(
                    fuse=1 if shared_cache else 2, inv_freq=fusion[0], rotary_dim=fusion[1], interleaved=fusion[2])),
            )
        elif self.hd in ops.FLASH_TC_HEAD_DIMS:
            a = ops.flash_prefill_tc(
                qkv, cache.k_pages, cache.v_pages, cache.block_table, step.seq_start, step.seq_pos0,
                step.max_q_len, self.H, self.K, self.hd, window=self.window, scale=self.scale,
            )
        else:
            a = ops.flash_prefill(
                qkv, cache.k_pages, cache.v_pages, cache.block_table, step.seq_start, step.seq_pos0,
                step.max_q_len, self.H, self.K, self.hd, window=self.window, scale=self.scale,
            )
        return a, self.w_o
