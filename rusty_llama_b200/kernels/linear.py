"""y = x . W^T for the model's projections, chosen by precision and row count.

float32 runs use the library's own 32-bit FMA kernel for every shape.  bfloat16 runs use the
persistent TMA-fed streaming kernel for up to 8 rows (a decode step; the older register-streaming
kernel where k is no multiple of 64) and the TMA + tcgen05 kernel above that (a prompt step).  The
reference makes the same split, its own GEMV kernels for decode and a cuBLASLt call for prompts
(src/backend/cuda.rs:354-442, :717-758); `use_library_gemm(True)` puts the vendor GEMM
(torch.matmul) in the place of the tcgen05 kernel, for comparisons only.  Those kernels move rows in
16-byte pieces; a product whose k is no multiple of 8, or whose rows do not start on 16 bytes, goes to a
plain FMA kernel instead (slow, but every size that a configuration allows has to run).
"""

from __future__ import annotations

from typing import Optional

import torch

from ..errors import KernelError
from . import ops
from .device import sm_count

_library_gemm = False

# Rows up to which the weight-streaming kernel is used.  Above it every warp of that kernel re-reads
# the activations for its 16 features and the L1/L2 traffic, not HBM, sets the pace; the tcgen05
# kernel stages the activations in shared memory once per tile and streams weights at HBM rate.
STREAM_MAX_ROWS = 8


def _streams(M: int, K: int, whole: bool) -> bool:
    """Whether the persistent streaming kernel takes the product; whole: only with all of k in one
    slice (the result goes on as it is, not as partial sums)."""
    slices = ops.gemv_stream_slices(M, K, 1)
    return slices == 1 or (slices > 1 and not whole)


def _odd(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the operands' rows cannot be moved in 16-byte pieces."""
    return bool(
        x.shape[1] % 8 or x.stride(0) % 8 or w.stride(0) % 8 or x.data_ptr() % 16 or w.data_ptr() % 16
    )


def use_library_gemm(on: bool) -> None:
    """Route bfloat16 products of more than 64 rows through torch.matmul instead of `gemm_tc`."""
    global _library_gemm
    _library_gemm = bool(on)


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """x[M, K] (dense rows), w[N, K] -> [M, N] in `out_dtype` (default: x's dtype)."""
    if out_dtype is None:
        out_dtype = x.dtype
    if x.dtype == torch.float32:
        if w.dtype != torch.float32 or out_dtype != torch.float32:
            raise KernelError(f"linear: a float32 input needs float32 weights and output, got {w.dtype}, {out_dtype}")
        return ops.gemm_f32(x, w)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"linear: unsupported dtypes {x.dtype} x {w.dtype}")
    M, K = x.shape
    if _odd(x, w):
        return ops.gemm_bf16_any(x, w, out_dtype)
    if M <= STREAM_MAX_ROWS:
        if _streams(M, K, whole=True):
            return ops.gemv_stream(x, w, out_dtype)
        return ops.gemv_bf16(x, w, out_dtype)
    if M <= 32 and ((M + 127) // 128) * ((w.shape[0] + 255) // 256) < sm_count(x.device) // 2:
        # too few output tiles to keep the SMs busy, and nothing downstream that could add up
        # partial sums: the streaming kernel's many small blocks still win here (measured)
        return ops.gemv_bf16(x, w, out_dtype)
    if _library_gemm and out_dtype == torch.bfloat16 and x.is_cuda:
        return torch.matmul(x, w.t())
    return ops.gemm_tc(x, w, out_dtype)


def linear_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """h[M, ff] = silu(x . Wg^T) * (x . Wu^T) in one kernel, for bfloat16.

    w_gate_up[2 ff, K] holds the rows of Wg and Wu alternately (row 2i is gate i, row 2i + 1 is up i);
    the product's 32-bit sums go through the activation before anything is rounded or stored."""
    if x.dtype != torch.bfloat16 or w_gate_up.dtype != torch.bfloat16:
        raise KernelError(f"linear_swiglu: bfloat16 only, got {x.dtype} x {w_gate_up.dtype}")
    if _odd(x, w_gate_up):
        return ops.gemm_bf16_any(x, w_gate_up, torch.bfloat16, swiglu=True)
    if x.shape[0] <= STREAM_MAX_ROWS:
        if _streams(x.shape[0], x.shape[1], whole=True):
            return ops.gemv_stream(x, w_gate_up, torch.bfloat16, swiglu=True)
        return ops.gemv_bf16(x, w_gate_up, torch.bfloat16, swiglu=True)
    return ops.gemm_tc(x, w_gate_up, torch.bfloat16, swiglu=True)


# resident blocks of the register-streaming kernel per SM: its splits of k aim at filling the GPU once
_STREAM_BLOCKS_PER_SM = 6


def linear_to_stream(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """A projection whose result is added to the residual stream (attention output, feed-forward
    down projection).  In bfloat16, when the output alone gives the GPU too few blocks (a decode
    step, a short prompt), the k range is split and the float32 partial sums [parts, M, N] are
    returned, which the next norm's kernel adds up in 32-bit; otherwise the same as `linear`."""
    M, K = x.shape
    N = w.shape[0]
    if x.dtype != torch.bfloat16 or _odd(x, w):
        return linear(x, w)
    if M <= STREAM_MAX_ROWS and _streams(M, K, whole=False):
        # as few slices of k as the kernel allows (each costs a partial result to write and to add)
        if ops.gemv_stream_slices(M, K, 1) > 1:
            return ops.gemv_stream(x, w, torch.float32, k_splits=2)
        return ops.gemv_stream(x, w)
    if M <= STREAM_MAX_ROWS and K <= 8192:
        # (for a long k the tcgen05 kernel below is faster even at one row: 25 us against 32 us
        # for the 8B down projection)
        blocks = (N + 15) // 16
        target = _STREAM_BLOCKS_PER_SM * sm_count(x.device)
        splits = min((target + blocks - 1) // blocks, 8, max(1, K // 1024))
        if splits > 1:
            return ops.gemv_bf16(x, w, torch.float32, k_splits=splits)
        return ops.gemv_bf16(x, w)
    if _library_gemm:
        return linear(x, w)
    sms = sm_count(x.device)
    if 32 < M <= 128:
        # One row of tiles (a decode step of 33 to 128 sequences): tiles of 128 columns with half as many slices of k
        # take the same time as tiles of 256 (measured at 64 rows: QKV 12.9 against 14.0 us, output 10.3 against
        # 10.1, down 24.5 against 24.5) and leave half the partial sums for the next kernel to add up (a layer of a
        # decode step: 254 against 258 us at 64 sequences, 395 against 408 at 128; at 16 sequences it loses 2 %).
        # Only where that still gives most SMs a unit of work: with the short k of the 1.1B sizes it does not (32 units
        # of 16 k slices each), and a layer at 64 sequences took 71 instead of 66 us.
        tiles = (N + 127) // 128
        splits = min(sms // tiles, 8, max(1, K // 1024)) if tiles <= sms // 2 else 1
        if splits > 1 and tiles * splits * 5 >= sms * 4:
            return ops.gemm_tc(x, w, torch.float32, k_splits=splits, tile_n=128)
    tiles = ((M + 127) // 128) * ((N + 255) // 256)
    splits = min(sms // tiles, 8, max(1, K // 512)) if tiles <= sms // 2 else 1
    if splits > 1:
        return ops.gemm_tc(x, w, torch.float32, k_splits=splits)
    return ops.gemm_tc(x, w)
