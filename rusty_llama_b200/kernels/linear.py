"""y = x . W^T for the model's projections, chosen by precision and row count.

float32 runs use the library's own 32-bit kernel for every shape.  bfloat16
runs use the library's weight-streaming kernel for up to 64 rows (a decode
step) and, above that, the vendor GEMM through torch.matmul: the reference does
the same split, its own GEMV kernels for decode and cuBLASLt for prompts
(src/backend/cuda.rs:717-758, :354-442).
"""

from __future__ import annotations

from typing import Optional

import torch

from ..errors import KernelError
from . import ops


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
    M = x.shape[0]
    if M <= ops.GEMV_MAX_ROWS:
        return ops.gemv_bf16(x, w, out_dtype)
    if out_dtype == torch.bfloat16:
        if not x.is_cuda:
            raise KernelError("linear: tensors must be on a CUDA device")
        return torch.matmul(x, w.t())
    # float32 results of many rows (logits of every position of a prompt): keep the
    # 32-bit accumulator's value by going through the streaming kernel in groups of rows
    out = torch.empty((M, w.shape[0]), dtype=out_dtype, device=x.device)
    for r0 in range(0, M, ops.GEMV_MAX_ROWS):
        r1 = min(M, r0 + ops.GEMV_MAX_ROWS)
        ops.gemv_bf16(x[r0:r1], w, out_dtype, out=out[r0:r1])
    return out
