"""The kernels as Python functions on torch tensors.

Each function checks what the kernel cannot check for itself (device, dtype,
contiguity, sizes that index arithmetic relies on), passes raw pointers and the
current stream to the launcher and raises KernelError when the launcher refuses
or the launch fails.  Nothing here computes with torch: if the extension cannot
be built or loaded, every call fails.
"""

from __future__ import annotations

import ctypes
import math
from typing import Optional, Sequence

import torch

from ..errors import KernelError
from . import build

PAGE_SIZE = 64  # tokens per cache page; the attention kernels' key tile

_F32, _BF16 = 0, 1
_DT = {torch.float32: _F32, torch.bfloat16: _BF16}

c_int, c_ll, c_float, c_void_p = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p


def _dt(t: torch.Tensor, what: str) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"{what}: dtype {t.dtype} is neither float32 nor bfloat16") from None


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _cuda(t: torch.Tensor, what: str, dtype=None, contiguous=True) -> torch.Tensor:
    _need(isinstance(t, torch.Tensor), f"{what}: not a tensor")
    _need(t.is_cuda, f"{what}: tensor is on {t.device}, the kernels run on CUDA only")
    if dtype is not None:
        _need(t.dtype == dtype, f"{what}: dtype {t.dtype}, expected {dtype}")
    if contiguous:
        _need(t.is_contiguous(), f"{what}: tensor is not contiguous")
    return t


def _rows(t: torch.Tensor, what: str) -> int:
    """Row stride of a 2-D tensor whose rows are dense."""
    _need(t.dim() == 2 and t.stride(1) == 1, f"{what}: expected a 2-D tensor with dense rows")
    return t.stride(0)


def _p(t: Optional[torch.Tensor]):
    return c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


_launches = 0


def launch_count() -> int:
    """Kernels of this library launched so far in this process (replayed graph nodes included)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(lib, rc: int, name: str, kernels: int = 1) -> None:
    global _launches
    _launches += kernels
    if rc != 0:
        text = lib.rl_error_text().decode("utf-8", "replace")
        kind = "refused its arguments" if rc < 0 else f"failed to launch (CUDA error {rc})"
        raise KernelError(f"{name} {kind}: {text}")


# ------------------------------------------------------------------ row kernels
def embed_gather(tokens: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = table[tokens[t]] as float32.  Token ids must already be known to lie in the table."""
    _cuda(tokens, "embed_gather tokens", torch.int32)
    _cuda(table, "embed_gather table")
    _need(tokens.dim() == 1 and table.dim() == 2, "embed_gather: tokens[T] and table[V, d] expected")
    T, d = tokens.numel(), table.shape[1]
    if out is None:
        out = torch.empty((T, d), dtype=torch.float32, device=table.device)
    _cuda(out, "embed_gather out", torch.float32)
    _need(tuple(out.shape) == (T, d), "embed_gather: out has the wrong shape")
    _need(table.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0, "embed_gather: tensors must be 16-byte aligned")
    lib = build.load("elementwise")
    rc = lib.rl_embed_gather(_p(tokens), _p(table), c_int(_dt(table, "embed_gather table")), _p(out), c_int(T), c_int(d), _stream())
    _check(lib, rc, "embed_gather")
    return out


def add_rmsnorm(
    x: torch.Tensor,
    delta: Optional[torch.Tensor],
    weight: Optional[torch.Tensor],
    eps: float,
    act_dtype: torch.dtype,
    rows: Optional[torch.Tensor] = None,
    write_x: bool = True,
    out: Optional[torch.Tensor] = None,
) -> Optional[torch.Tensor]:
    """x (float32 [T, d]) += sum of delta parts; returns rmsnorm(x) * weight in `act_dtype`.

    delta: None, [T, d] or [parts, T, d], in `act_dtype` or in float32 (partial sums of a product
    split over k).  weight None: only the sum.
    rows: int32 indices of the rows to produce (all rows if None).
    """
    _cuda(x, "add_rmsnorm x", torch.float32)
    _need(x.dim() == 2, "add_rmsnorm: x must be [T, d]")
    T, d = x.shape
    n_parts, part_stride = 0, 0
    delta_dt = _DT[act_dtype]
    if delta is not None:
        _cuda(delta, "add_rmsnorm delta")
        _need(delta.dtype in (act_dtype, torch.float32), f"add_rmsnorm: delta is {delta.dtype} in a run of {act_dtype}")
        delta_dt = _DT[delta.dtype]
        if delta.dim() == 2:
            _need(tuple(delta.shape) == (T, d), f"add_rmsnorm: delta {tuple(delta.shape)} does not match x {(T, d)}")
            n_parts = 1
        else:
            _need(delta.dim() == 3 and tuple(delta.shape[1:]) == (T, d), f"add_rmsnorm: delta {tuple(delta.shape)} does not match x {(T, d)}")
            n_parts, part_stride = delta.shape[0], T * d
    n_rows = T
    if rows is not None:
        _cuda(rows, "add_rmsnorm rows", torch.int32)
        n_rows = rows.numel()
    w_dt = _F32
    if weight is not None:
        _cuda(weight, "add_rmsnorm weight")
        _need(tuple(weight.shape) == (d,), f"add_rmsnorm: weight {tuple(weight.shape)} does not match d={d}")
        w_dt = _dt(weight, "add_rmsnorm weight")
        if out is None:
            out = torch.empty((n_rows, d), dtype=act_dtype, device=x.device)
        _cuda(out, "add_rmsnorm out", act_dtype)
        _need(tuple(out.shape) == (n_rows, d), "add_rmsnorm: out has the wrong shape")
    else:
        _need(delta is not None, "add_rmsnorm: neither a delta nor a weight, nothing to do")
        out = None
    if n_rows == 0:
        return out
    for name, t in (("x", x), ("delta", delta), ("weight", weight), ("out", out)):
        _need(t is None or t.data_ptr() % 16 == 0, f"add_rmsnorm: {name} is not 16-byte aligned")
    lib = build.load("elementwise")
    rc = lib.rl_add_rmsnorm(
        _p(x), _p(delta), c_int(delta_dt), c_int(n_parts), c_ll(part_stride), _p(weight), c_int(w_dt), _p(out),
        c_int(_DT[act_dtype]), _p(rows), c_int(n_rows), c_int(d), c_float(eps), c_int(1 if write_x else 0), _stream(),
    )
    _check(lib, rc, "add_rmsnorm")
    return out


def swiglu(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """h[t, i] = silu(gate_up[t, i]) * gate_up[t, ff + i]."""
    _cuda(gate_up, "swiglu input")
    _need(gate_up.dim() == 2 and gate_up.shape[1] % 2 == 0, "swiglu: input must be [T, 2*ff]")
    T, ff = gate_up.shape[0], gate_up.shape[1] // 2
    if out is None:
        out = torch.empty((T, ff), dtype=gate_up.dtype, device=gate_up.device)
    _cuda(out, "swiglu out", gate_up.dtype)
    _need(tuple(out.shape) == (T, ff), "swiglu: out has the wrong shape")
    lib = build.load("elementwise")
    rc = lib.rl_swiglu(_p(gate_up), _p(out), c_int(_dt(gate_up, "swiglu")), c_int(T), c_int(ff), _stream())
    _check(lib, rc, "swiglu")
    return out


# ------------------------------------------------------------------ per-sequence records
SEQ_FIELDS = 4  # a record: positions held, tokens decoded, the most it may decode, flags
SEQ_LEN, SEQ_DECODED, SEQ_MAX_NEW, SEQ_FLAGS = 0, 1, 2, 3


def seq_begin_decode(state: torch.Tensor, slot_ids: torch.Tensor, tok_pos: torch.Tensor, seq_pos0: torch.Tensor, seq_len: torch.Tensor) -> None:
    """A decode step's positions from the records on the device (int32 [slots, 4]): row i of the batch, which belongs
    to slot slot_ids[i], stands at position record.len; the record moves on by one position and one decoded token."""
    _cuda(state, "seq_begin_decode state", torch.int32)
    _need(state.dim() == 2 and state.shape[1] == SEQ_FIELDS, f"seq_begin_decode: records must be [slots, {SEQ_FIELDS}]")
    S = slot_ids.numel()
    for name, t in (("slot_ids", slot_ids), ("tok_pos", tok_pos), ("seq_pos0", seq_pos0), ("seq_len", seq_len)):
        _cuda(t, f"seq_begin_decode {name}", torch.int32)
        _need(t.numel() == S, f"seq_begin_decode: {name} has {t.numel()} entries for {S} sequences")
    lib = build.load("elementwise")
    rc = lib.rl_seq_begin_decode(_p(state), _p(slot_ids), c_int(S), _p(tok_pos), _p(seq_pos0), _p(seq_len), _stream())
    _check(lib, rc, "seq_begin_decode")


def seq_set_len(state: torch.Tensor, slot_ids: torch.Tensor, seq_len: torch.Tensor) -> None:
    """record.len = seq_len[i] for the sequences of a step whose positions the host gave."""
    _cuda(state, "seq_set_len state", torch.int32)
    _need(state.dim() == 2 and state.shape[1] == SEQ_FIELDS, f"seq_set_len: records must be [slots, {SEQ_FIELDS}]")
    _cuda(slot_ids, "seq_set_len slot_ids", torch.int32)
    _cuda(seq_len, "seq_set_len seq_len", torch.int32)
    _need(slot_ids.numel() == seq_len.numel(), "seq_set_len: one length per sequence")
    lib = build.load("elementwise")
    rc = lib.rl_seq_set_len(_p(state), _p(slot_ids), _p(seq_len), c_int(slot_ids.numel()), _stream())
    _check(lib, rc, "seq_set_len")


# ------------------------------------------------------------------ position encoding + cache write
def rope_kv_write(
    qkv: torch.Tensor,
    tok_pos: torch.Tensor,
    tok_seq: torch.Tensor,
    block_table: Optional[torch.Tensor],
    k_pages: Optional[torch.Tensor],
    v_pages: Optional[torch.Tensor],
    inv_freq: Optional[torch.Tensor],
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    rotary_dim: int,
    interleaved: bool,
    write_kv: bool = True,
) -> None:
    """Rotate q (in place) and k, store k and v at each token's place in the paged cache.

    qkv: [T, >= (H + 2K) * hd] rows holding q heads, k heads, v heads.
    k_pages, v_pages: [pages, K, PAGE_SIZE, hd] of qkv's dtype.
    """
    _cuda(qkv, "rope_kv_write qkv", contiguous=False)
    stride = _rows(qkv, "rope_kv_write qkv")
    T = qkv.shape[0]
    _cuda(tok_pos, "rope_kv_write tok_pos", torch.int32)
    _cuda(tok_seq, "rope_kv_write tok_seq", torch.int32)
    _need(tok_pos.numel() == T and tok_seq.numel() == T, "rope_kv_write: one position and one sequence index per token")
    width = 0
    if write_kv:
        _cuda(block_table, "rope_kv_write block_table", torch.int32)
        _need(block_table.dim() == 2, "rope_kv_write: block_table must be [S, width]")
        width = block_table.shape[1]
        for name, pages in (("k_pages", k_pages), ("v_pages", v_pages)):
            _cuda(pages, f"rope_kv_write {name}", qkv.dtype)
            _need(
                pages.dim() == 4 and tuple(pages.shape[1:]) == (num_kv_heads, PAGE_SIZE, head_dim),
                f"rope_kv_write: {name} {tuple(pages.shape)} is not [pages, {num_kv_heads}, {PAGE_SIZE}, {head_dim}]",
            )
        _need(qkv.shape[1] >= (num_heads + 2 * num_kv_heads) * head_dim, "rope_kv_write: qkv rows too short")
    _need(qkv.data_ptr() % 16 == 0, "rope_kv_write: qkv is not 16-byte aligned")
    if rotary_dim:
        _cuda(inv_freq, "rope_kv_write inv_freq", torch.float32)
        _need(inv_freq.numel() == rotary_dim // 2, "rope_kv_write: inv_freq must hold rotary_dim/2 values")
    lib = build.load("rope")
    rc = lib.rl_rope_kv_write(
        _p(qkv), c_int(_dt(qkv, "rope_kv_write")), c_int(stride), _p(tok_pos), _p(tok_seq), _p(block_table), c_int(width),
        _p(k_pages), _p(v_pages), _p(inv_freq), c_int(T), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
        c_int(rotary_dim), c_int(1 if interleaved else 0), c_int(PAGE_SIZE), c_int(1 if write_kv else 0), _stream(),
    )
    _check(lib, rc, "rope_kv_write")


# ------------------------------------------------------------------ attention
def _check_pages(k_pages, v_pages, dtype, K, hd, what):
    for name, pages in (("k_pages", k_pages), ("v_pages", v_pages)):
        _cuda(pages, f"{what} {name}", dtype)
        _need(
            pages.dim() == 4 and tuple(pages.shape[1:]) == (K, PAGE_SIZE, hd),
            f"{what}: {name} {tuple(pages.shape)} is not [pages, {K}, {PAGE_SIZE}, {hd}]",
        )


def attn_generic(
    q: torch.Tensor, k_pages, v_pages, block_table, tok_seq, tok_pos, num_heads: int, num_kv_heads: int,
    head_dim: int, window: int = 0, scale: Optional[float] = None, out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Attention of each token over its sequence's cached keys 0..pos; any head size up to 256, both dtypes.

    q: [T, >= H*hd] rows (the q part of the fused projection may be passed as is)."""
    _cuda(q, "attn_generic q", contiguous=False)
    qs = _rows(q, "attn_generic q")
    T = q.shape[0]
    _need(q.shape[1] >= num_heads * head_dim, "attn_generic: q rows too short")
    _check_pages(k_pages, v_pages, q.dtype, num_kv_heads, head_dim, "attn_generic")
    _cuda(block_table, "attn_generic block_table", torch.int32)
    _cuda(tok_seq, "attn_generic tok_seq", torch.int32)
    _cuda(tok_pos, "attn_generic tok_pos", torch.int32)
    _need(tok_seq.numel() == T and tok_pos.numel() == T and block_table.dim() == 2, "attn_generic: metadata sizes")
    if out is None:
        out = torch.empty((T, num_heads * head_dim), dtype=q.dtype, device=q.device)
    _cuda(out, "attn_generic out", q.dtype)
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    lib = build.load("attention_generic")
    rc = lib.rl_attn_generic(
        _p(q), c_int(_dt(q, "attn_generic")), c_int(qs), _p(k_pages), _p(v_pages), _p(block_table),
        c_int(block_table.shape[1]), _p(tok_seq), _p(tok_pos), _p(out), c_int(out.stride(0)), c_int(T),
        c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(PAGE_SIZE), c_int(window), c_float(scale), _stream(),
    )
    _check(lib, rc, "attn_generic")
    return out


ATTN_DECODE_TMA_HEAD_DIMS = (64, 128)  # head sizes the TMA-fed decode kernel is built for


def attn_decode_scratch_floats(n_seqs: int, num_heads: int, head_dim: int, n_splits: int) -> int:
    return n_seqs * num_heads * n_splits * (head_dim + 2)


def attn_decode(
    q: torch.Tensor, k_pages, v_pages, block_table, seq_len, num_heads: int, num_kv_heads: int, head_dim: int,
    n_splits: int, scratch: torch.Tensor, window: int = 0, scale: Optional[float] = None,
    out: Optional[torch.Tensor] = None, impl: str = "auto", fuse: int = 0,
    inv_freq: Optional[torch.Tensor] = None, rotary_dim: int = 0, interleaved: bool = False,
    counters: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """One query token per sequence over keys 0..seq_len-1, the key range cut into `n_splits`.

    counters (the "tma" kernel only): int32 zeros, one per sequence and group of 8 query heads of a kv
    head; with them the splits are added up by the block that finishes last instead of by a second
    kernel, and the counters are zeros again afterwards.

    fuse (the "tma" kernel only): 0 = q is position-encoded and the new key and value are in the cache
    (what `rope_kv_write` leaves); 1 = q's rows are raw projections, the kernel turns the queries by
    `inv_freq` / `rotary_dim` / `interleaved`; 2 = as 1, and the kernel also takes the new token's key and
    value from q's rows, turns the key and stores both into the cache (k_pages and v_pages are written).

    scratch: float32 tensor of at least attn_decode_scratch_floats(...) elements.
    impl: "warp" = one-warp blocks that copy their own tiles, "tma" = four-warp blocks on a TMA-fed
    ring of whole pages (head sizes 64 and 128), "auto" = "tma" where it applies, else "warp"."""
    q_parts = None
    if q.dim() == 3:
        # the projection as float32 partial sums [parts, S, columns] (a product that was split over k): the
        # fused TMA kernel adds them up as it reads them
        _cuda(q, "attn_decode q (partial sums)", torch.float32, contiguous=False)
        _need(fuse > 0, "attn_decode: partial sums of the projection need fuse > 0")
        _need(q.stride(2) == 1 and q.stride(1) % 4 == 0 and q.stride(0) % 4 == 0, "attn_decode: partial sums must have dense, 16-byte aligned rows")
        q_parts, act = q, k_pages.dtype
        qs, S, q_cols = q.stride(1), q.shape[1], q.shape[2]
    else:
        _cuda(q, "attn_decode q", contiguous=False)
        qs, act = _rows(q, "attn_decode q"), q.dtype
        S, q_cols = q.shape
    _need(q_cols >= num_heads * head_dim, "attn_decode: q rows too short")
    _need(q.data_ptr() % 16 == 0, "attn_decode: q is not 16-byte aligned")
    _check_pages(k_pages, v_pages, act, num_kv_heads, head_dim, "attn_decode")
    _cuda(block_table, "attn_decode block_table", torch.int32)
    _cuda(seq_len, "attn_decode seq_len", torch.int32)
    _need(block_table.dim() == 2 and block_table.shape[0] >= S and seq_len.numel() == S, "attn_decode: metadata sizes")
    _cuda(scratch, "attn_decode scratch", torch.float32)
    need = attn_decode_scratch_floats(S, num_heads, head_dim, n_splits)
    _need(scratch.numel() >= need, f"attn_decode: scratch holds {scratch.numel()} floats, {need} needed")
    if out is None:
        out = torch.empty((S, num_heads * head_dim), dtype=act, device=q.device)
    _cuda(out, "attn_decode out", act)
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    n_o = S * num_heads * n_splits * head_dim
    part_o = c_void_p(scratch.data_ptr())
    part_ml = c_void_p(scratch.data_ptr() + 4 * n_o)
    _need(impl in ("auto", "warp", "tma"), f"attn_decode: unknown impl {impl!r}")
    if impl == "auto":
        impl = "tma" if (head_dim in ATTN_DECODE_TMA_HEAD_DIMS and act == torch.bfloat16) else "warp"
    _need(fuse in (0, 1, 2), f"attn_decode: fuse={fuse}")
    if fuse:
        _need(impl == "tma", "attn_decode: only the TMA kernel fuses the position encoding")
        if rotary_dim:
            _cuda(inv_freq, "attn_decode inv_freq", torch.float32)
            _need(inv_freq.numel() >= rotary_dim // 2, "attn_decode: too few angles for the rotary size")
        if fuse == 2:
            _need(q_cols >= (num_heads + 2 * num_kv_heads) * head_dim, "attn_decode: q rows hold no key and value")
    if counters is not None:
        _need(impl == "tma", "attn_decode: only the TMA kernel adds the splits up itself")
        _cuda(counters, "attn_decode counters", torch.int32)
        groups = num_kv_heads * ((num_heads // num_kv_heads + 7) // 8)
        _need(counters.numel() >= S * groups, f"attn_decode: {counters.numel()} counters, {S * groups} needed")
    _need(q_parts is None or impl == "tma", "attn_decode: only the TMA kernel takes partial sums")
    if impl == "tma":
        _need(act == torch.bfloat16, "attn_decode: the TMA kernel is bfloat16 only")
        status = _tc_status_word(q.device)
        lib = build.load("attention_decode_tma")
        rc = lib.rl_attn_decode_tma(
            c_void_p(0) if q_parts is not None else _p(q), c_int(qs), _p(k_pages), _p(v_pages), c_int(k_pages.shape[0]), _p(block_table),
            c_int(block_table.shape[1]), _p(seq_len), part_o, part_ml, _p(out), c_int(out.stride(0)), c_int(S),
            c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(PAGE_SIZE), c_int(window), c_float(scale),
            c_int(n_splits), _p(status), c_int(fuse), _p(inv_freq) if (fuse and rotary_dim) else c_void_p(0), c_int(rotary_dim if fuse else 0),
            c_int(1 if interleaved else 0), _p(counters) if counters is not None else c_void_p(0),
            _p(q_parts) if q_parts is not None else c_void_p(0), c_int(0 if q_parts is None else q_parts.shape[0]),
            c_ll(0 if q_parts is None else q_parts.stride(0)), *_wt(), _stream(),
        )
        _check(lib, rc, "attn_decode_tma", kernels=1 if counters is not None else 2)
        return out
    lib = build.load("attention_decode")
    rc = lib.rl_attn_decode(
        _p(q), c_int(_dt(q, "attn_decode")), c_int(qs), _p(k_pages), _p(v_pages), _p(block_table),
        c_int(block_table.shape[1]), _p(seq_len), part_o, part_ml, _p(out), c_int(out.stride(0)), c_int(S),
        c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(PAGE_SIZE), c_int(window), c_float(scale),
        c_int(n_splits), _stream(),
    )
    _check(lib, rc, "attn_decode", kernels=2)
    return out


def flash_prefill(
    q: torch.Tensor, k_pages, v_pages, block_table, seq_start, seq_pos0, max_q_len: int, num_heads: int,
    num_kv_heads: int, head_dim: int, window: int = 0, scale: Optional[float] = None,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """bfloat16 causal attention of a ragged batch over the paged cache (tensor cores)."""
    _cuda(q, "flash_prefill q", torch.bfloat16, contiguous=False)
    qs = _rows(q, "flash_prefill q")
    T = q.shape[0]
    _need(q.shape[1] >= num_heads * head_dim, "flash_prefill: q rows too short")
    _need(q.data_ptr() % 16 == 0, "flash_prefill: q is not 16-byte aligned")
    _check_pages(k_pages, v_pages, torch.bfloat16, num_kv_heads, head_dim, "flash_prefill")
    _cuda(block_table, "flash_prefill block_table", torch.int32)
    _cuda(seq_start, "flash_prefill seq_start", torch.int32)
    _cuda(seq_pos0, "flash_prefill seq_pos0", torch.int32)
    S = seq_pos0.numel()
    _need(seq_start.numel() == S + 1 and block_table.dim() == 2 and block_table.shape[0] >= S, "flash_prefill: metadata sizes")
    if out is None:
        out = torch.empty((T, num_heads * head_dim), dtype=torch.bfloat16, device=q.device)
    _cuda(out, "flash_prefill out", torch.bfloat16)
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    lib = build.load("attention_prefill")
    rc = lib.rl_flash_prefill(
        _p(q), c_int(qs), _p(k_pages), _p(v_pages), _p(block_table), c_int(block_table.shape[1]), _p(seq_start),
        _p(seq_pos0), _p(out), c_int(out.stride(0)), c_int(S), c_int(max_q_len), c_int(num_heads),
        c_int(num_kv_heads), c_int(head_dim), c_int(PAGE_SIZE), c_int(window), c_float(scale), _stream(),
    )
    _check(lib, rc, "flash_prefill")
    return out


FLASH_TC_HEAD_DIMS = (64, 128)  # head sizes the tcgen05 prompt attention is built for


def flash_prefill_tc(
    q: torch.Tensor, k_pages, v_pages, block_table, seq_start, seq_pos0, max_q_len: int, num_heads: int,
    num_kv_heads: int, head_dim: int, window: int = 0, scale: Optional[float] = None,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """`flash_prefill` on the tcgen05 tensor cores (TMA-fed, S and P V in tensor memory); head sizes 64 and 128."""
    _need(head_dim in FLASH_TC_HEAD_DIMS, f"flash_prefill_tc: head size {head_dim}, this kernel is built for {FLASH_TC_HEAD_DIMS}")
    _cuda(q, "flash_prefill_tc q", torch.bfloat16, contiguous=False)
    qs = _rows(q, "flash_prefill_tc q")
    T = q.shape[0]
    _need(q.shape[1] >= num_heads * head_dim, "flash_prefill_tc: q rows too short")
    _check_pages(k_pages, v_pages, torch.bfloat16, num_kv_heads, head_dim, "flash_prefill_tc")
    _need(k_pages.shape[0] == v_pages.shape[0], "flash_prefill_tc: k and v have different page counts")
    _cuda(block_table, "flash_prefill_tc block_table", torch.int32)
    _cuda(seq_start, "flash_prefill_tc seq_start", torch.int32)
    _cuda(seq_pos0, "flash_prefill_tc seq_pos0", torch.int32)
    S = seq_pos0.numel()
    _need(seq_start.numel() == S + 1 and block_table.dim() == 2 and block_table.shape[0] >= S, "flash_prefill_tc: metadata sizes")
    if out is None:
        out = torch.empty((T, num_heads * head_dim), dtype=torch.bfloat16, device=q.device)
    _cuda(out, "flash_prefill_tc out", torch.bfloat16)
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    status = _tc_status_word(q.device)
    lib = build.load("attention_prefill_tc")
    rc = lib.rl_flash_prefill_tc(
        _p(q), c_int(qs), c_int(T), _p(k_pages), _p(v_pages), c_int(k_pages.shape[0]), _p(block_table),
        c_int(block_table.shape[1]), _p(seq_start), _p(seq_pos0), _p(out), c_int(out.stride(0)), c_int(S), c_int(max_q_len),
        c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(PAGE_SIZE), c_int(window), c_float(scale), _p(status), *_wt(), _stream(),
    )
    _check(lib, rc, "flash_prefill_tc")
    return out


# ------------------------------------------------------------------ matrix products
GEMV_MAX_ROWS = 64


def gemm_f32(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T in true 32-bit."""
    _cuda(x, "gemm_f32 x", torch.float32, contiguous=False)
    _cuda(w, "gemm_f32 w", torch.float32, contiguous=False)
    ldx, ldw = _rows(x, "gemm_f32 x"), _rows(w, "gemm_f32 w")
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K, f"gemm_f32: x[{M}, {K}] against w[{N}, {w.shape[1]}]")
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    _cuda(out, "gemm_f32 out", torch.float32, contiguous=False)
    _need(tuple(out.shape) == (M, N), "gemm_f32: out has the wrong shape")
    lib = build.load("gemm_f32")
    rc = lib.rl_gemm_f32(_p(x), c_int(ldx), _p(w), c_int(ldw), _p(out), c_int(_rows(out, "gemm_f32 out")), c_int(M), c_int(N), c_int(K), _stream())
    _check(lib, rc, "gemm_f32")
    return out


def gemm_bf16_any(
    x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16, swiglu: bool = False
) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T for bfloat16 operands of any k and alignment, 32-bit sums on the
    CUDA cores: the slow kernel behind the shapes that the 16-byte-row kernels refuse.

    swiglu: w's rows alternate gate and up; out[M, N/2] = silu(gate) * up, from the 32-bit sums."""
    _cuda(x, "gemm_bf16_any x", torch.bfloat16, contiguous=False)
    _cuda(w, "gemm_bf16_any w", torch.bfloat16, contiguous=False)
    ldx, ldw = _rows(x, "gemm_bf16_any x"), _rows(w, "gemm_bf16_any w")
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K, f"gemm_bf16_any: x[{M}, {K}] against w[{N}, {w.shape[1]}]")
    out = torch.empty((M, N // 2 if swiglu else N), dtype=out_dtype, device=x.device)
    lib = build.load("gemm_f32")
    rc = lib.rl_gemm_bf16_any(
        _p(x), c_int(ldx), _p(w), c_int(ldw), _p(out), c_int(_dt(out, "gemm_bf16_any out")), c_int(out.shape[1]),
        c_int(M), c_int(N), c_int(K), c_int(1 if swiglu else 0), _stream(),
    )
    _check(lib, rc, "gemm_bf16_any")
    return out


def gemv_bf16(
    x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16, out: Optional[torch.Tensor] = None,
    swiglu: bool = False, k_splits: int = 1,
) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T for M <= 64 rows, bfloat16 in, 32-bit accumulate.

    swiglu: w's rows alternate gate and up; out[M, N/2] = silu(gate) * up, from the 32-bit sums.
    k_splits > 1: returns float32 [k_splits, M, N], one partial sum per slice of k, for a consumer
    that adds them (`add_rmsnorm`): more blocks in flight when N is small."""
    _cuda(x, "gemv_bf16 x", torch.bfloat16, contiguous=False)
    _cuda(w, "gemv_bf16 w", torch.bfloat16, contiguous=False)
    ldx, ldw = _rows(x, "gemv_bf16 x"), _rows(w, "gemv_bf16 w")
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K, f"gemv_bf16: x[{M}, {K}] against w[{N}, {w.shape[1]}]")
    _need(x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0, "gemv_bf16: operands must be 16-byte aligned")
    n_out = N // 2 if swiglu else N
    if k_splits > 1:
        _need(out_dtype == torch.float32 and not swiglu, "gemv_bf16: partial sums over k slices are float32, without activation")
        if out is None:
            out = torch.empty((k_splits, M, n_out), dtype=torch.float32, device=x.device)
        _cuda(out, "gemv_bf16 out", torch.float32)
        _need(tuple(out.shape) == (k_splits, M, n_out), "gemv_bf16: out has the wrong shape")
        ldo = n_out
    else:
        if out is None:
            out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
        _cuda(out, "gemv_bf16 out", out_dtype, contiguous=False)
        _need(tuple(out.shape) == (M, n_out), "gemv_bf16: out has the wrong shape")
        ldo = _rows(out, "gemv_bf16 out")
    lib = build.load("gemv_bf16")
    rc = lib.rl_gemv_bf16(
        _p(x), c_int(ldx), _p(w), c_int(ldw), _p(out), c_int(_dt(out, "gemv_bf16 out")), c_int(ldo),
        c_int(M), c_int(N), c_int(K), c_int(1 if swiglu else 0), c_int(k_splits), _stream(),
    )
    _check(lib, rc, "gemv_bf16")
    return out


def gemv_stream_slices(M: int, K: int, k_splits: int = 1) -> int:
    """How many slices of k `gemv_stream` produces for these arguments: 1 is a finished result, more
    are float32 partial sums, 0 means that the kernel does not take the shape (more than 16 rows, k
    no multiple of 64).  A slice is at most 4096 long, or 5120 when k is longer than 4096, so longer k always comes in slices."""
    lib = build.load("gemv_stream")
    return int(lib.rl_gemv_stream_slices(c_int(M), c_int(K), c_int(k_splits)))


def gemv_stream_into_stream(
    x: torch.Tensor, w: torch.Tensor, resid: torch.Tensor, next_w: torch.Tensor, xw: Optional[torch.Tensor] = None,
    sumsq: Optional[torch.Tensor] = None,
):
    """The product before an RMSNorm that is folded into its neighbours (at most 8 rows, k a multiple of 64 up to 5120):

        resid (float32 [M, N], in place) += x[M, K] . w[N, K]^T
        xw[M, N] = bfloat16(resid * next_w)           the activations of the product after the norm
        sumsq[blocks, 8]                              each block's share of the rows' sum(resid^2)

    Returns (xw, sumsq, blocks); hand them to `gemv_stream(xw, ..., row_scale=(sumsq, blocks, N, eps))`."""
    _cuda(x, "gemv_stream_into_stream x", torch.bfloat16, contiguous=False)
    _cuda(w, "gemv_stream_into_stream w", torch.bfloat16, contiguous=False)
    _cuda(resid, "gemv_stream_into_stream resid", torch.float32, contiguous=False)
    _cuda(next_w, "gemv_stream_into_stream next_w")
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K and tuple(resid.shape) == (M, N) and tuple(next_w.shape) == (N,),
          f"gemv_stream_into_stream: x{tuple(x.shape)} w{tuple(w.shape)} resid{tuple(resid.shape)} next_w{tuple(next_w.shape)} do not fit")
    lib = build.load("gemv_stream")
    blocks = int(lib.rl_gemv_stream_blocks(c_int(N), c_int(K)))
    _need(blocks > 0, f"gemv_stream_into_stream: the kernel does not take N={N}, K={K}")
    if xw is None:
        xw = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    if sumsq is None:
        sumsq = torch.empty(blocks * 8, dtype=torch.float32, device=x.device)
    _cuda(xw, "gemv_stream_into_stream xw", torch.bfloat16, contiguous=False)
    _cuda(sumsq, "gemv_stream_into_stream sumsq", torch.float32)
    _need(tuple(xw.shape) == (M, N) and sumsq.numel() >= blocks * 8, "gemv_stream_into_stream: xw or sumsq of the wrong size")
    used = c_int(0)
    status = _tc_status_word(x.device)
    rc = lib.rl_gemv_stream_into_stream(
        _p(x), c_int(_rows(x, "gemv_stream_into_stream x")), _p(w), c_int(_rows(w, "gemv_stream_into_stream w")), _p(resid),
        c_int(_rows(resid, "gemv_stream_into_stream resid")), _p(next_w), c_int(_dt(next_w, "gemv_stream_into_stream next_w")), _p(xw),
        c_int(_rows(xw, "gemv_stream_into_stream xw")), _p(sumsq), c_int(M), c_int(N), c_int(K), ctypes.byref(used), _p(status), *_wt(), _stream(),
    )
    _check(lib, rc, "gemv_stream_into_stream")
    _need(used.value == blocks, f"gemv_stream_into_stream: the kernel ran {used.value} blocks, the wrapper planned {blocks}")
    return xw, sumsq, blocks


def gemv_stream(
    x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16, out: Optional[torch.Tensor] = None,
    swiglu: bool = False, k_splits: int = 1, row_scale=None,
) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T for M <= 16 rows: the persistent weight-streaming kernel of
    decode steps (bulk copies into a ring of shared memory, one block per SM).

    swiglu: w's rows alternate gate and up; out[M, N/2] = silu(gate) * up, from the 32-bit sums.
    k_splits > 1: returns float32 [slices, M, N] partial sums over slices of k (`gemv_stream_slices`
    says how many: each is a multiple of 1024 and at most 5120 long), for a consumer that adds them up.
    row_scale = (sumsq, blocks, norm_k, eps), as left by `gemv_stream_into_stream`: an RMSNorm folded into this
    product, whose x is then `xw`; every row's sums are multiplied by 1 / sqrt(sum(shares) / norm_k + eps) before
    they are stored or go through the activation (at most 8 rows, k in one slice)."""
    _cuda(x, "gemv_stream x", torch.bfloat16, contiguous=False)
    _cuda(w, "gemv_stream w", torch.bfloat16, contiguous=False)
    ldx, ldw = _rows(x, "gemv_stream x"), _rows(w, "gemv_stream w")
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K, f"gemv_stream: x[{M}, {K}] against w[{N}, {w.shape[1]}]")
    n_out = N // 2 if swiglu else N
    used = c_int(1)
    slices = max(1, gemv_stream_slices(M, K, k_splits))  # (0: the launcher says what it does not take)
    _need(k_splits > 1 or slices == 1, f"gemv_stream: k = {K} comes in {slices} slices, whose float32 partial sums have to be asked for (k_splits > 1)")
    if k_splits > 1 and slices > 1:
        _need(out is None and out_dtype == torch.float32 and not swiglu, "gemv_stream: partial sums over k slices are float32, without activation")
        out = torch.empty((slices, M, n_out), dtype=torch.float32, device=x.device)
        ldo = n_out
    else:
        if out is None:
            out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
        _cuda(out, "gemv_stream out", out_dtype, contiguous=False)
        _need(tuple(out.shape) == (M, n_out), "gemv_stream: out has the wrong shape")
        ldo = _rows(out, "gemv_stream out")
    status = _tc_status_word(x.device)
    lib = build.load("gemv_stream")
    if row_scale is not None:
        sumsq, blocks, norm_k, eps = row_scale
        _cuda(sumsq, "gemv_stream row_scale", torch.float32)
        _need(k_splits == 1 and slices == 1 and sumsq.numel() >= blocks * 8, "gemv_stream: a row scale goes with whole sums and needs its shares")
        rc = lib.rl_gemv_stream_scaled(
            _p(x), c_int(ldx), _p(w), c_int(ldw), _p(out), c_int(_dt(out, "gemv_stream out")), c_int(ldo), c_int(M), c_int(N), c_int(K),
            c_int(1 if swiglu else 0), _p(sumsq), c_int(blocks), c_int(norm_k), c_float(eps), _p(status), *_wt(), _stream(),
        )
        _check(lib, rc, "gemv_stream")
        return out
    rc = lib.rl_gemv_stream(
        _p(x), c_int(ldx), _p(w), c_int(ldw), _p(out), c_int(_dt(out, "gemv_stream out")), c_int(ldo),
        c_int(M), c_int(N), c_int(K), c_int(1 if swiglu else 0), c_int(k_splits), ctypes.byref(used), _p(status), *_wt(), _stream(),
    )
    _check(lib, rc, "gemv_stream")
    _need(used.value == slices, f"gemv_stream: kernel used {used.value} slices, the wrapper planned {slices}")
    return out


_tc_status = {}
_wait_test = (0, 0)  # (role code, limit in nanoseconds) handed to the launchers with bounded waits; (0, 0): none


class short_wait:
    """For tests of the give-up paths: inside `with ops.short_wait(code, ns):` the kernels with bounded waits
    let the role whose status code is `code` wait `ns` nanoseconds instead of a second (every other role keeps
    its limit, and so do the waits that keep a block alive until its copies have landed).  The codes are the
    ones `tc_status_check` names."""

    def __init__(self, role_code: int, limit_ns: int):
        self.value = (int(role_code), int(limit_ns))

    def __enter__(self):
        global _wait_test
        self.before, _wait_test = _wait_test, self.value
        return self

    def __exit__(self, *exc):
        global _wait_test
        _wait_test = self.before
        return False


def _wt():
    return c_int(_wait_test[0]), ctypes.c_uint(_wait_test[1])


def _tc_status_word(device: torch.device) -> torch.Tensor:
    key = (device.type, device.index)
    if key not in _tc_status:
        _tc_status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _tc_status[key]


_STATUS_NAMES = {
    1: "gemm_tc: the TMA producer (for a free stage)", 2: "gemm_tc: the tensor-core issuer (for a stage's data)",
    3: "gemm_tc: an epilogue warp (for a finished accumulator)", 4: "gemm_tc: the tensor-core issuer (for a free accumulator)",
    11: "flash_prefill_tc: the TMA producer (for a free key stage)", 12: "flash_prefill_tc: the TMA producer (for a free value stage)",
    13: "flash_prefill_tc: the tensor-core issuer (for the queries)", 14: "flash_prefill_tc: the tensor-core issuer (for a key tile)",
    15: "flash_prefill_tc: the tensor-core issuer (for the probabilities)", 16: "flash_prefill_tc: the tensor-core issuer (for a value tile)",
    17: "flash_prefill_tc: a softmax warp (for the scores)", 18: "flash_prefill_tc: a softmax warp (for the product before a rescale)",
    20: "flash_prefill_tc: a softmax warp (for the last product)",
    23: "flash_prefill_tc: shared memory not aligned",
    32: "gemv_stream: the copying lane (for a free stage)", 34: "gemv_stream: a product warp (for a stage's weights)",
    35: "gemv_stream: a storing warp (for an item's sums)", 36: "gemv_stream: shared memory not aligned",
    37: "gemv_stream: a product warp (for a free sum buffer)",
    51: "attn_decode_tma: the copying lane (for a free stage)", 52: "attn_decode_tma: a product warp (for a page)",
    56: "attn_decode_tma: shared memory not aligned",
}


def tc_status_check() -> None:
    """Raise if a bounded wait inside a TMA / tensor-core kernel expired since the last check (synchronises);
    the status word is zero again afterwards."""
    for word in _tc_status.values():
        code = int(word.item())
        if code:
            word.zero_()
            who = _STATUS_NAMES.get(code, "a role")
            raise KernelError(f"{who} gave up waiting on a barrier (code {code}); results of that step are not valid")


def gemm_tc(
    x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16, out: Optional[torch.Tensor] = None,
    swiglu: bool = False, k_splits: int = 1, tile_n: int = 0,
) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T on the tcgen05 tensor cores (TMA-fed, accumulator in tensor memory).

    tile_n: 0 (the launcher chooses), or the width of the output tiles, a multiple of 16 up to 256.

    swiglu: w's rows alternate gate and up; out[M, N/2] = silu(gate) * up, from the 32-bit accumulators.
    k_splits > 1: returns float32 [slices, M, N] partial sums over slices of k (at most k_splits of
    them), for a consumer that adds them up: more blocks at work when the output has few tiles."""
    _cuda(x, "gemm_tc x", torch.bfloat16, contiguous=False)
    _cuda(w, "gemm_tc w", torch.bfloat16, contiguous=False)
    ldx, ldw = _rows(x, "gemm_tc x"), _rows(w, "gemm_tc w")
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K, f"gemm_tc: x[{M}, {K}] against w[{N}, {w.shape[1]}]")
    n_out = N // 2 if swiglu else N
    used = c_int(1)
    if k_splits > 1:
        _need(out is None and out_dtype == torch.float32 and not swiglu, "gemm_tc: partial sums over k slices are float32, without activation")
        slices = (K + 63) // 64
        per = (slices + min(k_splits, slices) - 1) // min(k_splits, slices)
        k_splits = (slices + per - 1) // per
        out = torch.empty((k_splits, M, n_out), dtype=torch.float32, device=x.device)
        ldo = n_out
    else:
        if out is None:
            out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
        _cuda(out, "gemm_tc out", out_dtype, contiguous=False)
        _need(tuple(out.shape) == (M, n_out), "gemm_tc: out has the wrong shape")
        ldo = _rows(out, "gemm_tc out")
    status = _tc_status_word(x.device)
    lib = build.load("gemm_tc")
    rc = lib.rl_gemm_tc(
        _p(x), c_int(ldx), _p(w), c_int(ldw), _p(out), c_int(_dt(out, "gemm_tc out")), c_int(ldo),
        c_int(M), c_int(N), c_int(K), c_int(1 if swiglu else 0), c_int(k_splits), ctypes.byref(used), c_int(tile_n), _p(status), *_wt(), _stream(),
    )
    _check(lib, rc, "gemm_tc")
    if k_splits > 1:
        _need(used.value == k_splits, f"gemm_tc: kernel used {used.value} slices, the wrapper planned {k_splits}")
    return out


# ------------------------------------------------------------------ sampling
def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Index of the largest logit of each row, the last one among equals."""
    _cuda(logits, "argmax logits", torch.float32, contiguous=False)
    stride = _rows(logits, "argmax logits")
    R, n = logits.shape
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    _cuda(out, "argmax out", torch.int32)
    lib = build.load("sampling")
    rc = lib.rl_argmax(_p(logits), c_ll(stride), c_int(R), c_int(n), _p(out), _stream())
    _check(lib, rc, "argmax")
    return out


def sample(
    logits: torch.Tensor, temperature: float, top_p: float, rng_states: torch.Tensor, rng_index: torch.Tensor,
    scratch: torch.Tensor, out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """One draw per row from softmax(logits / temperature), cut to the top-p nucleus when 0 < top_p < 1.

    rng_states: int64 tensor of xorshift64* states; row r uses and advances rng_states[rng_index[r]].
    scratch: float32, at least rows * vocabulary elements."""
    _cuda(logits, "sample logits", torch.float32, contiguous=False)
    stride = _rows(logits, "sample logits")
    R, n = logits.shape
    _cuda(rng_states, "sample rng_states", torch.int64)
    _cuda(rng_index, "sample rng_index", torch.int32)
    _need(rng_index.numel() == R, "sample: one random-state index per row")
    _cuda(scratch, "sample scratch", torch.float32)
    _need(scratch.numel() >= R * n, f"sample: scratch holds {scratch.numel()} floats, {R * n} needed")
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    _cuda(out, "sample out", torch.int32)
    lib = build.load("sampling")
    rc = lib.rl_sample(
        _p(logits), c_ll(stride), c_int(R), c_int(n), c_float(temperature), c_float(top_p), _p(rng_states),
        _p(rng_index), _p(scratch), _p(out), _stream(),
    )
    _check(lib, rc, "sample")
    return out


SAMPLE_HISTORY_MAX = 1024


def sample_chain(
    logits: torch.Tensor, temperature: float, top_p: float, top_k: int, min_p: float, repeat_penalty: float,
    last_n: int, frequency_penalty: float, presence_penalty: float, rng_states: torch.Tensor, slot_of_row: torch.Tensor,
    history: torch.Tensor, history_count: torch.Tensor, work: torch.Tensor, out: Optional[torch.Tensor] = None,
    mirostat: int = 0, mirostat_tau: float = 5.0, mirostat_eta: float = 0.1, mirostat_mu: Optional[torch.Tensor] = None,
    xtc_probability: float = 0.0, xtc_threshold: float = 0.1, xtc_states: Optional[torch.Tensor] = None,
    dry_multiplier: float = 0.0, dry_base: float = 1.75, dry_allowed_length: int = 2, dry_last_n: int = 0,
    dry_breakers: Sequence[int] = (),
) -> torch.Tensor:
    """One token per row through penalties -> top-k -> top-p -> min-p -> temperature -> draw (temperature 0:
    the argmax of the penalised logits, no draw).

    Row r belongs to slot slot_of_row[r]: it uses and advances rng_states[slot], reads the last `last_n`
    chosen tokens of history[slot] (int32 [slots, 1024] with history_count[slot] tokens written so far) for
    the penalties and appends its choice.  work: float32, at least rows * 2 * (vocabulary rounded up to 4).
    mirostat 1 or 2: penalties -> temperature -> mirostat's own cut and draw; mirostat_mu: float32 [slots], NaN
    for a sequence that has not drawn yet.  xtc_probability > 0: the "exclude top choices" filter after min-p, with
    a generator of its own per slot (xtc_states, int64 like rng_states).  dry_multiplier > 0: the DRY penalty
    after the other penalties, over the last dry_last_n chosen tokens, with up to 8 breaker tokens.
    history[slot] is a ring over all 1024 places (the p-th chosen token at p % 1024), whatever the windows."""
    _cuda(logits, "sample_chain logits", torch.float32, contiguous=False)
    stride = _rows(logits, "sample_chain logits")
    R, n = logits.shape
    _cuda(rng_states, "sample_chain rng_states", torch.int64)
    _cuda(slot_of_row, "sample_chain slot_of_row", torch.int32)
    _need(slot_of_row.numel() == R, "sample_chain: one slot per row")
    _cuda(history, "sample_chain history", torch.int32)
    _cuda(history_count, "sample_chain history_count", torch.int32)
    _need(history.dim() == 2 and history.shape[1] == SAMPLE_HISTORY_MAX and history.shape[0] == history_count.numel(),
          f"sample_chain: history must be [slots, {SAMPLE_HISTORY_MAX}] with one count per slot")
    _cuda(work, "sample_chain work", torch.float32)
    need = R * 2 * ((n + 3) // 4 * 4)
    _need(work.numel() >= need, f"sample_chain: work holds {work.numel()} floats, {need} needed")
    _need(work.data_ptr() % 16 == 0, "sample_chain: work must be 16-byte aligned")
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    _cuda(out, "sample_chain out", torch.int32)
    if mirostat:
        _need(mirostat_mu is not None, "sample_chain: mirostat needs its state")
        _cuda(mirostat_mu, "sample_chain mirostat_mu", torch.float32)
        _need(mirostat_mu.numel() == history_count.numel(), "sample_chain: one mirostat state per slot")
    if xtc_probability > 0.0:
        _need(xtc_states is not None, "sample_chain: XTC needs its random states")
        _cuda(xtc_states, "sample_chain xtc_states", torch.int64)
        _need(xtc_states.numel() == history_count.numel(), "sample_chain: one XTC state per slot")
    breakers = (ctypes.c_int * max(len(dry_breakers), 1))(*[int(b) for b in dry_breakers])
    lib = build.load("sampling")
    rc = lib.rl_sample_chain(
        _p(logits), c_ll(stride), c_int(R), c_int(n), c_float(temperature), c_float(top_p), c_int(top_k), c_float(min_p),
        c_float(repeat_penalty), c_int(last_n), c_float(frequency_penalty), c_float(presence_penalty), c_int(mirostat),
        c_float(mirostat_tau), c_float(mirostat_eta), c_float(xtc_probability), c_float(xtc_threshold),
        c_float(dry_multiplier), c_float(dry_base), c_int(dry_allowed_length), c_int(dry_last_n), breakers, c_int(len(dry_breakers)),
        _p(rng_states),
        _p(slot_of_row), _p(history), _p(history_count), _p(mirostat_mu) if mirostat_mu is not None else c_void_p(0),
        _p(xtc_states) if xtc_states is not None else c_void_p(0), _p(work), _p(out), _stream(),
    )
    _check(lib, rc, "sample_chain")
    return out
