"""Each kernel alone against a plain float32/float64 reference of the same formula, at sizes the
engine's own models do not use (head sizes 24, 40, 128, 256; widths that are no power of two;
groups of 1, 3, 4, 5; pages in scrambled order)."""

import math

import numpy as np
import pytest
import torch

from plain_llama import PlainChain, PlainRng, plain_argmax, plain_rmsnorm, plain_rope, plain_sample, plain_silu

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
PAGE = 64


@pytest.fixture(scope="module")
def ops():
    from rusty_llama_b200.kernels import ops as o

    return o


def bf16_round(t):
    return t.to(torch.bfloat16).to(torch.float32)


def close_f32(got, ref, rel=2e-5):
    got, ref = got.detach().cpu().double(), ref.detach().cpu().double()
    tol = rel * float(ref.abs().max()) + 1e-7
    err = float((got - ref).abs().max())
    assert err <= tol, f"max error {err:.3e} exceeds {tol:.3e}"


def close_dot_f32(got, x, w):
    """32-bit results of K-term inner products accumulated in 32-bit: the rounding of a running sum
    grows like sqrt(K) units in the last place of the sum of the terms' magnitudes (a random walk of
    K roundings), whatever order the hardware adds in."""
    ref = x.double() @ w.double().T
    mags = x.abs().double() @ w.abs().double().T
    K = x.shape[1]
    tol = math.sqrt(K) * 2.0 ** -24 * mags + 1e-7
    err = (got.detach().cpu().double() - ref).abs()
    worst = float((err / tol).max())
    assert worst <= 1.0, f"error reaches {worst:.2f} of sqrt(K) ulp of the summed magnitudes (K={K})"


def close_bf16(got, ref):
    """bfloat16 keeps 8 bits: an element may be off by 2^-8 of its own size from the final rounding,
    plus what rounding the operands of an inner product adds, which scales with the result's range."""
    got, ref = got.detach().cpu().double(), ref.detach().cpu().double()
    scale = float(ref.abs().max()) + 1e-6
    err = (got - ref).abs()
    assert float(err.max()) <= 1.2e-2 * scale, f"max error {float(err.max()):.3e} vs range {scale:.3e}"
    assert float(err.mean()) <= 2e-3 * scale, f"mean error {float(err.mean()):.3e} vs range {scale:.3e}"


def guarded_out(M, n_out, dtype, pad_cols=8):
    """A NaN-filled flat buffer and the [M, n_out] window inside it that a product is asked to write: rows
    n_out + pad_cols apart (so ldo > N, and as ragged as N is), the first one on a 16-byte boundary, a row's
    worth of guard on both sides.  `untouched` says whether everything around the window is still NaN: a
    store past a ragged edge, or with the wrong row stride, lands there."""
    ld = n_out + pad_cols
    lead = (ld + 7) // 8 * 8
    buf = torch.full((lead + (M + 1) * ld,), float("nan"), dtype=dtype, device=DEV)
    return buf, buf[lead : lead + M * ld].view(M, ld)[:, :n_out]


def untouched(buf, M, n_out, pad_cols=8):
    ld = n_out + pad_cols
    lead = (ld + 7) // 8 * 8
    b = buf.float().cpu()
    inside = b[lead : lead + M * ld].view(M, ld)
    return bool(torch.isnan(b[:lead]).all() and torch.isnan(b[lead + M * ld :]).all() and torch.isnan(inside[:, n_out:]).all()
                and not torch.isnan(inside[:, :n_out]).any())


class PagedKV:
    """Dense keys/values of several sequences laid out in scrambled pages."""

    def __init__(self, lens, K, hd, dtype, seed=0, extra_pages=3):
        g = torch.Generator().manual_seed(seed)
        self.lens, self.K, self.hd = lens, K, hd
        self.k = [torch.randn(n, K, hd, generator=g) for n in lens]
        self.v = [torch.randn(n, K, hd, generator=g) for n in lens]
        if dtype == torch.bfloat16:
            self.k = [bf16_round(t) for t in self.k]
            self.v = [bf16_round(t) for t in self.v]
        n_pages = sum((n + PAGE - 1) // PAGE for n in lens) + extra_pages
        order = torch.randperm(n_pages, generator=g).tolist()
        width = max((n + PAGE - 1) // PAGE for n in lens)
        self.table = torch.zeros(len(lens), width, dtype=torch.int32)
        # unwritten pages hold large finite junk: reading them shows up in the result
        self.k_pages = torch.full((n_pages, K, PAGE, hd), 77.0)
        self.v_pages = torch.full((n_pages, K, PAGE, hd), -55.0)
        for s, n in enumerate(lens):
            for j in range((n + PAGE - 1) // PAGE):
                page = order.pop()
                self.table[s, j] = page
                lo, hi = j * PAGE, min(n, (j + 1) * PAGE)
                self.k_pages[page, :, : hi - lo] = self.k[s][lo:hi].transpose(0, 1)
                self.v_pages[page, :, : hi - lo] = self.v[s][lo:hi].transpose(0, 1)
        self.k_pages = self.k_pages.to(dtype).to(DEV)
        self.v_pages = self.v_pages.to(dtype).to(DEV)
        self.table = self.table.to(DEV)


def ref_attention_rows(q_rows, kv: PagedKV, s, positions, window=0, scale=None):
    """Attention of query rows at `positions` of sequence s over its keys 0..pos (float64)."""
    H, hd = q_rows.shape[1], q_rows.shape[2]
    K = kv.K
    scale = scale or 1.0 / math.sqrt(hd)
    out = torch.zeros(len(positions), H, hd, dtype=torch.float64)
    for i, pos in enumerate(positions):
        lo = max(0, pos + 1 - window) if window else 0
        for h in range(H):
            g = h // (H // K)
            sc = (kv.k[s][lo : pos + 1, g].double() @ q_rows[i, h].double()) * scale
            p = torch.softmax(sc, dim=0)
            out[i, h] = p @ kv.v[s][lo : pos + 1, g].double()
    return out


# --------------------------------------------------------------------------- row kernels
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d", [72, 70, 4096])
def test_embed_gather(ops, dtype, d):
    table = torch.randn(300, d).to(dtype)
    toks = torch.tensor([0, 299, 17, 17, 5], dtype=torch.int32)
    out = ops.embed_gather(toks.to(DEV), table.to(DEV))
    assert out.dtype == torch.float32
    assert torch.equal(out.cpu(), table[toks.long()].float())


@pytest.mark.parametrize("act", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("wdt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d, parts", [(200, 0), (72, 1), (4104, 3), (201, 2)])
def test_add_rmsnorm(ops, act, wdt, d, parts):
    T, eps = 5, 3e-6
    x = torch.randn(T, d) * 3
    w = (1 + 0.1 * torch.randn(d)).to(wdt)
    delta = None if parts == 0 else torch.randn(parts, T, d).to(act)
    ref_x = x.clone()
    if delta is not None:
        for p in range(parts):
            ref_x = ref_x + delta[p].float()
    ref = plain_rmsnorm(ref_x.double(), w.double(), eps)
    xd = x.to(DEV)
    dd = None if delta is None else (delta[0] if parts == 1 else delta).contiguous().to(DEV)
    out = ops.add_rmsnorm(xd, dd, w.to(DEV), eps, act)
    assert out.dtype == act
    close_f32(xd, ref_x, 1e-6)  # the stream holds the 32-bit sum
    (close_f32 if act == torch.float32 else close_bf16)(out, ref)
    # a subset of rows, stream untouched
    xd2 = x.to(DEV)
    rows = torch.tensor([4, 1], dtype=torch.int32, device=DEV)
    out2 = ops.add_rmsnorm(xd2, dd, w.to(DEV), eps, act, rows=rows, write_x=False)
    assert torch.equal(xd2.cpu(), x)
    assert torch.equal(out2.cpu(), out[[4, 1]].cpu())
    # the sum alone
    if delta is not None:
        xd3 = x.to(DEV)
        assert ops.add_rmsnorm(xd3, dd, None, 0.0, act) is None
        close_f32(xd3, ref_x, 1e-6)


@pytest.mark.parametrize("wdt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T, d, parts, part_dtype", [(70, 4096, 1, torch.bfloat16), (64, 520, 2, torch.float32), (300, 4100, 0, None), (65, 72, 3, torch.bfloat16)])
def test_add_rmsnorm_many_rows_in_bfloat16(ops, wdt, T, d, parts, part_dtype):
    """From 64 rows on a bfloat16 run takes the kernel that keeps a row in registers: widths that
    fill all of a thread's pieces, some of them and (4100) more than it holds, which falls back."""
    eps = 1e-5
    x = torch.randn(T, d) * 2
    w = (1 + 0.1 * torch.randn(d)).to(wdt)
    delta = None if parts == 0 else torch.randn(parts, T, d).to(part_dtype)
    ref_x = x.clone()
    for p in range(parts):
        ref_x = ref_x + delta[p].float()
    xd = x.to(DEV)
    dd = None if delta is None else (delta[0] if parts == 1 and part_dtype == torch.bfloat16 else delta).contiguous().to(DEV)
    out = ops.add_rmsnorm(xd, dd, w.to(DEV), eps, torch.bfloat16)
    close_f32(xd, ref_x, 1e-6)
    close_bf16(out, plain_rmsnorm(ref_x.double(), w.double(), eps))
    rows = torch.arange(T - 1, -1, -1, dtype=torch.int32, device=DEV)  # every row, backwards, stream untouched
    xd2 = x.to(DEV)
    out2 = ops.add_rmsnorm(xd2, dd, w.to(DEV), eps, torch.bfloat16, rows=rows, write_x=False)
    assert torch.equal(xd2.cpu(), x)
    assert torch.equal(out2.cpu(), out.flip(0).cpu())


def test_rmsnorm_of_ones_and_eps(ops):
    # src/backend/cpu.rs:750-771
    x = torch.ones(2, 64, device=DEV)
    out = ops.add_rmsnorm(x, None, torch.ones(64, device=DEV), 1e-5, torch.float32)
    assert abs(float(out[0, 0]) - 1 / math.sqrt(1 + 1e-5)) < 1e-7
    out = ops.add_rmsnorm(torch.zeros(1, 64, device=DEV), None, torch.ones(64, device=DEV), 1e-5, torch.float32)
    assert torch.isfinite(out).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("ff", [100, 101, 14336])
def test_swiglu(ops, dtype, ff):
    gu = (torch.randn(3, 2 * ff) * 4).to(dtype)
    ref = plain_silu(gu[:, :ff].double()) * gu[:, ff:].double()
    out = ops.swiglu(gu.to(DEV))
    (close_f32 if dtype == torch.float32 else close_bf16)(out, ref)
    one = torch.tensor([[1.0, 2.0]], device=DEV)
    assert abs(float(ops.swiglu(one)[0, 0]) - 0.7310586 * 2) < 1e-6  # src/backend/cpu.rs:781-787


# --------------------------------------------------------------------------- rotary + cache write
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("H, K, hd, rot", [(6, 3, 40, 40), (4, 4, 24, 16), (5, 1, 128, 128), (3, 1, 18, 10)])
def test_rope_kv_write(ops, dtype, interleaved, H, K, hd, rot):
    lens = [70, 3]  # the first sequence crosses a page
    pos0 = [60, 130]  # and both start late in their sequences
    T = sum(lens)
    qkv = torch.randn(T, (H + 2 * K) * hd + 8).to(dtype)  # rows longer than needed: the stride is honoured
    tok_seq = torch.tensor(sum(([s] * n for s, n in enumerate(lens)), []), dtype=torch.int32)
    tok_pos = torch.tensor(sum((list(range(p, p + n)) for p, n in zip(pos0, lens)), []), dtype=torch.int32)
    inv = torch.tensor([10000.0 ** (-2 * j / rot) for j in range(rot // 2)], dtype=torch.float32)
    n_pages = 8
    table = torch.tensor([[5, 2, 7], [1, 0, 3]], dtype=torch.int32)
    kp = torch.zeros(n_pages, K, PAGE, hd, dtype=dtype, device=DEV)
    vp = torch.zeros_like(kp)
    qd = qkv.to(DEV)
    ops.rope_kv_write(qd, tok_pos.to(DEV), tok_seq.to(DEV), table.to(DEV), kp, vp, inv.to(DEV), H, K, hd, rot, interleaved)
    q = qkv[:, : H * hd].float().view(T, H, hd)
    k = qkv[:, H * hd : (H + K) * hd].float().view(T, K, hd)
    v = qkv[:, (H + K) * hd : (H + 2 * K) * hd].float().view(T, K, hd)

    def rotated(x):
        out = x.clone().double()
        out[..., :rot] = plain_rope(x[..., :rot].double(), tok_pos, inv, interleaved)
        return out

    cmp = close_f32 if dtype == torch.float32 else close_bf16
    cmp(qd[:, : H * hd].view(T, H, hd), rotated(q))
    assert torch.equal(qd[:, H * hd :].cpu(), qkv[:, H * hd :])  # k, v and the padding of the row are not touched
    kr = rotated(k)
    got_k = torch.zeros(T, K, hd)
    got_v = torch.zeros(T, K, hd)
    for t in range(T):
        s, p = int(tok_seq[t]), int(tok_pos[t])
        page = int(table[s, p // PAGE])
        got_k[t] = kp[page, :, p % PAGE].float().cpu()
        got_v[t] = vp[page, :, p % PAGE].float().cpu()
    cmp(got_k, kr)
    assert torch.equal(got_v, v)
    # nothing else was written
    written = torch.zeros(n_pages, PAGE, dtype=torch.bool)
    for t in range(T):
        s, p = int(tok_seq[t]), int(tok_pos[t])
        written[int(table[s, p // PAGE]), p % PAGE] = True
    assert (kp.float().cpu().abs().sum(dim=(1, 3))[~written] == 0).all()


# --------------------------------------------------------------------------- attention
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, K, hd, window", [(4, 2, 40, 0), (3, 3, 24, 0), (6, 2, 256, 0), (4, 1, 16, 37)])
def test_attn_generic(ops, dtype, H, K, hd, window):
    lens = [150, 64, 1]
    kv = PagedKV(lens, K, hd, dtype, seed=1)
    # queries: every position of sequence 1, a few of the others
    queries = [(0, [0, 63, 64, 149]), (1, list(range(64))), (2, [0])]
    tok_seq = torch.tensor(sum(([s] * len(p) for s, p in queries), []), dtype=torch.int32)
    tok_pos = torch.tensor(sum((p for _, p in queries), []), dtype=torch.int32)
    T = len(tok_seq)
    q = torch.randn(T, H * hd + 16)
    if dtype == torch.bfloat16:
        q = bf16_round(q)
    out = ops.attn_generic(q.to(dtype).to(DEV), kv.k_pages, kv.v_pages, kv.table, tok_seq.to(DEV), tok_pos.to(DEV), H, K, hd, window=window)
    ref = torch.cat([
        ref_attention_rows(q[tok_seq == s][:, : H * hd].view(-1, H, hd), kv, s, p, window) for s, p in queries
    ]).view(T, H * hd)
    (close_f32 if dtype == torch.float32 else close_bf16)(out, ref)


def test_attn_generic_bits_do_not_depend_on_the_batch(ops):
    """32-bit attention of a token is the same bits alone or among others."""
    H, K, hd = 4, 2, 48
    kv = PagedKV([200, 90], K, hd, torch.float32, seed=2)
    q = torch.randn(5, H * hd)
    tok_seq = torch.tensor([0, 0, 1, 0, 1], dtype=torch.int32)
    tok_pos = torch.tensor([10, 199, 89, 64, 0], dtype=torch.int32)
    full = ops.attn_generic(q.to(DEV), kv.k_pages, kv.v_pages, kv.table, tok_seq.to(DEV), tok_pos.to(DEV), H, K, hd)
    for i in range(5):
        one = ops.attn_generic(q[i : i + 1].to(DEV), kv.k_pages, kv.v_pages, kv.table, tok_seq[i : i + 1].to(DEV), tok_pos[i : i + 1].to(DEV), H, K, hd)
        assert torch.equal(one[0], full[i])


@pytest.mark.parametrize("H, K, hd", [(8, 2, 128), (6, 2, 24), (5, 1, 64), (3, 3, 256), (16, 2, 40), (40, 2, 64)])
@pytest.mark.parametrize("n_splits, window", [(1, 0), (3, 0), (8, 0), (2, 100)])
def test_attn_decode(ops, H, K, hd, n_splits, window):
    lens = [1, 64, 65, 300, 128]
    S = len(lens)
    kv = PagedKV(lens, K, hd, torch.bfloat16, seed=3)
    q = bf16_round(torch.randn(S, (H + 2 * K) * hd))
    scratch = torch.full((ops.attn_decode_scratch_floats(S, H, hd, n_splits) + 7,), float("nan"), device=DEV)
    seq_len = torch.tensor(lens, dtype=torch.int32, device=DEV)
    out = ops.attn_decode(q.to(torch.bfloat16).to(DEV), kv.k_pages, kv.v_pages, kv.table, seq_len, H, K, hd, n_splits, scratch, window=window,
                          impl="warp")  # (the one-warp kernel, also at the head sizes that "auto" gives to the TMA kernel)
    ref = torch.cat([
        ref_attention_rows(q[s : s + 1, : H * hd].view(1, H, hd), kv, s, [lens[s] - 1], window) for s in range(S)
    ]).view(S, H * hd)
    close_bf16(out, ref)
    assert torch.isnan(scratch[-7:]).all()  # the kernel stays inside the scratch it asked for


@pytest.mark.parametrize("H, K", [(8, 2), (4, 4), (32, 8), (24, 1), (5, 1)])
@pytest.mark.parametrize("n_splits, window", [(1, 0), (3, 0), (8, 0), (2, 100), (64, 0), (5, 333)])
@pytest.mark.parametrize("hd", [128, 64])
def test_attn_decode_tma(ops, H, K, n_splits, window, hd):
    """The four-warp kernel on a TMA-fed ring of pages (head sizes 64 and 128): lengths that end at a page's
    first and last key and inside a warp's 16 keys, more splits than pages (empty splits), groups
    of 1, 4, 5 and 24 query heads per kv head (fewer than 8, and more than one block per kv head)."""
    lens = [1, 64, 65, 300, 128, 1000, 17]
    S = len(lens)
    kv = PagedKV(lens, K, hd, torch.bfloat16, seed=3)
    q = bf16_round(torch.randn(S, (H + 2 * K) * hd))
    scratch = torch.full((ops.attn_decode_scratch_floats(S, H, hd, n_splits) + 7,), float("nan"), device=DEV)
    seq_len = torch.tensor(lens, dtype=torch.int32, device=DEV)
    out = ops.attn_decode(q.to(torch.bfloat16).to(DEV), kv.k_pages, kv.v_pages, kv.table, seq_len, H, K, hd, n_splits, scratch,
                          window=window, impl="tma")
    torch.cuda.synchronize()
    ops.tc_status_check()
    ref = torch.cat([
        ref_attention_rows(q[s : s + 1, : H * hd].view(1, H, hd), kv, s, [lens[s] - 1], window) for s in range(S)
    ]).view(S, H * hd)
    close_bf16(out, ref)
    assert torch.isnan(scratch[-7:]).all()  # the kernel stays inside the scratch it asked for


@pytest.mark.parametrize("H, K", [(8, 2), (32, 8), (24, 1)])
@pytest.mark.parametrize("hd, rot, interleaved", [(128, 128, False), (128, 128, True), (128, 64, False), (128, 0, False),
                                                  (64, 64, False), (64, 64, True), (64, 32, False), (64, 0, False), (64, 24, True)])
@pytest.mark.parametrize("n_splits, window", [(1, 0), (4, 0), (3, 150)])
def test_attn_decode_tma_with_rotary_and_cache_write_fused(ops, H, K, hd, rot, interleaved, n_splits, window):
    """fuse = 2 against the two kernels it stands for (rope_kv_write, then attention): the same keys
    and values end up in the cache, bit for bit, at a page's first and last slot and in every warp's
    quarter of a page, and the same attention comes out; fuse = 1 turns the queries only."""
    lens = [1, 64, 65, 300, 128, 1000, 17, 81, 112]
    S = len(lens)
    kv = PagedKV(lens, K, hd, torch.bfloat16, seed=9)
    g = torch.Generator().manual_seed(rot + H)
    raw = bf16_round(torch.randn(S, (H + 2 * K) * hd, generator=g)).to(torch.bfloat16).to(DEV)
    inv_freq = (10000.0 ** (-torch.arange(0, max(rot, 2), 2, dtype=torch.float32) / max(rot, 2))).to(DEV)
    seq_len = torch.tensor(lens, dtype=torch.int32, device=DEV)
    tok_pos = (seq_len - 1).contiguous()
    tok_seq = torch.arange(S, dtype=torch.int32, device=DEV)
    scratch = torch.empty(ops.attn_decode_scratch_floats(S, H, hd, n_splits), device=DEV)
    # the two-kernel way, on copies
    qkv_a, k_a, v_a = raw.clone(), kv.k_pages.clone(), kv.v_pages.clone()
    ops.rope_kv_write(qkv_a, tok_pos, tok_seq, kv.table, k_a, v_a, inv_freq if rot else None, H, K, hd, rot, interleaved, write_kv=True)
    out_a = ops.attn_decode(qkv_a, k_a, v_a, kv.table, seq_len, H, K, hd, n_splits, scratch, window=window, impl="tma").clone()
    # the fused way: the new position's slot holds junk before the call
    qkv_b, k_b, v_b = raw.clone(), kv.k_pages.clone(), kv.v_pages.clone()
    out_b = ops.attn_decode(qkv_b, k_b, v_b, kv.table, seq_len, H, K, hd, n_splits, scratch, window=window, impl="tma",
                            fuse=2, inv_freq=inv_freq, rotary_dim=rot, interleaved=interleaved)
    torch.cuda.synchronize()
    ops.tc_status_check()
    assert torch.equal(k_b, k_a) and torch.equal(v_b, v_a)  # the cache holds what the rotary kernel would have stored
    assert torch.equal(qkv_b, raw)  # the projection's output is only read
    assert torch.equal(out_b, out_a)
    # and the two-kernel way is right: against the plain formula for one sequence
    s = 3
    q_rot = qkv_a[s : s + 1, : H * hd].float().cpu().view(1, H, hd)
    k_all = torch.stack([k_a[int(kv.table[s, p // PAGE]), :, p % PAGE].float().cpu() for p in range(lens[s])])  # [len, K, hd]
    ref = torch.zeros(H, hd, dtype=torch.float64)
    lo = max(0, lens[s] - window) if window else 0
    for h in range(H):
        kh = h // (H // K)
        sc = (k_all[lo:, kh].double() @ q_rot[0, h].double()) / math.sqrt(hd)
        vv = torch.stack([v_a[int(kv.table[s, p // PAGE]), kh, p % PAGE].float().cpu() for p in range(lo, lens[s])]).double()
        ref[h] = torch.softmax(sc, dim=0) @ vv
    close_bf16(out_b[s].view(H, hd), ref)
    # queries only (the cache is complete, as when a layer reads another layer's cache)
    out_c = ops.attn_decode(raw.clone(), k_a, v_a, kv.table, seq_len, H, K, hd, n_splits, scratch, window=window, impl="tma",
                            fuse=1, inv_freq=inv_freq, rotary_dim=rot, interleaved=interleaved)
    assert torch.equal(out_c, out_a)


@pytest.mark.parametrize("H, K", [(8, 2), (32, 8), (24, 1)])
@pytest.mark.parametrize("n_splits, window", [(1, 0), (4, 0), (64, 0), (3, 150)])
@pytest.mark.parametrize("hd", [128, 64])
def test_attn_decode_tma_adds_its_splits_up_itself(ops, H, K, n_splits, window, hd):
    """With counters the block that finishes last merges the splits: the same result as with the merge
    kernel, call after call (the counters are zeros again each time), also with splits that hold no key."""
    lens = [1, 64, 65, 300, 128, 1000, 17]
    S = len(lens)
    kv = PagedKV(lens, K, hd, torch.bfloat16, seed=6)
    q = bf16_round(torch.randn(S, (H + 2 * K) * hd)).to(torch.bfloat16).to(DEV)
    seq_len = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scratch = torch.empty(ops.attn_decode_scratch_floats(S, H, hd, n_splits), device=DEV)
    two = ops.attn_decode(q, kv.k_pages, kv.v_pages, kv.table, seq_len, H, K, hd, n_splits, scratch, window=window, impl="tma").clone()
    groups = K * ((H // K + 7) // 8)
    counters = torch.zeros(S * groups + 3, dtype=torch.int32, device=DEV)
    for _ in range(3):
        one = ops.attn_decode(q, kv.k_pages, kv.v_pages, kv.table, seq_len, H, K, hd, n_splits, scratch, window=window, impl="tma",
                              counters=counters, out=torch.full((S, H * hd), float("nan"), dtype=torch.bfloat16, device=DEV))
        torch.cuda.synchronize()
        ops.tc_status_check()
        assert int(counters.abs().sum()) == 0
        close_bf16(one, two.double())
        assert float((one.float() - two.float()).abs().max()) <= 2.0 ** -7 * float(two.float().abs().max())  # sums in another order at most
    ref = torch.cat([
        ref_attention_rows(q[s : s + 1, : H * hd].float().cpu().view(1, H, hd), kv, s, [lens[s] - 1], window) for s in range(S)
    ]).view(S, H * hd)
    close_bf16(one, ref)


@pytest.mark.parametrize("parts", [1, 3])
@pytest.mark.parametrize("fuse", [1, 2])
@pytest.mark.parametrize("hd", [128, 64])
def test_attn_decode_tma_takes_the_projection_as_partial_sums(ops, parts, fuse, hd):
    """The fused kernel fed with float32 partial sums [parts, S, columns] of the projection against the
    same kernel fed with their bfloat16 sum: the same cache contents and the same result, bit for bit."""
    H, K, rot = 8, 2, hd
    lens = [1, 64, 65, 300, 128, 17]
    S = len(lens)
    kv = PagedKV(lens, K, hd, torch.bfloat16, seed=12)
    g = torch.Generator().manual_seed(parts)
    pieces = torch.randn(parts, S, (H + 2 * K) * hd, generator=g).to(DEV)
    whole = pieces.sum(dim=0) if parts > 1 else pieces[0]
    # the sum the kernel makes: part after part in 32-bit
    acc = torch.zeros_like(pieces[0])
    for p in range(parts):
        acc = acc + pieces[p]
    raw = acc.to(torch.bfloat16)
    inv_freq = (10000.0 ** (-torch.arange(0, rot, 2, dtype=torch.float32) / rot)).to(DEV)
    seq_len = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scratch = torch.empty(ops.attn_decode_scratch_floats(S, H, hd, 2), device=DEV)
    k_a, v_a, k_b, v_b = kv.k_pages.clone(), kv.v_pages.clone(), kv.k_pages.clone(), kv.v_pages.clone()
    kw = dict(impl="tma", fuse=fuse, inv_freq=inv_freq, rotary_dim=rot, interleaved=False)
    out_a = ops.attn_decode(raw, k_a, v_a, kv.table, seq_len, H, K, hd, 2, scratch, **kw).clone()
    out_b = ops.attn_decode(pieces, k_b, v_b, kv.table, seq_len, H, K, hd, 2, scratch, **kw)
    torch.cuda.synchronize()
    ops.tc_status_check()
    assert out_b.dtype == torch.bfloat16 and torch.equal(out_b, out_a)
    assert torch.equal(k_b, k_a) and torch.equal(v_b, v_a)
    if fuse == 2:
        assert not torch.equal(k_a, kv.k_pages)  # the new keys were stored
    with pytest.raises(Exception, match="fuse > 0"):
        ops.attn_decode(pieces, k_b, v_b, kv.table, seq_len, H, K, hd, 2, scratch, impl="tma")


@pytest.mark.parametrize("hd", [128, 64])
def test_attn_decode_tma_finds_a_far_key(ops, hd):
    """One key far back among hundreds carries almost all the weight: a kernel that skips a page, a
    split, a warp's 16 keys or a swizzled piece returns something else entirely."""
    H, K = 4, 1
    for far in (0, 15, 16, 63, 64, 127, 450, 512):
        kv = PagedKV([513], K, hd, torch.bfloat16, seed=4)
        q = bf16_round(torch.randn(1, H * hd))
        page, slot = int(kv.table[0, far // PAGE]), far % PAGE
        boost = bf16_round(q.view(H, hd).mean(dim=0) * 4)
        kv.k[0][far, 0] = boost
        kv.k_pages[page, 0, slot] = boost.to(torch.bfloat16).to(DEV)
        qq = bf16_round(boost.repeat(H) * 1.0)[None]
        scratch = torch.empty(ops.attn_decode_scratch_floats(1, H, hd, 4), device=DEV)
        out = ops.attn_decode(qq.to(torch.bfloat16).to(DEV), kv.k_pages, kv.v_pages, kv.table, torch.tensor([513], dtype=torch.int32, device=DEV),
                              H, K, hd, 4, scratch, impl="tma")
        torch.cuda.synchronize()
        ops.tc_status_check()
        ref = ref_attention_rows(qq.view(1, H, hd), kv, 0, [512]).view(1, H * hd)
        close_bf16(out, ref)
        assert float((ref.view(H, hd)[0] - kv.v[0][far, 0].double()).abs().max()) < 0.05


def test_attn_decode_finds_a_far_key(ops):
    """One key far back among hundreds carries almost all the weight: a kernel that skips a page,
    a split or a tile edge returns something else entirely."""
    H, K, hd = 4, 1, 64
    for far in (0, 63, 64, 127, 450):
        kv = PagedKV([513], K, hd, torch.bfloat16, seed=4)
        q = bf16_round(torch.randn(1, H * hd))
        # make key `far` point along each head's query
        page, slot = int(kv.table[0, far // PAGE]), far % PAGE
        boost = bf16_round(q.view(H, hd).mean(dim=0) * 4)
        kv.k[0][far, 0] = boost
        kv.k_pages[page, 0, slot] = boost.to(torch.bfloat16).to(DEV)
        qq = bf16_round(boost.repeat(H) * 1.0)[None]
        scratch = torch.empty(ops.attn_decode_scratch_floats(1, H, hd, 4), device=DEV)
        out = ops.attn_decode(qq.to(torch.bfloat16).to(DEV), kv.k_pages, kv.v_pages, kv.table, torch.tensor([513], dtype=torch.int32, device=DEV), H, K, hd, 4, scratch, impl="warp")
        ref = ref_attention_rows(qq.view(1, H, hd), kv, 0, [512]).view(1, H * hd)
        close_bf16(out, ref)
        # and the weight really is on that key
        assert float((ref.view(H, hd)[0] - kv.v[0][far, 0].double()).abs().max()) < 0.05


@pytest.mark.parametrize("H, K, hd", [(4, 2, 128), (6, 6, 24), (5, 1, 64), (2, 1, 256), (8, 2, 40)])
@pytest.mark.parametrize("window", [0, 70])
def test_flash_prefill(ops, H, K, hd, window):
    # sequence 0: a whole prompt; 1: a chunk appended to 100 cached positions; 2: a single row deep in a sequence;
    # 3: exactly one tile
    pos0 = [0, 100, 199, 0]
    q_lens = [150, 77, 1, 64]
    lens = [p + n for p, n in zip(pos0, q_lens)]
    kv = PagedKV(lens, K, hd, torch.bfloat16, seed=5)
    T = sum(q_lens)
    q = bf16_round(torch.randn(T, H * hd + 24))
    seq_start = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32, device=DEV)
    out = ops.flash_prefill(
        q.to(torch.bfloat16).to(DEV), kv.k_pages, kv.v_pages, kv.table, seq_start,
        torch.tensor(pos0, dtype=torch.int32, device=DEV), max(q_lens), H, K, hd, window=window,
    )
    refs, at = [], 0
    for s, (p, n) in enumerate(zip(pos0, q_lens)):
        refs.append(ref_attention_rows(q[at : at + n, : H * hd].view(n, H, hd), kv, s, list(range(p, p + n)), window))
        at += n
    close_bf16(out, torch.cat(refs).view(T, H * hd))


@pytest.mark.parametrize("H, K", [(4, 2), (3, 3), (8, 1)])
@pytest.mark.parametrize("window", [0, 200])
@pytest.mark.parametrize("hd", [128, 64])
def test_flash_prefill_tc(ops, H, K, window, hd):
    """The tcgen05 prompt-attention kernel (head sizes 64 and 128): whole prompts, a chunk behind cached positions,
    single rows, tile-sized and ragged lengths, several key tiles per row tile."""
    pos0 = [0, 100, 199, 0, 300]
    q_lens = [150, 77, 1, 128, 257]
    lens = [p + n for p, n in zip(pos0, q_lens)]
    kv = PagedKV(lens, K, hd, torch.bfloat16, seed=15)
    T = sum(q_lens)
    q = bf16_round(torch.randn(T, (H + 2 * K) * hd))
    seq_start = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32, device=DEV)
    out = ops.flash_prefill_tc(
        q.to(torch.bfloat16).to(DEV), kv.k_pages, kv.v_pages, kv.table, seq_start,
        torch.tensor(pos0, dtype=torch.int32, device=DEV), max(q_lens), H, K, hd, window=window,
    )
    torch.cuda.synchronize()
    ops.tc_status_check()
    refs, at = [], 0
    for s, (p, n) in enumerate(zip(pos0, q_lens)):
        refs.append(ref_attention_rows(q[at : at + n, : H * hd].view(n, H, hd), kv, s, list(range(p, p + n)), window))
        at += n
    close_bf16(out, torch.cat(refs).view(T, H * hd))


@pytest.mark.parametrize("hd", [128, 64])
def test_long_context_attention_kernels(ops, hd):
    """20 000 cached positions (313 pages in a scrambled table): a chunk of 200 prompt rows appended far
    into the sequence through the tcgen05 kernel, then a decode row through the TMA kernel with few and
    many key splits, with and without a window.  One key far back (position 77) is made to matter, so
    that a page skipped hundreds of pages away would show."""
    H, K = 4, 2
    n, q_len = 20000, 200
    kv = PagedKV([n], K, hd, torch.bfloat16, seed=31, extra_pages=5)
    g = torch.Generator().manual_seed(7)
    q = bf16_round(torch.randn(q_len, (H + 2 * K) * hd, generator=g))
    far = 77
    boost = bf16_round(q[-1, :hd] * 0.6)  # along the last row's first head
    kv.k[0][far, 0] = boost
    kv.k_pages[int(kv.table[0, far // PAGE]), 0, far % PAGE] = boost.to(torch.bfloat16).to(DEV)
    qd = q.to(torch.bfloat16).to(DEV)
    pos0 = n - q_len
    for window in (0, 5000):
        out = ops.flash_prefill_tc(qd, kv.k_pages, kv.v_pages, kv.table, torch.tensor([0, q_len], dtype=torch.int32, device=DEV),
                                   torch.tensor([pos0], dtype=torch.int32, device=DEV), q_len, H, K, hd, window=window)
        torch.cuda.synchronize()
        ops.tc_status_check()
        rows = [0, 63, 64, 127, 128, 199]
        ref = ref_attention_rows(q[rows, : H * hd].view(len(rows), H, hd), kv, 0, [pos0 + r for r in rows], window).view(len(rows), H * hd)
        close_bf16(out[rows], ref)
        for n_splits in (3, 64):
            scratch = torch.empty(ops.attn_decode_scratch_floats(1, H, hd, n_splits), device=DEV)
            dec = ops.attn_decode(qd[-1:], kv.k_pages, kv.v_pages, kv.table, torch.tensor([n], dtype=torch.int32, device=DEV),
                                  H, K, hd, n_splits, scratch, window=window, impl="tma")
            torch.cuda.synchronize()
            ops.tc_status_check()
            close_bf16(dec, ref[-1:])
    # without a window the far key carries visible weight in the last row's first head
    full = ref_attention_rows(q[-1:, : H * hd].view(1, H, hd), kv, 0, [n - 1], 0).view(H, hd)
    near = ref_attention_rows(q[-1:, : H * hd].view(1, H, hd), kv, 0, [n - 1], 5000).view(H, hd)
    assert float((full[0] - near[0]).abs().max()) > 0.05


@pytest.mark.parametrize("hd", [128, 64])
def test_flash_prefill_tc_whole_prompts_of_the_benchmarks_length(ops, hd):
    """Two whole prompts in one call, 2113 and 700 tokens from position 0 (17 and 6 row tiles, up to 34 key tiles
    for a row tile; blocks are handed out with the longest row tiles first): rows at tile edges, in the middle and
    at the ends against the float64 attention, and one early key that late rows must still see."""
    H, K = 4, 2
    q_lens = [2113, 700]
    kv = PagedKV(q_lens, K, hd, torch.bfloat16, seed=41)
    T = sum(q_lens)
    q = bf16_round(torch.randn(T, (H + 2 * K) * hd, generator=torch.Generator().manual_seed(8)))
    far = 3
    boost = bf16_round(q[2100, :hd] * 1.0)  # along row 2100's first head
    kv.k[0][far, 0] = boost
    kv.k_pages[int(kv.table[0, far // PAGE]), 0, far % PAGE] = boost.to(torch.bfloat16).to(DEV)
    out = ops.flash_prefill_tc(
        q.to(torch.bfloat16).to(DEV), kv.k_pages, kv.v_pages, kv.table, torch.tensor([0, q_lens[0], T], dtype=torch.int32, device=DEV),
        torch.tensor([0, 0], dtype=torch.int32, device=DEV), max(q_lens), H, K, hd,
    )
    torch.cuda.synchronize()
    ops.tc_status_check()
    for s, (start, rows) in enumerate([(0, [0, 1, 63, 64, 127, 128, 1000, 1023, 1024, 2047, 2048, 2100, 2111, 2112]), (q_lens[0], [0, 64, 639, 640, 699])]):
        qr = q[[start + r for r in rows], : H * hd].view(len(rows), H, hd)
        ref = ref_attention_rows(qr, kv, s, rows).view(len(rows), H * hd)
        close_bf16(out[[start + r for r in rows]], ref)
    # the early key carries visible weight in row 2100's first head (so a row tile that skipped its first key tile fails above)
    scores = (kv.k[0][:2101, 0].double() @ q[2100, :hd].double()) / math.sqrt(hd)
    assert float(torch.softmax(scores, dim=0)[far]) > 0.2


@pytest.mark.parametrize("hd", [128, 64])
def test_flash_prefill_tc_each_key_and_dimension_lands_where_it_should(ops, hd):
    """Values that name their own key and dimension, queries that each pick one key: any mix-up of pages,
    swizzled pieces, k steps or the transposed V operand shows as a wrong number, not as noise."""
    H, K, n = 1, 1, 320
    kv = PagedKV([n], K, hd, torch.bfloat16, seed=16)
    # keys: orthogonal-ish directions; query t points at key pick(t) <= t
    keys = bf16_round(torch.randn(n, hd, generator=torch.Generator().manual_seed(3)))
    vals = torch.zeros(n, hd)
    vals[torch.arange(n), torch.arange(n) % hd] = 1.0  # value row t is a one-hot at dimension t % 128
    vals += (torch.arange(n)[:, None] // hd) * 0.25    # plus a step that tells the three 128-key tiles apart
    vals = bf16_round(vals)
    pick = (torch.arange(n) * 5) % (torch.arange(n) + 1)
    q = bf16_round(keys[pick] * 2.0)
    for t in range(n):
        page, slot = int(kv.table[0, t // PAGE]), t % PAGE
        kv.k_pages[page, 0, slot] = keys[t].to(torch.bfloat16).to(DEV)
        kv.v_pages[page, 0, slot] = vals[t].to(torch.bfloat16).to(DEV)
    kv.k[0][:, 0] = keys
    kv.v[0][:, 0] = vals
    out = ops.flash_prefill_tc(
        q.to(torch.bfloat16).to(DEV), kv.k_pages, kv.v_pages, kv.table, torch.tensor([0, n], dtype=torch.int32, device=DEV),
        torch.tensor([0], dtype=torch.int32, device=DEV), n, H, K, hd,
    )
    torch.cuda.synchronize()
    ops.tc_status_check()
    ref = ref_attention_rows(q.view(n, H, hd), kv, 0, list(range(n))).view(n, hd)
    close_bf16(out, ref)
    # the picked key dominates: the output is close to that key's value row
    got = out.float().cpu()
    assert float((got - vals[pick]).abs().max()) < 0.1


def test_flash_prefill_finds_a_far_key_and_respects_the_causal_edge(ops):
    H, K, hd = 2, 1, 64
    n = 400
    kv = PagedKV([n], K, hd, torch.bfloat16, seed=6)
    direction = bf16_round(torch.randn(hd))
    far = 130
    kv.k[0][far, 0] = direction * 3
    kv.k_pages[int(kv.table[0, far // PAGE]), 0, far % PAGE] = (direction * 3).to(torch.bfloat16).to(DEV)
    q = bf16_round(direction.repeat(n, H) * 1.0)
    out = ops.flash_prefill(
        q.to(torch.bfloat16).to(DEV), kv.k_pages, kv.v_pages, kv.table, torch.tensor([0, n], dtype=torch.int32, device=DEV),
        torch.tensor([0], dtype=torch.int32, device=DEV), n, H, K, hd,
    )
    ref = ref_attention_rows(q.view(n, H, hd), kv, 0, list(range(n))).view(n, H * hd)
    close_bf16(out, ref)
    # rows before the far key cannot see it, rows from it on are dominated by its value
    v_far = kv.v[0][far, 0].double()
    assert float((ref[far + 5].view(H, hd)[0] - v_far).abs().max()) < 0.05
    assert float((ref[far - 1].view(H, hd)[0] - v_far).abs().max()) > 0.5
    got = out.float().cpu().view(n, H, hd)
    assert float((got[far, 0] - v_far.float()).abs().max()) < 0.08 and float((got[far - 1, 0] - v_far.float()).abs().max()) > 0.5


# --------------------------------------------------------------------------- matrix products
@pytest.mark.parametrize("M, N, K", [(1, 130, 50), (70, 130, 50), (5, 64, 17), (129, 65, 257)])
def test_gemm_f32(ops, M, N, K):
    x, w = torch.randn(M, K), torch.randn(N, K)
    out = ops.gemm_f32(x.to(DEV), w.to(DEV))
    close_f32(out, x.double() @ w.double().T, 1e-6)


def test_gemm_f32_rows_do_not_depend_on_the_batch(ops):
    x, w = torch.randn(100, 300).to(DEV), torch.randn(77, 300).to(DEV)
    full = ops.gemm_f32(x, w)
    for r in (0, 63, 64, 99):
        assert torch.equal(ops.gemm_f32(x[r : r + 1], w)[0], full[r])
    assert torch.equal(ops.gemm_f32(x[10:50], w), full[10:50])


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 17, 33, 64])
@pytest.mark.parametrize("N, K", [(100, 72), (48, 4096), (257, 1000)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemv_bf16(ops, M, N, K, out_dtype):
    x = bf16_round(torch.randn(M, K))
    w = bf16_round(torch.randn(N, K) * 0.05)
    buf, out = guarded_out(M, N, out_dtype)
    ops.gemv_bf16(x.to(torch.bfloat16).to(DEV), w.to(torch.bfloat16).to(DEV), out_dtype, out=out)
    assert untouched(buf, M, N)
    if out_dtype == torch.float32:
        close_dot_f32(out, x, w)
    else:
        close_bf16(out, x.double() @ w.double().T)


@pytest.mark.parametrize(
    "M, N, K",
    [(128, 256, 64), (128, 256, 256), (200, 300, 72), (2048, 512, 4096), (65, 1000, 1000), (129, 257, 4104),
     (640, 17920, 128), (1280, 25600, 64)],  # the last two give every block several tiles: both accumulators, many rounds
)
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tc(ops, M, N, K, out_dtype):
    """The tcgen05 kernel at full tiles, at ragged edges in M, N and K, and with a long K; the result goes
    into the middle of a NaN-filled buffer whose surroundings must stay as they were."""
    g = torch.Generator().manual_seed(M + N + K)
    x = bf16_round(torch.randn(M, K, generator=g))
    w = bf16_round(torch.randn(N, K, generator=g) * 0.05)
    buf, out = guarded_out(M, N, out_dtype)
    ops.gemm_tc(x.to(torch.bfloat16).to(DEV), w.to(torch.bfloat16).to(DEV), out_dtype, out=out)
    torch.cuda.synchronize()
    ops.tc_status_check()
    assert untouched(buf, M, N)
    if out_dtype == torch.float32:
        close_dot_f32(out, x, w)
    else:
        close_bf16(out, x.double() @ w.double().T)


@pytest.mark.parametrize("M, N, K, splits", [(64, 512, 4096, 8), (20, 300, 1000, 3), (200, 256, 640, 64), (64, 4096, 14336, 8)])
def test_gemm_tc_partial_sums_over_k_slices(ops, M, N, K, splits):
    g = torch.Generator().manual_seed(M + N)
    x = bf16_round(torch.randn(M, K, generator=g))
    w = bf16_round(torch.randn(N, K, generator=g) * 0.05)
    parts = ops.gemm_tc(x.to(torch.bfloat16).to(DEV), w.to(torch.bfloat16).to(DEV), torch.float32, k_splits=splits)
    torch.cuda.synchronize()
    ops.tc_status_check()
    assert parts.dim() == 3 and parts.shape[1:] == (M, N) and 1 < parts.shape[0] <= splits
    close_dot_f32(parts.sum(dim=0), x, w)
    per = ((K + 63) // 64 + parts.shape[0] - 1) // parts.shape[0] * 64
    for i in range(parts.shape[0]):
        close_dot_f32(parts[i], x[:, i * per : (i + 1) * per], w[:, i * per : (i + 1) * per])


def test_gemm_tc_each_output_sees_its_own_row_and_column(ops):
    """x = one-hot rows, w = distinct rows: out[m, n] must be w[n, pick(m)], which exposes any mix-up of
    rows, columns, k slices or the swizzle."""
    M, N, K = 512, 768, 320
    pick = torch.arange(M) * 7 % K
    x = torch.zeros(M, K)
    x[torch.arange(M), pick] = 1.0
    w = bf16_round(torch.randn(N, K, generator=torch.Generator().manual_seed(1)))
    out = ops.gemm_tc(x.to(torch.bfloat16).to(DEV), w.to(torch.bfloat16).to(DEV), torch.float32)
    torch.cuda.synchronize()
    ops.tc_status_check()
    assert torch.equal(out.cpu(), w[:, pick].T.contiguous())


@pytest.mark.parametrize("M", [1, 8, 40, 64, 65, 300])
@pytest.mark.parametrize("ff, K", [(100, 72), (1432, 512)])
def test_fused_gate_up_swiglu(ops, M, ff, K):
    """silu(x Wg^T) * (x Wu^T) from one kernel over row-interleaved weights, for decode-sized and
    prompt-sized M (the streaming kernel and the tcgen05 kernel)."""
    from rusty_llama_b200.kernels.linear import linear_swiglu

    g = torch.Generator().manual_seed(M + ff)
    x = bf16_round(torch.randn(M, K, generator=g))
    wg = bf16_round(torch.randn(ff, K, generator=g) * 0.1)
    wu = bf16_round(torch.randn(ff, K, generator=g) * 0.1)
    w = torch.stack([wg, wu], dim=1).reshape(2 * ff, K)
    out = linear_swiglu(x.to(torch.bfloat16).to(DEV), w.to(torch.bfloat16).to(DEV))
    torch.cuda.synchronize()
    ops.tc_status_check()
    assert out.shape == (M, ff)
    ref = plain_silu(x.double() @ wg.double().T) * (x.double() @ wu.double().T)
    close_bf16(out, ref)


@pytest.mark.parametrize("M, N, K, splits", [(8, 100, 4096, 4), (1, 48, 1000, 3), (64, 257, 2048, 8), (3, 16, 72, 2)])
def test_gemv_bf16_partial_sums_over_k_slices(ops, M, N, K, splits):
    x = bf16_round(torch.randn(M, K))
    w = bf16_round(torch.randn(N, K) * 0.05)
    parts = ops.gemv_bf16(x.to(torch.bfloat16).to(DEV), w.to(torch.bfloat16).to(DEV), torch.float32, k_splits=splits)
    assert parts.shape == (splits, M, N) and parts.dtype == torch.float32
    close_dot_f32(parts.sum(dim=0), x, w)
    # each slice really is its own range of k
    per = ((K + 31) // 32 + splits - 1) // splits * 32
    for i in range(splits):
        lo, hi = i * per, min(K, (i + 1) * per)
        if lo < hi:
            close_dot_f32(parts[i], x[:, lo:hi], w[:, lo:hi])
        else:
            assert float(parts[i].abs().max()) == 0.0


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N, K", [(100, 64), (48, 4096), (257, 960), (4099, 2112), (20000, 1024), (72, 5120), (40, 4160)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemv_stream(ops, M, N, K, out_dtype):
    """The persistent TMA-fed kernel: row counts on both sides of 8, feature counts that are no
    multiple of 8 (a last unit with fewer rows), k that ends inside a stage, fewer items than SMs
    and many items per block."""
    g = torch.Generator().manual_seed(M * 7 + N)
    x = bf16_round(torch.randn(M, K, generator=g))
    w = bf16_round(torch.randn(N, K, generator=g) * 0.05)
    buf, out = guarded_out(M, N, out_dtype)
    ops.gemv_stream(x.to(torch.bfloat16).to(DEV), w.to(torch.bfloat16).to(DEV), out_dtype, out=out)
    torch.cuda.synchronize()
    ops.tc_status_check()
    assert untouched(buf, M, N)
    if out_dtype == torch.float32:
        close_dot_f32(out, x, w)
    else:
        close_bf16(out, x.double() @ w.double().T)


@pytest.mark.parametrize("M, N, K, splits", [(8, 100, 4096, 4), (1, 48, 960, 3), (16, 257, 3136, 2), (3, 4096, 14336, 7), (8, 24, 2048, 2), (9, 40, 14336, 2), (2, 24, 10304, 2), (8, 16, 5184, 2)])
def test_gemv_stream_partial_sums_over_k_slices(ops, M, N, K, splits):
    x = bf16_round(torch.randn(M, K))
    w = bf16_round(torch.randn(N, K) * 0.05)
    parts = ops.gemv_stream(x.to(torch.bfloat16).to(DEV), w.to(torch.bfloat16).to(DEV), torch.float32, k_splits=splits)
    torch.cuda.synchronize()
    ops.tc_status_check()
    chunks = (K + 1023) // 1024
    per = min(5 if K > 4096 else 4, (chunks + min(splits, chunks) - 1) // min(splits, chunks))  # a slice is at most 4096 long, 5120 when k is longer than that
    used = (chunks + per - 1) // per
    assert used == ops.gemv_stream_slices(M, K, splits)
    if used == 1:
        assert parts.shape == (M, N)
        close_dot_f32(parts, x, w)
        return
    assert parts.shape == (used, M, N) and parts.dtype == torch.float32
    close_dot_f32(parts.sum(dim=0), x, w)
    for i in range(used):  # each slice really is its own range of k
        lo, hi = i * per * 1024, min(K, (i + 1) * per * 1024)
        close_dot_f32(parts[i], x[:, lo:hi], w[:, lo:hi])


@pytest.mark.parametrize("M", [1, 8, 13])
@pytest.mark.parametrize("ff, K", [(100, 64), (1432, 512), (7168, 1024), (104, 5120)])
def test_gemv_stream_fused_swiglu(ops, M, ff, K):
    g = torch.Generator().manual_seed(M + ff)
    x = bf16_round(torch.randn(M, K, generator=g))
    wg = bf16_round(torch.randn(ff, K, generator=g) * 0.1)
    wu = bf16_round(torch.randn(ff, K, generator=g) * 0.1)
    w = torch.stack([wg, wu], dim=1).reshape(2 * ff, K)
    buf, out = guarded_out(M, ff, torch.bfloat16)
    ops.gemv_stream(x.to(torch.bfloat16).to(DEV), w.to(torch.bfloat16).to(DEV), out=out, swiglu=True)
    torch.cuda.synchronize()
    ops.tc_status_check()
    assert untouched(buf, M, ff)
    close_bf16(out, plain_silu(x.double() @ wg.double().T) * (x.double() @ wu.double().T))


def test_gemv_stream_strided_operands_and_repeat(ops):
    """Operands that are column slices of wider tensors, and the same bits on every run."""
    big_x = bf16_round(torch.randn(5, 3000))
    big_w = bf16_round(torch.randn(300, 2600) * 0.05)
    xd, wd = big_x.to(torch.bfloat16).to(DEV), big_w.to(torch.bfloat16).to(DEV)
    x, w = xd[:, 8 : 8 + 2048], wd[:, 16 : 16 + 2048]
    out = ops.gemv_stream(x, w, torch.float32)
    close_dot_f32(out, big_x[:, 8 : 8 + 2048], big_w[:, 16 : 16 + 2048])
    assert torch.equal(out, ops.gemv_stream(x, w, torch.float32))


def test_gemv_stream_refuses_what_it_cannot_do(ops):
    from rusty_llama_b200.errors import KernelError

    with pytest.raises(KernelError, match="multiple of 64"):
        ops.gemv_stream(torch.zeros(2, 72, dtype=torch.bfloat16, device=DEV), torch.zeros(8, 72, dtype=torch.bfloat16, device=DEV))
    assert ops.gemv_stream_slices(2, 72) == 0
    with pytest.raises(KernelError, match="at most 16"):
        ops.gemv_stream(torch.zeros(17, 64, dtype=torch.bfloat16, device=DEV), torch.zeros(8, 64, dtype=torch.bfloat16, device=DEV))
    assert ops.gemv_stream_slices(16, 4096) == 1 and ops.gemv_stream_slices(16, 5120) == 1 and ops.gemv_stream_slices(16, 5184) == 2
    assert ops.gemv_stream_slices(16, 14336) == 3   # a block keeps at most 5120 activations per row
    assert ops.gemv_stream_slices(16, 14336, 7) == 7
    with pytest.raises(KernelError, match="comes in 3 slices"):
        ops.gemv_stream(torch.zeros(16, 14336, dtype=torch.bfloat16, device=DEV), torch.zeros(8, 14336, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(KernelError, match="comes in 3 slices"):  # also with a 32-bit result: there is room for one result only
        ops.gemv_stream(torch.zeros(2, 10304, dtype=torch.bfloat16, device=DEV), torch.zeros(8, 10304, dtype=torch.bfloat16, device=DEV), torch.float32)


@pytest.mark.parametrize("M", [1, 5, 8])
@pytest.mark.parametrize("d, q_dim, ff, norm_dtype", [(256, 128, 320, torch.float32), (1024, 2048, 2752, torch.bfloat16), (4096, 4096, 14336, torch.bfloat16), (192, 64, 96, torch.float32), (5120, 5120, 1728, torch.bfloat16), (4608, 4160, 200, torch.float32)])
def test_gemv_stream_with_a_folded_norm(ops, M, d, q_dim, ff, norm_dtype):
    """An RMSNorm folded into the two products around it: the first adds its sums to the 32-bit stream, writes
    x * w beside it and leaves the rows' sums of squares; the second takes x * w and scales its sums by the rows'
    1 / sqrt(mean(x^2) + eps).  Against the three steps done plainly in float64 (stream, norm, gated product),
    with roundings to bfloat16 where the kernels store bfloat16."""
    g = torch.Generator().manual_seed(M + d)
    a = bf16_round(torch.randn(M, q_dim, generator=g))
    w_o = bf16_round(torch.randn(d, q_dim, generator=g) * (q_dim ** -0.5))
    x = torch.randn(M, d, generator=g) * 2
    nw = (1 + 0.1 * torch.randn(d, generator=g)).to(norm_dtype)
    wg = bf16_round(torch.randn(ff, d, generator=g) * (d ** -0.5))
    wu = bf16_round(torch.randn(ff, d, generator=g) * (d ** -0.5))
    w_gu = torch.stack([wg, wu], dim=1).reshape(2 * ff, d)
    eps = 1e-5
    xd = x.to(DEV)
    xw, sumsq, blocks = ops.gemv_stream_into_stream(a.to(torch.bfloat16).to(DEV), w_o.to(torch.bfloat16).to(DEV), xd, nw.to(DEV))
    torch.cuda.synchronize()
    ops.tc_status_check()
    x_new = x.double() + a.double() @ w_o.double().T
    close_f32(xd, x_new, 2e-6)
    got_x = xd.cpu().double()
    assert torch.equal(xw.cpu(), (xd.cpu() * nw.float()).to(torch.bfloat16))  # x * w from the stream as stored, rounded once
    shares = sumsq[: blocks * 8].view(blocks, 8).cpu().double()
    close_f32(shares.sum(dim=0)[:M], (got_x * got_x).sum(dim=1), 1e-5)
    assert float(shares[:, M:].abs().max()) == 0.0 if M < 8 else True
    buf, h = guarded_out(M, ff, torch.bfloat16)
    ops.gemv_stream(xw, w_gu.to(torch.bfloat16).to(DEV), torch.bfloat16, out=h, swiglu=True, row_scale=(sumsq, blocks, d, eps))
    torch.cuda.synchronize()
    ops.tc_status_check()
    assert untouched(buf, M, ff)
    inv = 1.0 / torch.sqrt((got_x * got_x).mean(dim=1, keepdim=True) + eps)
    xwf = xw.float().cpu().double()
    close_bf16(h, plain_silu((xwf @ wg.double().T) * inv) * ((xwf @ wu.double().T) * inv))
    # and that is the plain norm followed by the plain gated product, up to the roundings
    xn = bf16_round(plain_rmsnorm(got_x, nw.double(), eps).float()).double()
    close_bf16(h, plain_silu(xn @ wg.double().T) * (xn @ wu.double().T))
    # a plain (not gated) product with a row scale, 32-bit out
    out = ops.gemv_stream(xw, wg.to(torch.bfloat16).to(DEV), torch.float32, row_scale=(sumsq, blocks, d, eps))
    close_f32(out, (xwf @ wg.double().T) * inv, 3e-5)


def test_add_rmsnorm_takes_float32_partial_sums_in_a_bfloat16_run(ops):
    T, d = 6, 520
    x = torch.randn(T, d)
    parts = torch.randn(3, T, d)
    w = (1 + 0.1 * torch.randn(d)).to(torch.bfloat16)
    xd = x.to(DEV)
    out = ops.add_rmsnorm(xd, parts.to(DEV), w.to(DEV), 1e-5, torch.bfloat16)
    total = x + parts[0] + parts[1] + parts[2]
    close_f32(xd, total, 1e-6)
    close_bf16(out, plain_rmsnorm(total.double(), w.double(), 1e-5))


def test_gemv_bf16_refuses_what_it_cannot_do(ops):
    from rusty_llama_b200.errors import KernelError

    x = torch.zeros(2, 20, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(8, 20, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(KernelError, match="multiples of 8"):
        ops.gemv_bf16(x, w)
    with pytest.raises(KernelError, match="at most 64"):
        ops.gemv_bf16(torch.zeros(65, 16, dtype=torch.bfloat16, device=DEV), torch.zeros(8, 16, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(KernelError, match="CUDA only"):
        ops.gemv_bf16(x.cpu(), w.cpu())


@pytest.mark.parametrize("M, N, K", [(1, 34, 100), (7, 258, 250), (70, 130, 129), (200, 66, 1001)])
@pytest.mark.parametrize("swiglu", [False, True])
def test_gemm_bf16_any_takes_every_k(ops, M, N, K, swiglu):
    """The plain FMA kernel behind the shapes that the 16-byte-row kernels refuse: any k, rows that start
    anywhere."""
    g = torch.Generator().manual_seed(M * N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / K ** 0.5).to(torch.bfloat16)
    ref = x.double() @ w.double().t()
    if swiglu:
        gate, up = ref[:, 0::2], ref[:, 1::2]
        ref = gate / (1 + torch.exp(-gate)) * up
    for out_dtype in (torch.bfloat16, torch.float32):
        got = ops.gemm_bf16_any(x.to(DEV), w.to(DEV), out_dtype, swiglu=swiglu).cpu().double()
        assert got.shape == ref.shape
        err = (got - ref).abs().max().item()
        bound = 2e-5 * ref.abs().max().item() + (ref.abs().max().item() * 2 ** -8 if out_dtype == torch.bfloat16 else 0)
        assert err <= bound + 1e-6, f"{out_dtype}: {err} against {bound}"


# --------------------------------------------------------------------------- sampling
def test_argmax_last_of_ties(ops):
    logits = torch.randn(6, 1000)
    logits[0, [5, 700, 999]] = 9.0
    logits[1, :] = 1.0
    logits[2, 0] = 50.0
    out = ops.argmax(logits.to(DEV)).cpu().tolist()
    assert out == [plain_argmax(row.tolist()) for row in logits]
    assert out[0] == 999 and out[1] == 999 and out[2] == 0


def test_argmax_with_nans_follows_the_reference(ops):
    """The reference's comparison `!(best > x)` lets a NaN take the running maximum's place and whatever
    follows take the NaN's (src/sampler.rs:76-84, test :983-988): the winner is the last of the equal maxima
    among the elements after the row's last NaN, or that NaN when it ends the row."""
    nan = float("nan")
    small = [[1.0, nan, 0.5], [nan, 3.0, 2.0], [5.0, 1.0, nan], [nan, nan, nan], [2.0, nan, 1.0, 1.0], [nan, 9.0, nan, 0.0, -1.0]]
    for row in small:
        got = ops.argmax(torch.tensor([row], device=DEV)).item()
        assert got == plain_argmax(row), f"{row}: kernel {got}, reference {plain_argmax(row)}"
    assert plain_argmax([1.0, nan, 0.5]) == 2 and plain_argmax([5.0, 1.0, nan]) == 2  # the reference's own cases
    g = torch.Generator().manual_seed(5)
    big = torch.randn(6, 5003, generator=g)
    big[0, 4000] = nan                      # the maximum before the NaN does not count
    big[0, 100] = 50.0
    big[1, [7, 4999]] = nan                 # two NaNs: only what follows the last one counts
    big[2, 5002] = nan                      # a NaN at the end wins
    big[3, 0] = nan                         # a NaN at the start changes nothing
    big[4, 2500:] = nan                     # a tail of NaNs
    want = [plain_argmax(r.tolist()) for r in big]
    assert want[0] > 4000 and want[1] > 4999 and want[2] == 5002 and want[4] == 5002
    assert ops.argmax(big.to(DEV)).cpu().tolist() == want


def draw_interval(logits64, temperature, top_p, token):
    """[lo, hi) of `token` in the exact (float64) cumulative distribution that a draw runs over, and the mass the
    coin is scaled by: all tokens in index order, or with 0 < top_p < 1 the nucleus in descending order of
    probability (src/sampler.rs:116-164, :190-216)."""
    z = logits64 / temperature
    p = np.exp(z - z.max())
    p /= p.sum()
    n = len(p)
    if not (0.0 < top_p < 1.0):
        cum = np.cumsum(p)
        return (cum[token - 1] if token else 0.0), cum[token], 1.0
    kept = np.nonzero(p >= (1.0 - top_p) / max(n - 1, 1))[0]
    order = kept[np.argsort(-p[kept], kind="stable")]
    cum = np.cumsum(p[order])
    last = int(np.argmax(cum > top_p)) if (cum > top_p).any() else len(order) - 1
    where = np.nonzero(order[: last + 2] == token)[0]
    assert len(where) == 1, f"token {token} is not in the nucleus of {last + 1} tokens"
    k = int(where[0])
    return (cum[k - 1] if k else 0.0), cum[k], cum[last]


@pytest.mark.parametrize("rows", [1, 8, 64])
def test_sample_kernels_at_a_vocabulary_of_128256(ops, rows):
    """The classifier's width in the benchmark: greedy, temperature and temperature + top-p for 1, 8 and 64 rows,
    each row with its own seed; a few rows of each batch are replayed by the plain sampler (it is slow), all rows
    must be valid and the same on a second run from the same states."""
    n = 128256
    g = torch.Generator().manual_seed(rows)
    logits = torch.randn(rows, n, generator=g) * 3.0
    ld = logits.to(DEV)
    assert ops.argmax(ld).cpu().tolist() == [int(r.argmax()) for r in logits]  # (no ties in random floats)
    seeds = [1000 + 17 * r for r in range(rows)]
    index = torch.arange(rows, dtype=torch.int32, device=DEV)
    scratch = torch.empty(rows * n, device=DEV)
    check = sorted({0, rows // 2, rows - 1})
    for temperature, top_p in ((0.8, 0.0), (1.1, 0.9)):
        states = torch.from_numpy(np.array(seeds, dtype=np.uint64).view(np.int64).copy()).to(DEV)
        got = ops.sample(ld, temperature, top_p, states, index, scratch).cpu().tolist()
        again_states = torch.from_numpy(np.array(seeds, dtype=np.uint64).view(np.int64).copy()).to(DEV)
        assert ops.sample(ld, temperature, top_p, again_states, index, scratch).cpu().tolist() == got
        for r in range(rows):
            # Over 128k probabilities of 1e-5 or so each, the reference's running 32-bit sum (src/sampler.rs:205-214)
            # is itself off by more than one token's probability, so the draw is checked against the exact
            # distribution instead: the coin, times the kept mass, must lie in the chosen token's own interval of
            # the cumulative distribution, give or take the 32-bit sum's error (sqrt(n) roundings of 2^-24: 2e-5).
            lo, hi, mass = draw_interval(logits[r].double().numpy(), temperature, top_p, got[r])
            target = PlainRng(seeds[r]).next_f32() * mass
            assert lo - 1e-4 <= target < hi + 1e-4, f"row {r}: token {got[r]} owns [{lo}, {hi}), the draw was {target}"
        for r in check[:1]:  # (slow) the plain sampler itself, which must at least land next to the kernel's token
            want = plain_sample(logits[r].tolist(), temperature, top_p, PlainRng(seeds[r]))
            lo, hi, mass = draw_interval(logits[r].double().numpy(), temperature, top_p, want)
            target = PlainRng(seeds[r]).next_f32() * mass
            assert lo - 1e-3 <= target < hi + 1e-3
    # the longer chain on the same rows: top-k, then the nucleus, then min-p, then the draw
    history = torch.zeros(rows, ops.SAMPLE_HISTORY_MAX, dtype=torch.int32, device=DEV)
    count = torch.zeros(rows, dtype=torch.int32, device=DEV)
    work = torch.empty(rows * 2 * n, device=DEV)
    states = torch.from_numpy(np.array(seeds, dtype=np.uint64).view(np.int64).copy()).to(DEV)
    got = ops.sample_chain(ld, 0.9, 0.95, 50, 0.01, 1.0, 0, 0.0, 0.0, states, index, history, count, work).cpu().tolist()
    for r in check:
        want = PlainChain(temperature=0.9, top_p=0.95, top_k=50, min_p=0.01, seed=seeds[r]).sample(logits[r].numpy())
        assert got[r] == want, f"row {r}: chain kernel {got[r]}, plain {want}"


@pytest.mark.parametrize("n, temperature, top_p", [(300, 1.0, 0.9), (300, 0.7, 0.0), (5000, 1.3, 0.5), (5000, 0.8, 0.95), (8, 1.0, 0.9)])
def test_sample_follows_the_plain_sampler(ops, n, temperature, top_p):
    rows = 6
    g = torch.Generator().manual_seed(n)
    logits = torch.randn(rows, n, generator=g) * 2.0
    logits[1] = torch.round(logits[1] * 2) / 2  # many equal probabilities
    logits[2, 3] = 30.0  # one dominant token
    if n == 8:
        logits[0] = torch.tensor([2.0, 1.8, 1.6, 1.4, 1.2, 1.0, 0.8, 0.6])
    seeds = [12345, 1, 2, 3, 99, 2**63 + 5]
    states = torch.from_numpy(np.array(seeds, dtype=np.uint64).view(np.int64).copy()).to(DEV)
    index = torch.arange(rows, dtype=torch.int32, device=DEV)
    scratch = torch.empty(rows * n, device=DEV)
    rngs = [PlainRng(s) for s in seeds]
    ld = logits.to(DEV)
    draws, total, same = 12, 0, 0
    for d in range(draws):
        got = ops.sample(ld, temperature, top_p, states, index, scratch).cpu().tolist()
        want = [plain_sample(logits[r].tolist(), temperature, top_p, rngs[r]) for r in range(rows)]
        total += rows
        same += sum(int(a == b) for a, b in zip(got, want))
        if n == 8 and top_p == 0.9 and d < 8:
            assert got[0] == [2, 4, 0, 4, 0, 0, 6, 2][d]  # the reference's golden stream (src/sampler.rs:1009-1014)
    # tokens of equal probability are ordered by the reference's unstable sort, here by index; rows without
    # ties must agree draw for draw
    assert same >= total - draws, f"{total - same} of {total} draws differ"
    # the generator states advanced exactly as the plain ones
    want_states = np.array([r.state for r in rngs], dtype=np.uint64)
    assert np.array_equal(states.cpu().numpy().view(np.uint64), want_states)


@pytest.mark.parametrize("n, temperature, top_p", [(9000, 0.8, 0.5), (20000, 1.0, 0.0), (40001, 0.9, 0.9), (40001, 1.5, 0.99)])
def test_sample_rows_shared_by_several_blocks(ops, n, temperature, top_p):
    """Rows long enough that 2, 4 and 8 blocks share one (a length that is no multiple of 4 among them):
    the blocks' sums, histograms and counts have to meet in index order."""
    rows = 4
    g = torch.Generator().manual_seed(n)
    logits = torch.randn(rows, n, generator=g) * 2.5
    logits[1] = torch.round(logits[1] * 2) / 2  # many equal probabilities, spread over all blocks
    logits[2, n - 2] = 30.0  # one dominant token in the last block's part
    logits[3, :] = -20.0
    logits[3, [1, n // 2, n - 1]] = torch.tensor([3.0, 3.0, 3.0])  # equals in the first, a middle and the last part
    seeds = [4242, 17, 3, 2**62 + 11]
    states = torch.from_numpy(np.array(seeds, dtype=np.uint64).view(np.int64).copy()).to(DEV)
    index = torch.arange(rows, dtype=torch.int32, device=DEV)
    scratch = torch.empty(rows * n, device=DEV)
    rngs = [PlainRng(s) for s in seeds]
    ld = logits.to(DEV)
    draws = 5
    for d in range(draws):
        got = ops.sample(ld, temperature, top_p, states, index, scratch).cpu().tolist()
        want = [plain_sample(logits[r].tolist(), temperature, top_p, rngs[r]) for r in range(rows)]
        assert got[0] == want[0] and got[2] == want[2], f"draw {d}: {got} against {want}"
        # equal probabilities are ordered by the reference's unstable sort, here by index: the draw lands
        # on the same value, maybe at another index
        assert logits[1, got[1]] == logits[1, want[1]]
        # the three equal tokens hold nearly all the mass: whichever the coin picks, it is one of them
        assert got[3] in (1, n // 2, n - 1) and want[3] in (1, n // 2, n - 1)
    want_states = np.array([r.state for r in rngs], dtype=np.uint64)
    assert np.array_equal(states.cpu().numpy().view(np.uint64), want_states)


CHAINS = [
    dict(temperature=0.8, top_p=0.9, top_k=40),
    dict(temperature=1.0, top_p=0.0, top_k=5),
    dict(temperature=1.2, top_p=0.95, min_p=0.05),
    dict(temperature=0.7, top_p=0.0, min_p=0.2, top_k=50),
    dict(temperature=1.0, top_p=0.9, repeat_penalty=1.3, repeat_last_n=8),
    dict(temperature=1.0, top_p=0.0, frequency_penalty=0.7, presence_penalty=0.4, repeat_last_n=5),
    dict(temperature=0.0, top_p=0.9, repeat_penalty=1.5, frequency_penalty=0.3, repeat_last_n=64),
    dict(temperature=0.9, top_p=0.8, top_k=30, min_p=0.02, repeat_penalty=1.1, presence_penalty=0.2, repeat_last_n=16),
    dict(temperature=1.0, top_p=0.9, top_k=1),
    dict(temperature=1.5, top_p=0.3, min_p=1.5),
    dict(temperature=0.8, top_p=0.0, xtc_probability=0.7, xtc_threshold=0.02),
    dict(temperature=1.0, top_p=0.95, top_k=50, xtc_probability=1.0, xtc_threshold=0.05),
    dict(temperature=0.0, top_p=0.0, xtc_probability=1.0, xtc_threshold=0.01),
    dict(temperature=0.9, top_p=0.9, min_p=0.01, repeat_penalty=1.2, repeat_last_n=8, xtc_probability=0.5, xtc_threshold=0.1),
    dict(temperature=1.0, top_p=0.0, top_k=3, xtc_probability=1.0, xtc_threshold=0.0),
]


@pytest.mark.parametrize("n", [300, 20001])
@pytest.mark.parametrize("chain", CHAINS, ids=lambda c: ",".join(f"{k}={v}" for k, v in c.items()))
def test_sample_chain_follows_the_plain_chain(ops, n, chain):
    """penalties -> top-k -> top-p -> min-p -> temperature -> draw against the reference's stages run one
    after the other on the host: rows without equal logits agree draw for draw, the chosen tokens feed the
    penalties of the next draw, and the generator advances once per drawn token (never for the argmax)."""
    rows, slots = 3, 5
    g = torch.Generator().manual_seed(n + len(chain))
    logits = [torch.randn(rows, n, generator=g) * 2.5 for _ in range(10)]
    for l in logits:
        l[1, 7] = 9.0  # a dominant token: penalties have something to push down
    seeds = [11, 2**40 + 3, 7]
    slot_of_row = [4, 0, 2]
    states = torch.ones(slots, dtype=torch.int64, device=DEV)
    states[slot_of_row] = torch.tensor(seeds, dtype=torch.int64, device=DEV)
    index = torch.tensor(slot_of_row, dtype=torch.int32, device=DEV)
    history = torch.zeros(slots, 1024, dtype=torch.int32, device=DEV)
    count = torch.zeros(slots, dtype=torch.int32, device=DEV)
    work = torch.empty(rows * 2 * ((n + 3) // 4 * 4), device=DEV)
    c = dict(temperature=1.0, top_p=0.9, top_k=0, min_p=0.0, repeat_penalty=1.0, repeat_last_n=64, frequency_penalty=0.0, presence_penalty=0.0,
             xtc_probability=0.0, xtc_threshold=0.1)
    c.update(chain)
    xtc_states = states.clone()  # XTC's own generator starts from the same seeds
    penalties = c["repeat_penalty"] != 1.0 or c["frequency_penalty"] != 0.0 or c["presence_penalty"] != 0.0
    plain = [PlainChain(seed=s, **c) for s in seeds]
    # (with XTC the candidates stay in index order on the draws where its gate does not open)
    index_order = c["top_k"] == 0 and c["min_p"] == 0.0 and not (0.0 < c["top_p"] < 1.0) and n > 10000
    for d, l in enumerate(logits):
        got = ops.sample_chain(
            l.to(DEV), c["temperature"], c["top_p"], c["top_k"], c["min_p"], c["repeat_penalty"],
            c["repeat_last_n"] if penalties else 0, c["frequency_penalty"], c["presence_penalty"], states, index, history, count, work,
            xtc_probability=c["xtc_probability"], xtc_threshold=c["xtc_threshold"], xtc_states=xtc_states,
        ).cpu().tolist()
        want = [plain[r].sample(l[r].tolist()) for r in range(rows)]
        if got != want and index_order:
            # a walk over the whole row in index order: the plain chain adds 20001 probabilities one after the
            # other in 32-bit, the kernel in blocks; a draw within that rounding of a boundary may take the
            # neighbour (or the one after, where the token between them has next to no mass).  The penalties then go
            # on from the kernel's token.
            for r in range(rows):
                assert abs(got[r] - want[r]) <= 3, f"draw {d}: {got} against {want}"
                if plain[r].ring:
                    plain[r].ring[-1] = got[r]
        else:
            assert got == want, f"draw {d}: {got} against {want}"
    want_states = np.array([p.rng.state for p in plain], dtype=np.uint64)
    assert np.array_equal(states.cpu().numpy().view(np.uint64)[slot_of_row], want_states)
    if penalties:
        assert count.cpu().tolist() == [10 if s in slot_of_row else 0 for s in range(slots)]
    if c["xtc_probability"] > 0.0:
        want_xtc = np.array([p.xtc_rng.state for p in plain], dtype=np.uint64)
        assert np.array_equal(xtc_states.cpu().numpy().view(np.uint64)[slot_of_row], want_xtc)


@pytest.mark.parametrize("n", [300, 20001])
@pytest.mark.parametrize("mode, tau, eta, t, penalised", [(2, 3.0, 0.1, 0.8, False), (2, 6.0, 0.3, 1.2, True), (1, 3.0, 0.1, 0.9, False), (1, 5.0, 0.2, 1.0, True)])
def test_sample_chain_mirostat_follows_the_plain_chain(ops, n, mode, tau, eta, t, penalised):
    """Mirostat 1 and 2 (penalties -> temperature -> its own cut and draw): the same tokens as the plain chain
    draw after draw, with the surprise ceiling mu carried from one draw to the next on the device."""
    rows = 3
    g = torch.Generator().manual_seed(n + mode)
    logits = [torch.randn(rows, n, generator=g) * 3.0 for _ in range(12)]
    seeds = [5, 2**33 + 1, 77]
    states = torch.tensor(seeds, dtype=torch.int64, device=DEV)
    index = torch.arange(rows, dtype=torch.int32, device=DEV)
    history = torch.zeros(rows, 1024, dtype=torch.int32, device=DEV)
    count = torch.zeros(rows, dtype=torch.int32, device=DEV)
    mu = torch.full((rows,), float("nan"), device=DEV)
    work = torch.empty(rows * 2 * ((n + 3) // 4 * 4), device=DEV)
    pen = dict(repeat_penalty=1.2, presence_penalty=0.3, repeat_last_n=8) if penalised else {}
    plain = [PlainChain(temperature=t, seed=s, mirostat=mode, mirostat_lr=eta, mirostat_ent=tau, **pen) for s in seeds]
    same = total = 0
    for d, l in enumerate(logits):
        got = ops.sample_chain(
            l.to(DEV), t, 0.9, 0, 0.0, pen.get("repeat_penalty", 1.0), pen.get("repeat_last_n", 0) if penalised else 0, 0.0,
            pen.get("presence_penalty", 0.0), states, index, history, count, work, mirostat=mode, mirostat_tau=tau, mirostat_eta=eta,
            mirostat_mu=mu,
        ).cpu().tolist()
        want = [plain[r].sample(l[r].tolist()) for r in range(rows)]
        for r in range(rows):
            total += 1
            if got[r] == want[r]:
                same += 1
            else:
                # (mirostat 1 rounds a real number down to the count of candidates it keeps, from sums of a hundred
                # logarithms: a count that differs by one now and then moves a draw); go on from the kernel's state
                plain[r].mu = np.float32(mu[r].item())
                if plain[r].ring:
                    plain[r].ring[-1] = got[r]
        got_mu = mu.cpu().numpy()
        want_mu = np.array([p.mu for p in plain], dtype=np.float32)
        for r in range(rows):
            if got[r] == want[r]:
                assert abs(got_mu[r] - want_mu[r]) <= 2e-4 * max(1.0, abs(want_mu[r])), f"draw {d} row {r}: mu {got_mu[r]} against {want_mu[r]}"
    assert same >= total - (0 if mode == 2 else 3), f"{total - same} of {total} draws differ"
    assert np.array_equal(states.cpu().numpy().view(np.uint64), np.array([p.rng.state for p in plain], dtype=np.uint64))


@pytest.mark.parametrize("n", [12, 9000])
@pytest.mark.parametrize("extra", [dict(), dict(repeat_penalty=1.1, repeat_last_n=5), dict(dry_sequence_breakers=(2,)), dict(mirostat=2, mirostat_ent=2.0)])
def test_sample_chain_dry_follows_the_plain_chain(ops, n, extra):
    """DRY over a history in which stretches do repeat (a handful of likely tokens), with its own window beside
    the penalties' window, with a breaker token, and inside the mirostat mode: the plain chain's tokens draw for
    draw, 80 draws, so the ring of 1024 places is read at many phases."""
    rows = 2
    g = torch.Generator().manual_seed(n)
    seeds = [9, 2**35 + 7]
    states = torch.tensor(seeds, dtype=torch.int64, device=DEV)
    index = torch.arange(rows, dtype=torch.int32, device=DEV)
    history = torch.zeros(rows, 1024, dtype=torch.int32, device=DEV)
    count = torch.zeros(rows, dtype=torch.int32, device=DEV)
    mu = torch.full((rows,), float("nan"), device=DEV)
    work = torch.empty(rows * 2 * ((n + 3) // 4 * 4), device=DEV)
    knobs = dict(temperature=0.9, top_p=0.0, dry_multiplier=0.8, dry_base=1.75, dry_allowed_length=2, dry_penalty_last_n=16, repeat_last_n=0)
    knobs.update(extra)
    plain = [PlainChain(seed=s, **knobs) for s in seeds]
    penalised = knobs.get("repeat_penalty", 1.0) != 1.0
    same = 0
    for d in range(80):
        l = torch.randn(rows, n, generator=g)
        l[:, :5] += 7.0  # five likely tokens: their stretches repeat soon
        got = ops.sample_chain(
            l.to(DEV), knobs["temperature"], knobs["top_p"], 0, 0.0, knobs.get("repeat_penalty", 1.0),
            knobs["repeat_last_n"] if penalised else 0, 0.0, 0.0, states, index, history, count, work,
            mirostat=knobs.get("mirostat", 0), mirostat_tau=knobs.get("mirostat_ent", 5.0), mirostat_eta=0.1, mirostat_mu=mu,
            dry_multiplier=knobs["dry_multiplier"], dry_base=knobs["dry_base"], dry_allowed_length=knobs["dry_allowed_length"],
            dry_last_n=knobs["dry_penalty_last_n"], dry_breakers=knobs.get("dry_sequence_breakers", ()),
        ).cpu().tolist()
        want = [plain[r].sample(l[r].tolist()) for r in range(rows)]
        if got != want:
            # (without a filter the walk is in index order over the whole row: a draw within rounding of a boundary
            # may take the neighbour; the histories then go on from the kernel's token)
            assert n > 1000 and all(abs(a - b) <= 3 for a, b in zip(got, want)), f"draw {d}: {got} against {want}"
            for r in range(rows):
                for ring in (plain[r].ring, plain[r].dry_ring):
                    if ring:
                        ring[-1] = got[r]
        else:
            same += 1
    assert same >= 76
    assert count.cpu().tolist() == [80, 80]


def test_sample_chain_on_the_reference_cases(ops):
    """The kernel on the inputs and outcomes of the reference's own unit tests of its stages
    (src/sampler.rs:1064-1211)."""

    def run(logits, draws=1, ring=(), seed=3, **kw):
        c = dict(temperature=1.0, top_p=0.0, top_k=0, min_p=0.0, repeat_penalty=1.0, repeat_last_n=64, frequency_penalty=0.0,
                 presence_penalty=0.0, mirostat=0, mirostat_tau=5.0, mirostat_eta=0.1, xtc_probability=0.0, xtc_threshold=0.1,
                 dry_multiplier=0.0, dry_base=1.75, dry_allowed_length=2, dry_last_n=0, dry_breakers=())
        c.update(kw)
        n = len(logits)
        l = torch.tensor([logits], dtype=torch.float32, device=DEV)
        states = torch.tensor([seed], dtype=torch.int64, device=DEV)
        history = torch.zeros(1, 1024, dtype=torch.int32, device=DEV)
        count = torch.zeros(1, dtype=torch.int32, device=DEV)
        last_n = c["repeat_last_n"]
        for t in ring:  # as the kernel itself files chosen tokens
            history[0, int(count.item()) % 1024] = t
            count += 1
        mu = torch.full((1,), float("nan"), device=DEV)
        work = torch.empty(2 * ((n + 3) // 4 * 4), device=DEV)
        out = [
            ops.sample_chain(
                l, c["temperature"], c["top_p"], c["top_k"], c["min_p"], c["repeat_penalty"], last_n, c["frequency_penalty"],
                c["presence_penalty"], states, torch.zeros(1, dtype=torch.int32, device=DEV), history, count, work,
                mirostat=c["mirostat"], mirostat_tau=c["mirostat_tau"], mirostat_eta=c["mirostat_eta"], mirostat_mu=mu,
                xtc_probability=c["xtc_probability"], xtc_threshold=c["xtc_threshold"], xtc_states=states.clone(),
                dry_multiplier=c["dry_multiplier"], dry_base=c["dry_base"], dry_allowed_length=c["dry_allowed_length"],
                dry_last_n=c["dry_last_n"], dry_breakers=c["dry_breakers"],
            ).item()
            for _ in range(draws)
        ]
        return out, mu.item()

    assert set(run([3.0, 1.0, 4.0, 1.0, 5.0], draws=40, top_k=2)[0]) == {2, 4}
    assert set(run([10.0, 9.0, 2.0, 1.0], draws=20, min_p=0.5)[0]) == {0}
    assert run([4.5, 1.0, 5.0], ring=[2], temperature=0.0, repeat_penalty=1.3)[0] == [0]
    assert run([0.0, 0.0, 0.0], ring=[0, 1, 2], temperature=0.0, presence_penalty=5.0, repeat_last_n=2)[0] == [0]
    assert run([0.0, 0.0, -1.5], ring=[0, 0, 1], temperature=0.0, frequency_penalty=1.0)[0] == [1]
    assert run([0.0, 0.0, -0.5], ring=[0, 0, 1], temperature=0.0, frequency_penalty=1.0)[0] == [2]
    got, mu = run([10.0, 0.0, 0.0], seed=1, mirostat=2, repeat_last_n=0)
    assert got == [0] and abs(mu - 10.5) < 1e-4
    assert run([10.0, 9.0, 0.0, -1.0], seed=7, temperature=0.0, xtc_probability=1.0, xtc_threshold=0.2)[0] == [1]
    assert run([1.0, 2.0, 3.0, 4.0, 5.0], xtc_probability=1.0, xtc_threshold=0.0)[0] == [0]
    assert run([10.0, 9.0, 0.0, -1.0], temperature=0.0, top_k=4, xtc_probability=0.0)[0] == [0]
    # dry_short_repeat_at_allowed_length_boundary_hand_computed (src/sampler.rs:1247-1262): after A, B, A the
    # token B would repeat "A, B": a repeat of 2 = the allowed length, so it loses the bare multiplier
    dry = dict(temperature=0.0, repeat_last_n=0, dry_multiplier=1.0, dry_base=2.0, dry_allowed_length=2, dry_last_n=64)
    assert run([0.0, 0.0, 0.5], ring=[1, 2, 1], **dry)[0] == [1]   # token 2 at 0.5 - 1.0 falls behind; last of the equal 0, 1
    assert run([0.0, 0.0, 1.5], ring=[1, 2, 1], **dry)[0] == [2]   # 1.5 - 1.0 still leads
    # dry_no_repeat_no_penalty: all different, nothing changes
    assert run([0.0, 0.3, 0.0, 0.0, 0.0, 0.0], ring=[1, 2, 3, 4, 5], **dry)[0] == [1]
    # a breaker between the two stretches stops the match
    assert run([0.0, 0.0, 0.5, 0.0], ring=[1, 2, 3, 1], **dict(dry, dry_breakers=(3,)))[0] == [2]
    assert run([0.0, 0.0, 0.5, 0.0], ring=[1, 2, 3, 1], **dry)[0] == [3]  # without it, 2 after the last 1 would repeat "1, 2"


def test_sample_chain_takes_equal_logits_in_index_order(ops):
    """Equal logits at the edge of top-k and inside the draw: the first by index stay, as in the plain chain's
    stable sorts."""
    n = 50
    logits = torch.full((1, n), -3.0)
    logits[0, [4, 9, 20, 33, 41]] = 2.0
    logits[0, 12] = 5.0
    states = torch.tensor([99], dtype=torch.int64, device=DEV)
    index = torch.zeros(1, dtype=torch.int32, device=DEV)
    history = torch.zeros(1, 1024, dtype=torch.int32, device=DEV)
    count = torch.zeros(1, dtype=torch.int32, device=DEV)
    work = torch.empty(2 * 52, device=DEV)
    plain = PlainChain(temperature=2.0, top_p=0.0, seed=99, top_k=4)
    seen = set()
    for _ in range(40):
        got = ops.sample_chain(logits.to(DEV), 2.0, 0.0, 4, 0.0, 1.0, 0, 0.0, 0.0, states, index, history, count, work).item()
        assert got == plain.sample(logits[0].tolist())
        seen.add(got)
    assert seen == {12, 4, 9, 20}  # the largest and the first three of the five equals


def test_sample_rows_without_ties_agree_exactly(ops):
    n, rows = 2000, 8
    logits = torch.randn(rows, n, generator=torch.Generator().manual_seed(5)) * 3
    seeds = list(range(1, rows + 1))
    states = torch.tensor(seeds, dtype=torch.int64, device=DEV)
    index = torch.arange(rows, dtype=torch.int32, device=DEV)
    scratch = torch.empty(rows * n, device=DEV)
    rngs = [PlainRng(s) for s in seeds]
    for _ in range(10):
        got = ops.sample(logits.to(DEV), 1.0, 0.9, states, index, scratch).cpu().tolist()
        want = [plain_sample(logits[r].tolist(), 1.0, 0.9, rngs[r]) for r in range(rows)]
        assert got == want


def test_sample_empty_nucleus_collapses_to_argmax(ops):
    # src/sampler.rs:1035-1043: uniform distribution and a tiny top-p
    logits = torch.ones(1, 4, device=DEV)
    states = torch.tensor([7], dtype=torch.int64, device=DEV)
    out = ops.sample(logits, 1.0, 0.1, states, torch.zeros(1, dtype=torch.int32, device=DEV), torch.empty(4, device=DEV))
    assert out.item() == 3 and states.item() != 7  # the coin is still drawn


def test_pipeline_probes_run():
    """The measuring aids of csrc/probe_pipeline.cu on small buffers: no wait runs out, the handshake's consumer
    reports a time for every block, the tensor core is not faster than its nominal rate."""
    import ctypes

    from rusty_llama_b200.kernels import build

    lib = build.load("probe_pipeline")
    lib.rl_error_text.restype = ctypes.c_char_p
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    nbytes = 64 << 20
    buf = torch.zeros(nbytes // 2, dtype=torch.bfloat16, device=DEV)
    for rows, kc, stages, walk in [(8, 1024, 13, 0), (2, 4096, 6, 0), (256, 64, 6, 1), (64, 256, 3, 1)]:
        rc = lib.rl_probe_tma_stream(ctypes.c_void_p(buf.data_ptr()), ctypes.c_longlong(nbytes), ctypes.c_int(4096), ctypes.c_int(rows),
                                     ctypes.c_int(kc), ctypes.c_int(stages), ctypes.c_int(walk), ctypes.c_int(256), ctypes.c_void_p(err.data_ptr()), stream)
        assert rc == 0, lib.rl_error_text().decode()
    rc = lib.rl_probe_tma_stream(ctypes.c_void_p(buf.data_ptr()), ctypes.c_longlong(nbytes), ctypes.c_int(4096), ctypes.c_int(8), ctypes.c_int(1000),
                                 ctypes.c_int(6), ctypes.c_int(0), ctypes.c_int(256), ctypes.c_void_p(err.data_ptr()), stream)
    assert rc < 0  # k per stage must be a multiple of 64
    out = torch.zeros(16, dtype=torch.int64, device=DEV)
    small = torch.zeros(64 * 16 * 64, dtype=torch.bfloat16, device=DEV)
    for mode in (0, 1, 3, 4, 5, 8, 9):
        out.zero_()
        rc = lib.rl_probe_handshake(ctypes.c_void_p(small.data_ptr()), ctypes.c_int(16), ctypes.c_int(mode), ctypes.c_int(4), ctypes.c_int(64),
                                    ctypes.c_int(16), ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(err.data_ptr()), stream)
        assert rc == 0, lib.rl_error_text().decode()
        torch.cuda.synchronize()
        assert int(err.item()) == 0 and int(out.min().item()) > 0
    assert lib.rl_probe_handshake(ctypes.c_void_p(small.data_ptr()), ctypes.c_int(16), ctypes.c_int(2), ctypes.c_int(4), ctypes.c_int(64),
                                  ctypes.c_int(16), ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(err.data_ptr()), stream) < 0
    # the tensor core's rate per instruction: every form runs, no wait runs out, a long run of 128 x 256 x 16 takes at
    # least its nominal 128 cycles an instruction
    rows256 = torch.zeros(256 * 16 * 64, dtype=torch.bfloat16, device=DEV)
    cycles = torch.zeros(2 * 4, dtype=torch.int64, device=DEV)
    for n, form in [(256, 0), (256, 1), (128, 2), (64, 3), (256, 4), (128, 6), (256, 8), (256, 24), (256, 56), (256, 64), (128, 68)]:
        cycles.zero_()
        rc = lib.rl_probe_mma_rate(ctypes.c_void_p(rows256.data_ptr()), ctypes.c_int(16), ctypes.c_int(n), ctypes.c_int(form), ctypes.c_int(512),
                                   ctypes.c_int(4), ctypes.c_void_p(cycles.data_ptr()), ctypes.c_void_p(err.data_ptr()), stream)
        assert rc == 0, lib.rl_error_text().decode()
        torch.cuda.synchronize()
        assert int(err.item()) == 0, f"form {form}: a wait ran out"
        assert int(cycles[:4].min().item()) >= 512 * (n // 2) * 0.98, f"n {n} form {form}: {cycles[:4].tolist()} cycles for 512 instructions"
    assert lib.rl_probe_mma_rate(ctypes.c_void_p(rows256.data_ptr()), ctypes.c_int(16), ctypes.c_int(256), ctypes.c_int(2), ctypes.c_int(512),
                                 ctypes.c_int(4), ctypes.c_void_p(cycles.data_ptr()), ctypes.c_void_p(err.data_ptr()), stream) < 0  # A in tensor memory: n <= 128

