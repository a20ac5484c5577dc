"""The decode-attention entry point that brings its own scratch memory (for callers that cannot
allocate on the device), called through its exported C symbol, twice in a row so that the second call
finds the first call's leftovers in the shared array.  Each result is compared with a float64 attention
computed here from the dense keys and values, and with the ordinary entry point: bit for bit where both run
the same kernel.  One case needs all but a few floats of the array, the next size up is refused.
This file sorts last on purpose: a run that stops at the first failure has then run everything else."""

import ctypes
import math

import pytest
import torch

from test_kernels import PagedKV, bf16_round, close_bf16, ref_attention_rows

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = 64
LIMIT = 1 << 20  # RL_ATTN_DECODE_STATIC_FLOATS


def make_case(lens, H, K, hd, seed):
    kv = PagedKV(list(lens), K, hd, torch.bfloat16, seed=seed)
    q = bf16_round(torch.randn(len(lens), H * hd, generator=torch.Generator().manual_seed(seed + 1)))
    seq_len = torch.tensor(list(lens), dtype=torch.int32, device=DEV)
    return kv, q, q.to(torch.bfloat16).to(DEV), seq_len


def call_static(lib, qd, kv, seq_len, H, K, hd, n_splits, window=0):
    """rl_attn_decode_static through ctypes: inputs and the output only, no scratch argument."""
    S = qd.shape[0]
    out = torch.empty(S, H * hd, dtype=torch.bfloat16, device=DEV)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    i = ctypes.c_int
    rc = lib.rl_attn_decode_static(
        p(qd), i(1), i(qd.stride(0)), p(kv.k_pages), p(kv.v_pages), p(kv.table), i(kv.table.shape[1]), p(seq_len), p(out), i(out.stride(0)),
        i(S), i(H), i(K), i(hd), i(PAGE), i(window), ctypes.c_float(1.0 / math.sqrt(hd)), i(n_splits),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
    )
    return rc, out


def oracle(kv, q, lens, H, hd, window, seqs=None):
    seqs = range(len(lens)) if seqs is None else seqs
    return torch.stack([ref_attention_rows(q[s : s + 1].view(1, H, hd), kv, s, [lens[s] - 1], window).view(H * hd) for s in seqs])


def test_static_scratch_entry_point_matches_float64_attention_and_the_ordinary_one_twice_in_a_row():
    from rusty_llama_b200.kernels import build, ops

    lib = build.load("attention_decode")
    assert hasattr(lib, "rl_attn_decode_static")
    # the later cases are smaller and cut differently: they run over what the earlier ones left in the array
    cases = [((300, 64, 65, 1, 513), 16, 4, 128, 6, 0), ((70, 200), 6, 2, 40, 3, 0), ((300, 90, 513), 8, 2, 64, 4, 100)]
    for lens, H, K, hd, n_splits, window in cases:
        kv, q, qd, seq_len = make_case(lens, H, K, hd, seed=H + hd)
        rc, got = call_static(lib, qd, kv, seq_len, H, K, hd, n_splits, window)
        assert rc == 0, lib.rl_error_text().decode()
        torch.cuda.synchronize()
        close_bf16(got, oracle(kv, q, lens, H, hd, window))
        # the ordinary entry point with the caller's scratch runs the same kernel: the same bits
        scratch = torch.empty(ops.attn_decode_scratch_floats(len(lens), H, hd, n_splits), device=DEV)
        same = ops.attn_decode(qd, kv.k_pages, kv.v_pages, kv.table, seq_len, H, K, hd, n_splits, scratch, window=window, impl="warp")
        assert torch.equal(got, same)


def test_static_scratch_entry_point_at_its_limit():
    """n_seqs * H * n_splits * (hd + 2) floats are needed.  With head sizes that are multiples of 8 no case needs
    exactly 2^20, so the limit is met from both sides within one unit: 4559 * 23 * 1 * (8 + 2) = 1048570 fits
    (and the maxima and sums, which lie behind the outputs at the array's far end, must still be right), while
    52429 * 2 * 1 * (8 + 2) = 1048580 is refused before anything is launched."""
    from rusty_llama_b200.kernels import build, ops

    lib = build.load("attention_decode")
    lib.rl_error_text.restype = ctypes.c_char_p
    S, H, K, hd = 4559, 23, 1, 8
    assert S * H * (hd + 2) <= LIMIT < S * H * (hd + 2) + (hd + 2)
    lens = [1 + (7 * s) % 64 for s in range(S)]
    kv, q, qd, seq_len = make_case(lens, H, K, hd, seed=5)
    rc, got = call_static(lib, qd, kv, seq_len, H, K, hd, 1)
    assert rc == 0, lib.rl_error_text().decode()
    torch.cuda.synchronize()
    some = [0, 1, 63, 64, 2000, S - 2, S - 1]
    close_bf16(got[some], oracle(kv, q, lens, H, hd, 0, some))
    scratch = torch.empty(ops.attn_decode_scratch_floats(S, H, hd, 1), device=DEV)
    assert torch.equal(got, ops.attn_decode(qd, kv.k_pages, kv.v_pages, kv.table, seq_len, H, K, hd, 1, scratch, impl="warp"))
    # one unit more
    S2, H2 = 52429, 2
    assert S2 * H2 * (hd + 2) == S * H * (hd + 2) + (hd + 2) and S2 * H2 * (hd + 2) > LIMIT
    q2 = torch.zeros(S2, H2 * hd, dtype=torch.bfloat16, device=DEV)
    kv2 = PagedKV([1], H2, hd, torch.bfloat16, seed=6)
    kv2.table = torch.zeros(S2, 1, dtype=torch.int32, device=DEV)
    rc, _ = call_static(lib, q2, kv2, torch.ones(S2, dtype=torch.int32, device=DEV), H2, H2, hd, 1)
    assert rc < 0
    text = lib.rl_error_text().decode()
    assert "1048580 floats of scratch" in text and "1048576" in text
    torch.cuda.synchronize()


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from rusty_llama_b200.kernels import build

    lib = build.load("attention_decode")
    lib.rl_error_text.restype = ctypes.c_char_p
    kv, q, qd, seq_len = make_case([64] * 40, 32, 8, 128, seed=1)
    rc, _ = call_static(lib, qd, kv, seq_len, 32, 8, 128, 64)  # 40 * 32 * 64 * 130 floats > 2^20
    assert rc < 0
    text = lib.rl_error_text().decode()
    assert "floats of scratch" in text and "1048576" in text
    torch.cuda.synchronize()
