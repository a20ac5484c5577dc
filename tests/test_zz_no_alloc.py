"""The decode-attention entry point that brings its own scratch memory (for callers that cannot
allocate on the device), called through its exported C symbol and compared with the ordinary entry
point, twice in a row so that the second call finds the first call's leftovers in the shared array.
This file sorts last on purpose: a run that stops at the first failure has then run everything else."""

import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = 64


def make_case(seqs_lens, H, K, hd, seed):
    g = torch.Generator().manual_seed(seed)
    n_pages = sum((n + PAGE - 1) // PAGE for n in seqs_lens) + 2
    k_pages = torch.randn(n_pages, K, PAGE, hd, generator=g).to(torch.bfloat16).to(DEV)
    v_pages = torch.randn(n_pages, K, PAGE, hd, generator=g).to(torch.bfloat16).to(DEV)
    width = max((n + PAGE - 1) // PAGE for n in seqs_lens)
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.zeros(len(seqs_lens), width, dtype=torch.int32)
    for s, n in enumerate(seqs_lens):
        for j in range((n + PAGE - 1) // PAGE):
            table[s, j] = order.pop()
    q = torch.randn(len(seqs_lens), H * hd, generator=g).to(torch.bfloat16).to(DEV)
    seq_len = torch.tensor(seqs_lens, dtype=torch.int32, device=DEV)
    return q, k_pages, v_pages, table.to(DEV), seq_len


def call_static(lib, q, k_pages, v_pages, table, seq_len, H, K, hd, n_splits):
    """rl_attn_decode_static through ctypes: inputs and the output only, no scratch argument."""
    S = q.shape[0]
    out = torch.empty(S, H * hd, dtype=torch.bfloat16, device=DEV)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    i = ctypes.c_int
    rc = lib.rl_attn_decode_static(
        p(q), i(1), i(q.stride(0)), p(k_pages), p(v_pages), p(table), i(table.shape[1]), p(seq_len), p(out), i(out.stride(0)),
        i(S), i(H), i(K), i(hd), i(PAGE), i(0), ctypes.c_float(1.0 / math.sqrt(hd)), i(n_splits),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
    )
    return rc, out


def test_static_scratch_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from rusty_llama_b200.kernels import build, ops

    lib = build.load("attention_decode")
    assert hasattr(lib, "rl_attn_decode_static")
    # the second case is smaller and cut differently: it runs over what the first left in the array
    cases = [((300, 64, 65, 1, 513), 16, 4, 128, 6), ((70, 200), 6, 2, 40, 3)]
    for lens, H, K, hd, n_splits in cases:
        q, kp, vp, table, seq_len = make_case(list(lens), H, K, hd, seed=H + hd)
        scratch = torch.empty(ops.attn_decode_scratch_floats(len(lens), H, hd, n_splits), device=DEV)
        want = ops.attn_decode(q, kp, vp, table, seq_len, H, K, hd, n_splits, scratch)
        rc, got = call_static(lib, q, kp, vp, table, seq_len, H, K, hd, n_splits)
        assert rc == 0, lib.rl_error_text().decode()
        torch.cuda.synchronize()
        err = (got.float() - want.float()).abs()
        scale = float(want.float().abs().max())
        # the tolerance of the other bfloat16 kernel tests; the two entry points run the same kernels
        assert float(err.max()) <= 1.2e-2 * scale and float(err.mean()) <= 2e-3 * scale
        assert torch.isfinite(got.float()).all()


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from rusty_llama_b200.kernels import build

    lib = build.load("attention_decode")
    lib.rl_error_text.restype = ctypes.c_char_p
    q, kp, vp, table, seq_len = make_case([64] * 40, 32, 8, 128, seed=1)
    rc, _ = call_static(lib, q, kp, vp, table, seq_len, 32, 8, 128, 64)  # 40 * 32 * 64 * 130 floats > 2^20
    assert rc < 0
    text = lib.rl_error_text().decode()
    assert "floats of scratch" in text and "1048576" in text
    torch.cuda.synchronize()
