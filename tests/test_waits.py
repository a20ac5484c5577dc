"""The give-up paths of the kernels with bounded waits, taken on purpose and from the host: one role of a
kernel is given a wait limit of zero for one launch (`ops.short_wait`), so its first wait runs out.  The call
must return, the status word must name that role, the other roles must drain (they see the block's abort flag;
the waits that keep a block alive until its copies have landed keep their long limit), the status must read
zero after the check, and the same kernel must give right results on the next launch.  No kernel faults,
traps or hangs for this: the role simply stops waiting.  Counterpart of the reference's `expect()` on every
CUDA call (src/backend/cuda.rs:652, :755): an error the host can read instead of a hang."""

import time

import numpy as np
import pytest
import torch

from test_kernels import DEV, PagedKV, bf16_round, close_bf16, close_dot_f32, ref_attention_rows

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from rusty_llama_b200.kernels import ops as o

    return o


def expect_give_up(ops, code, text, launch):
    """Run `launch` with role `code` on a zero limit; the status check must raise with `text` and clear the word."""
    from rusty_llama_b200.errors import KernelError

    ops.tc_status_check()
    t0 = time.perf_counter()
    with ops.short_wait(code, 0):
        launch()
    torch.cuda.synchronize()
    took = time.perf_counter() - t0
    with pytest.raises(KernelError, match=text) as e:
        ops.tc_status_check()
    assert f"code {code})" in str(e.value)
    assert int(ops._tc_status_word(torch.device(DEV)).item()) == 0
    ops.tc_status_check()  # nothing left to report
    # the other roles leave when they see the abort flag; nobody sits out its second
    assert took < 5.0, f"the abandoned launch took {took:.1f} s"


def test_gemm_tc_issuer_gives_up_and_the_next_launch_is_right(ops):
    g = torch.Generator().manual_seed(1)
    x = bf16_round(torch.randn(200, 512, generator=g))
    w = bf16_round(torch.randn(700, 512, generator=g) * 0.05)
    xd, wd = x.to(torch.bfloat16).to(DEV), w.to(torch.bfloat16).to(DEV)
    expect_give_up(ops, 2, r"gemm_tc: the tensor-core issuer \(for a stage's data\)", lambda: ops.gemm_tc(xd, wd, torch.float32))
    out = ops.gemm_tc(xd, wd, torch.float32)
    torch.cuda.synchronize()
    ops.tc_status_check()
    close_dot_f32(out, x, w)
    # few rows: the kernel asks for its first weights before its activations (the drain has to cope with both)
    expect_give_up(ops, 2, "gemm_tc: the tensor-core issuer", lambda: ops.gemm_tc(xd[:24], wd, torch.float32))
    close_dot_f32(ops.gemm_tc(xd[:24], wd, torch.float32), x[:24], w)
    # an epilogue warp that stops waiting for its accumulator
    expect_give_up(ops, 3, "gemm_tc: an epilogue warp", lambda: ops.gemm_tc(xd, wd, torch.float32))
    close_dot_f32(ops.gemm_tc(xd, wd, torch.float32), x, w)
    ops.tc_status_check()


def test_gemv_stream_product_warp_gives_up_and_the_next_launch_is_right(ops):
    g = torch.Generator().manual_seed(2)
    x = bf16_round(torch.randn(5, 2048, generator=g))
    w = bf16_round(torch.randn(3000, 2048, generator=g) * 0.05)
    xd, wd = x.to(torch.bfloat16).to(DEV), w.to(torch.bfloat16).to(DEV)
    expect_give_up(ops, 34, r"gemv_stream: a product warp \(for a stage's weights\)", lambda: ops.gemv_stream(xd, wd, torch.float32))
    out = ops.gemv_stream(xd, wd, torch.float32)
    torch.cuda.synchronize()
    ops.tc_status_check()
    close_dot_f32(out, x, w)
    expect_give_up(ops, 35, "gemv_stream: a storing warp", lambda: ops.gemv_stream(xd, wd, torch.float32))
    close_dot_f32(ops.gemv_stream(xd, wd, torch.float32), x, w)
    ops.tc_status_check()


def test_attn_decode_tma_product_warp_gives_up_and_the_next_launch_is_right(ops):
    H, K, hd, n = 8, 2, 128, 700
    kv = PagedKV([n], K, hd, torch.bfloat16, seed=3)
    q = bf16_round(torch.randn(1, H * hd, generator=torch.Generator().manual_seed(3)))
    qd = q.to(torch.bfloat16).to(DEV)
    lens = torch.tensor([n], dtype=torch.int32, device=DEV)
    ref = ref_attention_rows(q.view(1, H, hd), kv, 0, [n - 1]).view(1, H * hd)
    for n_splits in (1, 3):
        scratch = torch.zeros(ops.attn_decode_scratch_floats(1, H, hd, n_splits), device=DEV)
        run = lambda: ops.attn_decode(qd, kv.k_pages, kv.v_pages, kv.table, lens, H, K, hd, n_splits, scratch, impl="tma")
        expect_give_up(ops, 52, r"attn_decode_tma: a product warp \(for a page\)", run)
        out = run()
        torch.cuda.synchronize()
        ops.tc_status_check()
        close_bf16(out, ref)


def test_flash_prefill_tc_issuer_gives_up_and_the_next_launch_is_right(ops):
    H, K, hd, n = 2, 1, 128, 300
    kv = PagedKV([n], K, hd, torch.bfloat16, seed=4)
    q = bf16_round(torch.randn(n, H * hd, generator=torch.Generator().manual_seed(4)))
    qd = q.to(torch.bfloat16).to(DEV)
    start = torch.tensor([0, n], dtype=torch.int32, device=DEV)
    pos0 = torch.tensor([0], dtype=torch.int32, device=DEV)
    run = lambda: ops.flash_prefill_tc(qd, kv.k_pages, kv.v_pages, kv.table, start, pos0, n, H, K, hd)
    ref = ref_attention_rows(q.view(n, H, hd), kv, 0, list(range(n))).view(n, H * hd)
    for code, text in ((14, r"the tensor-core issuer \(for a key tile\)"), (17, r"a softmax warp \(for the scores\)")):
        expect_give_up(ops, code, "flash_prefill_tc: " + text, run)
        out = run()
        torch.cuda.synchronize()
        ops.tc_status_check()
        close_bf16(out, ref)


def test_generate_reports_a_decode_kernel_that_gave_up(tmp_path):
    """The generation loop looks at the status word after the prompt step and once more when it returns: a
    decode kernel that gave up must not hand back its tokens as if nothing had happened."""
    import rusty_llama_b200 as rl
    from rusty_llama_b200.errors import KernelError
    from rusty_llama_b200.kernels import ops

    import __graft_entry__ as entry

    model_dir = rl.write_random_model(str(tmp_path / "m"), entry.SMOKE_CONFIG, seed=3)
    llm = rl.load(model_dir, dtype="bfloat16", max_tokens=64 * 4, use_graphs=False)  # (a captured graph would keep the test's limit)
    prompt = np.random.default_rng(0).integers(0, 320, 20).tolist()
    want = llm.generate(prompt, max_new_tokens=5, temperature=0.0, stop_token_ids=[])
    with ops.short_wait(52, 0):  # the decode attention's product warps; the prompt step does not run that kernel
        with pytest.raises(KernelError, match="attn_decode_tma: a product warp"):
            llm.generate(prompt, max_new_tokens=5, temperature=0.0, stop_token_ids=[])
    assert llm.engine.cache.n_open == 0
    assert llm.generate(prompt, max_new_tokens=5, temperature=0.0, stop_token_ids=[]) == want
