"""Time one kernel of the library at a given shape, with CUDA events.

    python -m rusty_llama_b200.kernels.microbench gemv --rows 8 --n 28672 --k 4096
    python -m rusty_llama_b200.kernels.microbench attn_decode --seqs 8 --ctx 4096
    python -m rusty_llama_b200.kernels.microbench flash_prefill --tokens 2048
    python -m rusty_llama_b200.kernels.microbench gemm --rows 2048 --n 6144 --k 4096

Each timed call works on its own copy of the large operand (weights, cache pages), and the copies
together exceed the 126 MB L2, so the figures are HBM figures.  Prints one JSON line: microseconds
per call, and GB/s or TFLOP/s of the bytes or flops the call has to move or do.
"""

from __future__ import annotations

import argparse
import json
import math
import sys

import torch

from . import ops
from .linear import linear

L2_BYTES = 126 * 1024 * 1024


USE_GRAPH = True


def _time(fn, n_variants: int, iters: int, warmup: int) -> float:
    """Microseconds per call.  The timed calls are captured into one CUDA graph and replayed, so that
    short kernels are not measured by how fast Python can launch them."""
    for i in range(warmup):
        fn(i % n_variants)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if USE_GRAPH:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(iters):
                fn(i % n_variants)
        graph.replay()  # once untimed
        torch.cuda.synchronize()
        e0.record()
        graph.replay()
        e1.record()
    else:
        e0.record()
        for i in range(iters):
            fn(i % n_variants)
        e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1000.0 / iters


def _copies(nbytes: int) -> int:
    return max(2, math.ceil(2 * L2_BYTES / max(nbytes, 1)))


def bench_gemv(a) -> dict:
    dev = "cuda:0"
    wbytes = a.n * a.k * 2
    nv = min(_copies(wbytes), 64)
    ws = [torch.randn(a.n, a.k, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(nv)]
    x = torch.randn(a.rows, a.k, device=dev, dtype=torch.bfloat16)
    out = torch.empty(a.rows, a.n, device=dev, dtype=torch.bfloat16)
    fn = ops.gemv_stream if a.impl == "stream" else ops.gemv_bf16
    if a.splits > 1:
        us = _time(lambda i: fn(x, ws[i], torch.float32, k_splits=a.splits), nv, a.iters, a.warmup)
    else:
        us = _time(lambda i: fn(x, ws[i], torch.bfloat16, out=out), nv, a.iters, a.warmup)
    ops.tc_status_check()
    return {"kernel": "gemv_stream" if a.impl == "stream" else "gemv_bf16", "rows": a.rows, "n": a.n, "k": a.k, "us": round(us, 2), "GBps": round(wbytes / us / 1e3, 1), "weight_copies": nv}


def bench_gemm(a) -> dict:
    dev = "cuda:0"
    nv = min(_copies(a.n * a.k * 2), 16)
    ws = [torch.randn(a.n, a.k, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(nv)]
    x = torch.randn(a.rows, a.k, device=dev, dtype=torch.bfloat16)
    if a.impl == "tc":
        out = torch.empty(a.rows, a.n, device=dev, dtype=torch.bfloat16)
        if a.splits > 1:
            us = _time(lambda i: ops.gemm_tc(x, ws[i], torch.float32, k_splits=a.splits), nv, a.iters, a.warmup)
        else:
            us = _time(lambda i: ops.gemm_tc(x, ws[i], torch.bfloat16, out=out), nv, a.iters, a.warmup)
        ops.tc_status_check()
    else:
        us = _time(lambda i: linear(x, ws[i]), nv, a.iters, a.warmup)
    flops = 2.0 * a.rows * a.n * a.k
    return {"kernel": "gemm_tc" if a.impl == "tc" else "linear(bf16)", "rows": a.rows, "n": a.n, "k": a.k, "us": round(us, 2), "TFLOPs": round(flops / us / 1e6, 1)}


def bench_linear(a) -> dict:
    """A projection as the model runs it: `linear`, `linear_swiglu` (a.swiglu: n counts gate and up rows) or
    `linear_to_stream` (a.to_stream: the result may come as partial sums), whichever kernel the dispatch picks
    for a.rows rows."""
    from .linear import linear_swiglu, linear_to_stream

    dev = "cuda:0"
    wbytes = a.n * a.k * 2
    nv = min(_copies(wbytes), 16)
    ws = [torch.randn(a.n, a.k, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(nv)]
    x = torch.randn(a.rows, a.k, device=dev, dtype=torch.bfloat16)
    out_dtype = getattr(a, "out_dtype", None)
    if getattr(a, "swiglu", False):
        fn = lambda i: linear_swiglu(x, ws[i])
    elif getattr(a, "to_stream", False):
        fn = lambda i: linear_to_stream(x, ws[i])
    else:
        fn = lambda i: linear(x, ws[i], out_dtype)
    us = _time(fn, nv, a.iters, a.warmup)
    ops.tc_status_check()
    return {"kernel": "linear", "rows": a.rows, "n": a.n, "k": a.k, "us": round(us, 2), "GBps": round(wbytes / us / 1e3, 1),
            "TFLOPs": round(2.0 * a.rows * a.n * a.k / us / 1e6, 1)}


def _paged(seqs: int, ctx: int, K: int, hd: int, copies: int):
    dev = "cuda:0"
    pages_per_seq = (ctx + 63) // 64
    n_pages = seqs * pages_per_seq
    ks = [torch.randn(n_pages, K, 64, hd, device=dev, dtype=torch.bfloat16) for _ in range(copies)]
    vs = [torch.randn(n_pages, K, 64, hd, device=dev, dtype=torch.bfloat16) for _ in range(copies)]
    table = torch.randperm(n_pages, device=dev).to(torch.int32).view(seqs, pages_per_seq).contiguous()
    return ks, vs, table


def bench_attn_decode(a) -> dict:
    from ..parts.attention import decode_splits

    dev = "cuda:0"
    H, K, hd = a.heads, a.kv_heads, a.head_dim
    kv_bytes = a.seqs * a.ctx * K * hd * 2 * 2
    nv = min(_copies(kv_bytes), 16)
    ks, vs, table = _paged(a.seqs, a.ctx, K, hd, nv)
    q = torch.randn(a.seqs, (H + 2 * K) * hd, device=dev, dtype=torch.bfloat16)
    seq_len = torch.full((a.seqs,), a.ctx, dtype=torch.int32, device=dev)
    n_splits = a.splits or decode_splits(a.seqs, H, K, a.ctx, 0 if a.impl == 'warp' else hd)
    scratch = torch.empty(ops.attn_decode_scratch_floats(a.seqs, H, hd, n_splits), device=dev)
    out = torch.empty(a.seqs, H * hd, device=dev, dtype=torch.bfloat16)
    impl = {"tma": "tma", "warp": "warp"}.get(a.impl, "auto")
    us = _time(lambda i: ops.attn_decode(q, ks[i], vs[i], table, seq_len, H, K, hd, n_splits, scratch, out=out, impl=impl), nv, a.iters, a.warmup)
    ops.tc_status_check()
    return {"kernel": "attn_decode", "impl": impl, "seqs": a.seqs, "ctx": a.ctx, "H": H, "K": K, "hd": hd, "splits": n_splits, "us": round(us, 2),
            "GBps": round(kv_bytes / us / 1e3, 1)}


def bench_flash_prefill(a) -> dict:
    dev = "cuda:0"
    H, K, hd, T = a.heads, a.kv_heads, a.head_dim, a.tokens
    ks, vs, table = _paged(1, T, K, hd, 1)
    q = torch.randn(T, (H + 2 * K) * hd, device=dev, dtype=torch.bfloat16)
    seq_start = torch.tensor([0, T], dtype=torch.int32, device=dev)
    pos0 = torch.zeros(1, dtype=torch.int32, device=dev)
    tc = a.impl == "tc" or (a.impl == "auto" and hd in ops.FLASH_TC_HEAD_DIMS)
    fn = ops.flash_prefill_tc if tc else ops.flash_prefill
    us = _time(lambda i: fn(q, ks[0], vs[0], table, seq_start, pos0, T, H, K, hd), 1, a.iters, a.warmup)
    if tc:
        ops.tc_status_check()
    flops = 4.0 * T * T * hd * H / 2
    return {"kernel": "flash_prefill_tc" if tc else "flash_prefill", "tokens": T, "H": H, "K": K, "hd": hd, "us": round(us, 2), "causal_TFLOPs": round(flops / us / 1e6, 1)}


def bench_rows(a) -> dict:
    dev = "cuda:0"
    d = a.k
    x = torch.randn(a.rows, d, device=dev)
    delta = torch.randn(a.rows, d, device=dev, dtype=torch.bfloat16)
    w = torch.ones(d, device=dev, dtype=torch.bfloat16)
    us = _time(lambda i: ops.add_rmsnorm(x, delta, w, 1e-5, torch.bfloat16), 1, a.iters, a.warmup)
    return {"kernel": "add_rmsnorm", "rows": a.rows, "d": d, "us": round(us, 2)}


def bench_sample(a) -> dict:
    """One sampling call for `--rows` sequences over a vocabulary of `--vocab`: greedy, temperature,
    temperature + top-p (the reference's default chain), and the longer chain with top-k, min-p and penalties."""
    from ..sampling.sampler import Sampler, SamplingParams

    global USE_GRAPH
    USE_GRAPH = False  # a call uploads the rows' slot numbers, which a capture does not take: plain launches
    dev = "cuda:0"
    logits = [torch.randn(a.rows, a.vocab, device=dev) * 3 for _ in range(4)]
    smp = Sampler(dev, max(a.rows, 1), a.vocab)
    slots = list(range(a.rows))
    smp.seed_slots(slots, [7 + i for i in slots])
    out = {"kernel": "sample", "rows": a.rows, "vocab": a.vocab, "us": {}}
    for name, params in (
        ("greedy", SamplingParams(0.0)),
        ("temperature", SamplingParams(1.0, 0.0, 7)),
        ("temperature_top_p", SamplingParams(0.8, 0.9, 7)),
        ("longer_chain", SamplingParams(0.8, 0.9, 7, top_k=40, min_p=0.05, repeat_penalty=1.1)),
    ):
        out["us"][name] = round(_time(lambda i: smp.sample(logits[i % 4], slots, params), 4, a.iters, a.warmup), 2)
    return out


def bench_step_trace(a) -> dict:
    """Durations of the kernels inside ONE replayed decode step (a CUDA graph with programmatic
    launches, where a profiler would serialise them): every kernel's first thread notes the time at
    which its dependency wait returned, i.e. when its predecessor had finished.  Needs libraries built
    with -DRL_TRACE:

        RUSTY_LLAMA_NVCC_EXTRA=-DRL_TRACE RUSTY_LLAMA_BUILD_DIR=/tmp/rl_trace \\
            python -m rusty_llama_b200.kernels.microbench step_trace --layers 4 --seqs 8
    """
    import ctypes

    from .. import load_random
    from ..engine import StepEntry
    from ..parts.attention import decode_splits
    from . import build as kbuild

    cfg = {
        "architectures": ["LlamaForCausalLM"], "hidden_size": a.heads * a.head_dim, "intermediate_size": a.ff,
        "num_hidden_layers": a.layers, "num_attention_heads": a.heads, "num_key_value_heads": a.kv_heads, "head_dim": a.head_dim,
        "vocab_size": a.vocab, "max_position_embeddings": a.ctx + 64, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
        "rope_scaling": None, "tie_word_embeddings": False, "torch_dtype": "bfloat16",
    }
    llm = load_random(cfg, seed=0, max_tokens=a.seqs * (a.ctx + 128), max_seqs=a.seqs)
    gen = torch.Generator().manual_seed(0)
    slots = [llm.open_sequence() for _ in range(a.seqs)]
    for s in slots:
        llm.step([StepEntry(s, torch.randint(0, a.vocab, (a.ctx - 400,), generator=gen).tolist(), [])])  # warm-up and traced steps stay inside one page-table width

    def decode():
        return llm.step([StepEntry(s, [5], [0]) for s in slots])

    for _ in range(300):  # a plain run, the capture, and enough replays for the SM clock to have come up
        decode()
    torch.cuda.synchronize()
    cap = 8192
    buf = torch.zeros(cap, dtype=torch.int64, device="cuda:0")
    count = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    for name in kbuild.loaded_libraries():
        lib = kbuild.load(name)
        if not hasattr(lib, "rl_trace_set"):
            raise SystemExit("the kernel libraries were built without -DRL_TRACE:\n" + bench_step_trace.__doc__)
        rc = lib.rl_trace_set(ctypes.c_void_p(buf.data_ptr()), ctypes.c_void_p(count.data_ptr()), ctypes.c_uint(cap))
        if rc:
            raise SystemExit(f"rl_trace_set of {name} failed with CUDA error {rc}")
    runs = []
    for _ in range(a.iters):
        count.zero_()
        torch.cuda.synchronize()
        decode()
        torch.cuda.synchronize()
        raw = buf[: int(count.item())].cpu().tolist()
        notes = sorted((v & ((1 << 56) - 1), (v >> 56) & 0xFF) for v in raw)  # (time, number); 0: a wait that returned
        t = [when for when, what in notes if what == 0]
        runs.append([(y - x) / 1000.0 for x, y in zip(t, t[1:])])
    # the kernels that call the dependency wait, in a step's order; an interval runs from the end of a
    # kernel's predecessor to its own end (the classifier product and the sampler follow the last mark)
    fused = a.head_dim in ops.ATTN_DECODE_TMA_HEAD_DIMS
    one_split = decode_splits(a.seqs, a.heads, a.kv_heads, a.ctx, a.head_dim) == 1
    import os

    from .linear import STREAM_MAX_ROWS

    folded = a.seqs <= STREAM_MAX_ROWS and os.environ.get("RL_FOLD_NORM", "1") != "0"  # the second norm has no kernel of its own then
    layer = (["norm1", "qkv"] + ([] if fused else ["rope"]) + ["attention"] + ([] if (fused and one_split) else ["merge"])
             + ["o_proj"] + ([] if folded else ["norm2"]) + ["gate_up", "down"])
    names = ["positions", "embed"] + layer * a.layers + ["final_norm"]  # (the step's first kernel takes the positions from the sequences' records)
    if any(len(r) != len(names) for r in runs):
        raise SystemExit(f"expected {len(names)} intervals per step, got {[len(r) for r in runs]}: the step's kernel list has changed")
    per = {}
    for r in runs:
        for nm, dt in zip(names, r):
            per.setdefault(nm, []).append(dt)
    # the median over the steps: a step that crosses into a wider page table runs plainly once more
    med = lambda v: sorted(v)[len(v) // 2]
    out = {"kernel": "step_trace", "seqs": a.seqs, "ctx": a.ctx, "layers": a.layers, "us": {k: round(med(v), 2) for k, v in per.items()},
           "step_spans_us": [round(sum(r), 1) for r in runs]}
    out["layer_us"] = round(sum(out["us"][k] for k in layer), 1)
    if a.events:
        # the last traced step's second layer with the numbered notes that some kernels leave besides
        # (csrc/gemv_stream.cu: 1 block 0 runs, 2 first copy issued, 3 ring full of requests, 4 activations
        # requested, 5 first stage consumed, 6 last sums handed over, 7 last copy issued, 8 last result
        # stored); every note is taken after an atomic's round trip, about a microsecond late
        marks = [i for i, (_, what) in enumerate(notes) if what == 0]
        first = 2 + len(layer)  # marks: positions, embed, the first layer's kernels, then the second layer's
        lo, hi = marks[first], marks[min(first + len(layer) + 1, len(marks) - 1)]
        kernel_at = {marks[first + j]: nm for j, nm in enumerate(layer + layer[:1]) if first + j < len(marks)}
        out["events_us"] = [
            [round((when - notes[lo][0]) / 1000.0, 2), ("wait returned: " + kernel_at.get(i, "?")) if what == 0 else what]
            for i, (when, what) in enumerate(notes[lo : hi + 1], start=lo)
        ]
    return out


def bench_probe_stream(a) -> dict:
    """What HBM delivers to a bare ring of TMA copies (csrc/probe_pipeline.cu), nothing done with the data: 1 GiB
    read once by one block per SM, for stages of several shapes and rings of several depths."""
    import ctypes

    from . import build as kbuild

    lib = kbuild.load("probe_pipeline")
    nbytes = 1 << 30
    buf = torch.zeros(nbytes // 2, dtype=torch.bfloat16, device="cuda:0")
    err = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    rows_out = []
    K = a.k
    # (rows, k per stage, walk): the streaming product's stage, the same bytes as fewer and longer rows, a GEMM operand's tile
    shapes = [(8, 1024, 0), (4, 2048, 0), (2, 4096, 0), (256, 64, 1), (128, 128, 1), (64, 256, 1)]
    for rows, kc, walk in shapes:
        if kc > K:
            continue
        for stages in (6, 13) if rows * kc * 2 == 16384 else (6,):
            ms = []
            for _ in range(3):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                reps = 6  # (the first launch of a burst waits for the host; it is not timed)
                for i in range(reps):
                    if i == 1:
                        e0.record()
                    rc = lib.rl_probe_tma_stream(ctypes.c_void_p(buf.data_ptr()), ctypes.c_longlong(nbytes), ctypes.c_int(K), ctypes.c_int(rows),
                                                 ctypes.c_int(kc), ctypes.c_int(stages), ctypes.c_int(walk), ctypes.c_int(256),
                                                 ctypes.c_void_p(err.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
                    if rc != 0:
                        raise SystemExit(f"probe_tma_stream refused or failed: {rc} {lib.rl_error_text().decode()}")
                e1.record()
                torch.cuda.synchronize()
                ms.append(e0.elapsed_time(e1) / (reps - 1))
            if int(err.item()):
                raise SystemExit("probe_tma_stream: a wait ran out")
            rows_out.append({"rows": rows, "bytes_per_row": kc * 2, "stage_KB": rows * kc * 2 // 1024, "stages": stages,
                             "walk": "gemm operand" if walk else "rows along k", "GBps": round(nbytes / (min(ms) * 1e-3) / 1e9, 0)})
    return {"kernel": "probe_tma_stream", "k": K, "results": rows_out}


def bench_probe_handshake(a) -> dict:
    """What one trip of a producer / consumer pair of single threads costs (csrc/probe_pipeline.cu), in nanoseconds
    per stage: 128 blocks, 512 stages each, the slowest block."""
    import ctypes

    from . import build as kbuild

    lib = kbuild.load("probe_pipeline")
    k_blocks, n_blocks, n_iters = 256, 128, 512
    buf = torch.zeros(64 * k_blocks * 64, dtype=torch.bfloat16, device="cuda:0")
    out = torch.zeros(n_blocks, dtype=torch.int64, device="cuda:0")
    err = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    modes = [(0, "arrival only, counters"), (4, "arrival only, divisions by the ring's depth"), (8, "arrival only, counters, the timer read per wait"),
             (1, "one TMA box, counters"), (3, "two TMA boxes, counters"), (5, "one TMA box, divisions"), (9, "one TMA box, counters, the timer read per wait")]
    res = []
    for mode, what in modes:
        for stages in (4, 16):
            best = None
            for _ in range(3):
                rc = lib.rl_probe_handshake(ctypes.c_void_p(buf.data_ptr()), ctypes.c_int(k_blocks), ctypes.c_int(mode), ctypes.c_int(stages),
                                            ctypes.c_int(n_iters), ctypes.c_int(n_blocks), ctypes.c_void_p(out.data_ptr()),
                                            ctypes.c_void_p(err.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
                torch.cuda.synchronize()
                if rc != 0:
                    raise SystemExit(f"probe_handshake refused or failed: {rc} {lib.rl_error_text().decode()}")
                worst = int(out.max().item())
                best = worst if best is None else min(best, worst)
            if int(err.item()):
                raise SystemExit("probe_handshake: a wait ran out")
            res.append({"what": what, "stages": stages, "ns_per_stage": round(best / n_iters, 1)})
    return {"kernel": "probe_handshake", "results": res}


def bench_probe_mma(a) -> dict:
    """What the tensor core takes per tcgen05.mma of M 128, N n, K 16 when one thread issues a long run of them on
    operands that lie still (csrc/probe_pipeline.cu): SM cycles per instruction (the slowest block) against the
    n / 2 cycles of the nominal rate, on one SM and on all of them."""
    import ctypes

    from . import build as kbuild

    lib = kbuild.load("probe_pipeline")
    k_blocks, n_mma = 64, 4096
    buf = torch.zeros(256 * k_blocks * 64, dtype=torch.bfloat16, device="cuda:0")
    err = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    forms = [(0, "A and B from shared memory, one accumulator"), (1, "the same, two accumulators in turn"),
             (2, "A from tensor memory, one accumulator"), (3, "A from tensor memory, two accumulators in turn"),
             (4, "A and B from shared memory, one accumulator, TMA copies landing meanwhile"),
             (6, "A from tensor memory, one accumulator, TMA copies landing meanwhile"),
             (8, "A and B from shared memory, a commit after every fourth"),
             (16, "A and B from shared memory, a wait that succeeds and a fence before every fourth"),
             (48, "A and B from shared memory, a wait that succeeds before every fourth, no fence"),
             (56, "A and B from shared memory, wait, four instructions, commit, no fence"),
             (24, "A and B from shared memory, wait, fence, four instructions, commit: a GEMM's k slice"),
             (28, "the same with TMA copies landing meanwhile"),
             (64, "the slice with the wait's question asked before its four instructions and read after the commit"),
             (68, "the same with TMA copies landing meanwhile")]
    res = []
    for n in (16, 32, 64, 128, 256):
        for form, what in forms:
            if (form & 2) and n > 128:
                continue
            for n_blocks in (148,):
                out = torch.zeros(2 * n_blocks, dtype=torch.int64, device="cuda:0")
                best = None
                for _ in range(3):
                    rc = lib.rl_probe_mma_rate(ctypes.c_void_p(buf.data_ptr()), ctypes.c_int(k_blocks), ctypes.c_int(n), ctypes.c_int(form),
                                               ctypes.c_int(n_mma), ctypes.c_int(n_blocks), ctypes.c_void_p(out.data_ptr()),
                                               ctypes.c_void_p(err.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
                    torch.cuda.synchronize()
                    if rc != 0:
                        raise SystemExit(f"probe_mma_rate refused or failed: {rc} {lib.rl_error_text().decode()}")
                    worst = int(out[:n_blocks].max().item())
                    if best is None or worst < best[0]:
                        best = (worst, int(out[n_blocks:].min().item()))
                if int(err.item()):
                    raise SystemExit("probe_mma_rate: a wait ran out")
                row = {"n": n, "what": what, "blocks": n_blocks, "cycles_per_mma": round(best[0] / n_mma, 1), "nominal": n // 2}
                if form & 4:
                    row["copied_bytes_per_cycle"] = round(best[1] * 32768 / best[0], 1)
                res.append(row)
    return {"kernel": "probe_mma_rate", "mmas": n_mma, "results": res}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("kernel", choices=["gemv", "gemm", "linear", "attn_decode", "flash_prefill", "add_rmsnorm", "sample", "step_trace", "probe_stream", "probe_handshake", "probe_mma"])
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--seqs", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--layers", type=int, default=4, help="step_trace: layers of the model")
    ap.add_argument("--ff", type=int, default=14336, help="step_trace: width of the feed-forward")
    ap.add_argument("--vocab", type=int, default=128256, help="step_trace, sample: vocabulary")
    ap.add_argument("--events", action="store_true", help="step_trace: also the numbered notes inside one layer's kernels")
    ap.add_argument("--splits", type=int, default=0, help="attn_decode: key splits; gemv/gemm: slices of k with float32 partial sums")
    ap.add_argument("--impl", default="linear", choices=["linear", "auto", "tc", "stream", "tma", "warp"], help="gemm: the dispatching linear() or the tcgen05 kernel; flash_prefill: tc = the tcgen05 kernel, auto = by head size; gemv: stream = the persistent TMA-fed kernel; attn_decode: tma or warp = one of its two kernels")
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--swiglu", action="store_true", help="linear: the fused gate/up product (n counts both)")
    ap.add_argument("--to-stream", action="store_true", help="linear: a projection into the residual stream (may split k)")
    ap.add_argument("--no-graph", action="store_true", help="launch the timed calls one by one instead of as one graph")
    a = ap.parse_args(argv)
    global USE_GRAPH
    USE_GRAPH = not a.no_graph
    fn = {"gemv": bench_gemv, "gemm": bench_gemm, "linear": bench_linear, "attn_decode": bench_attn_decode, "flash_prefill": bench_flash_prefill,
          "add_rmsnorm": bench_rows, "sample": bench_sample, "step_trace": bench_step_trace, "probe_stream": bench_probe_stream,
          "probe_handshake": bench_probe_handshake, "probe_mma": bench_probe_mma}[a.kernel]
    print(json.dumps(fn(a)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
