"""Decode and prefill throughput of the library on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--reps R]
    python bench.py --sizes 1b|13b --workload

The default run has the layer sizes of Llama-3.1-8B (BASELINE.json configs[2]) with random
bfloat16 weights, a batch of 8 sequences and a context of 4096.  A step is one decode step of the
whole batch through `Engine.step` (the CUDA graph the generation loop replays).  `value` is decoded
tokens per second at the full context: R repetitions (default 5; mean and standard deviation under
`reps`), each a fresh prefill to a length from which W untimed (at least 64, see `warmup` in the line)
and exactly K timed steps end at position 4096, timed with CUDA events.  `points` holds decoding at batch 1, 8 and 64 at half the
context, at the full context and averaged over the way between them (the workload BASELINE.json names:
from 2,048-token prompts to 4,096).  `prefill` is one step of 2,048 tokens.  `e2e` is decoding through
the Python entry point `LLM.generate`, host token lists in and out, timed on the host per token over
at least 512 steps.  `kernels` times the step's main kernels alone at this configuration's shapes.
Inputs are larger than L2 (a decode step reads every weight: 16 GB), so no explicit L2 flush.
If a kernel reports that one of its bounded waits ran out, the run is discarded and measured once more
(`measured_again` in the line then holds the report).
With `--workload`, the unequal-prompt workloads that BASELINE.json names for the 1b and 13b sizes run
through `LLM.generate` instead.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode_tokens_per_second_batch{batch}_ctx{ctx}"  # at the defaults: batch 8, context 4096


SIZES = {
    # BASELINE.json's configs are prose; their sizes as config.json keys.  "8b" is configs[2], the default run.
    "8b": ("Llama-3.1-8B sizes (BASELINE.json configs[2])", dict(
        hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8,
        head_dim=128, vocab_size=128256, max_position_embeddings=131072, rms_norm_eps=1e-5, rope_theta=500000.0,
        rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                      "original_max_position_embeddings": 8192})),
    "1b": ("TinyLlama-1.1B sizes (BASELINE.json configs[3])", dict(
        hidden_size=2048, intermediate_size=5632, num_hidden_layers=22, num_attention_heads=32, num_key_value_heads=4,
        head_dim=64, vocab_size=32000, max_position_embeddings=2048, rms_norm_eps=1e-5, rope_theta=10000.0, rope_scaling=None)),
    "13b": ("Llama-2-13B sizes (BASELINE.json configs[4])", dict(
        hidden_size=5120, intermediate_size=13824, num_hidden_layers=40, num_attention_heads=40, num_key_value_heads=40,
        head_dim=128, vocab_size=32000, max_position_embeddings=4096, rms_norm_eps=1e-5, rope_theta=10000.0, rope_scaling=None)),
}


def load_config(sizes: str = "8b") -> dict:
    cfg = {"architectures": ["LlamaForCausalLM"], "tie_word_embeddings": False, "torch_dtype": "bfloat16"}
    cfg.update(SIZES[sizes][1])
    return cfg


def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    except (OSError, KeyError, ValueError, TypeError):
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs; every sample
    carries the host's time at which it was read."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, period_ms: int = 100):
        self.samples = []  # (host time, MHz, max MHz, active reasons)
        self.proc = None
        self.period_ms = period_ms

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", str(self.period_ms)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                mhz, mx = float(parts[0]), float(parts[1])
            except ValueError:
                continue
            self.samples.append((time.time(), mhz, mx, [n for n, v in zip(self.NAMES, parts[2:6]) if v.lower().startswith("active")]))

    def median_mhz(self, t0: float, t1: float):
        """Median SM clock of the samples read between two host times (None if there is none)."""
        mhz = sorted(m for t, m, _, _ in self.samples if t0 <= t <= t1)
        return mhz[len(mhz) // 2] if mhz else None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        mhz = sorted(m for _, m, _, _ in self.samples)
        reasons = sorted({r for _, _, _, rs in self.samples for r in rs})
        mx = self.samples[-1][2] if self.samples else None
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": reasons, "samples": len(mhz)}


def model_bytes_and_flops(cfg: dict, n_layers: int):
    d, ff, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    qd = cfg["num_attention_heads"] * cfg["head_dim"]
    kvd = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = d * (qd + 2 * kvd) + qd * d + 3 * d * ff
    weights = per_layer * n_layers + V * d  # matrices a decode step reads: the layers and the classifier
    kv_per_token = 2 * kvd * n_layers
    return per_layer, weights, kv_per_token


def mean_sd(xs):
    m = sum(xs) / len(xs)
    return m, (sum((x - m) ** 2 for x in xs) / max(len(xs) - 1, 1)) ** 0.5


def kernel_breakdown(cfg: dict, batch: int, ctx: int, T: int, peaks: dict) -> dict:
    """The kernels that a prompt step and a decode step spend their time in, each timed alone at this
    configuration's shapes (CUDA events around a replayed graph of calls, every call on its own copy of the
    weights or pages so that HBM is read): microseconds, and the fraction of the measured peak that the flops
    it must do or the bytes it must read amount to."""
    from types import SimpleNamespace

    import torch

    from rusty_llama_b200.kernels import microbench as mb

    d, ff, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    H, K, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    qkv = (H + 2 * K) * hd
    base = dict(iters=10, warmup=2, splits=0, heads=H, kv_heads=K, head_dim=hd)
    out = {}
    for name, n, k in (("qkv", qkv, d), ("attn_out", d, H * hd), ("gate_up", 2 * ff, d), ("down", d, ff)):
        kind = dict(swiglu=name == "gate_up", to_stream=name in ("attn_out", "down"))
        r = mb.bench_linear(SimpleNamespace(rows=T, n=n, k=k, **kind, **base))
        out[f"prefill_{name}"] = {"us": r["us"], "frac": round(r["TFLOPs"] / peaks["bf16_tflops"], 3)}
        r = mb.bench_linear(SimpleNamespace(rows=batch, n=n, k=k, **kind, **base))
        out[f"decode_{name}"] = {"us": r["us"], "frac": round(r["GBps"] / peaks["hbm_gbs"], 3)}
    r = mb.bench_linear(SimpleNamespace(rows=batch, n=V, k=d, out_dtype=torch.float32, **base))
    out["decode_classifier"] = {"us": r["us"], "frac": round(r["GBps"] / peaks["hbm_gbs"], 3)}
    r = mb.bench_flash_prefill(SimpleNamespace(tokens=T, impl="auto", **base))
    out["prefill_attention"] = {"us": r["us"], "frac": round(r["causal_TFLOPs"] / peaks["bf16_tflops"], 3)}
    r = mb.bench_attn_decode(SimpleNamespace(seqs=batch, ctx=ctx, impl="auto", **base))
    out["decode_attention"] = {"us": r["us"], "frac": round(r["GBps"] / peaks["hbm_gbs"], 3)}
    return out


def run_ours(args) -> dict:
    import torch

    import rusty_llama_b200 as rl
    from rusty_llama_b200 import StepEntry
    from rusty_llama_b200.kernels import ops

    cfg = load_config(args.sizes)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    L = cfg["num_hidden_layers"]
    ctx = min(args.context, cfg["max_position_embeddings"])
    batch, K, W, R = args.batch, args.steps, args.warmup, args.reps
    # Untimed steps before the timed ones.  A repetition starts with a prompt step of tens of thousands of
    # tokens, which runs into the power cap; the SM clock takes about 0.13 s to come back from it (the
    # end-to-end figure below shows that transient on its own), so at least 64 steps are run untimed.
    W = max(W, 64)
    peaks = measured_peaks()
    torch.cuda.set_device(0)
    t_load = time.time()
    # the cache holds 64 sequences of the context where that fits beside the weights (it does at the default
    # context); with a longer --context the batch-64 point is left out instead of running out of memory
    per_layer, weight_elems, kv_per_token = model_bytes_and_flops(cfg, L)
    # (beside the weights: the activations of the end-to-end run's prompt step, which takes all prompts at once,
    # about 2 * (q + k + v + 3 widths + 3 feed-forward widths) bytes a token, and 12 GB for everything else)
    act_per_token = 2 * (cfg["num_attention_heads"] * cfg["head_dim"] * 2 + 4 * cfg["hidden_size"] + 3 * cfg["intermediate_size"]) + 8 * cfg["hidden_size"]
    free_bytes = (torch.cuda.mem_get_info(0)[0] - 2 * (weight_elems + cfg["vocab_size"] * cfg["hidden_size"])
                  - batch * ctx * act_per_token - (12 << 30))
    tokens_that_fit = max(free_bytes // (2 * kv_per_token), 0) // 64 * 64
    need = batch * ctx + 64 * 64
    if tokens_that_fit < need:
        print(json.dumps({"error": f"a cache for {batch} sequences of {ctx} tokens does not fit this GPU's memory"}))
        raise SystemExit(1)
    max_tokens = min(max(64 * ctx, batch * ctx) + 64 * 64, tokens_that_fit)
    llm = rl.load_random(cfg, seed=0, dtype="bfloat16", device="cuda:0", max_tokens=max_tokens, max_seqs=64,
                         use_graphs=not args.no_graphs)
    torch.cuda.synchronize()
    print(f"[bench] model of {L} layers ready in {time.time() - t_load:.1f} s", file=sys.stderr, flush=True)
    gen = torch.Generator().manual_seed(0)
    V = cfg["vocab_size"]

    def extend(slots, n):
        """n more (random) tokens for each of `slots`, as prompt steps of at most 8192 tokens."""
        if n <= 0:
            return
        group = max(1, 8192 // n)
        for i in range(0, len(slots), group):
            llm.step([StepEntry(s, torch.randint(0, V, (n,), generator=gen).tolist(), []) for s in slots[i : i + group]])

    def timed_decode(slots, steps):
        """Exactly `steps` decode steps of the batch between two CUDA events (synchronised on both sides);
        returns (milliseconds per step, kernels launched)."""
        B = len(slots)
        toks = torch.randint(0, V, (steps, B), generator=gen).tolist()
        torch.cuda.synchronize()
        l0 = ops.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for k in range(steps):
            # (the logits are borrowed: this loop does not keep them, and the copy that would make them
            # the caller's own is not part of a decode step)
            llm.step([StepEntry(s, [toks[k][j]], [0]) for j, s in enumerate(slots)], borrow=True)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps, ops.launch_count() - l0

    def step_bytes(B, mean_ctx):
        return 2 * weight_elems + 2 * kv_per_token * mean_ctx * B

    def headline_rep(B, steps, warm):
        """B sequences prefilled so that `warm + steps` decode steps end at position ctx."""
        slots = [llm.open_sequence() for _ in range(B)]
        extend(slots, ctx - (warm + steps))
        timed_decode(slots, warm)
        ms, launches = timed_decode(slots, steps)
        for s in slots:
            llm.close_sequence(s)
        return ms, launches

    def trajectory(B, win):
        """Decode rates along the way from half the context to all of it: windows of `win` timed steps at
        five contexts, the sequences brought from one to the next by prompt steps.  Returns {context: tokens/s}."""
        slots = [llm.open_sequence() for _ in range(B)]
        have, rates = 0, {}
        start = ctx // 2
        for c in [start + (ctx - start) * i // 4 for i in range(4)] + [ctx - win]:
            c = max(c, have)
            extend(slots, c - have)
            timed_decode(slots, 2)  # (a new page-table width: plain run and capture, untimed)
            ms, _ = timed_decode(slots, win - 2)
            have = c + win
            rates[c] = B * 1000.0 / ms
        for s in slots:
            llm.close_sequence(s)
        return rates

    if args.only == "prefill":
        value, ms_step, clocks, launches, rep_rates = 0.0, 1.0, None, 0, [0.0]
    else:
        # ---- headline: batch `batch`, R repetitions of exactly K timed steps that end at the context
        headline_rep(batch, K, W)  # untimed: graphs are captured, workspaces sized, clocks settle
        sampler = ClockSampler().start()
        reps = [headline_rep(batch, K, W) for _ in range(R)]
        clocks = sampler.stop()
        rep_rates = [batch * 1000.0 / ms for ms, _ in reps]
        ms_step = sum(ms for ms, _ in reps) / R
        value = batch * 1000.0 / ms_step
        launches = reps[-1][1]
    bytes_step = step_bytes(batch, ctx - K / 2.0)
    achieved = bytes_step / (ms_step * 1e-3) / 1e9
    if args.only == "decode":
        print(json.dumps({"only": "decode", "batch": batch, "ms_per_step": ms_step, "tokens_per_s": value, "GBps": achieved, "layers": L}))
        return None

    # ---- decoding along the trajectory, at batch 1, the headline's batch and 64
    points = {}
    win = max(64, min(K, 256))
    for B in sorted({1, batch, 64}):
        if args.only == "prefill":
            break
        if B * ctx + 64 * 64 > max_tokens:
            points[f"decode_b{B}"] = None  # its cache does not fit at this context
            continue
        rates = trajectory(B, win)
        cs = sorted(rates)
        points[f"decode_b{B}"] = round(rates[cs[-1]], 1)                    # at the full context, like the headline
        points[f"decode_b{B}_c{cs[0]}"] = round(rates[cs[0]], 1)             # at half the context
        points[f"decode_b{B}_mean"] = round(sum(rates.values()) / len(rates), 1)  # over the way from one to the other
        points[f"decode_b{B}_frac_of_hbm_peak"] = round(step_bytes(B, cs[-1] + win / 2.0) * rates[cs[-1]] / B / 1e9 / peaks["hbm_gbs"], 4)
    points["window_steps"] = win

    # ---- prefill of 2048 tokens
    T = min(2048, ctx)
    slot_times = []
    for rep in range(W + 5):
        s = llm.open_sequence()
        prompt = torch.randint(0, V, (T,), generator=gen).tolist()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        llm.step([StepEntry(s, prompt, [T - 1])])
        e1.record()
        torch.cuda.synchronize()
        if rep >= W:
            slot_times.append(e0.elapsed_time(e1))
        llm.close_sequence(s)
    pre_ms, pre_sd = mean_sd(slot_times)
    H, hd = cfg["num_attention_heads"], cfg["head_dim"]
    flops = 2.0 * T * per_layer * L + 4.0 * T * T * hd * H / 2 * L + 2.0 * V * cfg["hidden_size"]
    pre_frac = flops / (pre_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12)
    if args.only == "prefill":
        print(json.dumps({"only": "prefill", "tokens": T, "ms": pre_ms, "sd_ms": pre_sd, "tokens_per_s": T * 1000.0 / pre_ms, "frac": pre_frac, "layers": L}))
        return None

    # ---- end to end through the Python entry point: host token lists in, host token lists out.  Long enough
    # (at least 512 decode steps) to outlast what the prompt step leaves behind: its power-capped SM clock
    # takes a tenth of a second to recover.  The figure is taken over the last 256 steps, which end at the
    # context like the device-timed steps; the first 256 are reported beside it, each with the SM clock that
    # nvidia-smi showed meanwhile, so that milliseconds times megahertz can be compared.
    E = max(512, 2 * K)
    prompts = [torch.randint(0, V, (ctx - E - 1,), generator=gen).tolist() for _ in range(batch)]
    llm.generate(prompts[:1], max_new_tokens=4, temperature=0.0, stop_token_ids=[])  # warm the batch-1 paths
    llm.generate(prompts, max_new_tokens=8, temperature=0.0, stop_token_ids=[])
    stamps = []
    sent0 = llm.engine.upload_bytes
    sampler = ClockSampler(period_ms=20).start()
    llm.generate(prompts, max_new_tokens=E + 1, temperature=0.0, stop_token_ids=[],
                 on_token=lambda r, t: stamps.append(time.time()) if r == 0 else None)
    sampler.stop()
    st = llm.last_stats
    n_e2e = 256
    assert len(stamps) == E + 1
    first_ms = 1000.0 * (stamps[n_e2e] - stamps[0]) / n_e2e
    last_ms = 1000.0 * (stamps[E] - stamps[E - n_e2e]) / n_e2e
    mhz_first, mhz_last = sampler.median_mhz(stamps[0], stamps[n_e2e]), sampler.median_mhz(stamps[E - n_e2e], stamps[E])
    # what went to the device during the call: the prompts' tokens and positions once, then a step's slot numbers and
    # page tables only when a sequence takes a new page (the sampled tokens never leave the device on their way into
    # the next step; every step's tokens are read back by the host)
    h2d_per_step = (llm.engine.upload_bytes - sent0) / (E + 1)

    out = {
        "metric": METRIC.format(batch=batch, ctx=ctx),
        "value": round(value, 1),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": K,
        "warmup": W,
        "ms_per_step": round(ms_step, 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: random token ids, random-init weights N(0, 0.02)",
        "impl": "ours",
        "reps": {"n": R, "each": f"{W} untimed and {K} timed decode steps ending at position {ctx}, after a fresh prefill",
                 "tokens_per_s_mean": round(mean_sd(rep_rates)[0], 1), "tokens_per_s_sd": round(mean_sd(rep_rates)[1], 1)},
        "config": {
            "model": SIZES[args.sizes][0],
            "global_batch": batch,
            "seq_len": ctx,
            "parallelism": "single GPU",
            "layers": L,
            "layers_of_full_config": full_layers,
            "hidden_size": cfg["hidden_size"],
            "intermediate_size": cfg["intermediate_size"],
            "num_attention_heads": cfg["num_attention_heads"],
            "num_key_value_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"],
            "vocab_size": V,
            "rope_theta": cfg["rope_theta"],
            "rope_scaling": "llama3 factor 8 low 1 high 4 original 8192" if cfg["rope_scaling"] else "none",
            "rms_norm_eps": cfg["rms_norm_eps"],
            "tie_word_embeddings": False,
            "prefill_tokens": T,
            "l2": "inputs larger than L2 (each step reads all weights); no flush",
        },
        "e2e": {
            "value": round(batch * 1000.0 / last_ms, 1),
            "unit": "tokens/s",
            "steps": n_e2e,
            "h2d_bytes_per_step": round(h2d_per_step, 1),
            "d2h_bytes_per_step": 4 * batch,
            "what": f"LLM.generate, greedy, host lists in and out, host clock per token: the last {n_e2e} of {E} decode steps, which end at position {ctx}",
            "ms_per_step": round(last_ms, 4),
            "sm_mhz": mhz_last,
            "first_steps_ms_per_step": round(first_ms, 4),
            "first_steps_sm_mhz": mhz_first,
            "ms_x_mhz_last_over_first": None if not (mhz_first and mhz_last) else round(last_ms * mhz_last / (first_ms * mhz_first), 3),
            "whole_decode_phase_tokens_per_s": round(st.decode_steps * batch / st.decode_seconds, 1) if st.decode_seconds > 0 else None,
            "host_ms_per_step_in_step_call": round(1000.0 * st.decode_step_call_seconds / max(st.decode_steps, 1), 4),
            "host_ms_per_step_in_sample_call": round(1000.0 * st.decode_sample_call_seconds / max(st.decode_steps, 1), 4),
        },
        "gpu_launches": launches,
        "prefill": {"value": round(T * 1000.0 / pre_ms, 1), "tokens": T, "ms": round(pre_ms, 3), "sd_ms": round(pre_sd, 3), "reps": len(slot_times),
                    "frac": round(pre_frac, 4), "peak_tflops": peaks["bf16_tflops"], "of": peaks["source"],
                    "frac_of_sustained_peak": round(flops / (pre_ms * 1e-3) / (peaks["bf16_tflops_sustained"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4), "of": peaks["source"]},
        "points": points,
        "clocks": clocks,
    }
    if not args.no_kernels:
        del llm
        torch.cuda.empty_cache()
        out["kernels"] = kernel_breakdown(cfg, batch, ctx, T, peaks)
    return out


# BASELINE.json's configs[3] and [4] name workloads of unequal prompts; (sizes) -> (prompts, shortest, longest, new tokens)
WORKLOADS = {"1b": (64, 128, 1024, 256), "13b": (8, 512, 3072, None)}  # None: every sequence decodes up to the context


def run_workload(args) -> dict:
    """`--workload`: the unequal-prompt workload that BASELINE.json names for these sizes, through `LLM.generate`
    (prompts in one step, then one token each, sequences leaving as they finish), timed on the host."""
    import random

    import torch

    import rusty_llama_b200 as rl

    cfg = load_config(args.sizes)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    n, lo, hi, new = WORKLOADS[args.sizes]
    ctx = min(args.context, cfg["max_position_embeddings"])
    rnd = random.Random(0)
    lens = [rnd.randint(lo, hi) for _ in range(n)]
    budgets = [new if new is not None else ctx - l for l in lens]
    budgets = [min(b, ctx - l) for b, l in zip(budgets, lens)]
    torch.cuda.set_device(0)
    llm = rl.load_random(cfg, seed=0, dtype="bfloat16", device="cuda:0", max_tokens=n * ctx + 64 * 64, max_seqs=n)
    V = cfg["vocab_size"]
    prompts = [[rnd.randrange(V) for _ in range(l)] for l in lens]
    runs = []
    for rep in range(1 + args.reps):  # the first run captures the graphs of every batch size it passes through
        llm.generate(prompts, max_new_tokens=budgets, temperature=0.0, stop_token_ids=[])
        st = llm.last_stats
        if rep:
            runs.append((st.generated_tokens / (st.prefill_seconds + st.decode_seconds), (st.generated_tokens - n) / st.decode_seconds,
                         st.prompt_tokens / st.prefill_seconds))
    return {
        "workload": f"{n} prompts of {lo} to {hi} random ids (seeded), " + (f"{new} new tokens each" if new else f"each decoding to position {ctx}"),
        "impl": "ours", "sizes": SIZES[args.sizes][0], "layers": cfg["num_hidden_layers"], "dtype": "bf16",
        "prompt_tokens": sum(lens), "generated_tokens": sum(budgets), "reps": len(runs),
        "generated_tokens_per_s": round(mean_sd([r[0] for r in runs])[0], 1), "generated_tokens_per_s_sd": round(mean_sd([r[0] for r in runs])[1], 1),
        "decode_phase_tokens_per_s": round(mean_sd([r[1] for r in runs])[0], 1),
        "prompt_step_tokens_per_s": round(mean_sd([r[2] for r in runs])[0], 1),
        "through": "LLM.generate, greedy, host token lists in and out, host clock",
    }


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--sizes", default="8b", choices=sorted(SIZES), help="layer sizes: 8b is BASELINE.json's configs[2] (the default run), 1b and 13b its configs[3] and [4]")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (named in the output)")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"], help="profiling aid: run one phase only")
    ap.add_argument("--no-graphs", action="store_true", help="profiling aid: launch decode kernels one by one")
    ap.add_argument("--reps", type=int, default=5, help="repetitions of the timed steps (mean and standard deviation are reported)")
    ap.add_argument("--no-kernels", action="store_true", help="leave out the kernel-by-kernel table")
    ap.add_argument("--workload", action="store_true", help="with --sizes 1b or 13b: BASELINE.json's workload of unequal prompts through LLM.generate, instead of the contract line")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({
            "impl": "reference",
            "unavailable": "the reference is a Rust crate (Cargo.toml, no setup.py/pyproject.toml): pip cannot install it "
                           "offline and neither cargo nor rustc exists on this machine",
        }))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this library has no multi-GPU path (asked for --gpus {args.gpus})")
        return 2
    args.warmup = max(args.warmup, 3)
    args.reps = max(args.reps, 1)
    if args.workload:
        if args.sizes not in WORKLOADS:
            print(f"--workload goes with --sizes {' or '.join(sorted(WORKLOADS))}")
            return 2
        print(json.dumps(run_workload(args)))
        return 0
    out = measured_again_if_a_kernel_gave_up(lambda: run_ours(args))
    if out is not None:
        print(json.dumps(out))
    return 0


def measured_again_if_a_kernel_gave_up(run):
    """run() once; if a kernel of the library reported that one of its bounded waits ran out (a KernelError: that
    run's numbers are not valid), say so on stderr, give the device memory back and measure once more from the
    start.  A second failure is raised.  The line of a repeated run says so under `measured_again`."""
    from rusty_llama_b200.errors import KernelError

    try:
        return run()
    except KernelError as e:
        why = str(e)
    print(f"[bench] this run is discarded: {why}; measuring once more", file=sys.stderr, flush=True)
    import gc

    import torch

    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
    out = run()
    if isinstance(out, dict):
        out["measured_again"] = why
    return out


if __name__ == "__main__":
    sys.exit(main())
