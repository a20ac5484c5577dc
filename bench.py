"""Decode and prefill throughput of the library on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run has the layer sizes of Llama-3.1-8B (BASELINE.json configs[2]) with random
bfloat16 weights, a batch of 8 sequences and a context of 4096: each sequence is prefilled to a
length such that the K timed decode steps end at position 4096.  A step is one decode step of the
whole batch through `Engine.step` (the CUDA graph the generation loop replays); `value` is decoded
tokens per second, timed with CUDA events around exactly K steps.  `e2e` is the same through the
Python entry point `LLM.generate`, host token lists in and out, timed on the host around its decode
phase.  `prefill` is one step of 2,048 tokens; `points` holds decoding at batch 1 and 64.
Inputs are larger than L2 (a decode step reads every weight: 16 GB), so no explicit L2 flush.
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
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            parts = [p.strip() for p in s.split(",")]
            if len(parts) < 6:
                continue
            try:
                mhz.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(mhz)}


def model_bytes_and_flops(cfg: dict, n_layers: int):
    d, ff, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    qd = cfg["num_attention_heads"] * cfg["head_dim"]
    kvd = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = d * (qd + 2 * kvd) + qd * d + 3 * d * ff
    weights = per_layer * n_layers + V * d  # matrices a decode step reads: the layers and the classifier
    kv_per_token = 2 * kvd * n_layers
    return per_layer, weights, kv_per_token


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
    ctx, batch, K, W = args.context, args.batch, args.steps, args.warmup
    peaks = measured_peaks()
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
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

    def decode_run(B: int, steps: int, warm: int, sample_clocks: bool):
        """B sequences prefilled so that `warm + steps` decode steps end at position ctx; returns
        (tokens/s, ms/step, bytes a step must read, clocks, launches)."""
        start = ctx - (warm + steps)
        slots = [llm.open_sequence() for _ in range(B)]
        # prefill in pieces of at most 8192 tokens per step
        group = max(1, 8192 // start)
        for i in range(0, B, group):
            ents = [StepEntry(s, torch.randint(0, V, (start,), generator=gen).tolist(), []) for s in slots[i : i + group]]
            llm.step(ents)
        toks = torch.randint(0, V, (warm + steps, B), generator=gen).tolist()
        for w in range(warm):
            llm.step([StepEntry(s, [toks[w][j]], [0]) for j, s in enumerate(slots)])
        torch.cuda.synchronize()
        sampler = ClockSampler()
        if sample_clocks:
            sampler.start()
        l0 = ops.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for k in range(steps):
            llm.step([StepEntry(s, [toks[warm + k][j]], [0]) for j, s in enumerate(slots)])
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        launches = ops.launch_count() - l0
        clocks = sampler.stop() if sample_clocks else None
        mean_ctx = ctx - steps / 2.0
        bytes_step = 2 * weight_elems + 2 * kv_per_token * mean_ctx * B
        for s in slots:
            llm.close_sequence(s)
        return B * 1000.0 / ms, ms, bytes_step, clocks, launches

    if args.only == "prefill":
        value, ms_step, bytes_step, clocks, launches = 0.0, 1.0, 0.0, None, 0
    else:
        # ---- headline: batch `batch`
        value, ms_step, bytes_step, clocks, launches = decode_run(batch, K, W, True)
    achieved = bytes_step / (ms_step * 1e-3) / 1e9
    if args.only == "decode":
        print(json.dumps({"only": "decode", "batch": batch, "ms_per_step": ms_step, "tokens_per_s": value, "GBps": achieved, "layers": L}))
        return None

    # ---- other batch sizes
    points = {}
    for B in (1, 64):
        if args.only == "prefill":
            break
        if B * ctx + 64 * 64 > max_tokens:
            points[f"decode_b{B}"] = None  # its cache does not fit at this context
            continue
        v, _, _, _, _ = decode_run(B, max(8, K // 2), W, False)
        points[f"decode_b{B}"] = round(v, 1)

    # ---- prefill of 2048 tokens
    T = 2048
    slot_times = []
    for rep in range(W + 3):
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
    pre_ms = sorted(slot_times)[len(slot_times) // 2]
    H, hd = cfg["num_attention_heads"], cfg["head_dim"]
    flops = 2.0 * T * per_layer * L + 4.0 * T * T * hd * H / 2 * L + 2.0 * V * cfg["hidden_size"]
    pre_frac = flops / (pre_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12)
    if args.only == "prefill":
        print(json.dumps({"only": "prefill", "tokens": T, "ms": pre_ms, "tokens_per_s": T * 1000.0 / pre_ms, "frac": pre_frac, "layers": L}))
        return None

    # ---- end to end through the Python entry point: host token lists in, host token lists out
    prompts = [torch.randint(0, V, (ctx - (K + 1),), generator=gen).tolist() for _ in range(batch)]
    llm.generate(prompts[:1], max_new_tokens=4, temperature=0.0, stop_token_ids=[])  # warm the batch-1 paths
    llm.generate(prompts, max_new_tokens=W + 1, temperature=0.0, stop_token_ids=[])
    llm.generate(prompts, max_new_tokens=K + 1, temperature=0.0, stop_token_ids=[])
    st = llm.last_stats
    e2e_value = st.decode_steps * batch / st.decode_seconds if st.decode_seconds > 0 else None
    meta_ints = 4 * (3 * batch + (batch + 1) + 3 * batch + batch + batch * 64)

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
            "value": None if e2e_value is None else round(e2e_value, 1),
            "unit": "tokens/s",
            "h2d_bytes_per_step": meta_ints,
            "d2h_bytes_per_step": 4 * batch,
            "what": "LLM.generate decode phase, greedy, host lists in and out, host clock; starts right after the prompt step, whose power-capped SM clock takes about 130 ms to recover",
            "host_ms_per_step_in_step_call": round(1000.0 * st.decode_step_call_seconds / max(st.decode_steps, 1), 4),
            "host_ms_per_step_in_sample_call": round(1000.0 * st.decode_sample_call_seconds / max(st.decode_steps, 1), 4),
        },
        "gpu_launches": launches,
        "prefill": {"value": round(T * 1000.0 / pre_ms, 1), "tokens": T, "ms": round(pre_ms, 3), "frac": round(pre_frac, 4),
                    "peak_tflops": peaks["bf16_tflops"], "of": peaks["source"]},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4), "of": peaks["source"]},
        "points": points,
        "clocks": clocks,
    }
    return out


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
    out = run_ours(args)
    if out is not None:
        print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
