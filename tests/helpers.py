"""Helpers shared by the GPU tests: the plain implementation's logits, tolerances, trace replay."""

import json
import os
import subprocess
import sys

import numpy as np
import torch

from plain_llama import plain_logits

from conftest import rounded_weights

REPO = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")


def plain_all_logits(cfg, weights, dtype_name, requests):
    """request id -> float64 logits [len, vocab] of the whole sequence, from the weights as a run of
    `dtype_name` holds them."""
    w = rounded_weights(weights, dtype_name)
    return {rid: plain_logits(cfg, w, toks, torch.float64).numpy() for rid, toks in requests.items()}


def check_logits(got, ref, dtype_name, what=""):
    """float32 runs: the engine and the plain float64 result differ by 32-bit rounding only.
    bfloat16 runs: every activation between two kernels is rounded to 8 bits; over the few dozen
    roundings of a tiny model that is a few percent of the logits' range at worst, well under one
    percent on average."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    scale = float(np.abs(ref).max())
    err = np.abs(got - ref)
    if dtype_name == "float32":
        assert err.max() <= 5e-5 * scale + 1e-6, f"{what}: max error {err.max():.3e} at range {scale:.3e}"
    else:
        assert err.max() <= 3e-2 * scale, f"{what}: max error {err.max():.3e} at range {scale:.3e}"
        assert err.mean() <= 6e-3 * scale, f"{what}: mean error {err.mean():.3e} at range {scale:.3e}"


class TraceRun:
    """bin/trace_run as a child process: send a step, wait for its `done` line, read its file."""

    def __init__(self, model_dir, dtype, out_dir, max_tokens, vocab):
        self.out_dir, self.vocab = out_dir, vocab
        self.proc = subprocess.Popen(
            [sys.executable, os.path.join(REPO, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
             "--out", out_dir, "--max-tokens", str(max_tokens)],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1,
        )
        self.n = 0

    def step(self, entries, end=()):
        """entries: list of (id, tokens, want).  Returns float32 [wanted, vocab] or None."""
        rec = {"step": self.n, "entries": [{"id": i, "tokens": list(map(int, t)), "want": list(w)} for i, t, w in entries], "end": list(end)}
        self.proc.stdin.write(json.dumps(rec) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline()
        assert line.strip() == f"done {self.n}", f"trace_run answered {line!r} (exit {self.proc.poll()})"
        path = os.path.join(self.out_dir, f"{self.n}.f32")
        self.n += 1
        wanted = sum(len(w) for _, _, w in entries)
        if wanted == 0:
            assert not os.path.exists(path)
            return None
        arr = np.fromfile(path, dtype="<f4")
        assert arr.size == wanted * self.vocab
        return arr.reshape(wanted, self.vocab)

    def close(self):
        self.proc.stdin.close()
        rc = self.proc.wait(timeout=120)
        assert rc == 0, f"trace_run exited with {rc}"
