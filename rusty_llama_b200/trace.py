"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and owns no model code: it builds the same `LLM` that generation
uses and calls its step function.  The reference has no stand-alone program for this;
its tests do the same in-process (tests/prefill.rs:25-65, tests/integration.rs:236-286).

Input, one JSON object per line on standard input:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
`entries`: the next tokens of each request and the places among them whose logits are
wanted.  `end`: requests that are finished after this step; their slots and pages are
given back.  For a step in which something is wanted, `<out>/<step>.f32` receives the
logits [wanted, vocab] as little-endian float32, in the order of the entries and of
`want`.  After every step a line `done <step>` is printed and flushed.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True, help="positions live requests hold at most, each rounded up to 64")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    from . import load
    from .cache import PAGE_SIZE
    from .engine import StepEntry

    os.makedirs(args.out, exist_ok=True)
    max_seqs = max(1, (args.max_tokens + PAGE_SIZE - 1) // PAGE_SIZE)
    llm = load(args.model, dtype=args.dtype, device=args.device, max_tokens=args.max_tokens, max_seqs=max_seqs)
    slots: Dict[str, int] = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step_id = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = str(e["id"])
            if rid not in slots:
                slots[rid] = llm.open_sequence()
            entries.append(StepEntry(slots[rid], [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])]))
        if entries:
            logits = llm.step(entries)
            arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
            llm.engine.check_device_status()  # every step: a kernel that gave up on a wait ends the run here
            if logits.shape[0] > 0:
                tmp = os.path.join(args.out, f"{step_id}.f32.tmp")
                arr.tofile(tmp)
                os.replace(tmp, os.path.join(args.out, f"{step_id}.f32"))
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid in slots:
                llm.close_sequence(slots.pop(rid))
        print(f"done {step_id}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
