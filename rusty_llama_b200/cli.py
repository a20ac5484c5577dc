"""Command line, with the reference's option names and meanings (src/main.rs:24-66).

    rusty_llama <model_dir> [-t temperature] [-p top_p] [-s seed] [-n steps] [-i prompt]

    -t <float>  temperature, 0 = greedy     (default: 1.0)
    -p <float>  top-p / nucleus sampling    (default: 0.9)
    -s <int>    RNG seed                    (default: wall-clock time)
    -n <int>    number of steps to run      (default: 256): positions in total, the prompt included
    -i <ids>    prompt                      token ids separated by commas or spaces, or @file
                                            with one prompt per line (the reference takes text;
                                            tokenisation is the caller's here)
    --top-k <int>  --min-p <float>  --repeat-penalty <float>  --repeat-last-n <int>
    --frequency-penalty <float>  --presence-penalty <float>
    --mirostat <0|1|2>  --mirostat-lr <float>  --mirostat-ent <float>
    --xtc-probability <float>  --xtc-threshold <float>
    --dry-multiplier <float>  --dry-base <float>  --dry-allowed-length <int>  --dry-penalty-last-n <int>
    --dry-sequence-breaker <id>   (may be given up to 8 times; a token id where the reference takes a string)
                the reference's further sampling knobs, with its defaults (0, 0, 1.0, 64, 0, 0; 0, 0.1, 5.0; 0, 0.1;
                0, 1.75, 2, 64, none; src/main.rs:478-495); its grammar options, which work on token strings, are not built
Where the reference has `-z tokenizer` and `--backend`, this program has `--dtype bfloat16|float32`
(the second is the true 32-bit path) and `--random SEED` to run a folder that holds only a
config.json with random weights.  Generated ids go to standard output, one line per prompt, and
`[N tokens, X tok/s]` to standard error as in src/main.rs:410-413.
"""

from __future__ import annotations

import sys
import time
from typing import List

USAGE = __doc__


def parse_prompts(text: str) -> List[List[int]]:
    if text.startswith("@"):
        with open(text[1:], "r", encoding="utf-8") as f:
            lines = [ln for ln in f.read().splitlines() if ln.strip()]
    else:
        lines = [text]
    prompts = []
    for ln in lines:
        ids = [int(tok) for tok in ln.replace(",", " ").split()]
        prompts.append(ids)
    return prompts


def parse_args(argv: List[str]) -> dict:
    if not argv or argv[0] in ("-h", "--help"):
        print(USAGE)
        sys.exit(0 if argv else 1)
    args = {
        "model": argv[0], "temperature": 1.0, "top_p": 0.9, "seed": None, "steps": 256, "prompt": "",
        "dtype": "bfloat16", "random": None, "device": "cuda:0", "max_tokens": None,
        "top_k": 0, "min_p": 0.0, "repeat_penalty": 1.0, "repeat_last_n": 64, "frequency_penalty": 0.0,
        "presence_penalty": 0.0, "mirostat": 0, "mirostat_lr": 0.1, "mirostat_ent": 5.0,
        "xtc_probability": 0.0, "xtc_threshold": 0.1,
        "dry_multiplier": 0.0, "dry_base": 1.75, "dry_allowed_length": 2, "dry_penalty_last_n": 64, "dry_sequence_breakers": [],
    }
    flags = {
        "-t": ("temperature", float), "-p": ("top_p", float), "-s": ("seed", int), "-n": ("steps", int),
        "-i": ("prompt", str), "--dtype": ("dtype", str), "--random": ("random", int), "--device": ("device", str),
        "--max-tokens": ("max_tokens", int),
        "--top-k": ("top_k", int), "--min-p": ("min_p", float), "--repeat-penalty": ("repeat_penalty", float),
        "--repeat-last-n": ("repeat_last_n", int), "--frequency-penalty": ("frequency_penalty", float),
        "--presence-penalty": ("presence_penalty", float),
        "--mirostat": ("mirostat", int), "--mirostat-lr": ("mirostat_lr", float), "--mirostat-ent": ("mirostat_ent", float),
        "--xtc-probability": ("xtc_probability", float), "--xtc-threshold": ("xtc_threshold", float),
        "--dry-multiplier": ("dry_multiplier", float), "--dry-base": ("dry_base", float),
        "--dry-allowed-length": ("dry_allowed_length", int), "--dry-penalty-last-n": ("dry_penalty_last_n", int),
        "--dry-sequence-breaker": ("dry_sequence_breakers", int),
    }
    i = 1
    while i < len(argv):
        flag = argv[i]
        if flag in ("-h", "--help"):
            print(USAGE)
            sys.exit(0)
        if flag not in flags:
            raise SystemExit(f"unknown option '{flag}'\n\n{USAGE}")
        if i + 1 >= len(argv):
            raise SystemExit(f"missing value for '{flag}'")
        name, conv = flags[flag]
        try:
            if isinstance(args[name], list):
                args[name].append(conv(argv[i + 1]))  # an option that may be given more than once
            else:
                args[name] = conv(argv[i + 1])
        except ValueError:
            raise SystemExit(f"bad value '{argv[i + 1]}' for '{flag}'")
        i += 2
    return args


def main(argv=None) -> int:
    args = parse_args(list(sys.argv[1:] if argv is None else argv))
    prompts = parse_prompts(args["prompt"]) if args["prompt"] else []
    if not prompts or any(not p for p in prompts):
        print("error: the prompt is empty: give token ids with -i", file=sys.stderr)  # src/main.rs:294-296
        return 1
    from . import load, load_random

    if args["random"] is not None:
        llm = load_random(args["model"], seed=args["random"], dtype=args["dtype"], device=args["device"], max_tokens=args["max_tokens"])
    else:
        llm = load(args["model"], dtype=args["dtype"], device=args["device"], max_tokens=args["max_tokens"])
    t0 = time.perf_counter()
    outs = llm.generate(
        prompts, steps=args["steps"], temperature=args["temperature"], top_p=args["top_p"], seed=args["seed"],
        top_k=args["top_k"], min_p=args["min_p"], repeat_penalty=args["repeat_penalty"], repeat_last_n=args["repeat_last_n"],
        frequency_penalty=args["frequency_penalty"], presence_penalty=args["presence_penalty"],
        mirostat=args["mirostat"], mirostat_lr=args["mirostat_lr"], mirostat_ent=args["mirostat_ent"],
        xtc_probability=args["xtc_probability"], xtc_threshold=args["xtc_threshold"],
        dry_multiplier=args["dry_multiplier"], dry_base=args["dry_base"], dry_allowed_length=args["dry_allowed_length"],
        dry_penalty_last_n=args["dry_penalty_last_n"], dry_sequence_breakers=args["dry_sequence_breakers"],
    )
    dt = time.perf_counter() - t0
    n = 0
    for ids in outs:
        print(" ".join(str(t) for t in ids), flush=True)
        n += len(ids)
    print(f"[{n} tokens, {n / dt:.1f} tok/s]", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
