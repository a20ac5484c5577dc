"""Trace replay through bin/trace_run, the way a user drives it: the same requests whole, with their
last 32 tokens one by one, and in batches of unequal lengths that run one after another in a cache too
small for all of them, in 32-bit and in bfloat16, every logit compared with the plain implementation."""

import numpy as np
import pytest

from conftest import TINY
from helpers import TraceRun, check_logits, plain_all_logits

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 9, 13, 40, 70, 100, 128], "B": [1, 4, 17, 33, 60, 130, 200, 256]}


def make_requests(name):
    cfg = TINY[name][0]
    rng = np.random.default_rng(11 + len(name))
    return {f"r{n}": rng.integers(0, cfg["vocab_size"], n).tolist() for n in LENGTHS[name]}


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_whole_one_by_one_and_in_batches(name, dtype, tiny_dirs, tiny_weights, tmp_path):
    cfg = TINY[name][0]
    V = cfg["vocab_size"]
    requests = make_requests(name)
    ref = plain_all_logits(cfg, tiny_weights[name], dtype, requests)
    # room for the second and third longest requests at once, each rounded up to 64 (the longest fits
    # alone): the batches below are planned to fit, and the cache has to be used again and again
    some = sorted(LENGTHS[name])[-3:-1]
    max_tokens = sum((n + 63) // 64 * 64 for n in some)
    run = TraceRun(tiny_dirs[name], dtype, str(tmp_path / "out"), max_tokens, V)
    try:
        # 1. each request alone and whole, logits at every position
        for rid, toks in requests.items():
            got = run.step([(rid + "w", toks, range(len(toks)))], end=[rid + "w"])
            check_logits(got, ref[rid], dtype, f"{rid} whole")
        # 2. the last 32 tokens one by one (short requests: every token one by one, from the first)
        for rid, toks in requests.items():
            n = len(toks)
            head = max(n - 32, 0)
            rows = []
            if head:
                got = run.step([(rid + "s", toks[:head], range(head))])
                rows.append(got)
            for t in range(head, n):
                rows.append(run.step([(rid + "s", [toks[t]], [0])], end=[rid + "s"] if t == n - 1 else []))
            check_logits(np.concatenate(rows), ref[rid], dtype, f"{rid} last 32 one by one")
        # 3. batches of unequal lengths; a prefix of each prompt in one step, then one token each; the
        #    shorter requests end earlier; one batch after another in the slots the last one gave back
        ids = list(requests)
        batches, cur, used = [], [], 0
        for rid in ids:
            need = (len(requests[rid]) + 63) // 64 * 64
            if cur and used + need > max_tokens:
                batches.append(cur)
                cur, used = [], 0
            cur.append(rid)
            used += need
        batches.append(cur)
        assert len(batches) >= 3
        for batch in batches:
            got = {rid: [] for rid in batch}
            heads = {rid: max(1, len(requests[rid]) - 10 - 3 * i) for i, rid in enumerate(batch)}
            out = run.step([(rid + "b", requests[rid][: heads[rid]], range(heads[rid])) for rid in batch],
                           end=[rid + "b" for rid in batch if heads[rid] == len(requests[rid])])
            at = 0
            for rid in batch:
                got[rid].append(out[at : at + heads[rid]])
                at += heads[rid]
            pos = dict(heads)
            while True:
                live = [rid for rid in batch if pos[rid] < len(requests[rid])]
                if not live:
                    break
                ending = [rid + "b" for rid in live if pos[rid] + 1 == len(requests[rid])]
                out = run.step([(rid + "b", [requests[rid][pos[rid]]], [0]) for rid in live], end=ending)
                for i, rid in enumerate(live):
                    got[rid].append(out[i : i + 1])
                    pos[rid] += 1
            for rid in batch:
                check_logits(np.concatenate(got[rid]), ref[rid], dtype, f"{rid} in a batch of {len(batch)}")
        # a step that wants nothing writes no file
        assert run.step([("x", [1, 2, 3], [])], end=["x"]) is None
    finally:
        run.close()
