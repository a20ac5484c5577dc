"""The generation loop's decisions, with a scripted engine and sampler (no GPU)."""

import pytest
import torch

from rusty_llama_b200.cache import Cache
from rusty_llama_b200.engine import GenerationStats, generate, plan_batches
from rusty_llama_b200.engine.generate import MAX_NEW_TOKENS, POSITION_LIMIT, STOP_TOKEN
from rusty_llama_b200.errors import CacheError, StepError
from rusty_llama_b200.parts import KVNeed
from rusty_llama_b200.sampling import SamplingParams, sequence_seed


class FakeSpec:
    stop_token_ids = (0,)


class FakeModel:
    spec = FakeSpec()


class FakeEngine:
    """Keeps a real Cache (so slots and pages are really taken and given back) and answers a step with
    'logits' that encode (slot, position of the row): the fake sampler turns them into scripted tokens."""

    def __init__(self, max_tokens=64 * 8, max_seqs=4, max_positions=40):
        self.cache = Cache([(0, KVNeed(1, 8, 0))], max_tokens, max_seqs, torch.float32, "cpu")
        self.model = FakeModel()
        self.max_positions = max_positions
        self.steps = []  # per step: list of (slot, n tokens)
        self.fed = {}  # slot -> tokens fed so far
        self.peak_open = 0

    def open_sequence(self):
        s = self.cache.open_sequence()
        self.fed[s] = []
        self.peak_open = max(self.peak_open, self.cache.n_open)
        return s

    def close_sequence(self, slot):
        self.cache.close_sequence(slot)

    def step(self, entries):
        slots = [e.slot for e in entries]
        lens = [len(e.tokens) for e in entries]
        self.cache.reserve(slots, lens)
        self.cache.commit(slots, lens)
        self.steps.append(list(zip(slots, lens)))
        rows = []
        for e in entries:
            self.fed[e.slot].extend(e.tokens)
            assert list(e.want) == [len(e.tokens) - 1]
            rows.append([float(e.slot), float(self.cache.length(e.slot))])
        return torch.tensor(rows)


class ScriptedSampler:
    """Token for the row of a sequence of length n that began with prompt token p: script[p][n]."""

    def __init__(self, engine, script):
        self.engine, self.script, self.seeded = engine, script, {}

    def seed_slots(self, slots, seeds):
        for s, sd in zip(slots, seeds):
            self.seeded[s] = sd

    def sample(self, logits, slots, params):
        out = []
        for row, slot in zip(logits.tolist(), slots):
            assert int(row[0]) == slot
            first = self.engine.fed[slot][0]
            out.append(self.script(first, int(row[1])))
        return torch.tensor(out, dtype=torch.int32)


def test_plan_batches_respects_pages_and_batch_size():
    assert plan_batches([10, 10, 10], [20, 20, 20], 1000, page_budget=2, max_batch=8) == [[0, 1], [2]]
    assert plan_batches([10] * 5, [5] * 5, 1000, page_budget=100, max_batch=2) == [[0, 1], [2, 3], [4]]
    assert plan_batches([100], [1000], 128, page_budget=2, max_batch=8) == [[0]]  # clamped by the position limit
    with pytest.raises(StepError, match="pages"):
        plan_batches([200], [10], 1000, page_budget=2, max_batch=8)


def test_unequal_prompts_stop_tokens_and_early_leavers():
    eng = FakeEngine()
    # sequences are known by their first prompt token; token 0 stops
    script = lambda first, n: {11: 0 if n == 6 else 50 + n, 12: 60 + n, 13: 0 if n == 3 else 70 + n}[first]
    smp = ScriptedSampler(eng, script)
    prompts = [[11, 1, 1, 1], [12, 2], [13, 3, 3]]
    stats = GenerationStats()
    res = generate(eng, smp, prompts, 5, SamplingParams(0.0, 0.9, 7), stats=stats)
    assert [r.tokens for r in res] == [[54, 55], [62, 63, 64, 65, 66], []]
    assert [r.finish_reason for r in res] == [STOP_TOKEN, MAX_NEW_TOKENS, STOP_TOKEN]
    # first step: the three prompts together, with their own lengths; then shrinking decode batches
    assert sorted(n for _, n in eng.steps[0]) == [2, 3, 4]
    assert [len(s) for s in eng.steps[1:]] == [2, 2, 1, 1]
    assert all(n == 1 for st in eng.steps[1:] for _, n in st)
    # the last emitted token is not fed back; a stop token is never fed
    for slot, fed in eng.fed.items():
        assert 0 not in fed
    assert eng.cache.n_open == 0 and eng.cache.pages_free() == eng.cache.n_pages
    assert stats.prompt_tokens == 9 and stats.generated_tokens == 7 and stats.decode_steps == 4 and stats.batches == 1
    assert smp.seeded and set(smp.seeded.values()) == {sequence_seed(7, i) for i in range(3)}


def test_include_stop_and_callback_order():
    eng = FakeEngine()
    smp = ScriptedSampler(eng, lambda first, n: 0 if n == 4 else 9)
    seen = []
    res = generate(eng, smp, [[5, 5]], 10, SamplingParams(0.0), include_stop=True, on_token=lambda r, t: seen.append((r, t)))
    assert res[0].tokens == [9, 9, 0] and res[0].finish_reason == STOP_TOKEN
    assert seen == [(0, 9), (0, 9)]


def test_more_requests_than_slots_run_batch_after_batch_in_the_same_slots():
    eng = FakeEngine(max_seqs=2)
    smp = ScriptedSampler(eng, lambda first, n: first)
    prompts = [[20 + i] * (1 + i) for i in range(5)]
    res = generate(eng, smp, prompts, 3, SamplingParams(0.0), stop_token_ids=[])
    assert [r.tokens for r in res] == [[20 + i] * 3 for i in range(5)]
    assert eng.peak_open == 2 and set(eng.fed) == {0, 1}  # only two slots ever existed
    assert eng.cache.n_open == 0
    eng.cache.check_consistent()


def test_position_limit_and_budget_per_prompt():
    eng = FakeEngine(max_positions=6)
    smp = ScriptedSampler(eng, lambda first, n: 9)
    res = generate(eng, smp, [[1, 1, 1, 1], [2]], [10, 2], SamplingParams(0.0), stop_token_ids=[])
    # 4 prompt positions + 2 fed tokens fill the 6 positions; the third token is produced but cannot be fed
    assert res[0].tokens == [9, 9, 9] and res[0].finish_reason == POSITION_LIMIT
    assert res[1].tokens == [9, 9] and res[1].finish_reason == MAX_NEW_TOKENS
    with pytest.raises(StepError, match="limit"):
        generate(eng, smp, [[1] * 7], 1, SamplingParams(0.0))
    with pytest.raises(StepError, match="empty"):
        generate(eng, smp, [[]], 1, SamplingParams(0.0))
    assert generate(eng, smp, [[1]], 0, SamplingParams(0.0))[0].tokens == []


class AheadEngine(FakeEngine):
    """A FakeEngine that also steps on tokens it is handed as a tensor, as the real engine does for
    tokens that are still on the device; it records which steps were launched that way."""

    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        self.ahead_steps = []

    def step_device_tokens(self, slots, tokens):
        from rusty_llama_b200.engine import StepEntry

        assert tokens.dtype == torch.int32 and tuple(tokens.shape) == (len(slots),)
        self.ahead_steps.append(len(self.steps))
        return self.step([StepEntry(s, [int(t)], [0]) for s, t in zip(slots, tokens.tolist())])


@pytest.mark.parametrize("case", ["stops", "budgets", "limit"])
def test_launching_ahead_gives_the_same_tokens_and_frees_everything(case):
    """Steps launched before the host has read the tokens: same results, reasons and callbacks as
    the plain loop; a sequence that drew a stop token has been stepped once more (its stop token
    was fed) and nothing of it is kept; no step is launched ahead when a budget or the position
    limit may end a sequence."""
    if case == "stops":
        script = lambda first, n: {11: 0 if n == 6 else 50 + n, 12: 60 + n, 13: 0 if n == 5 else 70 + n}[first]
        prompts, budget, kw = [[11, 1, 1, 1], [12, 2], [13, 3, 3]], 6, {}
    elif case == "budgets":
        script = lambda first, n: 30 + n
        prompts, budget, kw = [[11, 1], [12, 2, 2], [13]], [2, 5, 3], {"stop_token_ids": []}
    else:
        script = lambda first, n: 9
        prompts, budget, kw = [[1, 1, 1, 1], [2]], [10, 4], {"stop_token_ids": []}
    runs = []
    for ahead in (False, True):
        eng = AheadEngine(max_positions=8 if case == "limit" else 40)
        smp = ScriptedSampler(eng, script)
        seen = []
        stats = GenerationStats()
        res = generate(eng, smp, prompts, budget, SamplingParams(0.0, 0.9, 7), on_token=lambda r, t: seen.append((r, t)),
                       stats=stats, launch_ahead=ahead, **kw)
        assert eng.cache.n_open == 0 and eng.cache.pages_free() == eng.cache.n_pages
        eng.cache.check_consistent()
        runs.append(([(r.tokens, r.finish_reason) for r in res], seen, stats.generated_tokens))
        if not ahead:
            assert eng.ahead_steps == []
        else:
            assert eng.ahead_steps, "no step was launched ahead"
            assert stats.decode_steps == len(eng.steps) - 1
            if case == "stops":
                # a stop token is fed only by a step that was launched ahead
                assert any(0 in fed for fed in eng.fed.values())
    assert runs[0] == runs[1]


def test_launching_ahead_never_steps_past_a_budget_or_the_position_limit():
    eng = AheadEngine(max_positions=7)
    smp = ScriptedSampler(eng, lambda first, n: 9)
    res = generate(eng, smp, [[1, 1, 1, 1], [2]], [10, 3], SamplingParams(0.0), stop_token_ids=[])
    assert res[0].tokens == [9, 9, 9, 9] and res[0].finish_reason == POSITION_LIMIT
    assert res[1].tokens == [9, 9, 9] and res[1].finish_reason == MAX_NEW_TOKENS
    # positions fed: the long one 4 + 3, the short one 1 + 2; the cache never saw more
    assert sorted(len(f) for f in eng.fed.values()) == [3, 7]


def test_slots_are_given_back_when_a_step_fails():
    eng = FakeEngine()
    smp = ScriptedSampler(eng, lambda first, n: 9)

    def boom(entries):
        raise CacheError("scripted failure")

    eng.step = boom
    with pytest.raises(CacheError, match="scripted"):
        generate(eng, smp, [[1, 2], [3]], 4, SamplingParams(0.0))
    assert eng.cache.n_open == 0


def test_sequence_seeds():
    assert sequence_seed(12345, 0) == 12345 and sequence_seed(0, 0) == 1
    seeds = {sequence_seed(12345, i) for i in range(100)}
    assert len(seeds) == 100 and 0 not in seeds


def test_command_line_options_follow_the_reference(tmp_path):
    """-t -p -s -n -i with the reference's names, meanings and defaults (src/main.rs:24-66)."""
    from rusty_llama_b200.cli import main, parse_args, parse_prompts

    a = parse_args(["some/dir"])
    assert (a["temperature"], a["top_p"], a["seed"], a["steps"], a["prompt"], a["dtype"]) == (1.0, 0.9, None, 256, "", "bfloat16")
    a = parse_args(["m", "-t", "0", "-p", "0.5", "-s", "42", "-n", "17", "-i", "1, 2 3", "--dtype", "float32"])
    assert (a["temperature"], a["top_p"], a["seed"], a["steps"], a["prompt"], a["dtype"]) == (0.0, 0.5, 42, 17, "1, 2 3", "float32")
    assert (a["top_k"], a["min_p"], a["repeat_penalty"], a["repeat_last_n"], a["frequency_penalty"], a["presence_penalty"]) == (0, 0.0, 1.0, 64, 0.0, 0.0)  # src/main.rs:478-485
    a = parse_args(["m", "--top-k", "40", "--min-p", "0.05", "--repeat-penalty", "1.1", "--repeat-last-n", "32", "--frequency-penalty", "0.2", "--presence-penalty", "0.3"])
    assert (a["top_k"], a["min_p"], a["repeat_penalty"], a["repeat_last_n"], a["frequency_penalty"], a["presence_penalty"]) == (40, 0.05, 1.1, 32, 0.2, 0.3)
    a = parse_args(["m", "--mirostat", "2", "--mirostat-lr", "0.2", "--mirostat-ent", "4"])
    assert (a["mirostat"], a["mirostat_lr"], a["mirostat_ent"]) == (2, 0.2, 4.0)
    assert (parse_args(["m"])["mirostat"], parse_args(["m"])["mirostat_lr"], parse_args(["m"])["mirostat_ent"]) == (0, 0.1, 5.0)
    a = parse_args(["m", "--xtc-probability", "0.5", "--xtc-threshold", "0.2"])
    assert (a["xtc_probability"], a["xtc_threshold"]) == (0.5, 0.2)
    assert (parse_args(["m"])["xtc_probability"], parse_args(["m"])["xtc_threshold"]) == (0.0, 0.1)
    a = parse_args(["m", "--dry-multiplier", "0.8", "--dry-base", "2", "--dry-allowed-length", "3", "--dry-penalty-last-n", "128",
                    "--dry-sequence-breaker", "13", "--dry-sequence-breaker", "198"])
    assert (a["dry_multiplier"], a["dry_base"], a["dry_allowed_length"], a["dry_penalty_last_n"], a["dry_sequence_breakers"]) == (0.8, 2.0, 3, 128, [13, 198])
    d = parse_args(["m"])
    assert (d["dry_multiplier"], d["dry_base"], d["dry_allowed_length"], d["dry_penalty_last_n"], d["dry_sequence_breakers"]) == (0.0, 1.75, 2, 64, [])
    with pytest.raises(SystemExit, match="unknown option"):
        parse_args(["m", "--grammar", "root ::= x"])  # not built: works on token strings
    assert parse_prompts("1, 2 3") == [[1, 2, 3]]
    f = tmp_path / "prompts.txt"
    f.write_text("5 6\n\n7,8,9\n")
    assert parse_prompts("@" + str(f)) == [[5, 6], [7, 8, 9]]
    with pytest.raises(SystemExit, match="unknown option"):
        parse_args(["m", "-z", "tok.bin"])
    with pytest.raises(SystemExit, match="missing value"):
        parse_args(["m", "-t"])
    with pytest.raises(SystemExit, match="bad value"):
        parse_args(["m", "-n", "many"])
    assert main(["m", "-n", "4"]) == 1  # an empty prompt is an error before anything is loaded (src/main.rs:294-296)


def test_sampling_params_pick_the_chain_as_the_reference_does():
    """The longer chain is built as soon as one of its knobs leaves its neutral value (src/sampler.rs:868-876)."""
    from rusty_llama_b200.errors import ConfigError
    from rusty_llama_b200.sampling import SamplingParams

    assert not SamplingParams(0.8, 0.9, 1).longer_chain
    assert not SamplingParams(0.8, 0.9, 1, repeat_last_n=8).longer_chain  # a window alone changes nothing
    for kw in (dict(top_k=5), dict(min_p=0.1), dict(repeat_penalty=1.1), dict(frequency_penalty=0.5), dict(presence_penalty=-0.5), dict(mirostat=2), dict(xtc_probability=0.3), dict(dry_multiplier=0.8)):
        p = SamplingParams(0.8, 0.9, 1, **kw)
        p.validate()
        assert p.longer_chain
    for kw in (dict(top_k=-1), dict(repeat_penalty=0.0), dict(repeat_last_n=5000), dict(min_p=float("nan")), dict(mirostat=3)):
        with pytest.raises(ConfigError):
            SamplingParams(0.8, 0.9, 1, **kw).validate()
    with pytest.raises(ConfigError, match="temperature"):
        SamplingParams(0.0, 0.9, 1, mirostat=1).validate()


def test_bench_answers_for_more_gpus_and_for_the_reference_arm():
    """`bench.py --gpus 2` says in one line that it measures one GPU and exits with 2; `--impl reference` prints
    its `unavailable` line and exits with 0.  Neither touches a GPU."""
    import json
    import os
    import subprocess
    import sys

    bench = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "bench.py")
    two = subprocess.run([sys.executable, bench, "--gpus", "2"], capture_output=True, text=True, timeout=120)
    assert two.returncode == 2 and len(two.stdout.strip().splitlines()) == 1 and "one GPU" in two.stdout
    ref = subprocess.run([sys.executable, bench, "--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3"],
                         capture_output=True, text=True, timeout=120)
    line = json.loads(ref.stdout.strip())
    assert ref.returncode == 0 and line["impl"] == "reference" and isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]


def test_bench_measures_again_when_a_kernel_gave_up():
    """A run in which a bounded wait ran out is discarded and repeated once; the line says so; a second failure is
    the caller's."""
    import bench
    from rusty_llama_b200.errors import KernelError

    calls = []

    def flaky():
        calls.append(1)
        if len(calls) == 1:
            raise KernelError("gemm_tc: the tensor-core issuer gave up waiting on a barrier (code 2)")
        return {"value": 1.0}

    out = bench.measured_again_if_a_kernel_gave_up(flaky)
    assert len(calls) == 2 and out["value"] == 1.0 and "code 2" in out["measured_again"]
    assert bench.measured_again_if_a_kernel_gave_up(lambda: {"value": 2.0}) == {"value": 2.0}

    def broken():
        raise KernelError("again")

    with pytest.raises(KernelError):
        bench.measured_again_if_a_kernel_gave_up(broken)
