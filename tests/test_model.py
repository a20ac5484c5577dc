"""The engine in-process against the plain implementation: whole sequences, cuts, batches, long decoding,
slot reuse, generation through the entry point."""

import numpy as np
import pytest
import torch

from conftest import TINY, rounded_weights
from helpers import check_logits, plain_all_logits
from plain_llama import plain_generate, plain_logits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def llms(tiny_dirs):
    import rusty_llama_b200 as rl

    made = {}

    def get(name, dtype, **kw):
        key = (name, dtype, tuple(sorted(kw.items())))
        if key not in made:
            made[key] = rl.load(tiny_dirs[name], dtype=dtype, max_tokens=kw.pop("max_tokens", 64 * 16), **kw)
        return made[key]

    return get


class ShiftedRng:
    """The plain generator with its draw number `at` moved by `shift` (for `parted_within_rounding`)."""

    def __init__(self, seed, at, shift):
        from plain_llama import PlainRng

        self.inner, self.at, self.shift, self.n = PlainRng(seed), at, shift, 0

    def next_f32(self):
        v = self.inner.next_f32()
        if self.n == self.at:
            v = min(max(v + self.shift, 0.0), 0.99999994)
        self.n += 1
        return v


def parted_within_rounding(cfg, w, prompt, got, want, make_sampler):
    """Where the engine's sampled stream `got` leaves the plain stream `want`, is the engine's token what the
    plain sampler draws when that one draw's coin, or its temperature, moves by 1e-5 or less?  The engine's
    32-bit logits equal the plain ones to a few 1e-5 of their range, so a draw that lands that close to a
    boundary of the cumulative distribution (or a nucleus that closes that close to top-p) may fall on either
    side; any other parting is a fault.  make_sampler(rng) -> callable(logits) with fresh state."""
    k = next(i for i, (a, b) in enumerate(zip(got, want)) if a != b)
    trials = [(d, 1.0) for d in (1e-6, -1e-6, 1e-5, -1e-5)] + [(0.0, 1.0 + d) for d in (1e-5, -1e-5, 3e-5, -3e-5)]
    for shift, t_scale in trials:
        sampler = make_sampler(lambda seed: ShiftedRng(seed, k, shift))
        seq = list(prompt)
        for j in range(k + 1):
            logits = plain_logits(cfg, w, seq)[-1].to(torch.float32).numpy()
            tok = sampler(logits / np.float32(t_scale) if j == k else logits)
            if j < k:
                if tok != want[j]:
                    break
                seq.append(tok)
        else:
            if tok == got[k]:
                return True
    return False


def step_all(llm, slot, tokens):
    from rusty_llama_b200 import StepEntry

    return llm.step([StepEntry(slot, tokens, list(range(len(tokens))))]).cpu().numpy()


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_sequence_logits(name, dtype, llms, tiny_weights):
    cfg = TINY[name][0]
    llm = llms(name, dtype)
    rng = np.random.default_rng(3)
    for n in (1, 7, 64, 65, cfg["max_position_embeddings"]):
        toks = rng.integers(0, cfg["vocab_size"], n).tolist()
        ref = plain_all_logits(cfg, tiny_weights[name], dtype, {"r": toks})["r"]
        slot = llm.open_sequence()
        got = step_all(llm, slot, toks)
        llm.close_sequence(slot)
        check_logits(got, ref, dtype, f"tiny {name}, {n} tokens")


@pytest.mark.parametrize("name", ["A", "B"])
def test_float32_bits_do_not_depend_on_cut_or_batch(name, llms):
    """In 32-bit every kernel adds in an order that depends on the token alone, so the logits at a
    position are the same bits whole, one by one, chunked, or next to other sequences."""
    from rusty_llama_b200 import StepEntry

    cfg = TINY[name][0]
    llm = llms(name, "float32")
    rng = np.random.default_rng(5)
    a = rng.integers(0, cfg["vocab_size"], 90).tolist()
    b = rng.integers(0, cfg["vocab_size"], 37).tolist()
    s = llm.open_sequence()
    whole = torch.from_numpy(step_all(llm, s, a))
    llm.close_sequence(s)
    s = llm.open_sequence()
    parts = [torch.from_numpy(step_all(llm, s, a[:50]))]
    parts.append(torch.from_numpy(step_all(llm, s, a[50:58])))
    for t in a[58:]:
        parts.append(torch.from_numpy(step_all(llm, s, [t])))
    llm.close_sequence(s)
    assert torch.equal(torch.cat(parts), whole)
    s1, s2 = llm.open_sequence(), llm.open_sequence()
    out = llm.step([StepEntry(s2, b, [len(b) - 1]), StepEntry(s1, a, list(range(90)))]).cpu()
    llm.close_sequence(s1)
    llm.close_sequence(s2)
    assert torch.equal(out[1:], whole)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_with_and_without_graphs(dtype, llms, tiny_weights):
    """A prompt of 3 tokens, then one token per step up to the position limit: the decode kernels and
    the captured graph see every length, page boundaries included."""
    from rusty_llama_b200 import StepEntry

    name = "B"
    cfg = TINY[name][0]
    n = cfg["max_position_embeddings"]
    toks = np.random.default_rng(9).integers(0, cfg["vocab_size"], n).tolist()
    ref = plain_all_logits(cfg, tiny_weights[name], dtype, {"r": toks})["r"]
    for graphs in (True, False):
        llm = llms(name, dtype, use_graphs=graphs)
        s = llm.open_sequence()
        rows = [step_all(llm, s, toks[:3])]
        for t in toks[3:]:
            rows.append(llm.step([StepEntry(s, [t], [0])]).cpu().numpy())
        llm.close_sequence(s)
        check_logits(np.concatenate(rows), ref, dtype, f"decoding to {n}, graphs={graphs}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batched_decoding_with_leavers_and_slot_reuse(dtype, llms, tiny_weights):
    """Batches of unequal prompts decode together; the short ones end; their slots and pages go to the
    next batch, whose logits must not see what the slots held before."""
    from rusty_llama_b200 import StepEntry

    name = "A"
    cfg = TINY[name][0]
    llm = llms(name, dtype, max_tokens=64 * 5, max_seqs=3)
    rng = np.random.default_rng(21)
    for round_ in range(3):
        lens = [(5, 12), (9, 30), (13, 66)] if round_ % 2 == 0 else [(70, 75), (1, 20), (64, 65)]
        seqs = {i: rng.integers(0, cfg["vocab_size"], total).tolist() for i, (_, total) in enumerate(lens)}
        ref = plain_all_logits(cfg, tiny_weights[name], dtype, seqs)
        slots = {i: llm.open_sequence() for i in seqs}
        assert set(slots.values()) == {0, 1, 2}
        got = {i: [] for i in seqs}
        out = llm.step([StepEntry(slots[i], seqs[i][: lens[i][0]], [lens[i][0] - 1]) for i in seqs]).cpu().numpy()
        pos = {}
        for j, i in enumerate(seqs):
            got[i].append(out[j : j + 1])
            pos[i] = lens[i][0]
        while True:
            live = [i for i in seqs if pos[i] < lens[i][1]]
            if not live:
                break
            out = llm.step([StepEntry(slots[i], [seqs[i][pos[i]]], [0]) for i in live]).cpu().numpy()
            for j, i in enumerate(live):
                got[i].append(out[j : j + 1])
                pos[i] += 1
                if pos[i] == lens[i][1]:
                    llm.close_sequence(slots[i])
        for i in seqs:
            check_logits(np.concatenate(got[i]), ref[i][lens[i][0] - 1 :], dtype, f"round {round_}, sequence {i}")
        llm.engine.cache.check_consistent()
        assert llm.engine.cache.n_open == 0


@pytest.mark.parametrize("name, n_seqs", [("A", 12), ("B", 40)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_steps_of_more_than_eight_sequences(name, n_seqs, dtype, llms, tiny_weights):
    """Batches of 12 and 40 unequal prompts: above 8 rows the bfloat16 decode step takes other kernels (the
    tensor-core products, the norm folded into them) than the small batches of the other tests."""
    from rusty_llama_b200 import StepEntry

    cfg = TINY[name][0]
    llm = llms(name, dtype, max_tokens=64 * 2 * n_seqs, max_seqs=n_seqs)
    rng = np.random.default_rng(n_seqs)
    new = 6
    lens = [int(rng.integers(1, 70)) for _ in range(n_seqs)]
    seqs = {i: rng.integers(0, cfg["vocab_size"], lens[i] + new).tolist() for i in range(n_seqs)}
    ref = plain_all_logits(cfg, tiny_weights[name], dtype, seqs)
    slots = {i: llm.open_sequence() for i in seqs}
    got = {i: [] for i in seqs}
    out = llm.step([StepEntry(slots[i], seqs[i][: lens[i]], [lens[i] - 1]) for i in seqs]).cpu().numpy()
    for i in seqs:
        got[i].append(out[i : i + 1])
    for t in range(new):
        out = llm.step([StepEntry(slots[i], [seqs[i][lens[i] + t]], [0]) for i in seqs]).cpu().numpy()
        for i in seqs:
            got[i].append(out[i : i + 1])
    for i in seqs:
        llm.close_sequence(slots[i])
        check_logits(np.concatenate(got[i]), ref[i][lens[i] - 1 :], dtype, f"sequence {i} of {n_seqs}")
    llm.engine.cache.check_consistent()


def test_step_errors_come_before_any_launch(llms):
    from rusty_llama_b200 import CacheError, StepEntry, StepError

    llm = llms("A", "float32", max_tokens=64 * 2, max_seqs=2)
    s = llm.open_sequence()
    with pytest.raises(StepError, match="outside the vocabulary"):
        llm.step([StepEntry(s, [1, 256], [0])])
    with pytest.raises(StepError, match="no token"):
        llm.step([StepEntry(s, [], [])])
    with pytest.raises(StepError, match="limit"):
        llm.step([StepEntry(s, [1] * 129, [])])
    with pytest.raises(StepError, match="index 3"):
        llm.step([StepEntry(s, [1, 2, 3], [3])])
    with pytest.raises(StepError, match="twice"):
        llm.step([StepEntry(s, [1], []), StepEntry(s, [2], [])])
    with pytest.raises(StepError, match="at least one"):
        llm.step([])
    with pytest.raises(CacheError, match="not open"):
        llm.step([StepEntry(1, [1], [])])
    assert llm.engine.cache.length(s) == 0
    s2 = llm.open_sequence()
    llm.step([StepEntry(s, [1] * 100, [])])
    with pytest.raises(CacheError, match="out of cache pages"):
        llm.step([StepEntry(s2, [1] * 10, [])])
    assert llm.engine.cache.length(s2) == 0 and llm.engine.cache.length(s) == 100
    llm.close_sequence(s)
    llm.close_sequence(s2)


@pytest.mark.parametrize("name, dtype", [("A", "float32"), ("A", "bfloat16"), ("B", "float32")])
def test_greedy_generation_through_the_entry_point(name, dtype, llms, tiny_weights):
    """Tiny A's workload: prompts of 5, 9 and 13 tokens, 8 greedy tokens each, one batch."""
    cfg = TINY[name][0]
    llm = llms(name, dtype)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (5, 9, 13)]
    outs = llm.generate(prompts, max_new_tokens=8, temperature=0.0, stop_token_ids=[])
    w = rounded_weights(tiny_weights[name], dtype)
    for p, got in zip(prompts, outs):
        want = plain_generate(cfg, w, p, 8, temperature=0.0)
        if dtype == "float32":
            assert got == want
        else:
            # bfloat16 may pick the other of two nearly equal logits; up to there the streams agree, and
            # the token it picked is within rounding of the best one
            k = next((i for i, (a, b) in enumerate(zip(got, want)) if a != b), None)
            if k is not None:
                l = plain_logits(cfg, w, p + want[:k])[-1]
                assert float(l[want[k]] - l[got[k]]) <= 3e-2 * float(l.abs().max())
    assert llm.last_stats.prompt_tokens == 27 and llm.last_stats.generated_tokens == 24
    assert llm.engine.cache.n_open == 0
    # the reference's `steps` counts positions, prompt included (src/model.rs:1668-1690)
    assert len(llm.generate(prompts[0], steps=9, temperature=0.0, stop_token_ids=[])) == 4
    # one prompt, one list back; stop tokens end a sequence and are not returned
    first = llm.generate(prompts[1], max_new_tokens=8, temperature=0.0, stop_token_ids=[])
    k = max(i for i in range(8) if first[i] not in first[:i])  # the last token that did not occur before
    res = llm.generate(prompts[1], max_new_tokens=8, temperature=0.0, stop_token_ids=[first[k]], return_results=True)
    assert res.tokens == first[:k] and res.finish_reason == "stop_token"


def test_sampled_generation_follows_the_plain_sampler(llms, tiny_weights):
    """Tiny B's workload: prompts of 1, 4, 17, 33 and 60 tokens, 16 tokens each at temperature 0.8, top-p 0.9.
    In 32-bit the engine's logits equal the plain ones to rounding, so the same seeds give the same draws
    unless a draw lands within rounding of a boundary; then the streams part and are compared up to there."""
    from rusty_llama_b200.sampling import sequence_seed

    name = "B"
    cfg = TINY[name][0]
    llm = llms(name, "float32")
    rng = np.random.default_rng(1)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (1, 4, 17, 33, 60)]
    outs = llm.generate(prompts, max_new_tokens=16, temperature=0.8, top_p=0.9, seed=4242, stop_token_ids=[])
    again = llm.generate(prompts, max_new_tokens=16, temperature=0.8, top_p=0.9, seed=4242, stop_token_ids=[])
    assert outs == again
    alone = llm.generate(prompts[2], max_new_tokens=16, temperature=0.8, top_p=0.9, seed=sequence_seed(4242, 2), stop_token_ids=[])
    w = rounded_weights(tiny_weights[name], "float32")
    from plain_llama import plain_sample

    agree = 0
    for i, (p, got) in enumerate(zip(prompts, outs)):
        want = plain_generate(cfg, w, p, 16, temperature=0.8, top_p=0.9, seed=sequence_seed(4242, i))
        agree += int(got == want)
        assert len(got) == 16
        if got != want:  # only a draw within rounding of a boundary may part the streams
            def make(rng_of, seed=sequence_seed(4242, i)):
                rng = rng_of(seed)
                return lambda logits: plain_sample(logits, 0.8, 0.9, rng)

            assert parted_within_rounding(cfg, w, p, got, want, make), f"sequence {i}: {got} left {want} at a clear margin"
    assert agree >= 4
    assert alone == outs[2]  # a sequence's draws do not depend on its neighbours


def test_generation_with_the_longer_sampler_chain(llms, tiny_weights):
    """top-k, min-p and the penalties through the entry point, in 32-bit, against the plain chain fed by the
    plain model: the kernel keeps each sequence's ring of chosen tokens itself, across steps and batches."""
    from plain_llama import PlainChain
    from rusty_llama_b200.sampling import sequence_seed

    name = "A"
    cfg = TINY[name][0]
    llm = llms(name, "float32")
    rng = np.random.default_rng(8)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (3, 20, 41)]
    knobs = dict(temperature=0.9, top_p=0.95, top_k=20, min_p=0.02, repeat_penalty=1.3, repeat_last_n=6, frequency_penalty=0.2, presence_penalty=0.1)
    outs = llm.generate(prompts, max_new_tokens=24, seed=77, stop_token_ids=[], **knobs)
    assert outs == llm.generate(prompts, max_new_tokens=24, seed=77, stop_token_ids=[], **knobs)  # the rings start empty again
    assert outs == llm.generate(prompts, max_new_tokens=24, seed=77, stop_token_ids=[], launch_ahead=False, **knobs)
    w = rounded_weights(tiny_weights[name], "float32")
    agree = 0
    for i, (p, got) in enumerate(zip(prompts, outs)):
        want = plain_generate(cfg, w, p, 24, stop_token_ids=[], chain=PlainChain(seed=sequence_seed(77, i), **knobs))
        agree += int(got == want)
        assert len(got) == 24
        if got != want:  # only a draw within rounding of a boundary may part the streams
            def make(rng_of, seed=sequence_seed(77, i)):
                chain = PlainChain(seed=seed, **knobs)
                chain.rng = rng_of(seed)
                return chain.sample

            assert parted_within_rounding(cfg, w, p, got, want, make), f"sequence {i}: {got} left {want} at a clear margin"
    assert agree >= 2
    # mirostat keeps its surprise ceiling per sequence on the device, from the first draw of a call on
    miro = dict(temperature=0.9, mirostat=2, mirostat_ent=3.0, mirostat_lr=0.2)
    outs = llm.generate(prompts, max_new_tokens=24, seed=5, stop_token_ids=[], **miro)
    assert outs == llm.generate(prompts, max_new_tokens=24, seed=5, stop_token_ids=[], **miro)
    agree = 0
    for i, (p, got) in enumerate(zip(prompts, outs)):
        want = plain_generate(cfg, w, p, 24, stop_token_ids=[], chain=PlainChain(seed=sequence_seed(5, i), **miro))
        agree += int(got == want)
        if got != want:
            def make(rng_of, seed=sequence_seed(5, i)):
                chain = PlainChain(seed=seed, **miro)
                chain.rng = rng_of(seed)
                return chain.sample

            assert parted_within_rounding(cfg, w, p, got, want, make), f"mirostat, sequence {i}: {got} left {want} at a clear margin"
    assert agree >= 2
    # greedy with a strong repetition penalty: no token twice within the window, and not the plain greedy's run
    greedy = llm.generate(prompts[0], max_new_tokens=20, temperature=0.0, stop_token_ids=[])
    pen = llm.generate(prompts[0], max_new_tokens=20, temperature=0.0, repeat_penalty=50.0, presence_penalty=100.0, repeat_last_n=4, stop_token_ids=[])
    want = plain_generate(cfg, w, prompts[0], 20, stop_token_ids=[], chain=PlainChain(temperature=0.0, repeat_penalty=50.0, presence_penalty=100.0, repeat_last_n=4))
    assert pen == want and pen != greedy
    assert all(pen[k] not in pen[max(0, k - 4) : k] for k in range(len(pen)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("temperature", [0.0, 0.8])
def test_launching_ahead_changes_no_token(dtype, temperature, llms):
    """Steps launched on tokens that are still on the device, against the loop that reads every token
    first: the same tokens and finish reasons, for sequences that end on stop tokens at different
    times, on their budgets and together; slots and pages all come back."""
    name = "B"
    cfg = TINY[name][0]
    llm = llms(name, dtype)
    rng = np.random.default_rng(5)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (3, 11, 20, 34)]
    kw = dict(temperature=temperature, top_p=0.9, seed=99, return_results=True)
    free = llm.engine.cache.pages_free()
    plain = llm.generate(prompts, max_new_tokens=[12, 20, 7, 20], stop_token_ids=[], launch_ahead=False, **kw)
    # stop tokens taken from what the sequences really produce, so that they end at different steps
    stops = [plain[0].tokens[5], plain[1].tokens[9], plain[3].tokens[14]]
    for stop_ids in ([], stops):
        a = llm.generate(prompts, max_new_tokens=[12, 20, 7, 20], stop_token_ids=stop_ids, launch_ahead=False, **kw)
        steps_plain = llm.last_stats.decode_steps
        b = llm.generate(prompts, max_new_tokens=[12, 20, 7, 20], stop_token_ids=stop_ids, launch_ahead=True, **kw)
        assert [(r.tokens, r.finish_reason) for r in a] == [(r.tokens, r.finish_reason) for r in b]
        assert llm.last_stats.decode_steps >= steps_plain
        assert llm.engine.cache.n_open == 0 and llm.engine.cache.pages_free() == free
        llm.engine.cache.check_consistent()
    assert any(r.finish_reason == "stop_token" for r in b)


def test_command_line_generates_what_the_entry_point_generates(tmp_path, capsys, tiny_weights):
    """bin/rusty_llama's main on a model folder: `-n` counts positions, prompt included; ids on standard
    output, one line per prompt; the rate on standard error."""
    import rusty_llama_b200 as rl
    from rusty_llama_b200.cli import main

    cfg = TINY["A"][0]
    model_dir = rl.write_random_model(str(tmp_path / "m"), cfg, seed=3)
    prompts = tmp_path / "p.txt"
    prompts.write_text("5 17 3 9\n7, 7\n")
    assert main([model_dir, "-t", "0", "-n", "12", "-i", "@" + str(prompts), "--dtype", "float32", "--max-tokens", "256"]) == 0
    out, err = capsys.readouterr()
    lines = [[int(t) for t in ln.split()] for ln in out.splitlines()]
    assert len(lines) == 2 and len(lines[0]) <= 8 and len(lines[1]) <= 10  # 12 positions each, 4 and 2 of them the prompt
    assert "tokens" in err and "tok/s" in err
    llm = rl.load(model_dir, dtype="float32", max_tokens=256)
    assert llm.generate([[5, 17, 3, 9], [7, 7]], steps=12, temperature=0.0) == lines
    # without the model's stop tokens the count is exact
    assert [len(o) for o in llm.generate([[5, 17, 3, 9], [7, 7]], steps=12, temperature=0.0, stop_token_ids=[])] == [8, 10]
    # sampled, with a seed: the same call twice gives the same ids
    assert main([model_dir, "-t", "0.9", "-p", "0.8", "-s", "5", "-n", "9", "-i", "1 2 3", "--max-tokens", "256"]) == 0
    first = capsys.readouterr().out
    assert main([model_dir, "-t", "0.9", "-p", "0.8", "-s", "5", "-n", "9", "-i", "1 2 3", "--max-tokens", "256"]) == 0
    assert capsys.readouterr().out == first and len(first.split()) <= 6


def test_one_layer_at_the_sizes_of_the_benchmark(tmp_path):
    """The benchmark's layer sizes (width 4096, 32 / 8 heads of 128, feed-forward 14336, llama3 rope
    scaling) with one layer and a smaller vocabulary, in bfloat16: prompts of unequal lengths in one
    step, then tokens one by one, with and without graphs, as a batch of 2 (the streaming products, key
    splits with a merge kernel) and as a batch of 12 (the tcgen05 product with narrowed tiles and with
    split k, attention that writes its result itself).  This is where the kernels that only these
    sizes select are checked inside a model."""
    import bench
    import rusty_llama_b200 as rl
    from conftest import read_weights

    cfg = dict(bench.load_config())
    cfg.update(num_hidden_layers=1, vocab_size=8200, max_position_embeddings=1024)
    model_dir = rl.write_random_model(str(tmp_path / "big"), cfg, seed=21, std=0.03, norm_jitter=0.1)
    w = read_weights(model_dir)
    rng = np.random.default_rng(4)
    reqs = {"a": rng.integers(0, 8200, 580).tolist(), "b": rng.integers(0, 8200, 71).tolist()}  # a: long enough for four key splits
    for i in range(10):
        reqs[f"s{i}"] = rng.integers(0, 8200, 12 + 3 * i).tolist()
    refs = plain_all_logits(cfg, w, "bfloat16", reqs)
    n_decode = 6
    for graphs in (True, False):
        for names in (["a", "b"], list(reqs)):
            llm = rl.load(model_dir, dtype="bfloat16", max_tokens=64 * 24, max_seqs=len(names), use_graphs=graphs)
            slots = {n: llm.open_sequence() for n in names}
            cut = {n: len(reqs[n]) - n_decode for n in names}
            out = llm.step([rl.StepEntry(slots[n], reqs[n][: cut[n]], [0, cut[n] - 1]) for n in names]).cpu().numpy()
            for i, n in enumerate(names):
                check_logits(out[2 * i : 2 * i + 2], refs[n][[0, cut[n] - 1]], "bfloat16", f"prompt {n}")
            for t in range(n_decode):
                out = llm.step([rl.StepEntry(slots[n], [reqs[n][cut[n] + t]], [0]) for n in names]).cpu().numpy()
                for i, n in enumerate(names):
                    check_logits(out[i : i + 1], refs[n][[cut[n] + t]], "bfloat16", f"decode {n} {t} (graphs={graphs}, batch {len(names)})")
            for n in names:
                llm.close_sequence(slots[n])
            llm.engine.check_device_status()
            del llm
            torch.cuda.empty_cache()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_across_graph_buckets_and_kept_logits(dtype, tmp_path, tiny_weights):
    """Decode graphs are captured per (batch size, page-table width 4, 8, 16, 32, ...).  One sequence and a
    batch of three, whose members stand on different pages, decode from below position 256 to above 1024
    (tiny B with room for 1100 positions): every new width means a plain run, a capture and then replays,
    and the number of key splits changes with it.  Every step's logits are kept on the device and read only
    at the end, so a result that a later step overwrote would show; all are compared with the plain model,
    and in 32-bit the runs with and without graphs must agree in every bit."""
    import rusty_llama_b200 as rl
    from conftest import read_weights
    from rusty_llama_b200 import StepEntry

    cfg = dict(TINY["B"][0], max_position_embeddings=1100)
    model_dir = rl.write_random_model(str(tmp_path / "long_b"), cfg, seed=1, norm_jitter=0.1)
    w = read_weights(model_dir)
    rng = np.random.default_rng(12)
    seqs = {"solo": rng.integers(0, cfg["vocab_size"], 1100).tolist(), "x": rng.integers(0, cfg["vocab_size"], 1050).tolist(),
            "y": rng.integers(0, cfg["vocab_size"], 930).tolist(), "z": rng.integers(0, cfg["vocab_size"], 860).tolist()}
    prompt = {"solo": 200, "x": 250, "y": 130, "z": 60}
    ref = plain_all_logits(cfg, w, dtype, seqs)
    kept = {}
    for graphs in (True, False):
        llm = rl.load(model_dir, dtype=dtype, max_tokens=64 * 48, max_seqs=3, use_graphs=graphs)
        got = {n: [] for n in seqs}
        for batch in (["solo"], ["x", "y", "z"]):
            slots = {n: llm.open_sequence() for n in batch}
            out = llm.step([StepEntry(slots[n], seqs[n][: prompt[n]], [prompt[n] - 1]) for n in batch])
            for i, n in enumerate(batch):
                got[n].append(out[i : i + 1])
            pos = {n: prompt[n] for n in batch}
            while True:
                live = [n for n in batch if pos[n] < len(seqs[n])]
                if not live:
                    break
                out = llm.step([StepEntry(slots[n], [seqs[n][pos[n]]], [0]) for n in live])  # stays on the device
                for i, n in enumerate(live):
                    got[n].append(out[i : i + 1])
                    pos[n] += 1
                    if pos[n] == len(seqs[n]):
                        llm.close_sequence(slots[n])
        llm.engine.check_device_status()
        if graphs:
            widths = sorted({k[1] for k in llm.engine._graphs})
            assert widths == [4, 8, 16, 32], widths
        kept[graphs] = {n: torch.cat(got[n]).cpu() for n in seqs}
        for n in seqs:
            check_logits(kept[graphs][n].numpy(), ref[n][prompt[n] - 1 :], dtype, f"{n}, graphs={graphs}")
    if dtype == "float32":
        for n in seqs:
            assert torch.equal(kept[True][n], kept[False][n]), f"{n}: graphs change bits"


def test_borrowed_logits_are_the_graphs_buffer_and_owned_ones_are_not(llms):
    """`step` hands out logits that are the caller's to keep; `borrow=True` (what the generation loop uses) hands
    out the replayed graph's own buffer, which the next step of the same shape overwrites."""
    from rusty_llama_b200 import StepEntry

    llm = llms("A", "bfloat16")
    s = llm.open_sequence()
    llm.step([StepEntry(s, [1, 2, 3], [])])
    for t in (4, 5, 6):  # plain run, capture, replay
        llm.step([StepEntry(s, [t], [0])])
    own = llm.step([StepEntry(s, [7], [0])])
    own_then = own.clone()
    lent = llm.step([StepEntry(s, [8], [0])], borrow=True)
    lent_then = lent.clone()
    after = llm.step([StepEntry(s, [9], [0])], borrow=True)
    llm.close_sequence(s)
    assert torch.equal(own, own_then)
    assert lent.data_ptr() == after.data_ptr() and torch.equal(lent, after) and not torch.equal(lent, lent_then)


def test_sequence_records_on_the_device_follow_every_kind_of_step(llms):
    """Each slot has a record on the device (positions held, tokens decoded, budget, open).  A decode step that is
    replayed as a graph takes its positions from there, so once the slots and their page tables are on the device
    a step launched on device tokens uploads nothing; the records must agree with the host's bookkeeping after
    prompt steps, chunks, plain and replayed decode steps, and a slot that is opened again starts from zero."""
    from rusty_llama_b200 import StepEntry

    for graphs in (True, False):
        llm = llms("B", "bfloat16", use_graphs=graphs, max_tokens=64 * 8, max_seqs=2)
        eng = llm.engine
        a, b = llm.open_sequence(), llm.open_sequence()
        eng.note_budget(a, 77)
        llm.step([StepEntry(a, [1, 2, 3, 4, 5], []), StepEntry(b, [9] * 70, [])])
        assert eng.sequence_record(a) == {"len": 5, "decoded": 0, "max_new": 77, "open": True}
        assert eng.sequence_record(b)["len"] == 70
        llm.step([StepEntry(a, [6, 7], [])])  # a chunk
        for t in range(4):
            llm.step([StepEntry(a, [10 + t], [0]), StepEntry(b, [20 + t], [0])])
        ra, rb = eng.sequence_record(a), eng.sequence_record(b)
        assert (ra["len"], rb["len"]) == (11, 74) == (eng.cache.length(a), eng.cache.length(b))
        assert ra["decoded"] == rb["decoded"] == (4 if graphs else 0)  # (the plain path's positions come from the host)
        if graphs:
            # steps on tokens that lie on the device: nothing is uploaded while the members and their pages stay
            toks = torch.tensor([3, 4], dtype=torch.int32, device="cuda:0")
            eng.step_device_tokens([a, b], toks)  # (the first one sends the slots and tables of this batch)
            before = eng.uploads
            for _ in range(20):
                eng.step_device_tokens([a, b], toks)
            assert eng.uploads == before, "a replayed step on device tokens uploaded its integers"
            assert eng.sequence_record(a)["len"] == 11 + 21 == eng.cache.length(a)
            for _ in range(40):  # ... until a sequence crosses into a new page (b: 74 + 21 + 40 = 135 > 128)
                eng.step_device_tokens([a, b], toks)
            assert eng.uploads > before
            assert eng.sequence_record(b)["len"] == eng.cache.length(b) == 135
        llm.close_sequence(a)
        assert eng.sequence_record(a)["open"] is False
        a2 = llm.open_sequence()
        assert a2 == a and eng.sequence_record(a2) == {"len": 0, "decoded": 0, "max_new": 0, "open": True}
        llm.close_sequence(a2)
        llm.close_sequence(b)
