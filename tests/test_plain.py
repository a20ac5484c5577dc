"""The plain implementation against the numbers the reference's own unit tests pin down (no GPU)."""

import math

import numpy as np
import torch

from plain_llama import (
    PlainRng, plain_argmax, plain_attention, plain_generate, plain_logits, plain_rmsnorm, plain_rope,
    plain_sample, plain_silu,
)

from conftest import TINY


def test_silu_known_value():
    # src/backend/cpu.rs:781-787: silu(1) * 2
    assert abs(float(plain_silu(torch.tensor(1.0))) - 0.7310586) < 1e-6


def test_rmsnorm_of_ones():
    # src/backend/cpu.rs:750-759: 1/sqrt(1 + 1e-5); and eps matters (:762)
    y = plain_rmsnorm(torch.ones(4), torch.ones(4), 1e-5)
    assert torch.allclose(y, torch.full((4,), 1.0 / math.sqrt(1.0 + 1e-5)), atol=1e-7)
    z = plain_rmsnorm(torch.zeros(4), torch.ones(4), 1e-5)
    assert torch.isfinite(z).all() and (z == 0).all()


def test_rope_position_zero_is_identity_and_angle():
    # src/backend/cpu.rs:797-835
    v = torch.randn(1, 2, 8)
    inv = torch.tensor([1.0, 0.1, 0.01, 0.001])
    for inter in (True, False):
        assert torch.equal(plain_rope(v, torch.tensor([0]), inv, inter), v)
    x = torch.zeros(1, 1, 8)
    x[0, 0, 0] = 1.0
    y = plain_rope(x, torch.tensor([3]), inv, interleaved=True)
    assert abs(float(y[0, 0, 0]) - math.cos(3.0)) < 1e-6 and abs(float(y[0, 0, 1]) - math.sin(3.0)) < 1e-6
    y = plain_rope(x, torch.tensor([3]), inv, interleaved=False)
    assert abs(float(y[0, 0, 0]) - math.cos(3.0)) < 1e-6 and abs(float(y[0, 0, 4]) - math.sin(3.0)) < 1e-6


def test_rope_pairings_agree_after_row_permutation():
    # a half-split head equals an interleaved head whose dims were permuted (src/model.rs:1953-1963)
    hd = 8
    v = torch.randn(5, 3, hd)
    inv = torch.tensor([1.0, 0.1, 0.01, 0.001])
    pos = torch.arange(5)
    perm = torch.tensor([j // 2 + (hd // 2) * (j % 2) for j in range(hd)])  # interleaved index -> half-split index
    a = plain_rope(v, pos, inv, interleaved=False)
    b = plain_rope(v[..., perm], pos, inv, interleaved=True)
    assert torch.allclose(a[..., perm], b, atol=1e-6)


def test_attention_single_key_and_uniform_scores():
    # src/backend/cpu.rs:930-1019: one key -> its value; equal scores -> mean of the values
    q = torch.randn(1, 2, 4)
    k = torch.randn(1, 1, 4)
    v = torch.randn(1, 1, 4)
    out = plain_attention(q, k, v)
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 1], v[0, 0])
    T = 5
    q = torch.zeros(T, 1, 4)
    k = torch.randn(T, 1, 4)
    v = torch.randn(T, 1, 4)
    out = plain_attention(q, k, v)
    for r in range(T):
        assert torch.allclose(out[r, 0], v[: r + 1, 0].mean(dim=0), atol=1e-6)
    out_w = plain_attention(q, k, v, window=2)
    assert torch.allclose(out_w[4, 0], v[3:5, 0].mean(dim=0), atol=1e-6)


def test_argmax_last_of_ties_and_nan():
    # src/sampler.rs:976-988
    assert plain_argmax([0.1, 0.2, 5.0, 0.3]) == 2
    assert plain_argmax([1.0, 1.0, 1.0]) == 2
    assert plain_argmax([float("nan"), 0.0, 5.0]) == 2


def test_sampler_golden_stream():
    # src/sampler.rs:1009-1014
    logits = [2.0, 1.8, 1.6, 1.4, 1.2, 1.0, 0.8, 0.6]
    rng = PlainRng(12345)
    assert [plain_sample(logits, 1.0, 0.9, rng) for _ in range(8)] == [2, 4, 0, 4, 0, 0, 6, 2]


def test_top_p_edge_cases():
    # src/sampler.rs:1025-1060
    rng = PlainRng(1)
    assert plain_sample([0.0, 0.0, 10.0, 0.0], 1.0, 0.9, rng) == 2
    assert plain_sample([1.0, 1.0, 1.0, 1.0], 1.0, 0.1, rng) == 3  # empty nucleus -> argmax, last of ties
    assert plain_sample([42.0], 1.0, 0.9, rng) == 0 and plain_sample([42.0], 0.0, 0.9, rng) == 0
    a = [plain_sample([1.0, 2.0, 3.0, 4.0], 1.0, 0.0, PlainRng(12345)) for _ in range(2)]
    assert a[0] == a[1]


def test_float32_tracks_float64(tiny_weights):
    """float32 is a faithful stand-in for exact arithmetic at these sizes, which bounds what any
    32-bit engine can be asked to match."""
    for name, (cfg, _, _) in TINY.items():
        w = {k: v.to(torch.float32) for k, v in tiny_weights[name].items()}
        toks = list(np.random.default_rng(7).integers(0, cfg["vocab_size"], 40))
        l32 = plain_logits(cfg, w, toks, torch.float32)
        l64 = plain_logits(cfg, w, toks, torch.float64)
        assert float((l32.double() - l64).abs().max()) < 2e-5 * float(l64.abs().max()) + 1e-6


def test_whole_equals_prefix(tiny_weights):
    """Causality: logits at position t do not change when later tokens are appended."""
    cfg, _, _ = TINY["A"]
    w = {k: v.to(torch.float32) for k, v in tiny_weights["A"].items()}
    toks = [5, 17, 3, 99, 200, 41, 7]
    full = plain_logits(cfg, w, toks)
    part = plain_logits(cfg, w, toks[:4])
    assert torch.allclose(full[:4], part, atol=1e-6)


def test_greedy_generation_is_reproducible(tiny_weights):
    cfg, _, _ = TINY["A"]
    w = {k: v.to(torch.float32) for k, v in tiny_weights["A"].items()}
    a = plain_generate(cfg, w, [1, 2, 3], 6)
    assert a == plain_generate(cfg, w, [1, 2, 3], 6) and len(a) == 6


def test_longer_chain_stages_on_the_reference_cases():
    """The stages of the longer chain on the inputs and outcomes of the reference's own unit tests
    (src/sampler.rs:1064-1211)."""
    from plain_llama import PlainChain

    # top_k_keeps_k_highest: of [3, 1, 4, 1, 5] with k = 2 only ids 2 and 4 can be drawn
    c = PlainChain(temperature=1.0, top_p=0.0, seed=3, top_k=2)
    assert {c.sample([3.0, 1.0, 4.0, 1.0, 5.0]) for _ in range(40)} == {2, 4}
    # min_p_drops_low_probability_tail: 10 + ln 0.5 = 9.31, only id 0 clears it
    c = PlainChain(temperature=1.0, top_p=0.0, seed=3, min_p=0.5)
    assert {c.sample([10.0, 9.0, 2.0, 1.0]) for _ in range(20)} == {0}
    # penalty_demotes_repeated_token: id 2 (5.0) falls below id 0 (4.5) once it was chosen before
    c = PlainChain(temperature=0.0, repeat_penalty=1.3)
    c.ring = [2]
    assert c.sample([4.5, 1.0, 5.0]) == 0
    # penalty_ring_evicts_past_window: a window of 2 after 0, 1, 2: token 0 is no longer penalised
    c = PlainChain(temperature=0.0, presence_penalty=5.0, repeat_last_n=2)
    for tok in (0, 1, 2):
        c._accept(tok)
    assert c.ring == [1, 2] and c.sample([0.0, 0.0, 0.0]) == 0
    # penalty_frequency_scales_with_count: seen twice costs more than seen once
    c = PlainChain(temperature=0.0, frequency_penalty=1.0)
    c.ring = [0, 0, 1]
    assert c.sample([0.0, 0.0, -1.5]) == 1  # -2 (seen twice), -1 (seen once), -1.5
    c.ring = [0, 0, 1]
    assert c.sample([0.0, 0.0, -0.5]) == 2  # -2, -1, -0.5
    # mirostat_v2_truncates_and_updates_mu: only token 0 survives, p = 1, mu = 10 - 0.1 * (0 - 5)
    c = PlainChain(temperature=1.0, seed=1, mirostat=2, mirostat_ent=5.0, mirostat_lr=0.1)
    assert float(c.mu) == 10.0 and c.sample([10.0, 0.0, 0.0]) == 0 and abs(float(c.mu) - 10.5) < 1e-4
    # xtc_drops_leading_above_threshold_run: p = 0.73, 0.27, ...: id 0 goes, id 1 is then the largest
    c = PlainChain(temperature=0.0, seed=7, xtc_probability=1.0, xtc_threshold=0.2)
    assert c.sample([10.0, 9.0, 0.0, -1.0]) == 1
    # xtc_always_keeps_at_least_one_token: threshold 0 leaves the least probable alone
    c = PlainChain(temperature=1.0, top_p=0.0, seed=3, xtc_probability=1.0, xtc_threshold=0.0)
    assert c.sample([1.0, 2.0, 3.0, 4.0, 5.0]) == 0
    # xtc_zero_probability_is_noop (and draws nothing from its generator)
    c = PlainChain(temperature=0.0, top_k=4, xtc_probability=0.0)
    assert c.sample([10.0, 9.0, 0.0, -1.0]) == 0 and c.xtc_rng.state == c.rng.state
    # DRY (src/sampler.rs:1231-1262): no repeat, no penalty; after A, B, A the token B loses the bare multiplier
    dry = dict(temperature=0.0, repeat_last_n=0, dry_multiplier=1.0, dry_base=2.0, dry_allowed_length=2)
    c = PlainChain(**dry)
    c.dry_ring = [1, 2, 3, 4, 5]
    assert c.sample([0.0, 0.3, 0.0, 0.0, 0.0, 0.0]) == 1
    c = PlainChain(**dry)
    c.dry_ring = [1, 2, 1]
    assert c.sample([0.0, 0.0, 0.5]) == 1 and c.sample([0.0, 0.0, 1.5]) == 2
    assert PlainChain._z_array([1, 2, 1, 2]) == [4, 0, 2, 0] and PlainChain._z_array([1, 2, 3, 4]) == [4, 0, 0, 0]
    c = PlainChain(dry_sequence_breakers=(3,), **dry)
    c.dry_ring = [1, 2, 3, 1]
    assert c.sample([0.0, 0.0, 0.5, 0.0]) == 2  # the breaker keeps "1, 2" out of reach
