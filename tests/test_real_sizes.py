"""The benchmark's layer sizes inside a model, compared and not only timed: Llama-3.1-8B widths (4096, 32
query heads over 8 kv heads of 128, feed-forward 14336, llama3 rope scaling) and its whole vocabulary of
128256, with 2 of its 32 layers, random weights.

32-bit runs: every request whole, with its last 32 tokens one by one, and in batches of unequal lengths
whose members leave at different times and whose slots are used again: the same bits on all three
schedules (the reference's own guarantee for its 32-bit path, tests/prefill.rs:25-65 and
tests/integration.rs:236-286), within 1e-4 of the range of the plain float64 logits, the same argmax.
bfloat16 runs: the same three schedules within the tolerance of the tiny models, and a decode step of 64
sequences (graphs on and off), where the tcgen05 product with few rows, the fused attention kernel and
the projection as partial sums meet.
"""

import numpy as np
import pytest
import torch

from helpers import check_logits
from plain_llama import plain_hidden, plain_rmsnorm

pytestmark = pytest.mark.gpu

LAYERS = 2
VOCAB = 128256
LENGTHS = {"a": 5, "b": 33, "c": 70, "d": 96}


def config():
    import bench

    cfg = dict(bench.load_config("8b"))
    assert cfg["vocab_size"] == VOCAB and cfg["hidden_size"] == 4096
    cfg.update(num_hidden_layers=LAYERS, max_position_embeddings=256)
    return cfg


@pytest.fixture(scope="module")
def world():
    """Weights made once on the device from the library's seeded generator and handed both to the engine
    (by name, like a checkpoint) and, copied to the host, to the plain implementation; the requests; the
    plain float64 logits of every request at the rows that are compared."""
    from rusty_llama_b200.registry import describe_model
    from rusty_llama_b200.weights.random_init import _param_infos, random_tensors

    cfg = config()
    infos = _param_infos(cfg)
    weights = dict(random_tensors(infos, seed=17, dtype=torch.bfloat16, std=0.03, norm_jitter=0.1, device="cuda:0"))
    host = {k: v.cpu().float() for k, v in weights.items()}
    rng = np.random.default_rng(2)
    requests = {rid: rng.integers(0, VOCAB, n).tolist() for rid, n in LENGTHS.items()}
    # rows compared with the plain model: every row of the short requests; of the long ones the first
    # three, every seventh, and the last 34 (what the one-by-one schedule decodes, and a little before it)
    rows = {}
    for rid, n in LENGTHS.items():
        keep = set(range(min(n, 3))) | set(range(0, n, 7)) | set(range(max(0, n - 34), n))
        rows[rid] = sorted(keep)
    ref = {}
    head = host["lm_head.weight"].double()
    for rid, toks in requests.items():
        x = plain_hidden(cfg, host, toks, torch.float64)[rows[rid]]
        xn = plain_rmsnorm(x, host["model.norm.weight"], cfg["rms_norm_eps"])
        ref[rid] = (xn @ head.T).numpy()
    del head
    return {"cfg": cfg, "weights": weights, "requests": requests, "rows": rows, "ref": ref, "spec": describe_model(cfg)}


def make_llm(world, dtype, **kw):
    import rusty_llama_b200 as rl
    from rusty_llama_b200.models.model import Model
    from rusty_llama_b200.parts.base import Runtime
    from rusty_llama_b200.weights.loader import load_tensors

    model = Model(world["spec"], Runtime.create("cuda:0", dtype))
    load_tensors(model, world["weights"])
    return rl.LLM(model, **kw)


def three_schedules(llm, requests):
    """request -> [logits of every position] for: whole; last 32 one by one; batches of two with leavers,
    the second batch in the slots of the first."""
    from rusty_llama_b200 import StepEntry

    whole, single, batched = {}, {}, {}
    for rid, toks in requests.items():
        s = llm.open_sequence()
        whole[rid] = llm.step([StepEntry(s, toks, list(range(len(toks))))]).cpu()
        llm.close_sequence(s)
    for rid, toks in requests.items():
        n = len(toks)
        head = max(n - 32, 0)
        s = llm.open_sequence()
        parts = []
        if head:
            parts.append(llm.step([StepEntry(s, toks[:head], list(range(head)))]).cpu())
        for t in range(head, n):
            parts.append(llm.step([StepEntry(s, [toks[t]], [0])]).cpu())
        llm.close_sequence(s)
        single[rid] = torch.cat(parts)
    ids = list(requests)
    for batch in (ids[:2], ids[2:]):
        slots = {rid: llm.open_sequence() for rid in batch}
        heads = {rid: max(1, len(requests[rid]) - 6 - 5 * i) for i, rid in enumerate(batch)}
        got = {rid: [] for rid in batch}
        out = llm.step([StepEntry(slots[rid], requests[rid][: heads[rid]], list(range(heads[rid]))) for rid in batch]).cpu()
        at = 0
        for rid in batch:
            got[rid].append(out[at : at + heads[rid]])
            at += heads[rid]
        pos = dict(heads)
        while True:
            live = [rid for rid in batch if pos[rid] < len(requests[rid])]
            if not live:
                break
            out = llm.step([StepEntry(slots[rid], [requests[rid][pos[rid]]], [0]) for rid in live]).cpu()
            for i, rid in enumerate(live):
                got[rid].append(out[i : i + 1])
                pos[rid] += 1
                if pos[rid] == len(requests[rid]):
                    llm.close_sequence(slots[rid])
        for rid in batch:
            batched[rid] = torch.cat(got[rid])
    llm.engine.check_device_status()
    llm.engine.cache.check_consistent()
    assert llm.engine.cache.n_open == 0
    return whole, single, batched


def test_float32_at_benchmark_sizes_2_of_32_layers_three_schedules(world):
    llm = make_llm(world, "float32", max_tokens=64 * 4, max_seqs=2)
    whole, single, batched = three_schedules(llm, world["requests"])
    for rid in world["requests"]:
        assert torch.equal(whole[rid], single[rid]), f"request {rid}: one by one differs from whole in its bits"
        assert torch.equal(whole[rid], batched[rid]), f"request {rid}: in a batch differs from whole in its bits"
        got = whole[rid][world["rows"][rid]].double().numpy()
        ref = world["ref"][rid]
        scale = float(np.abs(ref).max())
        err = float(np.abs(got - ref).max())
        assert err <= 1e-4 * scale, f"request {rid}: max error {err:.3e} at range {scale:.3e}"
        # the same argmax wherever the plain model's best two logits are further apart than the error bound
        top2 = np.sort(ref, axis=1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 2e-4 * scale
        assert clear.sum() >= len(clear) // 2
        assert np.array_equal(got.argmax(axis=1)[clear], ref.argmax(axis=1)[clear])


def test_bfloat16_at_benchmark_sizes_2_of_32_layers_three_schedules(world):
    llm = make_llm(world, "bfloat16", max_tokens=64 * 4, max_seqs=2)
    for name, got in zip(("whole", "last 32 one by one", "in batches"), three_schedules(llm, world["requests"])):
        for rid in world["requests"]:
            check_logits(got[rid][world["rows"][rid]].numpy(), world["ref"][rid], "bfloat16", f"request {rid} {name}")


@pytest.mark.parametrize("graphs", [True, False])
def test_bfloat16_decode_step_of_64_sequences_2_of_32_layers(world, graphs):
    """64 sequences, each a prefix of one of the four requests cut at a row whose plain logits are known, take
    one more token together, then another: every row of both steps must be the plain model's row."""
    from rusty_llama_b200 import StepEntry

    requests, rows, ref = world["requests"], world["rows"], world["ref"]
    llm = make_llm(world, "bfloat16", max_tokens=64 * 2 * 64, max_seqs=64, use_graphs=graphs)
    # (request, position p): the sequence holds tokens [0, p), then decodes tokens p and p + 1;
    # rows p and p + 1 must both be among the compared rows, which the last 34 of each request are
    cuts = []
    for rid in ("b", "c", "d"):
        n = len(requests[rid])
        cuts += [(rid, p) for p in range(max(1, n - 34), n - 1)]
    cuts = [cuts[i] for i in np.linspace(0, len(cuts) - 1, 61).astype(int)] + [("a", p) for p in (1, 2, 3)]
    assert len(cuts) == 64 and len(set(cuts)) == 64
    slots = [llm.open_sequence() for _ in cuts]
    llm.step([StepEntry(s, requests[rid][:p], []) for s, (rid, p) in zip(slots, cuts)])
    for k in range(2):
        out = llm.step([StepEntry(s, [requests[rid][p + k]], [0]) for s, (rid, p) in zip(slots, cuts)]).cpu().numpy()
        want = np.stack([ref[rid][rows[rid].index(p + k)] for rid, p in cuts])
        check_logits(out, want, "bfloat16", f"decode step {k} of 64 sequences, graphs={graphs}")
    for s in slots:
        llm.close_sequence(s)
    llm.engine.check_device_status()


# --------------------------------------------------------------------------- kernels at the sizes only these models reach
@pytest.mark.parametrize("M", [1, 8])
def test_gemv_stream_classifier_of_128256_rows(M):
    from rusty_llama_b200.kernels import ops
    from test_kernels import bf16_round, close_dot_f32

    g = torch.Generator().manual_seed(M)
    x = bf16_round(torch.randn(M, 4096, generator=g))
    w = bf16_round(torch.randn(VOCAB, 4096, generator=g) * 0.05)
    out = ops.gemv_stream(x.to(torch.bfloat16).cuda(), w.to(torch.bfloat16).cuda(), torch.float32)
    torch.cuda.synchronize()
    ops.tc_status_check()
    close_dot_f32(out, x, w)


def test_gemm_tc_classifier_of_128256_rows_for_64_tokens():
    from rusty_llama_b200.kernels import ops
    from test_kernels import bf16_round, close_dot_f32

    g = torch.Generator().manual_seed(64)
    x = bf16_round(torch.randn(64, 4096, generator=g))
    w = bf16_round(torch.randn(VOCAB, 4096, generator=g) * 0.05)
    out = ops.gemm_tc(x.to(torch.bfloat16).cuda(), w.to(torch.bfloat16).cuda(), torch.float32)
    torch.cuda.synchronize()
    ops.tc_status_check()
    close_dot_f32(out, x, w)
