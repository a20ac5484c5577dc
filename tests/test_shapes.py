"""Every size that a configuration allows: head sizes in steps of 16 up to 256, head counts and groups
that are no power of two, one kv head for all, widths, feed-forward sizes and vocabularies that are odd
or no multiple of 8 (which the 16-byte-row kernels refuse, so a plain kernel has to take over).  Each
shape runs prompts of unequal lengths in one step and then tokens one by one, in 32-bit and in bfloat16,
against the plain implementation."""

import numpy as np
import pytest
import torch

from conftest import read_weights
from helpers import check_logits, plain_all_logits

pytestmark = pytest.mark.gpu

# head size, heads, kv heads, width, feed-forward, vocabulary, layers
SHAPES = [
    (16, 7, 7, 112, 48, 129, 3),
    (32, 5, 5, 96, 200, 300, 2),
    (32, 4, 2, 129, 255, 257, 1),
    (48, 6, 2, 100, 250, 1001, 2),
    (64, 8, 1, 512, 1088, 777, 1),
    (64, 3, 1, 66, 90, 131, 2),
    (80, 3, 3, 120, 136, 515, 2),
    (96, 4, 2, 192, 520, 2000, 1),
    (112, 2, 1, 72, 96, 260, 2),
    (128, 9, 3, 576, 600, 900, 2),
    (128, 16, 1, 256, 320, 333, 1),
    (128, 3, 3, 200, 176, 4099, 1),
    (128, 2, 1, 100, 172, 515, 2),
    (160, 2, 1, 64, 128, 256, 1),
    (192, 2, 2, 128, 256, 256, 1),
    (256, 2, 1, 128, 192, 384, 1),
]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "hd{}_h{}k{}_d{}_ff{}_v{}".format(*s[:6]))
def test_shape_runs_and_agrees_with_the_plain_model(shape, tmp_path):
    import rusty_llama_b200 as rl

    hd, H, K, d, ff, V, L = shape
    seed = SHAPES.index(shape)
    cfg = {
        "architectures": ["LlamaForCausalLM"], "hidden_size": d, "intermediate_size": ff, "num_hidden_layers": L,
        "num_attention_heads": H, "num_key_value_heads": K, "head_dim": hd, "vocab_size": V,
        "max_position_embeddings": 512, "rms_norm_eps": 3e-6, "rope_theta": 25000.0, "rope_scaling": None,
        "tie_word_embeddings": bool(seed % 2), "torch_dtype": "bfloat16", "eos_token_id": 1,
    }
    model_dir = rl.write_random_model(str(tmp_path / "m"), cfg, seed=seed, norm_jitter=0.1)
    w = read_weights(model_dir)
    rng = np.random.default_rng(seed)
    reqs = {"a": rng.integers(0, V, 150).tolist(), "b": rng.integers(0, V, 67).tolist(), "c": rng.integers(0, V, 12).tolist()}
    n_decode = 8
    for dtype in ("float32", "bfloat16"):
        refs = plain_all_logits(cfg, w, dtype, reqs)
        llm = rl.load(model_dir, dtype=dtype, max_tokens=64 * 8, max_seqs=3)
        slots = {n: llm.open_sequence() for n in reqs}
        cut = {n: len(reqs[n]) - n_decode for n in reqs}
        out = llm.step([rl.StepEntry(slots[n], reqs[n][: cut[n]], list(range(cut[n]))) for n in reqs]).cpu().numpy()
        at = 0
        for n in reqs:
            check_logits(out[at : at + cut[n]], refs[n][: cut[n]], dtype, f"{shape}: prompt {n}")
            at += cut[n]
        for t in range(n_decode):
            out = llm.step([rl.StepEntry(slots[n], [reqs[n][cut[n] + t]], [0]) for n in reqs]).cpu().numpy()
            for i, n in enumerate(reqs):
                check_logits(out[i : i + 1], refs[n][[cut[n] + t]], dtype, f"{shape}: decode {n} {t}")
        for n in reqs:
            llm.close_sequence(slots[n])
        llm.engine.check_device_status()
        del llm
    torch.cuda.empty_cache()


# head size, heads, kv heads, width, feed-forward, vocabulary, layers: head sizes that are even but no multiple of 8
SHAPES_32_BIT_ONLY = [(12, 3, 1, 36, 40, 50, 2), (20, 4, 2, 80, 72, 90, 1), (6, 2, 2, 12, 20, 33, 1), (250, 1, 1, 250, 64, 40, 1)]


@pytest.mark.parametrize("shape", SHAPES_32_BIT_ONLY, ids=lambda s: "hd{}_h{}k{}_d{}_ff{}_v{}".format(*s[:6]))
def test_head_sizes_that_only_a_32_bit_run_takes(shape, tmp_path):
    """The 32-bit kernels take every even head size up to 256; the bfloat16 kernels move heads in 16-byte pieces
    and say so instead of computing something else."""
    import rusty_llama_b200 as rl

    hd, H, K, d, ff, V, L = shape
    cfg = {
        "architectures": ["LlamaForCausalLM"], "hidden_size": d, "intermediate_size": ff, "num_hidden_layers": L,
        "num_attention_heads": H, "num_key_value_heads": K, "head_dim": hd, "vocab_size": V,
        "max_position_embeddings": 256, "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "rope_scaling": None,
        "tie_word_embeddings": True, "torch_dtype": "float32",
    }
    model_dir = rl.write_random_model(str(tmp_path / "m"), cfg, seed=hd, norm_jitter=0.1)
    w = read_weights(model_dir)
    rng = np.random.default_rng(hd)
    reqs = {"a": rng.integers(0, V, 80).tolist(), "b": rng.integers(0, V, 9).tolist()}
    refs = plain_all_logits(cfg, w, "float32", reqs)
    llm = rl.load(model_dir, dtype="float32", max_tokens=64 * 4, max_seqs=2)
    slots = {n: llm.open_sequence() for n in reqs}
    cut = {n: len(reqs[n]) - 4 for n in reqs}
    out = llm.step([rl.StepEntry(slots[n], reqs[n][: cut[n]], list(range(cut[n]))) for n in reqs]).cpu().numpy()
    at = 0
    for n in reqs:
        check_logits(out[at : at + cut[n]], refs[n][: cut[n]], "float32", f"{shape}: prompt {n}")
        at += cut[n]
    for t in range(4):
        out = llm.step([rl.StepEntry(slots[n], [reqs[n][cut[n] + t]], [0]) for n in reqs]).cpu().numpy()
        for i, n in enumerate(reqs):
            check_logits(out[i : i + 1], refs[n][[cut[n] + t]], "float32", f"{shape}: decode {n} {t}")
    if hd % 8:
        with pytest.raises(rl.ConfigError, match="multiple of 8"):
            rl.load(model_dir, dtype="bfloat16", max_tokens=64)
