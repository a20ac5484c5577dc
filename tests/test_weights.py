"""Safetensors reading, name/shape checks and random weights (no GPU)."""

import json
import os
import struct

import pytest
import torch

import rusty_llama_b200 as rl
from rusty_llama_b200.errors import WeightsError
from rusty_llama_b200.models.model import Model
from rusty_llama_b200.parts import Runtime
from rusty_llama_b200.weights import Checkpoint, SafetensorsFile, load_tensors, write_random_model, write_safetensors

from conftest import TINY, TINY_A, TINY_B, read_weights


def test_writer_is_read_by_the_reference_package_and_back(tmp_path):
    t = {
        "a": torch.randn(3, 5),
        "b": torch.randn(7).to(torch.bfloat16),
        "c": torch.arange(6, dtype=torch.int32).reshape(2, 3),
    }
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, t)
    from safetensors.torch import load_file, save_file

    theirs = load_file(path)
    for k in t:
        assert theirs[k].dtype == t[k].dtype and torch.equal(theirs[k], t[k])
    save_file(t, str(tmp_path / "y.safetensors"))
    f = SafetensorsFile(str(tmp_path / "y.safetensors"))
    for k in t:
        got = f.read(k)
        assert got.dtype == t[k].dtype and torch.equal(got, t[k])
    f.close()


def test_random_model_folder_has_every_tensor(tiny_dirs):
    for name, (cfg, _, _) in TINY.items():
        w = read_weights(tiny_dirs[name])
        L = cfg["num_hidden_layers"]
        expect = 2 + 9 * L + (0 if cfg["tie_word_embeddings"] else 1)
        assert len(w) == expect
        assert ("lm_head.weight" in w) == (not cfg["tie_word_embeddings"])
        dt = torch.float32 if cfg["torch_dtype"] == "float32" else torch.bfloat16
        assert all(t.dtype == dt for t in w.values())
        assert w["model.layers.0.self_attn.k_proj.weight"].shape == (cfg["num_key_value_heads"] * cfg["head_dim"], cfg["hidden_size"])
        with open(os.path.join(tiny_dirs[name], "config.json")) as f:
            assert json.load(f)["hidden_size"] == cfg["hidden_size"]
    a = read_weights(tiny_dirs["A"])
    assert (a["model.norm.weight"] == 1).all()
    b = read_weights(tiny_dirs["B"])
    assert (b["model.norm.weight"].float() != 1).any()
    assert abs(float(a["model.layers.1.mlp.up_proj.weight"].std()) - 0.02) < 0.002


def test_random_weights_depend_on_seed_and_name_only(tmp_path):
    d1 = write_random_model(str(tmp_path / "m1"), TINY_A, 3)
    d2 = write_random_model(str(tmp_path / "m2"), TINY_A, 3)
    d3 = write_random_model(str(tmp_path / "m3"), TINY_A, 4)
    w1, w2, w3 = read_weights(d1), read_weights(d2), read_weights(d3)
    assert all(torch.equal(w1[k], w2[k]) for k in w1)
    assert not torch.equal(w1["model.embed_tokens.weight"], w3["model.embed_tokens.weight"])
    assert not torch.equal(w1["model.layers.0.mlp.gate_proj.weight"], w1["model.layers.0.mlp.up_proj.weight"])


def _cpu_model(cfg, dtype="float32"):
    return Model(rl.describe_model(cfg), Runtime.create("cpu", dtype))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tiny_weights):
    w = dict(tiny_weights["B"])
    del w["model.layers.1.mlp.down_proj.weight"]
    del w["lm_head.weight"]
    w["model.layers.7.extra.weight"] = torch.zeros(2, 2, dtype=torch.bfloat16)
    w["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(10, 144, dtype=torch.bfloat16)
    w["model.norm.weight"] = torch.zeros(144, dtype=torch.int32)
    with pytest.raises(WeightsError) as e:
        load_tensors(_cpu_model(TINY_B), w)
    err = e.value
    assert err.missing == ["lm_head.weight", "model.layers.1.mlp.down_proj.weight"]
    assert err.unexpected == ["model.layers.7.extra.weight"]
    assert err.wrong_shape == [("model.layers.0.self_attn.q_proj.weight", (10, 144), (144, 144))]
    assert err.wrong_dtype == [("model.norm.weight", "I32")]
    text = str(err)
    for needle in ("missing (2)", "unexpected (1)", "wrong shape (1)", "is [10, 144], expected [144, 144]", "unusable type"):
        assert needle in text


def test_run_types_of_loaded_tensors(tiny_weights):
    # a bfloat16 run: matrices in bfloat16, a vector stored in 32-bit stays 32-bit
    m = _cpu_model(TINY_A, "bfloat16")
    load_tensors(m, tiny_weights["A"])  # stored float32
    assert m.blocks[0].mixer.w_qkv.dtype == torch.bfloat16 and m.blocks[0].mixer.w_qkv.shape == (64 + 2 * 32, 64)
    assert m.blocks[0].norms["mixer"].weight.dtype == torch.float32
    assert m.head.weight is m.embedding.weight  # tied: the same tensor, not a copy
    m = _cpu_model(TINY_B, "bfloat16")
    load_tensors(m, tiny_weights["B"])  # stored bfloat16
    assert m.final_norm.weight.dtype == torch.bfloat16 and m.blocks[2].feed_forward.w_gate_up.shape == (768, 144)
    # bfloat16 runs keep gate and up rows alternating for the fused kernel
    gu = m.blocks[2].feed_forward.w_gate_up
    assert torch.equal(gu[0::2], tiny_weights["B"]["model.layers.2.mlp.gate_proj.weight"])
    assert torch.equal(gu[1::2], tiny_weights["B"]["model.layers.2.mlp.up_proj.weight"])
    # a 32-bit run widens everything exactly
    m = _cpu_model(TINY_B, "float32")
    load_tensors(m, tiny_weights["B"])
    assert m.head.weight.dtype == torch.float32
    assert torch.equal(m.head.weight, tiny_weights["B"]["lm_head.weight"].float())


def test_truncated_and_corrupt_files_are_errors_not_crashes(tiny_dirs, tmp_path):
    src = os.path.join(tiny_dirs["A"], "model.safetensors")
    blob = open(src, "rb").read()
    d = tmp_path / "trunc"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(TINY_A))
    for cut in (4, 100, len(blob) // 2, len(blob) - 1):
        (d / "model.safetensors").write_bytes(blob[:cut])
        with pytest.raises(WeightsError):
            Checkpoint(str(d))
    (d / "model.safetensors").write_bytes(struct.pack("<Q", 1 << 60) + b"{}")
    with pytest.raises(WeightsError, match="truncated or not safetensors"):
        Checkpoint(str(d))
    (d / "model.safetensors").write_bytes(struct.pack("<Q", 9) + b"{not json")
    with pytest.raises(WeightsError, match="not valid JSON"):
        Checkpoint(str(d))
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}, "b": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}).encode()
    (d / "model.safetensors").write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 12)
    with pytest.raises(WeightsError, match="overlap"):
        Checkpoint(str(d))
    os.remove(d / "model.safetensors")
    with pytest.raises(WeightsError, match="neither model.safetensors"):
        Checkpoint(str(d))


def test_sharded_checkpoint(tiny_weights, tmp_path):
    w = tiny_weights["A"]
    names = sorted(w)
    half = len(names) // 2
    write_safetensors(str(tmp_path / "s1.safetensors"), {n: w[n] for n in names[:half]})
    write_safetensors(str(tmp_path / "s2.safetensors"), {n: w[n] for n in names[half:]})
    index = {"weight_map": {n: ("s1.safetensors" if i < half else "s2.safetensors") for i, n in enumerate(names)}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    with Checkpoint(str(tmp_path)) as c:
        assert sorted(c.names()) == names
        assert torch.equal(c.read(names[-1]), w[names[-1]])
        m = _cpu_model(TINY_A)
        load_tensors(m, c)
    assert m.loaded


def test_known_redundant_tensors_are_passed_over_and_unknown_ones_are_not(tiny_weights, capsys):
    """Llama folders often carry rotary tables as buffers and, beside tied embeddings, a copy of the matrix as
    lm_head.weight: the architecture names those patterns and the loader passes over them with a note; a
    tensor that nobody names stays an error, and so does lm_head.weight's absence in an untied model."""
    w = dict(tiny_weights["A"])  # tied
    w["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    w["lm_head.weight"] = w["model.embed_tokens.weight"].clone()
    m = _cpu_model(TINY_A)
    load_tensors(m, w)
    assert m.loaded and m.head.weight is m.embedding.weight
    assert "passing over 2 tensors" in capsys.readouterr().err
    w["model.layers.0.self_attn.rotary_emb.cos_cached"] = torch.zeros(8)
    with pytest.raises(WeightsError) as e:
        load_tensors(_cpu_model(TINY_A), w)
    assert e.value.unexpected == ["model.layers.0.self_attn.rotary_emb.cos_cached"]
    b = dict(tiny_weights["B"])  # untied: lm_head.weight is wanted, not redundant
    del b["lm_head.weight"]
    with pytest.raises(WeightsError) as e:
        load_tensors(_cpu_model(TINY_B), b)
    assert e.value.missing == ["lm_head.weight"]


def test_a_checkpoint_stored_in_float16_loads_into_either_run_type(tmp_path):
    cfg = dict(TINY_A, torch_dtype="float16")
    d = write_random_model(str(tmp_path / "h"), cfg, 5)
    w = read_weights(d)
    assert all(t.dtype == torch.float16 for t in w.values())
    for run, want in (("bfloat16", torch.bfloat16), ("float32", torch.float32)):
        m = _cpu_model(cfg, run)
        load_tensors(m, w)
        assert m.blocks[0].mixer.w_o.dtype == want
        assert torch.equal(m.blocks[0].mixer.w_o, w["model.layers.0.self_attn.o_proj.weight"].to(want))
