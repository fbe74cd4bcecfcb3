"""Weights by tensor name: reading, writing, the one error, the random-weights mode (no GPU)."""
import json
import os
import struct

import pytest
import torch

from helpers import TINY_A, TINY_B, make_model_folder
from llm_inference_lab_b200.config import Qwen2Config, qwen2_blueprint
from llm_inference_lab_b200.models.builder import _tied_extras, expected_tensors
from llm_inference_lab_b200.weights import (ModelFiles, SafetensorsError, WeightsError, kept_dtype, load_weights,
                                            save_file, write_random_model)


def specs_of(raw):
    bp = qwen2_blueprint(Qwen2Config.from_dict(raw))
    return bp, expected_tensors(bp)


def test_random_model_is_complete_and_reproducible(tmp_path):
    a = make_model_folder(str(tmp_path / "a"), TINY_A, seed=0, dtype="bfloat16")
    b = make_model_folder(str(tmp_path / "b"), TINY_A, seed=0, dtype="bfloat16")
    c = make_model_folder(str(tmp_path / "c"), TINY_A, seed=1, dtype="bfloat16")
    assert sorted(os.listdir(a)) == ["config.json", "model.safetensors"]
    bp, specs = specs_of(TINY_A)
    wa, wb, wc = (load_weights(f, specs, "cpu") for f in (a, b, c))
    assert set(wa) == {s.name for s in specs}
    assert all(torch.equal(wa[n], wb[n]) for n in wa) and any(not torch.equal(wa[n], wc[n]) for n in wa)
    assert all(t.dtype == torch.bfloat16 for t in wa.values())
    norm = wa["model.norm.weight"].float()
    assert 0.5 < norm.mean() < 1.5 and abs(wa["model.layers.0.mlp.up_proj.weight"].float().mean()) < 0.01
    # the library's reader agrees with ours on every byte
    from safetensors.torch import load_file
    theirs = load_file(os.path.join(a, "model.safetensors"))
    assert set(theirs) == set(wa) and all(torch.equal(theirs[n], wa[n]) for n in wa)
    assert json.load(open(os.path.join(a, "config.json")))["architectures"] == ["Qwen2ForCausalLM"]


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = make_model_folder(str(tmp_path / "m"), TINY_B, seed=1, dtype="float32")
    bp, specs = specs_of(TINY_B)
    files = ModelFiles(folder)
    tensors = {n: files.get(n).clone() for n in files.names()}
    del tensors["model.layers.1.mlp.up_proj.weight"], tensors["lm_head.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(7)
    tensors["model.layers.2.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    with pytest.raises(WeightsError) as err:
        load_weights(folder, specs, "cpu")
    e = err.value
    assert e.missing == ["lm_head.weight", "model.layers.1.mlp.up_proj.weight"]
    assert e.unexpected == ["model.layers.2.self_attn.rotary_emb.inv_freq"]
    assert [w[0] for w in e.wrong_shape] == ["model.layers.0.self_attn.q_proj.bias"]
    text = str(e)
    assert "missing (2)" in text and "unexpected (1)" in text and "is [7], wanted [192]" in text


def test_tied_checkpoint_may_carry_a_head_copy(tmp_path):
    folder = make_model_folder(str(tmp_path / "m"), TINY_A, seed=0, dtype="float32")
    bp, specs = specs_of(TINY_A)
    files = ModelFiles(folder)
    tensors = {n: files.get(n).clone() for n in files.names()}
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    out = load_weights(folder, specs, "cpu", optional=_tied_extras(bp))
    assert "lm_head.weight" not in out


def test_kept_dtypes(tmp_path):
    assert kept_dtype(torch.bfloat16) == torch.bfloat16 and kept_dtype(torch.float16) == torch.float32
    assert kept_dtype(torch.float32) == torch.float32 and kept_dtype(torch.float64) == torch.float32
    assert kept_dtype(torch.int64) == torch.int32
    path = str(tmp_path / "t.safetensors")
    save_file({"a": torch.tensor([1.5, -0.0], dtype=torch.float32), "b": torch.arange(4, dtype=torch.int64),
               "c": torch.tensor([[1.0, 2.0]], dtype=torch.bfloat16),
               "h": torch.tensor([1.0009765625, 3.0e-5], dtype=torch.float16)}, path)
    from llm_inference_lab_b200.parts.spec import TensorSpec
    os.rename(path, str(tmp_path / "model.safetensors"))
    out = load_weights(str(tmp_path), [TensorSpec("a", (2,)), TensorSpec("b", (4,)), TensorSpec("c", (1, 2)),
                                       TensorSpec("h", (2,))], "cpu")
    assert out["a"].dtype == torch.float32 and out["b"].dtype == torch.int32 and out["c"].dtype == torch.bfloat16
    assert torch.signbit(out["a"][1]) and out["b"].tolist() == [0, 1, 2, 3]
    # float16 reaches a 32-bit engine exactly (1 + 2^-10 has no bfloat16)
    assert out["h"].dtype == torch.float32
    assert out["h"].tolist() == torch.tensor([1.0009765625, 3.0e-5], dtype=torch.float16).float().tolist()


def test_sharded_index_and_broken_files(tmp_path):
    folder = str(tmp_path)
    save_file({"x": torch.ones(2, 3)}, os.path.join(folder, "part-1.safetensors"))
    save_file({"y": torch.zeros(4)}, os.path.join(folder, "part-2.safetensors"))
    index = {"weight_map": {"x": "part-1.safetensors", "y": "part-2.safetensors"}}
    open(os.path.join(folder, "model.safetensors.index.json"), "w").write(json.dumps(index))
    files = ModelFiles(folder)
    assert sorted(files.names()) == ["x", "y"] and files.get("x").shape == (2, 3)
    with pytest.raises(SafetensorsError, match="not found"):
        files.get("z")
    index["weight_map"]["y"] = "../part-2.safetensors"
    open(os.path.join(folder, "model.safetensors.index.json"), "w").write(json.dumps(index))
    with pytest.raises(SafetensorsError, match="plain"):
        ModelFiles(folder)
    open(os.path.join(folder, "model.safetensors.index.json"), "w").write("{")
    with pytest.raises(SafetensorsError, match="broken index"):
        ModelFiles(folder)          # a broken index never falls back to a single file
    os.remove(os.path.join(folder, "model.safetensors.index.json"))
    with pytest.raises(SafetensorsError, match="no model.safetensors"):
        ModelFiles(folder)
    with open(os.path.join(folder, "model.safetensors"), "wb") as fh:
        fh.write(struct.pack("<Q", 10**9) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        ModelFiles(folder)
    header = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    with open(os.path.join(folder, "model.safetensors"), "wb") as fh:
        fh.write(struct.pack("<Q", len(header)) + header + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="holds 8 bytes"):
        ModelFiles(folder)


def test_scales_make_attention_peaky(tmp_path):
    cfg = Qwen2Config.from_dict(TINY_A)
    write_random_model(cfg, str(tmp_path / "a"), seed=3, dtype=torch.float32)
    write_random_model(cfg, str(tmp_path / "b"), seed=3, dtype=torch.float32, scales={"q_proj.weight": 4.0})
    fa, fb = ModelFiles(str(tmp_path / "a")), ModelFiles(str(tmp_path / "b"))
    n = "model.layers.0.self_attn.q_proj.weight"
    assert torch.allclose(fa.get(n) * 4, fb.get(n)) and torch.equal(fa.get("model.norm.weight"),
                                                                    fb.get("model.norm.weight"))
