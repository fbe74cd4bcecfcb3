"""The reference's own tiny Qwen2 model, restated: its shape and its closed-form weights.

pochenai/llm-inference-lab's engine tests build a small model without checkpoint files
(rust/engine/src/runner/model/qwen2/engine.rs:2360-2454): hidden 128, two query heads and one
key/value head of 64, intermediate 64, vocabulary 257, two layers, theta 1e6, eps 1e-6, tied head,
64 positions.  A tensor with seed s holds, at flat row-major index i,

    ((i * 13 + s * 7) % 59) * 0.003 - 0.087        (32-bit arithmetic; s == 0 means all ones)

with seed 1 for the embedding, 0 for every norm, and for the layers with base seeds 2 and 13:
q +0, k +1, v +2, o +3, q bias +4, k bias +5, v bias +6, gate +7, up +8, down +9.  This is the one
piece of the reference's test data that can be rebuilt bit for bit without its toolchain; this file
writes it as a model folder (config.json, model.safetensors) with the `safetensors` library.  Its
head size of 64 with two query heads on one key/value head and a tied head is the shape family the
tcgen05 attention serves.
"""
from __future__ import annotations

import json
import os

import numpy as np

REFERENCE_TINY = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=257, hidden_size=128, intermediate_size=64,
    num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1, rms_norm_eps=1e-6, rope_theta=1000000.0,
    max_position_embeddings=64, tie_word_embeddings=True, eos_token_id=256, hidden_act="silu")

# The reference's own bounds for this model (absolute, on logits): 32-bit packed against serial
# (engine.rs:3512); bfloat16 cached against whole, and bfloat16 against 32-bit (engine.rs:4814-4820).
F32_ABS, BF16_CUT_ABS, BF16_F32_ABS = 1e-4, 0.01, 0.03
# The histories of the reference's bfloat16 test (engine.rs:4782).
HISTORIES = [[1] * 33, [4, 9, 7], [3, 5, 8, 13, 21]]


def closed_form(shape, seed):
    n = int(np.prod(shape))
    if seed == 0:
        return np.ones(shape, dtype=np.float32)
    k = ((np.arange(n, dtype=np.int64) * 13 + seed * 7) % 59).astype(np.float32)
    return (k * np.float32(0.003) - np.float32(0.087)).astype(np.float32).reshape(shape)


def reference_tiny_tensors():
    t = {"model.embed_tokens.weight": closed_form((257, 128), 1), "model.norm.weight": closed_form((128,), 0)}
    for layer, seed in enumerate((2, 13)):
        p = f"model.layers.{layer}."
        t[p + "input_layernorm.weight"] = closed_form((128,), 0)
        t[p + "post_attention_layernorm.weight"] = closed_form((128,), 0)
        for offset, (name, shape) in enumerate([
                ("self_attn.q_proj.weight", (128, 128)), ("self_attn.k_proj.weight", (64, 128)),
                ("self_attn.v_proj.weight", (64, 128)), ("self_attn.o_proj.weight", (128, 128)),
                ("self_attn.q_proj.bias", (128,)), ("self_attn.k_proj.bias", (64,)), ("self_attn.v_proj.bias", (64,)),
                ("mlp.gate_proj.weight", (64, 128)), ("mlp.up_proj.weight", (64, 128)),
                ("mlp.down_proj.weight", (128, 64))]):
            t[p + name] = closed_form(shape, seed + offset)
    return t


def write_reference_tiny(folder, dtype="float32"):
    """The model folder; `dtype` bfloat16 rounds every tensor to nearest even, as the reference's
    decoding of 32-bit weights into a bfloat16 model does (rust/engine/src/runner/loader.rs:57-133)."""
    import torch
    from safetensors.torch import save_file

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(REFERENCE_TINY, fh)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    save_file({k: torch.from_numpy(v).to(tdt).contiguous() for k, v in reference_tiny_tensors().items()},
              os.path.join(folder, "model.safetensors"))
    return folder
