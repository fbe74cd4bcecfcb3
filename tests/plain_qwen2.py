"""A plain, slow Qwen2 forward pass: the yardstick of every numerical test.

Whole sequences, no cache, no batching, one function for each part, NumPy in
float64 over the stored weights.  It shares no code with the package: it reads
the model folder with the `safetensors` library and its own few lines of JSON
handling.

It rests on the reference's formulas, not on the reference's code being run:
pochenai/llm-inference-lab is Rust + cuTile and cannot be compiled or imported
on a machine without cargo and the cuTile toolchain, and its own Python
fixture script only wraps a library's model code with a downloaded checkpoint
(rust/engine/examples/qwen2_reference.py:21-63).  Every function below cites
the lines of the reference whose formula it restates.  Where the reference
rounds to its storage type T between operators, this file does not (T is
float64 here); the 32-bit engine is compared with a tight tolerance and the
bfloat16 engine with the band the reference itself uses for T = bf16.

How far rounding alone moves the logits of a given model is measured with the same
functions: inside `plain_precision(np.float32)` they compute in 32-bit, and inside
`plain_precision(edge=round_bfloat16)` every operator's result is rounded to
bfloat16 where the reference's T = bf16 kernels round (kernels.rs:393-418 one
rounding per product, 546-582 norm, 587-631 rotation, 802-828 p rounded before
P V, 1469-1486 the gated product, the residual sum).  A test may hold an engine's
error against such a twin where it exceeds its fixed bound.
"""
from __future__ import annotations

import contextlib
import json
import os

import numpy as np

_COMPUTE = np.float64   # the type the parts compute in
_EDGE = None            # what every operator's result goes through (None: nothing)


@contextlib.contextmanager
def plain_precision(compute=np.float64, edge=None):
    """Within the block the parts compute in `compute` and pass each operator's result through `edge`."""
    global _COMPUTE, _EDGE
    saved = (_COMPUTE, _EDGE)
    _COMPUTE, _EDGE = compute, edge
    try:
        yield
    finally:
        _COMPUTE, _EDGE = saved


def round_bfloat16(x):
    """x rounded to the nearest bfloat16 (ties to even), as float32."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    finite = (bits & np.uint32(0x7F800000)) != np.uint32(0x7F800000)
    rounded = (bits + np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return np.where(finite, rounded, bits).astype(np.uint32).view(np.float32)


def _edge(y):
    return y if _EDGE is None else np.asarray(_EDGE(y), dtype=_COMPUTE)


# ----------------------------------------------------------------------------------------
# Parts
# ----------------------------------------------------------------------------------------

def plain_embedding(ids, table):
    """x[t, :] = table[ids[t], :], no scaling.  rust/engine/src/runner/model/qwen2/kernels.rs:46-57"""
    return _edge(np.asarray(table, dtype=_COMPUTE)[np.asarray(ids, dtype=np.int64)])


def plain_rms_norm(x, weight, eps):
    """y = x * rsqrt(mean(x^2) + eps) * w, mean over the true width.  kernels.rs:546-582"""
    x = np.asarray(x, dtype=_COMPUTE)
    inv = 1.0 / np.sqrt((x * x).mean(axis=-1, keepdims=True) + _COMPUTE(eps))
    return _edge(x * inv * np.asarray(weight, dtype=_COMPUTE))


def _product(x, weight, bias=None):
    y = np.asarray(x, dtype=_COMPUTE) @ np.asarray(weight, dtype=_COMPUTE).T
    if bias is not None:
        y = y + np.asarray(bias, dtype=_COMPUTE)
    return y


def plain_linear(x, weight, bias=None):
    """y = x W^T (+ b); W is stored [out, in].  kernels.rs:156-178, 393-418"""
    return _edge(_product(x, weight, bias))


def plain_inv_freq(head_dim, theta):
    """inv_freq[i] = theta^(-2i/d), i in [0, d/2), held in 32-bit.  engine.rs:304-311"""
    i = np.arange(head_dim // 2, dtype=np.float64)
    return (float(theta) ** (-2.0 * i / head_dim)).astype(np.float32)


def plain_rope(x, positions, theta):
    """Split-half rotation of each head: out = [lo*c - hi*s, hi*c + lo*s] with the angle
    f32(pos) * inv_freq formed in 32-bit.  kernels.rs:587-631

    x: [T, heads, d]; positions: [T].
    """
    x = np.asarray(x, dtype=_COMPUTE)
    d = x.shape[-1]
    inv = plain_inv_freq(d, theta)
    ang = (np.asarray(positions, dtype=np.float32)[:, None] * inv[None, :]).astype(np.float32)
    c = np.cos(ang.astype(np.float64))[:, None, :].astype(_COMPUTE)
    s = np.sin(ang.astype(np.float64))[:, None, :].astype(_COMPUTE)
    lo, hi = x[..., : d // 2], x[..., d // 2:]
    return _edge(np.concatenate([lo * c - hi * s, hi * c + lo * s], axis=-1))


def plain_attention(q, k, v, positions, window=0):
    """Causal softmax attention with grouped key/value heads.

    score(p, j) = q_p . k_j / sqrt(d) for j <= p (and p - j < window when a window is
    set), else -inf; kv head of query head h is h // (n_h / n_kv).
    kernels.rs:736-766 (scores, mask), 802-828 (softmax), engine.rs:1589-1617 (grouping).
    The window rule is this engine's own (the reference refuses windows, engine.rs:262).

    q: [T, n_h, d]; k, v: [T, n_kv, d]; positions: [T] absolute, increasing.
    """
    q = np.asarray(q, dtype=_COMPUTE)
    k = np.asarray(k, dtype=_COMPUTE)
    v = np.asarray(v, dtype=_COMPUTE)
    T, n_h, d = q.shape
    n_kv = k.shape[1]
    group = n_h // n_kv
    pos = np.asarray(positions, dtype=np.int64)
    diff = pos[:, None] - pos[None, :]
    visible = diff >= 0
    if window:
        visible &= diff < window
    out = np.empty_like(q)
    scale = _COMPUTE(1.0 / np.sqrt(d))
    for h in range(n_h):
        g = h // group
        s = (q[:, h, :] @ k[:, g, :].T) * scale
        s = np.where(visible, s, -np.inf)
        s = s - s.max(axis=-1, keepdims=True)
        p = np.exp(s)
        if _EDGE is None:
            p = p / p.sum(axis=-1, keepdims=True)
            out[:, h, :] = p @ v[:, g, :]
        else:
            # p is rounded before P V, the sum runs over the unrounded p (kernels.rs:802-828, 946-1124)
            out[:, h, :] = (_edge(p) @ v[:, g, :]) / p.sum(axis=-1, keepdims=True)
    return _edge(out)


def plain_silu(x):
    """silu(g) = g / (1 + exp(-g)).  kernels.rs:1469-1486"""
    x = np.asarray(x, dtype=_COMPUTE)
    return x / (1.0 + np.exp(-x))


def plain_gated_mlp(x, w_gate, w_up, w_down):
    """down( silu(x Wg^T) * (x Wu^T) ), no biases.  kernels.rs:1469-1486; engine.rs:1242-1293"""
    return plain_linear(_edge(plain_silu(_product(x, w_gate)) * _product(x, w_up)), w_down)


def plain_attention_part(x, w, prefix, cfg, positions, window):
    """q/k/v projections with bias, rotation of q and k, attention, output projection
    without bias.  engine.rs:1133-1214 (project_qkv), 1225-1232 (o_proj)."""
    n_h, n_kv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], head_dim_of(cfg)
    T = x.shape[0]
    q = plain_linear(x, w[prefix + "q_proj.weight"], w[prefix + "q_proj.bias"]).reshape(T, n_h, d)
    k = plain_linear(x, w[prefix + "k_proj.weight"], w[prefix + "k_proj.bias"]).reshape(T, n_kv, d)
    v = plain_linear(x, w[prefix + "v_proj.weight"], w[prefix + "v_proj.bias"]).reshape(T, n_kv, d)
    q = plain_rope(q, positions, cfg["rope_theta"])
    k = plain_rope(k, positions, cfg["rope_theta"])
    a = plain_attention(q, k, v, positions, window).reshape(T, n_h * d)
    return plain_linear(a, w[prefix + "o_proj.weight"])


def plain_block(x, w, layer, cfg, positions):
    """Pre-norm block: r = x + attn(norm1(x)); out = r + mlp(norm2(r)).  engine.rs:1216-1296"""
    p = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    a = plain_attention_part(plain_rms_norm(x, w[p + "input_layernorm.weight"], eps), w, p + "self_attn.",
                             cfg, positions, layer_window(cfg, layer))
    r = _edge(x + a)
    f = plain_gated_mlp(plain_rms_norm(r, w[p + "post_attention_layernorm.weight"], eps),
                        w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return _edge(r + f)


# ----------------------------------------------------------------------------------------
# The whole model
# ----------------------------------------------------------------------------------------

def head_dim_of(cfg):
    return cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]


def layer_window(cfg, layer):
    if cfg.get("use_sliding_window") and layer >= cfg["max_window_layers"]:
        return int(cfg["sliding_window"])
    return 0


def plain_hidden(cfg, w, ids):
    """The final norm's output [T, hidden] of one whole sequence.  engine.rs:916-1130, 1298-1311"""
    ids = np.asarray(ids, dtype=np.int64)
    positions = np.arange(len(ids))
    x = plain_embedding(ids, w["model.embed_tokens.weight"])
    for layer in range(cfg["num_hidden_layers"]):
        x = plain_block(x, w, layer, cfg, positions)
    return plain_rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])


def plain_head(cfg, w, hidden):
    """Logits of rows of the final norm's output; the head is the embedding table when tied.
    engine.rs:299-303, 1312-1341"""
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    return _product(hidden, head)     # the logits stay 32-bit: no rounding at this edge


def plain_forward(cfg, w, ids):
    """Logits [T, vocab] of one whole sequence."""
    return plain_head(cfg, w, plain_hidden(cfg, w, ids))


def plain_argmax(logits):
    """Greedy pick; ties go to the smallest index.  kernels.rs:1488-1552"""
    return int(np.argmax(np.asarray(logits)))


def plain_greedy(cfg, w, prompt, n_new, eos=()):
    """Greedy continuation by running the whole sequence again for every token."""
    ids = list(prompt)
    out = []
    for _ in range(n_new):
        tok = plain_argmax(plain_forward(cfg, w, ids)[-1])
        out.append(tok)
        ids.append(tok)
        if tok in eos:
            break
    return out


# ----------------------------------------------------------------------------------------
# Temperature sampling (this engine's own rule; the reference is greedy only,
# rust/engine/src/runner/model_runner.rs:615-623).
# ----------------------------------------------------------------------------------------

def _mix32(x):
    x = np.asarray(x, dtype=np.uint64) & np.uint64(0xFFFFFFFF)
    x ^= x >> np.uint64(16)
    x = (x * np.uint64(0x7FEB352D)) & np.uint64(0xFFFFFFFF)
    x ^= x >> np.uint64(15)
    x = (x * np.uint64(0x846CA68B)) & np.uint64(0xFFFFFFFF)
    x ^= x >> np.uint64(16)
    return x


def plain_uniform(seed, position, vocab):
    """u[i] in (0, 1) from a 32-bit integer hash of (seed, position, i), 23 bits wide."""
    i = np.arange(vocab, dtype=np.uint64)
    h = _mix32(np.uint64(seed & 0xFFFFFFFF) ^ np.uint64(0x9E3779B9))
    h = _mix32(h ^ np.uint64(position & 0xFFFFFFFF))
    h = _mix32((h + i * np.uint64(0x85EBCA6B)) & np.uint64(0xFFFFFFFF))
    return ((h >> np.uint64(9)).astype(np.float64) + 0.5) / 8388608.0


def plain_sample(logits, temperature, seed, position):
    """Gumbel-max: argmax_i( logit_i / temperature - log(-log u_i) ); temperature 0 is greedy."""
    logits = np.asarray(logits, dtype=np.float64)
    if temperature == 0:
        return plain_argmax(logits), None
    u = plain_uniform(seed, position, logits.shape[-1])
    scores = logits / float(temperature) - np.log(-np.log(u))
    return int(np.argmax(scores)), scores


# ----------------------------------------------------------------------------------------
# Reading a model folder
# ----------------------------------------------------------------------------------------

def read_model_folder(folder):
    """(config dict, {name: float64 array}) of a folder with config.json + model.safetensors."""
    import torch
    from safetensors.torch import load_file

    with open(os.path.join(folder, "config.json")) as fh:
        cfg = json.load(fh)
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    weights = {name: t.to(torch.float64).numpy() for name, t in tensors.items()}
    return cfg, weights
