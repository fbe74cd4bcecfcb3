"""Shared pieces of the tests: tiny configurations, model folders, replay drivers."""
from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# Three tiny Qwen2 configurations that differ in every size and option: head counts and
# groups (4/2, 6/1, 3/3), head sizes (16, 32, 48), widths that are no power of two,
# number of layers, vocabulary (one of them prime), theta, eps, tying, page size, and a
# window on some layers of the third.
TINY_A = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=256, hidden_size=64, intermediate_size=128,
    num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, rms_norm_eps=1e-6, rope_theta=10000.0,
    max_position_embeddings=128, hidden_act="silu", tie_word_embeddings=True, use_sliding_window=False,
    eos_token_id=255)
TINY_B = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=503, hidden_size=192, intermediate_size=320,
    num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=1, rms_norm_eps=1e-5, rope_theta=1e6,
    max_position_embeddings=256, hidden_act="silu", tie_word_embeddings=False, use_sliding_window=False,
    eos_token_id=[501, 502])
TINY_C = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=331, hidden_size=104, intermediate_size=200,
    num_hidden_layers=4, num_attention_heads=3, num_key_value_heads=3, head_dim=48, rms_norm_eps=3e-6,
    rope_theta=50000.0, max_position_embeddings=192, hidden_act="silu", tie_word_embeddings=False,
    use_sliding_window=True, sliding_window=20, max_window_layers=2, eos_token_id=None)

# Two with sizes the tensor-core kernels cannot take as they are: a width and an intermediate size
# that are no multiples of 8 (rows of no 16-byte multiple), a head of 80, and a head of 160 (beyond
# the tensor-core attention); heads * head size differs from the width.
TINY_D = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=257, hidden_size=100, intermediate_size=90,
    num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1, head_dim=80, rms_norm_eps=1e-5,
    rope_theta=10000.0, max_position_embeddings=160, hidden_act="silu", tie_word_embeddings=True,
    use_sliding_window=False, eos_token_id=3)
TINY_E = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=129, hidden_size=72, intermediate_size=136,
    num_hidden_layers=2, num_attention_heads=5, num_key_value_heads=5, head_dim=160, rms_norm_eps=1e-6,
    rope_theta=500000.0, max_position_embeddings=128, hidden_act="silu", tie_word_embeddings=False,
    use_sliding_window=False, eos_token_id=None)

# Two whose heads are the sizes the tcgen05 attention is built for (64 and 128), with positions enough for
# portions of more than 64 tokens, which is where that kernel takes over from the mma.sync one.
TINY_F = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=311, hidden_size=256, intermediate_size=176,
    num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6,
    rope_theta=1e6, max_position_embeddings=448, hidden_act="silu", tie_word_embeddings=True,
    use_sliding_window=False, eos_token_id=None)
TINY_G = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=205, hidden_size=160, intermediate_size=232,
    num_hidden_layers=3, num_attention_heads=2, num_key_value_heads=1, head_dim=128, rms_norm_eps=1e-5,
    rope_theta=10000.0, max_position_embeddings=400, hidden_act="silu", tie_word_embeddings=False,
    use_sliding_window=True, sliding_window=150, max_window_layers=2, eos_token_id=None)

TINY = {"A": (TINY_A, dict(seed=0, page_size=4)), "B": (TINY_B, dict(seed=1, page_size=16)),
        "C": (TINY_C, dict(seed=2, page_size=8)), "D": (TINY_D, dict(seed=3, page_size=32)),
        "E": (TINY_E, dict(seed=4, page_size=64)), "F": (TINY_F, dict(seed=5, page_size=16)),
        "G": (TINY_G, dict(seed=6, page_size=32))}

# Random weights N(0, 0.02) make attention nearly uniform and would hide a misplaced key;
# the q and k projections are scaled up so that scores spread over several units (more would only amplify rounding).
PEAKY = {"q_proj.weight": 3.0, "k_proj.weight": 3.0, "q_proj.bias": 3.0, "k_proj.bias": 3.0}


def make_model_folder(folder, cfg_dict, seed, dtype="float32", std=0.05, scales=PEAKY):
    import torch
    from llm_inference_lab_b200.registry import resolve
    from llm_inference_lab_b200.weights import write_random_model

    arch = resolve(cfg_dict)
    cfg = arch.config_class.from_dict(cfg_dict)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    write_random_model(cfg, folder, seed=seed, dtype=tdt, std=std, scales=scales)
    return folder


def random_tokens(rng, n, vocab):
    return [int(t) for t in rng.integers(0, vocab, size=n)]


def plain_logits(folder, sequences, twin=None):
    """{name: [len, vocab] float64} of whole sequences by the plain implementation.  `twin`: "float32"
    computes in 32-bit, "bfloat16" rounds every operator's result to bfloat16: what the arithmetic of an
    engine of that type alone does to these logits."""
    import contextlib

    from plain_qwen2 import plain_forward, plain_precision, read_model_folder, round_bfloat16

    cfg, w = read_model_folder(folder)
    how = {None: contextlib.nullcontext(), "float32": plain_precision(np.float32),
           "bfloat16": plain_precision(edge=round_bfloat16)}[twin]
    with how:
        return {name: np.asarray(plain_forward(cfg, w, ids), dtype=np.float64) for name, ids in sequences.items()}


# ----------------------------------------------------------------------------------------
# Traces: lists of steps in bin/trace_run's format, built for the ways of cutting.
# ----------------------------------------------------------------------------------------

def trace_whole(sequences):
    steps = []
    for i, (name, ids) in enumerate(sequences.items()):
        steps.append({"step": i, "entries": [{"id": name, "tokens": ids, "want": list(range(len(ids)))}],
                      "end": [name]})
    return steps


def trace_tail_decode(sequences, tail=32):
    steps = []
    n = 0
    for name, ids in sequences.items():
        head = max(len(ids) - tail, 1)
        steps.append({"step": n, "entries": [{"id": name, "tokens": ids[:head], "want": list(range(head))}],
                      "end": []})
        n += 1
        for p in range(head, len(ids)):
            steps.append({"step": n, "entries": [{"id": name, "tokens": [ids[p]], "want": [0]}],
                          "end": [name] if p == len(ids) - 1 else []})
            n += 1
        if head == len(ids):
            steps[-1]["end"] = [name]
    return steps


def trace_portions(sequences, sizes=(7, 2, 5, 3, 2, 11, 4, 2, 9)):
    steps = []
    n = 0
    for name, ids in sequences.items():
        at = 0
        k = 0
        while at < len(ids):
            size = min(sizes[k % len(sizes)], len(ids) - at)
            k += 1
            end = [name] if at + size == len(ids) else []
            steps.append({"step": n, "entries": [{"id": name, "tokens": ids[at:at + size],
                                                  "want": list(range(size))}], "end": end})
            at += size
            n += 1
    return steps


def trace_mixed(sequences, rng, max_live=4, max_portion=9, decode_after=0.6):
    """Up to `max_live` requests at a time: portions of some beside single tokens of others;
    a request may sit a step out; finished requests end and new ones start on their pages."""
    names = list(sequences)
    waiting = list(names)
    live = {}
    steps = []
    n = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            live[waiting.pop(0)] = 0
        entries = []
        end = []
        for name in list(live):
            ids = sequences[name]
            at = live[name]
            if len(live) > 1 and rng.random() < 0.2:
                continue   # left out of this step, goes on later
            left = len(ids) - at
            if at >= decode_after * len(ids):
                size = 1
            else:
                size = int(min(left, rng.integers(2, max_portion + 1)))
            entries.append({"id": name, "tokens": ids[at:at + size], "want": list(range(size))})
            live[name] = at + size
            if live[name] == len(ids):
                end.append(name)
                del live[name]
        if entries:
            steps.append({"step": n, "entries": entries, "end": end})
            n += 1
    return steps


def random_config(rng, layers=None):
    """A random Qwen2 configuration and page size: head sizes in steps of 16, any number of heads and
    groups, widths and intermediate sizes that are multiples of 8 or only of 2, any vocabulary,
    sometimes a window on the later layers."""
    head_dim = int(rng.choice([16, 32, 48, 64, 64, 80, 96, 112, 128, 128]))
    n_kv = int(rng.choice([1, 2, 3, 4]))
    n_heads = n_kv * int(rng.choice([1, 2, 3, 4, 7, 8]))
    n_layers = int(rng.integers(1, 4)) if layers is None else layers
    cfg = dict(
        architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=int(rng.integers(40, 3000)),
        hidden_size=int(rng.choice([8, 8, 8, 2])) * int(rng.integers(4, 40)),
        intermediate_size=int(rng.choice([8, 8, 16, 2])) * int(rng.integers(4, 60)),
        num_hidden_layers=n_layers, num_attention_heads=n_heads, num_key_value_heads=n_kv, head_dim=head_dim,
        rms_norm_eps=float(rng.choice([1e-6, 1e-5, 3e-6])), rope_theta=float(rng.choice([1e4, 1e6, 5e4])),
        max_position_embeddings=int(rng.choice([96, 200, 400, 700])), hidden_act="silu",
        tie_word_embeddings=bool(rng.random() < 0.5), use_sliding_window=bool(rng.random() < 0.25), eos_token_id=None)
    if cfg["use_sliding_window"]:
        cfg.update(sliding_window=int(rng.integers(3, 150)), max_window_layers=int(rng.integers(0, n_layers)))
    return cfg, int(rng.choice([16, 16, 16, 4, 8, 32, 64]))


def trace_random(sequences, rng, max_live=4, sizes=(1, 1, 1, 2, 3, 7, 16, 40, 65, 130, 300)):
    """Requests start in random order and at random times; every step takes a portion of random size
    (single tokens, a few, or hundreds) from most of the live ones."""
    waiting = list(sequences)
    rng.shuffle(waiting)
    at = {name: 0 for name in waiting}
    live, steps = [], []
    while live or waiting:
        while waiting and len(live) < max_live and rng.random() < 0.7:
            live.append(waiting.pop())
        if not live:
            live.append(waiting.pop())
        entries, end = [], []
        for name in list(live):
            if rng.random() < 0.2 and len(live) > 1:
                continue
            size = int(min(len(sequences[name]) - at[name], rng.choice(list(sizes))))
            entries.append({"id": name, "tokens": sequences[name][at[name]: at[name] + size],
                            "want": list(range(size))})
            at[name] += size
            if at[name] == len(sequences[name]):
                end.append(name)
                live.remove(name)
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


def tokens_needed(steps, page=64):
    """Most tokens live requests hold at any time, each rounded up to a multiple of `page`."""
    held = {}
    most = 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        most = max(most, sum(-(-v // page) * page for v in held.values()))
        for name in st["end"]:
            held.pop(name, None)
    return most


def run_trace_inprocess(engine, steps):
    """Drives `Engine.step` the way bin/trace_run does; returns {(name, position): logits}."""
    from llm_inference_lab_b200.engine import Entry
    from llm_inference_lab_b200.kernels import ops

    ids = {}
    at = {}
    out = {}
    counter = 0
    for st in steps:
        entries = []
        for e in st["entries"]:
            if e["id"] not in ids:
                ids[e["id"]] = counter
                counter += 1
            entries.append(Entry(ids[e["id"]], e["tokens"], e["want"]))
        logits = engine.step(entries)
        if logits is not None:
            arr = logits.float().cpu().numpy()
            k = 0
            for e in st["entries"]:
                base = at.get(e["id"], 0)
                for w in e["want"]:
                    out[(e["id"], base + w)] = arr[k]
                    k += 1
        for e in st["entries"]:
            at[e["id"]] = at.get(e["id"], 0) + len(e["tokens"])
        for name in st["end"]:
            engine.close(ids.pop(name))
            at.pop(name)
    ops.take_device_errors()
    return out


def run_trace_program(folder, dtype, steps, out_dir, max_tokens, page_size=None, timeout=600):
    """Runs bin/trace_run as a user would; returns {(name, position): logits}."""
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens)]
    if page_size:
        cmd += ["--page-size", str(page_size)]
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=timeout)
    if proc.returncode != 0:
        raise RuntimeError(f"trace_run failed ({proc.returncode}):\n{proc.stdout[-2000:]}\n{proc.stderr[-4000:]}")
    done = [line for line in proc.stdout.splitlines() if line.startswith("done ")]
    assert [int(d.split()[1]) for d in done] == [s["step"] for s in steps], "a 'done' line per step, in order"
    with open(os.path.join(folder, "config.json")) as fh:
        vocab = json.load(fh)["vocab_size"]
    out = {}
    at = {}
    for st in steps:
        n_want = sum(len(e["want"]) for e in st["entries"])
        path = os.path.join(out_dir, f"{st['step']}.f32")
        if n_want:
            arr = np.fromfile(path, dtype="<f4").reshape(n_want, vocab)
            k = 0
            for e in st["entries"]:
                base = at.get(e["id"], 0)
                for w in e["want"]:
                    out[(e["id"], base + w)] = arr[k]
                    k += 1
        else:
            assert not os.path.exists(path)
        for e in st["entries"]:
            at[e["id"]] = at.get(e["id"], 0) + len(e["tokens"])
        for name in st["end"]:
            at.pop(name, None)
    return out


def worst_error(got, want_by_name):
    """(max abs error, max |reference|, where) over every (name, position) in `got`."""
    worst, where, scale = 0.0, None, 0.0
    for (name, pos), row in got.items():
        ref = want_by_name[name][pos]
        scale = max(scale, float(np.abs(ref).max()))
        err = float(np.abs(row.astype(np.float64) - ref).max())
        if not np.isfinite(err):
            return float("inf"), scale, (name, pos)
        if err > worst:
            worst, where = err, (name, pos)
    return worst, scale, where


def error_stats(got, want_by_name):
    """(max abs error / max |ref|, rms error / rms ref, where the worst lies)."""
    worst, where = 0.0, None
    se, sr, peak = 0.0, 0.0, 0.0
    for (name, pos), row in got.items():
        ref = want_by_name[name][pos]
        diff = row.astype(np.float64) - ref
        if not np.isfinite(diff).all():
            return float("inf"), float("inf"), (name, pos)
        peak = max(peak, float(np.abs(ref).max()))
        se += float((diff * diff).sum())
        sr += float((ref * ref).sum())
        err = float(np.abs(diff).max())
        if err > worst:
            worst, where = err, (name, pos)
    return worst / max(peak, 1e-30), (se / max(sr, 1e-30)) ** 0.5, where
