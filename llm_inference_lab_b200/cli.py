"""Command line: run one prompt through scheduler, step function and sampler.

Options keep the names and meanings of the reference's example program
(rust/engine/examples/qwen2.rs:38-73): ``--dtype bf16|f32``, ``--model-dir``,
``--prompt``, ``--max-new-tokens`` (8), ``--max-batch-tokens`` (512),
``--repeat``, ``--cuda-graph``, ``--trace-steps``; it prints one JSON line with
model, dtype, input_ids, text, elapsed, ttft, generated_tokens, tok/s and
kv_released (qwen2.rs:262-268).  Not taken over: ``--disable-overlap`` (there is
one step in flight at a time), ``--prefix-cache`` and ``--reference-dir``
(prefix sharing and checkpoint fixtures are out of scope).  Added:
``--prompt-ids`` for models without a tokenizer (random weights),
``--temperature`` and ``--seed``, ``--random-config`` to make a random model.

    python -m llm_inference_lab_b200.cli --model-dir DIR --prompt-ids 1,2,3 --max-new-tokens 8
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time


def chat_prompt(user: str) -> str:
    """The two-message chat template the reference hard-codes (rust/engine/examples/qwen2.rs:121-129)."""
    return ("<|im_start|>system\nYou are Qwen, created by Alibaba Cloud. You are a helpful assistant.<|im_end|>\n"
            f"<|im_start|>user\n{user}<|im_end|>\n<|im_start|>assistant\n")


def load_tokenizer(model_dir: str):
    path = os.path.join(model_dir, "tokenizer.json")
    if not os.path.exists(path):
        return None
    from tokenizers import Tokenizer
    return Tokenizer.from_file(path)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="llm_inference_lab_b200.cli", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f32"],
                    help="weight, activation and cache storage; sums stay 32-bit")
    ap.add_argument("--model-dir", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--prompt", default="Say hello.", help="user message (needs tokenizer.json in the folder)")
    ap.add_argument("--prompt-ids", default=None, help="comma-separated token ids instead of --prompt")
    ap.add_argument("--max-new-tokens", type=int, default=8)
    ap.add_argument("--max-batch-tokens", type=int, default=512,
                    help="most new tokens per step, shared by decode and prefill")
    ap.add_argument("--temperature", type=float, default=None, help="sample with this temperature (default greedy)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--repeat", type=int, default=1, help="run the same prompt again and check the tokens are equal")
    ap.add_argument("--cuda-graph", action="store_true", help="replay decode steps from a CUDA graph")
    ap.add_argument("--trace-steps", action="store_true", help="one JSON line per step on stderr")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--kv-tokens", type=int, default=None, help="size of the cache pool in tokens")
    ap.add_argument("--random-config", default=None,
                    help="a config.json: write a random model into --model-dir first (with --seed)")
    args = ap.parse_args(argv)
    if args.max_new_tokens <= 0:
        ap.error("--max-new-tokens must be positive")

    if args.random_config:
        import torch
        from .registry import resolve
        from .config.base import read_config_json
        from .weights import write_random_model
        raw = read_config_json(args.random_config)
        cfg = resolve(raw).config_class.from_dict(raw)
        write_random_model(cfg, args.model_dir, seed=args.seed, dtype=torch.bfloat16)

    from .engine.llm import LLM
    from .sampling import SamplingConfig

    tokenizer = load_tokenizer(args.model_dir)
    if args.prompt_ids is not None:
        input_ids = [int(t) for t in args.prompt_ids.split(",") if t.strip()]
    elif tokenizer is not None:
        input_ids = tokenizer.encode(chat_prompt(args.prompt), add_special_tokens=False).ids
    else:
        ap.error("the model folder has no tokenizer.json: give --prompt-ids")

    t_load = time.perf_counter()
    llm = LLM(args.model_dir, args.dtype, max_batch_tokens=args.max_batch_tokens, page_size=args.page_size,
              kv_tokens=args.kv_tokens, cuda_graph=args.cuda_graph)
    if args.trace_steps:
        llm.trace = lambda rec: print(json.dumps(rec), file=sys.stderr, flush=True)
    load_s = time.perf_counter() - t_load
    sampling = SamplingConfig(max_new_tokens=args.max_new_tokens, do_sample=args.temperature is not None,
                              temperature=args.temperature, seed=args.seed)
    first = None
    for _ in range(args.repeat):
        t0 = time.perf_counter()
        result = llm.generate([input_ids], sampling)[0]
        elapsed = time.perf_counter() - t0
        if first is None:
            first = result
        elif result.tokens != first.tokens:
            print("repeat produced other tokens", file=sys.stderr)
            return 1
    text = tokenizer.decode(result.tokens) if tokenizer is not None else None
    free = llm.engine.free_pages()
    print(json.dumps({
        "model": os.path.abspath(args.model_dir), "dtype": args.dtype, "input_ids": input_ids,
        "request_id": result.request_id, "generated_ids": result.tokens, "text": text,
        "finish_reason": result.finish_reason, "load_seconds": round(load_s, 3), "elapsed": round(elapsed, 6),
        "ttft": None if result.ttft is None else round(result.ttft, 6), "generated_tokens": len(result.tokens),
        "tok/s": round(len(result.tokens) / elapsed, 2) if elapsed > 0 else None,
        "kv_released": all(f == llm.engine.num_pages for f in free) and llm.engine.cache.live_requests == 0,
    }))
    return 0 if result.finish_reason in ("length", "eos") else 1


if __name__ == "__main__":
    sys.exit(main())
