"""Generation through the Python entry point and the command line, against the plain
implementation: greedy tokens, temperature sampling with a seed, continuous batching with
portions of prompts, end-of-sequence, and preemption when pages run out."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from helpers import ROOT, TINY, make_model_folder, random_config, random_tokens
from plain_qwen2 import plain_forward, plain_greedy, plain_sample, read_model_folder

pytestmark = pytest.mark.gpu
_folders = {}


def folder_of(tmp_path_factory, name, dtype):
    if (name, dtype) not in _folders:
        cfg, opt = TINY[name]
        f = str(tmp_path_factory.mktemp(f"gen{name}{dtype}"))
        make_model_folder(f, cfg, opt["seed"], dtype)
        _folders[(name, dtype)] = f
    return _folders[(name, dtype)]


def check_teacher_forced(folder, prompt, tokens, temperature, seed, slack):
    """Every generated token is what the plain implementation picks at its position, given the
    tokens before it; where two candidates lie within `slack` of each other either may win."""
    cfg, w = read_model_folder(folder)
    logits = plain_forward(cfg, w, list(prompt) + list(tokens))
    for i, tok in enumerate(tokens):
        pos = len(prompt) + i
        row = logits[pos - 1]
        want, scores = plain_sample(row, temperature, seed, pos)
        if tok != want:
            s = scores if scores is not None else row
            assert abs(s[tok] - s[want]) <= slack, f"token {i}: got {tok}, plain picks {want}"


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_equals_plain_in_32_bit(tmp_path_factory, name):
    from llm_inference_lab_b200.engine.llm import LLM
    from llm_inference_lab_b200.sampling import SamplingConfig

    cfg, opt = TINY[name]
    folder = folder_of(tmp_path_factory, name, "float32")
    rng = np.random.default_rng(0)
    prompts = [random_tokens(rng, n, cfg["vocab_size"]) for n in (5, 9, 17)]
    llm = LLM(folder, "f32", page_size=opt["page_size"], kv_tokens=256, max_requests=4)
    results = llm.generate(prompts, SamplingConfig(max_new_tokens=8, ignore_eos=True))
    pcfg, w = read_model_folder(folder)
    for prompt, res in zip(prompts, results):
        assert res.finish_reason == "length" and res.prompt_tokens == prompt
        assert res.tokens == plain_greedy(pcfg, w, prompt, 8)
    assert llm.engine.cache.live_requests == 0 and llm.engine.free_pages()[0] == llm.engine.num_pages


@pytest.mark.parametrize("graph", [False, True])
def test_prompt_that_fills_the_maximum_length(tmp_path_factory, graph):
    """A prompt of most of the model's positions, generated up to the very last one: the step function
    counts the tokens the scheduler has reserved once, not twice.  One token more is refused."""
    from llm_inference_lab_b200.engine.llm import LLM
    from llm_inference_lab_b200.sampling import SamplingConfig

    cfg, opt = TINY["A"]
    most = cfg["max_position_embeddings"]
    folder = folder_of(tmp_path_factory, "A", "float32")
    rng = np.random.default_rng(4)
    fits = random_tokens(rng, most - 8, cfg["vocab_size"])      # the ninth token is sampled at the last position
    too_long = random_tokens(rng, most - 7, cfg["vocab_size"])
    llm = LLM(folder, "f32", page_size=opt["page_size"], kv_tokens=2 * most, max_requests=4, max_batch_tokens=64,
              cuda_graph=graph)
    a, b = llm.generate([fits, too_long], SamplingConfig(max_new_tokens=9, ignore_eos=True))
    pcfg, w = read_model_folder(folder)
    assert a.finish_reason == "length" and a.tokens == plain_greedy(pcfg, w, fits, 9)
    assert b.finish_reason == "invalid" and "maximum sequence length" in b.message and b.tokens == []
    assert llm.engine.cache.live_requests == 0 and llm.engine.free_pages()[0] == llm.engine.num_pages


@pytest.mark.parametrize("dtype,slack", [("float32", 1e-4), ("bfloat16", 0.25)])
def test_mixed_batch_with_temperature(tmp_path_factory, dtype, slack):
    """Configuration B's workload: four requests with prompts of 1/7/33/70 tokens, portions of at
    most 8 tokens, 12 new tokens each at temperature 0.8 with seed 7."""
    from llm_inference_lab_b200.engine.llm import LLM
    from llm_inference_lab_b200.sampling import SamplingConfig

    cfg, opt = TINY["B"]
    folder = folder_of(tmp_path_factory, "B", dtype)
    rng = np.random.default_rng(1)
    prompts = [random_tokens(rng, n, cfg["vocab_size"]) for n in (1, 7, 33, 70)]
    llm = LLM(folder, dtype, max_batch_tokens=8, page_size=16, kv_tokens=512, max_requests=4)
    sampling = SamplingConfig(max_new_tokens=12, do_sample=True, temperature=0.8, seed=7, ignore_eos=True)
    results = llm.generate(prompts, sampling)
    assert llm.steps > 14, "prompts were cut into portions"
    for prompt, res in zip(prompts, results):
        assert len(res.tokens) == 12
        check_teacher_forced(folder, prompt, res.tokens, 0.8, 7, slack)
    again = llm.generate(prompts[2:3], sampling)[0]
    assert again.tokens == results[2].tokens, "the draw depends on seed and position, not on the batch"
    other = llm.generate(prompts[2:3], SamplingConfig(max_new_tokens=12, do_sample=True, temperature=0.8, seed=8,
                                                      ignore_eos=True))[0]
    assert other.tokens != results[2].tokens


def test_bfloat16_greedy_is_near_plain(tmp_path_factory):
    from llm_inference_lab_b200.engine.llm import LLM
    from llm_inference_lab_b200.sampling import SamplingConfig

    cfg, opt = TINY["C"]
    folder = folder_of(tmp_path_factory, "C", "bfloat16")
    prompts = [random_tokens(np.random.default_rng(2), n, cfg["vocab_size"]) for n in (3, 40, 64)]
    llm = LLM(folder, "bf16", page_size=8, kv_tokens=512, max_requests=4, max_batch_tokens=16)
    for prompt, res in zip(prompts, llm.generate(prompts, SamplingConfig(max_new_tokens=30))):
        check_teacher_forced(folder, prompt, res.tokens, 0.0, 0, 0.2)


@pytest.mark.parametrize("name,requests", [("F", 130), ("G", 200)])
@pytest.mark.parametrize("graph", [False, True])
def test_bfloat16_decoding_of_many_requests_at_once(tmp_path_factory, name, requests, graph):
    """Decode steps of 128 rows and more take other routes than small ones (the rotation reads its
    angles from a table that the step's layers share, the products run with tokens on the 128-row
    side): eagerly and from CUDA graphs, whose captured kernels must fill that table themselves in every
    replay.  Every token is near the plain implementation's best at its position."""
    from llm_inference_lab_b200.engine.llm import LLM
    from llm_inference_lab_b200.kernels import ops
    from llm_inference_lab_b200.sampling import SamplingConfig

    cfg, opt = TINY[name]
    folder = folder_of(tmp_path_factory, name, "bfloat16")
    rng = np.random.default_rng(31)
    prompts = [random_tokens(rng, int(rng.integers(1, 12)), cfg["vocab_size"]) for _ in range(requests)]
    llm = LLM(folder, "bf16", page_size=opt["page_size"], kv_tokens=requests * 32, max_requests=requests,
              cuda_graph=graph)
    results = llm.generate(prompts, SamplingConfig(max_new_tokens=6, ignore_eos=True))
    ops.take_device_errors()
    if graph:
        assert any(rows >= 128 for rows, _ in llm.graphs.cached), "no decode step of 128 rows or more"
    for i in range(0, requests, 7):
        check_teacher_forced(folder, prompts[i], results[i].tokens, 0.0, 0, 0.2)
    assert llm.engine.cache.live_requests == 0


def test_eos_and_options(tmp_path_factory):
    from llm_inference_lab_b200.engine.llm import LLM
    from llm_inference_lab_b200.sampling import SamplingConfig

    cfg, opt = TINY["B"]
    folder = folder_of(tmp_path_factory, "B", "float32")
    prompt = random_tokens(np.random.default_rng(3), 6, cfg["vocab_size"])
    llm = LLM(folder, "f32", kv_tokens=256, max_requests=2)
    free = llm.generate([prompt], SamplingConfig(max_new_tokens=6))[0].tokens
    stop = llm.generate([prompt], SamplingConfig(max_new_tokens=6, eos_token_id=free[2]))[0]
    assert stop.tokens == free[:3] and stop.finish_reason == "eos", "the end token is returned and counted"
    assert llm.generate([prompt], SamplingConfig())[0].tokens == free[:1], "max_new_tokens defaults to 1"
    with pytest.raises(ValueError, match="top_k"):
        llm.generate([prompt], SamplingConfig(top_k=5))
    bad = llm.generate([[cfg["vocab_size"]], prompt], SamplingConfig(max_new_tokens=2))
    assert bad[0].finish_reason == "invalid" and bad[1].tokens == free[:2], "an invalid peer does not stop the others"
    assert llm.engine.cache.live_requests == 0


def test_pages_run_out_preempt_and_recompute(tmp_path_factory):
    """Optimistic admission with a pool too small for all: requests are preempted and recomputed,
    and every request still gets the tokens it gets alone."""
    from llm_inference_lab_b200.engine.llm import LLM
    from llm_inference_lab_b200.sampling import SamplingConfig

    cfg, opt = TINY["A"]
    folder = folder_of(tmp_path_factory, "A", "float32")
    rng = np.random.default_rng(4)
    prompts = [random_tokens(rng, n, cfg["vocab_size"]) for n in (20, 24, 9, 30)]
    sampling = SamplingConfig(max_new_tokens=20, ignore_eos=True)
    roomy = LLM(folder, "f32", page_size=4, kv_tokens=1024, max_requests=4)
    alone = [r.tokens for r in roomy.generate(prompts, sampling)]
    tight = LLM(folder, "f32", page_size=4, kv_tokens=112, max_requests=4, reserve_future=False, max_batch_tokens=32)
    results = tight.generate(prompts, sampling)
    assert tight.scheduler.preemptions >= 1 and sum(r.preemptions for r in results) >= 1
    assert [r.tokens for r in results] == alone
    assert tight.engine.cache.live_requests == 0 and tight.engine.free_pages()[0] == tight.engine.num_pages
    # with reservation (the default) the same pool makes requests wait instead
    waiting = LLM(folder, "f32", page_size=4, kv_tokens=112, max_requests=4, max_batch_tokens=32)
    assert [r.tokens for r in waiting.generate(prompts, sampling)] == alone and waiting.scheduler.preemptions == 0


def test_command_line(tmp_path_factory):
    cfg, opt = TINY["A"]
    folder = folder_of(tmp_path_factory, "A", "float32")
    prompt = random_tokens(np.random.default_rng(5), 7, cfg["vocab_size"])
    cmd = [sys.executable, "-m", "llm_inference_lab_b200.cli", "--model-dir", folder, "--dtype", "f32",
           "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "5", "--repeat", "2", "--trace-steps"]
    proc = subprocess.run(cmd, capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    line = json.loads(proc.stdout.strip().splitlines()[-1])
    pcfg, w = read_model_folder(folder)
    expect = plain_greedy(pcfg, w, prompt, 5, eos=[255])
    assert line["generated_ids"] == expect and line["kv_released"] is True and line["input_ids"] == prompt
    assert line["dtype"] == "f32" and line["generated_tokens"] == len(expect)
    steps = [json.loads(s) for s in proc.stderr.splitlines() if s.startswith('{"event"')]
    assert len(steps) >= len(expect)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_lookahead_decoding_gives_the_same_tokens(tmp_path_factory, dtype):
    """Decode steps launched ahead of the host (the device feeds the sampled ids forward) give what
    step-by-step decoding gives: greedy and with temperature, requests of different lengths that end
    by length and by their end-of-sequence token at different steps, more requests than slots."""
    from llm_inference_lab_b200.engine.llm import LLM
    from llm_inference_lab_b200.sampling import SamplingConfig

    cfg, opt = TINY["B"]
    folder = folder_of(tmp_path_factory, "B", dtype)
    rng = np.random.default_rng(11)
    prompts = [random_tokens(rng, n, cfg["vocab_size"]) for n in (3, 17, 8, 30, 1, 12)]
    short = "f32" if dtype == "float32" else "bf16"
    outs = {}
    for ahead in (False, True):
        llm = LLM(folder, short, page_size=opt["page_size"], kv_tokens=512, max_requests=4, cuda_graph=True,
                  lookahead=ahead)
        free = llm.generate(prompts, SamplingConfig(max_new_tokens=24, ignore_eos=True))
        if dtype == "float32":
            pcfg, w = read_model_folder(folder)
            for prompt, res in zip(prompts, free):
                assert res.tokens == plain_greedy(pcfg, w, prompt, 24), "graphs and lookahead against the plain model"
        # end tokens taken from the free run: every request stops somewhere in the middle
        configs = [SamplingConfig(max_new_tokens=5 + 4 * i, eos_token_id=free[i].tokens[3 + i], temperature=0.7,
                                  do_sample=(i % 2 == 1), seed=5 + i) for i in range(len(prompts))]
        stopped = llm.generate(prompts, configs)
        outs[ahead] = ([r.tokens for r in free], [(r.tokens, r.finish_reason) for r in stopped])
        assert llm.engine.cache.live_requests == 0 and llm.engine.free_pages()[0] == llm.engine.num_pages
        llm.engine.cache.check_consistency()
        if ahead:
            assert llm.graphs.replays > 20
        # batches of three ran from the graph of four, with a request of length zero beside them
        assert {k[0] for k in llm.graphs.cached} <= {1, 2, 4}
    assert outs[True] == outs[False]
    assert any(reason == "eos" for _, reason in outs[True][1]) and any(reason == "length" for _, reason in outs[True][1])


def test_temperatures_and_seeds_follow_a_batch_from_graph_to_graph(tmp_path_factory):
    """Decode graphs are captured per context bucket, each with buffers of its own: when a batch's
    longest context crosses a bucket's edge (256 tokens), its temperatures and seeds must move to the
    next graph with it, and a greedy batch that later uses a graph must not inherit them."""
    from llm_inference_lab_b200.engine.llm import LLM
    from llm_inference_lab_b200.sampling import SamplingConfig

    cfg, opt = TINY["B"]
    cfg = dict(cfg, max_position_embeddings=512)
    folder = str(tmp_path_factory.mktemp("genB512"))
    make_model_folder(folder, cfg, opt["seed"], "float32")
    rng = np.random.default_rng(21)
    prompts = [random_tokens(rng, n, cfg["vocab_size"]) for n in (246, 240, 250)]
    hot = SamplingConfig(max_new_tokens=20, do_sample=True, temperature=0.8, seed=13, ignore_eos=True)
    cold = SamplingConfig(max_new_tokens=20, ignore_eos=True)
    outs = {}
    for graph in (False, True):
        llm = LLM(folder, "f32", page_size=16, kv_tokens=1024, max_requests=4, max_batch_tokens=512, cuda_graph=graph)
        first = [r.tokens for r in llm.generate(prompts, hot)]
        second = [r.tokens for r in llm.generate(prompts, cold)]     # same batch size, same graphs, greedy
        third = [r.tokens for r in llm.generate(prompts, hot)]
        outs[graph] = (first, second, third)
        if graph:
            assert len(llm.graphs.cached) >= 2, "the batch crossed from one context bucket to the next"
    assert outs[True] == outs[False]
    assert outs[True][0] == outs[True][2] and outs[True][0] != outs[True][1]
    pcfg, w = read_model_folder(folder)
    for prompt, tokens in zip(prompts, outs[True][1]):
        assert tokens == plain_greedy(pcfg, w, prompt, 20)
    for prompt, tokens in zip(prompts, outs[True][0]):
        check_teacher_forced(folder, prompt, tokens, 0.8, 13, 1e-4)


@pytest.mark.parametrize("trial", range(int(os.environ.get("LAB_RANDOM_GENERATE", "12"))))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_generation_schedules(tmp_path, trial, dtype):
    """Random configurations, pool sizes, token budgets and options through `LLM.generate`:
    with and without reservation (so some runs preempt and recompute), decode graphs, lookahead, an
    end-of-sequence id, requests that arrive in a second call while nothing of the first is left.
    In 32-bit the greedy tokens equal the plain implementation's.  In bfloat16 (one layer; eager decode
    steps then run as the persistent stack kernel where the sizes allow) every token lies as near the
    plain implementation's best at its position as rounding allows: within four times the largest error
    of the plain implementation's bfloat16 twin on the same sequence.  Every page comes back.  (An
    earlier, longer run of this generator found that the step function counted the scheduler's reserved
    tokens twice.)  LAB_RANDOM_GENERATE=200 in the environment runs that many trials instead of twelve."""
    from plain_qwen2 import plain_precision, round_bfloat16
    from llm_inference_lab_b200.engine.llm import LLM
    from llm_inference_lab_b200.sampling import SamplingConfig

    rng = np.random.default_rng(9000 + trial)
    cfg, page = random_config(rng, layers=None if dtype == "float32" else 1)
    cfg["max_position_embeddings"] = min(cfg["max_position_embeddings"], 200)
    vocab = cfg["vocab_size"]
    prompts, news = [], []
    for _ in range(int(rng.integers(1, 7))):
        n_new = int(rng.integers(0, 20))
        prompts.append(random_tokens(rng, int(rng.integers(1, cfg["max_position_embeddings"] - n_new)), vocab))
        news.append(n_new)
    eos = int(rng.integers(0, vocab)) if rng.random() < 0.5 else None
    cfg["eos_token_id"] = eos
    graph, ahead, reserve = bool(rng.random() < 0.6), bool(rng.random() < 0.7), bool(rng.random() < 0.5)
    rounded = [-(-(len(p) + n) // page) * page for p, n in zip(prompts, news)]
    kv_tokens = int(rng.integers(max(rounded), max(sum(rounded), max(rounded)) + 1))
    folder = make_model_folder(str(tmp_path / "m"), cfg, trial, dtype)
    pcfg, w = read_model_folder(folder)
    llm = LLM(folder, dtype, max_batch_tokens=int(rng.choice([8, 16, 64, 512])), kv_tokens=kv_tokens, page_size=page,
              max_requests=8, reserve_future=reserve, cuda_graph=graph, lookahead=ahead)
    results = llm.generate(prompts, [SamplingConfig(max_new_tokens=n) for n in news])
    late = llm.generate(prompts[:2], [SamplingConfig(max_new_tokens=n) for n in news[:2]])
    what = f"page {page}, pool {kv_tokens}, graph {graph}, lookahead {ahead}, reservation {reserve}"
    for prompt, n, res in zip(prompts + prompts[:2], news + news[:2], results + late):
        if dtype == "float32":
            assert res.tokens == plain_greedy(pcfg, w, prompt, n, eos=() if eos is None else (eos,)), what
            continue
        assert len(res.tokens) <= n and (len(res.tokens) == n or res.tokens[-1] == eos), what
        assert eos not in res.tokens[:-1], what
        if not res.tokens:
            continue
        ids = prompt + res.tokens[:-1]
        rows = plain_forward(pcfg, w, ids)[len(prompt) - 1:]
        with plain_precision(edge=round_bfloat16):
            noise = float(np.abs(np.asarray(plain_forward(pcfg, w, ids), dtype=np.float64)[len(prompt) - 1:] - rows).max())
        for i, tok in enumerate(res.tokens):
            assert rows[i].max() - rows[i][tok] <= 4 * noise, f"token {i} lies {rows[i].max() - rows[i][tok]:.3e} below the best ({what})"
    llm.engine.cache.check_consistency()
    assert llm.engine.cache.live_requests == 0 and llm.engine.free_pages() == [llm.engine.num_pages] * \
        llm.engine.cache.num_groups, what
