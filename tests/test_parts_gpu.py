"""Each part of a layer alone against the plain function of the same part, and the proof that
the framework takes new kinds of parts without a change to its files: a toy mixer with a state
of its own, a toy feed-forward with routing, a toy position encoding, and the toy architectures
that use them beside the framework's parts, all defined here."""
import dataclasses

import numpy as np
import pytest
import torch

from helpers import TINY, make_model_folder, random_tokens
from plain_qwen2 import (plain_attention_part, plain_block, plain_embedding, plain_gated_mlp, plain_linear,
                         plain_rms_norm, read_model_folder)

pytestmark = pytest.mark.gpu


def engine_and_ctx(tmp_path, name, dtype, lengths):
    """An engine of a tiny configuration and the context of one step that holds whole prompts."""
    from llm_inference_lab_b200.engine import Engine, Entry

    cfg, opt = TINY[name]
    folder = make_model_folder(str(tmp_path / f"{name}{dtype}"), cfg, opt["seed"], dtype)
    engine = Engine(folder, dtype, max_tokens=512, page_size=opt["page_size"], max_requests=4)
    rng = np.random.default_rng(0)
    entries = [Entry(i, random_tokens(rng, n, cfg["vocab_size"]), [n - 1]) for i, n in enumerate(lengths)]
    for e in entries:
        engine.open(e.request)
        engine.cache.reserve(e.request, len(e.tokens))
    ctx, rows = engine._pack(entries)
    return engine, folder, cfg, ctx, rows, entries


def close(a, b, dtype):
    a = a.double().cpu().numpy()
    err = np.abs(a - b).max() / max(np.abs(b).max(), 1e-30)
    assert np.isfinite(a).all() and err < (2e-5 if dtype == "float32" else 3e-2), err


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_parts_alone(tmp_path, name, dtype):
    lengths = [19, 6, 33]
    engine, folder, cfg, ctx, rows, entries = engine_and_ctx(tmp_path, name, dtype, lengths)
    pcfg, w = read_model_folder(folder)
    model = engine.model
    T, H = sum(lengths), cfg["hidden_size"]
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    g = torch.Generator().manual_seed(1)
    x = torch.randn(T, H, generator=g).to(tdt)
    xd = x.double().numpy()
    bounds = np.concatenate([[0], np.cumsum(lengths)])

    # embedding
    ids = np.concatenate([e.tokens for e in entries])
    assert torch.equal(model.embedding.forward(ctx.token_ids).cpu(),
                       torch.from_numpy(plain_embedding(ids, w["model.embed_tokens.weight"])).to(tdt))
    # norm, alone and fused with the residual add
    block = model.blocks[-1]
    layer = len(model.blocks) - 1
    p = f"model.layers.{layer}."
    close(block.norms[0].forward(x.cuda()), plain_rms_norm(xd, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"]),
          dtype)
    delta = torch.randn(T, H, generator=g).to(tdt)
    xs = x.clone().cuda()
    y = block.norms[1].forward_add(xs, delta.cuda())
    summed = (x.float() + delta.float()).to(tdt)
    assert torch.equal(xs.cpu(), summed)
    close(y, plain_rms_norm(summed.double().numpy(), w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"]),
          dtype)
    # feed-forward
    close(block.ffn.forward(x.cuda(), ctx),
          plain_gated_mlp(xd, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"]),
          dtype)
    # mixer: attention of whole prompts, each request on its own
    view = engine.views[layer]
    out = block.mixer.forward(x.cuda(), ctx, view)
    if out.dim() == 3:
        out = out.sum(0)
    window = cfg["sliding_window"] if cfg.get("use_sliding_window") and layer >= cfg["max_window_layers"] else 0
    want = np.concatenate([plain_attention_part(xd[a:b], w, p + "self_attn.", pcfg, np.arange(b - a), window)
                           for a, b in zip(bounds[:-1], bounds[1:])])
    close(out, want, dtype)
    # whole block: residual stream in, (residual, pending product) out
    xs = x.clone().cuda()
    res, pending = block.forward(xs, None, ctx, view)
    if pending.dim() == 3:
        pending = pending.sum(0)
    want = np.concatenate([plain_block(xd[a:b], w, layer, pcfg, np.arange(b - a))
                           for a, b in zip(bounds[:-1], bounds[1:])])
    close(res.float() + pending.float(), want, dtype)
    # head at gathered rows
    h = torch.randn(3, H, generator=g).to(tdt)
    head_w = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    logits = model.head.forward(h.cuda())
    assert logits.dtype == torch.float32
    close(logits, plain_linear(h.double().numpy(), head_w), "float32" if dtype == "float32" else "bfloat16")


# ----------------------------------------------------------------------------------------
# A toy mixer with a state of its own, and a toy architecture, defined in this test only.
# ----------------------------------------------------------------------------------------

def define_toy():
    from llm_inference_lab_b200 import register_architecture
    from llm_inference_lab_b200.config.base import ModelConfig, optional, positive, required
    from llm_inference_lab_b200.parts import (FixedState, LayerCall, LayerSpec, Mixer, ModelBlueprint, PartSpec,
                                              TensorSpec, register_part)

    class RunningMean(Mixer):
        """out[t] = w * mean(x[0..t]): the state per request is the running sum and the count."""

        @classmethod
        def tensors(cls, spec):
            return [TensorSpec(spec.prefix + "mix.weight", (spec["hidden"],), init="norm")]

        @classmethod
        def cache_need(cls, spec):
            return FixedState((spec["hidden"] + 1,))

        def __init__(self, spec, weights, dtype, device):
            super().__init__(spec, weights, dtype, device)
            self.w = self._weight(weights, "mix.weight").float()
            self.h = spec["hidden"]

        def forward(self, x, ctx, cache):
            out = torch.empty_like(x)
            at = 0
            for n, slot in zip(ctx.q_lens, ctx.state_slots):
                state = cache.state[slot]
                sums = state[: self.h] + torch.cumsum(x[at: at + n].float(), dim=0)
                counts = state[self.h] + torch.arange(1, n + 1, device=x.device, dtype=torch.float32)
                out[at: at + n] = (sums / counts[:, None] * self.w).to(x.dtype)
                if cache.write:
                    state[: self.h] = sums[-1]
                    state[self.h] = counts[-1]
                at += n
            return out

    register_part("mixer", "running_mean", RunningMean)

    @dataclasses.dataclass
    class ToyConfig(ModelConfig):
        architecture = "ToyStateLM"
        vocab_size: int = required(int, positive)
        hidden_size: int = required(int, positive)
        num_layers: int = required(int, positive)
        inner_size: int = required(int, positive)
        heads: int = optional(int, 2)
        eps: float = optional(float, 1e-5)
        max_positions: int = optional(int, 256)

    def blueprint(cfg):
        layers = []
        for i in range(cfg.num_layers):
            p = f"blocks.{i}."
            if i % 2 == 0:
                mixer = PartSpec("running_mean", {"hidden": cfg.hidden_size}, prefix=p)
            else:
                mixer = PartSpec("gqa_attention", {
                    "hidden": cfg.hidden_size, "n_heads": cfg.heads, "n_kv_heads": 1,
                    "head_dim": cfg.hidden_size // cfg.heads, "qkv_bias": False, "out_bias": False, "window": 0,
                    "position": PartSpec("none", {})}, prefix=p + "attn.")
            ffn = PartSpec("gated_mlp", {"hidden": cfg.hidden_size, "intermediate": cfg.inner_size, "act": "silu"},
                           prefix=p + "ff.")
            norms = tuple(PartSpec("rmsnorm", {"hidden": cfg.hidden_size, "eps": cfg.eps}, prefix=p + f"n{j}.")
                          for j in range(2))
            layers.append(LayerSpec("prenorm", mixer, ffn, norms, hidden=cfg.hidden_size))
        # layer 0 runs a second time at the end, with a state of its own (cache id num_layers)
        order = tuple(LayerCall(i, i) for i in range(cfg.num_layers)) + (LayerCall(0, cfg.num_layers),)
        return ModelBlueprint(
            hidden=cfg.hidden_size, vocab=cfg.vocab_size,
            embedding=PartSpec("token_embedding", {"vocab": cfg.vocab_size, "hidden": cfg.hidden_size}, prefix="emb."),
            layers=tuple(layers), order=order,
            final_norm=PartSpec("rmsnorm", {"hidden": cfg.hidden_size, "eps": cfg.eps}, prefix="out_norm."),
            head=PartSpec("linear_head", {"vocab": cfg.vocab_size, "hidden": cfg.hidden_size, "tied_to": "emb.weight"},
                          prefix="head."),
            max_positions=cfg.max_positions)

    register_architecture("ToyStateLM", ToyConfig, blueprint)
    return ToyConfig


def toy_reference(folder, ids):
    """The toy model on one whole sequence, in plain NumPy."""
    from plain_qwen2 import plain_attention
    import json
    cfg = json.load(open(f"{folder}/config.json"))
    _, w = read_model_folder(folder)
    H, heads = cfg["hidden_size"], cfg["heads"]
    x = w["emb.weight"][np.asarray(ids)]
    T = len(ids)

    def run(i, x):
        p = f"blocks.{i}."
        h = plain_rms_norm(x, w[p + "n0.weight"], cfg["eps"])
        if i % 2 == 0:
            a = np.cumsum(h, axis=0) / np.arange(1, T + 1)[:, None] * w[p + "mix.weight"]
        else:
            d = H // heads
            q = plain_linear(h, w[p + "attn.q_proj.weight"]).reshape(T, heads, d)
            k = plain_linear(h, w[p + "attn.k_proj.weight"]).reshape(T, 1, d)
            v = plain_linear(h, w[p + "attn.v_proj.weight"]).reshape(T, 1, d)
            a = plain_linear(plain_attention(q, k, v, np.arange(T)).reshape(T, H), w[p + "attn.o_proj.weight"])
        r = x + a
        return r + plain_gated_mlp(plain_rms_norm(r, w[p + "n1.weight"], cfg["eps"]), w[p + "ff.gate_proj.weight"],
                                   w[p + "ff.up_proj.weight"], w[p + "ff.down_proj.weight"])

    for i in list(range(cfg["num_layers"])) + [0]:
        x = run(i, x)
    return plain_linear(plain_rms_norm(x, w["out_norm.weight"], cfg["eps"]), w["emb.weight"])


def test_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    from llm_inference_lab_b200.engine import Engine, Entry
    from llm_inference_lab_b200.weights import write_random_model

    ToyConfig = define_toy()
    cfg = ToyConfig.from_dict(dict(vocab_size=97, hidden_size=32, num_layers=3, inner_size=48, heads=2))
    folder = write_random_model(cfg, str(tmp_path / "toy"), seed=3, dtype=torch.float32, std=0.08)
    engine = Engine(folder, "float32", max_tokens=256, page_size=8, max_requests=3)
    plan = engine.model.cache_plan
    assert [type(n).__name__ for n in plan.needs] == ["FixedState", "PagedKV", "FixedState", "FixedState"]
    rng = np.random.default_rng(0)
    seqs = {0: random_tokens(rng, 37, 97), 1: random_tokens(rng, 12, 97)}
    want = {k: toy_reference(folder, ids) for k, ids in seqs.items()}
    got = {k: [] for k in seqs}
    # request 0 in portions of changing size beside request 1 token by token
    cuts0 = [5, 2, 9, 1, 1, 7, 3, 9]
    at0 = at1 = 0
    for n0 in cuts0:
        entries = [Entry(0, seqs[0][at0: at0 + n0], list(range(n0)))]
        if at1 < len(seqs[1]):
            entries.append(Entry(1, seqs[1][at1: at1 + 1], [0]))
        logits = engine.step(entries).cpu().numpy()
        got[0].append(logits[:n0])
        if len(entries) == 2:
            got[1].append(logits[n0:])
            at1 += 1
        at0 += n0
    assert at0 == 37
    engine.close(0)
    while at1 < len(seqs[1]):   # request 1 goes on alone; a new request takes request 0's state slot
        entries = [Entry(1, seqs[1][at1: at1 + 1], [0])]
        if at1 == 9:
            entries.append(Entry(2, seqs[0][:4], [3]))
        logits = engine.step(entries).cpu().numpy()
        got[1].append(logits[:1])
        if len(entries) == 2:
            assert np.abs(logits[1] - want[0][3]).max() < 1e-4, "a state slot used again starts from zero"
        at1 += 1
    for k in seqs:
        err = np.abs(np.concatenate(got[k]) - want[k]).max()
        assert err < 1e-4, (k, err)
    engine.close(1), engine.close(2)
    assert engine.cache.free_state_slots == 3


def toy_greedy(folder, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(np.argmax(toy_reference(folder, ids)[-1])))
    return ids[len(prompt):]


@pytest.mark.parametrize("graph", [False, True])
def test_toy_state_survives_the_scheduler(tmp_path, graph):
    """The toy architecture through `LLM.generate`: more requests than state slots, so slots are used
    again (whoever opened the request, its state starts from zero); prompts cut into portions; a pool
    so tight that a request is preempted and recomputed (its state starts over); with `cuda_graph`
    asked for, which a model with state of its own declines.  Greedy tokens equal the NumPy toy's."""
    from llm_inference_lab_b200.engine.llm import LLM
    from llm_inference_lab_b200.sampling import SamplingConfig
    from llm_inference_lab_b200.weights import write_random_model

    ToyConfig = define_toy()
    cfg = ToyConfig.from_dict(dict(vocab_size=97, hidden_size=32, num_layers=3, inner_size=48, heads=2))
    folder = write_random_model(cfg, str(tmp_path / "toy"), seed=5, dtype=torch.float32, std=0.08)
    rng = np.random.default_rng(1)
    prompts = [random_tokens(rng, n, 97) for n in (11, 3, 20, 7, 15)]
    want = [toy_greedy(folder, p, 10) for p in prompts]
    sampling = SamplingConfig(max_new_tokens=10, ignore_eos=True)
    llm = LLM(folder, "f32", page_size=4, kv_tokens=256, max_requests=2, max_batch_tokens=6, cuda_graph=graph)
    assert llm.engine.stateful and llm.graphs is None
    assert [r.tokens for r in llm.generate(prompts, sampling)] == want
    assert [r.tokens for r in llm.generate(prompts[::-1], sampling)] == want[::-1], "slots left dirty by the first run"
    tight = LLM(folder, "f32", page_size=4, kv_tokens=56, max_requests=3, max_batch_tokens=8, reserve_future=False,
                cuda_graph=graph)
    results = tight.generate(prompts, sampling)
    assert tight.scheduler.preemptions >= 1
    assert [r.tokens for r in results] == want
    for x in (llm, tight):
        assert x.engine.cache.live_requests == 0 and x.engine.free_pages()[0] == x.engine.num_pages
        x.engine.cache.check_consistency()


def test_a_failed_step_leaves_state_and_pages_as_they_were(tmp_path):
    """A step that fails after its mixers have advanced their state (here: the head raises) gives its
    pages back and puts the state of its requests back, so the same step can be run again."""
    from llm_inference_lab_b200.engine import Engine, Entry
    from llm_inference_lab_b200.engine.decode_graph import DecodeGraphs
    from llm_inference_lab_b200.weights import write_random_model

    ToyConfig = define_toy()
    cfg = ToyConfig.from_dict(dict(vocab_size=97, hidden_size=32, num_layers=3, inner_size=48, heads=2))
    folder = write_random_model(cfg, str(tmp_path / "toy"), seed=6, dtype=torch.float32, std=0.08)
    engine = Engine(folder, "float32", max_tokens=128, page_size=4, max_requests=3)
    with pytest.raises(ValueError, match="fixed-size per-request state"):
        DecodeGraphs(engine)
    rng = np.random.default_rng(2)
    a, b = random_tokens(rng, 14, 97), random_tokens(rng, 9, 97)
    engine.step([Entry(0, a[:6], []), Entry(1, b[:5], [])])
    free, states = engine.free_pages(), [v.state.clone() for v in engine.views if v.state is not None]
    head = engine.model.head.forward

    def broken(x):
        raise RuntimeError("the head fails")

    engine.model.head.forward = broken
    with pytest.raises(RuntimeError, match="the head fails"):
        engine.step([Entry(0, a[6:11], [4]), Entry(1, b[5:6], [0]), Entry(2, a[:3], [2])])
    engine.model.head.forward = head
    assert engine.free_pages() == free and not engine.has(2) and engine.length(0) == 6 and engine.length(1) == 5
    assert all(torch.equal(s, v.state) for s, v in zip(states, [v for v in engine.views if v.state is not None]))
    logits = engine.step([Entry(0, a[6:11], [4]), Entry(1, b[5:6], [0]), Entry(2, a[:3], [2])]).cpu().numpy()
    for row, (ids, pos) in zip(logits, [(a, 10), (b, 5), (a, 2)]):
        assert np.abs(row - toy_reference(folder, ids[: pos + 1])[pos]).max() < 1e-4
    engine.cache.check_consistency()


# ----------------------------------------------------------------------------------------
# A toy feed-forward with routing and a toy position encoding, again defined here only.
# ----------------------------------------------------------------------------------------

def define_toy_routed():
    from llm_inference_lab_b200 import register_architecture
    from llm_inference_lab_b200.config.base import ModelConfig, optional, positive, required
    from llm_inference_lab_b200.kernels import ops
    from llm_inference_lab_b200.parts import (FeedForward, LayerCall, LayerSpec, ModelBlueprint, PartSpec,
                                              PositionEncoding, TensorSpec, register_part)

    class Top1Experts(FeedForward):
        """Each token goes to the expert with the largest router logit (32-bit); the expert is a gated
        MLP and its output is weighted with the softmax probability of that logit."""

        @classmethod
        def tensors(cls, spec):
            h, i, p = spec["hidden"], spec["intermediate"], spec.prefix
            out = [TensorSpec(p + "router.weight", (spec["experts"], h))]
            for e in range(spec["experts"]):
                out += [TensorSpec(p + f"experts.{e}.gate_up.weight", (2 * i, h)),
                        TensorSpec(p + f"experts.{e}.down.weight", (h, i))]
            return out

        def __init__(self, spec, weights, dtype, device):
            super().__init__(spec, weights, dtype, device)
            self.router = self._weight(weights, "router.weight").contiguous()
            self.experts = [(self._weight(weights, f"experts.{e}.gate_up.weight").contiguous(),
                             self._weight(weights, f"experts.{e}.down.weight").contiguous())
                            for e in range(spec["experts"])]

        def forward(self, x, ctx):
            logits = ops.linear(x, self.router, None, out_f32=True)
            prob, choice = torch.softmax(logits, dim=-1).max(dim=-1)
            out = torch.zeros_like(x)
            for e, (w_gate_up, w_down) in enumerate(self.experts):
                rows = torch.nonzero(choice == e).flatten()
                if rows.numel():
                    y = ops.linear(ops.linear_gated(x[rows].contiguous(), w_gate_up), w_down)
                    out[rows] = (y.float() * prob[rows, None]).to(x.dtype)
            return out

    class StridedRope(PositionEncoding):
        """Rotary encoding whose angle grows `stride` times as fast: position p is encoded as
        p * stride.  It only encodes (here with the framework's rotation kernel and positions of its
        own); the paged store of k and v is the framework's."""

        def __init__(self, spec, weights, dtype, device):
            super().__init__(spec, weights, dtype, device)
            d = int(spec["rotary_dim"])
            inv = np.power(float(spec["theta"]), -2.0 * np.arange(d // 2, dtype=np.float64) / d).astype(np.float32)
            self.inv_freq, self.rotary_dim, self.stride = torch.from_numpy(inv).to(device), d, int(spec["stride"])

        def encode(self, qkv, positions, n_q, n_kv, head_dim):
            ops.rope_kv_write(qkv, positions * self.stride, self.inv_freq, self.rotary_dim, None, None, None, n_q,
                              n_kv, head_dim)

    register_part("feed_forward", "top1_experts", Top1Experts)
    register_part("position", "strided_rope", StridedRope)

    @dataclasses.dataclass
    class ToyRoutedConfig(ModelConfig):
        architecture = "ToyRoutedLM"
        vocab_size: int = required(int, positive)
        hidden_size: int = required(int, positive)
        num_layers: int = required(int, positive)
        inner_size: int = required(int, positive)
        experts: int = optional(int, 3)
        heads: int = optional(int, 2)
        stride: int = optional(int, 3)
        theta: float = optional(float, 100.0)
        eps: float = optional(float, 1e-5)
        max_positions: int = optional(int, 256)

    def blueprint(cfg):
        layers = []
        d = cfg.hidden_size // cfg.heads
        for i in range(cfg.num_layers):
            p = f"blocks.{i}."
            mixer = PartSpec("gqa_attention", {
                "hidden": cfg.hidden_size, "n_heads": cfg.heads, "n_kv_heads": 1, "head_dim": d, "qkv_bias": False,
                "out_bias": False, "window": 0,
                "position": PartSpec("strided_rope", {"rotary_dim": d, "theta": cfg.theta, "stride": cfg.stride})},
                prefix=p + "attn.")
            if i % 2 == 0:
                ffn = PartSpec("top1_experts", {"hidden": cfg.hidden_size, "intermediate": cfg.inner_size,
                                                "experts": cfg.experts}, prefix=p + "moe.")
            else:
                ffn = PartSpec("gated_mlp", {"hidden": cfg.hidden_size, "intermediate": cfg.inner_size,
                                             "act": "silu"}, prefix=p + "ff.")
            norms = tuple(PartSpec("rmsnorm", {"hidden": cfg.hidden_size, "eps": cfg.eps}, prefix=p + f"n{j}.")
                          for j in range(2))
            layers.append(LayerSpec("prenorm", mixer, ffn, norms, hidden=cfg.hidden_size))
        return ModelBlueprint(
            hidden=cfg.hidden_size, vocab=cfg.vocab_size,
            embedding=PartSpec("token_embedding", {"vocab": cfg.vocab_size, "hidden": cfg.hidden_size}, prefix="emb."),
            layers=tuple(layers), order=tuple(LayerCall(i, i) for i in range(cfg.num_layers)),
            final_norm=PartSpec("rmsnorm", {"hidden": cfg.hidden_size, "eps": cfg.eps}, prefix="out_norm."),
            head=PartSpec("linear_head", {"vocab": cfg.vocab_size, "hidden": cfg.hidden_size, "tied_to": None},
                          prefix="head."),
            max_positions=cfg.max_positions)

    register_architecture("ToyRoutedLM", ToyRoutedConfig, blueprint)
    return ToyRoutedConfig


def toy_routed_reference(folder, ids):
    """The routed toy model on one whole sequence, in plain NumPy."""
    import json
    from plain_qwen2 import plain_attention, plain_rope, plain_silu
    cfg = json.load(open(f"{folder}/config.json"))
    _, w = read_model_folder(folder)
    H, heads, T = cfg["hidden_size"], cfg["heads"], len(ids)
    d = H // heads
    x = w["emb.weight"][np.asarray(ids)].astype(np.float64)
    pos = np.arange(T)
    for i in range(cfg["num_layers"]):
        p = f"blocks.{i}."
        h = plain_rms_norm(x, w[p + "n0.weight"], cfg["eps"])
        q = plain_rope(plain_linear(h, w[p + "attn.q_proj.weight"]).reshape(T, heads, d), pos * cfg["stride"], cfg["theta"])
        k = plain_rope(plain_linear(h, w[p + "attn.k_proj.weight"]).reshape(T, 1, d), pos * cfg["stride"], cfg["theta"])
        v = plain_linear(h, w[p + "attn.v_proj.weight"]).reshape(T, 1, d)
        x = x + plain_linear(plain_attention(q, k, v, pos).reshape(T, H), w[p + "attn.o_proj.weight"])
        h = plain_rms_norm(x, w[p + "n1.weight"], cfg["eps"])
        if i % 2 == 0:
            logits = plain_linear(h, w[p + "moe.router.weight"])
            prob = np.exp(logits - logits.max(-1, keepdims=True))
            prob /= prob.sum(-1, keepdims=True)
            y = np.zeros_like(h)
            for t in range(T):
                e = int(np.argmax(logits[t]))
                gu = plain_linear(h[t: t + 1], w[p + f"moe.experts.{e}.gate_up.weight"])
                inner = gu.shape[1] // 2
                y[t] = plain_linear(plain_silu(gu[:, :inner]) * gu[:, inner:], w[p + f"moe.experts.{e}.down.weight"])[0] \
                    * prob[t, e]
            x = x + y
        else:
            x = x + plain_gated_mlp(h, w[p + "ff.gate_proj.weight"], w[p + "ff.up_proj.weight"],
                                    w[p + "ff.down_proj.weight"])
    return plain_linear(plain_rms_norm(x, w["out_norm.weight"], cfg["eps"]), w["head.weight"])


def test_toy_routed_feed_forward_and_position_encoding(tmp_path):
    """A feed-forward with routing and another position encoding register, build and step, whole and in
    portions beside a decoding request, without a change to the framework's files."""
    from llm_inference_lab_b200.engine import Engine, Entry
    from llm_inference_lab_b200.weights import write_random_model

    Config = define_toy_routed()
    cfg = Config.from_dict(dict(vocab_size=61, hidden_size=32, num_layers=3, inner_size=40, experts=3, heads=2))
    folder = write_random_model(cfg, str(tmp_path / "routed"), seed=5, dtype=torch.float32, std=0.2)
    engine = Engine(folder, "float32", max_tokens=256, page_size=8, max_requests=3)
    rng = np.random.default_rng(1)
    seqs = {0: random_tokens(rng, 33, 61), 1: random_tokens(rng, 9, 61)}
    want = {k: toy_routed_reference(folder, ids) for k, ids in seqs.items()}
    whole = engine.step([Entry(7, seqs[0], list(range(33)))]).cpu().numpy()
    engine.close(7)
    assert np.abs(whole - want[0]).max() < 1e-4
    got = {0: [], 1: []}
    at0 = at1 = 0
    for n0 in [4, 9, 2, 1, 8, 3, 6]:
        entries = [Entry(0, seqs[0][at0: at0 + n0], list(range(n0)))]
        if at1 < len(seqs[1]):
            entries.append(Entry(1, seqs[1][at1: at1 + 1], [0]))
        logits = engine.step(entries).cpu().numpy()
        got[0].append(logits[:n0])
        if len(entries) == 2:
            got[1].append(logits[n0:])
            at1 += 1
        at0 += n0
    assert at0 == 33
    for k in (0, 1):
        have = np.concatenate(got[k])
        assert np.abs(have - want[k][: len(have)]).max() < 1e-4, k
    engine.close(0), engine.close(1)


# ----------------------------------------------------------------------------------------
# A run order in which one layer reads the keys and values that another layer cached.
# ----------------------------------------------------------------------------------------

def define_toy_shared_cache():
    from llm_inference_lab_b200 import register_architecture
    from llm_inference_lab_b200.config.base import ModelConfig, optional, positive, required
    from llm_inference_lab_b200.parts import LayerCall, LayerSpec, ModelBlueprint, PartSpec

    @dataclasses.dataclass
    class SharedConfig(ModelConfig):
        architecture = "ToySharedCacheLM"
        vocab_size: int = required(int, positive)
        hidden_size: int = required(int, positive)
        inner_size: int = required(int, positive)
        heads: int = required(int, positive)
        kv_heads: int = required(int, positive)
        head_size: int = required(int, positive)
        theta: float = optional(float, 10000.0)
        eps: float = optional(float, 1e-5)
        max_positions: int = optional(int, 256)

    def blueprint(cfg):
        layers = []
        for i in range(3):
            p = f"blocks.{i}."
            mixer = PartSpec("gqa_attention", {
                "hidden": cfg.hidden_size, "n_heads": cfg.heads, "n_kv_heads": cfg.kv_heads,
                "head_dim": cfg.head_size, "qkv_bias": True, "out_bias": False, "window": 0,
                "position": PartSpec("rope", {"theta": cfg.theta, "rotary_dim": cfg.head_size})}, prefix=p + "attn.")
            ffn = PartSpec("gated_mlp", {"hidden": cfg.hidden_size, "intermediate": cfg.inner_size, "act": "silu"},
                           prefix=p + "ff.")
            norms = tuple(PartSpec("rmsnorm", {"hidden": cfg.hidden_size, "eps": cfg.eps}, prefix=p + f"n{j}.")
                          for j in range(2))
            layers.append(LayerSpec("prenorm", mixer, ffn, norms, hidden=cfg.hidden_size))
        # Layer 2 forms its own queries but attends over what layer 0 cached; it caches nothing.
        order = (LayerCall(0, 0), LayerCall(1, 1), LayerCall(2, 0, write=False))
        return ModelBlueprint(
            hidden=cfg.hidden_size, vocab=cfg.vocab_size,
            embedding=PartSpec("token_embedding", {"vocab": cfg.vocab_size, "hidden": cfg.hidden_size}, prefix="emb."),
            layers=tuple(layers), order=order,
            final_norm=PartSpec("rmsnorm", {"hidden": cfg.hidden_size, "eps": cfg.eps}, prefix="out_norm."),
            head=PartSpec("linear_head", {"vocab": cfg.vocab_size, "hidden": cfg.hidden_size, "tied_to": None},
                          prefix="head."),
            max_positions=cfg.max_positions)

    register_architecture("ToySharedCacheLM", SharedConfig, blueprint)
    return SharedConfig


def toy_shared_reference(folder, ids):
    from plain_qwen2 import plain_attention, plain_rope
    import json
    cfg = json.load(open(f"{folder}/config.json"))
    _, w = read_model_folder(folder)
    n_h, n_kv, d, theta, eps = cfg["heads"], cfg["kv_heads"], cfg["head_size"], cfg["theta"], cfg["eps"]
    T = len(ids)
    pos = np.arange(T)
    x = w["emb.weight"][np.asarray(ids)]
    cached = {}
    for layer, cache, write in ((0, 0, True), (1, 1, True), (2, 0, False)):
        p = f"blocks.{layer}."
        h = plain_rms_norm(x, w[p + "n0.weight"], eps)
        q = plain_rope(plain_linear(h, w[p + "attn.q_proj.weight"], w[p + "attn.q_proj.bias"]).reshape(T, n_h, d),
                       pos, theta)
        if write:
            k = plain_rope(plain_linear(h, w[p + "attn.k_proj.weight"], w[p + "attn.k_proj.bias"]).reshape(T, n_kv, d),
                           pos, theta)
            v = plain_linear(h, w[p + "attn.v_proj.weight"], w[p + "attn.v_proj.bias"]).reshape(T, n_kv, d)
            cached[cache] = (k, v)
        k, v = cached[cache]
        r = x + plain_linear(plain_attention(q, k, v, pos).reshape(T, n_h * d), w[p + "attn.o_proj.weight"])
        x = r + plain_gated_mlp(plain_rms_norm(r, w[p + "n1.weight"], eps), w[p + "ff.gate_proj.weight"],
                                w[p + "ff.up_proj.weight"], w[p + "ff.down_proj.weight"])
    return plain_linear(plain_rms_norm(x, w["out_norm.weight"], eps), w["head.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_layer_reads_the_cache_another_layer_fills(tmp_path, dtype):
    """The run order is data: its third call reads cache 0, which the first call fills, and writes
    nothing.  Whole prompts, portions beside single tokens, and pages used again."""
    from llm_inference_lab_b200.engine import Engine, Entry
    from llm_inference_lab_b200.weights import write_random_model

    Config = define_toy_shared_cache()
    cfg = Config.from_dict(dict(vocab_size=83, hidden_size=48, inner_size=72, heads=4, kv_heads=2, head_size=16))
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = write_random_model(cfg, str(tmp_path / "shared"), seed=11, dtype=tdt, std=0.15)
    engine = Engine(folder, dtype, max_tokens=128, page_size=8, max_requests=3)
    assert len(engine.model.cache_plan.needs) == 2 and len(engine.views) == 2, "three calls, two caches"
    rng = np.random.default_rng(2)
    seqs = {0: random_tokens(rng, 45, 83), 1: random_tokens(rng, 14, 83), 2: random_tokens(rng, 80, 83)}
    want = {k: toy_shared_reference(folder, ids) for k, ids in seqs.items()}

    def ok(have, ref, what):
        have = have.astype(np.float64)
        if dtype == "float32":
            assert np.abs(have - ref).max() < 1e-4, what
        else:
            assert np.abs(have - ref).max() <= 0.12 * np.abs(ref).max(), what

    got = {0: [], 1: []}
    at0 = at1 = 0
    for n0 in [6, 2, 9, 1, 1, 8, 3, 15]:
        entries = [Entry(0, seqs[0][at0: at0 + n0], list(range(n0)))]
        if at1 < len(seqs[1]):
            entries.append(Entry(1, seqs[1][at1: at1 + 1], [0]))
        logits = engine.step(entries).cpu().numpy()
        got[0].append(logits[:n0])
        if len(entries) == 2:
            got[1].append(logits[n0:])
            at1 += 1
        at0 += n0
    assert at0 == 45
    for k in (0, 1):
        have = np.concatenate(got[k])
        ok(have, want[k][: len(have)], f"request {k} in portions")
    engine.close(0), engine.close(1)
    # 80 tokens need 10 of the 16 pages: some of them held request 0's keys a moment ago.
    whole = engine.step([Entry(2, seqs[2], list(range(80)))]).cpu().numpy()
    ok(whole, want[2], "whole prompt on pages used again")
    engine.close(2)
    assert engine.free_pages() == [engine.num_pages]


@pytest.mark.parametrize("name,lengths", [("F", [5, 40, 130, 64, 65, 1, 300, 17, 33, 128, 2, 90, 70, 200, 9, 250]),
                                          ("G", [150, 3, 64])])
def test_decode_stack_equals_the_parts_it_replaces(tmp_path, name, lengths):
    """A decode step of few tokens that is launched kernel by kernel runs its layers as one persistent
    kernel (phases between grid-wide barriers) where the model's layers fit it.  The same steps run part
    by part give the same logits up to bfloat16 rounding, both are the plain implementation's, and the
    fused step is a handful of launches.  Heads of 64 and of 128, a window, batches of 16 and of 3,
    histories that end on page edges, a width that is no multiple of the k-tile."""
    from llm_inference_lab_b200.engine import Engine, Entry
    from llm_inference_lab_b200.kernels import ops
    from llm_inference_lab_b200.models import builder
    from plain_qwen2 import plain_forward

    cfg, opt = TINY[name]
    folder = make_model_folder(str(tmp_path / name), cfg, opt["seed"], "bfloat16")
    rng = np.random.default_rng(3)
    steps = 4
    seqs = [random_tokens(rng, n + steps, cfg["vocab_size"]) for n in lengths]
    outs, launches = {}, {}
    for fused in (False, True):
        builder.USE_DECODE_STACK = fused
        try:
            engine = Engine(folder, "bfloat16", max_tokens=4096, page_size=opt["page_size"], max_requests=len(lengths))
            assert engine.model.decode_stack is not None
            for i, ids in enumerate(seqs):
                engine.step([Entry(i, ids[: lengths[i]], [])])
            got = []
            for s in range(steps):
                before = ops.COUNTER.launches
                logits = engine.step([Entry(i, [ids[lengths[i] + s]], [0]) for i, ids in enumerate(seqs)])
                launches[fused] = ops.COUNTER.launches - before
                got.append(logits.float().cpu().numpy())
            ops.take_device_errors()
            outs[fused] = np.stack(got)           # [steps, requests, vocab]
            for i in range(len(seqs)):
                engine.close(i)
            assert engine.cache.live_requests == 0
        finally:
            builder.USE_DECODE_STACK = True
    assert launches[True] <= 6 < launches[False], launches
    pcfg, w = read_model_folder(folder)
    want = np.stack([np.stack([plain_forward(pcfg, w, ids)[lengths[i] + s] for i, ids in enumerate(seqs)])
                     for s in range(steps)])
    scale = np.abs(want).max()
    for fused in (False, True):
        err = np.abs(outs[fused] - want).max() / scale
        rms = np.sqrt(((outs[fused] - want) ** 2).mean() / (want ** 2).mean())
        assert err < 0.12 and rms < 0.045, (fused, err, rms)
    assert np.abs(outs[True] - outs[False]).max() / scale < 0.08
