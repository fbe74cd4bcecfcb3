"""The profiling ranges: off by default and then silent; when on, pushed and popped in pairs around
the step's scopes, named by layer call and by part kind (no GPU: NVTX is replaced by a recorder)."""
import types

import pytest
import torch

from llm_inference_lab_b200 import profiling


@pytest.fixture
def recorder(monkeypatch):
    events = []
    monkeypatch.setattr(torch.cuda.nvtx, "range_push", lambda name: events.append(("push", name)))
    monkeypatch.setattr(torch.cuda.nvtx, "range_pop", lambda: events.append(("pop",)))
    monkeypatch.setattr(profiling, "ON", True)
    return events


def test_ranges_are_silent_when_off(monkeypatch):
    calls = []
    monkeypatch.setattr(torch.cuda.nvtx, "range_push", lambda name: calls.append(name))
    monkeypatch.setattr(profiling, "ON", False)
    with profiling.scoped_range("quiet"):
        pass
    assert calls == []


def test_ranges_pair_up_and_survive_exceptions(recorder):
    with profiling.scoped_range("outer"):
        with pytest.raises(RuntimeError):
            with profiling.scoped_range("inner"):
                raise RuntimeError("boom")
    assert recorder == [("push", "outer"), ("push", "inner"), ("pop",), ("pop",)]


class _Stub:
    def __init__(self, kind):
        self.spec = types.SimpleNamespace(kind=kind)

    def forward(self, x, *rest):
        return x

    def forward_add(self, x, delta, rows=None):
        return x


def test_block_and_model_name_their_scopes(recorder):
    from llm_inference_lab_b200.models.builder import CausalLM
    from llm_inference_lab_b200.parts.block import PreNormBlock
    from llm_inference_lab_b200.parts.spec import LayerCall

    blocks = [PreNormBlock(_Stub("toy_mixer"), _Stub("toy_ffn"), [_Stub("n"), _Stub("n")]) for _ in range(2)]
    model = CausalLM.__new__(CausalLM)
    model.embedding, model.final_norm, model.head, model.blocks = _Stub("e"), _Stub("n"), _Stub("h"), blocks
    model.order = (LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2))       # layer 0 named twice
    model.range_names = [f"layer.{c.layer}" for c in model.order]
    ctx = types.SimpleNamespace(token_ids=torch.zeros(3))
    caches = [types.SimpleNamespace(write=True)] * 3
    out = model.forward(ctx, caches, torch.tensor([2]))
    assert out is not None
    pushes = [e[1] for e in recorder if e[0] == "push"]
    per_layer = ["mixer.toy_mixer", "feed_forward.toy_ffn"]
    assert pushes == (["embedding", "layer.0"] + per_layer + ["layer.1"] + per_layer + ["layer.0"] + per_layer
                      + ["final_norm+head"])
    assert sum(e[0] == "pop" for e in recorder) == len(pushes)
    depth = 0
    for e in recorder:
        depth += 1 if e[0] == "push" else -1
        assert 0 <= depth <= 2
    assert depth == 0
