"""NVTX ranges around the host's submission scopes, for timelines taken with a profiler.

The reference pushes thread-local NVTX ranges named per operator around the code that
submits each operator's kernels, and per step around the whole submission
(rust/engine/src/profiling.rs:4-18; rust/engine/src/runner/model/qwen2/engine.rs:922-935).
Here the scopes are the step (``step.prefill`` / ``step.decode``, by the reference's rule:
a step is a prefill step if any request brings more than one token or holds nothing yet,
engine.rs:862-864), each layer call of the run order (``layer.<index>``), and inside a block
its mixer and feed-forward by kind (``mixer.gqa_attention``, ``feed_forward.gated_mlp``).

Off unless the environment has ``LAB_NVTX=1`` or `enable()` is called: a range that is off
costs one attribute test.  A range marks host time (when the kernels were submitted); the
kernels themselves appear under it in a profiler's timeline by correlation.
"""
from __future__ import annotations

import os

ON = os.environ.get("LAB_NVTX", "") not in ("", "0")


def enable(on: bool = True) -> None:
    global ON
    ON = bool(on)


class scoped_range:
    """``with scoped_range("name"):`` pushes an NVTX range on entry and pops it on exit."""
    __slots__ = ("name", "pushed")

    def __init__(self, name: str):
        self.name = name
        self.pushed = False

    def __enter__(self):
        if ON:
            import torch
            torch.cuda.nvtx.range_push(self.name)
            self.pushed = True
        return self

    def __exit__(self, *exc):
        if self.pushed:
            import torch
            torch.cuda.nvtx.range_pop()
            self.pushed = False
        return False
