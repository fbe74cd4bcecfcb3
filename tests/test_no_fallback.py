"""There is no CPU path: without a GPU, with host tensors, or without a kernel's source the
product fails with an error that says so; it never computes something else instead."""
import pytest
import torch

from helpers import TINY, make_model_folder


def test_engine_refuses_to_start_without_a_gpu(tmp_path, monkeypatch):
    from llm_inference_lab_b200.engine import Engine
    from llm_inference_lab_b200.kernels.ops import KernelError

    cfg, opt = TINY["A"]
    folder = make_model_folder(str(tmp_path / "model"), cfg, opt["seed"], "float32")
    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    with pytest.raises(KernelError, match="no CPU fallback"):
        Engine(folder, "float32", max_tokens=64)


def test_kernels_refuse_host_tensors():
    from llm_inference_lab_b200.kernels import ops

    ids = torch.zeros(4, dtype=torch.int32)
    table = torch.zeros(8, 16)
    with pytest.raises(ops.KernelError, match="CUDA tensors"):
        ops.embed(ids, table)
    with pytest.raises(ops.KernelError, match="CUDA tensors"):
        ops.add_rmsnorm(torch.zeros(2, 16), torch.ones(16), 1e-6)
    with pytest.raises(ops.KernelError, match="float32 or bfloat16"):
        ops.dtype_code(torch.float16)


def test_a_missing_kernel_source_is_an_error():
    from llm_inference_lab_b200.kernels import build

    with pytest.raises(build.BuildError, match="no kernel source"):
        build.kernel_library("no_such_kernel")
