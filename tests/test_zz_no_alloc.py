"""The decode-attention entry point that allocates nothing, called through its exported C
symbol the way a caller without a tensor library would, against the ordinary entry point.

Some callers cannot allocate device memory (a plugin in a host that owns the device heap, a
callback during which allocation is forbidden, a real-time loop): for them the scratch of the
split-KV kernel is a fixed array inside the library.  Two calls in a row share that array and
must both be right, whatever the first one left in it.  This file is collected last, so a run
that stops at the first failure has already run every other test.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def make_case(seed, requests, n_q, n_kv, d, ps):
    rng = np.random.default_rng(seed)
    blocks = [-(-kv // ps) for kv in requests]
    n_pages = sum(blocks) + 2
    perm = rng.permutation(n_pages)
    ck = torch.from_numpy(rng.standard_normal((n_pages, n_kv, ps, d)).astype(np.float32)).bfloat16().to(DEV)
    cv = torch.from_numpy(rng.standard_normal((n_pages, n_kv, ps, d)).astype(np.float32)).bfloat16().to(DEV)
    width = max(blocks) + 1
    bt = np.full((len(requests), width), -1, dtype=np.int32)
    at = 0
    for b, n in enumerate(blocks):
        bt[b, :n] = perm[at: at + n]
        at += n
    B = len(requests)
    q = torch.from_numpy(rng.standard_normal((B, n_q * d)).astype(np.float32)).bfloat16().to(DEV)
    dev = lambda a: torch.from_numpy(np.asarray(a, dtype=np.int32)).to(DEV)  # noqa: E731
    return dict(q=q, ck=ck, cv=cv, bt=dev(bt), q_start=dev(np.arange(B + 1)), kv_len=dev(requests),
                pos0=dev(np.asarray(requests) - 1), width=width, n_pages=n_pages)


def test_no_alloc_entry_point_matches_the_ordinary_one():
    from llm_inference_lab_b200.kernels import ops

    n_q, n_kv, d, ps = 14, 2, 64, 16
    lib = ops.lib("attention_tc", {"LAB_HEAD_DIM": d})
    fn = lib.lab_attention_decode_noalloc
    fn.restype = ctypes.c_int
    lib.lab_attention_decode_noalloc_max_floats.restype = ctypes.c_longlong
    lib.lab_attention_decode_noalloc_strerror.restype = ctypes.c_char_p
    limit = lib.lab_attention_decode_noalloc_max_floats()
    assert limit == 1 << 20
    scale = 1.0 / math.sqrt(d)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def call(case, requests, splits):
        out = torch.full((len(requests), n_q * d), float("nan"), dtype=torch.bfloat16, device=DEV)
        torch.cuda.synchronize()
        held = (torch.cuda.memory_allocated(), torch.cuda.memory_reserved())
        code = fn(ctypes.c_void_p(out.data_ptr()), out.stride(0), ctypes.c_void_p(case["q"].data_ptr()),
                  case["q"].stride(0), ctypes.c_void_p(case["ck"].data_ptr()), ctypes.c_void_p(case["cv"].data_ptr()),
                  ctypes.c_void_p(case["q_start"].data_ptr()), ctypes.c_void_p(case["kv_len"].data_ptr()),
                  ctypes.c_void_p(case["bt"].data_ptr()), case["width"], len(requests), n_q, n_kv, ps,
                  case["n_pages"], 0, ctypes.c_float(scale), splits, stream)
        torch.cuda.synchronize()
        assert (torch.cuda.memory_allocated(), torch.cuda.memory_reserved()) == held, "the call allocated nothing"
        return code, out

    # two calls in a row, of different sizes and split counts: the second finds the first one's
    # partial results in the shared array and must not be disturbed by them
    for seed, requests, splits in ((1, [700, 33, 1, 260, 512], 7), (2, [90, 1500, 31], 4)):
        case = make_case(seed, requests, n_q, n_kv, d, ps)
        code, got = call(case, requests, splits)
        assert code == 0, lib.lab_attention_decode_noalloc_strerror(code)
        # the ordinary entry point, made to take the same road (partial results to a buffer, then the
        # merge kernel, instead of merging inside a thread-block cluster): the same kernels on the same
        # inputs give the same bits
        merge_in_cluster, ops.CLUSTER_MERGE = ops.CLUSTER_MERGE, False
        try:
            want = ops.attention_tc(case["q"], case["ck"], case["cv"], case["q_start"], case["kv_len"], case["pos0"],
                                    case["bt"], len(requests), [1] * len(requests), max(requests), n_q, n_kv, d, 0,
                                    scale, splits=splits)
        finally:
            ops.CLUSTER_MERGE = merge_in_cluster
        torch.cuda.synchronize()
        assert torch.equal(got, want), "the entry point that allocates nothing differs from the ordinary one"
        # and once against a plain 64-bit attention over the same pages
        for b, kv in enumerate(requests):
            pages = case["bt"][b, : -(-kv // ps)].long()
            k = case["ck"][pages].permute(0, 2, 1, 3).reshape(-1, n_kv, d)[:kv].double().cpu()
            v = case["cv"][pages].permute(0, 2, 1, 3).reshape(-1, n_kv, d)[:kv].double().cpu()
            q = case["q"][b].view(n_q, d).double().cpu()
            group = n_q // n_kv
            for h in range(n_q):
                p = torch.softmax((k[:, h // group] @ q[h]) * scale, dim=0)
                ref = p @ v[:, h // group]
                err = (got[b].view(n_q, d)[h].double().cpu() - ref).abs().max() / ref.abs().max()
                assert err < 2e-2, (b, h, float(err))
    ops.take_device_errors()

    # beyond the fixed scratch: refused with a clear message, nothing runs
    big = [8] * 700
    assert len(big) * n_q * 32 * (d + 2) > limit
    case = make_case(3, big, n_q, n_kv, d, ps)
    code, out = call(case, big, 32)
    assert code < 0 and b"exceeds the fixed scratch" in lib.lab_attention_decode_noalloc_strerror(code)
    torch.cuda.synchronize()
    assert torch.isnan(out.float()).all()
