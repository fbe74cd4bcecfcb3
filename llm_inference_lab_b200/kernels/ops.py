"""Python face of the CUDA kernels.

Each function checks shapes and types on the host, then calls one ``extern "C"``
entry point of a library built from ``csrc/kernels`` on the current CUDA stream.
There is no fallback: without a GPU, or without the built library, a call
raises.  Tensors are torch tensors on the GPU; a kernel never allocates.
"""
from __future__ import annotations

import ctypes
import threading

import torch

from . import build

F32, BF16 = 0, 1
_libs: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class KernelError(RuntimeError):
    pass


DEVICE_ERRORS = {1: "a page or slot index outside the pool", 2: "a bounded wait inside a kernel ran out",
                 3: "a gathered row index outside the batch"}


_fast: dict = {}    # (name, values of the defines) -> library handle; read without the lock on the hot path


def lib(name: str, defines: dict[str, int] | None = None) -> ctypes.CDLL:
    fast_key = (name, tuple(defines.values()) if defines else None)
    handle = _fast.get(fast_key)
    if handle is not None:
        return handle
    key = name + repr(sorted((defines or {}).items()))
    with _lock:
        if key in _libs:
            _fast[fast_key] = _libs[key]
            return _libs[key]
    path = build.kernel_library(name, defines)
    handle = ctypes.CDLL(path)
    with _lock:
        _libs[key] = handle
        _fast[fast_key] = handle
    return handle


def require_gpu() -> None:
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: the engine runs on a B200 only and has no CPU fallback")


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported storage type {dtype}: the kernels take float32 or bfloat16")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> ctypes.c_void_p:
    """The current CUDA stream's handle (also the capturing stream while a graph is recorded)."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def copy_to_device(dst: torch.Tensor, pinned_src: torch.Tensor, words_from: int, words_to: int) -> None:
    """dst[words_from:words_to] = pinned_src[words_from:words_to] (both int32, same layout) on the current
    stream, without the host-side cost of a tensor copy."""
    _check(lib("rowwise").lab_copy_to_device(
        ctypes.c_void_p(dst.data_ptr() + 4 * words_from), ctypes.c_void_p(pinned_src.data_ptr() + 4 * words_from),
        ctypes.c_longlong(4 * (words_to - words_from)), _stream()), "copy_to_device", 0)


_stream_objects: dict = {}


def current_stream() -> "torch.cuda.Stream":
    """torch's object for the current stream, found through its raw handle (the library's own
    lookup costs several microseconds a call)."""
    if _raw_stream is None:
        return torch.cuda.current_stream()
    device = torch.cuda.current_device()
    key = (device, _raw_stream(device))
    obj = _stream_objects.get(key)
    if obj is None:
        obj = _stream_objects[key] = torch.cuda.current_stream()
    return obj


def _ptr(t) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


class _Counter:
    """Kernel launches issued through this module (a graph replay adds what it captured)."""
    launches = 0


COUNTER = _Counter()


def _check(code: int, what: str, launches: int = 1) -> None:
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code}")
    COUNTER.launches += launches


def _on_gpu(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel arguments must be CUDA tensors")


_error_hooks: list = []


def on_device_error(method) -> None:
    """The bound method `method` is called when `take_device_errors` finds an error (to put scratch
    state right again); held weakly, so that it does not keep its object alive."""
    import weakref
    _error_hooks[:] = [h for h in _error_hooks if h() is not None]
    _error_hooks.append(weakref.WeakMethod(method))


def take_device_errors() -> None:
    """Synchronise and raise if any kernel left an error code."""
    for key, handle in list(_libs.items()):
        out = ctypes.c_int(0)
        _check(handle.lab_take_error_word(ctypes.byref(out)), "reading the error word", 0)
        if out.value:
            for hook in _error_hooks:
                method = hook()
                if method is not None:
                    method()
            raise KernelError(f"kernel library {key.split('[')[0]} reported: "
                              f"{DEVICE_ERRORS.get(out.value, out.value)}")


def wait_probe(limit_ms: float = 2.0) -> bool:
    """Runs the tensor-core product library's test kernel whose wait nothing ends, with a limit of
    `limit_ms` (50 at most).  Returns True if the wait gave up, as it must; the library's error word
    then says that a bounded wait ran out (`take_device_errors` raises)."""
    flag = torch.zeros((1,), dtype=torch.int32, device="cuda")
    _check(lib("gemm_tc").lab_gemm_tc_wait_probe(ctypes.c_ulonglong(int(limit_ms * 1e6)), _ptr(flag), _stream()),
           "wait_probe")
    return bool(flag.item())


# ----------------------------------------------------------------------------------------
def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    _on_gpu(ids, table)
    tokens, (vocab, hidden) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((tokens, hidden), dtype=table.dtype, device=table.device)
    assert ids.dtype == torch.int32 and table.is_contiguous() and out.is_contiguous()
    _check(lib("rowwise").lab_embed(_ptr(out), _ptr(table), _ptr(ids), tokens, hidden, vocab,
                                    dtype_code(table.dtype), _stream()), "embed")
    return out


def add_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, delta: torch.Tensor | None = None,
                partial: torch.Tensor | None = None, rows: torch.Tensor | None = None,
                out: torch.Tensor | None = None) -> torch.Tensor:
    """x += delta (+ sum of `partial` over its first axis), in place; returns rmsnorm(x) * weight.

    With `rows`, output row i is computed from x[rows[i]] and x is left as it is.
    """
    _on_gpu(x, weight, delta, partial, rows)
    n_in, hidden = x.shape
    n_out = n_in if rows is None else rows.numel()
    if out is None:
        out = torch.empty((n_out, hidden), dtype=x.dtype, device=x.device)
    assert x.is_contiguous() and weight.dtype == x.dtype and weight.numel() == hidden
    assert delta is None or (delta.shape == x.shape and delta.dtype == x.dtype and delta.is_contiguous())
    splits, stride = 0, 0
    if partial is not None:
        assert partial.dtype == torch.float32 and partial.is_contiguous() and partial.shape[1:] == x.shape
        splits, stride = partial.shape[0], n_in * hidden
    _check(lib("rowwise").lab_add_rmsnorm(_ptr(out), _ptr(x), _ptr(delta), _ptr(partial), splits,
                                          ctypes.c_longlong(stride), _ptr(weight), _ptr(rows), n_out, n_in, hidden,
                                          ctypes.c_float(eps), dtype_code(x.dtype), _stream()), "add_rmsnorm")
    return out


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor | None, inv_freq: torch.Tensor, rotary_dim: int,
                  slots: torch.Tensor | None, cache_k: torch.Tensor | None, cache_v: torch.Tensor | None,
                  n_q: int, n_kv: int, head_dim: int, bias: torch.Tensor | None = None,
                  q_out: torch.Tensor | None = None) -> torch.Tensor:
    """Rotate q and k, and write k and v to their cache slots.  Returns the rotated q.

    `qkv` is the fused projection [tokens, (n_q + 2 n_kv) * d] rounded to the storage type (q is
    rotated in place and the q columns are returned), or its 32-bit split-K partial products
    [splits, tokens, ...] with `bias` still to add (rotated q goes to a new tensor).
    """
    _on_gpu(qkv, positions, inv_freq, slots, cache_k, cache_v, bias, q_out)
    width = (n_q + 2 * n_kv) * head_dim
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() == rotary_dim // 2
    assert positions is not None or rotary_dim == 0
    page_size = num_pages = 0
    if cache_k is not None:
        num_pages, kvh, page_size, d = cache_k.shape
        assert kvh == n_kv and d == head_dim and cache_k.is_contiguous() and cache_v.is_contiguous()
        assert cache_v.shape == cache_k.shape and slots is not None
    if qkv.dim() == 3:
        splits, tokens = qkv.shape[0], qkv.shape[1]
        assert qkv.dtype == torch.float32 and qkv.is_contiguous() and qkv.shape[2] == width
        dt = cache_k.dtype if cache_k is not None else torch.bfloat16
        if q_out is None:
            q_out = torch.empty((tokens, n_q * head_dim), dtype=dt, device=qkv.device)
        _check(lib("rowwise").lab_rope_kv_write(
            None, width, _ptr(qkv), splits, ctypes.c_longlong(tokens * width), _ptr(bias), _ptr(q_out),
            _ptr(positions), _ptr(inv_freq), rotary_dim, _ptr(slots), _ptr(cache_k), _ptr(cache_v), tokens, n_q, n_kv,
            head_dim, page_size, num_pages, dtype_code(dt), _stream()), "rope_kv_write")
        return q_out
    tokens = qkv.shape[0]
    assert qkv.stride(1) == 1 and qkv.shape[1] == width and bias is None
    assert cache_k is None or cache_k.dtype == qkv.dtype
    _check(lib("rowwise").lab_rope_kv_write(
        _ptr(qkv), qkv.stride(0), None, 0, ctypes.c_longlong(0), None, None, _ptr(positions), _ptr(inv_freq),
        rotary_dim, _ptr(slots), _ptr(cache_k), _ptr(cache_v), tokens, n_q, n_kv, head_dim, page_size, num_pages,
        dtype_code(qkv.dtype), _stream()), "rope_kv_write")
    return qkv[:, : n_q * head_dim]


_no_freq: dict = {}


def kv_store(qkv: torch.Tensor, slots, cache_k, cache_v, n_q: int, n_kv: int, head_dim: int) -> torch.Tensor:
    """The framework's paged store: writes the k and v columns of the fused projection `qkv`
    [tokens, (n_q + 2 n_kv) * d] to their cache slots (nothing if `cache_k` is None) and returns the q
    columns.  What a position encoding that only encodes leaves to the framework."""
    key = str(qkv.device)
    none = _no_freq.get(key)
    if none is None:
        none = _no_freq[key] = torch.zeros((0,), dtype=torch.float32, device=qkv.device)
    return rope_kv_write(qkv, None, none, 0, slots, cache_k, cache_v, n_q, n_kv, head_dim)


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """(cos, sin) of pos * inv_freq for every row of a step: [tokens, rotary_dim / 2, 2] float32."""
    tokens, half = positions.numel(), inv_freq.numel()
    table = torch.empty((tokens, half, 2), dtype=torch.float32, device=positions.device)
    _check(lib("rowwise").lab_rope_table(_ptr(table), _ptr(positions), _ptr(inv_freq), tokens, half, _stream()),
           "rope_table")
    return table


def rope_kv_write_table(qkv, table, rotary_dim, slots, cache_k, cache_v, n_q, n_kv, head_dim) -> torch.Tensor:
    """The rotation and cache write for bfloat16 steps with many rows, with cos/sin from `rope_table`."""
    tokens = qkv.shape[0]
    page_size = num_pages = 0
    if cache_k is not None:
        num_pages, _, page_size, _ = cache_k.shape
    _check(lib("rowwise").lab_rope_kv_write_table(
        _ptr(qkv), qkv.stride(0), _ptr(table), rotary_dim, _ptr(slots), _ptr(cache_k), _ptr(cache_v), tokens, n_q,
        n_kv, head_dim, page_size, num_pages, _stream()), "rope_kv_write_table")
    return qkv[:, : n_q * head_dim]


def gemm_plain(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, gated: bool = False,
               out_f32: bool = False, out: torch.Tensor | None = None) -> torch.Tensor:
    """out = x @ w.T (+ bias) on the ordinary arithmetic units; `gated`: silu(x@wg.T) * (x@wu.T), w = [wg; wu]."""
    _on_gpu(x, w, bias, out)
    M, K = x.shape
    N = w.shape[0] // 2 if gated else w.shape[0]
    assert w.shape[1] == K and w.is_contiguous() and x.stride(1) == 1 and w.dtype == x.dtype
    assert bias is None or (bias.dtype == x.dtype and bias.numel() == N and not gated)
    odt = torch.float32 if (out_f32 or x.dtype == torch.float32) else x.dtype
    if out is None:
        out = torch.empty((M, N), dtype=odt, device=x.device)
    assert out.dtype == odt and out.stride(1) == 1 and out.shape == (M, N)
    _check(lib("gemm_plain").lab_gemm_plain(_ptr(out), _ptr(x), _ptr(w), _ptr(bias), M, N, K, x.stride(0),
                                            out.stride(0), int(gated), dtype_code(x.dtype), int(out_f32), _stream()),
           "gemm_plain")
    return out


def attention_plain(q: torch.Tensor, cache_k: torch.Tensor, cache_v: torch.Tensor, row_req: torch.Tensor,
                    row_pos: torch.Tensor, block_table: torch.Tensor, n_q: int, n_kv: int, head_dim: int,
                    window: int, scale: float, out: torch.Tensor | None = None) -> torch.Tensor:
    """Attention of every row over its request's pages; q may be a column slice of the fused projection."""
    _on_gpu(q, cache_k, cache_v, row_req, row_pos, block_table)
    tokens = q.shape[0]
    if out is None:
        out = torch.empty((tokens, n_q * head_dim), dtype=q.dtype, device=q.device)
    num_pages, kvh, page_size, d = cache_k.shape
    assert kvh == n_kv and d == head_dim and q.stride(1) == 1 and cache_k.dtype == q.dtype
    assert block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous()
    _check(lib("attention_plain").lab_attention_plain(
        _ptr(out), out.stride(0), _ptr(q), q.stride(0), _ptr(cache_k), _ptr(cache_v), _ptr(row_req), _ptr(row_pos),
        _ptr(block_table), block_table.shape[1], tokens, n_q, n_kv, head_dim, page_size, num_pages, window,
        ctypes.c_float(scale), dtype_code(q.dtype), _stream()), "attention_plain")
    return out


_sample_scratch: dict = {}
# Scratch that was outgrown stays alive: a CUDA graph captured earlier still launches kernels with its address.
_retired_scratch: list = []


def _sample_buffers(device, rows: int, chunks: int):
    """Scratch of the sampling kernel, kept per device (its counters must stay zero between calls)."""
    key = str(device)
    need = rows * chunks
    buf = _sample_scratch.get(key)
    if buf is None or buf[0].numel() < need or buf[2].numel() < rows:
        cap_rows, cap = max(rows, 256), max(need, 256 * chunks)
        buf = (torch.empty((cap,), dtype=torch.float32, device=device),
               torch.empty((cap,), dtype=torch.int32, device=device),
               torch.zeros((cap_rows,), dtype=torch.int32, device=device))
        _retired_scratch.append(_sample_scratch.get(key))
        _sample_scratch[key] = buf
    return buf


def sample(logits: torch.Tensor, temperature: torch.Tensor | None = None, seeds: torch.Tensor | None = None,
           positions: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """One token per row of 32-bit logits: greedy where temperature is 0 (or None), else Gumbel-max."""
    _on_gpu(logits, temperature, seeds, positions)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    if temperature is not None:
        assert temperature.dtype == torch.float32 and seeds.dtype == torch.int32 and positions.dtype == torch.int32
        assert temperature.numel() == rows and seeds.numel() == rows and positions.numel() == rows
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    L = lib("sampling")
    chunks = L.lab_sample_chunks(vocab)
    pv = pi = cnt = None
    if chunks > 1:
        pv, pi, cnt = _sample_buffers(logits.device, rows, chunks)
    _check(L.lab_sample(_ptr(out), _ptr(logits), ctypes.c_longlong(logits.stride(0)), rows, vocab, _ptr(temperature),
                        _ptr(seeds), _ptr(positions), _ptr(pv), _ptr(pi), _ptr(cnt), _stream()), "sample")
    return out


# ----------------------------------------------------------------------------------------
# Dispatch: which kernel serves a matrix product or an attention call.
#
# float32 always runs the plain kernels (a true 32-bit path: no tensor cores, no reduced
# precision).  bfloat16 runs the tensor-core kernels; `force_plain(True)` sends bfloat16 to
# the plain kernels as well, which tests use to tell a kernel fault from a model fault.
# ----------------------------------------------------------------------------------------
_force_plain = False
_sm_count = 0


def sm_count() -> int:
    """Streaming multiprocessors of the current device (the host's choices of tiles and splits go by
    it, as the kernels' own grids do); 148, a B200's, where no device is present."""
    global _sm_count
    if _sm_count == 0:
        if torch.cuda.is_available():
            _sm_count = int(torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count)
        else:
            _sm_count = 148
    return _sm_count


def forced_plain() -> bool:
    return _force_plain


def force_plain(flag: bool) -> bool:
    global _force_plain
    old, _force_plain = _force_plain, bool(flag)
    return old


def gemm_tc(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, gated: bool = False,
            out_f32: bool = False, swap: bool | None = None, bn: int | None = None, splits: int = 1,
            out: torch.Tensor | None = None) -> torch.Tensor:
    """out = x @ w.T (+ bias) on the tcgen05 tensor cores (bfloat16 in, 32-bit accumulate).

    `swap` puts output features on the M side of the MMA (few tokens); `bn` is the tile on the
    other side; `splits` > 1 returns 32-bit partial products [splits, tokens, out].
    """
    _on_gpu(x, w, bias, out)
    T, K = x.shape
    n_out = w.shape[0] // 2 if gated else w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc takes bfloat16 operands")
    if K % 8 or x.stride(0) % 8 or x.stride(1) != 1 or not w.is_contiguous() or w.shape[1] != K:
        raise KernelError(f"gemm_tc: K={K} and the row stride must be multiples of 8 (16-byte rows for TMA)")
    if x.data_ptr() % 16 or w.data_ptr() % 16:
        raise KernelError("gemm_tc: operands must start on a 16-byte boundary")
    if swap is None:
        swap = T <= (64 if gated else 128)
    if bn is None:
        if swap:
            bn = 16
            while bn < min(T, 64 if gated else 256):
                bn *= 2
        else:
            bn = 256 if gated else 128
    if splits > 1:
        if gated or bias is not None:
            raise KernelError("split-K takes no bias and no gate")
        k_tiles = -(-K // 64)
        per = -(-k_tiles // splits)
        splits = -(-k_tiles // per)       # no empty split
    if splits > 1:
        out = torch.empty((splits, T, n_out), dtype=torch.float32, device=x.device) if out is None else out
        ld_out, f32 = n_out, True
    else:
        odt = torch.float32 if out_f32 else torch.bfloat16
        if out is None:
            out = torch.empty((T, n_out), dtype=odt, device=x.device)
        assert out.dtype == odt and out.stride(1) == 1
        ld_out, f32 = out.stride(0), out_f32
    _check(lib("gemm_tc").lab_gemm_tc(_ptr(out), _ptr(x), _ptr(w), _ptr(bias), T, n_out, K, x.stride(0), ld_out,
                                      int(gated), int(f32), int(swap), bn, splits, _stream()), "gemm_tc")
    return out


def gemm_tc2(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, gated: bool = False,
             out_f32: bool = False, splits: int = 1, out: torch.Tensor | None = None, bn: int = 0) -> torch.Tensor:
    """out = x @ w.T (+ bias) on pairs of SMs (tcgen05.mma.cta_group::2): tiles of 256 tokens by 256
    accumulator columns, each CTA of a pair loading half of the weight tile.  For steps with many
    tokens; `splits` > 1 returns 32-bit partial products [splits, tokens, out].  `bn`: accumulator
    columns of a tile (256, 224 or 192; 0: the width whose tiles fill the rounds of the pairs best)."""
    _on_gpu(x, w, bias, out)
    T, K = x.shape
    n_out = w.shape[0] // 2 if gated else w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc2 takes bfloat16 operands")
    if not _tc_operands(x, w) or w.shape[1] != K:
        raise KernelError(f"gemm_tc2: K={K} and the row stride must be multiples of 8 (16-byte rows for TMA)")
    if splits > 1:
        if gated or bias is not None:
            raise KernelError("split-K takes no bias and no gate")
        k_tiles = -(-K // 64)
        per = -(-k_tiles // splits)
        splits = -(-k_tiles // per)       # no empty split
    if splits > 1:
        out = torch.empty((splits, T, n_out), dtype=torch.float32, device=x.device) if out is None else out
        ld_out, f32 = n_out, True
    else:
        odt = torch.float32 if out_f32 else torch.bfloat16
        if out is None:
            out = torch.empty((T, n_out), dtype=odt, device=x.device)
        assert out.dtype == odt and out.stride(1) == 1
        ld_out, f32 = out.stride(0), out_f32
    _check(lib("gemm_tc2").lab_gemm_tc2(_ptr(out), _ptr(x), _ptr(w), _ptr(bias), T, n_out, K, x.stride(0), ld_out,
                                        int(gated), int(f32), splits, bn, _stream()), "gemm_tc2")
    return out


def qkv_fusable(x, w, head_dim: int, rotary_dim: int) -> bool:
    """Whether `qkv_rope_store` serves this projection: bfloat16 operands the tensor-core product
    takes, heads of 64 or 128 (a head must lie whole inside a tile), rotation over the whole head."""
    return (x.dtype == torch.bfloat16 and not _force_plain and head_dim in (64, 128) and rotary_dim == head_dim
            and _tc_operands(x, w))


def qkv_rope_store(x, w_qkv, bias, table, slots, cache_k, cache_v, n_q: int, n_kv: int, head_dim: int,
                   bn: int | None = None) -> torch.Tensor:
    """The fused q/k/v projection with its epilogue in one kernel: x @ w_qkv.T + bias, rounded; q and k
    rotated with the cosines and sines of `table` ([tokens, head_dim / 2, 2] from `rope_table`); the
    rotated q returned [tokens, n_q * head_dim]; k and v written to their cache slots (`cache_k` None:
    the call does not write the cache).  Tokens lie on the 128-row side of the product: for steps of
    many tokens."""
    _on_gpu(x, w_qkv, bias, table, slots, cache_k, cache_v)
    T, K = x.shape
    width = (n_q + 2 * n_kv) * head_dim
    if not qkv_fusable(x, w_qkv, head_dim, head_dim):
        raise KernelError("qkv_rope_store takes bfloat16 operands with 16-byte rows and heads of 64 or 128")
    assert w_qkv.shape == (width, K) and (bias is None or (bias.numel() == width and bias.dtype == x.dtype))
    assert table.dtype == torch.float32 and table.is_contiguous() and table.shape == (T, head_dim // 2, 2)
    page_size = num_pages = 0
    if cache_k is not None:
        num_pages, kvh, page_size, d = cache_k.shape
        assert kvh == n_kv and d == head_dim and cache_k.is_contiguous() and cache_v.is_contiguous()
        assert cache_v.shape == cache_k.shape and cache_k.dtype == x.dtype and slots is not None
        assert slots.dtype == torch.int32 and slots.numel() >= T
    if bn is None:
        bn = _pick_prefill_tiles(T, width, K, False)[1]     # 128, or 256 where its waves cost less
    q = torch.empty((T, n_q * head_dim), dtype=x.dtype, device=x.device)
    _check(lib("gemm_tc").lab_gemm_tc_qkv(
        _ptr(q), _ptr(x), _ptr(w_qkv), _ptr(bias), T, n_q, n_kv, head_dim, K, x.stride(0), q.stride(0), _ptr(table),
        _ptr(slots), _ptr(cache_k), _ptr(cache_v), page_size, num_pages, bn, _stream()), "gemm_tc_qkv")
    return q


_pick_scratch: dict = {}
# Rows up to which a step's head picks its tokens itself (the kernel takes up to 128).  Measured at the
# Qwen2.5-0.5B sizes against the head that writes 32-bit logits for the sampling kernel: a decode step of
# 8 or 16 rows takes the same time (0.792 ms both ways; 0.812 against 0.814 ms) without the 5 to 10 MB of
# logits written and read back; at 32 rows the pick in the epilogue costs more than the logits' traffic
# (0.980 against 0.950 ms), at 64 rows 1.16 against 1.14 ms.
PICK_MAX_ROWS = 16


def head_pick_fusable(x, w) -> bool:
    """Whether `head_pick` serves this head: bfloat16 operands the tensor-core product takes, few rows."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and not _force_plain
            and x.shape[0] <= min(PICK_MAX_ROWS, 128) and _tc_operands(x, w))


def head_pick(x, w, temperature=None, seeds=None, positions=None, out=None) -> torch.Tensor:
    """One token per row of x from the head's logits x @ w.T without writing them: every tile of the
    product keeps its best candidate per row (greedy, or Gumbel-max where `temperature` > 0, by the
    sampling kernel's rule) and a second, tiny kernel picks each row's best."""
    _on_gpu(x, w, temperature, seeds, positions, out)
    T, K = x.shape
    vocab = w.shape[0]
    if not (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and T <= 128 and _tc_operands(x, w)):
        raise KernelError("head_pick takes bfloat16 operands with 16-byte rows and up to 128 rows")
    if temperature is not None:
        assert temperature.dtype == torch.float32 and seeds.dtype == torch.int32 and positions.dtype == torch.int32
        assert temperature.numel() >= T and seeds.numel() >= T and positions.numel() >= T
    if out is None:
        out = torch.empty((T,), dtype=torch.int32, device=x.device)
    assert out.dtype == torch.int32 and out.numel() >= T
    tiles = -(-vocab // 128)
    key = str(x.device)
    buf = _pick_scratch.get(key)
    if buf is None or buf[0].numel() < T * tiles:
        cap = max(T, 128) * tiles
        buf = (torch.empty((cap,), dtype=torch.float32, device=x.device),
               torch.empty((cap,), dtype=torch.int32, device=x.device))
        _retired_scratch.append(_pick_scratch.get(key))
        _pick_scratch[key] = buf
    bn = 16
    while bn < T:
        bn *= 2
    _check(lib("gemm_tc").lab_gemm_tc_pick(_ptr(out), _ptr(x), _ptr(w), T, vocab, K, x.stride(0), _ptr(temperature),
                                           _ptr(seeds), _ptr(positions), _ptr(buf[0]), _ptr(buf[1]), bn, _stream()),
           "gemm_tc_pick", 2)
    return out


def _pick_splits(T: int, n_out: int, K: int) -> int:
    """Split K when an output has too few tiles to keep the memory system busy (decode)."""
    if T > 128:
        return 1
    tiles = -(-n_out // 128)
    k_tiles = -(-K // 64)
    if tiles >= sm_count() // 2 or k_tiles < 8:
        return 1
    return max(1, min(-(-k_tiles // 4), sm_count() // tiles, 16))   # about 4 k-tiles per CTA (measured best)


def _pick_prefill_tiles(T: int, n_out: int, K: int, allow_partial: bool) -> tuple[str, int, int]:
    """(kernel, N tile, K splits) of a product with many tokens (tokens on the 128-row side);
    kernel is "pair" (two CTAs per 256 x 256 tile) or "tc".  Measured on the down and output
    projections of the 0.5B, 1.5B and 7B layer sizes at 256 to 4,096 tokens, together with the
    norm that sums the partial products:
    * a CTA fills shared memory from L2 at a limited rate, so tiles with more arithmetic per byte
      run closer to the tensor cores' pace: 128 x 128 tiles take about 420 cycles per 64 elements
      of K, 128 x 256 tiles 600, and a pair's 256 x 256 tile 900;
    * pairs win once there are enough tiles for most of the 74 pairs of SMs and K is long
      (down at 2,048 tokens, 1.5B: 61 against 75 us; 7B: 221 against 249 us);
    * while 128-wide tiles fill at most one wave, they win, with K split so that the wave is
      full and a split keeps 16 k-tiles or more (down at 2,048 tokens, 0.5B: 28 against 34 us
      for 256-wide tiles and two splits; at 512 tokens 15 against 21 us);
    * beyond one wave, the width whose waves cost less."""
    m_tiles, k_tiles = -(-T // 128), -(-K // 64)
    pairs = -(-T // 256) * (-(-n_out // 256))
    if k_tiles >= 32 and pairs >= 48:
        return "pair", 256, 1
    t128, t256 = m_tiles * (-(-n_out // 128)), m_tiles * (-(-n_out // 256))
    if t128 <= sm_count():
        splits = max(1, min(sm_count() // t128, k_tiles // 16)) if allow_partial else 1
        return "tc", 128, splits
    if -(-t256 // sm_count()) * 600 < -(-t128 // sm_count()) * 420:
        return "tc", 256, 1
    return "tc", 128, 1


def _tc_operands(x, w) -> bool:
    """Whether TMA can describe the operands: rows of 16-byte multiples that start on 16-byte
    boundaries.  Widths that are no multiple of 8 go to the plain kernel instead."""
    return (x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) == 1 and w.is_contiguous()
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def linear(x, w, bias=None, out_f32=False, allow_partial=False):
    """x @ w.T (+ bias).  With `allow_partial` the result may come back as 32-bit partial
    products [splits, tokens, out], without the bias, that the consumer sums (`add_rmsnorm`,
    `rope_kv_write`)."""
    if x.dtype == torch.float32 or _force_plain or not _tc_operands(x, w):
        return gemm_plain(x, w, bias, out_f32=out_f32)
    T = x.shape[0]
    if T > 128:
        kind, bn, splits = _pick_prefill_tiles(T, w.shape[0], x.shape[1],
                                               allow_partial and bias is None and not out_f32)
        if kind == "pair":
            return gemm_tc2(x, w, bias, out_f32=out_f32)
        if splits > 1:
            return gemm_tc(x, w, None, swap=False, bn=bn, splits=splits)
        return gemm_tc(x, w, bias, out_f32=out_f32, swap=False, bn=bn)
    splits = _pick_splits(T, w.shape[0], x.shape[1]) if allow_partial else 1
    if splits > 1:
        return gemm_tc(x, w, None, splits=splits)     # the consumer adds the bias
    return gemm_tc(x, w, bias, out_f32=out_f32)


def linear_gated(x, w_gate_up):
    """silu(x @ wg.T) * (x @ wu.T) with w_gate_up = [wg; wu]."""
    if x.dtype == torch.float32 or _force_plain or not _tc_operands(x, w_gate_up):
        return gemm_plain(x, w_gate_up, None, gated=True)
    # Pairs of SMs (256 tokens x 128 features per tile, gate rows in one CTA and up rows in the other)
    # once their tiles fill most of the 74 pairs: measured 6 to 12 % faster from there on at the 0.5B,
    # 1.5B and 7B layer sizes (2,048 tokens: 31.7 against 33.7, 76 against 85, 349 against 385 us).
    T, inter = x.shape[0], w_gate_up.shape[0] // 2
    if -(-T // 256) * (-(-inter // 128)) >= 64:
        return gemm_tc2(x, w_gate_up, None, gated=True)
    return gemm_tc(x, w_gate_up, None, gated=True)


# Which kernel serves requests that bring several tokens: "auto" (tcgen05 for heads of 64 and of 128
# once a request brings more than 64 tokens, else mma.sync), "mma" or "tc05".
PREFILL_KERNEL = "auto"


# With 2 to 8 splits, and all CTAs of the launch resident at once, the decode kernel merges the splits
# itself: the splits of a (request, kv head) form a thread-block cluster and read one another's shared
# memory.  (With more CTAs than SMs the cluster launch measured slower than the merge kernel.)
# False: always the merge kernel.
CLUSTER_MERGE = True


def attention_tc_supported(head_dim: int) -> bool:
    return head_dim % 16 == 0 and 16 <= head_dim <= 128


def decode_shape(head_dim: int) -> tuple[int, int]:
    """(keys a decode CTA takes in one round of its warps, decode CTAs an SM holds) of the kernel
    built for this head size."""
    shape = _decode_shapes.get(head_dim)
    if shape is None:
        L = lib("attention_tc", {"LAB_HEAD_DIM": head_dim})
        shape = _decode_shapes[head_dim] = (int(L.lab_attention_decode_keys_per_round()),
                                            int(L.lab_attention_decode_ctas_per_sm()))
    return shape


_decode_shapes: dict[int, tuple[int, int]] = {}


def decode_splits(n_decode: int, n_kv: int, group: int, max_kv_len: int, keys_per_round: int = 128,
                  ctas_per_sm: int = 2) -> int:
    """How many ways the keys of a decoding request are split across CTAs.  A warp needs about
    two microseconds per tile (its instructions depend on one another), so for latency a
    CTA's warps should get one tile each: one round (128 keys at heads of 64) per CTA while all
    CTAs of the launch find room at once and the splits (8 at most) can merge inside their cluster;
    else two rounds per CTA, as far as the GPU has room for the CTAs (the reference splits 1..16
    ways, rust/engine/src/runner/model/qwen2/engine.rs:1597-1617)."""
    ctas = max(1, n_decode * n_kv * (-(-group // 16)))
    if CLUSTER_MERGE and max_kv_len <= 16 * keys_per_round:     # beyond that, more than 8 splits serve better
        fine = min(8, -(-max_kv_len // keys_per_round), sm_count() // ctas)
        if fine >= 2:
            return int(fine)
    room = max(1, (ctas_per_sm * sm_count()) // ctas)      # no second round of CTAs
    return int(max(1, min(room, -(-max_kv_len // (2 * keys_per_round)), 32)))


def attention_tc(q, cache_k, cache_v, q_start, kv_len, pos0, block_table, n_requests, q_lens, max_kv_len,
                 n_q, n_kv, head_dim, window, scale, out=None, splits=None, scratch=None):
    """Tensor-core attention: the prefill kernel serves requests with several new tokens,
    the split-KV decode kernel those with one."""
    _on_gpu(q, cache_k, cache_v, q_start, kv_len, pos0, block_table)
    if q.dtype != torch.bfloat16 or not attention_tc_supported(head_dim):
        raise KernelError(f"attention_tc: bfloat16 and a head size multiple of 16 up to 128, got {q.dtype}, {head_dim}")
    tokens = q.shape[0]
    if out is None:
        out = torch.empty((tokens, n_q * head_dim), dtype=q.dtype, device=q.device)
    num_pages, kvh, page_size, d = cache_k.shape
    assert kvh == n_kv and d == head_dim and q.stride(1) == 1 and q.stride(0) % 8 == 0
    assert block_table.dim() == 2 and block_table.is_contiguous() and block_table.shape[0] >= n_requests
    L = lib("attention_tc", {"LAB_HEAD_DIM": head_dim})
    max_q = max(q_lens)
    n_decode = sum(1 for n in q_lens if n == 1)
    use_tc05 = PREFILL_KERNEL == "tc05" or (PREFILL_KERNEL == "auto" and max_q > 64)
    if max_q > 1 and use_tc05 and head_dim in (64, 128) and page_size >= 8 and page_size <= 128 and \
            page_size & (page_size - 1) == 0:
        # tcgen05 kernel: tiles of 128 query rows, scores and P V on the 5th-generation tensor cores
        L5 = lib("attention_tc05", {"LAB_HEAD_DIM": head_dim})
        _check(L5.lab_attention_prefill_tc05(
            _ptr(out), out.stride(0), _ptr(q), q.stride(0), tokens, _ptr(cache_k), _ptr(cache_v), _ptr(q_start),
            _ptr(kv_len), _ptr(pos0), _ptr(block_table), block_table.shape[1], n_requests, max_q, n_q, n_kv,
            page_size, num_pages, window, ctypes.c_float(scale), 2, _stream()), "attention_prefill_tc05")
    elif max_q > 1:
        _check(L.lab_attention_prefill(_ptr(out), out.stride(0), _ptr(q), q.stride(0), _ptr(cache_k), _ptr(cache_v),
                                       _ptr(q_start), _ptr(kv_len), _ptr(pos0), _ptr(block_table),
                                       block_table.shape[1], n_requests, max_q, n_q, n_kv, page_size, num_pages,
                                       window, ctypes.c_float(scale), 2, _stream()), "attention_prefill")
    if n_decode:
        if splits is None:
            span = min(max_kv_len, window) if window else max_kv_len
            splits = decode_splits(n_decode, n_kv, n_q // n_kv, span, *decode_shape(head_dim))
        ctas = n_decode * n_kv * (-(-(n_q // n_kv) // 16)) * splits
        in_cluster = CLUSTER_MERGE and 2 <= splits <= 8 and ctas <= sm_count()
        if splits > 1 and not in_cluster:
            need = n_requests * n_q * splits * (head_dim + 2)
            if scratch is None or scratch.numel() < need:
                scratch = torch.empty((need,), dtype=torch.float32, device=q.device)
        else:
            scratch = None
        _check(L.lab_attention_decode(_ptr(out), out.stride(0), _ptr(q), q.stride(0), _ptr(cache_k), _ptr(cache_v),
                                      _ptr(q_start), _ptr(kv_len), _ptr(block_table), block_table.shape[1],
                                      n_requests, n_q, n_kv, page_size, num_pages, window, ctypes.c_float(scale),
                                      splits, _ptr(scratch), 1 if in_cluster else 0, _stream()), "attention_decode",
               2 if splits > 1 and not in_cluster else 1)
    return out


def attention(q, cache_k, cache_v, ctx, group, n_q, n_kv, head_dim, window, scale):
    if q.dtype == torch.bfloat16 and not _force_plain and attention_tc_supported(head_dim):
        return attention_tc(q, cache_k, cache_v, ctx.q_start, ctx.kv_len, ctx.pos0, group.block_table,
                            ctx.n_requests, ctx.q_lens, ctx.max_kv_len, n_q, n_kv, head_dim, window, scale)
    return attention_plain(q, cache_k, cache_v, ctx.row_req, ctx.row_pos, group.block_table, n_q, n_kv, head_dim,
                           window, scale)
