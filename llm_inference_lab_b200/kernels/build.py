"""Building the native code: CUDA kernels for sm_100a and the C++ runtime.

Every ``.cu`` file under ``csrc/kernels`` becomes one shared library (loaded with
ctypes through its ``extern "C"`` entry points), the C++ runtime under
``csrc/runtime`` one pybind11 module.  Libraries are built on first use into
``_build/`` beside the package (or, when that is not writable, into a per-user
temporary folder), named by a hash of their sources and flags, so a stale
binary is never loaded.  A library that takes build-time sizes (the attention
kernels take the head size) is built for the sizes a model asks for, nothing
else.  Progress lines go to stderr while compilers run.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
import tempfile
import threading
import time

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(_PKG, "csrc")
NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC", "-Xcompiler",
              "-fvisibility=hidden", "--expt-relaxed-constexpr"]

_lock = threading.Lock()
_built: dict[str, str] = {}


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[llm_inference_lab_b200 build] {msg}", file=sys.stderr, flush=True)


_build_dir: str | None = None


def build_dir() -> str:
    global _build_dir
    with _lock:
        if _build_dir is None:
            _build_dir = _pick_build_dir()
        return _build_dir


def _pick_build_dir() -> str:
    override = os.environ.get("LAB_B200_BUILD_DIR")
    candidates = [override] if override else []
    candidates.append(os.path.join(_PKG, "_build"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"llm_inference_lab_b200_build_{os.getuid()}"))
    for path in candidates:
        try:
            os.makedirs(path, exist_ok=True)
            probe = os.path.join(path, f".probe{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return path
        except OSError:
            continue
    raise BuildError("no writable folder for built libraries: tried " + ", ".join(candidates))


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc not found: the CUDA kernels cannot be built, and there is no fallback")


def _digest(paths, flags) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:12]


def _headers(folder):
    return [os.path.join(folder, f) for f in os.listdir(folder) if f.endswith((".cuh", ".h", ".hpp"))]


def _run(cmd, what):
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            _say(f"still compiling {what} ({time.time() - t0:.0f} s)")

    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    out, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        raise BuildError(f"building {what} failed:\n{' '.join(cmd)}\n{out}")
    return out


def kernel_library(name: str, defines: dict[str, int] | None = None, verbose_ptxas: bool = False) -> str:
    """Path of the shared library built from ``csrc/kernels/<name>.cu`` with `defines`."""
    defines = defines or {}
    tag = name + "".join(f"_{k.lower()}{v}" for k, v in sorted(defines.items()))
    with _lock:
        if tag in _built:
            return _built[tag]
    src = os.path.join(CSRC, "kernels", name + ".cu")
    if not os.path.exists(src):
        raise BuildError(f"no kernel source {src}")
    flags = NVCC_ARCH + NVCC_FLAGS + [f"-D{k}={v}" for k, v in sorted(defines.items())]
    if verbose_ptxas:
        flags += ["-Xptxas", "-v"]
    digest = _digest([src] + _headers(os.path.join(CSRC, "kernels")), flags)
    out = os.path.join(build_dir(), f"lib{tag}-{digest}.so")
    if not os.path.exists(out):
        nvcc = find_nvcc()
        _say(f"compiling {tag} for sm_100a")
        tmp = out + f".tmp{os.getpid()}"
        log = _run([nvcc] + flags + ["-o", tmp, src], tag)
        if verbose_ptxas:
            _say(log)
        os.replace(tmp, out)
        _say(f"built {os.path.basename(out)}")
    with _lock:
        _built[tag] = out
    return out


def runtime_module_path() -> str:
    """Path of the pybind11 module built from ``csrc/runtime/*.cpp`` (host code only)."""
    with _lock:
        if "_runtime" in _built:
            return _built["_runtime"]
    import pybind11

    folder = os.path.join(CSRC, "runtime")
    srcs = sorted(os.path.join(folder, f) for f in os.listdir(folder) if f.endswith(".cpp"))
    options = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-Wall"]
    flags = options + [f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}", f"-I{folder}"]
    # the name depends on the sources, the options and the interpreter, not on where the checkout lies
    digest = _digest(srcs + _headers(folder), options + [sys.version, pybind11.__version__])
    out = os.path.join(build_dir(), f"_lab_runtime-{digest}.so")
    if not os.path.exists(out):
        cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
        if not cxx:
            raise BuildError("no C++ compiler found for the runtime module")
        _say("compiling the C++ runtime (cache manager, scheduler)")
        tmp = out + f".tmp{os.getpid()}"
        _run([cxx] + flags + ["-o", tmp] + srcs, "runtime")
        os.replace(tmp, out)
        _say(f"built {os.path.basename(out)}")
    with _lock:
        _built["_runtime"] = out
    return out


def build_many(jobs) -> list[str]:
    """Build several kernel libraries at once; `jobs` is a list of (name, defines)."""
    results: list = [None] * len(jobs)
    errors: list = []

    def work(i, name, defines):
        try:
            results[i] = kernel_library(name, defines)
        except Exception as exc:  # noqa: BLE001 - reported below
            errors.append(exc)

    threads = [threading.Thread(target=work, args=(i, n, d)) for i, (n, d) in enumerate(jobs)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise errors[0]
    return results


def prune() -> list[str]:
    """Removes libraries in the build folder that no source of this checkout produces any more (a
    changed source or flag gives a new name and leaves the old file behind).  Keeps what this process
    has built or found; returns the names it removed."""
    with _lock:
        keep = {os.path.basename(p) for p in _built.values()}
    removed = []
    for name in os.listdir(build_dir()):
        if name.endswith(".so") and name not in keep:
            try:
                os.remove(os.path.join(build_dir(), name))
                removed.append(name)
            except OSError:
                pass
    return removed
