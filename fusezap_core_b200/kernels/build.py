"""Builds the CUDA libraries for sm_100a with nvcc, in-tree, at first use.

A library is a set of `.cu` files of `csrc/` linked into `_lib/lib<name>.so`. A library is built only when something
asks for it (the float32 path never builds the tensor-core kernels), it is rebuilt when its sources or flags change
(a stamp file beside it holds their hash), and a line is printed while the compiler runs. There is no fallback: with no
`nvcc`, or a failed compile, loading raises with the compiler's output.
"""
from __future__ import annotations
import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
NVCC_FLAGS += os.environ.get("FZB200_NVCC_EXTRA", "").split()      # extra compiler flags (instrumented builds)
LIBRARIES: dict[str, list[str]] = {
    "fzb200_core": ["rowwise.cu", "gemm_simt.cu", "attn_simt.cu"],
    "fzb200_tc": ["gemm_tc.cu", "attn_decode.cu", "attn_prefill.cu", "attn_prefill_tc.cu"],          # bfloat16 only: tcgen05 / TMA kernels
}
_HEADERS = ["common.cuh", "attn_mma.cuh", "tma.cuh", "umma.cuh"]
_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class KernelBuildError(RuntimeError):
    pass


def register_library(name: str, sources: list[str]) -> None:
    LIBRARIES[name] = list(sources)


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")):
        if cand and os.path.isfile(cand):
            return cand
    raise KernelBuildError("nvcc was not found (PATH, $CUDA_HOME/bin, /usr/local/cuda/bin): the CUDA kernels cannot be built")


def lib_dir() -> str:
    """`_lib/` inside the package if it can be written, else a per-user folder under the temporary directory."""
    override = os.environ.get("FZB200_LIB_DIR")
    cands = [override] if override else []
    cands.append(os.path.join(os.path.dirname(CSRC), "_lib"))
    cands.append(os.path.join(tempfile.gettempdir(), f"fusezap_core_b200-{os.getuid()}", "_lib"))
    for d in cands:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".w{os.getpid()}")
            with open(probe, "w"):
                pass
            os.unlink(probe)
            return d
        except OSError:
            continue
    raise KernelBuildError(f"no writable folder for the built kernels among {cands}")


def _digest(sources: list[str]) -> str:
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for fn in sorted(set(sources + _HEADERS + [f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))])):
        with open(os.path.join(CSRC, fn), "rb") as f:
            h.update(fn.encode() + b"\0" + f.read())
    return h.hexdigest()


def _say(msg: str) -> None:
    print(f"fusezap_core_b200: {msg}", file=sys.stderr, flush=True)


def _run_with_progress(cmds: list[tuple[str, list[str]]], what: str) -> None:
    procs = [(label, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)) for label, cmd in cmds]
    t0 = last = time.time()
    pending = list(procs)
    while pending:
        pending = [(l, p) for l, p in pending if p.poll() is None]
        if pending and time.time() - last >= 5:
            last = time.time()
            _say(f"still compiling {what}: {', '.join(l for l, _ in pending)} ({last - t0:.0f}s)")
        time.sleep(0.1)
    for label, p in procs:
        out = p.stdout.read() if p.stdout else ""
        if p.returncode != 0:
            raise KernelBuildError(f"nvcc failed on {label} (exit {p.returncode}):\n{out}")


def build(name: str, force: bool = False) -> str:
    """Builds library `name` if it is missing or stale; returns the path of the .so."""
    if name not in LIBRARIES:
        raise KeyError(f"unknown kernel library {name!r} (have {sorted(LIBRARIES)})")
    sources = LIBRARIES[name]
    d = lib_dir()
    so, stamp = os.path.join(d, f"lib{name}.so"), os.path.join(d, f"lib{name}.stamp")
    want = _digest(sources)
    with open(os.path.join(d, f".{name}.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and os.path.isfile(so) and os.path.isfile(stamp) and open(stamp).read().strip() == want:
                return so
            nvcc = _nvcc()
            t0 = time.time()
            _say(f"compiling lib{name}.so for sm_100a from {', '.join(sources)} (first use; later runs reuse it)")
            objdir = tempfile.mkdtemp(prefix=f"{name}-", dir=d)
            try:
                objs, cmds = [], []
                for src in sources:
                    obj = os.path.join(objdir, src.replace(".cu", ".o"))
                    objs.append(obj)
                    cmds.append((src, [nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]))
                _run_with_progress(cmds, f"lib{name}.so")
                tmp_so = os.path.join(objdir, f"lib{name}.so")
                _run_with_progress([("link", [nvcc, "-shared", "-o", tmp_so, *objs, "-lcudart"])], f"lib{name}.so")
                os.replace(tmp_so, so)
                with open(stamp, "w") as f:
                    f.write(want)
            finally:
                shutil.rmtree(objdir, ignore_errors=True)
            _say(f"built lib{name}.so in {time.time() - t0:.0f}s")
            return so
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def load(name: str) -> ctypes.CDLL:
    with _lock:
        if name not in _loaded:
            _loaded[name] = ctypes.CDLL(build(name))
        return _loaded[name]


def build_all(force: bool = False) -> list[str]:
    return [build(name, force) for name in LIBRARIES]
