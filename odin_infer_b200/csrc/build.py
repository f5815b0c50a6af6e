"""Compiles the CUDA sources of this folder for sm_100a and loads them.

Each group of kernels becomes one small shared library next to its sources
(`libodin_<group>.so`), built with nvcc at its first use and again whenever a
source, a header or a flag changes (a stamp file holds their hash).  A model
asks only for the groups its parts use, so a first call compiles what that
model needs, several groups in parallel, and prints a line now and then while
it waits.  If the package folder cannot be written, the libraries go to a
per-user folder under the system's temporary directory.

There is no fallback: without nvcc and without a built library this raises.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

_HERE = os.path.dirname(os.path.abspath(__file__))

# group -> sources; every group also depends on every header of this folder
GROUPS = {
    "elementwise": ["elementwise.cu"],
    "gemm_plain": ["gemm_plain.cu"],
    "head_prep": ["head_prep.cu"],
    "attention_plain": ["attention_plain.cu"],
    "sampling": ["sampling.cu"],
    "gemm_tc": ["gemm_tc.cu", "gemm_tc2.cu"],
    "attention_decode": ["attention_decode.cu"],
    "attention_prefill": ["attention_prefill_tc.cu"],
    "mma_probe": ["mma_probe.cu"],   # a measuring tool (see microbench mma-rate), no part of a step
}

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared",
    "--expt-relaxed-constexpr",
]

# ODIN_KERNEL_TRACE=1: libraries of their own (libodin_<group>_trace.so) whose kernels record a
# timeline (see common.cuh); for tuning, never for serving
TRACE = os.environ.get("ODIN_KERNEL_TRACE", "0") not in ("", "0")
if TRACE:
    NVCC_FLAGS.append("-DODIN_TRACE")

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def register_group(name: str, sources: list[str]) -> None:
    GROUPS[name] = list(sources)


def _nvcc() -> str | None:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


def _group_hash(group: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for name in sorted(GROUPS[group]) + sorted(_all_headers()):
        h.update(name.encode())
        with open(os.path.join(_HERE, name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _all_headers() -> list[str]:
    return [f for f in os.listdir(_HERE) if f.endswith((".cuh", ".h"))]


def _out_dir() -> str:
    if os.access(_HERE, os.W_OK):
        return _HERE
    d = os.path.join(tempfile.gettempdir(), f"odin_infer_b200-{os.getuid()}")
    os.makedirs(d, exist_ok=True)
    return d


def lib_path(group: str) -> str:
    return os.path.join(_out_dir(), f"libodin_{group}{'_trace' if TRACE else ''}.so")


def _is_fresh(group: str) -> bool:
    lib = lib_path(group)
    stamp = lib + ".stamp"
    if not (os.path.exists(lib) and os.path.exists(stamp)):
        return False
    try:
        with open(stamp) as f:
            return f.read().strip() == _group_hash(group)
    except OSError:
        return False


def _compile(group: str) -> None:
    nvcc = _nvcc()
    if nvcc is None:
        raise RuntimeError(
            f"odin_infer_b200: kernel library '{group}' is not built and nvcc was not found; "
            "this package has no CPU or library fallback")
    lib = lib_path(group)
    tmp = f"{lib}.{os.getpid()}.tmp"
    srcs = [os.path.join(_HERE, s) for s in GROUPS[group]]
    cmd = [nvcc] + NVCC_FLAGS + ["-I", _HERE, "-o", tmp] + srcs
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise RuntimeError(f"odin_infer_b200: nvcc failed for '{group}':\n{' '.join(cmd)}\n{proc.stdout}")
    os.replace(tmp, lib)
    with open(lib + ".stamp", "w") as f:
        f.write(_group_hash(group))


def ensure_built(groups=None, verbose: bool = True) -> None:
    """Build every stale group of `groups` (default: all), in parallel."""
    groups = list(GROUPS) if groups is None else list(groups)
    stale = [g for g in groups if not _is_fresh(g)]
    if not stale:
        return
    with _lock:
        stale = [g for g in stale if not _is_fresh(g)]
        if not stale:
            return
        t0 = time.time()
        if verbose:
            print(f"odin_infer_b200: compiling {len(stale)} kernel group(s) for sm_100a: "
                  f"{', '.join(stale)}", file=sys.stderr, flush=True)
        errors: list[BaseException] = []
        done: list[str] = []

        def work(g):
            try:
                _compile(g)
                done.append(g)
            except BaseException as e:  # noqa: BLE001 - reported below
                errors.append(e)

        max_par = max(1, min(len(stale), (os.cpu_count() or 2)))
        pending = list(stale)
        running: list[threading.Thread] = []
        last = time.time()
        while pending or running:
            while pending and len(running) < max_par:
                th = threading.Thread(target=work, args=(pending.pop(0),), daemon=True)
                th.start()
                running.append(th)
            time.sleep(0.2)
            running = [t for t in running if t.is_alive()]
            if verbose and time.time() - last > 10:
                last = time.time()
                print(f"odin_infer_b200: still compiling ({len(done)}/{len(stale)} done, "
                      f"{time.time() - t0:.0f} s)", file=sys.stderr, flush=True)
        if errors:
            raise errors[0]
        if verbose:
            print(f"odin_infer_b200: compiled in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)


def load(group: str) -> ctypes.CDLL:
    lib = _loaded.get(group)
    if lib is None:
        ensure_built([group])
        lib = ctypes.CDLL(lib_path(group))
        _loaded[group] = lib
    return lib
