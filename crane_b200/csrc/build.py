"""Compiles the engine's native code at first use and loads it with ctypes.

Two shared objects: ``libcrane_host`` (C++: cache manager, scheduler; g++ only)
and ``libcrane_kernels`` (CUDA for sm_100a; nvcc).  Sources are hashed with the
flags; an up-to-date object is reused.  Objects go to ``_build/`` beside the
sources when that is writable, otherwise to a per-user folder under the
system's temporary directory, so a read-only checkout and an empty HOME both
work.  There is no fallback: a failed build raises.
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
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List, Optional, Sequence

HERE = os.path.dirname(os.path.abspath(__file__))

# "file@NAME=VALUE": the file compiled once more with -DNAME=VALUE into an object of its own.  The
# warp-level attention kernels are compiled per head size this way, side by side.
ATTENTION_HEAD_SIZES = (16, 32, 48, 64, 80, 96, 112, 128, 160, 192, 256)
KERNEL_SOURCES = (["elementwise.cu", "gemm_simt.cu", "gemm_tcgen05.cu", "attention_simt.cu",
                   "attention_decode.cu", "attention_prefill.cu", "attention_prefill_tc.cu",
                   "sampling.cu"]
                  # the slowest to compile first
                  + [f"attention_decode.cu@CRANE_HEAD_SIZE={d}" for d in reversed(ATTENTION_HEAD_SIZES)]
                  + [f"attention_prefill.cu@CRANE_HEAD_SIZE={d}" for d in reversed(ATTENTION_HEAD_SIZES)])
HOST_SOURCES = ["host/cache_manager.cpp", "host/scheduler.cpp"]

NVCC_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
CXX_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-fvisibility=hidden", "-Wall"]

_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[crane_b200 build] {msg}", file=sys.stderr, flush=True)


def _find(tool: str, env: str, extra: Sequence[str]) -> str:
    cand = os.environ.get(env)
    if cand and os.path.isfile(cand):
        return cand
    found = shutil.which(tool)
    if found:
        return found
    for p in extra:
        if os.path.isfile(p):
            return p
    raise BuildError(f"{tool} not found (set {env}); the engine has no path without its native code")


def nvcc_path() -> str:
    return _find("nvcc", "CRANE_NVCC", ["/usr/local/cuda/bin/nvcc"])


def build_dir() -> str:
    override = os.environ.get("CRANE_BUILD_DIR")
    cands = [override] if override else []
    cands.append(os.path.join(HERE, "_build"))
    cands.append(os.path.join(tempfile.gettempdir(), f"crane_b200_build_{os.getuid()}"))
    for d in cands:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".w{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return d
        except OSError:
            continue
    raise BuildError("no writable build folder: tried " + ", ".join(cands))


def _digest(paths: Sequence[str], flags: Sequence[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    headers = sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h", ".hpp")))
    host_headers = sorted(os.path.join("host", f) for f in os.listdir(os.path.join(HERE, "host"))
                          if f.endswith((".h", ".hpp")))
    for rel in list(paths) + headers + host_headers:
        with open(os.path.join(HERE, rel.split("@")[0]), "rb") as f:
            h.update(rel.encode())
            h.update(f.read())
    return h.hexdigest()[:16]


def _run(cmd: List[str], what: str) -> None:
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    out: List[str] = []

    def pump():
        for line in proc.stdout:          # type: ignore[union-attr]
            out.append(line)
    th = threading.Thread(target=pump, daemon=True)
    th.start()
    while True:
        try:
            proc.wait(timeout=10.0)
            break
        except subprocess.TimeoutExpired:
            _say(f"still compiling {what} ({time.time() - t0:.0f} s)")     # a line now and then
    th.join()
    if proc.returncode != 0:
        raise BuildError(f"compiling {what} failed:\n$ {' '.join(cmd)}\n{''.join(out)}")


def _build(lib: str, sources: Sequence[str], compiler: str, flags: Sequence[str],
           link_flags: Sequence[str], verbose_ptxas: bool = False) -> str:
    bdir = build_dir()
    tag = _digest(sources, list(flags) + [compiler])
    so = os.path.join(bdir, f"{lib}_{tag}.so")
    if os.path.isfile(so):
        return so
    _say(f"building {lib} ({len(sources)} source files) in {bdir}")
    t0 = time.time()
    objs = []

    def one(rel: str) -> str:
        path, _, define = rel.partition("@")
        obj = os.path.join(bdir, f"{lib}_{tag}_{os.path.basename(path)}{'_' + define.replace('=', '_') if define else ''}.o")
        cmd = [compiler, *flags, "-I", HERE, "-c", os.path.join(HERE, path), "-o", obj]
        if define:
            cmd.insert(1, "-D" + define)
        if verbose_ptxas:
            cmd.insert(1, "-Xptxas=-v")
        _run(cmd, rel)
        _say(f"compiled {rel} ({time.time() - t0:.0f} s)")
        return obj
    with ThreadPoolExecutor(max_workers=min(os.cpu_count() or 8, 16, len(sources))) as pool:
        objs = list(pool.map(one, sources))
    tmp = so + f".tmp{os.getpid()}"
    _run([compiler, "-shared", "-o", tmp, *objs, *link_flags], lib)
    os.replace(tmp, so)
    for name in os.listdir(bdir):                      # objects of earlier source versions
        if name.startswith(lib + "_") and name.endswith(".so") and name != os.path.basename(so):
            try:
                os.remove(os.path.join(bdir, name))
            except OSError:
                pass
    for o in objs:
        try:
            os.remove(o)
        except OSError:
            pass
    _say(f"built {os.path.basename(so)} in {time.time() - t0:.0f} s")
    return so


def build_host() -> str:
    cxx = _find("g++", "CXX", ["/usr/bin/g++"])
    return _build("libcrane_host", HOST_SOURCES, cxx, CXX_FLAGS, [])


def build_kernels() -> str:
    return _build("libcrane_kernels", KERNEL_SOURCES, nvcc_path(), NVCC_FLAGS, [])


def load_host() -> ctypes.CDLL:
    with _lock:
        if "host" not in _loaded:
            _loaded["host"] = ctypes.CDLL(build_host())
        return _loaded["host"]


def load_kernels() -> ctypes.CDLL:
    """The CUDA library.  Raises BuildError if it cannot be built or loaded."""
    with _lock:
        if "kernels" not in _loaded:
            path = build_kernels()
            try:
                _loaded["kernels"] = ctypes.CDLL(path)
            except OSError as e:
                raise BuildError(f"cannot load {path}: {e}") from None
        return _loaded["kernels"]


def build_all() -> Dict[str, str]:
    return {"host": build_host(), "kernels": build_kernels()}
