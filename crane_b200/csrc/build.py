"""Compiles the engine's native code at first use and loads it with ctypes.

Two shared objects: ``libcrane_host`` (C++: cache manager, scheduler; g++ only)
and ``libcrane_kernels`` (CUDA for sm_100a; nvcc).  Sources are hashed with the
flags; an up-to-date object is reused.  Objects go to ``_build/`` beside the
sources when that is writable, otherwise to a per-user folder under the
system's temporary directory, so a read-only checkout and an empty HOME both
work.  There is no fallback: a failed build raises.

The warp-level attention kernels are compiled per head size, two objects a
size.  The CUDA library is linked for a set of head sizes: all eleven
(``build_all``, what the build check and the tests use), or just the ones the
models at hand have, so that a first call compiles what its model needs and no
more.  A library that holds more sizes than asked for is taken as it is;
compiled objects are kept, so a library for one more size compiles two files.
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
BASE_SOURCES = ["elementwise.cu", "gemm_simt.cu", "gemm_tcgen05.cu", "attention_simt.cu",
                "attention_decode.cu", "attention_prefill.cu", "attention_prefill_tc.cu", "sampling.cu"]
# the two files whose entry points pick a head size's launcher: compiled for the library's set of sizes
DISPATCH_SOURCES = ("attention_decode.cu", "attention_prefill.cu")


def kernel_sources(head_sizes: Sequence[int]) -> List[str]:
    sizes = sorted(set(head_sizes), reverse=True)          # the slowest to compile first
    return (BASE_SOURCES + [f"attention_decode.cu@CRANE_HEAD_SIZE={d}" for d in sizes]
            + [f"attention_prefill.cu@CRANE_HEAD_SIZE={d}" for d in sizes])


KERNEL_SOURCES = kernel_sources(ATTENTION_HEAD_SIZES)
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
           link_flags: Sequence[str], verbose_ptxas: bool = False, label: str = "",
           per_file_flags: Optional[Dict[str, List[str]]] = None) -> str:
    """Compiles what is not yet compiled and links ``lib``.  ``label`` tells
    libraries of one name apart (the CUDA library's set of head sizes);
    ``per_file_flags``: further flags for single source files."""
    bdir = build_dir()
    per_file_flags = per_file_flags or {}
    extra = [f for rel in sorted(per_file_flags) for f in [rel] + per_file_flags[rel]]
    tag = _digest(sources, list(flags) + [compiler] + extra)
    so = os.path.join(bdir, f"{lib}{'_' + label if label else ''}_{tag}.so")
    if os.path.isfile(so):
        return so
    _say(f"building {lib}{' (' + label + ')' if label else ''}: {len(sources)} source files in {bdir}")
    t0 = time.time()

    def one(rel: str) -> str:
        path, _, define = rel.partition("@")
        mine = list(flags) + per_file_flags.get(rel, [])
        # an object is kept under the digest of its own source, the headers and its flags
        otag = _digest([rel], mine + [compiler])
        obj = os.path.join(bdir, f"obj_{otag}_{os.path.basename(path)}{'_' + define.replace('=', '_') if define else ''}.o")
        if os.path.isfile(obj):
            return obj
        tmp_obj = obj + f".tmp{os.getpid()}"
        cmd = [compiler, *mine, "-I", HERE, "-c", os.path.join(HERE, path), "-o", tmp_obj]
        if define:
            cmd.insert(1, "-D" + define)
        if verbose_ptxas:
            cmd.insert(1, "-Xptxas=-v")
        _run(cmd, rel)
        os.replace(tmp_obj, obj)
        suffix = obj[len(os.path.join(bdir, f"obj_{otag}")):]
        for name in os.listdir(bdir):                  # the same file's objects of earlier source versions
            if name.startswith("obj_") and name.endswith(suffix) and len(name) == len(os.path.basename(obj)) \
                    and name != os.path.basename(obj) and not per_file_flags.get(rel):
                try:
                    os.remove(os.path.join(bdir, name))
                except OSError:
                    pass
        _say(f"compiled {rel} ({time.time() - t0:.0f} s)")
        return obj
    with ThreadPoolExecutor(max_workers=min(os.cpu_count() or 8, 16, len(sources))) as pool:
        objs = list(pool.map(one, sources))
    tmp = so + f".tmp{os.getpid()}"
    _run([compiler, "-shared", "-o", tmp, *objs, *link_flags], lib)
    os.replace(tmp, so)
    prefix = f"{lib}{'_' + label if label else ''}_"
    for name in os.listdir(bdir):                      # libraries of earlier source versions
        stale_lib = (name.startswith(prefix) and name.endswith(".so") and name != os.path.basename(so)
                     and len(name) == len(os.path.basename(so)))
        if stale_lib:
            try:
                os.remove(os.path.join(bdir, name))
            except OSError:
                pass
    _say(f"built {os.path.basename(so)} in {time.time() - t0:.0f} s")
    return so


def build_host() -> str:
    cxx = _find("g++", "CXX", ["/usr/bin/g++"])
    return _build("libcrane_host", HOST_SOURCES, cxx, CXX_FLAGS, [])


def _size_list_flag(head_sizes: Sequence[int]) -> str:
    return "-DCRANE_HEAD_SIZE_LIST(X)=" + " ".join(f"X({d})" for d in sorted(set(head_sizes)))


def _kernels_label(head_sizes: Sequence[int]) -> str:
    sizes = sorted(set(head_sizes))
    if sizes == sorted(ATTENTION_HEAD_SIZES):
        return "all"
    return "d" + "-".join(str(d) for d in sizes) if sizes else "d0"


def build_kernels(head_sizes: Optional[Sequence[int]] = None) -> str:
    """The CUDA library with the attention kernels of ``head_sizes`` (None: of all
    head sizes there are kernels for).  Returns its path; compiles what is missing."""
    sizes = sorted(set(ATTENTION_HEAD_SIZES if head_sizes is None else head_sizes))
    unknown = [d for d in sizes if d not in ATTENTION_HEAD_SIZES]
    if unknown:
        raise BuildError(f"no attention kernels are written for head sizes {unknown}")
    per_file = {}
    if sizes != sorted(ATTENTION_HEAD_SIZES):
        per_file = {f: [_size_list_flag(sizes)] for f in DISPATCH_SOURCES}
    return _build("libcrane_kernels", kernel_sources(sizes), nvcc_path(), NVCC_FLAGS, [],
                  label=_kernels_label(sizes), per_file_flags=per_file)


def built_kernels_with(head_sizes: Sequence[int]) -> Optional[str]:
    """The path of an up-to-date library that is already built and holds at least
    ``head_sizes``: the one with every head size, if it is there."""
    bdir = build_dir()
    tag = _digest(KERNEL_SOURCES, list(NVCC_FLAGS) + [nvcc_path()])
    so = os.path.join(bdir, f"libcrane_kernels_all_{tag}.so")
    return so if os.path.isfile(so) else None


def load_host() -> ctypes.CDLL:
    with _lock:
        if "host" not in _loaded:
            _loaded["host"] = ctypes.CDLL(build_host())
        return _loaded["host"]


def load_kernels(head_sizes: Sequence[int] = ()) -> ctypes.CDLL:
    """The CUDA library with (at least) the attention kernels of ``head_sizes``:
    the library with every head size if that is built already, else one for
    just these sizes, compiled now.  Raises BuildError if it cannot be built or
    loaded."""
    sizes = tuple(sorted(set(head_sizes)))
    with _lock:
        key = "kernels:" + ",".join(map(str, sizes))
        if key not in _loaded:
            path = built_kernels_with(sizes) or build_kernels(sizes)
            try:
                _loaded[key] = ctypes.CDLL(path)
            except OSError as e:
                raise BuildError(f"cannot load {path}: {e}") from None
            _loaded[key]._crane_path = path
        return _loaded[key]


def load_microbench() -> ctypes.CDLL:
    """The two measurements of the machine in microbench.cu (a small library of
    its own: no model needs it, so no first call compiles it)."""
    with _lock:
        if "microbench" not in _loaded:
            path = _build("libcrane_microbench", ["microbench.cu"], nvcc_path(), NVCC_FLAGS, [])
            _loaded["microbench"] = ctypes.CDLL(path)
        return _loaded["microbench"]


def build_all() -> Dict[str, str]:
    return {"host": build_host(), "kernels": build_kernels(),
            "microbench": _build("libcrane_microbench", ["microbench.cu"], nvcc_path(), NVCC_FLAGS, [])}
