"""Compiles the sources in this folder into shared libraries, in-tree.

Three kinds of library exist:

* ``libtge_runtime.so`` - the host runtime (page pools, cache bookkeeping,
  scheduler, step packing): plain C++, needs no CUDA;
* ``libtge_core.so`` - every kernel that does not depend on the model;
* ``libtge_attn_hd<N>.so`` - the tensor-core attention kernels for one head
  size, compiled when a model with that head size is first built.

A library is rebuilt when the hash of its sources and flags changes.  Builds
print a line per file so that a first call on a fresh checkout shows progress.
The libraries land in ``csrc/_build`` (or, if that cannot be written, in a
per-user folder under the temporary directory).
"""
from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List, Sequence

CSRC = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
CORE_SOURCES = ["host_util.cu", "elementwise.cu", "gemm_simt.cu", "gemm_tcgen05.cu", "attention_simt.cu", "sampling.cu", "sampling_cuts.cu",
                "gemm_static_scratch.cu", "random_fill.cu"]
HEADERS = ["common.cuh", "gemm_static_scratch.h", "random_weights.h", "attention_tc.cuh", "attention_tc2.cuh"]
RUNTIME_SOURCES = ["runtime.cpp"]
RUNTIME_HEADERS = ["runtime.h", "random_weights.h"]


class BuildError(RuntimeError):
    pass


def _log(message: str) -> None:
    print(f"[tge build] {message}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    candidates = [os.environ.get("TGE_NVCC"), shutil.which("nvcc")]
    for root in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if root:
            candidates.append(os.path.join(root, "bin", "nvcc"))
    for path in candidates:
        if path and os.path.isfile(path) and os.access(path, os.X_OK):
            return path
    raise BuildError("nvcc not found (looked at TGE_NVCC, PATH, CUDA_HOME, /usr/local/cuda): "
                     "the CUDA kernels of this engine cannot be built, and there is no fallback")


def build_dir() -> str:
    preferred = os.path.join(CSRC, "_build")
    try:
        os.makedirs(preferred, exist_ok=True)
        probe = os.path.join(preferred, f".probe_{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return preferred
    except OSError:
        fallback = os.path.join(tempfile.gettempdir(), f"tge_b200_build_{os.getuid()}")
        os.makedirs(fallback, exist_ok=True)
        return fallback


def find_host_compiler() -> List[str]:
    """The C++ compiler for the host runtime: g++ or c++ if there is one, else nvcc (which calls one)."""
    for name in (os.environ.get("CXX"), "g++", "c++", "clang++"):
        path = shutil.which(name) if name else None
        if path:
            return [path]
    return [find_nvcc(), "-x", "c++"]


def _hash(sources: Sequence[str], flags: Sequence[str], headers: Sequence[str] = ()) -> str:
    digest = hashlib.sha256()
    for name in list(sources) + list(headers or HEADERS):
        path = os.path.join(CSRC, name)
        digest.update(name.encode())
        with open(path, "rb") as handle:
            digest.update(handle.read())
    digest.update(" ".join(flags).encode())
    return digest.hexdigest()[:16]


def _compile_one(nvcc: str, source: str, obj: str, flags: Sequence[str]) -> None:
    started = time.time()
    _log(f"compiling {source} {' '.join(f for f in flags if f.startswith('-D'))}".rstrip())
    cmd = [nvcc, *ARCH_FLAGS, *COMMON_FLAGS, *flags, "-c",
           os.path.join(CSRC, source), "-o", obj]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {source}:\n{proc.stdout}\n{proc.stderr}")
    _log(f"compiled {source} in {time.time() - started:.1f} s")


def _build(lib_name: str, sources: Sequence[str], flags: Sequence[str]) -> str:
    out_dir = build_dir()
    lib_path = os.path.join(out_dir, lib_name)
    stamp_path = lib_path + ".hash"
    wanted = _hash(sources, flags)

    def fresh() -> bool:
        if not os.path.isfile(lib_path) or not os.path.isfile(stamp_path):
            return False
        with open(stamp_path, "r") as handle:
            return handle.read().strip() == wanted

    if fresh():
        return lib_path
    lock_path = lib_path + ".lock"
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if fresh():
                return lib_path
            nvcc = find_nvcc()
            _log(f"building {lib_name} ({len(sources)} files) with {nvcc}")
            started = time.time()
            objects: Dict[str, str] = {s: os.path.join(out_dir, f"{lib_name}.{s}.o") for s in sources}
            with ThreadPoolExecutor(max_workers=min(len(sources), os.cpu_count() or 1)) as pool:
                list(pool.map(lambda s: _compile_one(nvcc, s, objects[s], flags), sources))
            tmp_path = lib_path + f".tmp{os.getpid()}"
            cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", tmp_path, *objects.values()]
            proc = subprocess.run(cmd, capture_output=True, text=True)
            if proc.returncode != 0:
                raise BuildError(f"linking {lib_name} failed:\n{proc.stdout}\n{proc.stderr}")
            os.replace(tmp_path, lib_path)
            with open(stamp_path, "w") as handle:
                handle.write(wanted)
            for obj in objects.values():
                try:
                    os.remove(obj)
                except OSError:
                    pass
            _log(f"built {lib_name} in {time.time() - started:.1f} s")
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return lib_path


def build_runtime() -> str:
    """The host runtime, one translation unit, compiled with the host compiler."""
    out_dir = build_dir()
    lib_path = os.path.join(out_dir, "libtge_runtime.so")
    stamp_path = lib_path + ".hash"
    flags = ["-O2", "-std=c++17", "-fPIC", "-shared", "-pthread"]
    wanted = _hash(RUNTIME_SOURCES, flags, RUNTIME_HEADERS)

    def fresh() -> bool:
        if not os.path.isfile(lib_path) or not os.path.isfile(stamp_path):
            return False
        with open(stamp_path, "r") as handle:
            return handle.read().strip() == wanted

    if fresh():
        return lib_path
    with open(lib_path + ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if fresh():
                return lib_path
            compiler = find_host_compiler()
            started = time.time()
            _log(f"building libtge_runtime.so with {compiler[0]}")
            tmp_path = lib_path + f".tmp{os.getpid()}"
            if os.path.basename(compiler[0]).startswith("nvcc"):
                cmd = [*compiler, "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-Xcompiler", "-pthread", "-shared"]
            else:
                cmd = [*compiler, *flags]
            cmd += [os.path.join(CSRC, name) for name in RUNTIME_SOURCES] + ["-o", tmp_path]
            proc = subprocess.run(cmd, capture_output=True, text=True)
            if proc.returncode != 0:
                raise BuildError(f"compiling the host runtime failed:\n{proc.stdout}\n{proc.stderr}")
            os.replace(tmp_path, lib_path)
            with open(stamp_path, "w") as handle:
                handle.write(wanted)
            _log(f"built libtge_runtime.so in {time.time() - started:.1f} s")
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return lib_path


def build_core() -> str:
    return _build("libtge_core.so", CORE_SOURCES, [])


def build_attention(head_dim: int) -> str:
    if head_dim % 16 != 0 or not 16 <= head_dim <= 256:
        raise BuildError(f"the tensor-core attention kernel takes head sizes that are multiples of 16 "
                         f"up to 256, not {head_dim}")
    return _build(f"libtge_attn_hd{head_dim}.so", ["host_util.cu", "attention_mma.cu"],
                  [f"-DTGE_HEAD_DIM={head_dim}"])


def build_all(head_dims: Sequence[int] = (16, 32, 64, 128)) -> List[str]:
    paths = [build_runtime(), build_core()]
    for head_dim in head_dims:
        paths.append(build_attention(head_dim))
    return paths


if __name__ == "__main__":
    for path in build_all():
        print(path)
