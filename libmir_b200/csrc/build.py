"""Compiling the CUDA sources for sm_100a with nvcc into shared libraries, and finding them again.

There are two libraries so that a run compiles only what its model needs:
  core   kernels of both engine dtypes (norms, rotary + cache write, reference attention, 32-bit
         matrix product, sampling) and the layer executor for the float32 engine
  bf16   the same, and what only the bfloat16 engine uses (tensor-core attention, cuBLASLt and tcgen05
         products, the choice between them), with the layer executor for both engine dtypes
A library is rebuilt when the hash of its sources and flags changes.  Objects are compiled in
parallel, and a line is printed for each so that a first call shows progress.  The libraries are
written beside the package (libmir_b200/_lib) when that folder can be written, else under the
system's temporary folder.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

from ..errors import KernelError

HERE = Path(__file__).resolve().parent
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden"]

LIBRARIES = {
    "core": {
        "sources": ["runtime.cu", "elementwise.cu", "qk_rope_store.cu", "attention_generic.cu", "gemm_f32.cu",
                    "sampling.cu", "executor.cu"],
        "link": [],
        "defines": [],
    },
    # everything of `core` as well: the layer executor of this library runs both engine dtypes
    "bf16": {
        "sources": ["runtime.cu", "elementwise.cu", "qk_rope_store.cu", "attention_generic.cu", "gemm_f32.cu",
                    "gemm_lt.cu", "attention_mma.cu", "gemm_tc.cu", "attention_tc.cu", "attention_tc_decode.cu",
                    "gemm_tc_stream.cu", "ops_bf16.cu", "executor.cu"],
        "headers": ["no_alloc.h", "tcgen05.cuh"],
        "link": ["-lcublasLt"],
        "defines": ["-DMIR_WITH_BF16"],
    },
}
# the bfloat16 library with time stamps inside its kernels (trace.cuh), for bench.py --phase trace
LIBRARIES["bf16_trace"] = dict(LIBRARIES["bf16"], defines=LIBRARIES["bf16"]["defines"] + ["-DMIR_TRACE"])
HEADERS = ["common.cuh", "launchers.h", "trace.cuh"]


def _nvcc() -> str:
    for candidate in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.access(candidate, os.X_OK):
            return candidate
    raise KernelError("nvcc was not found (looked on PATH and in /usr/local/cuda/bin): the CUDA kernels of "
                      "libmir_b200 cannot be compiled, and there is no fallback without them")


def _digest(name: str) -> str:
    h = hashlib.sha256()
    spec = LIBRARIES[name]
    for rel in spec["sources"] + HEADERS + spec.get("headers", []):
        h.update(rel.encode())
        h.update((HERE / rel).read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + spec["link"] + spec.get("defines", [])).encode())
    return h.hexdigest()[:16]


def _writable_dir() -> Path:
    in_tree = HERE.parent / "_lib"
    try:
        in_tree.mkdir(exist_ok=True)
        probe = in_tree / f".probe-{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return in_tree
    except OSError:
        fallback = Path(tempfile.gettempdir()) / f"libmir_b200-lib-{os.getuid()}"
        fallback.mkdir(exist_ok=True)
        return fallback


def _candidate_dirs() -> list:
    return [HERE.parent / "_lib", Path(tempfile.gettempdir()) / f"libmir_b200-lib-{os.getuid()}"]


def library_path(name: str) -> Path | None:
    """The built library for the current sources, if there is one."""
    file_name = f"libmir_{name}-{_digest(name)}.so"
    for folder in _candidate_dirs():
        if (folder / file_name).is_file():
            return folder / file_name
    return None


def _say(message: str, verbose: bool) -> None:
    if verbose:
        print(f"[libmir_b200 build] {message}", file=sys.stderr, flush=True)


def build(name: str, verbose: bool = True, force: bool = False) -> Path:
    """Compile library `name` if it is missing or stale; returns its path."""
    if name not in LIBRARIES:
        raise KernelError(f"unknown kernel library {name!r}; known: {', '.join(LIBRARIES)}")
    existing = None if force else library_path(name)
    if existing is not None:
        return existing
    nvcc = _nvcc()
    spec = LIBRARIES[name]
    out_dir = _writable_dir()
    digest = _digest(name)
    work = out_dir / "_build" / f"{name}-{digest}-{os.getpid()}"
    work.mkdir(parents=True, exist_ok=True)
    started = time.time()
    _say(f"compiling {name} ({len(spec['sources'])} files) for sm_100a with {nvcc}", verbose)

    def compile_one(rel: str) -> Path:
        obj = work / (Path(rel).stem + ".o")
        t0 = time.time()
        command = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *spec.get("defines", []), "-I", str(HERE), "-c", str(HERE / rel),
                   "-o", str(obj)]
        done = subprocess.run(command, capture_output=True, text=True)
        if done.returncode != 0:
            raise KernelError(f"nvcc failed on {rel}:\n{done.stdout}\n{done.stderr}")
        _say(f"  {rel} compiled in {time.time() - t0:.1f}s", verbose)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(spec["sources"]))) as pool:
        objects = list(pool.map(compile_one, spec["sources"]))
    target = out_dir / f"libmir_{name}-{digest}.so"
    partial = work / target.name
    command = [nvcc, "-shared", *ARCH_FLAGS, "-o", str(partial), *[str(o) for o in objects],
               "-L/usr/local/cuda/lib64", "-Xlinker", "-rpath=/usr/local/cuda/lib64", *spec["link"]]
    done = subprocess.run(command, capture_output=True, text=True)
    if done.returncode != 0:
        raise KernelError(f"linking {target.name} failed:\n{done.stdout}\n{done.stderr}")
    os.replace(partial, target)   # atomic: a concurrent builder sees the old state or the whole file
    shutil.rmtree(work, ignore_errors=True)
    for stale in out_dir.glob(f"libmir_{name}-*.so"):
        if stale != target:
            try:
                stale.unlink()
            except OSError:
                pass
    _say(f"{target.name} ready in {time.time() - started:.1f}s", verbose)
    return target


def build_all(verbose: bool = True, force: bool = False) -> dict:
    return {name: build(name, verbose=verbose, force=force) for name in LIBRARIES}


if __name__ == "__main__":
    for lib_name, lib_path in build_all(force="--force" in sys.argv).items():
        print(lib_name, lib_path)
