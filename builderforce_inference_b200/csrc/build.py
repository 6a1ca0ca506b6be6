"""Building the kernel libraries with nvcc for sm_100a.

The sources are grouped into libraries; a run builds only the groups it asks for, on first use,
and prints a line now and then while nvcc works.  Objects and libraries are kept beside the
sources (``_build/``), or in a per-user temporary folder when the package folder cannot be
written.  A library is rebuilt when a source, a header or the flags change.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List

HERE = os.path.dirname(os.path.abspath(__file__))

# library name -> sources.  "core": every kernel of the 32-bit path and the general fallbacks of
# the bfloat16 path.  "fast": the bfloat16 kernels written for the tensor cores and for
# streaming weights and the cache at memory speed.
LIBRARIES: Dict[str, List[str]] = {
    "core": ["errors.cu", "elementwise.cu", "gemm_simt.cu", "attention_paged.cu", "sampling.cu", "utility.cu"],
    "fast": ["errors.cu", "skinny_gemm.cu", "attention_decode.cu", "attention_prefill.cu", "gemm_tcgen05.cu",
             "attention_prefill_tcgen05.cu", "weight_stream.cu"],
}

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
# BFI_B200_TRACE=1 builds libraries whose kernels stamp a timeline (common.cuh); never the default
if os.environ.get("BFI_B200_TRACE", "0") == "1":
    NVCC_FLAGS = NVCC_FLAGS + ["-DBFI_TRACE"]


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for root in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if root and os.path.isfile(os.path.join(root, "bin", "nvcc")):
            return os.path.join(root, "bin", "nvcc")
    found = shutil.which("nvcc")
    if found:
        return found
    raise BuildError("nvcc not found (looked in $CUDA_HOME, /usr/local/cuda and PATH); "
                     "the CUDA kernels cannot be built and there is no other path")


def build_dir() -> str:
    override = os.environ.get("BFI_B200_BUILD_DIR")
    if override:
        os.makedirs(override, exist_ok=True)
        return override
    local = os.path.join(HERE, "_build")
    try:
        os.makedirs(local, exist_ok=True)
        probe = os.path.join(local, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return local
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"bfi_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h", ".inl")))


def _digest(src: str, extra_flags: List[str]) -> str:
    h = hashlib.sha256()
    for name in [src] + _headers():
        with open(os.path.join(HERE, name), "rb") as f:
            h.update(name.encode())
            h.update(f.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + extra_flags).encode())
    return h.hexdigest()[:16]


def _say(msg: str) -> None:
    print(f"[bfi-b200 build] {msg}", file=sys.stderr, flush=True)


def _compile_one(nvcc: str, src: str, obj: str, extra_flags: List[str]) -> None:
    cmd = [nvcc] + ARCH_FLAGS + NVCC_FLAGS + extra_flags + ["-I", HERE, "-c", os.path.join(HERE, src), "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"nvcc failed on {src}:\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")


def library_path(name: str, verbose_flags: bool = False) -> str:
    """Path of the up-to-date shared library ``name``, building whatever is stale."""
    if name not in LIBRARIES:
        raise BuildError(f"unknown kernel library '{name}'; known: {sorted(LIBRARIES)}")
    out_dir = build_dir()
    extra = ["-Xptxas", "-v"] if verbose_flags else []
    sources = LIBRARIES[name]
    digests = {s: _digest(s, extra) for s in sources}
    tag = hashlib.sha256("".join(digests[s] for s in sources).encode()).hexdigest()[:16]
    lib = os.path.join(out_dir, f"libbfi_b200_{name}_{tag}.so")
    if os.path.isfile(lib):
        return lib
    nvcc = find_nvcc()
    todo = []
    objs = []
    for s in sources:
        obj = os.path.join(out_dir, f"{os.path.splitext(s)[0]}_{digests[s]}.o")
        objs.append(obj)
        if not os.path.isfile(obj):
            todo.append((s, obj))
    _say(f"building library '{name}' for sm_100a: {len(todo)} of {len(sources)} files to compile")
    t0 = time.time()
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            _say(f"... still compiling '{name}' ({time.time() - t0:.0f} s)")

    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    try:
        with ThreadPoolExecutor(max_workers=min(8, max(1, len(todo)))) as pool:
            futs = []
            for s, obj in todo:
                tmp = f"{obj}.{os.getpid()}.tmp"
                futs.append((s, obj, tmp, pool.submit(_compile_one, nvcc, s, tmp, extra)))
            for s, obj, tmp, f in futs:
                f.result()
                os.replace(tmp, obj)
                _say(f"compiled {s}")
        tmp_lib = f"{lib}.{os.getpid()}.tmp"
        cmd = [nvcc, "-shared"] + ARCH_FLAGS + ["-o", tmp_lib] + objs + ["-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"linking {name} failed:\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
        os.replace(tmp_lib, lib)
    finally:
        done.set()
    _say(f"library '{name}' ready in {time.time() - t0:.0f} s: {lib}")
    return lib


def build_all() -> Dict[str, str]:
    return {name: library_path(name) for name in LIBRARIES}


if __name__ == "__main__":
    for n, p in build_all().items():
        print(n, p)
