"""Compiles the CUDA sources of this folder for sm_100a into one shared library, in-tree.

Objects and the library live in `_build/` beside the sources; a stamp of the sources' contents
and the flags decides whether anything has to be compiled again, so the first call in a fresh
checkout compiles everything (printing a line per file) and later calls only load.  Where the
folder is not writable the build goes to a per-user folder under the system's temp folder.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import time
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libwpc_kernels.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=default"]


class BuildError(RuntimeError):
    pass


def sources() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def headers() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def find_nvcc() -> str:
    for cand in (os.environ.get("WPC_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc not found (looked at WPC_NVCC, PATH, CUDA_HOME, /usr/local/cuda)")


def _digest(paths: List[str]) -> str:
    h = hashlib.sha256()
    for p in paths:
        h.update(p.encode())
        with open(os.path.join(HERE, p), "rb") as f:
            h.update(f.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()


def build_dir() -> str:
    d = os.path.join(HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"wpc_engine_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _say(msg: str) -> None:
    print(f"[wpc_engine_b200 build] {msg}", file=sys.stderr, flush=True)


def library_path(verbose: bool = True) -> str:
    """The path of an up-to-date library, compiling what is missing."""
    out_dir = build_dir()
    lib = os.path.join(out_dir, LIB_NAME)
    stamp_path = os.path.join(out_dir, "stamp.json")
    srcs, hdrs = sources(), headers()
    hdr_digest = _digest(hdrs)
    want = {s: _digest([s]) + hdr_digest for s in srcs}
    try:
        with open(stamp_path) as f:
            have = json.load(f)
    except (OSError, json.JSONDecodeError):
        have = {}
    stale = [s for s in srcs if have.get(s) != want[s] or not os.path.exists(os.path.join(out_dir, s + ".o"))]
    if not stale and os.path.exists(lib) and set(have) == set(want):
        return lib
    nvcc = find_nvcc()
    t0 = time.time()
    if verbose:
        _say(f"compiling {len(stale)} of {len(srcs)} CUDA files for sm_100a into {out_dir}")

    def compile_one(src: str) -> str:
        obj = os.path.join(out_dir, src + ".o")
        cmd = [nvcc] + ARCH_FLAGS + NVCC_FLAGS + ["-I", HERE, "-c", os.path.join(HERE, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        return src

    done = 0
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(stale)))) as pool:
        for fut in concurrent.futures.as_completed([pool.submit(compile_one, src) for src in stale]):
            src = fut.result()                 # in the order in which the files finish: a line now and then
            done += 1
            if verbose:
                _say(f"  {src} done ({done}/{len(stale)}, {time.time() - t0:.0f} s)")
    objs = [os.path.join(out_dir, s + ".o") for s in srcs]
    tmp_lib = lib + f".tmp{os.getpid()}"
    r = subprocess.run([nvcc] + ARCH_FLAGS + ["--shared", "-o", tmp_lib] + objs + ["-lcudart"],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"linking {LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp_lib, lib)
    with open(stamp_path, "w") as f:
        json.dump(want, f)
    if verbose:
        _say(f"built {lib} in {time.time() - t0:.0f} s")
    return lib


if __name__ == "__main__":
    print(library_path())
