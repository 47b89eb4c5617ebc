"""Builds the CUDA kernels into a shared library the first time they are needed.

The kernels are plain `extern "C"` entry points compiled with nvcc for sm_100a and
opened with ctypes, so nothing depends on a home directory, a network, or a Python
extension cache.  The library lands in `_build/` beside the sources when that folder
can be written, else in a per-user folder under the system's temporary directory.
Its file name carries a hash of the sources and flags: a changed source makes a new
library, an unchanged one is reused.
"""
from __future__ import annotations

import hashlib
import functools
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Sequence

CSRC = Path(__file__).resolve().parent

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]

# Sources that do not depend on a model size.
CORE_SOURCES = ["errors.cu", "elementwise.cu", "attn_simple.cu", "gemm_simt.cu", "gemm_tc.cu", "gemm_tc2.cu",
                "fused_reduce.cu", "sampling.cu"]
HEADERS = ["common.cuh", "rowscale.cuh", "streamk.cuh", "tcgen05.cuh", "attn_noalloc.h", "page.h", "trace.cuh"]


class BuildError(RuntimeError):
    pass


@functools.lru_cache(maxsize=None)
def page_size() -> int:
    """Positions per cache page: read from page.h, the one place the number is written."""
    import re
    m = re.search(r"^#define\s+BRAID_PAGE_SIZE\s+(\d+)\s*$", (CSRC / "page.h").read_text(), re.M)
    if not m:
        raise BuildError("page.h does not define BRAID_PAGE_SIZE")
    return int(m.group(1))


def find_nvcc() -> str:
    cands = []
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            cands.append(os.path.join(os.environ[var], "bin", "nvcc"))
    cands.append("/usr/local/cuda/bin/nvcc")
    which = shutil.which("nvcc")
    if which:
        cands.append(which)
    for c in cands:
        if os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise BuildError("nvcc was not found (looked in CUDA_HOME, /usr/local/cuda/bin and PATH); "
                     "the CUDA kernels cannot be compiled")


def _say(msg: str) -> None:
    print(f"[braidinfer_b200] {msg}", file=sys.stderr, flush=True)


def build_dir() -> Path:
    env = os.environ.get("BRAIDINFER_BUILD_DIR")
    if env:
        p = Path(env)
        p.mkdir(parents=True, exist_ok=True)
        return p
    local = CSRC / "_build"
    try:
        local.mkdir(exist_ok=True)
        probe = local / f".probe{os.getpid()}"
        probe.write_text("x")
        probe.unlink()
        return local
    except OSError:
        p = Path(tempfile.gettempdir()) / f"braidinfer_b200_build_{os.getuid()}"
        p.mkdir(parents=True, exist_ok=True)
        return p


def _digest(sources: Sequence[str], defines: Sequence[str]) -> str:
    h = hashlib.sha256()
    for name in list(sources) + HEADERS:
        h.update(name.encode())
        h.update((CSRC / name).read_bytes())
    h.update(" ".join(ARCH_FLAGS + COMMON_FLAGS + list(defines)).encode())
    return h.hexdigest()[:16]


def _run(cmd: List[str], what: str) -> None:
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    if r.returncode != 0:
        raise BuildError(f"{what} failed (exit {r.returncode}):\n{' '.join(cmd)}\n{r.stdout}")


def build_library(name: str, sources: Sequence[str], defines: Sequence[str] = (), verbose: bool = True) -> Path:
    """Compile `sources` (names under csrc/) into lib<name>-<hash>.so and return its path."""
    out_dir = build_dir()
    tag = _digest(sources, defines)
    target = out_dir / f"lib{name}-{tag}.so"
    if target.exists():
        return target
    nvcc = find_nvcc()
    work = Path(tempfile.mkdtemp(prefix=f"{name}-", dir=str(out_dir)))
    t0 = time.time()
    if verbose:
        _say(f"compiling {len(sources)} CUDA source file(s) for sm_100a into {target.name} ...")
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            _say(f"still compiling ({time.time() - t0:.0f} s) ...")

    th = threading.Thread(target=ticker, daemon=True)
    if verbose:
        th.start()
    try:
        objs = []

        def compile_one(src: str) -> str:
            obj = str(work / (Path(src).stem + ".o"))
            _run([nvcc, *ARCH_FLAGS, *COMMON_FLAGS, *defines, "-I", str(CSRC), "-c", str(CSRC / src), "-o", obj],
                 f"compiling {src}")
            return obj

        with ThreadPoolExecutor(max_workers=min(8, len(sources))) as ex:
            objs = list(ex.map(compile_one, sources))
        tmp_target = work / target.name
        _run([nvcc, "-shared", *ARCH_FLAGS, "-cudart", "static", "-o", str(tmp_target), *objs], "linking")
        os.replace(tmp_target, target)       # atomic: concurrent builders agree on the result
        for old in out_dir.glob(f"lib{name}-*.so"):      # libraries of earlier sources are of no use
            if old != target:
                try:
                    old.unlink()
                except OSError:
                    pass
    finally:
        done.set()
        shutil.rmtree(work, ignore_errors=True)
    if verbose:
        _say(f"built {target.name} in {time.time() - t0:.1f} s")
    return target


def trace_build() -> bool:
    """BRAIDINFER_TRACE=1: the library is built with phase time stamps in its product and reduce
    kernels (csrc/trace.cuh).  A library of its own name; the ordinary one is left alone."""
    return os.environ.get("BRAIDINFER_TRACE", "0") not in ("", "0")


def core_library(verbose: bool = True) -> Path:
    if trace_build():
        return build_library("braidinfer_core_trace", CORE_SOURCES, defines=["-DBRAID_TRACE"], verbose=verbose)
    return build_library("braidinfer_core", CORE_SOURCES, verbose=verbose)


def attention_library(head_dim: int, verbose: bool = True) -> Path:
    """The tensor-core attention kernels compiled for one head size (what a model needs
    is compiled when the model is first built)."""
    return build_library(f"braidinfer_attn_hd{head_dim}", ["errors.cu", "attn_mma.cu", "attn_tc.cu"],
                         defines=[f"-DBRAID_HD={head_dim}"], verbose=verbose)
