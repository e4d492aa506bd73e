"""nvcc driver and in-tree cache for the core library and the generated modules.

Everything is compiled for sm_100a only and written under ``fasteq_b200/lib``
(git-ignored, shipped with the working tree).  Generated modules are keyed by a
hash of their operator signature plus the emitter version, the same role as the
reference's on-disk JIT cache (fasteq/ops/uniform1d_jit.py:444-471, :614-674),
without the auto-tuning sweep.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import threading
from typing import List, Optional

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
INCLUDE = os.path.join(ROOT, "include")
LIB = os.path.join(PKG, "lib")
JIT = os.path.join(LIB, "jit")
CORE_SO = os.path.join(LIB, "libfasteq_b200_core.so")
CORE_SOURCES = ["core.cu", "eqlinear.cu", "eqlinear_api.cu", "gemm_tf32x3.cu", "radial_chain.cu", "gate.cu", "neighbors.cu", "edge_geometry.cu"]

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-shared", "-diag-suppress", "177",
          f"-I{INCLUDE}", f"-I{CSRC}"]
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def nvcc_path() -> str:
    for cand in (os.environ.get("FASTEQ_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc not found: fasteq_b200 compiles its sm_100a kernels with nvcc and has no fallback path")


def compile_shared(sources: List[str], out_so: str, extra: Optional[List[str]] = None, verbose: bool = False) -> str:
    os.makedirs(os.path.dirname(out_so), exist_ok=True)
    tmp = out_so + f".tmp{os.getpid()}_{threading.get_ident()}"
    cmd = [nvcc_path()] + ARCH + COMMON + (extra or []) + ["-o", tmp] + sources
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"nvcc failed ({' '.join(cmd)}):\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, out_so)
    if verbose:
        print(r.stdout, r.stderr)
    return r.stdout + r.stderr


def _newer(target: str, deps: List[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps if os.path.exists(d))


def headers() -> List[str]:
    hs = [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    hs += [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    return hs


def build_core(force: bool = False) -> str:
    srcs = [os.path.join(CSRC, s) for s in CORE_SOURCES]
    with _lock:
        if force or not _newer(CORE_SO, srcs + headers()):
            compile_shared(srcs, CORE_SO, extra=["-Xptxas", "-v"])
    return CORE_SO


def build_generated(name: str, source: str, extra: Optional[List[str]] = None, force: bool = False) -> str:
    """Compile generated CUDA text into ``lib/jit/<name>.so`` unless an up-to-date build exists."""
    so = os.path.join(JIT, name + ".so")
    cu = os.path.join(JIT, name + ".cu")
    if not force and os.path.exists(so) and os.path.exists(cu):
        with open(cu) as f:
            if f.read() == source and _newer(so, headers()):
                return so
    os.makedirs(JIT, exist_ok=True)
    tmp_cu = cu + f".tmp{os.getpid()}_{threading.get_ident()}.cu"
    with open(tmp_cu, "w") as f:
        f.write(source)
    try:
        log = compile_shared([tmp_cu], so, extra=["-Xptxas", "-v"] + (extra or []))
    finally:
        if os.path.exists(tmp_cu):
            os.replace(tmp_cu, cu)
    with open(os.path.join(JIT, name + ".log"), "w") as f:
        f.write(log)
    return so
