"""Build the PE-attention C-ABI library in-tree with nvcc for sm_100a.

``python -m pe_ablations_b200.build_ext`` (or ``build()``) compiles
``csrc/*.cu`` into ``pe_ablations_b200/libpe_attn.so``.  nvcc cross-compiles
without a GPU; the built library is what the GPU box loads.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libpe_attn.so")
SOURCES = ["pe_attn_abi.cu", "pe_attn_simt.cu", "pe_attn_tc.cu", "pe_attn_tc2.cu", "pe_attn_tc4.cu", "pe_attn_ce.cu", "pe_attn_elementwise.cu",
           "pe_attn_bwd.cu", "pe_attn_bwd_simt.cu", "pe_attn_xform.cu", "pe_attn_decode.cu", "pe_attn_gemm.cu"]
HEADERS = ["pe_attn_common.cuh", "pe_attn_ptx.cuh", "pe_attn_tc_common.cuh", os.path.join("..", "..", "include", "pe_attn.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or add it to PATH")


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False, defines: tuple[str, ...] = ()) -> str:
    """Compile (if stale) and return the path of the shared library.  ``defines`` adds -D macros
    to a forced build (e.g. ``PE_GEMM_TRACE``: per-role clock counters in the GEMM kernel, read
    by ``bench.py --workload gemm``); rebuild with ``--force`` afterwards to drop them."""
    nvcc = _nvcc()
    force = force or bool(defines)
    srcs = [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    hdrs = [os.path.join(CSRC, h) for h in HEADERS]
    objs = []
    procs = []
    for s in srcs:
        src = os.path.join(CSRC, s)
        obj = os.path.join(CSRC, s.replace(".cu", ".o"))
        objs.append(obj)
        if force or _stale(obj, [src] + hdrs):
            cmd = [nvcc, *NVCC_FLAGS, *[f"-D{d}" for d in defines], "-c", src, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for name, pr in procs:
        out, _ = pr.communicate()
        if verbose or pr.returncode != 0:
            sys.stderr.write(out)
        if pr.returncode != 0:
            raise RuntimeError(f"nvcc failed on {name}")
    if force or procs or _stale(LIB_PATH, objs):
        cmd = [nvcc, "-shared", "-o", LIB_PATH, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout)
            raise RuntimeError("link failed")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv,
                defines=tuple(a[2:] for a in sys.argv[1:] if a.startswith("-D"))))
