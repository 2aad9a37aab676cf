"""Builds tensorlisp_b200/libtlb200.so (sm_100a only) in-tree with nvcc.

    python -m tensorlisp_b200.build [--force] [--verbose]

Every .cu under csrc/ is compiled to an object (in parallel) and linked into one shared library
that exports exactly the C ABI of include/tlb200.h. k_quant.cu is compiled with -fmad=false: the
row quantizers must round every intermediate the way the reference's no-FMA build does.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "build"
LIB = HERE / "libtlb200.so"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", 
          "-Xcompiler", "-Wall", "--expt-relaxed-constexpr", "-DTLB_BUILDING"]
PER_FILE = {"k_quant.cu": ["-fmad=false"], "k_fused.cu": ["-fmad=false"]}


def _nvcc() -> str:
    for c in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if c and (os.path.sep not in c or os.path.exists(c)):
            return c
    raise RuntimeError("nvcc not found")


def _run(cmd: list[str], verbose: bool) -> str:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout[-6000:], r.stderr[-6000:]))
    if verbose:
        sys.stderr.write(r.stdout + r.stderr)
    return r.stdout + r.stderr


def build(force: bool = False, verbose: bool = False) -> Path:
    srcs = sorted(CSRC.glob("*.cu"))
    hdrs = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "tlb200.h"]
    newest_hdr = max(h.stat().st_mtime for h in hdrs)
    OBJ.mkdir(exist_ok=True)
    nvcc = _nvcc()
    jobs, objs = [], []
    for s in srcs:
        o = OBJ / (s.stem + ".o")
        objs.append(o)
        if force or not o.exists() or o.stat().st_mtime < max(s.stat().st_mtime, newest_hdr):
            extra = ["-Xptxas", "-v"] if verbose else []
            jobs.append([nvcc] + ARCH + COMMON + PER_FILE.get(s.name, []) + extra + ["-c", str(s), "-o", str(o)])
    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        list(ex.map(lambda c: _run(c, verbose), jobs))
    if jobs or force or not LIB.exists():
        _run([nvcc] + ARCH + ["-shared", "-o", str(LIB)] + [str(o) for o in objs] + ["-ldl"], verbose)
    return LIB


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))


if __name__ == "__main__":
    main()
