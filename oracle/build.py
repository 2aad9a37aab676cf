"""TEST INFRASTRUCTURE ONLY: builds the checkers, never anything the product path runs.

(a) ``liboracle.so``  -- the plain-C restatement of the reference's algorithms (oracle/oracle.c).
(b) ``_ref/libtlref_<variant>.so`` -- when a reference checkout is present, the reference's own
    vendored ggml CPU backend + row quantizers behind oracle/ref_harness.cpp. The sources are
    compiled where they lie (file list and defines of the reference's
    crates/ggml-sys/build.rs:357-418); nothing is copied into this repository.

Variants of (b):
  base : -O3 only, like the reference's own build (no -march, hence no FMA contraction).
         The canonical parity oracle; "bit-exact" quantizers are defined against this build.
  v3   : -O3 -march=x86-64-v3                 (AVX2+FMA)  } timed CPU baselines, picked at run
  v4   : -O3 -march=x86-64-v4 -mavx512vnni    (AVX-512)   } time from the host's cpu flags

Usage: python oracle/build.py [--ref /path/to/reference] [--variants base,v3,v4] [--force]
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"

VARIANT_FLAGS = {
    "base": [],
    "v3": ["-march=x86-64-v3"],
    "v4": ["-march=x86-64-v4", "-mavx512vnni"],
}

C_SRCS = ["ggml.c", "ggml-alloc.c", "ggml-quants.c", "ggml-cpu/quants.c", "ggml-cpu/ggml-cpu.c",
          "ggml-cpu/arch/x86/quants.c"]
CXX_SRCS = ["ggml-cpu/repack.cpp", "ggml-cpu/vec.cpp", "ggml-cpu/hbm.cpp", "ggml-cpu/traits.cpp",
            "ggml-cpu/binary-ops.cpp", "ggml-cpu/unary-ops.cpp", "ggml-cpu/ops.cpp",
            "ggml-cpu/ggml-cpu.cpp", "ggml-cpu/llamafile/sgemm.cpp", "ggml.cpp", "ggml-backend.cpp",
            "ggml-backend-meta.cpp", "ggml-backend-dl.cpp", "ggml-backend-reg.cpp",
            "ggml-threading.cpp", "gguf.cpp", "ggml-cpu/arch/x86/repack.cpp",
            "ggml-cpu/arch/x86/cpu-feats.cpp"]


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s" % (" ".join(cmd), r.stderr[-4000:]))


def build_oracle(force: bool = False) -> Path:
    so = HERE / "liboracle.so"
    srcs = [HERE / "oracle.c", HERE / "oracle.h"]
    if force or not so.exists() or any(s.stat().st_mtime > so.stat().st_mtime for s in srcs):
        # -ffp-contract=off: the reference's build has no FMA, and the Q4_K search depends on it.
        _run(["gcc", "-O2", "-fPIC", "-ffp-contract=off", "-fno-fast-math", "-shared",
              str(HERE / "oracle.c"), "-o", str(so), "-lm"])
    return so


def build_ref(ref: Path, variants: list[str], force: bool = False) -> list[Path]:
    ggml = ref / "vendor" / "ggml"
    src = ggml / "src"
    if not (src / "ggml.c").exists():
        return []
    defs = ['-DGGML_VERSION="unknown"', '-DGGML_COMMIT="unknown"', "-DGGML_USE_CPU",
            "-DGGML_USE_LLAMAFILE", "-D_GNU_SOURCE"]
    incs = ["-I%s" % (ggml / "include"), "-I%s" % src, "-I%s" % (src / "ggml-cpu")]
    built = []
    for v in variants:
        so = OUT / ("libtlref_%s.so" % v)
        harness = HERE / "ref_harness.cpp"
        if so.exists() and not force and so.stat().st_mtime > harness.stat().st_mtime:
            built.append(so)
            continue
        objdir = OUT / ("obj_" + v)
        objdir.mkdir(parents=True, exist_ok=True)
        flags = ["-O3", "-fPIC", "-w"] + VARIANT_FLAGS[v] + defs + incs
        jobs = []
        for s in C_SRCS:
            o = objdir / (s.replace("/", "_") + ".o")
            if force or not o.exists():
                jobs.append(["gcc"] + flags + ["-c", str(src / s), "-o", str(o)])
        for s in CXX_SRCS:
            o = objdir / (s.replace("/", "_") + ".o")
            if force or not o.exists():
                jobs.append(["g++", "-std=c++17"] + flags + ["-c", str(src / s), "-o", str(o)])
        with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
            list(ex.map(_run, jobs))
        objs = sorted(str(p) for p in objdir.glob("*.o"))
        tag = "-O3 " + " ".join(VARIANT_FLAGS[v])
        _run(["g++", "-std=c++17"] + flags + ['-DTLREF_FLAGS="%s"' % tag.strip(), "-shared", str(harness)]
             + objs + ["-o", str(so), "-lpthread", "-ldl", "-lm"])
        built.append(so)
    return built


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("TENSORLISP_REFERENCE") or str(Path(__file__).resolve().parent.parent.parent / "reference"),
                    help="checkout of the reference (default: TENSORLISP_REFERENCE, else a `reference` directory beside this repository)")
    ap.add_argument("--variants", default="base,v3,v4")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print("oracle:", build_oracle(a.force))
    for so in build_ref(Path(a.ref), a.variants.split(","), a.force):
        print("ref:", so)


if __name__ == "__main__":
    sys.exit(main())
