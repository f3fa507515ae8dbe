"""Build libflashdmla.so (sm_100a only) in-tree with nvcc.

    python ds-flashdmla-moe_b200/build.py [--force] [--verbose] [--timeline [--ablate BITS]]

Every .cu under csrc/ is compiled with
`-gencode arch=compute_100a,code=sm_100a -lineinfo` and linked into
flashdmla/libflashdmla.so.  The CUDA runtime is linked statically and the
driver API is reached through cudaGetDriverEntryPoint, so the library loads on
a machine without a GPU driver (symbol checks, CPU-only test runs).

--timeline builds a second library, flashdmla/libflashdmla_timeline.so, with
-DFDMLA_TIMELINE: the 2-CTA forward kernel then stamps what every CTA pair does
with the global timer and the launcher appends the stamps of every launch to
the file named by FDMLA_TIMELINE_FILE (select the library with FLASHDMLA_LIB;
timeline_report.py beside this file runs a decode launch that way and prints the
summary).  --ablate BITS (with --timeline) builds libflashdmla_timeline_ablBITS.so,
in which that kernel leaves out one stage of its pipeline - 1: the K/V copies, 2:
the softmax arithmetic, 4: the MMAs - so that the cost of the rest can be timed;
its results are garbage.  Development aids; the ordinary library contains none of it.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
OUT = os.path.join(HERE, "flashdmla", "libflashdmla.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-I", INCLUDE,
]


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _newest_header() -> float:
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(INCLUDE, "flashdmla.h"))
    return max(os.path.getmtime(h) for h in hs)


def build(force: bool = False, verbose: bool = False, timeline: bool = False, ablate: int = 0) -> str:
    tag = ("_timeline" + (f"_abl{ablate}" if ablate else "")) if timeline else ""
    obj_dir = OBJ + tag
    out = OUT.replace(".so", tag + ".so")
    extra = (["-DFDMLA_TIMELINE"] + ([f"-DFDMLA_ABLATE={ablate}"] if ablate else [])) if timeline else []
    os.makedirs(obj_dir, exist_ok=True)
    hdr = _newest_header()
    jobs = []
    for src in _sources():
        s = os.path.join(CSRC, src)
        o = os.path.join(obj_dir, src[:-3] + ".o")
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr):
            cmd = ["nvcc", *NVCC_FLAGS, *extra, "-c", s, "-o", o]
            if verbose:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))

    with ThreadPoolExecutor(max_workers=4) as ex:
        list(ex.map(run, jobs))
    objs = [os.path.join(obj_dir, s[:-3] + ".o") for s in _sources()]
    if jobs or not os.path.exists(out):
        run(["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", out, *objs])
    return out


if __name__ == "__main__":
    abl = int(sys.argv[sys.argv.index("--ablate") + 1]) if "--ablate" in sys.argv else 0
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, timeline="--timeline" in sys.argv, ablate=abl))
