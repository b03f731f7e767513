"""Builds the CUDA library (sm_100a only) in-tree with nvcc.

    python -m fp4_post_b200.build        # or: from fp4_post_b200.build import build; build()

Output: fp4_post_b200/_lib/libmetis_nvfp4.so.  nvcc cross-compiles without a GPU.

    python -m fp4_post_b200.build --timing-knobs

builds a second library, _lib/libmetis_nvfp4_knobs.so, with -DMETIS_TIMING_KNOBS: the GEMM then accepts
bits in metis_gemm_args.reserved that switch parts of it off (no loads, no MMAs, no scale copies, no
epilogue) and make the issuing warp of CTA 0 write its cycle counts to the status words.  Results of such
runs are meaningless; `bench.py --only gemm_accounting` uses them to say where a tile's cycles go.  The
shipped library rejects the bits and contains none of that code.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT_DIR = PKG / "_lib"
LIB = OUT_DIR / "libmetis_nvfp4.so"
KNOBS_LIB = OUT_DIR / "libmetis_nvfp4_knobs.so"
SOURCES = ["api.cu", "quantize.cu", "rmsnorm_quant.cu", "dequantize.cu", "gemm_tcgen05.cu", "gemm_tcgen05_pair.cu", "lowrank_bwd.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC or install the CUDA toolkit)")


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False, timing_knobs: bool = False) -> Path:
    """Compile every .cu file to an object and link the shared library. Returns its path."""
    nvcc = _nvcc()
    OUT_DIR.mkdir(exist_ok=True)
    obj_dir, lib, extra = OUT_DIR, LIB, []
    if timing_knobs:
        obj_dir, lib, extra = OUT_DIR / "knobs", KNOBS_LIB, ["-DMETIS_TIMING_KNOBS"]
        obj_dir.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "metis_nvfp4.h"]
    objs = []
    procs = []
    for src in SOURCES:
        obj = obj_dir / (src + ".o")
        objs.append(obj)
        if force or _stale(obj, [CSRC / src] + headers):
            cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", str(CSRC / src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
                print(" ".join(cmd), file=sys.stderr)
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = []
    for src, p in procs:
        out, _ = p.communicate()
        if verbose and out:
            print(out, file=sys.stderr)
        if p.returncode != 0:
            failed.append((src, out))
    if failed:
        raise RuntimeError("nvcc failed:\n" + "\n".join(f"--- {s} ---\n{o}" for s, o in failed))
    if force or procs or _stale(lib, objs):
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(lib), *map(str, objs)]
        subprocess.run(cmd, check=True)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, timing_knobs="--timing-knobs" in sys.argv))
