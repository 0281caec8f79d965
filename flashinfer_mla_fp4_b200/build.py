"""Build libmla_fp4_b200.so in-tree with nvcc for sm_100a (no torch dependency in the library)."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = Path(os.environ.get("MLA_FP4_B200_LIB") or (PKG_DIR / "libmla_fp4_b200.so"))
SOURCES = ["abi.cu", "kernels_simt.cu", "combine.cu", "cache_write.cu", "cp_exchange.cu", "decode_sm100.cu"]
HEADERS = ["common.cuh", "dequant.cuh", "launch.h", "ptx_sm100.cuh", "../../include/mla_fp4_b200.h"]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC")
    return cand


def needs_build() -> bool:
    if not LIB_PATH.exists():
        return True
    t = LIB_PATH.stat().st_mtime
    deps = [CSRC / s for s in SOURCES] + [(CSRC / h).resolve() for h in HEADERS] + [Path(__file__)]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every CUDA source for sm_100a into one shared library next to this file."""
    if not force and not needs_build():
        return LIB_PATH
    objs = []
    build_dir = PKG_DIR / "build"
    build_dir.mkdir(exist_ok=True)
    common = [
        _nvcc(), "-std=c++17", "-O3", "-lineinfo",
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-Xcompiler", "-fPIC", "-Xptxas", "-v" if verbose else "-O3",
        "--expt-relaxed-constexpr",
    ] + os.environ.get("MLA_FP4_NVCC_FLAGS", "").split()
    procs = []
    for s in SOURCES:
        o = build_dir / (s + ".o")
        objs.append(str(o))
        procs.append((s, subprocess.Popen(common + ["-c", str(CSRC / s), "-o", str(o)],
                                          stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for s, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(f"--- nvcc {s}\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    link = [_nvcc(), "-shared", "-o", str(LIB_PATH)] + objs + ["-cudart", "static"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("link failed")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
