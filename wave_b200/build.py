"""Build libwave_b200.so in-tree with nvcc for sm_100a (`python -m wave_b200.build`)."""

from __future__ import annotations

import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT = PKG / "libwave_b200.so"
SOURCES = [CSRC / "api.cu"]
HEADERS = sorted(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "wave_b200.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def needs_build() -> bool:
    if not OUT.exists():
        return True
    t = OUT.stat().st_mtime
    return any(p.stat().st_mtime > t for p in SOURCES + HEADERS)


TRACE_OUT = PKG / "libwave_b200_trace.so"
CHECKS_OUT = PKG / "libwave_b200_checks.so"
CEILING_OUT = PKG / "libwave_b200_mma_ceiling.so"


def _stale(out: Path) -> bool:
    return not out.exists() or any(p.stat().st_mtime > out.stat().st_mtime for p in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False, trace: bool = False, checks: bool = False,
          mma_ceiling: bool = False) -> Path:
    """Compile the library if it is missing or older than its sources. Returns its path.
    `trace`: the measurement variant with per-CTA timeline marks in the skinny kernels (-DWB200_TRACE), written to
    libwave_b200_trace.so; load it with WAVE_B200_LIB=... (see `python -m wave_b200.perf --timeline`).
    `checks`: the debug-checked variant (-DWB200_CHECKS: index predicates in front of every copy-engine issue and
    global store, see csrc/checks.cuh), written to libwave_b200_checks.so.
    `mma_ceiling`: a measurement variant of the tile kernels (-DWB200_MMA_CEILING) that loads only the first ring of
    stages and never reads the accumulators, so that what remains is the scale-factor copies and the MMAs on
    operands resident in shared memory: the tensor pipe's ceiling for this tile shape under the GPU's power limit
    (`python -m wave_b200.perf --mma-ceiling`). Its results are wrong by construction; never load it for anything else."""
    out = TRACE_OUT if trace else CHECKS_OUT if checks else CEILING_OUT if mma_ceiling else OUT
    if not force and not _stale(out):
        return out
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    variant = ["-DWB200_TRACE"] if trace else ["-DWB200_CHECKS"] if checks else ["-DWB200_MMA_CEILING"] if mma_ceiling else []
    cmd = [nvcc, *NVCC_FLAGS, *variant, "-o", str(out), *map(str, SOURCES)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
        print(" ".join(cmd))
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed ({res.returncode}):\n{res.stdout}\n{res.stderr}")
    if verbose:
        print(res.stderr)
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, trace="--trace" in sys.argv, checks="--checks" in sys.argv,
                mma_ceiling="--mma-ceiling" in sys.argv))
