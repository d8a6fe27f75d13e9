"""Compiles weft_b200/csrc into weft_b200/libweft_b200.so with nvcc for sm_100a.

The library is built in-tree so that it travels with the repository snapshot; nothing is cached
outside the tree.  ``python -m weft_b200.build`` rebuilds it; ``ensure_built()`` is what importers
call (it only compiles when a source is newer than the library).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
CSRC = PACKAGE / "csrc"
LIBRARY = PACKAGE / "libweft_b200.so"
SOURCES = ["abi.cu", "abi_noalloc.cu", "dequantize.cu", "quantize.cu", "gemv.cu", "gemv_q4k.cu", "gemv_ring.cu", "gemv_q4ki.cu", "prefill.cu", "prefill_pair.cu", "prefill_blocks.cu", "mma_peak.cu", "gather.cu"]
HEADERS = ["common.cuh", "quantize.cuh", "kernels.h", "gemv_units.cuh", "ring.cuh", "tcgen05.cuh", "tensormap.cuh", "prefill_common.cuh", "gather.cuh", "../../include/weft_b200.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    # IEEE division and square root, no flush-to-zero, no fused contraction surprises in the
    # bit-exact kernels (they spell their ops with __fmul_rn/__fsub_rn as well)
    "--prec-div=true", "--prec-sqrt=true", "--ftz=false",
]


def nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return found


def stale() -> bool:
    if not LIBRARY.exists():
        return True
    built = LIBRARY.stat().st_mtime
    return any((CSRC / name).stat().st_mtime > built for name in SOURCES + HEADERS)


def build(verbose: bool = False, extra: list[str] | None = None) -> Path:
    objects = []
    obj_dir = PACKAGE / "build"
    obj_dir.mkdir(exist_ok=True)
    procs = []
    for name in SOURCES:
        obj = obj_dir / (Path(name).stem + ".o")
        objects.append(str(obj))
        cmd = [nvcc(), *NVCC_FLAGS, *(extra or []), "-c", str(CSRC / name), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((name, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for name, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0:
            failed = True
            sys.stderr.write(f"--- nvcc {name} failed\n{out}\n")
        elif verbose or out.strip():
            sys.stderr.write(f"--- nvcc {name}\n{out}\n")
    if failed:
        raise RuntimeError("nvcc failed; see the compiler output above")
    # link under a temporary name and move it into place: a process that loads the library meanwhile sees the old
    # file or the new one, never a half-written one
    fresh = LIBRARY.with_suffix(f".so.{os.getpid()}.tmp")
    link = [nvcc(), "-shared", "-o", str(fresh), *objects, "-gencode", "arch=compute_100a,code=sm_100a"]
    try:
        subprocess.run(link, check=True)
        os.replace(fresh, LIBRARY)
    finally:
        fresh.unlink(missing_ok=True)
    return LIBRARY


def ensure_built(extra: list[str] | None = None) -> Path:
    """Build when a source is newer than the library.  Several ranks of one job may call this at once: they
    take a file lock in turn, and all but the first find the library fresh."""
    if not stale():
        return LIBRARY
    if os.environ.get("WEFT_B200_NO_BUILD"):
        raise RuntimeError(f"{LIBRARY} is missing or stale and WEFT_B200_NO_BUILD is set")
    import fcntl

    (PACKAGE / "build").mkdir(exist_ok=True)
    with open(PACKAGE / "build" / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if stale():
                build(extra=extra)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIBRARY


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
