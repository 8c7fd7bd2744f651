"""Builds librlk_b200.so from the CUDA sources beside this file with nvcc for sm_100a.

The library exposes a plain C ABI (every entry point is ``extern "C" rlk_*``) and is loaded
with ctypes by ``rl_kernel_b200.backends.extension``; it has no dependency on torch headers,
so a full rebuild takes seconds per file and cross-compiles on a machine without a GPU.

Usage: ``python -m rl_kernel_b200.csrc.build [--force] [--verbose]``
"""
from __future__ import annotations

import argparse
import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
BUILD_DIR = CSRC / "build"
LIB_PATH = CSRC.parent / "librlk_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
    "-I", str(CSRC / "include"),
]


def nvcc_path() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = Path(cuda_home) / "bin" / "nvcc"
    return str(cand) if cand.exists() else "nvcc"


def sources() -> list[Path]:
    return sorted(p for p in CSRC.rglob("*.cu") if BUILD_DIR not in p.parents)


def _digest(src: Path) -> str:
    h = hashlib.sha256()
    h.update(src.read_bytes())
    for hdr in sorted((CSRC / "include").rglob("*")):
        if hdr.is_file():
            h.update(hdr.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _compile_one(src: Path, force: bool, verbose: bool) -> tuple[Path, bool, str]:
    rel = src.relative_to(CSRC).with_suffix("")
    obj = BUILD_DIR / ("_".join(rel.parts) + ".o")
    stamp = obj.with_suffix(".sha")
    digest = _digest(src)
    if not force and obj.exists() and stamp.exists() and stamp.read_text() == digest:
        return obj, False, ""
    cmd = [nvcc_path(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{proc.stdout}\n{proc.stderr}")
    stamp.write_text(digest)
    return obj, True, proc.stderr


def build(force: bool = False, verbose: bool = False, jobs: int | None = None) -> Path:
    """Compile every ``*.cu`` under csrc/ for sm_100a and link ``librlk_b200.so`` in-tree."""
    BUILD_DIR.mkdir(exist_ok=True)
    srcs = sources()
    jobs = jobs or min(len(srcs), os.cpu_count() or 4)
    with ThreadPoolExecutor(max_workers=jobs) as pool:
        results = list(pool.map(lambda s: _compile_one(s, force, verbose), srcs))
    rebuilt = any(r[1] for r in results)
    if verbose:
        for _, _, log in results:
            if log:
                print(log)
    if rebuilt or not LIB_PATH.exists():
        tmp = LIB_PATH.with_suffix(f".so.tmp{os.getpid()}")       # link beside the target, then rename: readers never see half a file
        cmd = [nvcc_path(), "-shared", "-o", str(tmp), *[str(r[0]) for r in results],
               "-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            tmp.unlink(missing_ok=True)
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
        os.replace(tmp, LIB_PATH)
    return LIB_PATH


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="pass -Xptxas -v and print its report")
    args = ap.parse_args(argv)
    path = build(force=args.force, verbose=args.verbose)
    print(path)
    return 0


if __name__ == "__main__":
    sys.exit(main())
