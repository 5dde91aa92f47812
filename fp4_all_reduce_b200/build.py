"""In-tree build of the native libraries.

    python -m fp4_all_reduce_b200.build [--force] [--verbose]

produces, next to this file,

    lib/libfp4ar.so         CUDA kernels + host runtime for sm_100a (nvcc, cross-compiles without a GPU)
    lib/libfp4ar_oracle.so  the host-only bit-exact model (g++)

Each translation unit is compiled separately and in parallel; an object is rebuilt when its source or
any header under csrc/ changed.  ptxas resource usage of every kernel is appended to
lib/build_resources.log (registers, spills, shared memory) the way the reference project's build.sh:18-27
keeps its register / spill log.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OBJ = ROOT / "build"
LIB = ROOT / "lib"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
    "-diag-suppress", "177",
]
GXX_FLAGS = ["-O2", "-std=c++17", "-ffp-contract=off", "-fno-fast-math", "-fopenmp", "-fPIC", "-shared"]


def cuda_sources() -> list[Path]:
    return sorted(list((CSRC / "kernels").glob("*.cu")) + list((CSRC / "runtime").glob("*.cu")))


def _headers_digest() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _stamp(src: Path, hdr: str) -> str:
    return hashlib.sha256(src.read_bytes() + hdr.encode()).hexdigest()


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found")
    return exe


def _compile_one(src: Path, hdr: str, force: bool, verbose: bool) -> tuple[Path, str, bool]:
    obj = OBJ / (src.stem + ".o")
    stamp_file = OBJ / (src.stem + ".stamp")
    stamp = _stamp(src, hdr)
    if not force and obj.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return obj, "", False
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    stamp_file.write_text(stamp)
    if verbose:
        print(f"[build] {src.name}")
    return obj, r.stderr, True


def build_cuda(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    LIB.mkdir(exist_ok=True)
    out = LIB / "libfp4ar.so"
    hdr = _headers_digest()
    srcs = cuda_sources()
    logs: list[str] = []
    rebuilt = False
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        for obj, log, did in ex.map(lambda s: _compile_one(s, hdr, force, verbose), srcs):
            rebuilt |= did
            if log:
                logs.append(log)
    objs = [OBJ / (s.stem + ".o") for s in srcs]
    if rebuilt or not out.exists():
        cmd = [_nvcc(), "-shared", "-o", str(out), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a",
               "-Xcompiler", "-fPIC", "-lcuda"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        if logs:
            with open(LIB / "build_resources.log", "w") as f:
                f.write("\n".join(logs))
    return out


def build_oracle(force: bool = False, verbose: bool = False) -> Path:
    LIB.mkdir(exist_ok=True)
    out = LIB / "libfp4ar_oracle.so"
    src = CSRC / "oracle" / "oracle.cpp"
    stamp_file = LIB / "oracle.stamp"
    stamp = hashlib.sha256(src.read_bytes() + " ".join(GXX_FLAGS).encode()).hexdigest()
    if not force and out.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return out
    cmd = ["g++", *GXX_FLAGS, str(src), "-o", str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"g++ failed:\n{r.stdout}\n{r.stderr}")
    stamp_file.write_text(stamp)
    if verbose:
        print("[build] oracle.cpp")
    return out


def build_all(force: bool = False, verbose: bool = False) -> dict[str, Path]:
    return {"oracle": build_oracle(force, verbose), "cuda": build_cuda(force, verbose)}


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ns = ap.parse_args(argv)
    libs = build_all(ns.force, ns.verbose)
    for k, v in libs.items():
        print(f"{k}: {v}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
