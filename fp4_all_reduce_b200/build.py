"""In-tree build of the native libraries.

    python -m fp4_all_reduce_b200.build [--force] [--verbose]
    python -m fp4_all_reduce_b200.build --check        # compile every translation unit, do not link
    python -m fp4_all_reduce_b200.build --resources    # registers / spills per kernel from the last full build
    python -m fp4_all_reduce_b200.build --manifest     # record the sha256 of every native source in csrc/MANIFEST.sha256
    python -m fp4_all_reduce_b200.build --verify       # compare the sources with that record (exit 1 on any difference)

produces, next to this file,

    lib/libfp4ar.so         CUDA kernels + host runtime for sm_100a (nvcc, cross-compiles without a GPU)
    lib/libfp4ar_oracle.so  the host-only bit-exact model (g++)

Each translation unit is compiled separately and in parallel; an object is rebuilt when its source or
any header under csrc/ changed.  ptxas resource usage of every kernel is appended to
lib/build_resources.log (registers, spills, shared memory) the way the reference project's build.sh:18-27
keeps its register / spill log.  `--check` is its `build.sh check` (objects only, works on a machine without a
GPU); `--manifest` / `--verify` do what its kernels/verify_origin.sh:4-22 does with md5 sums: they tie measured
numbers to the exact sources that produced them.
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
    (OBJ / (src.stem + ".ptxas")).write_text(r.stderr)     # kept per unit, so the resource log of an incremental build is complete
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
        with open(LIB / "build_resources.log", "w") as f:
            for src in srcs:
                unit = OBJ / (src.stem + ".ptxas")
                if unit.exists():
                    f.write(unit.read_text() + "\n")
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


def check_compile(verbose: bool = False) -> int:
    """Compile every CUDA translation unit and the host model to objects; nothing is linked or installed."""
    OBJ.mkdir(exist_ok=True)
    hdr = _headers_digest()
    n = 0
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        for _obj, _log, _did in ex.map(lambda s: _compile_one(s, hdr, False, verbose), cuda_sources()):
            n += 1
    r = subprocess.run(["g++", *[f for f in GXX_FLAGS if f != "-shared"], "-c", str(CSRC / "oracle" / "oracle.cpp"),
                        "-o", str(OBJ / "oracle.o")], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"g++ failed:\n{r.stdout}\n{r.stderr}")
    return n + 1


def native_sources(root: Path = CSRC) -> list[Path]:
    exts = (".cu", ".cuh", ".h", ".cpp")
    return sorted(p for p in root.rglob("*") if p.suffix in exts and p.is_file())


def write_manifest(root: Path = CSRC, out: Path | None = None) -> Path:
    out = out or root / "MANIFEST.sha256"
    lines = [f"{hashlib.sha256(p.read_bytes()).hexdigest()}  {p.relative_to(root).as_posix()}" for p in native_sources(root)]
    out.write_text("\n".join(lines) + "\n")
    return out


def verify_manifest(root: Path = CSRC, manifest: Path | None = None) -> list[str]:
    """Differences between the sources under `root` and the manifest: changed, missing and unlisted files."""
    manifest = manifest or root / "MANIFEST.sha256"
    want = {}
    for line in manifest.read_text().splitlines():
        if line.strip():
            digest, name = line.split(None, 1)
            want[name.strip()] = digest
    have = {p.relative_to(root).as_posix(): hashlib.sha256(p.read_bytes()).hexdigest() for p in native_sources(root)}
    diffs = [f"changed: {n}" for n in sorted(want) if n in have and have[n] != want[n]]
    diffs += [f"missing: {n}" for n in sorted(want) if n not in have]
    diffs += [f"unlisted: {n}" for n in sorted(have) if n not in want]
    return diffs


def resources(log: Path | None = None) -> list[dict]:
    """Kernel name, registers, stack, spill bytes from the ptxas log of the last full build."""
    import re

    log = log or LIB / "build_resources.log"
    text = log.read_text()
    pat = re.compile(r"Compiling entry function '(\S+)' for 'sm_100a'\n.*?\n\s+(\d+) bytes stack frame, (\d+) bytes spill stores, "
                     r"(\d+) bytes spill loads\nptxas info\s+: Used (\d+) registers")
    out = []
    for m in pat.finditer(text):
        out.append({"symbol": m.group(1), "stack": int(m.group(2)), "spill_stores": int(m.group(3)),
                    "spill_loads": int(m.group(4)), "registers": int(m.group(5))})
    return out


def build_all(force: bool = False, verbose: bool = False) -> dict[str, Path]:
    return {"oracle": build_oracle(force, verbose), "cuda": build_cuda(force, verbose)}


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--check", action="store_true", help="compile objects only, no link")
    ap.add_argument("--resources", action="store_true", help="print registers / spills per kernel")
    ap.add_argument("--manifest", action="store_true", help="write csrc/MANIFEST.sha256")
    ap.add_argument("--verify", action="store_true", help="verify the sources against csrc/MANIFEST.sha256")
    ns = ap.parse_args(argv)
    if ns.check:
        print(f"compiled {check_compile(ns.verbose)} translation units (no link)")
        return 0
    if ns.manifest:
        print(f"wrote {write_manifest()}")
        return 0
    if ns.verify:
        diffs = verify_manifest()
        print("\n".join(diffs) if diffs else "sources match the manifest")
        return 1 if diffs else 0
    if ns.resources:
        rs = resources()
        for r in sorted(rs, key=lambda r: -r["registers"]):
            print(f"{r['registers']:4d} regs  stack {r['stack']:3d}  spill {r['spill_stores']:3d}/{r['spill_loads']:3d}  {r['symbol']}")
        spilled = [r for r in rs if r["spill_stores"] or r["spill_loads"]]
        print(f"{len(rs)} kernels, {len(spilled)} with spills")
        return 0
    libs = build_all(ns.force, ns.verbose)
    for k, v in libs.items():
        print(f"{k}: {v}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
