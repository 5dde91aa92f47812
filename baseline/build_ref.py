"""Build the reference project's own kernels, untouched, for sm_100a, plus the driver that calls them.

    python baseline/build_ref.py [--src /path/to/reference]

Copies the reference tree to baseline/_ref/src (that directory is not tracked), compiles
kernels/push/tp2_l2.cu (variant L2, -DLAMPORT_V2=1), kernels/push/tp4_l4.cu (variant L4) and
kernels/fused_norm/lnorm.cu exactly the way the reference's build.sh:18-31 does (same flags, same
-DFP4AR_NAME / -DFP4AR_REGISTER defines), and links them with baseline/ref_shim.cu into baseline/_ref/ref_shim.
The reference's harness itself cannot be linked here: it needs ncclGetLsaDevicePointer (NCCL >= 2.31).
"""
from __future__ import annotations

import argparse
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"


def reference_dir() -> str:
    """Where the reference project's tree is: FP4AR_REFERENCE_DIR, else `reference_path` of BASELINE.json at the
    repository root, else "" (nothing to build from)."""
    import json
    import os

    d = os.environ.get("FP4AR_REFERENCE_DIR", "")
    if d:
        return d
    try:
        with open(HERE.parent / "BASELINE.json") as f:
            return str(json.load(f).get("reference_path", ""))
    except Exception:
        return ""


def nccl_paths():
    import nvidia
    base = Path(list(nvidia.__path__)[0]) / "nccl"
    return base / "include", base / "lib"


def copy_sources(ref: str) -> Path | None:
    src = OUT / "src"
    if ref and Path(ref).exists():
        if src.exists():
            shutil.rmtree(src)
        shutil.copytree(ref, src, ignore=shutil.ignore_patterns(".git"))
    return src if src.exists() else None


def build_host_oracle(ref: str | None = None, force: bool = False) -> Path | None:
    """baseline/_ref/libref_oracle.so: the reference's own CPU oracle (bench/codec/codec_bench.cu, `namespace cpu`)
    behind two C functions (baseline/ref_oracle_shim.cu).  Host code only runs; no GPU is needed to use it."""
    out = OUT / "libref_oracle.so"
    if out.exists() and not force:
        return out
    src = OUT / "src"
    if not src.exists():
        src = copy_sources(ref if ref is not None else reference_dir())
    if src is None:
        return None
    OUT.mkdir(exist_ok=True)
    cmd = ["nvcc", "-O2", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC,-fopenmp",
           "-diag-suppress", "177,550", f"-I{src}", f"-I{src}/include", f"-I{src}/harness", str(HERE / "ref_oracle_shim.cu"),
           "-o", str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        print(r.stdout[-2000:], r.stderr[-3000:], file=sys.stderr)
        return None
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", default=reference_dir(), help="reference tree (default: FP4AR_REFERENCE_DIR or BASELINE.json)")
    ap.add_argument("--host-oracle", action="store_true", help="build only the CPU oracle bridge")
    ns = ap.parse_args(argv)
    if ns.host_oracle:
        out = build_host_oracle(ns.src, force=True)
        print(out if out else "failed")
        return 0 if out else 1
    src = copy_sources(ns.src)
    if src is None:
        print("reference sources not found", file=sys.stderr)
        return 1
    inc, lib = nccl_paths()
    nv = ["nvcc", "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
          f"-I{src}/include", f"-I{src}/harness", f"-I{src}/kernels/fused_norm", f"-I{inc}"]
    jobs = [
        (["-DLAMPORT_V2=1", "-DFP4AR_NAME=L2", "-DFP4AR_REGISTER=fp4ar_register_L2", "-c", f"{src}/kernels/push/tp2_l2.cu"], OUT / "v_L2.o"),
        (["-DFP4AR_NAME=L4", "-DFP4AR_REGISTER=fp4ar_register_L4", "-c", f"{src}/kernels/push/tp4_l4.cu"], OUT / "v_L4.o"),
        (["-c", f"{src}/kernels/fused_norm/lnorm.cu"], OUT / "lnorm.o"),
        (["-c", str(HERE / "ref_shim.cu")], OUT / "ref_shim.o"),
    ]
    procs = [(subprocess.Popen(nv + a + ["-o", str(o)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True), o) for a, o in jobs]
    ok = True
    for p, o in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            ok = False
            print(f"FAILED {o.name}\n{out[-3000:]}")
    if not ok:
        return 1
    link = ["nvcc", "-o", str(OUT / "ref_shim")] + [str(o) for _, o in jobs] + [f"-L{lib}", "-l:libnccl.so.2", "-lpthread", "-ldl",
            "-Xlinker", f"-rpath={lib}", "-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        print(r.stdout, r.stderr)
        return 1
    print(OUT / "ref_shim")
    return 0


if __name__ == "__main__":
    sys.exit(main())
