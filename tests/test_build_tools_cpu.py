"""Source manifest (provenance) and the ptxas resource parser of the build script, on the host."""
from pathlib import Path

from fp4_all_reduce_b200 import build as B


def test_manifest_round_trip_and_negative_control(tmp_path):
    root = tmp_path / "csrc"
    (root / "kernels").mkdir(parents=True)
    (root / "kernels" / "a.cu").write_text("__global__ void k() {}\n")
    (root / "kernels" / "b.cuh").write_text("#pragma once\n")
    (root / "notes.txt").write_text("not a source\n")
    man = B.write_manifest(root)
    assert [l.split()[1] for l in man.read_text().splitlines()] == ["kernels/a.cu", "kernels/b.cuh"]
    assert B.verify_manifest(root) == []
    with open(root / "kernels" / "a.cu", "a") as f:      # the negative control: one appended byte must be seen
        f.write(" ")
    assert B.verify_manifest(root) == ["changed: kernels/a.cu"]
    (root / "kernels" / "b.cuh").unlink()
    (root / "kernels" / "c.h").write_text("")
    assert B.verify_manifest(root) == ["changed: kernels/a.cu", "missing: kernels/b.cuh", "unlisted: kernels/c.h"]


def test_repository_manifest_matches_sources():
    """The committed manifest is regenerated with every change of the native sources."""
    assert B.verify_manifest() == []


def test_resource_log_parser(tmp_path):
    log = tmp_path / "r.log"
    log.write_text(
        "ptxas info    : Compiling entry function '_Z1kv' for 'sm_100a'\n"
        "ptxas info    : Function properties for _Z1kv\n"
        "    40 bytes stack frame, 4 bytes spill stores, 12 bytes spill loads\n"
        "ptxas info    : Used 168 registers, used 1 barriers\n"
        "ptxas info    : Compiling entry function '_Z1jv' for 'sm_100a'\n"
        "ptxas info    : Function properties for _Z1jv\n"
        "    0 bytes stack frame, 0 bytes spill stores, 0 bytes spill loads\n"
        "ptxas info    : Used 32 registers\n")
    rs = B.resources(log)
    assert rs == [{"symbol": "_Z1kv", "stack": 40, "spill_stores": 4, "spill_loads": 12, "registers": 168},
                  {"symbol": "_Z1jv", "stack": 0, "spill_stores": 0, "spill_loads": 0, "registers": 32}]
