"""The host (gloo) form of the AllReduce in real rank processes on the CPU: bit-identical to the host model fed with
all ranks' inputs for both algorithms and both input kinds, with a row count that does not divide by the group size;
and a rank that leaves between steps turns the survivors' next call into PeerTimeout instead of a hang."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(world, extra, port):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", "host_group_worker.py")] + extra
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    recs, dec, text, i = [], json.JSONDecoder(), p.stdout, 0
    while True:                      # ranks share one stdout: two records can land on one line
        i = text.find("{", i)
        if i < 0:
            break
        try:
            obj, end = dec.raw_decode(text, i)
            recs.append(obj)
            i = end
        except json.JSONDecodeError:
            i += 1
    return p.returncode, recs, p.stdout[-2000:] + p.stderr[-2000:]


@pytest.mark.parametrize("world", [2, 4])
def test_host_allreduce_matches_the_host_model_on_every_rank(world):
    rc, recs, log = _run(world, ["--rows", "37"], 29720 + world)
    assert rc == 0, log
    assert len(recs) == world, log
    for r in recs:
        assert r["mismatches"] == {"oneshot": 0, "twoshot": 0, "nvfp4_in": 0}, r


def test_a_rank_that_leaves_is_reported_not_waited_for_forever():
    rc, recs, log = _run(3, ["--rows", "16", "--leaves", "1"], 29731)
    survivors = [r for r in recs if "peer_timeout" in r]
    assert any(r.get("left") for r in recs), log
    assert len(survivors) == 2 and all(r["peer_timeout"] for r in survivors), log
    # the calls before the failure were correct on the survivors
    assert all(r["mismatches"] == {"oneshot": 0, "twoshot": 0, "nvfp4_in": 0} for r in survivors), survivors
