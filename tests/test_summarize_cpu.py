"""Summarizer and gate verdict on hand-made records (no GPU)."""
import json

from fp4_all_reduce_b200.harness import summarize as S


def _t(mode, us, **kw):
    r = {"kind": "timing", "variant": "fp4ar", "tp": 4, "rows": 4096, "input": "bf16", "epilogue": 0, "algo": "auto",
         "team_warps": 0, "lags": 0, "mode": mode, "med_us": us, "wire_gbs": 300.0 if mode == "fused" else None}
    r.update(kw)
    return r


def test_timing_table_overlap_and_speedup(tmp_path, capsys):
    recs = [_t("fused", 60.0), _t("xport", 45.0), _t("compute", 55.0), _t("empty", 5.0),
            {"kind": "timing", "variant": "nccl_bf16", "tp": 4, "rows": 4096, "input": "bf16", "epilogue": 0, "mode": "fused", "med_us": 150.0},
            _t("fused", 50.0, lags=66), _t("fused", 70.0, variant="pull"),
            {"kind": "bw", "method": "bulk_store", "chunk": 4096, "ctas": 148, "active": "bidir", "gbs_per_dir": 600.0},
            {"kind": "latency", "method": "x", "one_way_us": 1.2},
            {"kind": "publish", "tile": 4096, "publish": "none", "gbs_per_dir": 600.0, "vs_unpublished": 1.0},
            {"kind": "fence", "ns_per_remote_store": 10.0, "ns_per_remote_store_plus_fence_acq_rel_sys": 900.0},
            {"kind": "tear", "access": "16B_store_16B_load", "slots": 4096, "polls_per_slot": 3000, "torn_loads": 0, "value_changes_seen": 77}]
    f = tmp_path / "r.jsonl"
    f.write_text("noise line\n" + "\n".join(json.dumps(r) for r in recs) + "\n")
    assert S.main([str(f)]) == 0
    out = capsys.readouterr().out
    # corrected overlap (45 + 55 - 60 - 5) / min(40, 50) = 0.875 -> 0.88; speed-up 150 / 60 = 2.5; 300 / 600 = 0.5
    row = [l for l in out.splitlines() if l.startswith("| 4 | fp4ar |  |")][0]
    assert "| 0.88 |" in row and "| 2.5 |" in row and "| 0.5 |" in row
    assert any("lags 2,4" in l and "| 50.0 |" in l for l in out.splitlines())
    assert any("| pull |" in l and "| 70.0 |" in l for l in out.splitlines())
    assert "16-byte atomicity" in out and "Publication cost" in out and "fence.acq_rel.sys: 900.0 ns" in out


def test_gate_verdicts():
    ok = {"kind": "check", "tp": 2, "rows": 64, "input": 0, "epilogue": 0, "algo": 0, "pass": True, "mism_first": 0}
    bad = dict(ok, **{"pass": False, "mism_first": 12, "status": "ok"})
    assert S.verdict([])[0] == 3
    assert S.verdict([ok, ok]) == (0, "GATE GREEN: 2 cells")
    code, line = S.verdict([ok, bad])
    assert code == 3 and "1 of 2 cells failed" in line
    # negative controls: green only when every corrupted cell was caught
    assert S.verdict([bad, bad], expect_fail=True)[0] == 0
    assert S.verdict([bad, ok], expect_fail=True)[0] == 3


def test_verdict_cli(tmp_path, capsys):
    f = tmp_path / "g.jsonl"
    f.write_text(json.dumps({"kind": "check", "tp": 2, "rows": 64, "input": 0, "epilogue": 0, "algo": 0, "pass": True}) + "\n")
    assert S.main([str(f), "--verdict"]) == 0
    assert "GATE GREEN" in capsys.readouterr().out
