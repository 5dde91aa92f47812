"""Markdown tables from the JSON-lines records of the harness programs.

    python -m fp4_all_reduce_b200.harness.summarize timing.jsonl [more.jsonl ...] [--peaks MEASURED_PEAKS.json]

Understands the records of bench_cli ("timing", "overlap"), gate_dist ("check"), micro ("bw", "latency"),
gemm_ar_bench and ops_bench / gemm_bench (plain dicts with an "op" key).  For timing cells it prints
fused / xport / compute / empty, the NCCL baseline and the speed-up, the corrected overlap
(X + C - F - E) / min(X - E, C - E), and wire GB/s as a fraction of the bulk-store ceiling when a micro record is
present in the input.  The reference project's counterpart is scripts/summarize.py:55-105.
"""
from __future__ import annotations

import argparse
import json
import sys
from collections import defaultdict


def load(paths):
    recs = []
    for p in paths:
        with open(p) as f:
            for line in f:
                line = line.strip()
                if line.startswith("{"):
                    try:
                        recs.append(json.loads(line))
                    except json.JSONDecodeError:
                        pass
    return recs


def table(headers, rows):
    out = ["| " + " | ".join(headers) + " |", "| " + " | ".join("---" for _ in headers) + " |"]
    for r in rows:
        out.append("| " + " | ".join("" if v is None else str(v) for v in r) + " |")
    return "\n".join(out)


def timing_tables(recs, ceiling):
    cells = defaultdict(dict)
    nccl = {}
    for r in recs:
        if r.get("kind") != "timing" or "rows" not in r:
            continue
        if str(r.get("variant", "")).startswith("nccl"):
            nccl[(r["tp"], r["rows"], r["epilogue"])] = r["med_us"]
            continue
        key = (r["tp"], r.get("variant", "fp4ar"), r["input"], r["epilogue"], r.get("algo", "auto"), r.get("team_warps", 0),
               r.get("lags", 0), r["rows"])
        cells[key][r["mode"]] = r
    rows = []
    for key in sorted(cells, key=lambda k: (k[0], k[1], k[2], k[3], str(k[4]), k[5], k[6], k[7])):
        tp, variant, inp, epi, algo, tw, lags, nrows = key
        c = cells[key]
        F = c.get("fused", {}).get("med_us")
        X = c.get("xport", {}).get("med_us")
        Cc = c.get("compute", {}).get("med_us")
        E = c.get("empty", {}).get("med_us")
        ov = None
        if None not in (F, X, Cc, E) and min(X - E, Cc - E) > 0:
            ov = round((X + Cc - F - E) / min(X - E, Cc - E), 2)
        base = nccl.get((tp, nrows, epi))    # the BF16 NCCL baseline is the comparison point of both input kinds
        wire = c.get("fused", {}).get("wire_gbs")
        frac = round(wire / ceiling, 2) if wire and ceiling else None
        tune = ("T%d " % tw if tw else "") + ("lags %d,%d" % (lags & 15, lags >> 4) if lags else "")
        rows.append([tp, variant, tune.strip(), inp, epi, nrows, F, X, Cc, E, ov, base,
                     round(base / F, 2) if base and F else None, wire, frac])
    if not rows:
        return ""
    return table(["TP", "variant", "tune", "input", "epilogue", "rows", "fused us", "xport us", "compute us", "empty us", "corr. overlap",
                  "NCCL BF16 (+norm) us", "speed-up", "wire GB/s", "of push ceiling"], rows)


def verdict(recs, expect_fail: bool = False) -> tuple[int, str]:
    """Exit code and one line for a set of gate records: green when there is at least one cell and every cell
    passed; with expect_fail (negative controls) green when every cell FAILED with mismatches.  The reference
    project's counterpart is tests/gate_check.py:31-79."""
    checks = [r for r in recs if r.get("kind") == "check" and "pass" in r]
    if not checks:
        return 3, "GATE RED: no check records"
    if expect_fail:
        undetected = [r for r in checks if r["pass"] or not (r.get("mism_first", 0) or r.get("bad_calls_percall", 0))]
        if undetected:
            return 3, f"NEGATIVE CONTROL RED: {len(undetected)} of {len(checks)} corrupted cells were not detected"
        return 0, f"NEGATIVE CONTROL GREEN: all {len(checks)} corrupted cells were detected"
    bad = [r for r in checks if not r["pass"]]
    if bad:
        first = bad[0]
        where = {k: first.get(k) for k in ("tp", "rows", "input", "epilogue", "algo", "variant") if k in first}
        return 3, f"GATE RED: {len(bad)} of {len(checks)} cells failed, first {where}: {first.get('status', '')}"
    return 0, f"GATE GREEN: {len(checks)} cells"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("files", nargs="+")
    ap.add_argument("--verdict", action="store_true", help="print the gate verdict and exit 3 when it is red")
    ap.add_argument("--expect-fail", action="store_true", help="with --verdict: the records are negative controls")
    ap.add_argument("--ceiling", type=float, default=None, help="bulk-store payload ceiling in GB/s (default: from a micro record)")
    ns = ap.parse_args(argv)
    recs = load(ns.files)
    if ns.verdict:
        code, line = verdict(recs, ns.expect_fail)
        print(line)
        return code
    ceiling = ns.ceiling
    bw = [r for r in recs if r.get("kind") == "bw"]
    if ceiling is None and bw:
        ceiling = max((r["gbs_per_dir"] for r in bw if r["method"] == "bulk_store" and r["active"] == "bidir"), default=None)
    t = timing_tables(recs, ceiling)
    if t:
        print("### Fused AllReduce timing (graph, per call, max over ranks)\n")
        print(t + "\n")
    checks = [r for r in recs if r.get("kind") == "check" and "rows" in r and "input" in r]
    if checks:
        print("### Gate\n")
        print(table(["TP", "rows", "input", "epilogue", "algo", "pass", "mism first", "b2b", "bad per-call", "bad graph",
                     "bad skew", "rel-L2 vs FP32"],
                    [[r["tp"], r["rows"], r["input"], r["epilogue"], r["algo"], r["pass"], r.get("mism_first"),
                      r.get("mism_b2b_final"), r.get("bad_calls_percall"), r.get("bad_calls_graph"), r.get("bad_calls_skew"),
                      None if r.get("rel_l2_vs_fp32") is None else round(r["rel_l2_vs_fp32"], 4)] for r in checks]) + "\n")
    if bw:
        print("### NVLink payload bandwidth (GB/s per direction per GPU)\n")
        print(table(["method", "chunk B", "CTAs", "active", "GB/s"],
                    [[r["method"], r["chunk"], r["ctas"], r["active"], r["gbs_per_dir"]] for r in bw]) + "\n")
    for r in recs:
        if r.get("kind") == "latency":
            print(f"One-way hand-off latency ({r['method']}): {r['one_way_us']} us\n")
    pub = [r for r in recs if r.get("kind") == "publish"]
    if pub:
        print("### Publication cost per tile (st.v4 into the peer, 148 CTAs, both directions busy)\n")
        print(table(["tile B", "publication", "GB/s", "time vs unpublished"],
                    [[r["tile"], r["publish"], r["gbs_per_dir"], r["vs_unpublished"]] for r in pub]) + "\n")
    for r in recs:
        if r.get("kind") == "fence":
            print(f"Remote 16-byte store: {r['ns_per_remote_store']} ns; store + fence.acq_rel.sys: "
                  f"{r['ns_per_remote_store_plus_fence_acq_rel_sys']} ns (one thread, idle link)\n")
    tear = [r for r in recs if r.get("kind") == "tear"]
    if tear:
        print("### 16-byte atomicity over NVLink\n")
        print(table(["access", "loads", "torn", "value changes seen"],
                    [[r["access"], r["slots"] * r["polls_per_slot"], r["torn_loads"], r["value_changes_seen"]] for r in tear]) + "\n")
    g = [r for r in recs if r.get("kind") == "timing" and "M" in r]
    if g:
        print("### Row-parallel linear + AllReduce + residual + RMSNorm\n")
        print(table(["TP", "M", "K", "variant", "us", "TFLOP/s", "GEMM floor us", "link floor us"],
                    [[r["tp"], r["M"], r["K"], r["variant"], r["med_us"], r["tflops"], r["gemm_floor_us_at_1391T"],
                      r["link_floor_us_at_770GBs"]] for r in g]) + "\n")
    ops = [r for r in recs if "op" in r and "gbs" in r]
    if ops:
        print("### Stand-alone kernels\n")
        print(table(["op", "rows", "us", "GB/s", "of HBM copy (" + ops[0].get("peak_kind", "") + ")"],
                    [[r["op"], r["rows"], r["med_us"], r["gbs"], r["frac_of_hbm_copy"]] for r in ops]) + "\n")
    gm = [r for r in recs if r.get("op") == "gemm_nvfp4"]
    if gm:
        print("### tcgen05 GEMM with NVFP4 epilogue\n")
        print(table(["M", "K", "N", "us", "TFLOP/s", "of cuBLAS BF16 sustained", "cuBLAS us"],
                    [[r["M"], r["K"], r["N"], r["us"], r["tflops"], r["frac_of_cublas_bf16"], r["cublas_bf16_us"]] for r in gm]) + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
