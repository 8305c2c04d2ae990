"""Performance ledger, bottleneck classifier and report for the optimisation loop.

    python -m machx_inference_engine_b200.cli.perf ledger add --file L.jsonl --model gpt-oss-120b --phase prefill --target mxf4_gemm \\
        --variant "weights on N" --baseline-ms 1.19 --variant-ms 0.297 --quality-baseline 0.9996 --quality-variant 0.9984 --quality-floor 0.997
    python -m machx_inference_engine_b200.cli.perf ledger summary --file L.jsonl
    python -m machx_inference_engine_b200.cli.perf ledger check --file L.jsonl          # exit 1 when the last entry was rejected
    python -m machx_inference_engine_b200.cli.perf roofline --kprofile prof.txt [--ncu raw.csv] [--out capture.json]
    python -m machx_inference_engine_b200.cli.perf viz capture.json report.html

``ledger``: an append-only JSONL record of every variant that was measured: a change is ACCEPTED only when it is faster AND its quality
number (logit cosine against the fp32 path, or perplexity with ``--lower-is-better``) stays on the right side of the floor / gate and
does not regress by more than the tolerance.  ``roofline`` reads the per-op table printed by ``ie_bench --kprofile`` /
``--kprofile-decode`` and, when given, the raw counters of an ``ncu --page raw --csv`` export, and names for every hot op what bounds
it (launch, HBM bandwidth, tensor pipe, latency / occupancy) and the lever that matches, against the measured peaks in
MEASURED_PEAKS.json (copy bandwidth, cuBLAS bf16 rate).  ``viz`` turns that capture into a self-contained HTML page.

Reference parity: tools/perf/ledger.py (add / summary / check with a perplexity gate), tools/perf/roofline.py (bottleneck classes and
levers from a kprofile plus profiler counters), tools/perf/viz.py (HTML report).  Standard library only.
"""
from __future__ import annotations

import argparse
import csv
import datetime
import html
import json
import os
import re
import subprocess
import sys

from .kernel_bench import peaks


# ------------------------------------------------------------------------------------------------ ledger
def _commit() -> str:
    try:
        return subprocess.run(["git", "rev-parse", "--short", "HEAD"], capture_output=True, text=True, timeout=5).stdout.strip()
    except Exception:
        return ""


def gate(e: dict) -> tuple[bool, str]:
    """(accepted, reason) of a ledger entry."""
    sp = e["baseline_ms"] / e["variant_ms"] if e["variant_ms"] > 0 else 0.0
    if sp <= 1.0:
        return False, f"not faster (x{sp:.3f})"
    qb, qv = e.get("quality_baseline"), e.get("quality_variant")
    if qv is None:
        return True, f"x{sp:.3f}, no quality number recorded"
    lower = bool(e.get("lower_is_better"))
    floor, tol = e.get("quality_floor"), e.get("quality_tol_pct", 0.5)
    if floor is not None and ((qv > floor) if lower else (qv < floor)):
        return False, f"quality {qv} is past the gate {floor}"
    if qb is not None and qb != 0:
        delta = (qv - qb) / abs(qb) * 100.0 * (1 if lower else -1)          # > 0: worse
        if delta > tol:
            return False, f"quality regressed by {delta:.3f} % (tolerance {tol} %)"
    return True, f"x{sp:.3f}, quality held"


def _read(path: str) -> list:
    if not os.path.exists(path):
        return []
    return [json.loads(l) for l in open(path) if l.strip()]


def ledger_cmd(a) -> int:
    if a.verb == "add":
        e = {"date": datetime.date.today().isoformat(), "model": a.model, "phase": a.phase, "target": a.target, "variant": a.variant,
             "baseline_ms": a.baseline_ms, "variant_ms": a.variant_ms, "quality_baseline": a.quality_baseline, "quality_variant": a.quality_variant,
             "quality_floor": a.quality_floor, "quality_tol_pct": a.quality_tol, "lower_is_better": a.lower_is_better, "commit": a.commit or _commit(),
             "notes": a.notes}
        ok, why = gate(e)
        e["speedup"] = round(a.baseline_ms / a.variant_ms, 4) if a.variant_ms > 0 else 0.0
        e["accepted"], e["reason"] = ok, why
        with open(a.file, "a") as f:
            f.write(json.dumps(e) + "\n")
        print(("ACCEPT" if ok else "REJECT") + ": " + why)
        return 0
    rows = _read(a.file)
    if a.verb == "check":
        if not rows:
            print("empty ledger")
            return 1
        ok, why = gate(rows[-1])
        print(("ACCEPT" if ok else "REJECT") + ": " + why)
        return 0 if ok else 1
    acc = [r for r in rows if r.get("accepted")]
    print(f"{'date':10s} {'model':16s} {'phase':8s} {'target':18s} {'variant':28s} {'base ms':>9s} {'var ms':>9s} {'x':>6s} {'ok':>3s}  notes")
    for r in rows:
        print(f"{r['date']:10s} {r['model'][:16]:16s} {r['phase'][:8]:8s} {r['target'][:18]:18s} {r['variant'][:28]:28s} {r['baseline_ms']:9.3f} "
              f"{r['variant_ms']:9.3f} {r.get('speedup', 0):6.2f} {'yes' if r.get('accepted') else 'NO':>3s}  {r.get('notes') or r.get('reason', '')}")
    best = {}
    for r in acc:
        if r["target"] not in best or r["speedup"] > best[r["target"]]["speedup"]:
            best[r["target"]] = r
    print(f"{len(rows)} entries, {len(acc)} accepted; best accepted per target: " +
          ", ".join(f"{t} x{r['speedup']:.2f} ({r['variant']})" for t, r in sorted(best.items())))
    return 0


# ------------------------------------------------------------------------------------------------ roofline
_ROW = re.compile(r"^(\S+)\s+(\d+)\s+([\d.]+)\s+([\d.]+)\s+([\d.]+)%\s*$")

LEVERS = {
    "launch": "many launches of a few microseconds: fuse neighbours, capture the loop in a CUDA graph, use programmatic dependent launch",
    "bandwidth": "at the HBM ceiling: move fewer bytes (narrower weight / KV formats, fuse the producer, keep tiles in L2 or shared memory)",
    "tensor": "tensor pipe is the busiest unit: larger MMA tiles, cta_group::2, fewer padded rows, a narrower operand type",
    "latency": "neither bytes nor math: more bytes / MMAs in flight per SM (deeper TMA ring, more resident CTAs), shorter dependent chains",
    "unknown": "no counters: capture this op with `ncu --set full --clock-control none -k regex:<kernel> -c 2` on a small case",
}


def parse_kprofile(text: str) -> dict:
    ops, total = [], 0.0
    for line in text.splitlines():
        m = _ROW.match(line.strip())
        if m:
            ops.append({"name": m.group(1), "calls": int(m.group(2)), "total_ms": float(m.group(3)), "us_per_call": float(m.group(4)),
                        "share_pct": float(m.group(5))})
        elif line.startswith("TOTAL"):
            total = float(line.split()[-1])
    return {"ops": ops, "total_ms": total or sum(o["total_ms"] for o in ops)}


def parse_ncu_raw(path: str) -> dict:
    """kernel name -> {metric: value} from `ncu -i X.ncu-rep --page raw --csv` (first launch of each kernel)."""
    rows = list(csv.reader(open(path)))
    if len(rows) < 3:
        return {}
    hdr = rows[0]
    ki = hdr.index("Kernel Name")
    want = {"gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed": "dram_pct", "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active": "tensor_pct",
            "sm__warps_active.avg.pct_of_peak_sustained_active": "occupancy_pct", "gpu__time_duration.sum": "duration"}
    out = {}
    for r in rows[2:]:
        name = r[ki].split("(")[0].split("<")[0].split("::")[-1]
        if name in out:
            continue
        d = {}
        for col, key in want.items():
            if col in hdr:
                try:
                    d[key] = float(r[hdr.index(col)].replace(",", ""))
                except ValueError:
                    pass
        out[name] = d
    return out


def classify(op: dict, counters: dict | None) -> str:
    if op["us_per_call"] < 12.0 and op["calls"] >= 32:
        return "launch"
    if not counters:
        return "unknown"
    if counters.get("dram_pct", 0) >= 55.0:
        return "bandwidth"
    if counters.get("tensor_pct", 0) >= 45.0:
        return "tensor"
    return "latency"


def roofline_cmd(a) -> int:
    text = sys.stdin.read() if a.kprofile == "-" else open(a.kprofile).read()
    cap = parse_kprofile(text)
    ncu = parse_ncu_raw(a.ncu) if a.ncu else {}
    pk = peaks()
    cap["peaks"] = pk
    for op in cap["ops"]:
        c = ncu.get(op["name"] + "_kernel") or ncu.get(op["name"]) or next((v for k, v in ncu.items() if k.startswith(op["name"])), None)
        op["counters"] = c or {}
        op["bound"] = classify(op, c)
        op["lever"] = LEVERS[op["bound"]]
    cap["ops"].sort(key=lambda o: -o["total_ms"])
    if a.out:
        json.dump(cap, open(a.out, "w"), indent=1)
    print(f"total {cap['total_ms']:.3f} ms; peaks ({pk['src']}): HBM {pk['hbm_gbs']:.0f} GB/s, bf16 {pk['bf16_tflops']:.0f} TFLOP/s")
    for op in cap["ops"]:
        c = op["counters"]
        extra = f" dram {c['dram_pct']:.0f}% tensor {c.get('tensor_pct', 0):.0f}%" if "dram_pct" in c else ""
        print(f"{op['share_pct']:5.1f}%  {op['name']:22s} {op['us_per_call']:9.1f} us x {op['calls']:5d}  -> {op['bound']:9s}{extra}\n        {op['lever']}")
    return 0


# ------------------------------------------------------------------------------------------------ report
_COLOR = {"launch": "#b07aa1", "bandwidth": "#4e79a7", "tensor": "#59a14f", "latency": "#e15759", "unknown": "#9c9c9c"}


def viz_cmd(a) -> int:
    cap = json.load(open(a.capture))
    ops = cap["ops"]
    top = max((o["total_ms"] for o in ops), default=1.0) or 1.0
    rows = []
    for o in ops:
        w = 600.0 * o["total_ms"] / top
        rows.append(f"<tr><td>{html.escape(o['name'])}</td><td>{o['calls']}</td><td>{o['us_per_call']:.1f}</td><td>{o['share_pct']:.1f} %</td>"
                    f"<td><svg width='610' height='14'><rect width='{w:.1f}' height='14' fill='{_COLOR.get(o['bound'], '#999')}'/></svg></td>"
                    f"<td>{o['bound']}</td><td>{html.escape(o['lever'])}</td></tr>")
    pk = cap.get("peaks", {})
    page = ("<html><head><meta charset='utf-8'><title>per-op profile</title><style>body{font-family:sans-serif}td,th{padding:2px 8px;font-size:13px}"
            "</style></head><body>" + f"<h3>per-op device time: {cap['total_ms']:.3f} ms</h3><p>peaks ({pk.get('src', '?')}): HBM {pk.get('hbm_gbs', 0):.0f} GB/s, "
            f"bf16 {pk.get('bf16_tflops', 0):.0f} TFLOP/s</p><table><tr><th>op</th><th>calls</th><th>us / call</th><th>share</th><th></th><th>bound</th>"
            "<th>lever</th></tr>" + "".join(rows) + "</table></body></html>")
    open(a.out, "w").write(page)
    print(f"wrote {a.out} ({len(ops)} ops)")
    return 0


_TRACE_CATEGORY = (("attention", "attention"), ("qkv_post", "memory_kv"), ("kv", "memory_kv"), ("gemm", "matmul"), ("gemv", "matmul"), ("linear", "matmul"),
                   ("moe", "moe"), ("expert", "moe"), ("norm", "norm"), ("deltanet", "recurrence"), ("conv1d", "recurrence"))


def trace_cmd(a) -> int:
    """A per-op table of ``ie_bench --kprofile`` / ``--kprofile-decode`` as a timeline file for a trace viewer (the Trace Event JSON
    that chrome://tracing and Perfetto load).  The table is an aggregate, not a timeline: the ops are laid end to end by their total
    time, so the picture reads as shares of the step, one lane per category (src: tools/perf/benchscope_export.py, which feeds the same
    tables to the reference's own dashboard)."""
    text = sys.stdin.read() if a.kprofile == "-" else open(a.kprofile).read()
    prof = parse_kprofile(text)
    lanes, events, t = {}, [], 0.0
    meta = {k: v for k, v in (("model", a.model), ("quant", a.quant), ("ctx", a.ctx), ("tok_s", a.tok_s)) if v not in (None, "")}
    for o in prof["ops"]:
        cat = next((c for key, c in _TRACE_CATEGORY if key in o["name"]), "other")
        tid = lanes.setdefault(cat, len(lanes) + 1)
        dur = o["total_ms"] * 1e3
        events.append({"name": o["name"], "cat": cat, "ph": "X", "pid": 1, "tid": tid, "ts": round(t, 3), "dur": round(dur, 3),
                       "args": {"calls": o["calls"], "us_per_call": o["us_per_call"], "share_pct": o["share_pct"], **meta}})
        t += dur
    for cat, tid in lanes.items():
        events.append({"name": "thread_name", "ph": "M", "pid": 1, "tid": tid, "args": {"name": cat}})
    events.append({"name": "process_name", "ph": "M", "pid": 1, "args": {"name": a.session or "kprofile"}})
    json.dump({"traceEvents": events, "displayTimeUnit": "ms", "otherData": {"total_ms": prof["total_ms"], **meta}}, open(a.out, "w"))
    print(f"wrote {a.out} ({len(prof['ops'])} ops, {prof['total_ms']:.3f} ms)")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="perf")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("ledger")
    p.add_argument("verb", choices=["add", "summary", "check"])
    p.add_argument("--file", default="perf_ledger.jsonl")
    p.add_argument("--model", default="")
    p.add_argument("--phase", default="")
    p.add_argument("--target", default="")
    p.add_argument("--variant", default="")
    p.add_argument("--baseline-ms", type=float, default=0.0)
    p.add_argument("--variant-ms", type=float, default=0.0)
    p.add_argument("--quality-baseline", type=float, default=None)
    p.add_argument("--quality-variant", type=float, default=None)
    p.add_argument("--quality-floor", type=float, default=None, help="gate: the variant's quality must not pass it")
    p.add_argument("--quality-tol", type=float, default=0.5, help="allowed regression against the baseline, percent")
    p.add_argument("--lower-is-better", action="store_true", help="the quality number is a perplexity-like quantity")
    p.add_argument("--commit", default="")
    p.add_argument("--notes", default="")
    p = sub.add_parser("roofline")
    p.add_argument("--kprofile", required=True, help="file with the table of ie_bench --kprofile / --kprofile-decode, or - for stdin")
    p.add_argument("--ncu", default=None, help="csv from `ncu -i X.ncu-rep --page raw --csv`")
    p.add_argument("--out", default=None)
    p = sub.add_parser("viz")
    p.add_argument("capture")
    p.add_argument("out")
    p = sub.add_parser("trace")
    p.add_argument("--kprofile", required=True, help="file with a --kprofile table, or - for stdin")
    p.add_argument("--out", required=True)
    p.add_argument("--session", default="")
    p.add_argument("--model", default="")
    p.add_argument("--quant", default="")
    p.add_argument("--ctx", type=int, default=None)
    p.add_argument("--tok-s", type=float, default=None)
    a = ap.parse_args(argv)
    return {"ledger": ledger_cmd, "roofline": roofline_cmd, "viz": viz_cmd, "trace": trace_cmd}[a.cmd](a)


if __name__ == "__main__":
    sys.exit(main())
