"""The optimisation-loop tools: ledger gate, bottleneck classes from a per-op profile (+ ncu counters), HTML report."""
import json

from machx_inference_engine_b200.cli import perf

KPROFILE = """# kprofile prefill T=2048
op                         calls    total ms      avg us   share
mxf4_gemm                     72      19.588       272.1   53.2%
gemm                         108       6.248        57.8   17.0%
attention                     36       3.888       108.0   10.6%
rmsnorm                       38       0.245         6.4    0.7%
TOTAL                        254      29.969
"""


def test_ledger_gate_and_summary(tmp_path, capsys):
    f = str(tmp_path / "l.jsonl")
    base = ["ledger", "add", "--file", f, "--model", "gpt-oss-120b", "--phase", "prefill", "--target", "mxf4_gemm", "--commit", "abc"]
    assert perf.main(base + ["--variant", "weights on N", "--baseline-ms", "1.19", "--variant-ms", "0.297", "--quality-baseline", "0.9996",
                             "--quality-variant", "0.9984", "--quality-floor", "0.997"]) == 0
    assert perf.main(["ledger", "check", "--file", f]) == 0
    # faster but past the quality floor: rejected
    perf.main(base + ["--variant", "4-bit activations", "--baseline-ms", "0.297", "--variant-ms", "0.2", "--quality-baseline", "0.9984",
                      "--quality-variant", "0.95", "--quality-floor", "0.997"])
    assert perf.main(["ledger", "check", "--file", f]) == 1
    # slower: rejected; perplexity-style number with a regression beyond the tolerance: rejected
    perf.main(base + ["--variant", "slower", "--baseline-ms", "1.0", "--variant-ms", "1.1"])
    assert perf.main(["ledger", "check", "--file", f]) == 1
    perf.main(base + ["--variant", "ppl", "--baseline-ms", "2.0", "--variant-ms", "1.0", "--quality-baseline", "6.0", "--quality-variant", "6.1",
                      "--lower-is-better"])
    assert perf.main(["ledger", "check", "--file", f]) == 1
    rows = [json.loads(l) for l in open(f)]
    assert [r["accepted"] for r in rows] == [True, False, False, False] and abs(rows[0]["speedup"] - 4.0067) < 1e-3
    capsys.readouterr()
    perf.main(["ledger", "summary", "--file", f])
    out = capsys.readouterr().out
    assert "4 entries, 1 accepted" in out and "mxf4_gemm x4.01" in out


def test_roofline_classes_and_report(tmp_path, capsys):
    kp, ncu, cap, page = (str(tmp_path / n) for n in ("k.txt", "n.csv", "c.json", "r.html"))
    open(kp, "w").write(KPROFILE)
    hdr = ["ID", "Kernel Name", "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed", "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active"]
    open(ncu, "w").write(",".join(f'"{h}"' for h in hdr) + '\n"","","%","%"\n"0","mx::mxf4_gemm_kernel(CUtensorMap_st, Mxf4Params)","51.2","47.5"\n'
                         '"1","void mx::fa_prefill_kernel<64, 0>(FaParams)","1.2","17.3"\n"2","mx::gemm_kernel<0>(GemmParams)","70.0","30.0"\n')
    assert perf.main(["roofline", "--kprofile", kp, "--ncu", ncu, "--out", cap]) == 0
    c = json.load(open(cap))
    bound = {o["name"]: o["bound"] for o in c["ops"]}
    assert bound == {"mxf4_gemm": "tensor", "gemm": "bandwidth", "attention": "unknown", "rmsnorm": "launch"}
    assert abs(c["total_ms"] - 29.969) < 1e-6 and c["ops"][0]["name"] == "mxf4_gemm" and c["peaks"]["hbm_gbs"] > 1000
    assert perf.main(["viz", cap, page]) == 0
    html = open(page).read()
    assert "mxf4_gemm" in html and "tensor pipe is the busiest unit" in html


def test_trace_export(tmp_path, capsys):
    kp, out = str(tmp_path / "k.txt"), str(tmp_path / "t.json")
    open(kp, "w").write(KPROFILE)
    assert perf.main(["trace", "--kprofile", kp, "--out", out, "--session", "s1", "--model", "gpt-oss-120b", "--ctx", "2048", "--tok-s", "61000"]) == 0
    t = json.load(open(out))
    ev = [e for e in t["traceEvents"] if e["ph"] == "X"]
    assert [e["name"] for e in ev][0] == "mxf4_gemm" and ev[0]["ts"] == 0 and abs(ev[1]["ts"] - ev[0]["dur"]) < 1e-3     # laid end to end
    assert abs(sum(e["dur"] for e in ev) / 1e3 - t["otherData"]["total_ms"]) < 1e-2 and ev[0]["args"]["model"] == "gpt-oss-120b"
    lanes = {e["args"]["name"] for e in t["traceEvents"] if e["name"] == "thread_name"}
    assert {"matmul", "attention", "norm"} <= lanes
