"""The validation tools and the serving benchmark run end to end on the CPU path with a tiny model."""
import json

from machx_inference_engine_b200.cli import serve_bench, tools


def _last_json(capsys):
    return json.loads(capsys.readouterr().out.strip().splitlines()[-1])


def test_det_probe_chunk_check_perplexity(capsys):
    assert tools.main(["det-probe", "--model", "tiny-llama", "--device", "cpu", "--runs", "2", "--tokens-n", "120"]) == 0
    assert _last_json(capsys)["bit_identical"] is True
    assert tools.main(["chunk-check", "--model", "tiny-qwen3next", "--device", "cpu", "--tokens-n", "200", "--chunks", "64"]) == 0
    assert _last_json(capsys)["vs_whole_prompt"]["64"]["cos_min"] > 0.999
    assert tools.main(["perplexity", "--model", "tiny-llama", "--device", "cpu", "--ctx", "100"]) == 0
    r = _last_json(capsys)
    assert r["tokens"] == 99 and 1000 < r["perplexity"] < 20000          # random-init model: about the vocabulary size


def test_soak_and_serve_bench(capsys):
    assert tools.main(["soak", "--model", "tiny-llama", "--device", "cpu", "--seconds", "2", "--concurrency", "3"]) == 0
    r = _last_json(capsys)
    assert r["failures"] == 0 and r["completions"] > 0
    assert serve_bench.main(["--model", "tiny-gpt-oss", "--device", "cpu", "--requests", "5", "--min-prompt", "10", "--max-prompt", "150", "--decode", "6"]) == 0
    r = _last_json(capsys)
    assert r["errors"] == 0 and r["generated_tokens"] == 30 and r["ttft_p50_s"] > 0


def test_layer_dump_and_diff(tmp_path, capsys):
    from machx_inference_engine_b200.formats.model_config import preset
    from machx_inference_engine_b200.formats.synth import write_synthetic_gguf
    g = str(tmp_path / "m.gguf")
    write_synthetic_gguf(preset("tiny-qwen3next"), g, quant="q8_0", seed=5)
    a, b = str(tmp_path / "a.pt"), str(tmp_path / "b.pt")
    assert tools.main(["layer-dump", "--gguf", g, "--device", "cpu", "--out", a, "--tokens-n", "40", "--chunk", "16"]) == 0
    assert _last_json(capsys)["positions"] == 40
    assert tools.main(["layer-dump", "--gguf", g, "--device", "cpu", "--out", b, "--tokens-n", "40", "--chunk", "64"]) == 0
    capsys.readouterr()
    assert tools.main(["layer-diff", a, b]) == 0                      # chunked against whole-prompt: the same activations
    r = _last_json(capsys)
    assert r["first_layer_below_threshold"] is None and r["logits_cos_min"] > 0.999
    import torch
    d = torch.load(b, weights_only=False)
    d["layers"][1]["resid"] = d["layers"][1]["resid"] + torch.randn_like(d["layers"][1]["resid"])
    torch.save(d, b)
    assert tools.main(["layer-diff", a, b]) == 1
    assert _last_json(capsys)["first_layer_below_threshold"] == 1
    assert tools.main(["layer-parity", "--gguf", g, "--device", "cpu", "--tokens-n", "24"]) == 0


def test_spec_accept_kv_scale_partial_stack(capsys):
    # acceptance and speed-up of self-speculative decoding: the random-init head accepts nothing, perfect drafts accept everything,
    # and every variant reproduces plain greedy decoding
    assert tools.main(["spec-accept", "--model", "tiny-qwen3next", "--device", "cpu", "--max-tokens", "20", "--prompt-n", "40", "--accept", "0.0,1.0"]) == 0
    r = _last_json(capsys)
    acc = {row["draft"]: row for row in r["rows"]}
    assert all(row["lossless"] for row in r["rows"]) and acc["oracle, per-position hit rate 1.0"]["acceptance"] == 1.0
    assert acc["oracle, per-position hit rate 0.0"]["acceptance"] == 0.0
    assert acc["oracle, per-position hit rate 1.0"]["tok_s"] > acc["oracle, per-position hit rate 0.0"]["tok_s"]
    # int8 KV rows against bf16 rows
    assert tools.main(["kv-scale", "--model", "tiny-llama", "--device", "cpu", "--tokens-n", "150"]) == 0
    r = _last_json(capsys)
    assert r["cos_min"] > 0.999 and abs(r["nll_bf16"] - r["nll_int8"]) < 0.01
    # the model cut after one layer differs from the whole model; the last cut is the whole model
    assert tools.main(["partial-stack", "--model", "tiny-llama", "--device", "cpu", "--layers", "1", "--tokens-n", "48"]) == 0
    r = _last_json(capsys)
    assert [c["layers"] for c in r["cuts"]] == [1, 2] and r["cuts"][0]["argmax_checksum"] != r["cuts"][1]["argmax_checksum"]


def test_bug_monitor_finds_an_injected_divergence(capsys):
    """Identical decode chains stay bit-identical (one forward each, and as one batch); a single flipped bit in one chain's recurrent
    state or K rows is reported with its step, chain and buffer (the reference's 8-chain monitor: tools/ie_bug_monitor.cpp)."""
    for model in ("tiny-qwen3next", "tiny-llama"):
        for extra in ([], ["--batched"]):
            assert tools.main(["bug-monitor", "--model", model, "--device", "cpu", "--chains", "3", "--iters", "5"] + extra) == 0
            r = _last_json(capsys)
            assert r["diverged"] is False and r["chains"] == 3 and r["steps"] == 5
    assert tools.main(["bug-monitor", "--model", "tiny-qwen3next", "--device", "cpu", "--chains", "3", "--iters", "5", "--inject", "2,1,1"]) == 0
    r = _last_json(capsys)
    assert r["first_divergence"] == {"step": 2, "chain": 1, "buffer": "DN_state[1]"}
    assert tools.main(["bug-monitor", "--model", "tiny-llama", "--device", "cpu", "--chains", "4", "--iters", "5", "--batched", "--inject", "3,2,0"]) == 0
    r = _last_json(capsys)
    assert r["first_divergence"] == {"step": 3, "chain": 2, "buffer": "KV_K[0]"} and r["diverged_at_end"] == [{"chain": 2, "buffer": "KV_K[0]"}]


def test_kernel_monitor_and_attn_profile(capsys):
    assert tools.main(["kernel-monitor", "--model", "tiny-qwen3next", "--device", "cpu", "--decode", "4", "--warmup", "1", "--interval", "2", "--tokens-n", "20"]) == 0
    r = _last_json(capsys)
    ops = [o["op"] for o in r["ops"]]
    assert r["steps"] == 4 and ops[0] == "embed" and {"deltanet_scan", "attention", "linear", "argmax"} <= set(ops)
    assert abs(sum(o["share"] for o in r["ops"]) - 1.0) < 1e-6 and ops.index("embed") < ops.index("argmax")      # dispatch order
    assert tools.main(["attn-profile", "--device", "cpu", "--ctx", "200,300", "--steps", "2", "--warmup", "1", "--layers", "2", "--q-heads", "4",
                       "--kv-heads", "2", "--head-dim", "64"]) == 0
    r = _last_json(capsys)
    assert [x["ctx"] for x in r["rows"]] == [200, 300] and r["rows"][0]["int8"]["kv_bytes"] < r["rows"][0]["bf16"]["kv_bytes"]


def test_debug_prompt_loop(capsys, tmp_path):
    from machx_inference_engine_b200.formats.model_config import preset
    from machx_inference_engine_b200.formats.synth import write_synthetic_gguf
    assert tools.main(["debug", "--model", "tiny-llama", "--device", "cpu", "--script", "T 1 2 3;T 4 5;R;T 1 2 3 4 5;P hi;Z;Q;T 9"]) == 0
    rows = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
    assert [r.get("context_tokens") for r in rows] == [3, 5, None, 5, None, None] and rows[2] == {"reset": True}
    assert rows[1]["argmax"] == rows[3]["argmax"] and rows[1]["top5"] == rows[3]["top5"]        # appended context == the same ids at once
    assert "no tokenizer" in rows[4]["error"] and "unknown command" in rows[5]["error"]
    path = str(tmp_path / "m.gguf")
    write_synthetic_gguf(preset("tiny-llama"), path, quant="q8_0", seed=1)
    assert tools.main(["debug", "--gguf", path, "--device", "cpu", "--script", "P Hello world;P again"]) == 0
    rows = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
    assert rows[1]["context_tokens"] > rows[0]["context_tokens"] > 1 and "text" in rows[0]["top5"][0]


def test_perplexity_over_two_ranks_matches_one(capsys):
    """The same tool under torchrun (two gloo ranks, tensor-parallel graph): rank 0 reports, and the number is the single-rank one up to
    the summation order (the reference's multi-GPU perplexity / equality tools: tools/multi_gpu_ppl.cpp, tools/multi_gpu_equality_test.cpp)."""
    import os
    import socket
    import subprocess
    import sys
    assert tools.main(["perplexity", "--model", "tiny-llama", "--device", "cpu", "--ctx", "64"]) == 0
    one = _last_json(capsys)
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", str(port),
                        "-m", "machx_inference_engine_b200.cli.tools", "perplexity", "--model", "tiny-llama", "--device", "cpu", "--ctx", "64"],
                       capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    rows = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(rows) == 1 and rows[0]["tokens"] == one["tokens"]                     # one report for the job
    assert abs(rows[0]["perplexity"] - one["perplexity"]) / one["perplexity"] < 2e-2
