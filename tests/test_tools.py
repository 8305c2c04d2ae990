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
