"""Engine scheduling, prefix cache, failure handling and the HTTP server on the CPU oracle path.

Failure injection follows the host-side recipe: a request that cannot fit, a pool that runs dry, a client that goes
away, a step that raises -- none of them may take the other requests or the server down (reference tests:
tests/unit/prefix_cache_test.cpp, engine_test.cpp, openai_server_test.cpp)."""
import http.client
import json
import threading
import time

import pytest
import torch

from machx_inference_engine_b200.formats.model_config import preset
from machx_inference_engine_b200.formats.synth import write_synthetic_gguf
from machx_inference_engine_b200.models import build_model
from machx_inference_engine_b200.runtime.api import Engine, EngineLoop
from machx_inference_engine_b200.runtime.engine import (BlockManager, ContextLengthExceeded, EngineOptions, LLMEngine, OutOfBlocks,
                                                        SamplingParams, Sequence)

KV = 128


@pytest.fixture(scope="module")
def model():
    return build_model(preset("tiny-llama"), "cpu", quant="q8_0", max_ctx=1024)


def test_block_manager_prefix_sharing_and_lru():
    bm = BlockManager(6)
    toks = list(range(300))
    s = Sequence(0, toks, SamplingParams(), tokens=list(toks))
    s.blocks = bm.allocate(3)
    s.n_computed = 300
    bm.publish(s)
    assert len(s.block_hashes) == 2                                # only full blocks are indexed
    blocks, hashes = bm.match_prefix(toks)
    assert blocks == s.blocks[:2] and hashes == s.block_hashes and bm.ref[blocks[0]] == 2
    other = list(range(128)) + [999] * 172                          # shares the first block only
    b2, _ = bm.match_prefix(other)
    assert b2 == s.blocks[:1]
    assert bm.match_prefix(list(range(128)))[0] == []              # the last token is always recomputed
    bm.release(blocks); bm.release(b2); bm.release(s.blocks)
    assert bm.n_free() == 5 and len(bm.evictable) == 2             # cached blocks stay matchable until evicted
    again, _ = bm.match_prefix(toks)
    assert again == s.blocks[:2]
    bm.release(again)
    got = bm.allocate(5)                                           # pool pressure evicts the cached blocks, oldest first
    assert len(got) == 5 and bm.match_prefix(toks)[0] == []
    with pytest.raises(OutOfBlocks):
        bm.allocate(1)


def test_continuous_batching_matches_sequential(model):
    V = model.cfg.vocab
    prompts = [[(i * 7 + j) % V for i in range(n)] for j, n in enumerate((5, 140, 33, 260))]
    sp = SamplingParams(max_tokens=8, ignore_eos=True)
    solo = [LLMEngine(model, EngineOptions(max_ctx=512, max_seqs=4)).generate([p], sp)[0] for p in prompts]
    eng = LLMEngine(model, EngineOptions(max_ctx=512, max_seqs=4, max_batch_tokens=64))       # chunked prefill mixed with decode
    both = eng.generate(prompts, sp)
    assert [b[:4] for b in both] == [s[:4] for s in solo]
    assert eng.stats["prefill_tokens"] == sum(len(p) for p in prompts) and eng.stats["decode_tokens"] > 0


def test_prefix_cache_reuses_blocks_and_keeps_outputs(model):
    V = model.cfg.vocab
    shared = [(i * 13 + 1) % V for i in range(300)]
    eng = LLMEngine(model, EngineOptions(max_ctx=1024, max_seqs=2))
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    first = eng.generate([shared + [5, 6, 7]], sp)[0]
    pre = eng.stats["prefill_tokens"]
    seq = eng.add_request(shared + [5, 6, 7], sp)
    while not seq.finished:
        eng.step()
    assert seq.n_cached_prefix == 2 * KV and eng.stats["prefill_tokens"] - pre == len(shared) + 3 - 2 * KV
    assert seq.tokens[len(seq.prompt):] == first
    cold = LLMEngine(model, EngineOptions(max_ctx=1024, max_seqs=2, enable_prefix_cache=False)).generate([shared + [5, 6, 7]], sp)[0]
    assert cold == first


def test_stop_conditions_sampling_and_budget(model):
    V = model.cfg.vocab
    eng = LLMEngine(model, EngineOptions(max_ctx=256, max_seqs=2))
    with pytest.raises(ContextLengthExceeded):
        eng.add_request(list(range(250)))
    with pytest.raises(ValueError):
        eng.add_request([])
    greedy = eng.generate([[1, 2, 3]], SamplingParams(max_tokens=5, ignore_eos=True))[0]
    stop_at = greedy[2]
    seq = eng.add_request([1, 2, 3], SamplingParams(max_tokens=50, stop_ids=(stop_at,)))
    while not seq.finished:
        eng.step()
    assert seq.finish_reason == "stop" and seq.tokens[-1] == stop_at and seq.n_generated <= 3
    a = eng.generate([[1, 2, 3]], SamplingParams(max_tokens=12, temperature=1.0, top_k=50, seed=7, ignore_eos=True))[0]
    b = eng.generate([[1, 2, 3]], SamplingParams(max_tokens=12, temperature=1.0, top_k=50, seed=8, ignore_eos=True))[0]
    assert all(0 <= t < V for t in a) and a != b
    long = eng.add_request([1, 2, 3], SamplingParams(max_tokens=0, ignore_eos=True))      # unlimited: ends when the context is full
    while not long.finished:
        eng.step()
    assert long.finish_reason == "length" and len(long.tokens) == 256


def test_pool_exhaustion_preempts_and_recovers(model):
    V = model.cfg.vocab
    eng = LLMEngine(model, EngineOptions(max_ctx=512, max_seqs=3, num_blocks=5, enable_prefix_cache=False))   # 4 usable blocks
    prompts = [[(i + j) % V for i in range(200)] for j in range(3)]                                            # 2 blocks each
    sp = SamplingParams(max_tokens=70, ignore_eos=True)                                                        # grows into a third
    outs = eng.generate(prompts, sp)
    assert all(len(o) == 70 for o in outs)
    solo = LLMEngine(model, EngineOptions(max_ctx=512, max_seqs=1)).generate([prompts[2]], sp)[0]
    assert outs[2][:5] == solo[:5]
    tiny = LLMEngine(model, EngineOptions(max_ctx=512, max_seqs=1, num_blocks=2))
    tiny.add_request(list(range(200)))
    with pytest.raises(OutOfBlocks):
        tiny.step()


def test_engine_loop_isolates_failures(model):
    e = Engine(model, None, EngineOptions(max_ctx=256, max_seqs=4))
    loop = EngineLoop(e)
    loop.start()
    done = {}
    ev = {k: threading.Event() for k in ("ok", "long", "gone", "ok2")}

    def fin(k):
        return lambda res: (done.__setitem__(k, res), ev[k].set())
    loop.submit([1, 2, 3], SamplingParams(max_tokens=6, ignore_eos=True), None, fin("ok"))
    loop.submit(list(range(300)), SamplingParams(max_tokens=6), None, fin("long"))                       # does not fit the context
    tk = loop.submit([4, 5, 6], SamplingParams(max_tokens=200, ignore_eos=True), None, fin("gone"))
    time.sleep(0.05)
    loop.abort(tk)                                                                                       # client went away
    for k in ("ok", "long", "gone"):
        assert ev[k].wait(30), k
    assert done["ok"].completion_tokens == 6 and done["ok"].finish_reason == "length"
    assert done["long"].finish_reason == "context_length_exceeded" and "300" in done["long"].error
    assert done["gone"].finish_reason == "abort" and done["gone"].completion_tokens < 200
    # a step that raises fails the running requests, not the loop
    orig = e.llm.step
    calls = {"n": 0}

    def flaky():
        calls["n"] += 1
        if calls["n"] == 2:
            raise RuntimeError("injected step failure")
        return orig()
    e.llm.step = flaky
    loop.submit([7, 8, 9], SamplingParams(max_tokens=20, ignore_eos=True), None, fin("ok2"))
    assert ev["ok2"].wait(30) and done["ok2"].finish_reason == "error"
    e.llm.step = orig
    ev["ok"].clear()
    loop.submit([1, 2, 3], SamplingParams(max_tokens=6, ignore_eos=True), None, fin("ok"))
    assert ev["ok"].wait(30) and done["ok"].completion_tokens == 6
    assert loop.metrics["requests"] == 5 and loop.metrics["errors"] >= 2
    loop.stop()


@pytest.fixture(scope="module")
def server(tmp_path_factory):
    from machx_inference_engine_b200.server.openai_server import run_openai_server
    path = str(tmp_path_factory.mktemp("srv") / "m.gguf")
    write_synthetic_gguf(preset("tiny-qwen3"), path, quant="q8_0", seed=3)
    eng = Engine.load(path, "cpu", EngineOptions(max_ctx=512, max_seqs=4))
    ready = threading.Event()
    th = threading.Thread(target=run_openai_server, args=(eng, "tiny", "127.0.0.1", 0, ready), daemon=True)
    th.start()
    assert ready.wait(30)
    yield ready.httpd.server_address[1]
    ready.httpd.shutdown()


def _req(port, method, path, body=None):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=60)
    c.request(method, path, body=None if body is None else json.dumps(body), headers={"Content-Type": "application/json"})
    r = c.getresponse()
    data = r.read()
    c.close()
    return r.status, data


def test_server_routes_and_errors(server):
    assert _req(server, "GET", "/health") == (200, b'{"status": "ok"}')
    st, body = _req(server, "GET", "/v1/models")
    assert st == 200 and json.loads(body)["data"][0]["id"] == "tiny"
    assert _req(server, "POST", "/v1/embeddings", {"input": "x"})[0] == 501
    assert _req(server, "GET", "/nope")[0] == 404
    st, body = _req(server, "POST", "/v1/chat/completions", {"messages": []})
    assert st == 400 and json.loads(body)["error"]["type"] == "invalid_request_error"
    st, body = _req(server, "POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "x " * 2000}], "max_tokens": 4})
    assert st == 400 and json.loads(body)["error"]["code"] == "context_length_exceeded"
    st, body = _req(server, "GET", "/metrics")
    assert st == 200 and b"mx_requests_total" in body


def test_server_chat_json_stream_and_concurrency(server):
    msg = {"messages": [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hello"}], "max_tokens": 8, "temperature": 0}
    st, body = _req(server, "POST", "/v1/chat/completions", msg)
    r = json.loads(body)
    assert st == 200 and r["object"] == "chat.completion" and r["choices"][0]["finish_reason"] in ("stop", "length")
    assert r["usage"]["completion_tokens"] >= 1 and r["usage"]["prompt_tokens"] > 5
    st, body = _req(server, "POST", "/v1/chat/completions", {**msg, "stream": True})
    frames = [f for f in body.decode().split("\n\n") if f]
    assert st == 200 and frames[-1] == "data: [DONE]" and all(f.startswith("data: ") for f in frames)
    objs = [json.loads(f[6:]) for f in frames[:-1]]
    assert objs[0]["choices"][0]["delta"]["role"] == "assistant"
    assert any(o["choices"] and o["choices"][0]["finish_reason"] for o in objs) and "usage" in objs[-1]
    streamed = "".join(o["choices"][0]["delta"].get("content", "") for o in objs if o["choices"])
    assert streamed == (r["choices"][0]["message"]["content"] or "")              # greedy: both transports give the same text
    results = []

    def worker(i):
        results.append(_req(server, "POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": f"q{i}"}], "max_tokens": 6, "temperature": 0}))
    ths = [threading.Thread(target=worker, args=(i,)) for i in range(6)]
    [t.start() for t in ths]
    [t.join(60) for t in ths]
    assert len(results) == 6 and all(s == 200 for s, _ in results)
