"""Worker for the SPMD serving test: every rank runs the engine loop over its shard; rank 0 submits requests (one is
aborted, one does not fit) and prints what came back.  Mode "die": rank 1 leaves between steps; rank 0 must find out
through the control group's timeout instead of hanging."""
import json
import os
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from machx_inference_engine_b200.formats.model_config import preset
from machx_inference_engine_b200.models import build_model
from machx_inference_engine_b200.parallel.comm import init_from_env
from machx_inference_engine_b200.runtime.api import Engine, EngineLoop
from machx_inference_engine_b200.runtime.engine import EngineOptions, SamplingParams


def main():
    mode = sys.argv[1]
    par = init_from_env("cpu", timeout_s=8 if mode == "die" else 120)
    cfg = preset("tiny-llama")
    model = build_model(cfg, "cpu", par, quant="q8_0", max_ctx=512, gen_device="cpu")
    eng = Engine(model, None, EngineOptions(max_ctx=512, max_seqs=4))
    loop = EngineLoop(eng, par)
    if par.rank != 0:
        if mode == "die":
            # leaves before the first step plan: nothing of its own is in flight.  Exit code 0: a non-zero code makes the launcher
            # terminate the surviving rank, which would race with the detection that this test is about
            os._exit(0)
        loop.run()
        os._exit(0)
    done, evs = {}, {k: threading.Event() for k in ("a", "b", "long", "gone")}
    fin = lambda k: (lambda res: (done.__setitem__(k, res), evs[k].set()))
    if mode == "die":
        try:
            loop.run()                                    # the first broadcast of a step plan fails once the peer is gone
            print("RESULT " + json.dumps({"detected": False}))
        except Exception as e:
            print("RESULT " + json.dumps({"detected": True, "error": type(e).__name__}))
        sys.stdout.flush()
        os._exit(0)
    loop.start()
    V = cfg.vocab
    loop.submit([(i * 7) % V for i in range(40)], SamplingParams(max_tokens=8, ignore_eos=True), None, fin("a"))
    loop.submit([(i * 5 + 1) % V for i in range(150)], SamplingParams(max_tokens=8, ignore_eos=True), None, fin("b"))
    loop.submit(list(range(600)), SamplingParams(max_tokens=4), None, fin("long"))
    tk = loop.submit([3, 4, 5], SamplingParams(max_tokens=300, ignore_eos=True), None, fin("gone"))
    time.sleep(0.3)
    loop.abort(tk)
    ok = all(evs[k].wait(90) for k in evs)
    loop.stop()
    loop.join(30)
    print("RESULT " + json.dumps({"ok": ok, "a": done["a"].token_ids, "b": done["b"].token_ids, "long": done["long"].finish_reason,
                                  "gone": done["gone"].finish_reason, "world": par.world}))
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
