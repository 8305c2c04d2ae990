"""Expert banks past a device budget stay in host memory and are staged per forward: which layers spill, the accounting, and that a
graph with spilled layers computes what the resident graph computes (CPU here; on a GPU in test_gpu_models.py)."""
import torch

from machx_inference_engine_b200.formats.model_config import preset
from machx_inference_engine_b200.models import build_model, spill
from machx_inference_engine_b200.runtime.engine import EngineOptions, LLMEngine, SamplingParams


def _tokens(model, prompts):
    eng = LLMEngine(model, EngineOptions(max_ctx=256, max_batch_tokens=64, max_seqs=2))
    return eng.generate(prompts, SamplingParams(max_tokens=6))


def test_budget_decides_in_layer_order_and_outputs_do_not_change():
    cfg = preset("tiny-gpt-oss")
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (11, 40)]
    try:
        spill.configure(None)
        base = build_model(cfg, torch.device("cpu"), quant="mxfp4", max_ctx=256)
        bank = sum(b.nbytes for b in (base.layers[0]["moe"].gate_up, base.layers[0]["moe"].down))
        want = _tokens(base, prompts)
        assert all(L["moe"]._spill is None for L in base.layers)
        # room for one layer's banks and a half: the first layer stays, the rest spill
        acc = spill.configure(1.5 * bank / 1e9)
        m = build_model(cfg, torch.device("cpu"), quant="mxfp4", max_ctx=256)
        flags = [L["moe"]._spill is not None for L in m.layers]
        assert flags == [False] + [True] * (cfg.n_layers - 1)
        assert acc.resident_bytes == bank and acc.spilled_bytes == bank * (cfg.n_layers - 1) and acc.layers_spilled == cfg.n_layers - 1
        assert _tokens(m, prompts) == want
        # two spilled layers share one staging area: each forward re-stages its own banks
        a, b = m.layers[1]["moe"], m.layers[2]["moe"] if cfg.n_layers > 2 else m.layers[1]["moe"]
        a._stage_banks()
        pa = a.gate_up.p0.data_ptr()
        b._stage_banks()
        assert b.gate_up.p0.data_ptr() == pa
        # a budget of zero spills everything
        spill.configure(0.0)
        m0 = build_model(cfg, torch.device("cpu"), quant="mxfp4", max_ctx=256)
        assert all(L["moe"]._spill is not None for L in m0.layers) and _tokens(m0, prompts) == want
    finally:
        spill.configure(None)
