"""Model graphs.  ``load_model`` opens a GGUF checkpoint; ``build_model`` random-initialises a named architecture."""
from __future__ import annotations

from typing import Optional

from ..formats.model_config import ModelConfig, read_config
from ..parallel.comm import ParallelCtx


def _graph_class(cfg: ModelConfig):
    if cfg.is_hybrid:
        from .hybrid import HybridModel
        return HybridModel
    if cfg.arch == "gemma4":
        from .gemma4 import Gemma4Model
        return Gemma4Model
    from .transformer import TransformerModel
    return TransformerModel


def build_model(cfg: ModelConfig, device, par: Optional[ParallelCtx] = None, quant: str = "q8_0", max_ctx: int = 8192, seed: int = 0,
                gen_device=None):
    """Random-init weights of architecture ``cfg`` quantised with recipe ``quant`` directly on ``device``."""
    from .sources import SynthSource, default_policy
    src = SynthSource(device, default_policy(cfg.arch, quant), seed=seed, n_layers=cfg.n_layers, gen_device=gen_device)
    return _graph_class(cfg)(cfg, src, device, par or ParallelCtx(), max_ctx=max_ctx)


def load_model(path: str, device, par: Optional[ParallelCtx] = None, max_ctx: int = 8192):
    """Loads a GGUF checkpoint (split shards are merged) onto ``device``; returns (model, reader)."""
    from ..formats.gguf import GGUFReader
    from .sources import GGUFSource
    reader = GGUFReader(path)
    cfg = read_config(reader.kv, reader.tensors.keys())
    model = _graph_class(cfg)(cfg, GGUFSource(reader, device), device, par or ParallelCtx(), max_ctx=min(max_ctx, max(cfg.ctx_train, 256)))
    return model, reader
