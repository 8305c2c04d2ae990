"""Architecture detection and one typed config for every model family.

Reference parity: src/loaders/model_config.cpp:8-359 and include/ie/model_config.hpp:12-254
(``detect_arch``, ``read_dense_config``, ``read_{qwen35,qwen3moe,gptoss,qwen3next,gemma4}_config``,
template-family classification, sliding-window load guard, Granite scalars).  The reference
keeps one struct per family; here one dataclass serves all graphs.
"""
from __future__ import annotations

from dataclasses import dataclass, field, asdict
from typing import Any, Mapping

DENSE_ARCHS = ("llama", "qwen2", "qwen3", "phi3", "granite", "mistral")
MOE_ARCHS = ("qwen3moe", "gpt-oss")
HYBRID_ARCHS = ("qwen3next", "qwen35", "qwen35moe")
GEMMA_ARCHS = ("gemma4",)
SUPPORTED_ARCHS = DENSE_ARCHS + MOE_ARCHS + HYBRID_ARCHS + GEMMA_ARCHS


class ConfigError(ValueError):
    pass


@dataclass
class ModelConfig:
    arch: str = "llama"
    n_layers: int = 0
    hidden: int = 0
    n_heads: int = 0
    n_kv_heads: int = 0
    head_dim: int = 0
    ffn: int = 0
    vocab: int = 0
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0
    n_rot: int = 0
    ctx_train: int = 4096
    sliding_window: int = 0
    # rope scaling (YaRN for gpt-oss, llama3 frequency factors come as a tensor)
    rope_scaling_type: str = "none"
    rope_scaling_factor: float = 1.0
    rope_orig_ctx: int = 0
    yarn_beta_fast: float = 32.0
    yarn_beta_slow: float = 1.0
    # mixture of experts
    n_experts: int = 0
    n_experts_used: int = 0
    expert_ffn: int = 0
    shared_expert_ffn: int = 0
    # hybrid (gated DeltaNet) models
    full_attn_interval: int = 0
    ssm_inner: int = 0
    ssm_state: int = 0
    ssm_n_k_heads: int = 0
    ssm_n_v_heads: int = 0
    ssm_conv_kernel: int = 0
    nextn_predict_layers: int = 0
    # Gemma-4: two head geometries chosen per layer (include/ie/model_config.hpp:216-249); head_dim / n_rot / rope_theta above
    # describe the global (full-attention) layers, the *_swa fields the sliding-window layers
    head_dim_swa: int = 0
    n_rot_swa: int = 0
    rope_theta_swa: float = 10000.0
    layer_swa: list = field(default_factory=list)        # per layer: True = sliding-window layer
    layer_n_kv: list = field(default_factory=list)       # per layer: KV head count
    # Granite scalars
    embedding_scale: float = 1.0
    residual_scale: float = 1.0
    attention_scale: float = 0.0       # 0 -> 1/sqrt(head_dim)
    logit_scale: float = 1.0
    final_logit_softcap: float = 0.0
    template_family: str = "auto"      # chatml | llama3 | mistral | deepseek | granite | gemma | harmony | auto
    mistral_sysprompt: bool = False
    tie_embeddings: bool = False
    name: str = ""

    # ---- derived
    @property
    def is_moe(self) -> bool:
        return self.n_experts > 0

    @property
    def is_hybrid(self) -> bool:
        return self.arch in HYBRID_ARCHS

    def layer_is_full_attention(self, layer: int) -> bool:
        if not self.is_hybrid:
            return True
        return (layer + 1) % self.full_attn_interval == 0

    def layer_window(self, layer: int) -> int:
        """Sliding window of a layer (0 = full).  gpt-oss windows the even layers (src/model/gptoss.cpp:133), Gemma-4 the
        layers its pattern marks (src/model/gemma4.cpp:709-714)."""
        if self.arch == "gpt-oss":
            return self.sliding_window if layer % 2 == 0 else 0
        if self.arch == "gemma4":
            return self.sliding_window if self.layer_swa[layer] else 0
        return self.sliding_window

    def layer_geometry(self, layer: int) -> tuple:
        """(head_dim, n_kv_heads, n_rot, rope_theta) of a layer."""
        if self.arch == "gemma4":
            swa = bool(self.layer_swa[layer])
            return (self.head_dim_swa if swa else self.head_dim, int(self.layer_n_kv[layer]), self.n_rot_swa if swa else self.n_rot,
                    self.rope_theta_swa if swa else self.rope_theta)
        return (self.head_dim, self.n_kv_heads, self.n_rot, self.rope_theta)

    def to_dict(self) -> dict:
        return asdict(self)


def detect_arch(kv: Mapping[str, Any]) -> str:
    a = kv.get("general.architecture")
    if a is None:
        raise ConfigError("GGUF has no general.architecture")
    if a not in SUPPORTED_ARCHS:
        raise ConfigError(f"unsupported architecture '{a}' (supported: {', '.join(SUPPORTED_ARCHS)})")
    return a


def classify_template_family(chat_template: str, arch: str = "") -> str:
    ct = chat_template or ""
    if "[INST]" in ct:
        return "mistral"
    if "<|start_header_id|>" in ct:
        return "llama3"
    if "<｜Assistant｜>" in ct:
        return "deepseek"
    if "<|start_of_role|>" in ct:
        return "granite"
    if "<|start|>" in ct and "<|channel|>" in ct or arch == "gpt-oss":
        return "harmony"
    if "<start_of_turn>" in ct:
        return "gemma"
    if "<|im_start|>" in ct:
        return "chatml"
    return "auto"


def read_config(kv: Mapping[str, Any], tensor_names=()) -> ModelConfig:
    arch = detect_arch(kv)
    c = ModelConfig(arch=arch, name=str(kv.get("general.name", "")))

    def get(suffix, default=None, required=False):
        k = f"{arch}.{suffix}"
        if k in kv and kv[k] is not None:
            return kv[k]
        if required:
            raise ConfigError(f"missing {k}")
        return default

    c.n_layers = int(get("block_count", required=True))
    c.hidden = int(get("embedding_length", required=True))
    c.n_heads = int(get("attention.head_count", required=True))
    hkv = get("attention.head_count_kv", c.n_heads)
    if isinstance(hkv, (list, tuple)):                                     # per-layer arrays: take the max
        c.n_kv_heads = max([int(v) for v in hkv if v] or [c.n_heads])
    else:
        c.n_kv_heads = int(hkv)
    c.ffn = int(get("feed_forward_length", 0) or 0)
    c.head_dim = int(get("attention.key_length", c.hidden // c.n_heads))
    c.n_rot = int(get("rope.dimension_count", c.head_dim))
    c.ctx_train = int(get("context_length", 4096))
    c.rope_theta = float(get("rope.freq_base", 10000.0))
    c.rms_eps = float(get("attention.layer_norm_rms_epsilon", 1e-5))
    c.sliding_window = int(get("attention.sliding_window", 0) or 0)
    if arch != "gpt-oss" and c.sliding_window and c.sliding_window < c.ctx_train:
        # every attention kernel here takes a window argument, so a windowed dense checkpoint is
        # served correctly (the reference refuses to load it); nothing to do
        pass
    if c.sliding_window >= c.ctx_train:
        c.sliding_window = 0
    c.embedding_scale = float(get("embedding_scale", 1.0))
    c.residual_scale = float(get("residual_scale", 1.0))
    c.attention_scale = float(get("attention.scale", 0.0))
    ls = float(get("logit_scale", 1.0))
    c.logit_scale = 1.0 / ls if (arch == "granite" and ls) else 1.0       # Granite divides logits by logits_scaling
    c.final_logit_softcap = float(get("final_logit_softcapping", 0.0))
    toks = kv.get("tokenizer.ggml.tokens")
    c.vocab = len(toks) if toks is not None else int(get("vocab_size", 0) or 0)
    if c.vocab == 0:
        raise ConfigError("missing tokenizer.ggml.tokens (vocabulary size unknown)")
    c.template_family = classify_template_family(str(kv.get("tokenizer.chat_template", "")), arch)
    c.mistral_sysprompt = "[SYSTEM_PROMPT]" in str(kv.get("tokenizer.chat_template", ""))
    c.rope_scaling_type = str(get("rope.scaling.type", "none"))
    c.rope_scaling_factor = float(get("rope.scaling.factor", 1.0))
    c.rope_orig_ctx = int(get("rope.scaling.original_context_length", 0) or 0)

    if arch == "gemma4":
        c.head_dim_swa = int(get("attention.key_length_swa", required=True))
        c.n_rot_swa = int(get("rope.dimension_count_swa", c.head_dim_swa))
        c.rope_theta_swa = float(get("rope.freq_base_swa", 10000.0))
        pat = get("attention.sliding_window_pattern", None)
        c.layer_swa = [bool(v) for v in pat] if isinstance(pat, (list, tuple)) else [False] * c.n_layers
        hk = get("attention.head_count_kv", required=True)
        c.layer_n_kv = [int(v) for v in hk] if isinstance(hk, (list, tuple)) else [int(hk)] * c.n_layers
        if len(c.layer_swa) != c.n_layers or len(c.layer_n_kv) != c.n_layers:
            raise ConfigError("gemma4: per-layer arrays do not match block_count")
        if any(c.n_heads % max(v, 1) for v in c.layer_n_kv):
            raise ConfigError("gemma4: attention.head_count is not a multiple of a layer's head_count_kv")
        c.embedding_scale = float(c.hidden) ** 0.5
        c.attention_scale = 1.0                 # q and k are RMS-normalised per head; the reference's net scale is 1
        if int(get("expert_count", 0) or 0) > 0:
            c.n_experts = int(get("expert_count"))
            c.n_experts_used = int(get("expert_used_count", required=True))
            c.expert_ffn = int(get("expert_feed_forward_length", required=True))
    if arch in ("qwen3moe", "gpt-oss", "qwen3next", "qwen35moe"):
        c.n_experts = int(get("expert_count", required=True))
        c.n_experts_used = int(get("expert_used_count", required=True))
        c.expert_ffn = int(get("expert_feed_forward_length", c.ffn) or c.ffn)
        c.shared_expert_ffn = int(get("expert_shared_feed_forward_length", 0) or 0)
        if c.n_experts_used > c.n_experts:
            raise ConfigError("expert_used_count exceeds expert_count")
    if arch in HYBRID_ARCHS:
        c.full_attn_interval = int(get("full_attention_interval", 4))
        if c.full_attn_interval <= 0:
            raise ConfigError(f"{arch}.full_attention_interval is zero")
        c.ssm_inner = int(get("ssm.inner_size", required=True))
        c.ssm_state = int(get("ssm.state_size", required=True))
        c.ssm_n_k_heads = int(get("ssm.group_count", required=True))
        c.ssm_n_v_heads = int(get("ssm.time_step_rank", required=True))
        c.ssm_conv_kernel = int(get("ssm.conv_kernel", required=True))
        if c.ssm_n_v_heads == 0:
            raise ConfigError(f"{arch}.ssm.time_step_rank is zero")
        c.nextn_predict_layers = int(get("nextn_predict_layers", 0) or 0)
    names = set(tensor_names)
    c.tie_embeddings = bool(names) and "output.weight" not in names
    for f in ("n_layers", "hidden", "n_heads", "head_dim"):
        if getattr(c, f) <= 0:
            raise ConfigError(f"invalid {f}={getattr(c, f)}")
    if c.n_heads % max(c.n_kv_heads, 1):
        raise ConfigError("attention.head_count is not a multiple of head_count_kv")
    return c


def config_to_kv(c: ModelConfig) -> dict:
    """Inverse of :func:`read_config` for the synthetic-checkpoint generator."""
    a = c.arch
    kv = {
        "general.architecture": a, "general.name": c.name or f"synthetic-{a}",
        f"{a}.block_count": c.n_layers, f"{a}.embedding_length": c.hidden, f"{a}.attention.head_count": c.n_heads,
        f"{a}.attention.head_count_kv": c.n_kv_heads, f"{a}.feed_forward_length": c.ffn, f"{a}.attention.key_length": c.head_dim,
        f"{a}.attention.value_length": c.head_dim, f"{a}.rope.dimension_count": c.n_rot or c.head_dim, f"{a}.context_length": c.ctx_train,
        f"{a}.rope.freq_base": float(c.rope_theta), f"{a}.attention.layer_norm_rms_epsilon": float(c.rms_eps),
    }
    if c.sliding_window:
        kv[f"{a}.attention.sliding_window"] = c.sliding_window
    if c.rope_scaling_type != "none":
        kv[f"{a}.rope.scaling.type"] = c.rope_scaling_type
        kv[f"{a}.rope.scaling.factor"] = float(c.rope_scaling_factor)
        kv[f"{a}.rope.scaling.original_context_length"] = c.rope_orig_ctx
    if c.n_experts:
        kv[f"{a}.expert_count"] = c.n_experts
        kv[f"{a}.expert_used_count"] = c.n_experts_used
        kv[f"{a}.expert_feed_forward_length"] = c.expert_ffn
        if c.shared_expert_ffn:
            kv[f"{a}.expert_shared_feed_forward_length"] = c.shared_expert_ffn
    if c.is_hybrid:
        kv[f"{a}.full_attention_interval"] = c.full_attn_interval
        kv[f"{a}.ssm.inner_size"] = c.ssm_inner
        kv[f"{a}.ssm.state_size"] = c.ssm_state
        kv[f"{a}.ssm.group_count"] = c.ssm_n_k_heads
        kv[f"{a}.ssm.time_step_rank"] = c.ssm_n_v_heads
        kv[f"{a}.ssm.conv_kernel"] = c.ssm_conv_kernel
        if c.nextn_predict_layers:
            kv[f"{a}.nextn_predict_layers"] = c.nextn_predict_layers
    if a == "gemma4":
        kv[f"{a}.attention.head_count_kv"] = [int(v) for v in c.layer_n_kv]
        kv[f"{a}.attention.sliding_window_pattern"] = [bool(v) for v in c.layer_swa]
        kv[f"{a}.attention.key_length_swa"] = c.head_dim_swa
        kv[f"{a}.attention.value_length_swa"] = c.head_dim_swa
        kv[f"{a}.rope.dimension_count_swa"] = c.n_rot_swa or c.head_dim_swa
        kv[f"{a}.rope.freq_base_swa"] = float(c.rope_theta_swa)
        kv[f"{a}.final_logit_softcapping"] = float(c.final_logit_softcap)
    if a == "granite":
        kv[f"{a}.embedding_scale"] = float(c.embedding_scale)
        kv[f"{a}.residual_scale"] = float(c.residual_scale)
        kv[f"{a}.attention.scale"] = float(c.attention_scale)
        kv[f"{a}.logit_scale"] = float(1.0 / c.logit_scale) if c.logit_scale else 1.0
    return kv


# ---- named architectures used by the benches and tests (random-init; see formats/synth.py)
def preset(name: str) -> ModelConfig:
    p = {
        "tiny-llama": ModelConfig(arch="llama", n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=688, vocab=4096,
                                  rms_eps=1e-5, rope_theta=10000.0, n_rot=64, ctx_train=2048),
        "llama-3-8b": ModelConfig(arch="llama", n_layers=32, hidden=4096, n_heads=32, n_kv_heads=8, head_dim=128, ffn=14336,
                                  vocab=128256, rms_eps=1e-5, rope_theta=500000.0, n_rot=128, ctx_train=8192),
        "gpt-oss-20b": ModelConfig(arch="gpt-oss", n_layers=24, hidden=2880, n_heads=64, n_kv_heads=8, head_dim=64, ffn=2880,
                                   vocab=201088, rms_eps=1e-5, rope_theta=150000.0, n_rot=64, ctx_train=131072, sliding_window=128,
                                   n_experts=32, n_experts_used=4, expert_ffn=2880, rope_scaling_type="yarn", rope_scaling_factor=32.0,
                                   rope_orig_ctx=4096),
        "gpt-oss-120b": ModelConfig(arch="gpt-oss", n_layers=36, hidden=2880, n_heads=64, n_kv_heads=8, head_dim=64, ffn=2880,
                                    vocab=201088, rms_eps=1e-5, rope_theta=150000.0, n_rot=64, ctx_train=131072, sliding_window=128,
                                    n_experts=128, n_experts_used=4, expert_ffn=2880, rope_scaling_type="yarn",
                                    rope_scaling_factor=32.0, rope_orig_ctx=4096),
        "tiny-gpt-oss": ModelConfig(arch="gpt-oss", n_layers=4, hidden=256, n_heads=8, n_kv_heads=2, head_dim=64, ffn=256, vocab=2048,
                                    rms_eps=1e-5, rope_theta=150000.0, n_rot=64, ctx_train=4096, sliding_window=128, n_experts=8,
                                    n_experts_used=2, expert_ffn=256),
        "qwen3-moe-30b": ModelConfig(arch="qwen3moe", n_layers=48, hidden=2048, n_heads=32, n_kv_heads=4, head_dim=128, ffn=6144,
                                     vocab=151936, rms_eps=1e-6, rope_theta=1e6, n_rot=128, ctx_train=40960, n_experts=128,
                                     n_experts_used=8, expert_ffn=768),
        "tiny-qwen3moe": ModelConfig(arch="qwen3moe", n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=2048,
                                     rms_eps=1e-6, rope_theta=1e6, n_rot=64, ctx_train=4096, n_experts=8, n_experts_used=2, expert_ffn=256),
        "qwen3-next-80b": ModelConfig(arch="qwen3next", n_layers=48, hidden=2048, n_heads=16, n_kv_heads=2, head_dim=256, ffn=5120,
                                      vocab=151936, rms_eps=1e-6, rope_theta=1e7, n_rot=64, ctx_train=262144, n_experts=512,
                                      n_experts_used=10, expert_ffn=512, shared_expert_ffn=512, full_attn_interval=4, ssm_inner=4096,
                                      ssm_state=128, ssm_n_k_heads=16, ssm_n_v_heads=32, ssm_conv_kernel=4, nextn_predict_layers=1),
        "tiny-qwen3next": ModelConfig(arch="qwen3next", n_layers=4, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=2048,
                                      rms_eps=1e-6, rope_theta=1e7, n_rot=32, ctx_train=4096, n_experts=8, n_experts_used=2,
                                      expert_ffn=256, shared_expert_ffn=256, full_attn_interval=4, ssm_inner=512, ssm_state=128,
                                      ssm_n_k_heads=2, ssm_n_v_heads=4, ssm_conv_kernel=4, nextn_predict_layers=1),
        "tiny-qwen35": ModelConfig(arch="qwen35", n_layers=4, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=2048,
                                   rms_eps=1e-6, rope_theta=1e7, n_rot=32, ctx_train=4096, full_attn_interval=4, ssm_inner=512,
                                   ssm_state=128, ssm_n_k_heads=2, ssm_n_v_heads=4, ssm_conv_kernel=4, nextn_predict_layers=1),
        # "crown": Qwen3.6-35B-A3B (qwen36.cpp: 40 layers, full attention every 4th, 256 experts top-8 + shared expert, MTP block)
        "qwen3.6-35b-a3b": ModelConfig(arch="qwen35moe", n_layers=40, hidden=2048, n_heads=16, n_kv_heads=2, head_dim=256, ffn=5120,
                                       vocab=248320, rms_eps=1e-6, rope_theta=1e7, n_rot=64, ctx_train=262144, n_experts=256,
                                       n_experts_used=8, expert_ffn=512, shared_expert_ffn=512, full_attn_interval=4, ssm_inner=4096,
                                       ssm_state=128, ssm_n_k_heads=16, ssm_n_v_heads=32, ssm_conv_kernel=4, nextn_predict_layers=1),
        "tiny-qwen35moe": ModelConfig(arch="qwen35moe", n_layers=4, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=2048,
                                      rms_eps=1e-6, rope_theta=1e7, n_rot=32, ctx_train=4096, n_experts=8, n_experts_used=2,
                                      expert_ffn=256, shared_expert_ffn=256, full_attn_interval=4, ssm_inner=512, ssm_state=128,
                                      ssm_n_k_heads=2, ssm_n_v_heads=4, ssm_conv_kernel=4, nextn_predict_layers=1),
        "qwen3.6-27b": ModelConfig(arch="qwen35", n_layers=64, hidden=5120, n_heads=24, n_kv_heads=4, head_dim=256, ffn=17408, vocab=248320,
                                   rms_eps=1e-6, rope_theta=1e7, n_rot=64, ctx_train=262144, full_attn_interval=4, ssm_inner=6144,
                                   ssm_state=128, ssm_n_k_heads=16, ssm_n_v_heads=48, ssm_conv_kernel=4, nextn_predict_layers=1),
        # Gemma-4 shape in miniature: sliding layers with more, narrower KV heads and one global layer with wide heads; MoE dual path
        "tiny-gemma4": ModelConfig(arch="gemma4", n_layers=3, hidden=256, n_heads=4, n_kv_heads=2, head_dim=128, ffn=512, vocab=2048,
                                   rms_eps=1e-6, rope_theta=1e6, n_rot=128, ctx_train=4096, sliding_window=128, head_dim_swa=64, n_rot_swa=64,
                                   rope_theta_swa=10000.0, layer_swa=[True, True, False], layer_n_kv=[2, 2, 1], n_experts=8, n_experts_used=2,
                                   expert_ffn=128, final_logit_softcap=30.0, embedding_scale=16.0, attention_scale=1.0, tie_embeddings=True),
        "tiny-gemma4-dense": ModelConfig(arch="gemma4", n_layers=3, hidden=256, n_heads=4, n_kv_heads=2, head_dim=128, ffn=512, vocab=2048,
                                         rms_eps=1e-6, rope_theta=1e6, n_rot=128, ctx_train=4096, sliding_window=128, head_dim_swa=64,
                                         n_rot_swa=64, rope_theta_swa=10000.0, layer_swa=[True, True, False], layer_n_kv=[2, 2, 1],
                                         final_logit_softcap=30.0, embedding_scale=16.0, attention_scale=1.0, tie_embeddings=True),
        "tiny-qwen2": ModelConfig(arch="qwen2", n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=2048,
                                  rms_eps=1e-6, rope_theta=1e6, n_rot=64, ctx_train=4096),
        "tiny-phi3": ModelConfig(arch="phi3", n_layers=2, hidden=256, n_heads=4, n_kv_heads=4, head_dim=64, ffn=512, vocab=2048,
                                 rms_eps=1e-5, rope_theta=10000.0, n_rot=64, ctx_train=4096),
        "tiny-granite": ModelConfig(arch="granite", n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=2048,
                                    rms_eps=1e-5, rope_theta=10000.0, n_rot=64, ctx_train=4096, embedding_scale=12.0, residual_scale=0.22,
                                    attention_scale=0.0078125, logit_scale=0.125),
        "tiny-qwen3": ModelConfig(arch="qwen3", n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=2048,
                                  rms_eps=1e-6, rope_theta=1e6, n_rot=64, ctx_train=4096),
    }
    if name not in p:
        raise KeyError(f"unknown preset {name}; have {sorted(p)}")
    c = p[name]
    c.name = name
    return c
