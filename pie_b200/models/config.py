"""Model configuration parsed from a Hugging Face ``config.json``.

Keys consumed mirror the reference's HF config reader
(driver/cuda/src/loader/hf_config.hpp:145-215).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field, asdict
from pathlib import Path
from typing import Optional

LLAMA_LIKE = {"llama", "qwen2", "qwen3", "mistral", "phi3"}   # pre-norm decoder blocks with SwiGLU and rotate-half RoPE
# `model_type` strings of checkpoints this build loads (the architecture registry of the loader)
SUPPORTED_MODEL_TYPES = ("llama", "mistral", "qwen2", "qwen3", "phi3", "qwen3_moe", "mixtral", "olmo2", "olmo3", "gpt_oss",
                         "qwen3_5", "qwen3_next", "mamba2_hybrid", "gemma2", "gemma3_text", "gemma3", "qwen2_moe", "qwen2_vl",
                         "qwen2_audio")
MAMBA_TYPES = {"mamba2_hybrid"}         # Mamba-2 (state-space) mixers in llama-like blocks, between full-attention layers
GDN_TYPES = {"qwen3_5", "qwen3_next"}   # hybrids: Gated DeltaNet (linear attention) layers between full-attention layers
POST_NORM = {"olmo2", "olmo3"}       # same block with the norms after attention / MLP and q, k norms over all heads
MOE_TYPES = {"qwen3_moe", "mixtral", "gpt_oss", "qwen2_moe"}
# Gemma-2 / Gemma-3: norms before AND after attention and MLP, gains stored as (w - 1), GeGLU, scaled embeddings,
# alternating local / global layers (Gemma-3: a RoPE base of their own for the local ones; Gemma-2: soft-capped logits)
GEMMA_TYPES = {"gemma2", "gemma3_text", "gemma3"}


@dataclass
class ModelConfig:
    model_type: str = "llama"
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    vocab_size: int = 128256
    max_position_embeddings: int = 131072
    rms_norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    rope_scaling: Optional[dict] = None
    tie_word_embeddings: bool = False
    qk_norm: bool = False           # Qwen3: per-head RMSNorm on q and k
    attention_bias: bool = False    # Qwen2: bias on q/k/v projections
    sliding_window: int = -1
    post_norm: bool = False         # OLMo-2: h += norm(attn(h)); h += norm(mlp(h)); q/k RMSNorm over the whole projection
    layer_types: Optional[list] = None   # per layer "sliding_attention" | "full_attention" (GPT-OSS); None: all alike
    attention_sinks: bool = False   # GPT-OSS: a learned per-head logit in every softmax denominator
    o_bias: bool = False            # bias on the attention output projection
    sandwich_norm: bool = False     # Gemma-2/3: h += norm(attn(norm(h))); h += norm(mlp(norm(h)))
    norm_plus_one: bool = False     # checkpoints store RMSNorm gains as (w - 1); the loader adds the 1
    hidden_act: str = "silu"        # gate activation of the GLU: "silu" | "gelu_tanh"
    embed_scale: float = 1.0        # embeddings are multiplied by this (Gemma: sqrt(hidden_size))
    query_pre_attn_scalar: float = 0.0   # attention scale is this ** -0.5 (0: head_dim)
    attn_softcap: float = 0.0       # scores pass through cap * tanh(s / cap) before the softmax (0: off)
    final_softcap: float = 0.0      # same for the output logits
    rope_local_theta: float = 0.0   # RoPE base of the sliding-window layers, unscaled (0: same table as the others)
    # mixture of experts
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    # a dense expert that every token also passes through, scaled by sigmoid(x . shared_gate) (Qwen2-MoE, Qwen3-Next); 0: none
    shared_expert_intermediate_size: int = 0
    moe_style: str = "swiglu"       # "gpt_oss": expert and router biases, clamped (up + 1) * gate * sigmoid(1.702 gate)
    swiglu_limit: float = 7.0
    # Gated DeltaNet layers (layer_types entry "linear_attention"): heads and head sizes of the linear mixer
    linear_num_key_heads: int = 0
    linear_num_value_heads: int = 0
    linear_key_head_dim: int = 0
    linear_value_head_dim: int = 0
    linear_conv_kernel_dim: int = 4
    # Mamba-2 layers (layer_types entry "mamba2"): heads, head size, state size, B / C groups
    mamba_num_heads: int = 0
    mamba_head_dim: int = 0
    ssm_state_size: int = 0
    mamba_n_groups: int = 1
    mamba_norm_grouped: bool = False   # gated RMSNorm per B / C group (Nemotron-H) instead of over the whole inner width (Mamba-2)
    # quantisation of the linear weights: None | "fp8_block" (128x128 weight scales)
    quantization: Optional[str] = None
    dtype: str = "bfloat16"
    name: str = ""

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    def is_linear_layer(self, li: int) -> bool:
        return self.layer_types is not None and self.layer_types[li] == "linear_attention"

    @property
    def linear_layers(self) -> list:
        """Indices of the Gated DeltaNet layers (empty for pure-attention models)."""
        return [li for li in range(self.num_hidden_layers) if self.is_linear_layer(li)]

    def is_mamba_layer(self, li: int) -> bool:
        return self.layer_types is not None and self.layer_types[li] == "mamba2"

    @property
    def mamba_layers(self) -> list:
        return [li for li in range(self.num_hidden_layers) if self.is_mamba_layer(li)]

    @property
    def recurrent_layers(self) -> list:
        """Layers whose state lives in the recurrent-state cache (Gated DeltaNet or Mamba-2)."""
        return [li for li in range(self.num_hidden_layers) if self.is_linear_layer(li) or self.is_mamba_layer(li)]

    @property
    def mamba_inner(self) -> int:
        return self.mamba_num_heads * self.mamba_head_dim

    @property
    def mamba_conv_channels(self) -> int:
        """Channels of the short convolution: x, then B and C of every group."""
        return self.mamba_inner + 2 * self.mamba_n_groups * self.ssm_state_size

    @property
    def mamba_in_features(self) -> int:
        """Rows of the input projection: z (gate) | x B C | dt."""
        return self.mamba_inner + self.mamba_conv_channels + self.mamba_num_heads

    @property
    def gdn_conv_channels(self) -> int:
        """Channels of the short convolution: q and k of the key heads, v of the value heads."""
        return 2 * self.linear_num_key_heads * self.linear_key_head_dim + self.linear_num_value_heads * self.linear_value_head_dim

    @property
    def gdn_in_features(self) -> int:
        """Rows of the fused input projection: q | k | v | z (output gate) | b (beta) | a (decay)."""
        return self.gdn_conv_channels + self.linear_num_value_heads * self.linear_value_head_dim + 2 * self.linear_num_value_heads

    def layer_window_left(self, li: int) -> int:
        """Keys left of the query that layer `li` sees (-1: all). HF `sliding_window` counts the query itself."""
        if not self.sliding_window or self.sliding_window <= 0:
            return -1
        if self.layer_types is not None and self.layer_types[li] != "sliding_attention":
            return -1
        return self.sliding_window - 1

    @property
    def plan_window_left(self) -> int:
        """The window attention plans may be cut to: the widest any layer needs."""
        ws = [self.layer_window_left(li) for li in range(self.num_hidden_layers)]
        return -1 if any(w < 0 for w in ws) or not ws else max(ws)

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def to_dict(self) -> dict:
        return asdict(self)

    @staticmethod
    def from_hf(cfg: dict, name: str = "") -> "ModelConfig":
        mt = cfg.get("model_type", "llama")
        if mt == "gemma3" and "text_config" in cfg:       # multimodal wrapper: the language model's own section
            cfg = dict(cfg["text_config"], model_type="gemma3_text")
            mt = "gemma3_text"
        if mt == "qwen2_audio" and "text_config" in cfg:       # the language model of Qwen2-Audio is a plain Qwen2
            tc = dict(cfg["text_config"])
            tc.setdefault("tie_word_embeddings", cfg.get("tie_word_embeddings", False))
            cfg, mt = dict(tc, model_type="qwen2"), "qwen2"
        if mt in ("qwen2_vl", "qwen2_vl_text"):
            # the language model of Qwen2-VL is the Qwen2 block; its three-axis rotary positions are not built: tokens
            # take one-dimensional positions (the same thing for text; image rows then differ from the checkpoint's own code)
            tc = dict(cfg.get("text_config") or cfg)
            tc.setdefault("tie_word_embeddings", cfg.get("tie_word_embeddings", False))
            cfg, mt = dict(tc, model_type="qwen2"), "qwen2"
        cfg = _flatten_rope_parameters(dict(cfg))
        gemma = mt in GEMMA_TYPES
        if gemma:
            cfg.setdefault("head_dim", 256)
            cfg.setdefault("tie_word_embeddings", True)
            cfg.setdefault("rms_norm_eps", 1e-6)
            if cfg.get("layer_types") is None:
                # Gemma-2 alternates local / global; Gemma-3 runs `sliding_window_pattern - 1` local layers per global one
                pat = int(cfg.get("sliding_window_pattern") or cfg.get("_sliding_window_pattern") or (2 if mt == "gemma2" else 6))
                cfg["layer_types"] = ["full_attention" if (i + 1) % pat == 0 else "sliding_attention"
                                      for i in range(cfg["num_hidden_layers"])]
        heads = cfg["num_attention_heads"]
        hd = cfg.get("head_dim") or cfg["hidden_size"] // heads
        q = cfg.get("quantization_config") or {}
        quant = None
        if q.get("quant_method") == "fp8" and q.get("weight_block_size"):
            quant = "fp8_block"
        elif _is_fp8_weight_config(q):
            # per-tensor / per-channel fp8 checkpoints (`weight_scale` next to each weight): the loader spreads the scale
            # over the row blocks of the same runtime format; activations are quantised per call, a stored input scale is unused
            quant = "fp8_block"
        return ModelConfig(
            model_type=mt,
            hidden_size=cfg["hidden_size"],
            intermediate_size=cfg.get("intermediate_size", 0),
            num_hidden_layers=cfg["num_hidden_layers"],
            num_attention_heads=heads,
            num_key_value_heads=cfg.get("num_key_value_heads", heads),
            head_dim=hd,
            vocab_size=cfg["vocab_size"],
            max_position_embeddings=cfg.get("max_position_embeddings", 8192),
            rms_norm_eps=cfg.get("rms_norm_eps", 1e-5),
            rope_theta=cfg.get("rope_theta", 10000.0),
            rope_scaling=cfg.get("rope_scaling"),
            tie_word_embeddings=cfg.get("tie_word_embeddings", False),
            qk_norm=mt in ("qwen3", "qwen3_moe", "olmo2", "olmo3", "gemma3_text") or mt in GDN_TYPES or cfg.get("use_qk_norm", False),
            sandwich_norm=gemma, norm_plus_one=gemma,
            hidden_act="gelu_tanh" if gemma or "gelu" in str(cfg.get("hidden_act", "")) else "silu",
            embed_scale=float(cfg["hidden_size"]) ** 0.5 if gemma else 1.0,
            query_pre_attn_scalar=float(cfg.get("query_pre_attn_scalar") or 0.0) if gemma else 0.0,
            attn_softcap=float(cfg.get("attn_logit_softcapping") or 0.0), final_softcap=float(cfg.get("final_logit_softcapping") or 0.0),
            rope_local_theta=float(cfg.get("rope_local_base_freq") or 0.0) if mt == "gemma3_text" else 0.0,
            post_norm=mt in POST_NORM,
            attention_bias=cfg.get("attention_bias", mt in ("qwen2", "gpt_oss", "qwen2_moe")),
            # Qwen2 gates the window on use_sliding_window; Mistral applies it whenever it is set
            sliding_window=(cfg.get("sliding_window") or -1)
            if cfg.get("use_sliding_window", mt in ("mistral", "gpt_oss", "olmo3") or gemma) else -1,
            # OLMo-3 and GPT-OSS alternate sliding-window and full-attention layers
            layer_types=cfg.get("layer_types") if mt in ("gpt_oss", "olmo3") or gemma or mt in GDN_TYPES or mt in MAMBA_TYPES else None,
            mamba_num_heads=cfg.get("mamba_num_heads", 0), mamba_head_dim=cfg.get("mamba_head_dim", 0),
            ssm_state_size=cfg.get("ssm_state_size", 0), mamba_n_groups=cfg.get("mamba_n_groups", 1),
            mamba_norm_grouped=bool(cfg.get("mamba_norm_grouped", False)),
            linear_num_key_heads=cfg.get("linear_num_key_heads", 0), linear_num_value_heads=cfg.get("linear_num_value_heads", 0),
            linear_key_head_dim=cfg.get("linear_key_head_dim", 0), linear_value_head_dim=cfg.get("linear_value_head_dim", 0),
            linear_conv_kernel_dim=cfg.get("linear_conv_kernel_dim", 4),
            attention_sinks=mt == "gpt_oss",
            o_bias=mt == "gpt_oss" and cfg.get("attention_bias", True),
            moe_style="gpt_oss" if mt == "gpt_oss" else "swiglu",
            swiglu_limit=float(cfg.get("swiglu_limit", 7.0)),
            num_experts=cfg.get("num_experts", cfg.get("num_local_experts", 0)) or 0,
            num_experts_per_tok=cfg.get("num_experts_per_tok", 0) or 0,
            # Mixtral has no separate field: its intermediate_size is the expert FFN width
            moe_intermediate_size=cfg.get("moe_intermediate_size", 0)
            or (cfg.get("intermediate_size", 0) if mt in ("mixtral", "gpt_oss") else 0),
            norm_topk_prob=cfg.get("norm_topk_prob", mt != "qwen2_moe"),
            shared_expert_intermediate_size=cfg.get("shared_expert_intermediate_size", 0) or 0,
            quantization=quant,
            dtype=str(cfg.get("torch_dtype") or cfg.get("dtype") or "bfloat16"),      # newer files say `dtype`
            name=name,
        )

    @staticmethod
    def from_path(path) -> "ModelConfig":
        p = Path(path)
        with open(p / "config.json") as f:
            return ModelConfig.from_hf(json.load(f), name=p.name)


def _is_fp8_weight_config(q: dict) -> bool:
    """`quantization_config` of an 8-bit float weight checkpoint without block scales: `fp8` / `fbgemm_fp8`, or
    compressed-tensors groups whose weights are 8-bit floats with a tensor or channel strategy."""
    method = q.get("quant_method")
    if method in ("fp8", "fbgemm_fp8"):
        return True
    if method == "compressed-tensors":
        groups = (q.get("config_groups") or {}).values()
        ws = [g.get("weights") or {} for g in groups]
        return bool(ws) and all(w.get("type") == "float" and w.get("num_bits") == 8 and w.get("strategy") in ("tensor", "channel")
                                for w in ws)
    return False


def _flatten_rope_parameters(cfg: dict) -> dict:
    """Newer `config.json` files carry RoPE settings as `rope_parameters`: one dict (`rope_theta`, `rope_type`,
    scaling fields), or one such dict per layer type. Rewrites them as the older `rope_theta` / `rope_scaling` /
    `rope_local_base_freq` keys, which win when both are present."""
    rp = cfg.get("rope_parameters")
    if not isinstance(rp, dict):
        return cfg
    local = None
    if "full_attention" in rp or "sliding_attention" in rp:
        local = rp.get("sliding_attention")
        rp = rp.get("full_attention") or local or {}
    if "rope_theta" in rp:
        cfg.setdefault("rope_theta", rp["rope_theta"])
    if rp.get("rope_type", "default") != "default" and not cfg.get("rope_scaling"):
        cfg["rope_scaling"] = {k: v for k, v in rp.items() if k != "rope_theta"}
    if local and "rope_theta" in local:
        cfg.setdefault("rope_local_base_freq", local["rope_theta"])
    return cfg


# Architectures named by the benchmark configurations (random-init weights of these shapes).
PRESETS = {
    "tiny-llama": dict(model_type="llama", hidden_size=256, intermediate_size=688, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=64, vocab_size=32000,
                       rope_theta=10000.0, rms_norm_eps=1e-5, dtype="float32"),
    "llama-3.1-8b": dict(model_type="llama", hidden_size=4096, intermediate_size=14336,
                         num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8,
                         head_dim=128, vocab_size=128256, rope_theta=500000.0, rms_norm_eps=1e-5),
    "qwen3-32b": dict(model_type="qwen3", hidden_size=5120, intermediate_size=25600,
                      num_hidden_layers=64, num_attention_heads=64, num_key_value_heads=8, head_dim=128,
                      vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, qk_norm=True),
    "qwen3-32b-fp8": dict(model_type="qwen3", hidden_size=5120, intermediate_size=25600,
                          num_hidden_layers=64, num_attention_heads=64, num_key_value_heads=8,
                          head_dim=128, vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6,
                          qk_norm=True, quantization="fp8_block"),
    "qwen3-30b-a3b": dict(model_type="qwen3_moe", hidden_size=2048, intermediate_size=6144,
                          num_hidden_layers=48, num_attention_heads=32, num_key_value_heads=4,
                          head_dim=128, vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6,
                          qk_norm=True, num_experts=128, num_experts_per_tok=8,
                          moe_intermediate_size=768, norm_topk_prob=True),
    "qwen3-0.6b": dict(model_type="qwen3", hidden_size=1024, intermediate_size=3072,
                       num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8, head_dim=128,
                       vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, qk_norm=True,
                       tie_word_embeddings=True),
    "olmo-2-7b": dict(model_type="olmo2", hidden_size=4096, intermediate_size=11008, num_hidden_layers=32,
                      num_attention_heads=32, num_key_value_heads=32, head_dim=128, vocab_size=100352,
                      rope_theta=500000.0, rms_norm_eps=1e-6, qk_norm=True, post_norm=True),
    "tiny-olmo2": dict(model_type="olmo2", hidden_size=256, intermediate_size=688, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=64, vocab_size=32000,
                       rope_theta=10000.0, rms_norm_eps=1e-6, qk_norm=True, post_norm=True, dtype="float32"),
    "gpt-oss-20b": dict(model_type="gpt_oss", hidden_size=2880, intermediate_size=2880, num_hidden_layers=24,
                        num_attention_heads=64, num_key_value_heads=8, head_dim=64, vocab_size=201088,
                        rope_theta=150000.0, rms_norm_eps=1e-5, attention_bias=True, o_bias=True, attention_sinks=True,
                        sliding_window=128, layer_types=["sliding_attention", "full_attention"] * 12,
                        num_experts=32, num_experts_per_tok=4, moe_intermediate_size=2880, moe_style="gpt_oss",
                        rope_scaling=dict(rope_type="yarn", factor=32.0, beta_fast=32.0, beta_slow=1.0,
                                          original_max_position_embeddings=4096, truncate=False)),
    "tiny-gpt-oss": dict(model_type="gpt_oss", hidden_size=256, intermediate_size=128, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=64, vocab_size=32000,
                         rope_theta=10000.0, rms_norm_eps=1e-5, attention_bias=True, o_bias=True,
                         attention_sinks=True, sliding_window=20, layer_types=["sliding_attention", "full_attention"],
                         num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128, moe_style="gpt_oss",
                         rope_scaling=dict(rope_type="yarn", factor=4.0, beta_fast=32.0, beta_slow=1.0,
                                           original_max_position_embeddings=64, truncate=False), dtype="float32"),
    "tiny-qwen3.5": dict(model_type="qwen3_5", hidden_size=256, intermediate_size=512, num_hidden_layers=4,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=64, vocab_size=32000, qk_norm=True,
                         rope_theta=1e6, layer_types=["linear_attention", "linear_attention", "linear_attention", "full_attention"],
                         linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=32, linear_value_head_dim=32),
    "tiny-mamba2": dict(model_type="mamba2_hybrid", hidden_size=256, intermediate_size=512, num_hidden_layers=3,
                        num_attention_heads=4, num_key_value_heads=2, head_dim=64, vocab_size=32000,
                        layer_types=["mamba2", "mamba2", "full_attention"], mamba_num_heads=8, mamba_head_dim=32,
                        ssm_state_size=16, mamba_n_groups=2),
    "gemma-3-27b": dict(model_type="gemma3_text", hidden_size=5376, intermediate_size=21504, num_hidden_layers=62,
                        num_attention_heads=32, num_key_value_heads=16, head_dim=128, vocab_size=262208,
                        rope_theta=1e6, rope_scaling=dict(rope_type="linear", factor=8.0), rope_local_theta=10000.0,
                        rms_norm_eps=1e-6, qk_norm=True, sandwich_norm=True, norm_plus_one=True, hidden_act="gelu_tanh",
                        embed_scale=5376 ** 0.5, query_pre_attn_scalar=168.0, sliding_window=1024, tie_word_embeddings=True,
                        layer_types=(["sliding_attention"] * 5 + ["full_attention"]) * 10 + ["sliding_attention"] * 2),
    "tiny-gemma3": dict(model_type="gemma3_text", hidden_size=256, intermediate_size=512, num_hidden_layers=3,
                        num_attention_heads=4, num_key_value_heads=2, head_dim=64, vocab_size=32000, rope_theta=1e6,
                        rope_scaling=dict(rope_type="linear", factor=8.0), rope_local_theta=10000.0, rms_norm_eps=1e-6,
                        qk_norm=True, sandwich_norm=True, norm_plus_one=True, hidden_act="gelu_tanh", embed_scale=16.0,
                        query_pre_attn_scalar=48.0, sliding_window=8, tie_word_embeddings=True,
                        layer_types=["sliding_attention", "sliding_attention", "full_attention"], dtype="float32"),
    "tiny-gemma2": dict(model_type="gemma2", hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                        num_attention_heads=4, num_key_value_heads=2, head_dim=64, vocab_size=32000, rope_theta=10000.0,
                        rms_norm_eps=1e-6, sandwich_norm=True, norm_plus_one=True, hidden_act="gelu_tanh", embed_scale=16.0,
                        query_pre_attn_scalar=48.0, sliding_window=8, tie_word_embeddings=True, attn_softcap=50.0,
                        final_softcap=30.0, layer_types=["sliding_attention", "full_attention"], dtype="float32"),
    "tiny-qwen2-moe": dict(model_type="qwen2_moe", hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                           num_attention_heads=4, num_key_value_heads=2, head_dim=64, vocab_size=32000, rope_theta=10000.0,
                           rms_norm_eps=1e-6, attention_bias=True, num_experts=8, num_experts_per_tok=2,
                           moe_intermediate_size=128, norm_topk_prob=False, shared_expert_intermediate_size=192, dtype="float32"),
    "tiny-qwen3-moe": dict(model_type="qwen3_moe", hidden_size=256, intermediate_size=512,
                           num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                           vocab_size=32000, rope_theta=10000.0, rms_norm_eps=1e-6, qk_norm=True,
                           num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128,
                           dtype="float32"),
}


def preset(name: str, **overrides) -> ModelConfig:
    if name not in PRESETS:
        raise KeyError(f"unknown model preset {name!r}; known: {sorted(PRESETS)}")
    kw = dict(PRESETS[name])
    kw.update(overrides)
    return ModelConfig(name=name, **kw)
