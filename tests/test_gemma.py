"""Gemma-2 / Gemma-3 family: norms on both sides of each sub-block with gains stored as (w - 1), GeGLU, scaled
embeddings, a scale from `query_pre_attn_scalar`, local layers with a RoPE base of their own (Gemma-3), soft-capped
scores and logits (Gemma-2). CPU driver against the dense oracle and through the engine; configuration readers for
both `config.json` generations; checkpoints under a multimodal wrapper's prefix. transformers parity is in
test_hf_parity.py, the CUDA kernels in test_kernels_gpu.py / test_driver_gpu.py."""
import json

import pytest
import torch

from pie_b200.driver.executor import TorchDriver
from pie_b200.inferlets import install_all
from pie_b200.models import loader
from pie_b200.models.config import ModelConfig, preset
from pie_b200.models.transformer import dense_reference_forward
from pie_b200.models.weights import random_weights
from pie_b200.ops import reference as ref
from pie_b200.runtime.engine import Engine, EngineConfig
from pie_b200.runtime.tokenizer import ByteTokenizer


def oracle_greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(dense_reference_forward(cfg, w, torch.tensor(toks))[-1].argmax()))
    return toks[len(prompt):]


@pytest.mark.parametrize("name", ["tiny-gemma3", "tiny-gemma2"])
def test_engine_generates_the_oracle_tokens(name):
    cfg = preset(name)
    w = random_weights(cfg, "cpu", torch.float32, seed=4)
    drv = TorchDriver(cfg, "cpu", weights=w, num_pages=64, page_size=16, max_requests=8, max_tokens=64)
    assert drv.capabilities().cohort_decode
    e = Engine(EngineConfig())
    try:
        e.add_model("gemma", drv, tokenizer=ByteTokenizer(cfg.vocab_size))
        install_all(e)
        prompt = list(range(100, 190))          # 90 tokens: two prefill chunks, and far past the 8-token window
        out = json.loads(e.run("text-completion", {"prompt_tokens": prompt, "max_tokens": 6, "temperature": 0.0,
                                                   "stop_tokens": []}, 300))
        assert out["tokens"] == oracle_greedy(cfg, w, prompt, 6)
        assert e.models["gemma"].inference.cohorts
    finally:
        e.shutdown()


def test_local_layers_use_their_own_rope_base_and_window():
    cfg = preset("tiny-gemma3")
    w = random_weights(cfg, "cpu", torch.float32, seed=1)
    toks = torch.arange(300, 330)
    base = dense_reference_forward(cfg, w, toks)
    same_base = dense_reference_forward(preset("tiny-gemma3", rope_local_theta=0.0), w, toks)
    no_window = dense_reference_forward(preset("tiny-gemma3", sliding_window=1000), w, toks)
    assert (base - same_base).abs().max() > 1e-3 and (base - no_window).abs().max() > 1e-3
    # inside the window the local layers see everything: the first 8 positions do not depend on it
    assert (base[:8] - no_window[:8]).abs().max() < 1e-5


def test_config_readers_of_both_config_generations():
    old = dict(model_type="gemma3_text", hidden_size=256, intermediate_size=512, num_hidden_layers=8, num_attention_heads=4,
               num_key_value_heads=2, head_dim=64, vocab_size=32000, rope_theta=1e6, rope_local_base_freq=1e4,
               rope_scaling=dict(rope_type="linear", factor=8.0), sliding_window=512, sliding_window_pattern=4,
               query_pre_attn_scalar=64)
    c = ModelConfig.from_hf(old)
    assert c.layer_types == ["sliding_attention"] * 3 + ["full_attention"] + ["sliding_attention"] * 3 + ["full_attention"]
    assert (c.rope_theta, c.rope_local_theta, c.rope_scaling["factor"]) == (1e6, 1e4, 8.0)
    assert c.sandwich_norm and c.norm_plus_one and c.qk_norm and c.hidden_act == "gelu_tanh" and c.tie_word_embeddings
    assert c.embed_scale == 16.0 and c.sliding_window == 512 and c.layer_window_left(0) == 511 and c.layer_window_left(3) == -1
    new = dict(old)
    for k in ("rope_theta", "rope_local_base_freq", "rope_scaling", "sliding_window_pattern"):
        del new[k]
    new["rope_parameters"] = {"sliding_attention": {"rope_type": "default", "rope_theta": 1e4},
                              "full_attention": {"rope_type": "linear", "factor": 8.0, "rope_theta": 1e6}}
    new["layer_types"] = c.layer_types
    assert ModelConfig.from_hf(new).to_dict() == c.to_dict()
    # the multimodal wrapper's configuration nests the language model's
    assert ModelConfig.from_hf({"model_type": "gemma3", "text_config": {k: v for k, v in old.items() if k != "model_type"}}).to_dict() == c.to_dict()
    # one-level `rope_parameters` of the other families
    ll = ModelConfig.from_hf(dict(model_type="llama", hidden_size=256, num_hidden_layers=2, num_attention_heads=4, vocab_size=100,
                                  rope_parameters={"rope_type": "llama3", "rope_theta": 5e5, "factor": 8.0, "low_freq_factor": 1.0,
                                                   "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}))
    assert ll.rope_theta == 5e5 and ll.rope_scaling["rope_type"] == "llama3" and "rope_theta" not in ll.rope_scaling
    g2 = ModelConfig.from_hf(dict(model_type="gemma2", hidden_size=256, intermediate_size=512, num_hidden_layers=4, num_attention_heads=4,
                                  num_key_value_heads=2, head_dim=64, vocab_size=32000, sliding_window=16, query_pre_attn_scalar=32,
                                  attn_logit_softcapping=50.0, final_logit_softcapping=30.0))
    assert g2.layer_types == ["sliding_attention", "full_attention"] * 2 and (g2.attn_softcap, g2.final_softcap) == (50.0, 30.0)
    assert not g2.qk_norm and g2.rope_local_theta == 0.0


def test_checkpoint_under_a_wrapper_prefix_and_gain_offset(tmp_path):
    from safetensors.torch import load_file, save_file
    cfg = preset("tiny-gemma3")
    w = random_weights(cfg, "cpu", torch.float32, seed=6)
    loader.export_hf_checkpoint(cfg, w, tmp_path)
    t = load_file(str(tmp_path / "model.safetensors"))
    # the file holds (gain - 1), as the family's checkpoints do
    assert torch.allclose(t["model.layers.0.pre_feedforward_layernorm.weight"] + 1, w["layers"][0]["ln2"])
    assert torch.allclose(t["model.layers.1.self_attn.q_norm.weight"] + 1, w["layers"][1]["q_norm"])
    # same tensors under the multimodal wrapper's names, next to tensors of the vision tower that the loader ignores
    wrapped = {k.replace("model.", "model.language_model.", 1): v for k, v in t.items()}
    wrapped["model.vision_tower.patch_embedding.weight"] = torch.zeros(4, 4)
    save_file(wrapped, str(tmp_path / "model.safetensors"))
    cfg2, w2 = loader.load_checkpoint(tmp_path, "cpu", dtype="float32")
    toks = torch.arange(100, 120)
    assert (dense_reference_forward(cfg2, w2, toks) - dense_reference_forward(cfg, w, toks)).abs().max() < 1e-5
    for key in ("ln1", "ln_pa", "ln2", "ln_pf", "q_norm", "k_norm", "wqkv", "w_gate_up"):
        assert torch.allclose(w2["layers"][2][key], w["layers"][2][key], atol=1e-6), key


def test_glu_and_softcap_reference_ops():
    torch.manual_seed(0)
    y = torch.randn(5, 32)
    g, u = y[:, 0::2], y[:, 1::2]
    assert torch.allclose(ref.glu_interleaved(y, "gelu_tanh"), torch.nn.functional.gelu(g, approximate="tanh") * u)
    assert torch.allclose(ref.glu_interleaved(y, "silu"), ref.swiglu_interleaved(y))
    # soft-capped paged attention against a direct statement
    q = torch.randn(3, 4, 16) * 4
    kv = torch.randn(2, 2, 2, 16, 16) * 4               # [pages, k/v, hkv, page, d]
    import numpy as np
    out = ref.paged_attention(q, kv, np.array([0, 3]), np.array([0, 2]), torch.tensor([1, 0]), np.array([20]), 0.25, softcap=5.0)
    k = torch.cat([kv[1, 0], kv[0, 0]], 1)[:, :20].repeat_interleave(2, 0)
    v = torch.cat([kv[1, 1], kv[0, 1]], 1)[:, :20].repeat_interleave(2, 0)
    s = torch.einsum("qhd,hkd->hqk", q, k) * 0.25
    s = torch.tanh(s / 5.0) * 5.0
    allow = torch.arange(20)[None, :] < (17 + torch.arange(3)[:, None] + 1)
    want = torch.einsum("hqk,hkd->qhd", torch.softmax(s.masked_fill(~allow[None], float("-inf")), -1), v)
    assert torch.allclose(out, want, atol=1e-5)
