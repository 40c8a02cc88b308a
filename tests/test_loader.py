"""Weight loader: tiny synthetic checkpoints (HF names, safetensors) -> storage program -> runtime
layout; byte-exact against the weights they were exported from, tensor-parallel shards
reassemble to the unsharded tensors, programs survive serialisation. Same idea as the reference's
load-parity suite (driver/cuda/tests/load_parity/README.md: synthetic checkpoints, TP reassembly)."""
import tempfile

import pytest
import torch

from pie_b200.models import loader
from pie_b200.models.config import preset
from pie_b200.models.weights import random_weights


def _same(a, b):
    if isinstance(a, torch.Tensor):
        return torch.equal(a, b)
    if isinstance(a, dict):
        return all(_same(a[k], b[k]) for k in a if k != "lm_head_vocab_start")
    if isinstance(a, list):
        return all(_same(x, y) for x, y in zip(a, b))
    return a == b


@pytest.mark.parametrize("name,over", [("tiny-llama", {}), ("tiny-llama", {"qk_norm": True, "attention_bias": True,
                                                                            "model_type": "qwen2"}),
                                       ("tiny-qwen3-moe", {})])
def test_roundtrip_and_tp_shards(name, over):
    cfg = preset(name, vocab_size=512, **over)
    full = random_weights(cfg, "cpu", torch.float32, seed=3)
    d = tempfile.mkdtemp()
    loader.export_hf_checkpoint(cfg, full, d)
    cfg2, w = loader.load_checkpoint(d, dtype="float32")
    assert cfg2.hidden_size == cfg.hidden_size and cfg2.num_experts == cfg.num_experts
    assert _same(full, w)
    for rank in range(2):
        want = random_weights(cfg, "cpu", torch.float32, seed=3, tp_size=2, tp_rank=rank)
        _, got = loader.load_checkpoint(d, tp_size=2, tp_rank=rank, dtype="float32")
        assert _same(want, got)
        assert got["lm_head_vocab_start"] == rank * 256


def test_expert_parallel_split_and_program_serialisation():
    cfg = preset("tiny-qwen3-moe", vocab_size=512)
    full = random_weights(cfg, "cpu", torch.float32, seed=4)
    d = tempfile.mkdtemp()
    loader.export_hf_checkpoint(cfg, full, d)
    reader = loader.SafetensorsReader(d)
    prog = loader.compile_program(cfg, reader.names(), tp_size=4, tp_rank=1, ep=True, dtype="float32")
    prog2 = loader.program_from_json(loader.program_to_json(prog))
    w = loader.execute_program(prog2, reader)
    want = random_weights(cfg, "cpu", torch.float32, seed=4, tp_size=4, tp_rank=1, ep=True)
    assert _same(want, w)
    assert w["layers"][0]["experts_gate_up"].shape[0] == cfg.num_experts // 4      # whole experts per rank


def test_missing_tensor_is_reported():
    cfg = preset("tiny-llama", vocab_size=512)
    with pytest.raises(KeyError):
        loader.compile_program(cfg, ["model.embed_tokens.weight"])


def test_fp8_block_checkpoint_loads_and_matches_dequantised_oracle(tmp_path):
    """Block-scaled fp8 checkpoint (weight + weight_scale_inv per 128x128 block, ragged last
    block): the loader keeps the weights in fp8 with per-row scales, also through the fused
    QKV join and the gate/up interleave; the engine's tokens equal the dense forward over the
    dequantised weights."""
    import json as _json
    import numpy as np
    from safetensors.torch import save_file
    from pie_b200 import ops
    from pie_b200.driver.executor import TorchDriver
    from pie_b200.models import loader
    from pie_b200.models.config import preset
    from pie_b200.models.transformer import dense_reference_forward
    from pie_b200.models.weights import dequantized, random_weights
    from pie_b200.runtime.scheduler import PendingRequest, fold
    from pie_b200.driver.schema import SamplerKind, SamplerSpec

    cfg = preset("tiny-llama")
    w = random_weights(cfg, "cpu", torch.float32, seed=3)
    loader.export_hf_checkpoint(cfg, w, tmp_path)
    from safetensors import safe_open
    tensors = {}
    with safe_open(str(tmp_path / "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            tensors[k] = f.get_tensor(k)
    out = {}
    for k, t in tensors.items():
        if k.endswith("_proj.weight"):
            n, kk = t.shape
            nb, kb = -(-n // 128), -(-kk // 128)
            pad = torch.zeros(nb * 128, kb * 128)
            pad[:n, :kk] = t.float()
            blocks = pad.view(nb, 128, kb, 128)
            sc = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-12) / 448.0
            out[k] = (blocks / sc[:, None, :, None]).reshape(nb * 128, kb * 128)[:n, :kk].to(torch.float8_e4m3fn)
            out[k + "_scale_inv"] = sc.contiguous()
        else:
            out[k] = t
    save_file(out, str(tmp_path / "model.safetensors"))
    hf = _json.loads((tmp_path / "config.json").read_text())
    hf["quantization_config"] = {"quant_method": "fp8", "weight_block_size": [128, 128]}
    (tmp_path / "config.json").write_text(_json.dumps(hf))

    cfg2, w2 = loader.load_checkpoint(tmp_path, "cpu", dtype="float32")
    assert cfg2.quantization == "fp8_block"
    lw = w2["layers"][0]
    assert isinstance(lw["wqkv"], ops.Fp8Linear) and isinstance(lw["w_gate_up"], ops.Fp8Linear)
    assert lw["w_gate_up"].scale.shape == (2 * cfg.intermediate_size, cfg.hidden_size // 128)
    # dequantised values are within fp8 rounding of the originals
    err = (lw["wo"].dequant(torch.float32) - w["layers"][0]["wo"]).abs().max() / w["layers"][0]["wo"].abs().max()
    assert err < 0.07
    drv = TorchDriver(cfg2, "cpu", weights=w2, num_pages=16, page_size=16, max_requests=4, max_tokens=128)
    toks = list(range(40, 70))
    raw = SamplerSpec(SamplerKind.RAW_LOGITS)
    resp = drv.fire_batch(fold([PendingRequest(0, toks, list(range(len(toks))), list(range(4)), 0, [(len(toks) - 1, raw)])], 16))
    got = np.frombuffer(resp.slots[0].logits, dtype=np.float32)
    want = dense_reference_forward(cfg2, dequantized(w2), torch.tensor(toks))[-1].numpy()
    assert np.abs(got - want).max() < 1e-3
    # a tensor-parallel rank gets the matching scale columns of row-parallel weights
    _, wr = loader.load_checkpoint(tmp_path, "cpu", tp_size=2, tp_rank=1, dtype="float32")
    full, part = w2["layers"][0]["wo"], wr["layers"][0]["wo"]
    assert part.shape == (cfg.hidden_size, full.shape[1] // 2)
    assert torch.equal(part.dequant(torch.float32), full.dequant(torch.float32)[:, full.shape[1] // 2:])


def test_phi3_fused_projections_load_like_split_ones(tmp_path):
    """A checkpoint that stores qkv_proj and gate_up_proj fused (Phi-3 layout) loads into the same
    runtime weights as the split layout, also for a tensor-parallel rank."""
    import json as _json
    from safetensors import safe_open
    from safetensors.torch import save_file
    from pie_b200.models import loader
    from pie_b200.models.config import preset
    from pie_b200.models.weights import random_weights
    cfg = preset("tiny-llama")
    w = random_weights(cfg, "cpu", torch.float32, seed=5)
    split_dir, fused_dir = tmp_path / "split", tmp_path / "fused"
    loader.export_hf_checkpoint(cfg, w, split_dir)
    fused_dir.mkdir()
    tensors = {}
    with safe_open(str(split_dir / "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            tensors[k] = f.get_tensor(k)
    out = {k: v for k, v in tensors.items() if "_proj.weight" not in k or "o_proj" in k or "down_proj" in k}
    for li in range(cfg.num_hidden_layers):
        L = f"model.layers.{li}."
        out[L + "self_attn.qkv_proj.weight"] = torch.cat([tensors[L + f"self_attn.{x}_proj.weight"] for x in "qkv"], 0)
        out[L + "mlp.gate_up_proj.weight"] = torch.cat([tensors[L + "mlp.gate_proj.weight"], tensors[L + "mlp.up_proj.weight"]], 0)
    save_file(out, str(fused_dir / "model.safetensors"))
    hf = _json.loads((split_dir / "config.json").read_text())
    hf["model_type"] = "phi3"
    (fused_dir / "config.json").write_text(_json.dumps(hf))
    for tp, rank in [(1, 0), (2, 1)]:
        _, a = loader.load_checkpoint(split_dir, "cpu", tp, rank, dtype="float32")
        _, b = loader.load_checkpoint(fused_dir, "cpu", tp, rank, dtype="float32")
        for la, lb in zip(a["layers"], b["layers"]):
            assert torch.equal(la["wqkv"], lb["wqkv"]) and torch.equal(la["w_gate_up"], lb["w_gate_up"])


def test_mixtral_tensor_names(tmp_path):
    """block_sparse_moe.{gate, experts.N.w1/w3/w2} (Mixtral) load like mlp.{gate, experts.N.gate/up/down_proj}."""
    import json as _json
    from safetensors import safe_open
    from safetensors.torch import save_file
    from pie_b200.models import loader
    from pie_b200.models.config import preset
    from pie_b200.models.weights import random_weights
    cfg = preset("tiny-qwen3-moe")
    w = random_weights(cfg, "cpu", torch.float32, seed=2)
    a_dir, b_dir = tmp_path / "qwen", tmp_path / "mixtral"
    loader.export_hf_checkpoint(cfg, w, a_dir)
    b_dir.mkdir()
    out = {}
    with safe_open(str(a_dir / "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            nk = (k.replace("mlp.gate.weight", "block_sparse_moe.gate.weight")
                   .replace("mlp.experts.", "block_sparse_moe.experts.")
                   .replace("gate_proj", "w1").replace("up_proj", "w3").replace("down_proj", "w2"))
            out[nk] = f.get_tensor(k)
    save_file(out, str(b_dir / "model.safetensors"))
    hf = _json.loads((a_dir / "config.json").read_text())
    hf.update(model_type="mixtral", num_local_experts=hf.pop("num_experts"), intermediate_size=hf.pop("moe_intermediate_size"))
    hf["qk_norm"] = False
    (b_dir / "config.json").write_text(_json.dumps(hf))
    cfg_b, wb = loader.load_checkpoint(b_dir, "cpu", dtype="float32")
    _, wa = loader.load_checkpoint(a_dir, "cpu", dtype="float32")
    assert cfg_b.num_experts == cfg.num_experts and cfg_b.moe_intermediate_size == cfg.moe_intermediate_size
    for la, lb in zip(wa["layers"], wb["layers"]):
        assert torch.equal(la["experts_gate_up"], lb["experts_gate_up"]) and torch.equal(la["router"], lb["router"])
        assert torch.equal(la["experts_down"], lb["experts_down"])


def test_olmo2_post_norm_family_loads_and_matches_dense_oracle(tmp_path):
    """OLMo-2: no input norm, norms after attention and after the MLP, q/k RMSNorm over all
    heads together. A checkpoint under its Hugging Face names loads, and prefill + decode
    through the paged driver give the dense oracle's logits."""
    import numpy as np
    from pie_b200.driver.executor import TorchDriver
    from pie_b200.driver.schema import SamplerKind, SamplerSpec
    from pie_b200.models import loader
    from pie_b200.models.config import preset
    from pie_b200.models.transformer import dense_reference_forward
    from pie_b200.models.weights import random_weights
    from pie_b200.runtime.scheduler import PendingRequest, fold

    cfg = preset("tiny-olmo2")
    w = random_weights(cfg, "cpu", torch.float32, seed=5)
    assert "ln1" not in w["layers"][0] and w["layers"][0]["q_norm"].numel() == cfg.q_size
    loader.export_hf_checkpoint(cfg, w, tmp_path)
    cfg2, w2 = loader.load_checkpoint(tmp_path, "cpu", dtype="float32")
    assert cfg2.post_norm and cfg2.qk_norm and cfg2.model_type == "olmo2"
    for key in ("ln2", "ln3", "q_norm", "k_norm", "wqkv", "w_gate_up"):
        assert torch.equal(w2["layers"][1][key], w["layers"][1][key])
    drv = TorchDriver(cfg2, "cpu", weights=w2, num_pages=16, page_size=16, max_requests=4, max_tokens=128)
    toks = list(range(100, 137))
    raw = SamplerSpec(SamplerKind.RAW_LOGITS)
    resp = drv.fire_batch(fold([PendingRequest(0, toks, list(range(len(toks))), list(range(4)), 0, [(len(toks) - 1, raw)])], 16))
    got = np.frombuffer(resp.slots[0].logits, dtype=np.float32)
    want = dense_reference_forward(cfg2, w2, torch.tensor(toks))[-1].numpy()
    assert np.abs(got - want).max() < 1e-3
    # one decode step on top of the cached prefix
    resp = drv.fire_batch(fold([PendingRequest(0, [7], [len(toks)], list(range(4)), len(toks), [(0, raw)])], 16))
    got = np.frombuffer(resp.slots[0].logits, dtype=np.float32)
    want = dense_reference_forward(cfg2, w2, torch.tensor(toks + [7]))[-1].numpy()
    assert np.abs(got - want).max() < 1e-3
    # tensor-parallel shards keep the norm gains of their own heads
    _, wr = loader.load_checkpoint(tmp_path, "cpu", tp_size=2, tp_rank=1, dtype="float32")
    ws = random_weights(cfg, "cpu", torch.float32, seed=5, tp_size=2, tp_rank=1)
    assert torch.equal(wr["layers"][0]["q_norm"], ws["layers"][0]["q_norm"])
    assert torch.equal(wr["layers"][0]["k_norm"], ws["layers"][0]["k_norm"])
    assert torch.equal(wr["layers"][0]["q_norm"], w["layers"][0]["q_norm"][cfg.q_size // 2:])


def test_sliding_window_prefill_and_decode_match_windowed_oracle():
    """Mistral-style sliding window: prefill and decode through the paged driver see only the
    last `sliding_window` keys; config.json enables it for Mistral without a separate switch."""
    import numpy as np
    from pie_b200.driver.executor import TorchDriver
    from pie_b200.driver.schema import SamplerKind, SamplerSpec
    from pie_b200.models.config import ModelConfig, preset
    from pie_b200.models.transformer import dense_reference_forward
    from pie_b200.models.weights import random_weights
    from pie_b200.runtime.scheduler import PendingRequest, fold

    hf = dict(model_type="mistral", hidden_size=64, num_hidden_layers=1, num_attention_heads=2, vocab_size=100,
              sliding_window=4096)
    assert ModelConfig.from_hf(hf).sliding_window == 4096
    assert ModelConfig.from_hf(dict(hf, model_type="qwen2")).sliding_window == -1
    assert ModelConfig.from_hf(dict(hf, model_type="qwen2", use_sliding_window=True)).sliding_window == 4096

    cfg = preset("tiny-llama", sliding_window=21)
    w = random_weights(cfg, "cpu", torch.float32, seed=7, std=0.08)
    drv = TorchDriver(cfg, "cpu", weights=w, num_pages=16, page_size=16, max_requests=4, max_tokens=128)
    toks = list(range(200, 250))
    raw = SamplerSpec(SamplerKind.RAW_LOGITS)
    resp = drv.fire_batch(fold([PendingRequest(0, toks, list(range(len(toks))), list(range(5)), 0, [(len(toks) - 1, raw)])], 16))
    got = np.frombuffer(resp.slots[0].logits, dtype=np.float32)
    want = dense_reference_forward(cfg, w, torch.tensor(toks))[-1].numpy()
    full = dense_reference_forward(preset("tiny-llama"), w, torch.tensor(toks))[-1].numpy()
    assert np.abs(got - want).max() < 1e-3 and np.abs(want - full).max() > 1e-2      # the window matters
    resp = drv.fire_batch(fold([PendingRequest(0, [9], [len(toks)], list(range(5)), len(toks), [(0, raw)])], 16))
    got = np.frombuffer(resp.slots[0].logits, dtype=np.float32)
    want = dense_reference_forward(cfg, w, torch.tensor(toks + [9]))[-1].numpy()
    assert np.abs(got - want).max() < 1e-3


def test_rope_scaling_tables_match_transformers():
    """Llama-3, linear and YaRN frequency tables (and YaRN's attention factor) against the
    Hugging Face implementation."""
    from pie_b200.ops import reference as r
    tf = pytest.importorskip("transformers")
    from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
    for sc in [dict(rope_type="yarn", factor=4.0, original_max_position_embeddings=32768),
               dict(rope_type="linear", factor=2.0),
               dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                    original_max_position_embeddings=8192)]:
        cfg = tf.LlamaConfig(hidden_size=4096, num_attention_heads=32, rope_theta=1e6, max_position_embeddings=131072,
                             rope_scaling=dict(sc))
        inv, att = ROPE_INIT_FUNCTIONS[sc["rope_type"]](cfg, "cpu")
        mine = r.rope_inv_freq(128, 1e6, sc)
        assert float((inv - mine).abs().max() / inv.abs().max()) < 1e-6
        assert abs(att - r.rope_attention_factor(sc)) < 1e-9


def test_gguf_checkpoint_loads_like_safetensors(tmp_path):
    """A GGUF file (llama architecture: q/k rows in llama.cpp's interleaved order; F16, BF16, F32
    and Q8_0 tensors) loads through the same storage program as safetensors, also sharded."""
    import numpy as np
    from pie_b200.models import gguf, loader
    from pie_b200.models.config import preset
    from pie_b200.models.transformer import dense_reference_forward
    from pie_b200.models.weights import random_weights

    cfg = preset("tiny-llama")
    w = random_weights(cfg, "cpu", torch.float32, seed=9, std=0.05)
    d, hq, hkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    tensors = {"token_embd.weight": (w["embed"], gguf.T_F16), "output_norm.weight": (w["final_norm"], gguf.T_F32),
               "output.weight": (w["lm_head"], gguf.T_BF16)}
    for li, lw in enumerate(w["layers"]):
        q, k, v = lw["wqkv"].split([hq * d, hkv * d, hkv * d], 0)
        B = f"blk.{li}."
        tensors[B + "attn_norm.weight"] = (lw["ln1"], gguf.T_F32)
        tensors[B + "ffn_norm.weight"] = (lw["ln2"], gguf.T_F32)
        tensors[B + "attn_q.weight"] = (gguf.permute_rotary(q, hq), gguf.T_F16)
        tensors[B + "attn_k.weight"] = (gguf.permute_rotary(k, hkv), gguf.T_F16)
        tensors[B + "attn_v.weight"] = (v, gguf.T_Q8_0)
        tensors[B + "attn_output.weight"] = (lw["wo"], gguf.T_F16)
        tensors[B + "ffn_gate.weight"] = (lw["w_gate_up"][0::2], gguf.T_F16)
        tensors[B + "ffn_up.weight"] = (lw["w_gate_up"][1::2], gguf.T_F16)
        tensors[B + "ffn_down.weight"] = (lw["w_down"], gguf.T_Q8_0)
    meta = {"general.architecture": "llama", "general.name": "tiny", "llama.embedding_length": cfg.hidden_size,
            "llama.block_count": cfg.num_hidden_layers, "llama.attention.head_count": hq,
            "llama.attention.head_count_kv": hkv, "llama.feed_forward_length": cfg.intermediate_size,
            "llama.context_length": 4096, "llama.rope.freq_base": float(cfg.rope_theta),
            "llama.attention.layer_norm_rms_epsilon": float(cfg.rms_norm_eps), "llama.vocab_size": cfg.vocab_size,
            "tokenizer.ggml.tokens": ["a", "b", "c"]}
    path = tmp_path / "tiny.gguf"
    gguf.write_gguf(path, meta, tensors)

    rd = gguf.GGUFReader(path)
    assert rd.meta["tokenizer.ggml.tokens"] == ["a", "b", "c"] and rd.version == 3
    cfg2, w2 = loader.load_checkpoint(path, "cpu", dtype="float32")
    assert (cfg2.hidden_size, cfg2.num_hidden_layers, cfg2.num_key_value_heads, cfg2.head_dim, cfg2.vocab_size) == \
        (cfg.hidden_size, cfg.num_hidden_layers, hkv, d, cfg.vocab_size)
    assert not cfg2.tie_word_embeddings
    lw, lw2 = w["layers"][1], w2["layers"][1]
    assert (lw2["wqkv"][: (hq + hkv) * d] - lw["wqkv"][: (hq + hkv) * d]).abs().max() < 1e-3      # fp16 rounding, order restored
    assert (lw2["w_down"] - lw["w_down"]).abs().max() < 0.05 * lw["w_down"].abs().max() / 2          # Q8_0 steps
    assert (lw2["w_gate_up"] - lw["w_gate_up"]).abs().max() < 1e-3
    toks = torch.arange(50, 90)
    got = dense_reference_forward(cfg2, w2, toks)[-1]
    want = dense_reference_forward(cfg, w, toks)[-1]
    assert torch.nn.functional.cosine_similarity(got, want, dim=0) > 0.999
    # directory form and a tensor-parallel shard
    _, wr = loader.load_checkpoint(tmp_path, "cpu", tp_size=2, tp_rank=1, dtype="float32")
    assert torch.equal(wr["layers"][0]["wo"], w2["layers"][0]["wo"][:, hq * d // 2:])
    # Q4_0 blocks expand as scale * (nibble - 8)
    raw = np.zeros(18, dtype=np.uint8)
    raw[:2] = np.array([0.5], dtype=np.float16).view(np.uint8)
    raw[2] = 0x1F            # element 0 = 15, element 16 = 1
    x = gguf.dequantize(raw, gguf.T_Q4_0, 32)
    assert x[0] == 0.5 * (15 - 8) and x[16] == 0.5 * (1 - 8) and x[1] == 0.5 * (0 - 8)


def test_gpt_oss_family_runs_through_the_paged_driver():
    """GPT-OSS style blocks: alternating sliding / full attention layers, per-head attention sinks,
    biases on q/k/v/o, router and expert biases, clamped GLU experts, YaRN without truncation.
    Prefill and decode through the paged driver against the dense oracle."""
    import numpy as np
    from pie_b200.driver.executor import TorchDriver
    from pie_b200.driver.schema import SamplerKind, SamplerSpec
    from pie_b200.models.config import ModelConfig, preset
    from pie_b200.models.transformer import dense_reference_forward
    from pie_b200.models.weights import random_weights
    from pie_b200.runtime.scheduler import PendingRequest, fold

    hf = dict(model_type="gpt_oss", hidden_size=2880, intermediate_size=2880, num_hidden_layers=4, num_attention_heads=64,
              num_key_value_heads=8, head_dim=64, vocab_size=201088, num_local_experts=32, num_experts_per_tok=4,
              sliding_window=128, layer_types=["sliding_attention", "full_attention"] * 2, swiglu_limit=7.0)
    c = ModelConfig.from_hf(hf)
    assert c.is_moe and c.moe_intermediate_size == 2880 and c.attention_sinks and c.o_bias and c.attention_bias
    assert [c.layer_window_left(i) for i in range(4)] == [127, -1, 127, -1] and c.plan_window_left == -1

    cfg = preset("tiny-gpt-oss")
    w = random_weights(cfg, "cpu", torch.float32, seed=11, std=0.08)
    drv = TorchDriver(cfg, "cpu", weights=w, num_pages=16, page_size=16, max_requests=4, max_tokens=128)
    toks = list(range(300, 345))
    raw = SamplerSpec(SamplerKind.RAW_LOGITS)
    resp = drv.fire_batch(fold([PendingRequest(0, toks, list(range(len(toks))), list(range(4)), 0, [(len(toks) - 1, raw)])], 16))
    got = np.frombuffer(resp.slots[0].logits, dtype=np.float32)
    want = dense_reference_forward(cfg, w, torch.tensor(toks))[-1].numpy()
    assert np.abs(got - want).max() < 2e-3
    resp = drv.fire_batch(fold([PendingRequest(0, [5], [len(toks)], list(range(4)), len(toks), [(0, raw)])], 16))
    got = np.frombuffer(resp.slots[0].logits, dtype=np.float32)
    want = dense_reference_forward(cfg, w, torch.tensor(toks + [5]))[-1].numpy()
    assert np.abs(got - want).max() < 2e-3
    # the sinks and the window both matter in this setup
    w2 = {**w, "layers": [{k: v for k, v in lw.items() if k != "sinks"} for lw in w["layers"]]}
    assert np.abs(dense_reference_forward(cfg, w2, torch.tensor(toks + [5]))[-1].numpy() - want).max() > 1e-3


def test_gpt_oss_checkpoint_names_and_mxfp4_experts(tmp_path):
    """GPT-OSS checkpoints: stacked experts as [E, in, out] (bf16) or as MXFP4 blocks + e8m0
    scales, router / expert / o_proj biases, attention sinks."""
    from safetensors import safe_open
    from safetensors.torch import save_file
    from pie_b200.models import loader
    from pie_b200.models.config import preset
    from pie_b200.models.weights import random_weights

    cfg = preset("tiny-gpt-oss")
    w = random_weights(cfg, "cpu", torch.float32, seed=12, std=0.08)
    loader.export_hf_checkpoint(cfg, w, tmp_path)
    cfg2, w2 = loader.load_checkpoint(tmp_path, "cpu", dtype="float32")
    assert cfg2.model_type == "gpt_oss" and cfg2.layer_types == cfg.layer_types and cfg2.attention_sinks
    assert cfg2.rope_scaling["truncate"] is False
    for key in ("wqkv", "bqkv", "wo", "bo", "sinks", "router", "router_bias", "experts_gate_up", "experts_down",
                "experts_gate_up_bias", "experts_down_bias"):
        assert torch.equal(w2["layers"][1][key], w["layers"][1][key]), key
    # the same experts as MXFP4 blocks
    tensors = {}
    with safe_open(str(tmp_path / "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            tensors[k] = f.get_tensor(k)
    for li, lw in enumerate(w["layers"]):
        for src, dst in (("gate_up_proj", "experts_gate_up"), ("down_proj", "experts_down")):
            X = f"model.layers.{li}.mlp.experts.{src}"
            del tensors[X]
            tensors[X + "_blocks"], tensors[X + "_scales"] = loader.quant_mxfp4(lw[dst])
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(tmp_path / "model.safetensors"))
    _, w3 = loader.load_checkpoint(tmp_path, "cpu", dtype="float32")
    got, ref = w3["layers"][0]["experts_down"], w["layers"][0]["experts_down"]
    assert got.shape == ref.shape
    assert torch.equal(got, loader.dequant_mxfp4(*loader.quant_mxfp4(ref)))
    assert (got - ref).abs().max() <= 0.26 * ref.abs().amax()        # e2m1 steps: at most 1 in 6 of the block maximum... plus scale rounding
    # known values: byte 0x2C = low nibble 12 (-2.0), high nibble 2 (1.0); scale 128 -> 2.0
    blk = torch.zeros(1, 1, 16, dtype=torch.uint8)
    blk[0, 0, 0] = 0x2C
    out = loader.dequant_mxfp4(blk, torch.tensor([[128]], dtype=torch.uint8))
    assert out[0, 0].item() == -4.0 and out[0, 1].item() == 2.0 and out[0, 2].item() == 0.0


def test_gpt_oss_tensor_parallel_shards(tmp_path):
    """GPT-OSS under tensor parallelism: experts sharded on their intermediate dimension (gate/up
    pairs stay together, also in the bias), the output bias on rank 0 only, sinks by head; the loader
    and the random initialiser agree."""
    from pie_b200.models import loader
    from pie_b200.models.config import preset
    from pie_b200.models.weights import random_weights

    cfg = preset("tiny-gpt-oss")
    full = random_weights(cfg, "cpu", torch.float32, seed=13)
    loader.export_hf_checkpoint(cfg, full, tmp_path)
    Im = cfg.moe_intermediate_size
    for r in range(2):
        w = random_weights(cfg, "cpu", torch.float32, seed=13, tp_size=2, tp_rank=r)
        _, l = loader.load_checkpoint(tmp_path, "cpu", tp_size=2, tp_rank=r, dtype="float32")
        for key in ("experts_gate_up", "experts_down", "experts_gate_up_bias", "experts_down_bias", "sinks", "bo", "wo"):
            assert torch.equal(l["layers"][0][key], w["layers"][0][key]), (r, key)
        lw = w["layers"][0]
        assert torch.equal(lw["experts_gate_up"], full["layers"][0]["experts_gate_up"][:, r * Im:(r + 1) * Im])
        assert torch.equal(lw["experts_down"], full["layers"][0]["experts_down"][:, :, r * Im // 2:(r + 1) * Im // 2])
        assert (lw["experts_down_bias"].abs().sum() > 0) == (r == 0)


def test_weight_artifact_cache_round_trip_and_keying(tmp_path, monkeypatch):
    """PIE_WEIGHT_CACHE_DIR: the first load materialises and stores this rank's weights, the second
    reads the entry (equal tensors, no storage program run), another shard plan gets its own entry,
    a touched checkpoint invalidates, a damaged entry is rebuilt."""
    import os
    cfg = preset("tiny-qwen3-moe", vocab_size=512)
    full = random_weights(cfg, "cpu", torch.float32, seed=5)
    src = tmp_path / "ckpt"
    src.mkdir()
    loader.export_hf_checkpoint(cfg, full, str(src))
    cache = tmp_path / "cache"
    monkeypatch.setenv("PIE_WEIGHT_CACHE_DIR", str(cache))
    _, a = loader.load_checkpoint(str(src), dtype="float32")
    assert len(list(cache.glob("*.safetensors"))) == 1 and _same(full, a)
    calls = []
    real = loader.execute_program
    monkeypatch.setattr(loader, "execute_program", lambda *x, **k: calls.append(1) or real(*x, **k))
    _, b = loader.load_checkpoint(str(src), dtype="float32")
    assert calls == [] and _same(a, b) and b["lm_head_vocab_start"] == 0
    _, r1 = loader.load_checkpoint(str(src), tp_size=2, tp_rank=1, dtype="float32")
    assert len(calls) == 1 and len(list(cache.glob("*.safetensors"))) == 2
    assert _same(random_weights(cfg, "cpu", torch.float32, seed=5, tp_size=2, tp_rank=1), r1)
    f = next(src.glob("*.safetensors"))
    os.utime(f, ns=(f.stat().st_atime_ns, f.stat().st_mtime_ns + 10**9))       # the checkpoint changed
    loader.load_checkpoint(str(src), dtype="float32")
    assert len(calls) == 2 and len(list(cache.glob("*.safetensors"))) == 3
    for e in cache.glob("*.safetensors"):
        e.write_bytes(b"broken")
    _, c = loader.load_checkpoint(str(src), dtype="float32")
    assert len(calls) == 3 and _same(full, c)
    assert not list(cache.glob("*.tmp*"))


def test_olmo3_alternating_window_layers_load_and_match_dense_oracle(tmp_path):
    """OLMo-3 = the OLMo-2 block with sliding-window layers alternating with full-attention ones
    (`layer_types`). Context longer than the window, so the two kinds of layer differ."""
    import json
    import numpy as np
    from pie_b200.driver.executor import TorchDriver
    from pie_b200.driver.schema import SamplerKind, SamplerSpec
    from pie_b200.models import loader
    from pie_b200.models.config import ModelConfig, preset
    from pie_b200.models.transformer import dense_reference_forward
    from pie_b200.models.weights import random_weights
    from pie_b200.runtime.scheduler import PendingRequest, fold

    cfg = preset("tiny-olmo2", model_type="olmo3", sliding_window=8, layer_types=["sliding_attention", "full_attention"])
    w = random_weights(cfg, "cpu", torch.float32, seed=6)
    loader.export_hf_checkpoint(cfg, w, tmp_path)
    hf = json.loads((tmp_path / "config.json").read_text())
    hf.update(model_type="olmo3", sliding_window=8, layer_types=["sliding_attention", "full_attention"])
    (tmp_path / "config.json").write_text(json.dumps(hf))
    cfg2, w2 = loader.load_checkpoint(tmp_path, "cpu", dtype="float32")
    assert cfg2.model_type == "olmo3" and cfg2.post_norm and cfg2.qk_norm
    assert [cfg2.layer_window_left(i) for i in range(2)] == [7, -1] and cfg2.plan_window_left == -1
    drv = TorchDriver(cfg2, "cpu", weights=w2, num_pages=16, page_size=16, max_requests=4, max_tokens=128)
    toks = list(range(100, 140))
    raw = SamplerSpec(SamplerKind.RAW_LOGITS)
    resp = drv.fire_batch(fold([PendingRequest(0, toks, list(range(len(toks))), list(range(4)), 0, [(len(toks) - 1, raw)])], 16))
    got = np.frombuffer(resp.slots[0].logits, dtype=np.float32)
    want = dense_reference_forward(cfg2, w2, torch.tensor(toks))[-1].numpy()
    assert np.abs(got - want).max() < 1e-3
    full = dense_reference_forward(ModelConfig(**{**cfg2.to_dict(), "sliding_window": -1, "layer_types": None}), w2,
                                   torch.tensor(toks))[-1].numpy()
    assert np.abs(full - want).max() > 1e-3                     # the window really changes the result
    resp = drv.fire_batch(fold([PendingRequest(0, [7], [len(toks)], list(range(4)), len(toks), [(0, raw)])], 16))
    got = np.frombuffer(resp.slots[0].logits, dtype=np.float32)
    want = dense_reference_forward(cfg2, w2, torch.tensor(toks + [7]))[-1].numpy()
    assert np.abs(got - want).max() < 1e-3


def test_type_check_reports_every_misfit_before_reading_tensors(tmp_path):
    """The loader infers every runtime shape from the checkpoint's header and compares it with the
    configuration: a wrong config fails with the list of tensors that do not fit, and no tensor is read."""
    import json
    from pie_b200.models import loader
    from pie_b200.models.config import ModelConfig, preset
    from pie_b200.models.weights import random_weights
    cfg = preset("tiny-llama")
    loader.export_hf_checkpoint(cfg, random_weights(cfg, "cpu", torch.float32, seed=1), tmp_path)
    rd = loader.SafetensorsReader(tmp_path)
    prog = loader.compile_program(cfg, rd.names(), 2, 1)
    shapes = loader.typecheck_program(prog, cfg, rd)
    assert shapes["layers.0.wqkv"] == ((2 + 2 * 1) * cfg.head_dim, cfg.hidden_size)         # this rank's heads
    assert shapes["layers.1.w_down"] == (cfg.hidden_size, cfg.intermediate_size // 2)
    hf = json.loads((tmp_path / "config.json").read_text())
    hf["intermediate_size"] += 16
    hf["num_key_value_heads"] = 4
    (tmp_path / "config.json").write_text(json.dumps(hf))
    reads = []
    orig = loader.SafetensorsReader.get
    loader.SafetensorsReader.get = lambda self, name: reads.append(name) or orig(self, name)
    try:
        with pytest.raises(loader.LoaderTypeError) as e:
            loader.load_checkpoint(tmp_path, "cpu")
    finally:
        loader.SafetensorsReader.get = orig
    msg = str(e.value)
    assert "layers.0.w_gate_up" in msg and "layers.0.w_down" in msg and "rows" in msg and reads == []
    with pytest.raises(loader.LoaderTypeError, match="does not split over 3 ranks"):
        loader.infer_shape(loader.Shard(loader.Read("model.layers.0.mlp.down_proj.weight"), 1, 0, 3), rd)


@pytest.mark.parametrize("strategy", ["tensor", "channel"])
def test_fp8_per_tensor_and_per_channel_checkpoints_load(tmp_path, strategy):
    """fp8 checkpoints with one scale per weight tensor or per output channel (`weight_scale` beside each weight, the
    compressed-tensors / fbgemm layout) load into the block-scaled runtime format: the scale is spread over a row's
    blocks, also through the fused QKV join, the gate / up interleave and a tensor-parallel shard."""
    import json as _json
    import numpy as np
    from safetensors import safe_open
    from safetensors.torch import save_file
    from pie_b200 import ops
    from pie_b200.driver.executor import TorchDriver
    from pie_b200.driver.schema import SamplerKind, SamplerSpec
    from pie_b200.models import loader
    from pie_b200.models.config import ModelConfig, preset
    from pie_b200.models.transformer import dense_reference_forward
    from pie_b200.models.weights import dequantized, random_weights
    from pie_b200.runtime.scheduler import PendingRequest, fold
    cfg = preset("tiny-llama")
    w = random_weights(cfg, "cpu", torch.float32, seed=3)
    loader.export_hf_checkpoint(cfg, w, tmp_path)
    out = {}
    with safe_open(str(tmp_path / "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            t = f.get_tensor(k)
            if k.endswith("_proj.weight"):
                amax = t.abs().amax() if strategy == "tensor" else t.abs().amax(dim=1, keepdim=True)
                sc = (amax.clamp_min(1e-12) / 448.0).float()
                out[k] = (t / sc).to(torch.float8_e4m3fn)
                out[k + "_scale"] = sc.reshape(1) if strategy == "tensor" else sc          # [1] or [N, 1]
                out[k[:-len("weight")] + "input_scale"] = torch.ones(1)                       # a static activation scale: unused
            else:
                out[k] = t
    save_file(out, str(tmp_path / "model.safetensors"))
    hf = _json.loads((tmp_path / "config.json").read_text())
    hf["quantization_config"] = {"quant_method": "compressed-tensors", "config_groups": {"group_0": {
        "weights": {"num_bits": 8, "type": "float", "strategy": strategy}, "input_activations": {"num_bits": 8, "type": "float"}}}}
    (tmp_path / "config.json").write_text(_json.dumps(hf))
    assert ModelConfig.from_hf({**hf, "quantization_config": {"quant_method": "fbgemm_fp8"}}).quantization == "fp8_block"
    assert ModelConfig.from_hf({**hf, "quantization_config": {"quant_method": "compressed-tensors", "config_groups": {"g": {
        "weights": {"num_bits": 4, "type": "int", "strategy": "group"}}}}}).quantization is None
    cfg2, w2 = loader.load_checkpoint(tmp_path, "cpu", dtype="float32")
    lw = w2["layers"][0]
    assert cfg2.quantization == "fp8_block" and isinstance(lw["wqkv"], ops.Fp8Linear) and isinstance(lw["w_down"], ops.Fp8Linear)
    assert lw["w_gate_up"].scale.shape == (2 * cfg.intermediate_size, cfg.hidden_size // 128)
    if strategy == "tensor":        # q, k and v keep their own scales inside the fused tensor
        q_rows = cfg.num_attention_heads * cfg.head_dim
        assert lw["wqkv"].scale[:q_rows].unique().numel() == 1 and lw["wqkv"].scale.unique().numel() == 3
    err = (lw["wo"].dequant(torch.float32) - w["layers"][0]["wo"]).abs().max() / w["layers"][0]["wo"].abs().max()
    assert err < 0.07
    drv = TorchDriver(cfg2, "cpu", weights=w2, num_pages=16, page_size=16, max_requests=4, max_tokens=128)
    toks = list(range(40, 70))
    raw = SamplerSpec(SamplerKind.RAW_LOGITS)
    resp = drv.fire_batch(fold([PendingRequest(0, toks, list(range(len(toks))), list(range(4)), 0, [(len(toks) - 1, raw)])], 16))
    got = np.frombuffer(resp.slots[0].logits, dtype=np.float32)
    want = dense_reference_forward(cfg2, dequantized(w2), torch.tensor(toks))[-1].numpy()
    assert np.abs(got - want).max() < 1e-3
    _, wr = loader.load_checkpoint(tmp_path, "cpu", tp_size=2, tp_rank=1, dtype="float32")
    full, part = w2["layers"][0]["w_gate_up"], wr["layers"][0]["w_gate_up"]
    assert torch.equal(part.dequant(torch.float32), full.dequant(torch.float32)[full.shape[0] // 2:])
