"""Mamba-2 hybrid (state-space mixers in llama-like blocks between full-attention layers): the cached, chunked
path against an independent dense oracle and against transformers' Mamba2Mixer; the engine on top of the
recurrent-state slots; checkpoint round trip. CPU driver; the CUDA kernel is tested in test_kernels_gpu.py."""
import json

import numpy as np
import pytest
import torch

from pie_b200.driver.executor import TorchDriver
from pie_b200.driver.schema import ForwardRequest, SamplerKind, SamplerSpec
from pie_b200.inferlets import install_all
from pie_b200.models import loader
from pie_b200.models.config import preset
from pie_b200.models.transformer import _dense_mamba2, dense_reference_forward
from pie_b200.models.weights import random_weights
from pie_b200.runtime.engine import Engine, EngineConfig


def model(seed=3, **over):
    cfg = preset("tiny-mamba2", **over)
    cfg.dtype = "float32"
    return cfg, random_weights(cfg, "cpu", torch.float32, seed=seed)


@pytest.mark.parametrize("grouped", [False, True])
def test_driver_matches_dense_oracle_over_chunks(grouped):
    cfg, w = model(mamba_norm_grouped=grouped)
    drv = TorchDriver(cfg, "cpu", weights=w, num_pages=16, page_size=16, max_requests=4, max_tokens=128)
    assert drv.capabilities().rs_cache_slots > 0
    toks = list(range(50, 71))
    want = dense_reference_forward(cfg, w, torch.tensor(toks)).numpy()
    i32 = lambda *a: np.asarray(a, dtype=np.int32)
    raw = SamplerSpec(SamplerKind.RAW_LOGITS)
    for a, b, reset in ((0, 9, 1), (9, 20, 0), (20, 21, 0)):
        kv = b
        req = ForwardRequest(tokens=np.asarray(toks[a:b], np.int32), positions=np.arange(a, b, dtype=np.int32),
                             qo_indptr=i32(0, b - a), kv_page_indices=np.arange(-(-kv // 16), dtype=np.int32),
                             kv_page_indptr=i32(0, -(-kv // 16)), kv_last_page_lens=i32((kv - 1) % 16 + 1),
                             slot_req=i32(0), slot_row=i32(b - a - 1), slot_samplers=[raw], rs_slots=i32(2), rs_reset=i32(reset))
        got = np.frombuffer(drv.fire_batch(req).slots[0].logits, dtype=np.float32)
        assert np.abs(got - want[b - 1]).max() < 1e-4


def test_mixer_equals_transformers_mamba2_module():
    pytest.importorskip("transformers")
    from transformers.models.mamba2.configuration_mamba2 import Mamba2Config
    from transformers.models.mamba2.modeling_mamba2 import Mamba2Mixer
    cfg, w = model(seed=5)
    lw = w["layers"][0]
    mod = Mamba2Mixer(Mamba2Config(hidden_size=cfg.hidden_size, num_heads=cfg.mamba_num_heads, head_dim=cfg.mamba_head_dim,
                                   state_size=cfg.ssm_state_size, n_groups=cfg.mamba_n_groups, expand=1, conv_kernel=4,
                                   num_hidden_layers=2, layer_norm_epsilon=cfg.rms_norm_eps), 0).float()
    mod.load_state_dict({"in_proj.weight": lw["w_mamba_in"], "conv1d.weight": lw["mamba_conv"].unsqueeze(1),
                         "conv1d.bias": lw["mamba_conv_bias"], "A_log": lw["mamba_A_log"], "dt_bias": lw["mamba_dt_bias"],
                         "D": lw["mamba_D"], "norm.weight": lw["mamba_norm"], "out_proj.weight": lw["w_mamba_out"]}, strict=True)
    torch.manual_seed(0)
    x = torch.randn(19, cfg.hidden_size) * 0.5
    with torch.no_grad():
        want = mod(x[None])[0]
    got = _dense_mamba2(cfg, lw, x) @ lw["w_mamba_out"].t()
    assert float((got - want).abs().max()) < 1e-5


def test_engine_generation_fork_and_checkpoint_round_trip(tmp_path):
    cfg, w = model()
    loader.export_hf_checkpoint(cfg, w, tmp_path)
    cfg2, w2 = loader.load_checkpoint(tmp_path, "cpu", dtype="float32")
    assert cfg2.model_type == "mamba2_hybrid" and cfg2.mamba_layers == [0, 1] and cfg2.ssm_state_size == 16
    for key in ("w_mamba_in", "mamba_conv", "mamba_conv_bias", "mamba_A_log", "mamba_D", "mamba_norm", "w_mamba_out"):
        assert torch.equal(w2["layers"][0][key], w["layers"][0][key]), key
    prompt = list(range(100, 141))

    def oracle(n):
        toks = list(prompt)
        for _ in range(n):
            toks.append(int(dense_reference_forward(cfg, w, torch.tensor(toks))[-1].argmax()))
        return toks[len(prompt):]
    drv = TorchDriver(cfg2, "cpu", weights=w2, num_pages=64, page_size=16, max_requests=8, max_tokens=32, rs_slots=4)
    eng = Engine(EngineConfig())
    eng.add_model("m", drv)
    install_all(eng)
    try:
        out = json.loads(eng.run("text-completion", {"prompt_tokens": prompt, "max_tokens": 5, "temperature": 0.0,
                                                     "stop_tokens": []}, 300))
        assert out["tokens"] == oracle(5)                       # 41 prompt tokens > max_tokens 32: chunked prefill
        assert eng.models["m"].ctxm.rs[0].slot_of == {}
    finally:
        eng.shutdown()
