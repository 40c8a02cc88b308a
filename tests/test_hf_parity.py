"""Parity with Hugging Face transformers, an implementation independent of this repository: tiny random
checkpoints are exported under their Hugging Face names, loaded by `AutoModelForCausalLM` and by this
loader, and the paged driver's logits (prefill, then a decode step on the cached prefix) must agree with
transformers' to fp32 rounding. The Gated DeltaNet mixer is checked against transformers' Qwen3-Next module
through the checkpoint layout of the exporter."""
import json

import numpy as np
import pytest
import torch

transformers = pytest.importorskip("transformers")

from pie_b200 import parity  # noqa: E402
from pie_b200.models import loader  # noqa: E402
from pie_b200.models.config import preset  # noqa: E402
from pie_b200.models.weights import random_weights  # noqa: E402

FAMILIES = [
    ("llama", "tiny-llama", {}),
    ("qwen2", "tiny-llama", dict(model_type="qwen2", attention_bias=True)),
    ("qwen3", "tiny-llama", dict(model_type="qwen3", qk_norm=True)),
    ("mistral", "tiny-llama", dict(model_type="mistral", sliding_window=16)),
    ("olmo2", "tiny-olmo2", {}),
    ("olmo3", "tiny-olmo2", dict(model_type="olmo3", sliding_window=8, layer_types=["sliding_attention", "full_attention"])),
    ("qwen3_moe", "tiny-qwen3-moe", {}),
    ("gpt_oss", "tiny-gpt-oss", {}),
    ("mixtral", "tiny-qwen3-moe", dict(model_type="mixtral", qk_norm=False)),
    ("phi3", "tiny-llama", dict(model_type="phi3")),
    ("gemma3_text", "tiny-gemma3", {}),
    ("gemma2", "tiny-gemma2", {}),
    ("qwen2_moe", "tiny-qwen2-moe", {}),
]


@pytest.mark.parametrize("family,base,over", FAMILIES, ids=[f[0] for f in FAMILIES])
def test_driver_logits_equal_transformers(family, base, over, tmp_path):
    cfg = preset(base, **over)
    cfg.dtype = "float32"
    loader.export_hf_checkpoint(cfg, random_weights(cfg, "cpu", torch.float32, seed=2), tmp_path)
    hf = json.loads((tmp_path / "config.json").read_text())
    if cfg.sliding_window > 0:
        hf["sliding_window"] = cfg.sliding_window
    if cfg.layer_types:
        hf["layer_types"] = cfg.layer_types
    (tmp_path / "config.json").write_text(json.dumps(hf))
    toks = list(range(100, 137))
    want = parity.run_hf(str(tmp_path), toks)
    for decode in (False, True):
        got = parity.run(family, toks, "cpu", str(tmp_path), decode_after_prefill=decode)
        rep = parity.compare(got, want)
        assert rep["max_abs"] < 2e-4 and rep["argmax_equal"] and rep["cos"] > 0.99999, (family, decode, rep)


def test_gated_deltanet_mixer_equals_transformers_qwen3_next_module():
    from transformers.models.qwen3_next.configuration_qwen3_next import Qwen3NextConfig
    from transformers.models.qwen3_next.modeling_qwen3_next import Qwen3NextGatedDeltaNet
    from pie_b200.driver.recurrent import RecurrentStateCache
    from pie_b200.ops import reference as ref
    cfg = preset("tiny-qwen3.5")
    cfg.dtype = "float32"
    lw = random_weights(cfg, "cpu", torch.float32, seed=5)["layers"][0]
    hk, hv, dk, dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
    mod = Qwen3NextGatedDeltaNet(Qwen3NextConfig(
        hidden_size=cfg.hidden_size, linear_num_key_heads=hk, linear_num_value_heads=hv, linear_key_head_dim=dk,
        linear_value_head_dim=dv, linear_conv_kernel_dim=4, rms_norm_eps=cfg.rms_norm_eps, hidden_act="silu",
        num_hidden_layers=4), 0).float()
    # the runtime layout goes to the checkpoint's layout the way the exporter writes it
    rep = hv // hk
    q, k, v, z, b, a = lw["w_gdn_in"].split([hk * dk, hk * dk, hv * dv, hv * dv, hv, hv], 0)
    grp = lambda x, n: x.reshape(hk, n, -1)
    mod.load_state_dict({
        "in_proj_qkvz.weight": torch.cat([grp(q, dk), grp(k, dk), grp(v, rep * dv), grp(z, rep * dv)], 1).reshape(-1, cfg.hidden_size),
        "in_proj_ba.weight": torch.cat([grp(b, rep), grp(a, rep)], 1).reshape(-1, cfg.hidden_size),
        "conv1d.weight": lw["gdn_conv"].unsqueeze(1), "A_log": lw["gdn_A_log"], "dt_bias": lw["gdn_dt_bias"],
        "norm.weight": lw["gdn_norm"], "out_proj.weight": lw["w_gdn_out"]}, strict=True)
    torch.manual_seed(0)
    x = torch.randn(23, cfg.hidden_size) * 0.5
    with torch.no_grad():
        want = mod(x[None])[0]
    # the cached, chunked mixer: 9 tokens, then 13, then 1
    cache = RecurrentStateCache(cfg, 2, "cpu")
    outs = []
    for a0, a1, reset in ((0, 9, 1), (9, 22, 0), (22, 23, 0)):
        mix = x[a0:a1] @ lw["w_gdn_in"].t()
        o = ref.gdn_mixer(mix, lw["gdn_conv"], lw["gdn_A_log"], lw["gdn_dt_bias"], lw["gdn_norm"], cfg.rms_norm_eps,
                          hk, hv, dk, dv, [0, a1 - a0], cache.conv_state[0], cache.rec_state[0], [1], [reset])
        outs.append(o @ lw["w_gdn_out"].t())
    got = torch.cat(outs)
    assert float((got - want).abs().max()) < 1e-5
