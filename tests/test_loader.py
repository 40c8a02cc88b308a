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
