"""vLLM comparator arm: the benchmark's workload (same model shape, same synthetic prompts, same sampling) served
by vLLM from the image, with random-init weights (`load_format="dummy"`). vLLM is the engine the reference's own
benchmarks are quoted against (benches/results_vllm.json). One process; for N > 1 vLLM starts its own tensor-parallel
workers.

    python -m pie_b200.bench.vllm_arm [--model llama-3.1-8b] [--requests 512] [--out-tokens 256] [--gpus 1]

Measured: wall time of `generate` with max_tokens = 1 (prefill + one sample) and with max_tokens = out_tokens + 1;
the difference is the decode phase, so decode tokens/s = requests * out_tokens / (t_full - t_prefill); the
whole-workload rate (prefill included) is reported next to it. A warm-up generate precedes both.
"""
from __future__ import annotations

import argparse
import json
import os
import tempfile
import time


def write_config_dir(cfg) -> str:
    """A local directory vLLM can read the architecture from (no tokenizer, no weights)."""
    d = tempfile.mkdtemp(prefix="pie_b200_vllm_cfg_")
    arch = {"llama": "LlamaForCausalLM", "qwen3": "Qwen3ForCausalLM", "qwen2": "Qwen2ForCausalLM",
            "mistral": "MistralForCausalLM"}.get(cfg.model_type)
    if arch is None:
        raise ValueError(f"no vLLM arm for model type {cfg.model_type}")
    hf = {"architectures": [arch], "model_type": cfg.model_type, "hidden_size": cfg.hidden_size,
          "intermediate_size": cfg.intermediate_size, "num_hidden_layers": cfg.num_hidden_layers,
          "num_attention_heads": cfg.num_attention_heads, "num_key_value_heads": cfg.num_key_value_heads,
          "head_dim": cfg.head_dim, "vocab_size": cfg.vocab_size, "rms_norm_eps": cfg.rms_norm_eps,
          "rope_theta": cfg.rope_theta, "max_position_embeddings": min(cfg.max_position_embeddings, 8192),
          "tie_word_embeddings": cfg.tie_word_embeddings, "torch_dtype": "bfloat16", "hidden_act": "silu",
          "attention_bias": cfg.attention_bias, "bos_token_id": 1, "eos_token_id": 2}
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(hf, f)
    return d


def run(cfg, prompts, out_tokens: int, n_gpus: int = 1, temperature: float = 1.0, top_p: float = 0.9,
        max_num_seqs: int = 512) -> dict:
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    os.environ.setdefault("VLLM_NO_USAGE_STATS", "1")
    os.environ.setdefault("VLLM_WORKER_MULTIPROC_METHOD", "spawn")
    import vllm
    from vllm import LLM, SamplingParams
    from vllm.inputs import TokensPrompt
    path = write_config_dir(cfg)
    max_len = max(len(p) for p in prompts) + out_tokens + 8
    llm = LLM(model=path, load_format="dummy", skip_tokenizer_init=True, dtype="bfloat16", max_model_len=max_len,
              tensor_parallel_size=n_gpus, max_num_seqs=max_num_seqs, gpu_memory_utilization=0.9, seed=0,
              enable_prefix_caching=False, disable_log_stats=True)
    inputs = [TokensPrompt(prompt_token_ids=list(p)) for p in prompts]

    def gen(n):
        sp = SamplingParams(temperature=temperature, top_p=top_p, max_tokens=n, min_tokens=n, ignore_eos=True,
                            detokenize=False)
        t0 = time.perf_counter()
        outs = llm.generate(inputs, sp, use_tqdm=False)
        dt = time.perf_counter() - t0
        return dt, sum(len(o.outputs[0].token_ids) for o in outs)
    gen(4)                                              # warm-up: compilation, graph capture, allocator
    t_pre, n_pre = gen(1)
    t_full, n_full = gen(out_tokens + 1)
    decode_tokens = n_full - n_pre
    decode_s = max(t_full - t_pre, 1e-9)
    return {"impl": "vllm", "version": vllm.__version__, "n_gpus": n_gpus, "requests": len(prompts),
            "out_tokens": out_tokens, "prefill_s": t_pre, "full_s": t_full,
            "decode_tokens_per_s": decode_tokens / decode_s, "ms_per_step": decode_s / out_tokens * 1e3,
            "workload_tokens_per_s": n_full / t_full,
            "prefill_tokens_per_s": sum(len(p) for p in prompts) / t_pre,
            "sampler": f"temperature {temperature}, top-p {top_p}", "weights": "random (load_format=dummy)", "dtype": "bf16"}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3.1-8b")
    ap.add_argument("--requests", type=int, default=512)
    ap.add_argument("--prompt-min", type=int, default=128)
    ap.add_argument("--prompt-max", type=int, default=2048)
    ap.add_argument("--out-tokens", type=int, default=256)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--layers", type=int, default=0)
    a = ap.parse_args(argv)
    from ..models.config import preset
    from . import harness
    cfg = preset(a.model, **({"num_hidden_layers": a.layers} if a.layers else {}))
    prompts = harness.make_prompts(a.requests, a.prompt_min, a.prompt_max, cfg.vocab_size, seed=1)
    try:
        out = run(cfg, prompts, a.out_tokens, a.gpus)
    except Exception as e:  # noqa: BLE001 - a comparator that cannot start is reported, not fatal
        out = {"impl": "vllm", "unavailable": f"{type(e).__name__}: {e}"[:400]}
    print(json.dumps(out), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
