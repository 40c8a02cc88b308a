"""Tensor-parallel parity check, run as one process per GPU:

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29511 \
        tests/tp_check.py [--backend fused|nccl]

Rank 0 drives a prefill batch and two decode steps through the tensor-parallel driver (followers
mirror every fire from the control ring) and compares the logits with a single-GPU driver holding
the unsharded weights of the same seed. Same idea as the reference's tp=1 vs tp=2 parity script
(driver/cuda/tests/parity_tp.py:1-16: cosine, arg-max, top-5 overlap). Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os

os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # peer loads/stores only, no NVLS binding

import numpy as np
import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="fused")
    ap.add_argument("--hidden", type=int, default=512)
    ap.add_argument("--model", default="dense", choices=["dense", "dense-fp8", "moe", "moe-ep", "gpt-oss", "olmo2", "gemma3", "gemma2", "qwen2-moe"],
                    help="moe: experts sharded on their intermediate dimension; moe-ep: whole experts per rank")
    a = ap.parse_args()
    import torch.distributed as dist
    from pie_b200.driver.executor import TorchDriver
    from pie_b200.driver.schema import SamplerKind, SamplerSpec
    from pie_b200.models.config import preset
    from pie_b200.models.transformer import ParallelContext
    from pie_b200.runtime.scheduler import PendingRequest, fold
    from pie_b200.parallel.comm import TPComm

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    if a.model in ("dense", "dense-fp8"):
        cfg = preset("tiny-llama", hidden_size=a.hidden, intermediate_size=1536, num_attention_heads=8,
                     num_key_value_heads=2, head_dim=128, vocab_size=4096, num_hidden_layers=3, dtype="bfloat16",
                     quantization="fp8_block" if a.model == "dense-fp8" else None)
    elif a.model == "olmo2":
        cfg = preset("tiny-olmo2", hidden_size=a.hidden, intermediate_size=1536, num_attention_heads=8,
                     num_key_value_heads=2, head_dim=128, vocab_size=4096, num_hidden_layers=3, dtype="bfloat16")
    elif a.model in ("gemma3", "gemma2"):
        # sandwich norms, GeGLU, scaled embeddings, alternating local / global layers (gemma2: soft-capped scores and logits)
        cfg = preset("tiny-" + a.model, hidden_size=a.hidden, intermediate_size=1536, num_attention_heads=8,
                     num_key_value_heads=2, head_dim=128, vocab_size=4096, num_hidden_layers=3, dtype="bfloat16",
                     sliding_window=24, layer_types=["sliding_attention", "full_attention", "sliding_attention"],
                     embed_scale=float(a.hidden) ** 0.5, query_pre_attn_scalar=128.0)
    elif a.model == "qwen2-moe":
        # routed experts plus a shared expert gated per token; attention biases
        cfg = preset("tiny-qwen2-moe", hidden_size=a.hidden, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
                     vocab_size=4096, num_hidden_layers=3, dtype="bfloat16", num_experts=16, num_experts_per_tok=4,
                     moe_intermediate_size=256, shared_expert_intermediate_size=512)
    elif a.model == "gpt-oss":
        cfg = preset("tiny-gpt-oss", hidden_size=a.hidden, intermediate_size=256, moe_intermediate_size=256,
                     num_attention_heads=8, num_key_value_heads=2, head_dim=64, vocab_size=4096, num_hidden_layers=2,
                     sliding_window=24, dtype="bfloat16")
    else:
        cfg = preset("tiny-qwen3-moe", hidden_size=a.hidden, num_attention_heads=8, num_key_value_heads=2,
                     head_dim=128, vocab_size=4096, num_hidden_layers=3, dtype="bfloat16", num_experts=16,
                     num_experts_per_tok=4, moe_intermediate_size=256)
    comm = TPComm(rank, world, dev, fused=a.backend == "fused")
    drv = TorchDriver(cfg, dev, num_pages=64, page_size=16, max_requests=8, max_tokens=512,
                      par=ParallelContext(world, rank, comm, ep=a.model == "moe-ep"), seed=0)
    comm.attach(drv)
    # one-shot small all-reduce against NCCL, three sizes, twice each (buffer parity)
    ar_ok = True
    if comm.fused:
        for n in (8, 4096, 200 * 1024):
            for rep in range(2):
                g = torch.Generator(device="cpu").manual_seed(100 * rank + n + rep)
                x = torch.randn(n, generator=g).to(torch.bfloat16).to(dev)
                want = x.float().clone()
                dist.all_reduce(want)
                got = comm.all_reduce(x.clone())
                torch.cuda.synchronize()
                ar_ok &= bool((got.float() - want).abs().max() <= 0.02 * want.abs().max() + 1e-3)
    if rank != 0:
        comm.follower_loop(drv)
        comm.close()
        os._exit(0)
    ref = TorchDriver(cfg, dev, num_pages=64, page_size=16, max_requests=8, max_tokens=512, seed=0)
    rng = np.random.default_rng(0)
    lens = [37, 5, 64]
    prompts = [rng.integers(0, cfg.vocab_size, n).tolist() for n in lens]
    pages, nxt = [], 0
    for n in lens:
        k = -(-(n + 8) // 16)
        pages.append(list(range(nxt, nxt + k)))
        nxt += k
    raw = SamplerSpec(SamplerKind.RAW_LOGITS)
    report = {"backend": a.backend, "model": a.model, "world": world, "checks": []}

    def compare(tag, r_tp, r_ref):
        for i, (x, y) in enumerate(zip(r_tp.slots, r_ref.slots)):
            g = np.frombuffer(x.logits, dtype=np.float32)
            w = np.frombuffer(y.logits, dtype=np.float32)
            cos = float(np.dot(g, w) / (np.linalg.norm(g) * np.linalg.norm(w) + 1e-12))
            top5 = len(set(np.argsort(g)[-5:]) & set(np.argsort(w)[-5:]))
            report["checks"].append({"tag": tag, "req": i, "cos": cos, "max_abs": float(np.abs(g - w).max()),
                                     "argmax_equal": bool(g.argmax() == w.argmax()), "top5_overlap": top5})

    items = lambda: [PendingRequest(i, p, list(range(len(p))), pg, 0, [(len(p) - 1, raw)])
                     for i, (p, pg) in enumerate(zip(prompts, pages))]
    r_tp = drv.fire_batch(fold(items(), 16))
    r_ref = ref.fire_batch(fold(items(), 16))
    compare("prefill", r_tp, r_ref)
    toks = [int(np.frombuffer(s.logits, dtype=np.float32).argmax()) for s in r_ref.slots]
    for step in range(2):
        mk = lambda: [PendingRequest(i, [t], [len(p) + step], pg, len(p) + step, [(0, raw)])
                      for i, (t, p, pg) in enumerate(zip(toks, prompts, pages))]
        r_tp = drv.fire_batch(fold(mk(), 16))
        r_ref = ref.fire_batch(fold(mk(), 16))
        compare(f"decode{step}", r_tp, r_ref)
        toks = [int(np.frombuffer(s.logits, dtype=np.float32).argmax()) for s in r_ref.slots]
    # vocabulary-sharded sampler: one more decode step with a raw-logits probe and five token samplers
    # per request on the same row; the tokens must equal the single-GPU sampler's on the gathered logits
    from pie_b200 import ops
    from pie_b200.driver.schema import position_seed
    samplers = [SamplerSpec.greedy(), SamplerSpec(SamplerKind.TOP_P, 1.0, 0, 0.9, 0.0, 11),
                SamplerSpec(SamplerKind.TOP_K, 0.8, 50, 1.0, 0.0, 12), SamplerSpec(SamplerKind.MIN_P, 1.0, 0, 1.0, 0.02, 13),
                SamplerSpec(SamplerKind.MULTINOMIAL, 1.3, 0, 1.0, 0.0, 14)]
    step = 2
    mk = [PendingRequest(i, [t], [len(p) + step], pg, len(p) + step, [(0, raw)] + [(0, sp) for sp in samplers])
          for i, (t, p, pg) in enumerate(zip(toks, prompts, pages))]
    r_tp = drv.fire_batch(fold(mk, 16))
    sample_ok = True
    per = 1 + len(samplers)
    for i in range(len(prompts)):
        lg = torch.from_numpy(np.frombuffer(r_tp.slots[i * per].logits, dtype=np.float32).copy()).to(dev)
        lg = lg.to(torch.bfloat16).reshape(1, -1).contiguous()
        for j, sp in enumerate(samplers):
            f = lambda v, dt: torch.tensor([v], dtype=dt, device=dev)
            want = ops.sample(lg, f(sp.temperature, torch.float32),
                              f(sp.top_k if sp.kind == SamplerKind.TOP_K else 0, torch.int32),
                              f(sp.top_p if sp.kind == SamplerKind.TOP_P else 1.0, torch.float32),
                              f(sp.min_p if sp.kind == SamplerKind.MIN_P else 0.0, torch.float32),
                              f(int(position_seed(sp.seed, len(prompts[i]) + step)) if sp.seed else 1, torch.int64))
            got = r_tp.slots[i * per + 1 + j].token
            if int(want.item()) != got:
                sample_ok = False
                report.setdefault("sample_mismatch", []).append([i, j, int(want.item()), got])
    report["sharded_sampling"] = bool(drv.model.sharded_logits)
    report["sample_ok"] = sample_ok
    comm.stop_followers()
    torch.cuda.synchronize()
    ops.check_kernel_status(dev)
    report["allreduce_small_ok"] = ar_ok
    report["ok"] = ar_ok and sample_ok and all(c["cos"] > 0.995 and c["top5_overlap"] >= 3 for c in report["checks"])
    report["graph_replays"] = drv.stats["graph_replays"]
    print(json.dumps(report), flush=True)
    comm.close()
    os._exit(0)


if __name__ == "__main__":
    main()
