"""The other benchmark configurations (the headline one is bench.py at the repository root; `bench.py
--config N` lands here). On one GPU, or under `python -m torch.distributed.run --nproc-per-node T ...`
as ONE fused tensor-parallel group over T GPUs (config 4: whole experts per rank, i.e. expert
parallelism, with tensor-parallel attention), device-timed as the max over ranks:

    python -m pie_b200.bench.configs --config 3   # Qwen3-32B block-fp8, 4096-token prompts, 512 out, greedy
    python -m pie_b200.bench.configs --config 4   # Qwen3-30B-A3B MoE, prompts U[256,1024], 256 out
    python -m pie_b200.bench.configs --config 5   # agentic fork: 64 agents x 8-way fork x 4 rounds on Llama-3.1-8B
    python -m pie_b200.bench.configs --config 6   # GPT-OSS-20B shapes (not one of the reference's configs), prompts U[256,1024]

`--requests` / `--agents` scale the concurrency down to what one GPU's memory holds; a scaled run
prints "valid": false. One JSON line per run, same timing rules as bench.py (device-timed decode
steps with CUDA events after warm-up, clocks sampled during the timed region).
"""
from __future__ import annotations

import argparse
import json
import time


def _hang_dump() -> None:
    """PIE_HANG_DUMP_S=N: every N seconds write every thread's Python stack to stderr (all ranks), to see
    where a run that stopped making progress is waiting."""
    import os
    n = float(os.environ.get("PIE_HANG_DUMP_S", "0") or 0)
    if n > 0:
        import faulthandler
        faulthandler.dump_traceback_later(n, repeat=True)


def main(argv=None):
    import os
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=int, required=True, choices=[3, 4, 5, 6])
    ap.add_argument("--gpus", type=int, default=0, help="informational; the launcher's WORLD_SIZE decides")
    ap.add_argument("--requests", type=int, default=0)
    ap.add_argument("--agents", type=int, default=64)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--gemm", default="tcgen05", choices=["tcgen05", "cublas"])
    ap.add_argument("--layers", type=int, default=0, help="debug: fewer layers (marks the run invalid)")
    a = ap.parse_args(argv)
    _hang_dump()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    import torch
    from . import harness
    from ..driver.executor import TorchDriver
    from ..driver.schema import SamplerKind, SamplerSpec
    from ..inferlets import install_all
    from ..models.config import preset
    from ..runtime.engine import Engine, EngineConfig

    spec = {3: dict(model="qwen3-32b-fp8", requests=256, pmin=4096, pmax=4096, out=512,
                    sampler=SamplerSpec(SamplerKind.MULTINOMIAL, temperature=0.0), sampler_txt="greedy"),
            4: dict(model="qwen3-30b-a3b", requests=1024, pmin=256, pmax=1024, out=256,
                    sampler=SamplerSpec(SamplerKind.TOP_P, temperature=1.0, top_p=0.9), sampler_txt="temperature 1.0, top-p 0.9"),
            6: dict(model="gpt-oss-20b", requests=256, pmin=256, pmax=1024, out=256,
                    sampler=SamplerSpec(SamplerKind.TOP_P, temperature=1.0, top_p=0.9), sampler_txt="temperature 1.0, top-p 0.9"),
            5: dict(model="llama-3.1-8b", requests=64, pmin=2048, pmax=2048, out=128,
                    sampler=SamplerSpec(SamplerKind.TOP_K, temperature=1.0, top_k=50), sampler_txt="top-k 50, seeded")}[a.config]
    over = {"num_hidden_layers": a.layers} if a.layers else {}
    cfg = preset(spec["model"], **over)
    n_req = a.requests or spec["requests"]
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    par, comm = None, None
    if world > 1:
        import datetime
        import torch.distributed as dist
        from ..models.transformer import ParallelContext
        from ..parallel.comm import TPComm
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=300))
        comm = TPComm(rank, world, dev, fused=True)
        par = ParallelContext(world, rank, comm, ep=a.config == 4)
    drv = TorchDriver(cfg, dev, page_size=16, max_requests=max(n_req, a.agents * 8 if a.config == 5 else n_req),
                      max_tokens=16384, gemm_backend=a.gemm, par=par)
    if comm is not None:
        comm.attach(drv)
    drv.precapture_graphs()
    if comm is not None and rank != 0:
        comm.follower_loop(drv)
        comm.close()
        os._exit(0)
    parallelism = "tp1" if world == 1 else (f"ep{world} experts + tp{world} attention (fused)" if a.config == 4
                                             else f"tp{world} (fused)")
    line = {"config": a.config, "model": cfg.name, "n_gpus": world, "parallelism": parallelism,
            "dtype": "bf16" if cfg.quantization is None else "fp8 weights, bf16 activations",
            "data": "synthetic random-token prompts, random-init weights", "gemm": a.gemm,
            "valid": not a.layers and (n_req == spec["requests"] if a.config != 5 else a.agents == 64)}
    clk = harness.ClockSampler(local).start()
    if a.config == 5:
        eng = Engine(EngineConfig())
        eng.add_model(cfg.name, drv)
        install_all(eng)
        r = harness.run_agentic_fork(eng, cfg.name, a.agents, 2048, 8, 128, 4, cfg.vocab_size)
        eng.shutdown()
        line.update(metric="decode output tokens/s (whole workload, wall clock incl. prefill)", value=r["tokens_per_s"],
                    agents=a.agents, branches=8, rounds=4, **{k: v for k, v in r.items() if k != "tokens_per_s"})
    else:
        prompts = harness.make_prompts(n_req, spec["pmin"], spec["pmax"], cfg.vocab_size, seed=1)
        t0 = time.time()
        d = harness.run_pipelined_decode(drv, prompts, spec["out"], spec["sampler"], a.warmup, a.steps, comm=comm)
        line.update(metric="decode output tokens/s", value=d["tokens_per_s"], ms_per_step=d["ms_per_step"],
                    requests=n_req, steps=a.steps, warmup=a.warmup, prefill_tokens_per_s=d["prefill_tokens_per_s"],
                    sampler=spec["sampler_txt"], wall_s=time.time() - t0)
    line["clocks"] = clk.stop()
    print(json.dumps(line), flush=True)
    if comm is not None:
        comm.stop_followers()
        comm.close()
        os._exit(0)


if __name__ == "__main__":
    main()
