#!/usr/bin/env python
"""Headline benchmark: decode output tokens/s of Llama-3.1-8B-architecture serving (bf16,
random-init weights, synthetic random-token prompts), 512 concurrent text-completion
inferlets, prompts uniform in [128, 2048], 256 output tokens, temperature 1.0 / top-p 0.9,
KV page size 16. With --gpus N > 1 the model runs as ONE tensor-parallel group over the N GPUs
(fused peer-memory kernels: GEMM -> reduce-scatter epilogue, owner reduce + norm + push all-gather,
gated GEMM loads, vocabulary-sharded lm_head with a cross-rank sampler); `--parallelism dp` runs N
independent replicas instead and is labelled as such in the output.

    python bench.py --gpus 1 --steps 64 --warmup 8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 64 --warmup 8

Rank 0 prints ONE JSON line. `value` is device-timed (CUDA events, max over ranks) over
exactly --steps decode steps of the whole 512-request batch; `e2e.value` is the same metric
through the engine's public API (inferlets -> scheduler -> driver) with per-step pinned-host
H2D of the inputs and D2H of the sampled tokens. `--impl reference` reports why the reference
cannot run here. `--impl library` runs the library comparator alone (cuBLAS GEMMs, FlashInfer paged
attention / norms / RoPE / sampling, NCCL all-reduce twice per layer with rank-0 logits, CUDA graphs:
the structure of the reference's CUDA driver, none of this repository's kernels; see
pie_b200/bench/library_arm.py). The default run times that comparator first, on the same GPUs and
the same synthetic contexts, and reports `vs_baseline` = ours / library.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

REFERENCE_UNAVAILABLE = ("pip cannot install the reference (a Rust/C++ workspace without setup.py or "
                         "pyproject.toml); cargo/rustc, wasmtime and the CPM-fetched C++ dependencies are absent offline")


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--config", type=int, default=2, choices=[2, 3, 4, 5, 6],
                    help="2: the headline configuration (this file); 3 Qwen3-32B block-fp8, 4 Qwen3-30B-A3B MoE with "
                         "expert parallelism, 5 agentic fork, 6 GPT-OSS shapes: see pie_b200/bench/configs.py")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "library", "vllm"])
    ap.add_argument("--no-baseline", action="store_true", help="skip the library comparator (vs_baseline stays null)")
    ap.add_argument("--model", default="llama-3.1-8b")
    ap.add_argument("--requests", type=int, default=512)
    ap.add_argument("--prompt-min", type=int, default=128)
    ap.add_argument("--prompt-max", type=int, default=2048)
    ap.add_argument("--out-tokens", type=int, default=256)
    ap.add_argument("--gemm", default="tcgen05", choices=["tcgen05", "cublas"])
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count (marks the run invalid)")
    ap.add_argument("--kv-dtype", default="auto", choices=["auto", "fp8_e4m3"],
                    help="fp8_e4m3: KV pages stored in fp8 with per-(token, head) scales; NOT the named configuration "
                         "(its KV is bf16): the line is marked valid=false")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-per-step", action="store_true", help="skip the inferlet-driven (per-step) e2e variant")
    ap.add_argument("--skip-device", action="store_true")
    ap.add_argument("--max-tokens", type=int, default=16384)
    ap.add_argument("--device-loop", default="pipelined", choices=["pipelined", "staged"],
                    help="pipelined: decode_async with device-fed tokens (all N); staged: inputs pre-staged on the device (N=1)")
    ap.add_argument("--parallelism", default="tp", choices=["dp", "tp"],
                    help="N>1: tp = one tensor-parallel group over all GPUs (default, the named configuration); "
                         "dp = one replica per GPU, the inferlets spread over them")
    ap.add_argument("--tp-backend", default="fused", choices=["fused", "nccl"],
                    help="fused: GEMM epilogue reduce-scatter + push all-gather over peer memory; nccl: GEMM + all-reduce")
    return ap.parse_args()


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    if args.impl == "vllm":
        # the workload served by vLLM (one process; it starts its own tensor-parallel workers for --gpus N)
        if rank == 0:
            from pie_b200.bench import vllm_arm
            vllm_arm.main(["--model", args.model, "--requests", str(args.requests), "--prompt-min", str(args.prompt_min),
                           "--prompt-max", str(args.prompt_max), "--out-tokens", str(args.out_tokens),
                           "--gpus", str(args.gpus)] + (["--layers", str(args.layers)] if args.layers else []))
        return 0
    from pie_b200.bench import configs as _configs
    _configs._hang_dump()
    if args.config != 2:
        from pie_b200.bench import configs
        return configs.main(["--config", str(args.config), "--steps", str(args.steps), "--warmup", str(args.warmup),
                             "--gemm", args.gemm] + (["--layers", str(args.layers)] if args.layers else []))

    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # peer loads/stores only, no NVLS binding
    import torch

    if not torch.cuda.is_available():
        if rank == 0:
            print(json.dumps({"metric": "decode output tokens/s", "value": None, "unavailable": "no CUDA device"}))
        return 0
    from pie_b200.bench import harness
    from pie_b200.driver.executor import TorchDriver
    from pie_b200.driver.schema import SamplerKind, SamplerSpec
    from pie_b200.inferlets import install_all
    from pie_b200.models.config import preset
    from pie_b200.models.transformer import ParallelContext
    from pie_b200.ops import _lib
    from pie_b200.runtime.engine import Engine, EngineConfig

    torch.cuda.set_device(local_rank)
    par = ParallelContext()
    barrier = None
    comm = None
    dp = world > 1 and args.parallelism == "dp"
    if world > 1:
        import torch.distributed as dist
        import datetime
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank),
                                timeout=datetime.timedelta(seconds=180))
        barrier = dist.barrier
        if not dp:
            from pie_b200.parallel.comm import TPComm
            comm = TPComm(rank, world, torch.device("cuda", local_rank), fused=args.tp_backend == "fused")
            par = ParallelContext(world, rank, comm)
    if args.gpus != world and rank == 0:
        print(f"[bench] note: --gpus {args.gpus} but WORLD_SIZE={world}; using {world}", file=sys.stderr)

    overrides = {}
    if args.layers:
        overrides["num_hidden_layers"] = args.layers
    cfg = preset(args.model, **overrides)

    # ---- library comparator: first, so that its memory is back before the engine sizes its KV pool
    baseline = None
    if args.impl == "library" or not args.no_baseline:
        baseline = _library_arm(args, cfg, rank, world, local_rank)
        if args.impl == "library":
            if rank == 0:
                ok = "error" not in baseline
                print(json.dumps({
                    "metric": "decode output tokens/s", "value": baseline.get("tokens_per_s"), "unit": "tokens/s",
                    "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": baseline.get("ms_per_step"),
                    "higher_is_better": True, "scaling": "strong", "vs_baseline": 1.0 if ok else None, "dtype": "bf16",
                    "data": "synthetic random-token contexts (random KV content), random-init N(0,0.02) weights",
                    "impl": "library", "config": {"model": cfg.name, "global_batch": args.requests,
                                                  "seq_len": f"prompts U[{args.prompt_min},{args.prompt_max}] + {args.out_tokens} out",
                                                  "parallelism": f"tp{world}", "kv_page_size": 16,
                                                  "sampler": "temperature 1.0, top-p 0.9", "valid": not args.layers},
                    "detail": baseline}))
            if world > 1:
                _hard_exit(0)
            return 0
    t0 = time.time()
    driver = TorchDriver(cfg, torch.device("cuda", local_rank), page_size=16, max_requests=args.requests,
                         max_tokens=args.max_tokens, par=par, gemm_backend=args.gemm, kv_dtype=args.kv_dtype)
    if comm is not None:
        comm.attach(driver)
    driver.precapture_graphs()      # start-up work, as in a serving process: no fire pays for a graph capture
    torch.cuda.synchronize()
    t_init = time.time() - t0
    prompts = harness.make_prompts(args.requests, args.prompt_min, args.prompt_max, cfg.vocab_size, seed=1)
    if dp:
        prompts = prompts[rank::world]      # every replica serves its share of the same 512 inferlets
    sampler = SamplerSpec(SamplerKind.TOP_P, temperature=1.0, top_p=0.9)
    sampler_args = {"temperature": 1.0, "top_p": 0.9}

    if comm is not None and rank != 0:
        comm.follower_loop(driver)      # serves every fire rank 0 publishes, both phases
        comm.close()
        _hard_exit(0)

    e2e = None
    if not args.skip_e2e:
        eng = Engine(EngineConfig(batch_policy="adaptive", speculation_depth=1))
        from pie_b200.runtime.tokenizer import ByteTokenizer
        eng.add_model(cfg.name, driver, tokenizer=ByteTokenizer(cfg.vocab_size))   # byte-level ids for the constrained variant
        install_all(eng)
        before = _lib.LAUNCHES
        e2e = harness.run_engine_workload(eng, cfg.name, prompts, args.out_tokens, sampler_args,
                                          window_skip=args.warmup, window_steps=args.steps)
        e2e["launcher_calls"] = _lib.LAUNCHES - before
        if not args.skip_per_step:
            # the programmable path: every inferlet drives its own loop, one forward-pass.execute per
            # token (what constraints, custom speculators and probes use); one in sixteen of the inferlets also
            # decode under a JSON-schema grammar whose vocabulary mask is applied on the device
            schema = {"type": "object", "required": ["a"], "properties": {"a": {"type": "array", "items": {"type": "integer"}}}}
            n_ps = min(len(prompts), 512)
            ps = harness.run_engine_workload(
                eng, cfg.name, prompts[:n_ps], 24, sampler_args, window_skip=3, window_steps=12,
                extra_args=lambda i: {"per_step": True, **({"json_schema": schema} if i % 16 == 0 else {})})
            e2e["per_step"] = {"ms_per_step": ps.get("window_ms_per_step"), "value": ps.get("window_tokens_per_s"),
                               "unit": "tokens/s", "inferlets": n_ps, "constrained_inferlets": (n_ps + 15) // 16,
                               "out_tokens": 24, "workload_tokens_per_s": ps["workload_tokens_per_s"]}
        # keep the driver alive for the device-only phase
        for s in eng.model(cfg.name).schedulers:
            s.shutdown()
        eng.models.clear()
        eng.shutdown()

    dev = None
    clocks = None
    if not args.skip_device:
        sampler_clk = harness.ClockSampler(local_rank).start()
        if args.device_loop == "staged" and world == 1:
            dev = harness.run_device_decode(driver, prompts, args.out_tokens, sampler, args.warmup, args.steps)
        else:
            dev = harness.run_pipelined_decode(driver, prompts, args.out_tokens, sampler, args.warmup,
                                               args.steps, comm=comm, barrier=barrier if dp else None)
        clocks = sampler_clk.stop()
    if comm is not None:
        comm.stop_followers()
        comm.close()

    n_req = args.requests
    h2d = d2h = None
    if e2e is not None:
        # per decode fire: the fixed slab segment + the page table, copied from pinned memory
        o, n = driver.slab.offsets["tile_qstart"]
        avg_pages = sum(-(-(len(p) + args.out_tokens // 2) // 16) for p in prompts)
        h2d = (o + n) * 4 + avg_pages * 4
        d2h = len(prompts) * 4
    launches = (driver.launches_per_decode_step(dev["rb"]) * args.steps) if dev else 0
    if dp:
        # whole-job numbers: the slowest replica sets the step time, throughputs and bytes add up.
        # One fixed-size vector per reduction so that every rank issues the same collectives.
        def g(d, key):
            v = (d or {}).get(key)
            return float(v) if v is not None else 0.0
        mx = torch.tensor([g(dev, "ms_per_step"), g(e2e, "window_ms_per_step"), g(e2e, "p50_ttft_s"),
                           g(e2e, "p50_itl_s"), g(e2e, "wall_s"), -g(clocks, "sm_mhz")],
                          device="cuda", dtype=torch.float64)
        sm = torch.tensor([g(dev, "prefill_tokens_per_s"), float(launches), g(e2e, "workload_tokens_per_s"),
                           g(e2e, "fires"), float(h2d or 0), float(d2h or 0)], device="cuda", dtype=torch.float64)
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        mx, sm = mx.tolist(), sm.tolist()
        if rank != 0:
            _hard_exit(0)
        if dev:
            dev["ms_per_step"] = mx[0]
            dev["tokens_per_s"] = n_req / (mx[0] / 1e3) if mx[0] else None
            dev["prefill_tokens_per_s"] = sm[0]
            launches = int(sm[1])
            if clocks:
                clocks["sm_mhz"] = -mx[5]          # slowest GPU's median clock
        if e2e is not None:
            e2e["window_ms_per_step"] = mx[1] or None
            e2e["window_tokens_per_s"] = n_req / (mx[1] / 1e3) if mx[1] else None
            e2e["p50_ttft_s"], e2e["p50_itl_s"], e2e["wall_s"] = mx[2], mx[3], mx[4]
            e2e["workload_tokens_per_s"], e2e["fires"] = sm[2], int(sm[3])
            h2d, d2h = int(sm[4]), int(sm[5])
    value = dev["tokens_per_s"] if dev else None
    vs = None
    if baseline and baseline.get("tokens_per_s") and value:
        vs = value / baseline["tokens_per_s"]
    line = {
        "metric": "decode output tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev["ms_per_step"] if dev else None,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": vs, "dtype": "bf16",
        "data": "synthetic random-token prompts, random-init N(0,0.02) weights",
        "impl": "ours",
        # what vs_baseline divides by: the library comparator timed in this same run (the reference
        # itself cannot be built here and publishes no number for this configuration)
        "baseline": baseline,
        "config": {"model": cfg.name, "global_batch": n_req, "seq_len": f"prompts U[{args.prompt_min},{args.prompt_max}] + {args.out_tokens} out",
                   "parallelism": (f"dp{world}" if dp else f"tp{world}"),
                   "tp_backend": args.tp_backend if (world > 1 and not dp) else None, "kv_page_size": 16, "sampler": "temperature 1.0, top-p 0.9",
                   "gemm": args.gemm, "layers": cfg.num_hidden_layers, "kv_dtype": "bf16" if args.kv_dtype == "auto" else args.kv_dtype,
                   "l2": "working set per step (weights 16 GB + KV > 60 GB) exceeds the 126 MB L2; no flush needed",
                   "valid": not args.layers and args.kv_dtype == "auto"},
        "clocks": clocks,
        "gpu_launches": launches,
        "prefill_tokens_per_s": dev["prefill_tokens_per_s"] if dev else None,
        "init_s": t_init,
    }
    if e2e is not None:
        line["e2e"] = {"value": e2e.get("window_tokens_per_s"), "unit": "tokens/s",
                       "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                       "ms_per_step": e2e.get("window_ms_per_step"),
                       "workload_tokens_per_s": e2e["workload_tokens_per_s"],
                       "p50_ttft_s": e2e["p50_ttft_s"], "p50_itl_s": e2e["p50_itl_s"],
                       "wall_s": e2e["wall_s"], "fires": e2e["fires"],
                       "requests_per_fire": e2e.get("window_requests_per_fire"),
                       "steps_used": e2e.get("window_steps_used"),
                       # same metric with every inferlet driving its own decode loop (one execute per token)
                       "per_step": e2e.get("per_step")}
    print(json.dumps(line))
    if world > 1:
        _hard_exit(0)
    return 0


def _library_arm(args, cfg, rank: int, world: int, local_rank: int) -> dict:
    """Time the library comparator on this run's GPUs and contexts; every rank calls it. Failures are
    reported, not raised: the headline number does not depend on the comparator."""
    import gc

    import torch
    from pie_b200.bench import harness, library_arm
    cache = library_arm.configure_cache()
    if not os.path.isdir(os.path.join(cache, ".cache", "flashinfer")) and os.environ.get("PIE_LIBRARY_ARM_JIT") != "1":
        return {"impl": "library", "error": "FlashInfer kernel cache not prebuilt (python -m pie_b200.bench.library_arm "
                                            "--prebuild); set PIE_LIBRARY_ARM_JIT=1 to compile during the run"}
    lens = [len(p) for p in harness.make_prompts(args.requests, args.prompt_min, args.prompt_max, cfg.vocab_size, seed=1)]
    try:
        out = library_arm.run(cfg, lens, args.out_tokens, args.warmup, args.steps, rank, world,
                              torch.device("cuda", local_rank))
    except Exception as e:  # noqa: BLE001
        out = {"impl": "library", "error": f"{type(e).__name__}: {e}"[:300]}
    gc.collect()
    torch.cuda.empty_cache()
    return out


def _hard_exit(code: int) -> None:
    """Leave without tearing down NCCL communicators that CUDA graphs still reference (that
    teardown can block); everything this process owns dies with it."""
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(code)


if __name__ == "__main__":
    sys.exit(main())
