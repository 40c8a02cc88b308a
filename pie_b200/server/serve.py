"""Engine start-up from a configuration: build the drivers of every [[model]] (one per
data-parallel group), register tokenizer / instruct template, install the bundled inferlets,
bind the WebSocket server, supervise. Counterpart of server/src/serve.rs:272-418 (start_engine),
serve/topology.rs (DP x TP), serve/lifecycle.rs (watchdog) and bootstrap_translate.rs.

Tensor parallelism spans processes: start `pie serve` under
`python -m torch.distributed.run --nproc-per-node T ...`; rank 0 runs the engine and the server,
the other ranks serve its fires (`TPComm.follower_loop`).
"""
from __future__ import annotations

import logging
import os
import signal
import threading
from pathlib import Path
from typing import Optional

from ..inferlets import install_all
from ..models.config import ModelConfig, preset
from ..runtime import instruct as instruct_mod
from ..runtime.engine import Engine, EngineConfig
from ..runtime.tokenizer import ByteTokenizer, load_hf_tokenizer
from .auth import Authenticator, UserStore
from .config import Config, ModelSection, calculate_topology
from .server import PieServer

log = logging.getLogger("pie_b200")


def build_drivers(m: ModelSection):
    """Drivers of one model behind the configured channel (`[model.driver] ipc`): the driver objects
    themselves (`direct`), each behind a service thread (`inproc`, `latency`), or one in a process of its
    own reached through shared memory (`shmem`). Returns (drivers, cfg, tokenizer, comm)."""
    ipc = m.driver.ipc
    if ipc == "shmem":
        from dataclasses import asdict
        from ..driver.channel import spawn_driver_process
        cfg, tok = _config_and_tokenizer(m)
        sec = asdict(m)
        sec["driver"]["ipc"] = "direct"
        drv, _proc = spawn_driver_process(f"pie_b200_drv_{os.getpid()}_{m.name}".replace("/", "_"), sec)
        return [drv], cfg, tok, None
    drivers, cfg, tok, comm = _build_drivers_direct(m)
    if ipc in ("inproc", "latency") and comm is None:
        from ..driver.channel import ChannelDriver, make_channel
        drivers = [ChannelDriver(make_channel(drv, ipc), on_shutdown=getattr(drv, "shutdown", None)) for drv in drivers]
    return drivers, cfg, tok, comm


def _config_and_tokenizer(m: ModelSection):
    """What the runtime needs to know of a model whose driver lives elsewhere."""
    tok = None
    if not m.path:
        return (preset(m.preset) if m.preset else ModelConfig(name=m.name)), tok
    mp = Path(m.path)
    ggufs = [mp] if mp.suffix == ".gguf" else ([] if list(mp.glob("*.safetensors")) else sorted(mp.glob("*.gguf")))
    if ggufs:
        from ..models.gguf import GGUFReader
        from ..runtime.tokenizer import load_gguf_tokenizer
        rd = GGUFReader(ggufs[0])
        cfg = rd.config()
        if rd.meta.get("tokenizer.ggml.tokens") and rd.meta.get("tokenizer.ggml.model", "gpt2") == "gpt2":
            tok = load_gguf_tokenizer(rd)
    else:
        cfg = ModelConfig.from_path(m.path)
    cfg.name = m.name
    if tok is None and mp.is_dir() and (mp / "tokenizer.json").exists():
        tok = load_hf_tokenizer(m.path)
    return cfg, tok


def _vision_encoder(m: ModelSection, cfg, device, dtype):
    """The model's vision encoder per `[model.driver] vision`, or None for a text-only model."""
    kind = m.driver.vision
    if not kind:
        return None
    import json as _json
    from ..models import vision as V
    if kind == "checkpoint":
        from ..models.loader import SafetensorsReader
        hf = _json.loads((Path(m.path) / "config.json").read_text())
        if (hf.get("vision_config") or {}).get("model_type") == "siglip_vision_model":      # Gemma-3: SigLIP tower + pooling projector
            scfg = V.SiglipConfig.from_hf(hf, llm_hidden=cfg.hidden_size)
            enc = V.SiglipEncoder(scfg, V.load_siglip_weights(SafetensorsReader(m.path), device, dtype))
            enc.delimiters = ("\n\n<start_of_image>", "<end_of_image>\n\n")        # Gemma-3's image span markers
            return enc
        vcfg = V.VisionConfig.from_hf(hf.get("vision_config") or {}, llm_hidden=cfg.hidden_size)
        enc = V.VisionEncoder(vcfg, V.load_vision_weights(SafetensorsReader(m.path), device, dtype))
        enc.delimiters = ("<|vision_start|>", "<|vision_end|>")                        # Qwen-VL's
        return enc
    if kind in V.SIGLIP_PRESETS:
        scfg = V.siglip_preset(kind, hidden_size=cfg.hidden_size)
        return V.SiglipEncoder(scfg, V.random_siglip_weights(scfg, device, dtype))
    vcfg = V.vision_preset(kind, hidden_size=cfg.hidden_size)
    return V.VisionEncoder(vcfg, V.random_vision_weights(vcfg, device, dtype))


def _audio_encoder(m: ModelSection, cfg, device, dtype):
    """The model's audio encoder per `[model.driver] audio`, or None."""
    kind = m.driver.audio
    if not kind:
        return None
    import json as _json
    from ..models import audio as A
    if kind == "checkpoint":
        from ..models.loader import SafetensorsReader
        hf = _json.loads((Path(m.path) / "config.json").read_text())
        acfg = A.AudioConfig.from_hf(hf.get("audio_config") or {}, llm_hidden=cfg.hidden_size)
        enc = A.AudioEncoder(acfg, A.load_audio_weights(SafetensorsReader(m.path), device, dtype))
        enc.delimiters = ("<|audio_bos|>", "<|audio_eos|>")                            # Qwen2-Audio's clip markers
        return enc
    acfg = A.audio_preset(kind, hidden_size=cfg.hidden_size)
    return A.AudioEncoder(acfg, A.random_audio_weights(acfg, device, dtype))


def _build_drivers_direct(m: ModelSection):
    """Drivers of one model: one per data-parallel group. Returns (drivers, cfg, tokenizer, comm)."""
    d = m.driver
    tok = None
    comm = None
    if d.type == "dummy":
        from ..driver.mock import DummyDriver
        cfg = preset(m.preset) if m.preset else ModelConfig(name=m.name)
        return [DummyDriver(vocab=cfg.vocab_size, page_size=d.kv_page_size, total_pages=4096)], cfg, tok, comm
    import torch
    from ..driver.executor import TorchDriver
    from ..models.transformer import ParallelContext
    weights = None
    if m.path:
        from ..models import loader
        mp = Path(m.path)
        ggufs = [mp] if mp.suffix == ".gguf" else ([] if list(mp.glob("*.safetensors")) else sorted(mp.glob("*.gguf")))
        if ggufs:       # one file carries configuration, weights and tokenizer
            from ..models.gguf import GGUFReader
            from ..runtime.tokenizer import load_gguf_tokenizer
            rd = GGUFReader(ggufs[0])
            cfg = rd.config()
            if rd.meta.get("tokenizer.ggml.tokens") and rd.meta.get("tokenizer.ggml.model", "gpt2") == "gpt2":
                tok = load_gguf_tokenizer(rd)
        else:
            cfg = ModelConfig.from_path(m.path)
        cfg.name = m.name
        if tok is None and mp.is_dir() and (mp / "tokenizer.json").exists():
            tok = load_hf_tokenizer(m.path)
    else:
        cfg = preset(m.preset)
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if d.type == "cpu":
        w = None
        if m.path:
            _, w = loader.load_checkpoint(m.path, "cpu", dtype="float32")
            cfg.dtype = "float32"
        return [TorchDriver(cfg, "cpu", weights=w, num_pages=4096, page_size=d.kv_page_size,
                            vision=_vision_encoder(m, cfg, "cpu", torch.float32),
                            audio=_audio_encoder(m, cfg, "cpu", torch.float32))], cfg, tok, comm
    groups = calculate_topology(d.device, d.tensor_parallel_size)
    drivers = []
    if d.tensor_parallel_size > 1:
        if world != d.tensor_parallel_size:
            raise RuntimeError(f"tensor_parallel_size={d.tensor_parallel_size} needs that many ranks "
                               f"(start under torch.distributed.run); WORLD_SIZE is {world}")
        import torch.distributed as dist
        from ..parallel.comm import TPComm
        dev = torch.device("cuda", groups[0][rank])
        torch.cuda.set_device(dev)
        if not dist.is_initialized():
            # a rank that died ends the others' next collective with an error after this long (the control ring
            # notices sooner: PIE_TP_ACK_TIMEOUT_S), instead of the library's ten-minute default
            import datetime
            dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(
                seconds=float(os.environ.get("PIE_TP_COLLECTIVE_TIMEOUT_S", "120"))))
        comm = TPComm(rank, world, dev, fused=d.tp_backend == "fused")
        par = ParallelContext(world, rank, comm, ep=d.expert_parallel)
        if m.path:
            _, weights = loader.load_checkpoint(m.path, dev, world, rank, ep=d.expert_parallel)
        drv = TorchDriver(cfg, dev, weights=weights, page_size=d.kv_page_size, par=par, gemm_backend=d.gemm,
                          use_graphs=d.cuda_graphs, gpu_mem_utilization=d.gpu_mem_utilization,
                          memory_profile=d.memory_profile, kv_dtype=d.kv_dtype)
        comm.attach(drv)
        if d.cuda_graphs and os.environ.get("PIE_PRECAPTURE_GRAPHS", "1") != "0":
            n = drv.precapture_graphs()      # every rank is here: the warm-up forwards run in lock step
            log.info("model %s rank %d: %d decode graphs captured ahead of time", m.name, rank, n)
        return [drv], cfg, tok, comm
    for g in groups:
        dev = torch.device("cuda", g[0])
        if m.path:
            _, weights = loader.load_checkpoint(m.path, dev)
        per_page = cfg.num_hidden_layers * 2 * cfg.num_key_value_heads * d.kv_page_size * cfg.head_dim * 2
        swap = int(d.swap_pool_gb * (1 << 30) // per_page)
        drivers.append(TorchDriver(cfg, dev, weights=weights, page_size=d.kv_page_size, gemm_backend=d.gemm,
                                   use_graphs=d.cuda_graphs, gpu_mem_utilization=d.gpu_mem_utilization,
                                   swap_pages=swap, memory_profile=d.memory_profile, kv_dtype=d.kv_dtype,
                                   vision=_vision_encoder(m, cfg, dev, torch.bfloat16),
                                   audio=_audio_encoder(m, cfg, dev, torch.bfloat16)))
        if d.cuda_graphs and os.environ.get("PIE_PRECAPTURE_GRAPHS", "1") != "0":
            n = drivers[-1].precapture_graphs()
            log.info("model %s on %s: %d decode graphs captured ahead of time", m.name, dev, n)
    return drivers, cfg, tok, comm


class EngineHandle:
    def __init__(self, engine: Engine, server: Optional[PieServer], auth: Authenticator, comms: list):
        self.engine, self.server, self.auth, self.comms = engine, server, auth, comms
        self._stop = threading.Event()

    @property
    def port(self) -> int:
        return self.server.port if self.server else 0

    @property
    def uri(self) -> str:
        return f"ws://{self.server.host}:{self.server.port}"

    def wait_then_shutdown(self) -> None:
        for s in (signal.SIGINT, signal.SIGTERM):
            try:
                signal.signal(s, lambda *_: self._stop.set())
            except ValueError:      # not on the main thread
                pass
        self._stop.wait()
        self.shutdown()

    def shutdown(self) -> None:
        self._stop.set()
        if self.server:
            self.server.stop()
        for c in self.comms:
            c.stop_followers()
        self.engine.shutdown()
        for c in self.comms:
            c.close()


def start_engine(cfg: Config, serve: bool = True, port: Optional[int] = None) -> Optional[EngineHandle]:
    """Returns None on tensor-parallel follower ranks (after they served until STOP)."""
    rt = cfg.runtime
    first = cfg.model[0].scheduler if cfg.model else None
    engine = Engine(EngineConfig(batch_policy=first.batch_policy if first else "adaptive",
                                 speculation_depth=first.speculation_depth if first else 1,
                                 system_spec_tokens=first.system_spec_tokens if first else 0,
                                 max_concurrent_processes=rt.max_concurrent_processes,
                                 request_timeout_secs=rt.request_timeout_secs,
                                 default_token_budget=rt.default_token_budget,
                                 default_endowment_pages=rt.default_endowment_pages,
                                 admission_oversubscription_factor=rt.admission_oversubscription_factor,
                                 fs_policy="scratch" if rt.allow_fs else "none",
                                 network_allow=tuple(rt.allow_network)))
    if cfg.telemetry.enabled:
        from ..runtime import telemetry
        log_dir = Path(cfg.telemetry.log_dir).expanduser() if cfg.telemetry.log_dir else None
        if log_dir:
            log_dir.mkdir(parents=True, exist_ok=True)
        telemetry.configure(True, str(log_dir / "spans.jsonl") if log_dir else None, cfg.telemetry.service_name,
                            cfg.telemetry.endpoint or None)
    comms = []
    for m in cfg.model:
        drivers, mcfg, tok, comm = build_drivers(m)
        if comm is not None:
            comms.append(comm)
            if comm.rank != 0:
                comm.follower_loop(drivers[0])
                comm.close()
                engine.shutdown()
                return None
        if tok is None:
            tok = ByteTokenizer(mcfg.vocab_size)
        ins = instruct_mod.for_arch(m.instruct or (mcfg.model_type if m.path else "plain"))
        engine.add_model(m.name, drivers, tokenizer=tok, instruct=ins)
        log.info("model %s: %d driver(s), %d KV pages", m.name, len(drivers),
                 sum(d.capabilities().total_pages for d in drivers))
    install_all(engine)
    auth = Authenticator(cfg.auth.enabled, UserStore(cfg.auth.authorized_users) if cfg.auth.enabled else None)
    server = None
    if serve:
        server = PieServer(engine, cfg.server.host, cfg.server.port if port is None else port, auth,
                           rt.program_dir, cfg.server.max_message_bytes, registry_url=rt.registry_url,
                           allow_program_upload=cfg.server.allow_program_upload)
        server.start()
    return EngineHandle(engine, server, auth, comms)
