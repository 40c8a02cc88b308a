"""Engine configuration: a TOML file with [server], [auth], [telemetry], [runtime] and one or
more [[model]] tables (each with optional [model.scheduler] and [model.driver]). Unknown keys
are rejected. Drivers advertise capacity themselves: batch sizes and page counts are not
configurable, only the memory fraction and the KV page size are.

Counterpart of server/src/config.rs:25-88 (sections), :198-220 (runtime), :320-336 (scheduler),
:423-441 (driver), :556-590 (rejected capacity keys) and serve/topology.rs:32-46 (DP x TP groups).
"""
from __future__ import annotations

import os
import tomllib
from dataclasses import asdict, dataclass, field, fields
from pathlib import Path
from typing import List, Optional


class ConfigError(ValueError):
    pass


@dataclass
class ServerConfig:
    host: str = "127.0.0.1"
    port: int = 8080
    max_message_bytes: int = 64 << 20
    # Uploaded programs are Python source that runs inside the engine process (no sandbox): only
    # switch this on for clients you would give a shell on the machine.
    allow_program_upload: bool = False


@dataclass
class AuthConfig:
    enabled: bool = True
    authorized_users: str = "~/.pie_b200/authorized_users.json"


@dataclass
class TelemetryConfig:
    enabled: bool = False
    endpoint: str = ""
    service_name: str = "pie_b200"
    log_dir: str = ""


@dataclass
class RuntimeConfig:
    max_concurrent_processes: int = 4096
    request_timeout_secs: float = 120.0
    default_token_budget: Optional[int] = None
    default_endowment_pages: int = 64
    admission_oversubscription_factor: float = 4.0
    restore_pause_at_utilization: float = 0.85
    program_dir: str = "~/.pie_b200/programs"
    registry_url: str = ""                  # programs that are not installed are fetched from here on first use
    allow_network: List[str] = field(default_factory=list)     # CIDR[:port] allow-list for inferlets
    allow_fs: bool = True                                      # per-process scratch directory


@dataclass
class SchedulerConfig:
    batch_policy: str = "adaptive"        # adaptive | eager | greedy
    speculation_depth: int = 1
    system_spec_tokens: int = 0           # > 0: the runtime drafts this many tokens per generator step (prompt look-up)


@dataclass
class DriverConfig:
    type: str = "cuda_native"             # cuda_native | cpu | dummy
    device: List[int] = field(default_factory=lambda: [0])
    tensor_parallel_size: int = 1
    expert_parallel: bool = False
    gpu_mem_utilization: float = 0.9
    kv_page_size: int = 16
    swap_pool_gb: float = 0.0
    cuda_graphs: bool = True
    gemm: str = "tcgen05"
    tp_backend: str = "fused"
    memory_profile: str = ""              # "" = built-in limits; auto | latency | balanced | throughput | capacity
    kv_dtype: str = "auto"                # KV pages: auto / bf16 | fp8_e4m3 (one byte per element + a scale per token and head)
    vision: str = ""                      # "" = text only | "checkpoint" (the `visual.*` tower of [model] path) |
                                          # a preset of models.vision with random weights (e.g. "tiny-vit")
    audio: str = ""                       # the same for the audio encoder (`audio_tower.*`; preset e.g. "tiny-audio")
    ipc: str = "direct"                   # runtime -> driver: direct call | inproc (queue + service thread) |
                                          # latency (polled ring) | shmem (driver in a process of its own)


@dataclass
class ModelSection:
    name: str = ""
    path: str = ""                        # checkpoint directory; empty = random-init preset
    preset: str = ""
    instruct: str = ""
    scheduler: SchedulerConfig = field(default_factory=SchedulerConfig)
    driver: DriverConfig = field(default_factory=DriverConfig)


@dataclass
class Config:
    server: ServerConfig = field(default_factory=ServerConfig)
    auth: AuthConfig = field(default_factory=AuthConfig)
    telemetry: TelemetryConfig = field(default_factory=TelemetryConfig)
    runtime: RuntimeConfig = field(default_factory=RuntimeConfig)
    model: List[ModelSection] = field(default_factory=list)


_CAPACITY_KEYS = {"max_batch_size", "max_num_seqs", "num_pages", "total_pages", "max_forward_tokens",
                  "max_forward_requests", "max_num_batched_tokens"}


def _build(cls, data: dict, where: str):
    if not isinstance(data, dict):
        raise ConfigError(f"[{where}] must be a table")
    known = {f.name: f for f in fields(cls)}
    for k in data:
        if k in _CAPACITY_KEYS:
            raise ConfigError(f"[{where}] {k}: capacity is planned by the driver and cannot be configured")
        if k not in known:
            raise ConfigError(f"[{where}] unknown key {k!r}")
    kw = {}
    for k, v in data.items():
        sub = {"scheduler": SchedulerConfig, "driver": DriverConfig}.get(k) if cls is ModelSection else None
        kw[k] = _build(sub, v, f"{where}.{k}") if sub else v
    return cls(**kw)


def parse(text: str, driver_defaults: Optional[dict] = None) -> Config:
    raw = tomllib.loads(text)
    if driver_defaults:
        models = raw.get("model", [])
        for m in ([models] if isinstance(models, dict) else models):
            d = m.setdefault("driver", {}) if isinstance(m, dict) else {}
            for k, v in driver_defaults.get(d.get("type", DriverConfig.type), {}).items():
                d.setdefault(k, v)
    sections = {"server": ServerConfig, "auth": AuthConfig, "telemetry": TelemetryConfig, "runtime": RuntimeConfig}
    for k in raw:
        if k not in sections and k != "model":
            raise ConfigError(f"unknown section [{k}]")
    cfg = Config(**{k: _build(c, raw.get(k, {}), k) for k, c in sections.items()})
    models = raw.get("model", [])
    if isinstance(models, dict):
        models = [models]
    cfg.model = [_build(ModelSection, m, f"model[{i}]") for i, m in enumerate(models)]
    validate(cfg)
    return cfg


def validate(cfg: Config) -> None:
    used = {}
    for m in cfg.model:
        if not m.name:
            raise ConfigError("every [[model]] needs a name")
        if not m.path and not m.preset:
            raise ConfigError(f"model {m.name}: give a checkpoint `path` or a `preset`")
        if m.scheduler.batch_policy not in ("adaptive", "eager", "greedy"):
            raise ConfigError(f"model {m.name}: unknown batch_policy {m.scheduler.batch_policy!r}")
        d = m.driver
        if d.type not in ("cuda_native", "cpu", "dummy"):
            raise ConfigError(f"model {m.name}: unknown driver type {d.type!r}")
        if d.kv_page_size % 16:
            raise ConfigError(f"model {m.name}: kv_page_size must be a multiple of 16")
        if d.kv_dtype not in ("auto", "bf16", "fp8_e4m3"):
            raise ConfigError(f"model {m.name}: unknown kv_dtype {d.kv_dtype!r} (auto | bf16 | fp8_e4m3)")
        if d.kv_dtype == "fp8_e4m3" and d.type != "cuda_native":
            raise ConfigError(f"model {m.name}: fp8 KV pages need the cuda_native driver")
        if not 0.05 <= d.gpu_mem_utilization <= 0.98:
            raise ConfigError(f"model {m.name}: gpu_mem_utilization out of range")
        if d.type == "cuda_native":
            calculate_topology(d.device, d.tensor_parallel_size)
            for dev in d.device:
                if dev in used:
                    raise ConfigError(f"device {dev} is assigned to both {used[dev]} and {m.name}")
                used[dev] = m.name
    names = [m.name for m in cfg.model]
    if len(set(names)) != len(names):
        raise ConfigError("model names must be unique")


def calculate_topology(devices: List[int], tp_size: int) -> List[List[int]]:
    """Split the device list into data-parallel groups of `tp_size` tensor-parallel ranks."""
    if tp_size < 1 or not devices:
        raise ConfigError("need at least one device and tensor_parallel_size >= 1")
    if len(set(devices)) != len(devices):
        raise ConfigError("duplicate device ids")
    if len(devices) % tp_size:
        raise ConfigError(f"{len(devices)} devices cannot form groups of {tp_size}")
    return [devices[i:i + tp_size] for i in range(0, len(devices), tp_size)]


def _fmt(v) -> str:
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, str):
        return '"' + v.replace("\\", "\\\\").replace('"', '\\"') + '"'
    if isinstance(v, list):
        return "[" + ", ".join(_fmt(x) for x in v) + "]"
    return repr(v)


def dumps(cfg: Config) -> str:
    out = []
    for sec in ("server", "auth", "telemetry", "runtime"):
        out.append(f"[{sec}]")
        out += [f"{k} = {_fmt(v)}" for k, v in asdict(getattr(cfg, sec)).items() if v is not None]
        out.append("")
    for m in cfg.model:
        out.append("[[model]]")
        out += [f"{k} = {_fmt(v)}" for k, v in asdict(m).items() if k not in ("scheduler", "driver") and v != ""]
        out.append("[model.scheduler]")
        out += [f"{k} = {_fmt(v)}" for k, v in asdict(m.scheduler).items()]
        out.append("[model.driver]")
        out += [f"{k} = {_fmt(v)}" for k, v in asdict(m.driver).items()]
        out.append("")
    return "\n".join(out)


def default_path() -> Path:
    return Path(os.environ.get("PIE_B200_CONFIG", "~/.pie_b200/config.toml")).expanduser()


def load(path=None) -> Config:
    p = Path(path).expanduser() if path else default_path()
    return parse(p.read_text(), driver_defaults=_driver_defaults())


def _driver_defaults() -> dict:
    """Knobs persisted by `pie driver <type> set` (drivers.toml beside the default config)."""
    p = default_path().parent / "drivers.toml"
    return tomllib.loads(p.read_text()) if p.exists() else {}


def default_config() -> Config:
    cfg = Config()
    cfg.model = [ModelSection(name="llama-3.1-8b", preset="llama-3.1-8b")]
    return cfg


def set_key(cfg: Config, dotted: str, value: str) -> None:
    """`pie config set server.port 9000` / `model.0.driver.kv_page_size 32`."""
    parts = dotted.split(".")
    obj = cfg
    for p in parts[:-1]:
        obj = obj[int(p)] if isinstance(obj, list) else getattr(obj, p)
    cur = getattr(obj, parts[-1])
    if isinstance(cur, bool):
        val = value.lower() in ("1", "true", "yes")
    elif isinstance(cur, int):
        val = int(value)
    elif isinstance(cur, float):
        val = float(value)
    elif isinstance(cur, list):
        val = [int(x) if x.strip().lstrip("-").isdigit() else x.strip() for x in value.strip("[]").split(",") if x.strip()]
    else:
        val = value
    setattr(obj, parts[-1], val)
    validate(cfg)
