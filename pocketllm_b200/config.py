"""One typed configuration object for a deployment: model, parallel layout, caches, speculative decoding and
serving, filled from a JSON / YAML file, then environment variables, then command-line overrides.

The reference spreads these choices over about 330 environment variables plus argparse flags and shell-script
profiles (`SERVING_PROFILE=safe1|latency2|throughput4`, scripts/run_openai_server.sh:11-29); here the
environment surface is small and explicit: `POCKET_<SECTION>_<FIELD>` for any field below, nothing else.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field, fields
from pathlib import Path
from typing import Any


@dataclass
class ModelConfig:
    path: str = ""
    format: str = "auto"                 # auto | safetensors | gguf
    family: str = "auto"                 # auto | qwen_hybrid | deepseek_v4 | minimax-m2 | glm-dsa
    tokenizer: str = ""                  # directory with tokenizer.json, a GGUF file, or "chars"
    chat_format: str = "auto"            # auto | qwen | dsv4 | glm | minimax
    max_context: int = 4096


@dataclass
class ParallelConfig:
    world: int = 1
    policy: str = "tp"                   # replicated | tp | layer_pp
    peer_allreduce: bool = True          # peer-memory collectives (NCCL otherwise)
    comm_timeout_us: int = 2_000_000


@dataclass
class CacheConfig:
    prefill_chunk: int = 512
    prefix_cache: bool = False
    prefix_block: int = 256
    prefix_max_snapshots: int = 8
    cuda_graph: bool = True
    decode_splits: int = 8


@dataclass
class SpeculativeConfig:
    mode: str = "off"                    # off | ngram | mtp (the checkpoint's multi-token predictor) | dspark (DSV4 block drafter)
    draft_len: int = 4
    gate: bool = True


@dataclass
class ServingConfig:
    host: str = "127.0.0.1"
    port: int = 8000
    model_name: str = "pocketllm-b200"
    max_queue: int = 64
    max_tokens_default: int = 512
    native: bool = False                 # serve from the C++ front end (`pocket_engine --serve`)


PROFILES: dict[str, dict[str, dict[str, Any]]] = {
    # one request at a time, conservative memory use
    "safe1": {"serving": {"max_queue": 1}, "cache": {"prefill_chunk": 256}, "speculative": {"mode": "off"}},
    # lowest latency for one or two users: speculative decoding on, small prefill chunks so that decode is not starved
    "latency2": {"serving": {"max_queue": 2}, "cache": {"prefill_chunk": 256}, "speculative": {"mode": "ngram", "draft_len": 4}},
    # throughput: long prefill chunks, deeper queue
    "throughput4": {"serving": {"max_queue": 64}, "cache": {"prefill_chunk": 1024, "prefix_cache": True}, "speculative": {"mode": "off"}},
}


@dataclass
class Config:
    model: ModelConfig = field(default_factory=ModelConfig)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    cache: CacheConfig = field(default_factory=CacheConfig)
    speculative: SpeculativeConfig = field(default_factory=SpeculativeConfig)
    serving: ServingConfig = field(default_factory=ServingConfig)

    # -- construction ------------------------------------------------------------------
    @classmethod
    def load(cls, path: str | Path | None = None, *, profile: str | None = None, env: dict[str, str] | None = None,
             overrides: list[str] | None = None) -> "Config":
        """Precedence (lowest to highest): defaults, profile, file, environment, `section.field=value` overrides."""
        cfg = cls()
        if profile:
            if profile not in PROFILES:
                raise ValueError(f"unknown serving profile {profile!r}; known: {sorted(PROFILES)}")
            cfg.update(PROFILES[profile])
        if path:
            text = Path(path).read_text()
            if str(path).endswith((".yaml", ".yml")):
                import yaml
                data = yaml.safe_load(text) or {}
            else:
                data = json.loads(text)
            cfg.update(data)
        cfg.update_from_env(os.environ if env is None else env)
        for item in overrides or []:
            key, sep, value = item.partition("=")
            if not sep or "." not in key:
                raise ValueError(f"override {item!r} is not of the form section.field=value")
            section, name = key.split(".", 1)
            cfg.set(section, name, value)
        cfg.validate()
        return cfg

    def update(self, data: dict[str, dict[str, Any]]) -> None:
        for section, values in data.items():
            if not hasattr(self, section):
                raise ValueError(f"unknown config section {section!r}")
            for name, value in (values or {}).items():
                self.set(section, name, value)

    def update_from_env(self, env) -> None:
        for section in (f.name for f in fields(self)):
            for f in fields(getattr(self, section)):
                key = f"POCKET_{section.upper()}_{f.name.upper()}"
                if key in env:
                    self.set(section, f.name, env[key])

    def set(self, section: str, name: str, value: Any) -> None:
        obj = getattr(self, section, None)
        if obj is None or name not in {f.name for f in fields(obj)}:
            raise ValueError(f"unknown config field {section}.{name}")
        current = getattr(obj, name)
        if isinstance(value, str) and not isinstance(current, str):
            if isinstance(current, bool):
                if value.lower() not in ("1", "0", "true", "false", "yes", "no", "on", "off"):
                    raise ValueError(f"{section}.{name}: {value!r} is not a boolean")
                value = value.lower() in ("1", "true", "yes", "on")
            else:
                value = type(current)(value)
        if isinstance(current, bool) != isinstance(value, bool) or (not isinstance(value, type(current)) and not (isinstance(current, float) and isinstance(value, int))):
            raise ValueError(f"{section}.{name}: expected {type(current).__name__}, got {type(value).__name__}")
        setattr(obj, name, value)

    def validate(self) -> None:
        p, c, s = self.parallel, self.cache, self.speculative
        if not 1 <= p.world <= 8:
            raise ValueError("parallel.world must be between 1 and 8 (one NVSwitch node)")
        if p.policy not in ("replicated", "tp", "layer_pp"):
            raise ValueError(f"parallel.policy {p.policy!r} is not one of replicated, tp, layer_pp")
        if s.mode not in ("off", "ngram", "mtp", "dspark") or not 1 <= s.draft_len <= 7:
            raise ValueError("speculative.mode must be off | ngram | mtp | dspark and draft_len between 1 and 7")
        if p.policy == "layer_pp" and s.mode in ("mtp", "dspark"):
            raise ValueError("MTP / DSpark drafting needs the last layers' hidden states on every rank: not available with layer_pp")
        if s.mode == "dspark" and self.model.family not in ("auto", "deepseek_v4"):
            raise ValueError("speculative.mode dspark is the DeepSeek-V4 block drafter; the Qwen hybrid uses mtp")
        if c.prefill_chunk < 8 or self.model.max_context < c.prefill_chunk:
            raise ValueError("cache.prefill_chunk must be at least 8 and at most model.max_context")

    def native_engine_args(self, rank: int = 0) -> list[str]:
        """Flags of the native CLI (`pocket_engine`) that realise this configuration for tensor-parallel rank `rank`:
        what `serving.native` launches, and the one place where config names meet flag names."""
        m, p, c, s, v = self.model, self.parallel, self.cache, self.speculative, self.serving
        if p.policy != "tp" and p.world > 1:
            raise ValueError("the native engine shards by tensor parallelism only")
        args = ["--ckpt", m.path, "--max-context", str(m.max_context), "--prefill-chunk-tokens", str(c.prefill_chunk),
                "--tp-world", str(p.world), "--tp-rank", str(rank)]
        if not c.cuda_graph:
            args.append("--no-cuda-graph")
        if s.mode == "mtp":
            args += ["--qwen-mtp-tokens", str(s.draft_len)]
        elif s.mode != "off":
            raise ValueError(f"the native engine drafts with the checkpoint's multi-token predictor only (speculative.mode {s.mode!r})")
        if v.native:
            args += ["--serve", "--host", v.host, "--port", str(v.port), "--model-name", v.model_name]
            if m.tokenizer:
                args += ["--tokenizer", m.tokenizer if m.tokenizer == "chars" or ":" in m.tokenizer
                         else ("gguf:" if m.tokenizer.endswith(".gguf") else "hf:") + m.tokenizer]
            if m.chat_format != "auto":
                args += ["--chat-format", m.chat_format]
        return args

    def to_dict(self) -> dict:
        return asdict(self)

    def dump(self) -> str:
        return json.dumps(self.to_dict(), indent=2)
