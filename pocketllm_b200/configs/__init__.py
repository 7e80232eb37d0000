"""Model configuration files of the benchmark shapes, one JSON file per family:

* `qwen3_8_27b_fp8.json`  -- hybrid Gated-DeltaNet / GQA decoder, Hugging Face keys (read by `QwenHybridConfig.from_json`
                             and by the native `QwenConfig::from_json`)
* `deepseek_v4_flash.json` -- the keys of the reference's `configs/config.json` (read by `DSV4Config.from_json` and by the
                             native `Dsv4Config`)
* `minimax_m2.json`, `glm_5_dsa.json` -- fields of `MiniMaxM2Config` / `GLMDSAConfig` (the GGUF files carry the same
                             values as metadata; these files size synthetic models and placement reports)
"""
from __future__ import annotations

import json
from pathlib import Path

_DIR = Path(__file__).resolve().parent


def path(name: str) -> Path:
    p = _DIR / (name if name.endswith(".json") else name + ".json")
    if not p.exists():
        raise FileNotFoundError(f"no configuration named {name}; available: {sorted(x.stem for x in _DIR.glob('*.json'))}")
    return p


def load(name: str):
    """The typed configuration object of a bundled file."""
    d = json.loads(path(name).read_text())
    stem = path(name).stem
    if stem.startswith("qwen"):
        from ..models.qwen_hybrid import QwenHybridConfig
        return QwenHybridConfig.from_json(json.dumps(d))
    if stem.startswith("deepseek"):
        from ..models.deepseek_v4 import DSV4Config
        return DSV4Config.from_json(json.dumps(d))
    if stem.startswith("minimax"):
        from ..models.minimax_m2 import MiniMaxM2Config
        return MiniMaxM2Config(**d)
    from ..models.glm_dsa import GLMDSAConfig
    return GLMDSAConfig(**d)
