"""Typed model configuration for the Qwen2 dense decoder, read from config.json keys.

Parity: the reference validates the same keys in ``ModelDims.from_hf_config``
(src/cloud_engine/model.py:47-83): nine required keys, ``model_type``,
``hidden_act == "silu"``, no ``rope_scaling``, ``rope_theta`` default 10000 and
``attention_bias`` default true for qwen2.  This class additionally reads
``head_dim`` (default ``hidden_size // num_attention_heads``, the reference's fixed
rule, model.py:66-75), ``max_position_embeddings`` and the sliding-window keys, and
refuses a window that would be in use, because the reference computes full causal
attention always.
"""

from __future__ import annotations

import json
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """A config.json key is missing, has the wrong type or an unsupported value."""


def _require(raw: dict[str, Any], key: str, kind: type | tuple[type, ...]) -> Any:
    if key not in raw:
        raise ConfigError(f"config.json: required key {key!r} is missing")
    value = raw[key]
    if isinstance(value, bool) and kind is not bool:
        raise ConfigError(f"config.json: key {key!r} must be {kind}, got bool")
    if not isinstance(value, kind):
        raise ConfigError(
            f"config.json: key {key!r} must be {kind}, got {type(value).__name__} ({value!r})"
        )
    return value


def _positive(raw: dict[str, Any], key: str) -> int:
    value = _require(raw, key, int)
    if value < 1:
        raise ConfigError(f"config.json: key {key!r} must be positive, got {value}")
    return value


@dataclass(frozen=True)
class Qwen2Config:
    """Every size and constant of a Qwen2 dense decoder; nothing of it lives in code."""

    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    attention_bias: bool
    tie_word_embeddings: bool
    eos_token_id: int | None
    max_position_embeddings: int
    hidden_act: str = "silu"
    model_type: str = "qwen2"
    architecture: str = "Qwen2ForCausalLM"

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "Qwen2Config":
        model_type = raw.get("model_type")
        if model_type != "qwen2":
            raise ConfigError(
                f"config.json: key 'model_type' must be 'qwen2' for this class, got {model_type!r}"
            )
        hidden = _positive(raw, "hidden_size")
        layers = _positive(raw, "num_hidden_layers")
        heads = _positive(raw, "num_attention_heads")
        kv_heads = _positive(raw, "num_key_value_heads")
        inter = _positive(raw, "intermediate_size")
        vocab = _positive(raw, "vocab_size")
        eps = float(_require(raw, "rms_norm_eps", (int, float)))
        tied = _require(raw, "tie_word_embeddings", bool)
        if "eos_token_id" not in raw:
            raise ConfigError("config.json: required key 'eos_token_id' is missing")
        eos = raw["eos_token_id"]
        if isinstance(eos, list):
            eos = eos[0] if eos else None
        if eos is not None and (isinstance(eos, bool) or not isinstance(eos, int)):
            raise ConfigError(f"config.json: key 'eos_token_id' must be an int or null, got {eos!r}")
        if eps <= 0:
            raise ConfigError(f"config.json: key 'rms_norm_eps' must be > 0, got {eps}")
        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: key 'hidden_act' must be 'silu' (SwiGLU), got {act!r}")
        if raw.get("rope_scaling"):
            raise ConfigError("config.json: key 'rope_scaling' is set; only unscaled RoPE is built")
        if heads % kv_heads != 0:
            raise ConfigError(
                "config.json: 'num_attention_heads' must be a multiple of 'num_key_value_heads' "
                f"({heads} vs {kv_heads})"
            )
        if "head_dim" in raw and raw["head_dim"] is not None:
            head_dim = _positive(raw, "head_dim")
        else:
            if hidden % heads != 0:
                raise ConfigError(
                    "config.json: 'hidden_size' is not divisible by 'num_attention_heads' "
                    "and no 'head_dim' is given"
                )
            head_dim = hidden // heads
        if head_dim % 2 != 0:
            raise ConfigError(f"config.json: head size {head_dim} must be even for rotary pairs")
        theta = float(raw.get("rope_theta", 10_000.0))
        if theta <= 0:
            raise ConfigError(f"config.json: key 'rope_theta' must be > 0, got {theta}")
        if raw.get("use_sliding_window", False):
            window = raw.get("sliding_window")
            max_window_layers = raw.get("max_window_layers", layers)
            if window is not None and max_window_layers < layers:
                raise ConfigError(
                    "config.json: 'use_sliding_window' would put a window in use "
                    f"(sliding_window={window}, max_window_layers={max_window_layers} < "
                    f"{layers} layers); this architecture is built with full causal attention"
                )
        max_pos = raw.get("max_position_embeddings", 32768)
        if isinstance(max_pos, bool) or not isinstance(max_pos, int) or max_pos < 1:
            raise ConfigError(
                f"config.json: key 'max_position_embeddings' must be a positive int, got {max_pos!r}"
            )
        archs = raw.get("architectures") or ["Qwen2ForCausalLM"]
        return cls(
            hidden_size=hidden,
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            intermediate_size=inter,
            vocab_size=vocab,
            rms_norm_eps=eps,
            rope_theta=theta,
            attention_bias=bool(raw.get("attention_bias", True)),
            tie_word_embeddings=tied,
            eos_token_id=eos,
            max_position_embeddings=max_pos,
            hidden_act=act,
            model_type="qwen2",
            architecture=str(archs[0]),
        )

    def to_dict(self) -> dict[str, Any]:
        """The config.json content that reads back to this configuration."""
        raw = asdict(self)
        arch = raw.pop("architecture")
        raw["architectures"] = [arch]
        raw["use_sliding_window"] = False
        return raw


def read_config_json(model_dir: str | Path) -> dict[str, Any]:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"no config.json in model folder {model_dir}")
    with open(path, encoding="utf-8") as handle:
        raw = json.load(handle)
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be a JSON object")
    return raw
