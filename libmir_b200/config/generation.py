"""generation_config.json and per-request overrides.

models/src/generation/mod.rs:13-47 (fields), :68-112 (resolve), :149-166 (validation),
:197-208 (stop ids from eos_token_id, an integer or a list)."""

from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional

from ..errors import ConfigError

DEFAULT_MAX_TOKENS = 2048
DEFAULT_SAMPLE_TEMPERATURE = 1.0
DEFAULT_SEED = 0x4D49524D4952   # runtime/src/sampling/mod.rs:156


@dataclass
class GenerationOverrides:
    max_tokens: Optional[int] = None
    min_tokens: Optional[int] = None
    ignore_eos: Optional[bool] = None
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    top_k: Optional[int] = None
    repetition_penalty: Optional[float] = None


@dataclass
class GenerationSettings:
    max_tokens: int = DEFAULT_MAX_TOKENS
    min_tokens: int = 0
    ignore_eos: bool = False
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    repetition_penalty: float = 1.0
    stop_token_ids: tuple = ()

    def validate(self) -> None:
        if self.max_tokens <= 0:
            raise ConfigError("max_tokens must be greater than zero")
        if self.min_tokens > self.max_tokens:
            raise ConfigError("min_tokens cannot exceed max_tokens")
        if not math.isfinite(self.temperature) or self.temperature < 0.0:
            raise ConfigError("temperature must be finite and >= 0")
        if not math.isfinite(self.top_p) or self.top_p <= 0.0 or self.top_p > 1.0:
            raise ConfigError("top_p must be in (0, 1]")
        if self.top_k < 0:
            raise ConfigError("top_k must be >= 0")
        if not math.isfinite(self.repetition_penalty) or self.repetition_penalty < 1.0:
            raise ConfigError("repetition_penalty must be finite and >= 1")

    @property
    def greedy(self) -> bool:
        """src/generation/sampling.rs:49-60: greedy iff temperature <= epsilon or top_k == 1."""
        return self.temperature <= 1.1920929e-07 or self.top_k == 1


@dataclass
class GenerationConfig:
    max_tokens: Optional[int] = None
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    top_k: Optional[int] = None
    repetition_penalty: Optional[float] = None
    do_sample: Optional[bool] = None
    stop_token_ids: tuple = ()

    @classmethod
    def from_dict(cls, value: dict) -> "GenerationConfig":
        def number(key, kind):
            raw = value.get(key)
            if raw is None:
                return None
            if isinstance(raw, bool) or not isinstance(raw, (int, float)):
                raise ConfigError(f"{key} must be a number")
            return kind(raw)
        eos = value.get("eos_token_id")
        if eos is None:
            stops = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            stops = (eos,)
        elif isinstance(eos, list) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            stops = tuple(eos)
        else:
            raise ConfigError("eos_token_id must be an integer or a list of integers")
        do_sample = value.get("do_sample")
        if do_sample is not None and not isinstance(do_sample, bool):
            raise ConfigError("do_sample must be a boolean")
        return cls(number("max_new_tokens", int), number("temperature", float), number("top_p", float),
                   number("top_k", int), number("repetition_penalty", float), do_sample, stops)

    @classmethod
    def from_folder(cls, folder) -> "GenerationConfig":
        path = Path(folder) / "generation_config.json"
        if not path.is_file():
            return cls()
        return cls.from_dict(json.loads(path.read_text()))

    def resolve(self, overrides: Optional[GenerationOverrides] = None) -> GenerationSettings:
        o = overrides or GenerationOverrides()
        checkpoint_temperature = self.temperature if self.do_sample is not False else None
        if o.temperature is not None:
            temperature = o.temperature
        elif checkpoint_temperature is not None:
            temperature = checkpoint_temperature
        else:
            temperature = DEFAULT_SAMPLE_TEMPERATURE if self.do_sample else 0.0
        pick = lambda a, b, default: a if a is not None else (b if b is not None else default)
        settings = GenerationSettings(
            max_tokens=pick(o.max_tokens, self.max_tokens, DEFAULT_MAX_TOKENS),
            min_tokens=pick(o.min_tokens, None, 0),
            ignore_eos=pick(o.ignore_eos, None, False),
            temperature=float(temperature),
            top_p=float(pick(o.top_p, self.top_p, 1.0)),
            top_k=int(pick(o.top_k, self.top_k, 0)),
            repetition_penalty=float(pick(o.repetition_penalty, self.repetition_penalty, 1.0)),
            stop_token_ids=tuple(self.stop_token_ids),
        )
        settings.validate()
        return settings
