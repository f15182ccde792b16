"""One registry from an architecture's name to its builder, and one from a part's kind to its class.

libmir admits a checkpoint by what its configuration and tensors describe, not by a name list
(README.md:24-25, admission/src/cuda/admission.rs:45-76).  Here the name in config.json's
`architectures` selects a builder, and the builder performs that capability check itself
(every layer softmax attention + dense SwiGLU for the one architecture that is built).

Adding an architecture:  register_architecture("NameForCausalLM", builder) where
    builder(config_json: dict, catalog: dict[str, tuple] | None) -> ModelSpec
and `catalog` maps checkpoint tensor names to shapes when a checkpoint is at hand (None in
random-weights mode), so that optional tensors can be discovered by presence.

Adding a part:  register_part("kind", cls) where cls(spec, env) builds the part from its
PartSpec; see libmir_b200/parts/base.py for the interface each kind of part must have.
"""

from __future__ import annotations

from typing import Callable, Dict, Mapping, Optional

from .errors import ConfigError, RegistryError

_ARCHITECTURES: Dict[str, Callable] = {}
_PARTS: Dict[str, type] = {}


def register_architecture(name: str, builder: Callable) -> None:
    _ARCHITECTURES[name] = builder


def known_architectures() -> list:
    _load_builtin()
    return sorted(_ARCHITECTURES)


def architecture_of(config_json: Mapping) -> str:
    names = config_json.get("architectures")
    if not isinstance(names, list) or not names or not all(isinstance(n, str) for n in names):
        raise ConfigError("config.json must name the model class in `architectures`, e.g. [\"LlamaForCausalLM\"]; "
                          f"known: {', '.join(known_architectures())}")
    return names[0]


def build_spec(config_json: Mapping, catalog: Optional[Mapping[str, tuple]] = None):
    """config.json (+ the checkpoint's tensor names and shapes, if any) -> ModelSpec."""
    _load_builtin()
    name = architecture_of(config_json)
    builder = _ARCHITECTURES.get(name)
    if builder is None:
        raise RegistryError(f"unknown architecture {name!r}; known: {', '.join(sorted(_ARCHITECTURES))}")
    spec = builder(config_json, catalog)
    spec.validate()
    return spec


def register_part(kind: str, cls: type) -> None:
    _PARTS[kind] = cls


def build_part(spec, env):
    """PartSpec -> part object; `env` is the BuildEnv (dtype, device) shared by all parts."""
    _load_builtin()
    if spec is None:
        return None
    cls = _PARTS.get(spec.kind)
    if cls is None:
        raise RegistryError(f"unknown part kind {spec.kind!r}; known: {', '.join(sorted(_PARTS))}")
    return cls(spec, env)


_loaded = False


def _load_builtin() -> None:
    global _loaded
    if _loaded:
        return
    _loaded = True
    from . import models  # noqa: F401  registers the architectures
    from . import parts   # noqa: F401  registers the built-in parts
