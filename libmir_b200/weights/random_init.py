"""Random weights from a configuration and a seed.

`write_model_folder` writes config.json and model.safetensors: every matrix N(0, 0.02^2), norm
weights 1, drawn on the host from a generator seeded by (seed, tensor name), so a tensor's values
do not depend on which other tensors exist.  `bind_random` fills a built model directly in device
memory (for sizes that are not worth a trip through a file); it uses the device's generator, so
its values differ from the file's for the same seed.  libmir has no such mode (its fixtures use a
constant 0.125, metal/src/engine/dense/swiglu/tests.rs:130-137).
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Mapping, Optional

import torch

from ..registry import build_spec
from .safetensors_io import write_file

STD = 0.02


def _seed_for(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 63) - 1)


def _storage_dtype(store: str, dtype: torch.dtype) -> torch.dtype:
    return {"float32": torch.float32, "int32": torch.int32}.get(store, dtype)


def random_tensor(name: str, spec, seed: int, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    target = _storage_dtype(spec.store, dtype)
    if spec.init == "ones":
        return torch.ones(spec.shape, dtype=target, device=device)
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=target, device=device)
    if torch.device(device).type == "cuda" and target in (torch.float32, torch.bfloat16):
        from .. import kernels
        values = torch.empty(spec.shape, dtype=target, device=device)
        kernels.random_normal(values, _seed_for(seed, name), STD)     # the engine's own generator, on the device
        return values
    generator = torch.Generator(device=device)
    generator.manual_seed(_seed_for(seed, name))
    values = torch.randn(spec.shape, generator=generator, dtype=torch.float32, device=device) * STD
    return values.to(target)


def parameter_specs(config_json: Mapping):
    """name -> ParamSpec of the model that config_json describes, without building any device state."""
    from ..models.decoder import DecoderModel
    from ..parts.base import BuildEnv
    spec = build_spec(config_json, None)
    model = DecoderModel(spec, BuildEnv(torch.float32, torch.device("meta")))
    return {name: param for name, (_, _, param) in model.parameter_table().items()}


def write_model_folder(folder, config_json: Mapping, seed: int = 0, dtype: str = "bfloat16",
                       include_optional: bool = True) -> Path:
    """Write `folder/config.json` and `folder/model.safetensors`; returns the folder."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    torch_dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}[dtype]
    tensors = {}
    for name, spec in parameter_specs(config_json).items():
        if spec.optional and not include_optional:
            continue
        tensors[name] = random_tensor(name, spec, seed, torch_dtype)
    (folder / "config.json").write_text(json.dumps(dict(config_json), indent=2))
    write_file(folder / "model.safetensors", tensors, metadata={"format": "pt", "seed": str(seed)})
    return folder


def bind_random(model, seed: int = 0) -> None:
    """Fill `model` with random weights generated on its device."""
    tensors = {}
    for name, (_, _, spec) in model.parameter_table().items():
        tensors[name] = random_tensor(name, spec, seed, model.env.dtype, device=model.env.device)
    model.bind(tensors)
