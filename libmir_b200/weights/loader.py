"""Binding checkpoint tensors to a model by name.

The model says which tensors it wants (DecoderModel.parameter_table); the checkpoint says which it
has (safetensors headers).  Names are compared after stripping one wrapping prefix
(models/src/weights/binding/roles/parse.rs:46-57).  Everything that does not fit is collected and
raised as ONE WeightsError that lists missing tensors, unexpected tensors and wrong shapes, so a bad
checkpoint is fixed in one pass.  libmir's loader ignores unknown extras as auxiliary
(roles/parse.rs:26-34,140-141); here an unexpected tensor is an error, because a tensor nobody reads
is most often a wrong config.json.

Dtypes on the device follow ParamSpec.store: "compute" tensors are cast to the engine's dtype
(bfloat16 or float32; libmir casts F16/F32 checkpoints to BF16 on upload,
cuda/src/checkpoint/dense/source.rs:34-38), "float32" tensors are kept in 32-bit, "int32" tables stay
integers.
"""

from __future__ import annotations

from pathlib import Path
from typing import Dict, Iterable, Mapping, Tuple

import torch

from ..errors import WeightsError
from .safetensors_io import TensorEntry, load_tensor, read_catalog


def canonical(name: str, prefixes: Iterable[str]) -> str:
    for prefix in prefixes:
        if name.startswith(prefix):
            return name[len(prefix):]
    return name


def catalog_shapes(folder) -> Dict[str, tuple]:
    """Canonical-agnostic view for architecture builders: checkpoint name -> shape."""
    return {name: entry.shape for name, entry in read_catalog(Path(folder)).items()}


def match(expected: Mapping[str, tuple], available: Mapping[str, TensorEntry], prefixes: Iterable[str]):
    """Pair wanted names with checkpoint entries; returns (pairs, missing, unexpected, wrong_shape)."""
    prefixes = tuple(prefixes)
    by_canonical: Dict[str, list] = {}
    for name in available:
        by_canonical.setdefault(canonical(name, prefixes), []).append(name)
    pairs: Dict[str, TensorEntry] = {}
    missing, unexpected, wrong_shape, duplicated = [], [], [], []
    used = set()
    for name, (_, _, spec) in expected.items():
        found = by_canonical.get(canonical(name, prefixes), [])
        if len(found) > 1:
            duplicated.append(f"{name} (stored as {', '.join(sorted(found))})")
            used.update(found)
            continue
        if not found:
            if not spec.optional:
                missing.append(name)
            continue
        entry = available[found[0]]
        used.add(found[0])
        if tuple(entry.shape) != tuple(spec.shape):
            wrong_shape.append(f"{found[0]}: expected {list(spec.shape)}, checkpoint has {list(entry.shape)}")
            continue
        pairs[name] = entry
    unexpected = sorted(name for name in available if name not in used)
    return pairs, sorted(missing), unexpected, wrong_shape, duplicated


def _to_device(tensor: torch.Tensor, store: str, env) -> torch.Tensor:
    if store == "int32":
        return tensor.to(device=env.device, dtype=torch.int32)
    target = torch.float32 if store == "float32" else env.dtype
    if tensor.dtype not in (torch.float32, torch.float16, torch.bfloat16, torch.float64):
        raise WeightsError(f"a floating-point tensor is stored as {tensor.dtype}")
    return tensor.to(device=env.device).to(target)


def load_into(model, folder) -> None:
    """Read the checkpoint of `folder` and bind it to `model` (a DecoderModel); raises WeightsError."""
    available = read_catalog(Path(folder))
    expected = model.parameter_table()
    pairs, missing, unexpected, wrong_shape, duplicated = match(expected, available, model.spec.strip_prefixes)
    if missing or unexpected or wrong_shape or duplicated:
        lines = [f"checkpoint {folder} does not fit architecture {model.spec.architecture}:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shapes ({len(wrong_shape)}): " + "; ".join(wrong_shape))
        if duplicated:
            lines.append(f"  stored more than once ({len(duplicated)}): " + "; ".join(duplicated))
        raise WeightsError("\n".join(lines), missing, unexpected, wrong_shape)
    tensors = {}
    for name, entry in pairs.items():
        store = expected[name][2].store
        tensors[name] = _to_device(load_tensor(entry), store, model.env)
    model.bind(tensors)
