"""Binding checkpoint tensors to a model by name.

The model says which tensors it wants (DecoderModel.parameter_table); the checkpoint says which it
has (safetensors headers).  Names are compared after stripping one wrapping prefix
(models/src/weights/binding/roles/parse.rs:46-57).  A wanted tensor is bound to the stored tensor of its
name, or, where its ParamSpec lists `sources`, to a range of rows of another stored tensor (a fused
`qkv_proj.weight`, models/src/weights/binding/shapes/transforms.rs:22-35); a 2-d tensor stored with its two
dimensions swapped is recognised by its shape and transposed (transforms.rs:52-58, dimensions.rs:7-15).
A checkpoint that stores a tensor both ways is refused (grammar/mod.rs:23-41).  Everything that does not
fit is collected and raised as ONE WeightsError that lists missing tensors, unexpected tensors and wrong
shapes, so a bad checkpoint is fixed in one pass.  Stored tensors that nothing asks for are auxiliary, as in
libmir (roles/parse.rs:26-34,140-141: older Llama folders carry `rotary_emb.inv_freq` buffers): they are
ignored, and named in the error when there is one; with `strict=True` they are an error by themselves.

Dtypes on the device follow ParamSpec.store: "compute" tensors are cast to the engine's dtype
(bfloat16 or float32; libmir casts F16/F32 checkpoints to BF16 on upload,
cuda/src/checkpoint/dense/source.rs:34-38), "float32" tensors are kept in 32-bit, "int32" tables stay
integers.
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Iterable, Mapping, Optional, Tuple

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


@dataclass(frozen=True)
class Binding:
    """How one wanted tensor is read: the stored entry, the rows of it that are wanted (None: all), and whether
    the stored tensor has its two dimensions swapped."""

    entry: TensorEntry
    rows: Optional[tuple] = None
    transposed: bool = False


def _is_transpose(wanted: tuple, stored: tuple) -> bool:
    return len(wanted) == 2 and wanted != stored and stored == (wanted[1], wanted[0])


def match(expected: Mapping[str, tuple], available: Mapping[str, TensorEntry], prefixes: Iterable[str]):
    """Pair wanted names with checkpoint entries.
    Returns (bindings, missing, unexpected, wrong_shape, duplicated)."""
    prefixes = tuple(prefixes)
    by_canonical: Dict[str, list] = {}
    for name in available:
        by_canonical.setdefault(canonical(name, prefixes), []).append(name)
    bindings: Dict[str, Binding] = {}
    missing, wrong_shape, duplicated = [], [], []
    used = set()
    for name, (_, local, spec) in expected.items():
        wanted = tuple(spec.shape)
        found = by_canonical.get(canonical(name, prefixes), [])
        # the same tensor cut from another stored one: the source's name replaces the local name
        stem = name[:len(name) - len(local)] if local and name.endswith(local) else None
        fused = []
        for source in (spec.sources if stem is not None else ()):
            for stored in by_canonical.get(canonical(stem + source.name, prefixes), []):
                fused.append((source, stored))
        used.update(found)
        used.update(stored for _, stored in fused)
        if len(found) > 1 or len(fused) > 1:
            both = sorted(found) + sorted(stored for _, stored in fused)
            duplicated.append(f"{name} (stored as {', '.join(both)})")
            continue
        if found and fused:
            duplicated.append(f"{name} (stored as {found[0]} and also as rows of {fused[0][1]}: fused and separate "
                              "tensors for one projection)")
            continue
        if fused:
            source, stored = fused[0]
            entry = available[stored]
            whole = (source.total_rows,) + wanted[1:]
            if tuple(entry.shape) == whole:
                bindings[name] = Binding(entry, tuple(source.rows), False)
            elif spec.accept_transposed and _is_transpose(whole, tuple(entry.shape)):
                bindings[name] = Binding(entry, tuple(source.rows), True)
            else:
                wrong_shape.append(f"{stored}: expected {list(whole)} (rows {source.rows[0]}..{source.rows[1]} of it "
                                   f"are {name}), checkpoint has {list(entry.shape)}")
            continue
        if not found:
            if not spec.optional:
                missing.append(name)
            continue
        entry = available[found[0]]
        if tuple(entry.shape) == wanted:
            bindings[name] = Binding(entry)
        elif spec.accept_transposed and _is_transpose(wanted, tuple(entry.shape)):
            bindings[name] = Binding(entry, None, True)
        else:
            wrong_shape.append(f"{found[0]}: expected {list(spec.shape)}, checkpoint has {list(entry.shape)}")
    unexpected = sorted(name for name in available if name not in used)
    return bindings, sorted(missing), unexpected, wrong_shape, duplicated


def _to_device(tensor: torch.Tensor, store: str, env) -> torch.Tensor:
    if store == "int32":
        return tensor.to(device=env.device, dtype=torch.int32)
    target = torch.float32 if store == "float32" else env.dtype
    if tensor.dtype not in (torch.float32, torch.float16, torch.bfloat16, torch.float64):
        raise WeightsError(f"a floating-point tensor is stored as {tensor.dtype}")
    moved = tensor.to(device=env.device)
    if moved.dtype == target:
        return moved
    if moved.is_cuda and moved.is_contiguous() and (moved.dtype, target) in _kernels().CAST_KINDS:
        cast = torch.empty(moved.shape, dtype=target, device=moved.device)
        _kernels().cast(moved, cast)                 # the engine's own cast kernel (libmir: dense_cast.cu)
        return cast
    return moved.to(target)


def _kernels():
    from .. import kernels
    return kernels


def load_into(model, folder, strict: bool = False) -> None:
    """Read the checkpoint of `folder` and bind it to `model` (a DecoderModel); raises WeightsError.
    `strict`: stored tensors that the model does not ask for are an error too."""
    available = read_catalog(Path(folder))
    expected = model.parameter_table()
    bindings, missing, unexpected, wrong_shape, duplicated = match(expected, available, model.spec.strip_prefixes)
    if missing or wrong_shape or duplicated or (strict and unexpected):
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
    model.ignored_tensors = unexpected
    loaded: Dict[str, torch.Tensor] = {}                # a fused tensor is read once for all its parts
    tensors = {}
    for name, binding in bindings.items():
        stored = loaded.get(binding.entry.name)
        if stored is None:
            stored = load_tensor(binding.entry)
            if binding.rows is not None:
                loaded[binding.entry.name] = stored
        if binding.transposed:
            stored = stored.t()
        if binding.rows is not None:
            stored = stored[binding.rows[0]:binding.rows[1]]
        tensors[name] = _to_device(stored.contiguous(), expected[name][2].store, model.env)
    model.bind(tensors)
