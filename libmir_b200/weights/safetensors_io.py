"""Reading and writing safetensors files without any library.

Container layout as libmir reads it (models/src/weights/catalog.rs:125-168): an unsigned
64-bit little-endian header length, a JSON header of {name: {dtype, shape, data_offsets}},
`__metadata__` skipped, header at most 100 MiB; a tensor's payload starts at
8 + header_len + data_offsets[0] (catalog.rs:28-39).  Files are found through
model.safetensors.index.json's weight_map, else every *.safetensors of the folder
(models/src/layout/files.rs:116-142).
"""

from __future__ import annotations

import json
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Iterable, Mapping

import numpy as np
import torch

from ..errors import WeightsError

MAX_HEADER_BYTES = 100 * 1024 * 1024

_DTYPES = {
    "F64": (torch.float64, np.dtype("<f8")), "F32": (torch.float32, np.dtype("<f4")),
    "F16": (torch.float16, np.dtype("<f2")), "BF16": (torch.bfloat16, np.dtype("<u2")),
    "I64": (torch.int64, np.dtype("<i8")), "I32": (torch.int32, np.dtype("<i4")),
    "I16": (torch.int16, np.dtype("<i2")), "I8": (torch.int8, np.dtype("i1")),
    "U8": (torch.uint8, np.dtype("u1")), "BOOL": (torch.bool, np.dtype("?")),
}
_NAMES = {torch_dtype: name for name, (torch_dtype, _) in _DTYPES.items()}


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str
    shape: tuple
    file: Path
    begin: int        # absolute byte offset in the file
    nbytes: int


def read_header(path: Path) -> Dict[str, TensorEntry]:
    path = Path(path)
    with open(path, "rb") as handle:
        first = handle.read(8)
        if len(first) != 8:
            raise WeightsError(f"{path}: too short to be a safetensors file")
        (length,) = struct.unpack("<Q", first)
        if length > MAX_HEADER_BYTES:
            raise WeightsError(f"{path}: header of {length} bytes exceeds the limit of {MAX_HEADER_BYTES}")
        try:
            header = json.loads(handle.read(length))
        except (json.JSONDecodeError, UnicodeDecodeError) as error:
            raise WeightsError(f"{path}: header is not valid JSON: {error}") from error
    size = path.stat().st_size
    entries: Dict[str, TensorEntry] = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        dtype = meta.get("dtype")
        if dtype not in _DTYPES:
            raise WeightsError(f"{path}: tensor {name} has unsupported dtype {dtype}")
        shape = tuple(int(d) for d in meta["shape"])
        begin, end = (int(v) for v in meta["data_offsets"])
        expect = int(np.prod(shape, dtype=np.int64)) * _DTYPES[dtype][1].itemsize
        if end - begin != expect or 8 + length + end > size:
            raise WeightsError(f"{path}: tensor {name} spans bytes {begin}..{end}, which does not fit shape {shape} "
                               f"of {dtype} or the file's size")
        entries[name] = TensorEntry(name, dtype, shape, path, 8 + length + begin, end - begin)
    return entries


def checkpoint_files(folder: Path) -> list:
    folder = Path(folder)
    index = folder / "model.safetensors.index.json"
    if index.is_file():
        weight_map = json.loads(index.read_text()).get("weight_map", {})
        files = sorted({folder / name for name in weight_map.values()})
    else:
        files = sorted(folder.glob("*.safetensors"))
    if not files:
        raise WeightsError(f"{folder}: no *.safetensors file")
    return files


def read_catalog(folder: Path) -> Dict[str, TensorEntry]:
    """Names, dtypes and shapes of every tensor of a model folder; headers only."""
    catalog: Dict[str, TensorEntry] = {}
    for path in checkpoint_files(folder):
        for name, entry in read_header(path).items():
            if name in catalog:
                raise WeightsError(f"tensor {name} appears in both {catalog[name].file.name} and {path.name}")
            catalog[name] = entry
    return catalog


def load_tensor(entry: TensorEntry) -> torch.Tensor:
    """The tensor on the host, in its stored dtype (memory-mapped, then copied)."""
    torch_dtype, numpy_dtype = _DTYPES[entry.dtype]
    count = entry.nbytes // numpy_dtype.itemsize
    if count == 0:
        return torch.empty(entry.shape, dtype=torch_dtype)
    mapped = np.memmap(entry.file, dtype=numpy_dtype, mode="r", offset=entry.begin, shape=(count,))
    tensor = torch.from_numpy(np.array(mapped))
    if entry.dtype == "BF16":
        tensor = tensor.view(torch.bfloat16)
    return tensor.reshape(entry.shape)


def write_file(path: Path, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] | None = None) -> None:
    """Write tensors (host or device) in name order, payload aligned to 8 bytes."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order = sorted(tensors)
    for name in order:
        tensor = tensors[name]
        if tensor.dtype not in _NAMES:
            raise WeightsError(f"cannot store tensor {name} of dtype {tensor.dtype}")
        nbytes = tensor.numel() * tensor.element_size()
        header[name] = {"dtype": _NAMES[tensor.dtype], "shape": list(tensor.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(blob)))
        handle.write(blob)
        for name in order:
            tensor = tensors[name].detach().contiguous().cpu()
            if tensor.dtype == torch.bfloat16:
                tensor = tensor.view(torch.int16)
            handle.write(tensor.numpy().tobytes())
