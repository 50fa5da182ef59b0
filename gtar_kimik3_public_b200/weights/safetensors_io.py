"""Reading and writing of safetensors files, by tensor name.

The format is small enough to own: an 8-byte little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}}`` and the raw little-endian
tensor bytes.  Tensors are mapped from the file (no copy until a tensor is taken), so a
folder with several shards costs no host memory to open.

The reference has no such file format (it pickles a state dict, ``src/common.py:85-93``);
its tensor *names* are what is kept (``model.state_dict()`` of
``src/models/transformer.py:70-77``).
"""

from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path

import torch

_DTYPES = {
    "F64": torch.float64,
    "F32": torch.float32,
    "F16": torch.float16,
    "BF16": torch.bfloat16,
    "I64": torch.int64,
    "I32": torch.int32,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    """The file is not a well-formed safetensors file."""


class SafetensorsFile:
    """One opened file: a table of entries and a memory map of the data."""

    def __init__(self, path: str | Path):
        self.path = Path(path)
        with open(self.path, "rb") as handle:
            head = handle.read(8)
            if len(head) != 8:
                raise SafetensorsError(f"{self.path}: shorter than its 8-byte header length")
            (header_len,) = struct.unpack("<Q", head)
            size = self.path.stat().st_size
            if header_len > size - 8:
                raise SafetensorsError(f"{self.path}: header length {header_len} exceeds the file ({size} bytes)")
            try:
                header = json.loads(handle.read(header_len))
            except (json.JSONDecodeError, UnicodeDecodeError) as exc:
                raise SafetensorsError(f"{self.path}: header is not JSON: {exc}") from None
            self.data_start = 8 + header_len
            self.metadata = header.pop("__metadata__", {}) or {}
            self.entries: dict[str, dict] = header
            data_size = size - self.data_start
            for name, entry in self.entries.items():
                if entry.get("dtype") not in _DTYPES:
                    raise SafetensorsError(f"{self.path}: tensor {name!r} has unsupported dtype {entry.get('dtype')!r}")
                begin, end = entry["data_offsets"]
                numel = 1
                for dim in entry["shape"]:
                    numel *= dim
                want = numel * _DTYPES[entry["dtype"]].itemsize
                if end - begin != want:
                    raise SafetensorsError(
                        f"{self.path}: tensor {name!r} spans {end - begin} bytes but its shape needs {want}"
                    )
                if end > data_size:
                    raise SafetensorsError(
                        f"{self.path}: truncated: tensor {name!r} ends at byte {end} of a {data_size}-byte data section"
                    )
            self._map = mmap.mmap(handle.fileno(), 0, access=mmap.ACCESS_COPY) if size > 0 else None

    def names(self) -> list[str]:
        return list(self.entries)

    def shape(self, name: str) -> tuple[int, ...]:
        return tuple(self.entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name]["dtype"]]

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that aliases the mapped file (a private copy-on-write mapping: writing to the
        tensor never reaches the file)."""
        entry = self.entries[name]
        begin, end = entry["data_offsets"]
        dtype = _DTYPES[entry["dtype"]]
        if end == begin:
            return torch.empty(tuple(entry["shape"]), dtype=dtype)
        start = self.data_start + begin
        if start % dtype.itemsize == 0:
            flat = torch.frombuffer(self._map, dtype=dtype, count=(end - begin) // dtype.itemsize, offset=start)
        else:  # a writer that did not keep alignment: take the bytes and reinterpret a copy
            flat = torch.frombuffer(self._map, dtype=torch.uint8, count=end - begin, offset=start).clone().view(dtype)
        return flat.view(tuple(entry["shape"]))


def write_safetensors(path: str | Path, tensors: dict[str, torch.Tensor], metadata: dict[str, str] | None = None) -> None:
    """Write ``tensors``; the header keeps the given order of names.

    The data section has no gaps (readers of this format refuse holes), so alignment is
    kept the usual way: tensors are laid out by element size, largest first, and the header
    is padded to a multiple of 8 bytes.
    """
    header: dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    prepared = {}
    for name, tensor in tensors.items():
        if tensor.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store tensor {name!r} of dtype {tensor.dtype}")
        prepared[name] = tensor.detach().cpu().contiguous()
        header[name] = None
    layout = sorted(prepared, key=lambda n: -prepared[n].dtype.itemsize)
    offset = 0
    for name in layout:
        tensor = prepared[name]
        nbytes = tensor.numel() * tensor.dtype.itemsize
        header[name] = {
            "dtype": _NAMES[tensor.dtype],
            "shape": list(tensor.shape),
            "data_offsets": [offset, offset + nbytes],
        }
        offset += nbytes
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * ((-len(text)) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(text)))
        handle.write(text)
        for name in layout:
            tensor = prepared[name]
            if tensor.numel():
                handle.write(tensor.reshape(-1).view(torch.uint8).numpy().tobytes())


class ModelFolderTensors:
    """All tensors of a model folder: ``model.safetensors`` or the shards its index names."""

    def __init__(self, folder: str | Path):
        folder = Path(folder)
        self.folder = folder
        index = folder / "model.safetensors.index.json"
        single = folder / "model.safetensors"
        self.files: list[SafetensorsFile] = []
        self.where: dict[str, SafetensorsFile] = {}
        if single.exists():
            paths = [single]
        elif index.exists():
            weight_map = json.loads(index.read_text()).get("weight_map", {})
            paths = [folder / shard for shard in sorted(set(weight_map.values()))]
        else:
            raise FileNotFoundError(f"{folder}: neither model.safetensors nor model.safetensors.index.json is there")
        for path in paths:
            opened = SafetensorsFile(path)
            self.files.append(opened)
            for name in opened.names():
                self.where[name] = opened

    def names(self) -> list[str]:
        return list(self.where)

    def shape(self, name: str) -> tuple[int, ...]:
        return self.where[name].shape(name)

    def dtype(self, name: str) -> torch.dtype:
        return self.where[name].dtype(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self.where[name].tensor(name)
