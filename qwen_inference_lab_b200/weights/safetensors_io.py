"""Reading and writing safetensors files without any helper package.

File format: 8 bytes little-endian header length, a JSON header that maps tensor
names to ``{"dtype", "shape", "data_offsets"}`` (offsets relative to the end of
the header), then the raw little-endian tensor bytes.  The reference opens its
shards through the ``safetensors`` package (qil/model.py:180,189-190); this module
parses the same files itself so that the engine depends on nothing but torch.
"""
from __future__ import annotations

import json
import mmap
import struct
import warnings
from pathlib import Path

import torch

_DTYPES = {
    "F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {dtype: name for name, dtype in _DTYPES.items()}


class SafetensorsError(ValueError):
    """A file that is not a well-formed safetensors file."""


class SafetensorsFile:
    """A memory-mapped safetensors file; tensors are views of the mapping."""

    def __init__(self, path):
        self.path = Path(path)
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: truncated file ({size} bytes)")
        self._handle = open(self.path, "rb")
        self._map = mmap.mmap(self._handle.fileno(), 0, access=mmap.ACCESS_READ)
        (header_len,) = struct.unpack("<Q", self._map[:8])
        if header_len <= 0 or 8 + header_len > size:
            raise SafetensorsError(f"{self.path}: header length {header_len} exceeds the file")
        try:
            header = json.loads(self._map[8:8 + header_len].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as error:
            raise SafetensorsError(f"{self.path}: unreadable header: {error}") from None
        self.metadata = header.pop("__metadata__", {})
        self._data_start = 8 + header_len
        self.entries = {}
        for name, entry in header.items():
            dtype = _DTYPES.get(entry.get("dtype"))
            if dtype is None:
                raise SafetensorsError(f"{self.path}: tensor {name} has unsupported dtype {entry.get('dtype')}")
            shape = tuple(int(n) for n in entry["shape"])
            begin, end = (int(n) for n in entry["data_offsets"])
            count = 1
            for n in shape:
                count *= n
            if end - begin != count * torch.empty((), dtype=dtype).element_size():
                raise SafetensorsError(f"{self.path}: tensor {name} has {end - begin} bytes for shape {shape}")
            if begin < 0 or self._data_start + end > size:
                raise SafetensorsError(f"{self.path}: tensor {name} lies beyond the end of the file (truncated?)")
            self.entries[name] = (dtype, shape, begin, end)

    def keys(self):
        return list(self.entries)

    def shape(self, name):
        return self.entries[name][1]

    def dtype(self, name):
        return self.entries[name][0]

    def tensor(self, name) -> torch.Tensor:
        """A read-only CPU view of the tensor's bytes (copy before writing to it)."""
        dtype, shape, begin, end = self.entries[name]
        if begin == end:
            return torch.empty(shape, dtype=dtype)
        count = 1
        for n in shape:
            count *= n
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)   # the mapping is read-only by design
            flat = torch.frombuffer(self._map, dtype=dtype, count=count, offset=self._data_start + begin)
        return flat.reshape(shape)

    def close(self):
        # Views handed out by tensor() keep the mapping alive; closing is best effort.
        try:
            self._map.close()
        except BufferError:
            pass
        self._handle.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_safetensors(path, tensors: dict, metadata: dict | None = None) -> None:
    """Write ``tensors`` (name -> CPU tensor) as one safetensors file, names sorted."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    ordered = sorted(tensors)
    for name in ordered:
        tensor = tensors[name]
        if tensor.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {tensor.dtype} for {name}")
        size = tensor.numel() * tensor.element_size()
        header[name] = {"dtype": _NAMES[tensor.dtype], "shape": list(tensor.shape),
                        "data_offsets": [offset, offset + size]}
        offset += size
    encoded = json.dumps(header, separators=(",", ":")).encode("utf-8")
    encoded += b" " * (-len(encoded) % 8)
    with open(path, "wb") as out:
        out.write(struct.pack("<Q", len(encoded)))
        out.write(encoded)
        for name in ordered:
            tensor = tensors[name].detach().cpu().contiguous()
            out.write(tensor.reshape(-1).view(torch.uint8).numpy().tobytes())
