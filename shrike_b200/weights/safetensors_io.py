"""Reading and writing the safetensors container, by tensor name.

The format: 8 bytes little-endian header length, a JSON header
`{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__"?: {...}}`,
then one byte buffer; offsets count from its start.  Azimml/shrike calls
`safetensors.torch.load_file` (shrike/models/qwen.py:20,210); this reader maps the
file and hands out zero-copy views instead, so a tensor goes from the page cache to
the device in one copy.
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
    pass


class SafetensorsFile:
    """One mapped .safetensors file."""

    def __init__(self, path: str | Path):
        self.path = Path(path)
        with open(self.path, "rb") as handle:
            head = handle.read(8)
            if len(head) < 8:
                raise SafetensorsError(f"{self.path}: shorter than a safetensors header")
            (length,) = struct.unpack("<Q", head)
            size = self.path.stat().st_size
            if length > size - 8:
                raise SafetensorsError(f"{self.path}: header length {length} exceeds the file")
            try:
                header = json.loads(handle.read(length))
            except json.JSONDecodeError as error:
                raise SafetensorsError(f"{self.path}: header is not JSON ({error})") from None
            self._map = mmap.mmap(handle.fileno(), 0, access=mmap.ACCESS_COPY) if size else None
        self.metadata = header.pop("__metadata__", {})
        self._data_start = 8 + length
        self.entries: dict[str, dict] = header
        limit = size - self._data_start
        for name, entry in header.items():
            if entry.get("dtype") not in _DTYPES:
                raise SafetensorsError(f"{self.path}: tensor {name!r} has dtype {entry.get('dtype')!r}")
            begin, end = entry["data_offsets"]
            count = 1
            for extent in entry["shape"]:
                count *= extent
            width = torch.empty((), dtype=_DTYPES[entry["dtype"]]).element_size()
            if not (0 <= begin <= end <= limit) or end - begin != count * width:
                raise SafetensorsError(f"{self.path}: tensor {name!r} has bad offsets {begin}:{end}")

    def names(self) -> list[str]:
        return list(self.entries)

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name]["dtype"]]

    def shape(self, name: str) -> tuple[int, ...]:
        return tuple(self.entries[name]["shape"])

    def tensor(self, name: str) -> torch.Tensor:
        """A read-only CPU view of the mapped bytes."""
        entry = self.entries[name]
        begin, end = entry["data_offsets"]
        dtype = _DTYPES[entry["dtype"]]
        if end == begin:
            return torch.empty(self.shape(name), dtype=dtype)
        count = (end - begin) // torch.empty((), dtype=dtype).element_size()
        flat = torch.frombuffer(self._map, dtype=dtype, count=count, offset=self._data_start + begin)
        return flat.view(self.shape(name))


def write_safetensors(path: str | Path, tensors: dict[str, torch.Tensor], metadata: dict | None = None):
    """Writes `tensors` packed without gaps, widest element type first (then by
    name), so that every tensor starts on a multiple of its element size."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name, tensor in sorted(tensors.items(), key=lambda kv: (-kv[1].element_size(), kv[0])):
        if tensor.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {tensor.dtype} cannot be stored")
        data = tensor.detach().cpu().contiguous()
        raw = data.view(torch.uint8).numpy().tobytes() if data.numel() else b""
        header[name] = {
            "dtype": _NAMES[tensor.dtype],
            "shape": list(tensor.shape),
            "data_offsets": [offset, offset + len(raw)],
        }
        blobs.append(raw)
        offset += len(raw)
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * ((-len(text)) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(text)))
        handle.write(text)
        for blob in blobs:
            handle.write(blob)
