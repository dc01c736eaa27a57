"""Reading and writing the safetensors container: an 8-byte little-endian header length, a JSON
header {name: {dtype, shape, data_offsets}}, then raw little-endian tensor bytes.

Plays the role that the GGUF parser plays in integrallis/models (by-name lookup over a mapped
file; backend-java/.../gguf/GgufFile.java:38-48, size checks
backend-java/.../gguf/GgufTensorInfo.java:24-74), for the folder format this library reads.
"""

from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Dict, Iterable, Mapping, Tuple

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


# dtype tag -> (bytes per element, numpy dtype used to view the bytes)
_ITEM = {
    "BF16": (2, np.uint16),
    "F16": (2, np.float16),
    "F32": (4, np.float32),
    "F64": (8, np.float64),
    "I64": (8, np.int64),
    "I32": (4, np.int32),
    "I16": (2, np.int16),
    "I8": (1, np.int8),
    "U8": (1, np.uint8),
    "BOOL": (1, np.uint8),
}

_TAG_OF = {
    torch.bfloat16: "BF16",
    torch.float16: "F16",
    torch.float32: "F32",
    torch.float64: "F64",
    torch.int64: "I64",
    torch.int32: "I32",
    torch.int16: "I16",
    torch.int8: "I8",
    torch.uint8: "U8",
}


def _no_duplicates(pairs):
    out = {}
    for key, value in pairs:
        if key in out:
            raise SafetensorsError(f"tensor name {key!r} appears twice in the header")
        out[key] = value
    return out


class SafetensorsFile:
    """One mapped file; tensors are materialised by name."""

    def __init__(self, path):
        self.path = Path(path)
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: too short to hold a safetensors header ({size} bytes)")
        self._file = open(self.path, "rb")
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        (header_len,) = struct.unpack("<Q", self._map[:8])
        if header_len <= 0 or 8 + header_len > size:
            raise SafetensorsError(
                f"{self.path}: header length {header_len} does not fit the file of {size} bytes (truncated?)")
        try:
            header = json.loads(self._map[8 : 8 + header_len].decode("utf-8"), object_pairs_hook=_no_duplicates)
        except (UnicodeDecodeError, json.JSONDecodeError) as error:
            raise SafetensorsError(f"{self.path}: header is not valid JSON ({error})") from error
        except SafetensorsError as error:
            raise SafetensorsError(f"{self.path}: {error}") from error
        if not isinstance(header, dict):
            raise SafetensorsError(f"{self.path}: header must be an object")
        self.metadata = header.pop("__metadata__", None) or {}
        self._data_start = 8 + header_len
        data_size = size - self._data_start
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            try:
                tag, shape, (begin, end) = info["dtype"], tuple(int(s) for s in info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError) as error:
                raise SafetensorsError(f"{self.path}: malformed header entry for {name!r}") from error
            if tag not in _ITEM:
                raise SafetensorsError(f"{self.path}: tensor {name!r} has unsupported dtype {tag!r}")
            count = 1
            for s in shape:
                if s < 0:
                    raise SafetensorsError(f"{self.path}: tensor {name!r} has a negative dimension {shape}")
                count *= s
            if not (0 <= begin <= end <= data_size):
                raise SafetensorsError(
                    f"{self.path}: tensor {name!r} spans bytes {begin}..{end}, beyond the {data_size} data bytes "
                    "of the file (truncated?)")
            if end - begin != count * _ITEM[tag][0]:
                raise SafetensorsError(
                    f"{self.path}: tensor {name!r} of shape {list(shape)} and dtype {tag} needs "
                    f"{count * _ITEM[tag][0]} bytes, the header gives {end - begin}")
            self.entries[name] = (tag, shape, begin, end)

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.entries[name][1]

    def dtype_tag(self, name: str) -> str:
        return self.entries[name][0]

    def tensor(self, name: str) -> torch.Tensor:
        """A host tensor that owns its memory.  bfloat16 stays bfloat16, float16 becomes bfloat16,
        32-bit floats stay 32-bit, 64-bit floats become 32-bit, integer tables become int32."""
        if name not in self.entries:
            raise SafetensorsError(f"{self.path}: tensor not found: {name}")
        tag, shape, begin, end = self.entries[name]
        view = np.frombuffer(self._map, dtype=_ITEM[tag][1], count=(end - begin) // _ITEM[tag][0],
                             offset=self._data_start + begin)
        if tag == "BF16":
            out = torch.from_numpy(view.copy()).view(torch.bfloat16)
        elif tag == "F16":
            out = torch.from_numpy(view.copy()).to(torch.bfloat16)
        elif tag == "F32":
            out = torch.from_numpy(view.copy())
        elif tag == "F64":
            out = torch.from_numpy(view.astype(np.float32))
        else:
            out = torch.from_numpy(view.astype(np.int32))
        return out.reshape(shape)

    def close(self):
        if self._map is not None:
            try:
                self._map.close()
            except BufferError:
                pass
            self._map = None
            self._file.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_safetensors(path, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] | None = None) -> None:
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    ordered = sorted(tensors.items())
    for name, t in ordered:
        if t.dtype not in _TAG_OF:
            raise SafetensorsError(f"cannot write tensor {name!r} of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _TAG_OF[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as out:
        out.write(struct.pack("<Q", len(blob)))
        out.write(blob)
        for _, t in ordered:
            c = t.detach().cpu().contiguous()
            if c.dtype == torch.bfloat16:
                c = c.view(torch.int16)
            out.write(c.numpy().tobytes())
