"""Reader (and, for tests and synthetic checkpoints, writer) of the safetensors container.

Format: 8-byte little-endian header length, a JSON header mapping tensor names to
``{"dtype", "shape", "data_offsets": [begin, end]}`` relative to the end of the header, then the
raw little-endian tensor bytes.  bf16 has no numpy dtype and is returned as its uint16 bits, like the
reference's reader does (litespark_inference/torchless/safetensors_io.py:1-13, 26-33)."""
from __future__ import annotations

import json
import struct
from pathlib import Path
from typing import Dict, Tuple

import numpy as np

_DTYPES = {
    "F64": np.float64, "F32": np.float32, "F16": np.float16, "BF16": np.uint16,
    "I64": np.int64, "I32": np.int32, "I16": np.int16, "I8": np.int8,
    "U64": np.uint64, "U32": np.uint32, "U16": np.uint16, "U8": np.uint8, "BOOL": np.bool_,
}


class SafetensorsFile:
    """Memory-mapped safetensors file.  ``get`` copies a tensor out, ``view`` returns a zero-copy
    array over the mapping (valid while this object is alive)."""

    def __init__(self, path):
        self.path = str(path)
        with open(self.path, "rb") as f:
            head = f.read(8)
            if len(head) != 8:
                raise ValueError(f"{self.path}: not a safetensors file (shorter than 8 bytes)")
            (n,) = struct.unpack("<Q", head)
            if n > 100 * 1024 * 1024:
                raise ValueError(f"{self.path}: implausible header length {n}")
            raw = f.read(n)
            if len(raw) != n:
                raise ValueError(f"{self.path}: truncated header")
        self.header: Dict[str, dict] = json.loads(raw.decode("utf-8"))
        self.metadata = self.header.pop("__metadata__", {})
        self.data_start = 8 + n
        self._mm = np.memmap(self.path, dtype=np.uint8, mode="r")
        size = self._mm.shape[0] - self.data_start
        for name, meta in self.header.items():
            b, e = meta["data_offsets"]
            if meta["dtype"] not in _DTYPES:
                raise ValueError(f"{self.path}: tensor {name!r} has unsupported dtype {meta['dtype']}")
            want = int(np.prod(meta["shape"], dtype=np.int64)) * np.dtype(_DTYPES[meta["dtype"]]).itemsize
            if not (0 <= b <= e <= size) or e - b != want:
                raise ValueError(f"{self.path}: tensor {name!r} has inconsistent offsets / shape")

    def __contains__(self, name: str) -> bool:
        return name in self.header

    def keys(self):
        return self.header.keys()

    def view(self, name: str) -> Tuple[np.ndarray, str]:
        """(zero-copy array, dtype tag).  bf16 comes back as uint16 bits."""
        meta = self.header[name]
        b, e = meta["data_offsets"]
        a = self._mm[self.data_start + b:self.data_start + e].view(_DTYPES[meta["dtype"]])
        return a.reshape(meta["shape"]), meta["dtype"]

    def get(self, name: str) -> Tuple[np.ndarray, str]:
        a, tag = self.view(name)
        return np.array(a), tag

    def close(self):
        self._mm = None


def open_safetensors(path) -> SafetensorsFile:
    return SafetensorsFile(path)


def save_safetensors(path, tensors: Dict[str, Tuple[np.ndarray, str]]) -> None:
    """Write ``{name: (array, dtype tag)}``; pass bf16 tensors as uint16 bits with the tag "BF16"."""
    header, offset, blobs = {}, 0, []
    for name, (arr, tag) in tensors.items():
        a = np.ascontiguousarray(arr, dtype=_DTYPES[tag])
        blob = a.tobytes()
        header[name] = {"dtype": tag, "shape": list(a.shape), "data_offsets": [offset, offset + len(blob)]}
        offset += len(blob)
        blobs.append(blob)
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * (-len(raw) % 8)                     # keep the data section 8-byte aligned
    with open(Path(path), "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for blob in blobs:
            f.write(blob)
