"""A single-file safetensors reader and writer.

Format (src/models/loader.cpp:213-227): an unsigned 64-bit little-endian header
length, a JSON header mapping each tensor name to ``dtype``, ``shape`` and
``data_offsets`` (relative to the end of the header), then the raw
little-endian data.  ``__metadata__`` is skipped.  The reader maps the file and
hands out tensors by name without copying the whole file; every malformed
input the reference rejects (src/models/loader.cpp:79-140, 214-252) is rejected
here with :class:`SafetensorsError`.
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Dict, Iterable, List, Tuple

import numpy as np
import torch


class SafetensorsError(RuntimeError):
    pass


# stored dtype -> (numpy view dtype, bytes per element, torch dtype handed out)
_DTYPES = {
    "BF16": (np.uint16, 2, torch.bfloat16),
    "F16": (np.float16, 2, torch.float32),    # widened: exact
    "F32": (np.float32, 4, torch.float32),
    "I32": (np.int32, 4, torch.int32),
    "I64": (np.int64, 8, torch.int32),         # integer tables are kept as int32
}


class SafetensorsFile:
    def __init__(self, path):
        self.path = Path(path)
        try:
            self._fh = open(self.path, "rb")
        except OSError as e:
            raise SafetensorsError(f"cannot open {self.path}: {e}") from None
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: file is smaller than the 8-byte header length")
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._map[:8])
        if 8 + hlen > size:
            raise SafetensorsError(f"{self.path}: header length {hlen} exceeds the file size {size}")
        try:
            header = json.loads(bytes(self._map[8:8 + hlen]))
        except ValueError as e:
            raise SafetensorsError(f"{self.path}: header is not JSON: {e}") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{self.path}: header is not a JSON object")
        self._base = 8 + hlen
        self._entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            self._entries[name] = self._check_entry(name, meta, size)

    def _check_entry(self, name, meta, size):
        if not isinstance(meta, dict) or not isinstance(meta.get("dtype"), str):
            raise SafetensorsError(f"tensor '{name}': missing dtype")
        dtype = meta["dtype"]
        if dtype not in _DTYPES:
            raise SafetensorsError(f"tensor '{name}': Unsupported dtype {dtype}")
        shape = meta.get("shape")
        if not isinstance(shape, list) or not shape:
            raise SafetensorsError(f"tensor '{name}': missing or empty shape (scalars are not supported)")
        for s in shape:
            if isinstance(s, bool) or not isinstance(s, int) or s <= 0:
                raise SafetensorsError(f"tensor '{name}': bad dimension {s!r} in shape {shape}")
        offs = meta.get("data_offsets")
        if (not isinstance(offs, list) or len(offs) != 2
                or any(isinstance(o, bool) or not isinstance(o, int) or o < 0 for o in offs) or offs[1] < offs[0]):
            raise SafetensorsError(f"tensor '{name}': bad data_offsets {offs!r}")
        if self._base + offs[1] > size:
            raise SafetensorsError(f"tensor '{name}': data runs past the end of the file")
        numel = 1
        for s in shape:
            numel *= s
        if offs[1] - offs[0] != numel * _DTYPES[dtype][1]:
            raise SafetensorsError(f"tensor '{name}': {offs[1] - offs[0]} bytes stored, "
                                   f"shape {shape} of {dtype} needs {numel * _DTYPES[dtype][1]}")
        return dtype, tuple(shape), offs[0], offs[1]

    def names(self) -> List[str]:
        return sorted(self._entries)

    def __contains__(self, name: str) -> bool:
        return name in self._entries

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._entries[name][1]

    def stored_dtype(self, name: str) -> str:
        return self._entries[name][0]

    def tensor(self, name: str) -> torch.Tensor:
        """A host tensor owning its data.  BF16 stays bfloat16, F32 stays float32,
        F16 is widened to float32, integer tables become int32."""
        if name not in self._entries:
            raise KeyError(name)
        dtype, shape, lo, hi = self._entries[name]
        np_dtype, _, torch_dtype = _DTYPES[dtype]
        arr = np.frombuffer(self._map, dtype=np_dtype, count=(hi - lo) // np.dtype(np_dtype).itemsize,
                            offset=self._base + lo).reshape(shape)
        if dtype == "BF16":
            return torch.from_numpy(arr.copy()).view(torch.bfloat16)
        return torch.from_numpy(arr.copy()).to(torch_dtype)

    def close(self) -> None:
        try:
            self._map.close()
        except (BufferError, ValueError):
            pass
        self._fh.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


_STORE = {torch.bfloat16: "BF16", torch.float32: "F32", torch.float16: "F16", torch.int32: "I32", torch.int64: "I64"}


def write_safetensors(path, tensors: Iterable[Tuple[str, torch.Tensor]]) -> None:
    """Writes tensors in the order given.  Accepts a dict's ``items()`` or a
    generator, so that a large model never has to be held whole."""
    path = Path(path)
    pending = []
    header = {}
    offset = 0
    tmp = path.with_suffix(path.suffix + ".data")
    with open(tmp, "wb") as data:
        for name, t in tensors:
            t = t.detach().cpu().contiguous()
            if t.dtype not in _STORE:
                raise SafetensorsError(f"tensor '{name}': cannot store dtype {t.dtype}")
            raw = t.view(torch.uint8).numpy().tobytes() if t.dtype != torch.bfloat16 \
                else t.view(torch.int16).numpy().tobytes()
            header[name] = {"dtype": _STORE[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
            offset += len(raw)
            data.write(raw)
            pending.append(name)
    hs = json.dumps(header).encode()
    hs += b" " * ((8 - len(hs) % 8) % 8)
    with open(path, "wb") as out, open(tmp, "rb") as data:
        out.write(struct.pack("<Q", len(hs)))
        out.write(hs)
        while True:
            chunk = data.read(1 << 24)
            if not chunk:
                break
            out.write(chunk)
    tmp.unlink()
