"""Read and write safetensors files by tensor name.

Format facts (as the reference's reader relies on them, crates/engine/src/weights.rs:99-136):
an 8-byte little-endian header length, a JSON header mapping each name to
{dtype, shape, data_offsets}, then the raw little-endian data. This reader maps the
file and hands out tensors that view the mapping; nothing is converted here.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Tuple

import torch

from ..errors import WeightsFormatError

_ST_TO_TORCH = {
    "BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64,
    "I8": torch.int8, "U8": torch.uint8, "I16": torch.int16, "I32": torch.int32, "I64": torch.int64,
    "BOOL": torch.bool,
}
_TORCH_TO_ST = {v: k for k, v in _ST_TO_TORCH.items()}


class SafetensorsFile:
    """A mapped safetensors file: names, shapes, dtypes, and tensors on demand."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise WeightsFormatError(f"cannot open {path}: {e}") from e
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise WeightsFormatError(f"{path}: too short to be a safetensors file ({size} bytes)")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > size - 8 or hlen > (100 << 20):
            raise WeightsFormatError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightsFormatError(f"{path}: header is not JSON: {e}") from e
        if not isinstance(header, dict):
            raise WeightsFormatError(f"{path}: header is not a JSON object")
        self.metadata = header.pop("__metadata__", {})
        self._base = 8 + hlen
        self._entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            try:
                dt, shape, (b, en) = e["dtype"], tuple(int(s) for s in e["shape"]), e["data_offsets"]
            except (KeyError, TypeError, ValueError) as ex:
                raise WeightsFormatError(f"{path}: bad header entry for {name!r}: {ex}") from ex
            if not (0 <= b <= en <= size - self._base):
                raise WeightsFormatError(f"{path}: data of {name!r} lies outside the file")
            self._entries[name] = (dt, shape, int(b), int(en))
        # A private copy-on-write mapping: torch wants a writable buffer, the file stays untouched.
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_COPY) if size > 0 else None

    def names(self) -> Iterable[str]:
        return self._entries.keys()

    def __contains__(self, name: str) -> bool:
        return name in self._entries

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._entries[name][1]

    def dtype_name(self, name: str) -> str:
        return self._entries[name][0]

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapping (valid while this object lives)."""
        dt, shape, b, e = self._entries[name]
        if dt not in _ST_TO_TORCH:
            raise WeightsFormatError(f"{self.path}: {name}: dtype {dt} is not supported")
        tdt = _ST_TO_TORCH[dt]
        n = 1
        for s in shape:
            n *= s
        if n * torch.empty((), dtype=tdt).element_size() != e - b:
            raise WeightsFormatError(f"{self.path}: {name}: {e - b} bytes do not hold shape {list(shape)} of {dt}")
        if n == 0:
            return torch.empty(shape, dtype=tdt)
        t = torch.frombuffer(self._mm, dtype=tdt, count=n, offset=self._base + b)
        return t.reshape(shape)

    def close(self) -> None:
        # Tensors handed out may still view the mapping; leave unmapping to the collector.
        self._f.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] = None) -> None:
    """Write tensors (moved to the CPU, made contiguous) under their names, sorted."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    blobs = []
    for name in order:
        t = tensors[name].detach().to("cpu").contiguous()
        if t.dtype not in _TORCH_TO_ST:
            raise WeightsFormatError(f"cannot write {name}: dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _TORCH_TO_ST[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
        blobs.append(t)
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for t in blobs:
            if t.numel():
                f.write(t.view(torch.uint8).reshape(-1).numpy().tobytes() if t.numel() < (1 << 24)
                        else memoryview(t.view(torch.uint8).reshape(-1).numpy()))
    os.replace(tmp, path)
