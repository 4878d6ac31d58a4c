"""Weights by tensor name, checked against the model's manifest in one pass.

The reference takes each tensor by its checkpoint name with a dtype and shape check and
rejects leftovers (crates/engine/src/weights.rs:105-136,185-194), stopping at the first
problem. Here every problem of a file is collected and raised as ONE `WeightsError` that
lists missing tensors, unexpected tensors and wrong shapes together.

Storage rule: a floating tensor stays in the dtype it was stored in (bfloat16 stays
bfloat16, a tensor stored in 32-bit stays 32-bit; float16 is widened to float32 because no
kernel here computes in it); integer tables become int32. What a part does with a tensor
whose dtype differs from the compute dtype is the part's business.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Dict, Iterable, Mapping, Optional, Tuple

import torch

from ..errors import WeightsError, WeightsFormatError
from .safetensors_io import SafetensorsFile

_FLOAT_NAMES = ("BF16", "F16", "F32")
_INT_NAMES = ("I8", "U8", "I16", "I32", "I64")


@dataclass(frozen=True)
class TensorSpec:
    """What the model expects under one name."""
    shape: Tuple[int, ...]
    kind: str = "float"          # "float" or "int"
    init: str = "normal"         # random-weights rule: "normal", "ones" or "zeros"


class WeightSet:
    """Checked tensors by name; `take` hands each out once, `finish` insists all were used."""

    def __init__(self, tensors: Dict[str, torch.Tensor], source: str):
        self._tensors = dict(tensors)
        self._taken = set()
        self.source = source

    def take(self, name: str) -> torch.Tensor:
        if name not in self._tensors:
            raise WeightsError(self.source, missing=[name])
        self._taken.add(name)
        return self._tensors[name]

    def has(self, name: str) -> bool:
        return name in self._tensors

    def finish(self) -> None:
        left = set(self._tensors) - self._taken
        if left:
            raise WeightsError(self.source, other=[f"the model did not use: {', '.join(sorted(left))}"])

    def names(self) -> Iterable[str]:
        return self._tensors.keys()

    def param_count(self) -> int:
        return sum(t.numel() for t in self._tensors.values())


def _normalise(t: torch.Tensor, kind: str) -> torch.Tensor:
    if kind == "int":
        return t.to(torch.int32)
    if t.dtype == torch.float16:
        return t.to(torch.float32)
    return t


def check_against_manifest(source: str, found: Mapping[str, Tuple[Tuple[int, ...], str]],
                           manifest: Mapping[str, TensorSpec]) -> None:
    """Raise one WeightsError for everything in `found` ({name: (shape, dtype name)}) that
    does not fit `manifest`."""
    missing = [n for n in manifest if n not in found]
    unexpected = [n for n in found if n not in manifest]
    wrong_shape, wrong_dtype = [], []
    for n, spec in manifest.items():
        if n not in found:
            continue
        shape, dt = found[n]
        if tuple(shape) != tuple(spec.shape):
            wrong_shape.append((n, tuple(spec.shape), tuple(shape)))
        ok = _FLOAT_NAMES if spec.kind == "float" else _INT_NAMES
        if dt not in ok:
            wrong_dtype.append((n, dt))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightsError(source, missing, unexpected, wrong_shape, wrong_dtype)


def _checkpoint_files(model_dir: str):
    """The safetensors files of a model folder: `model.safetensors`, or, for a checkpoint in
    shards, the files that `model.safetensors.index.json` names (its `weight_map` gives the shard
    of every tensor; the reference reads a single file only, crates/engine/src/weights.rs:139-150).
    Returns (source name for messages, [paths])."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.exists(single) or not os.path.exists(index):
        return single, [single]
    try:
        with open(index) as f:
            weight_map = json.load(f)["weight_map"]
        shards = sorted(set(weight_map.values()))
        if not shards or not all(isinstance(x, str) for x in shards):
            raise ValueError("empty weight_map")
    except (OSError, ValueError, KeyError, TypeError, AttributeError) as e:
        raise WeightsFormatError(f"{index}: not a shard index ({type(e).__name__}: {e})") from None
    return index, [os.path.join(model_dir, os.path.basename(x)) for x in shards]


def load_safetensors_weights(model_dir: str, manifest: Mapping[str, TensorSpec],
                             device: Optional[str] = None) -> WeightSet:
    """Read <model_dir>/model.safetensors (or the shards its index names), check what was found
    against the manifest, return a WeightSet.

    With `device`, tensors are copied there (the file mappings are not kept); without, they are
    private CPU copies."""
    source, paths = _checkpoint_files(model_dir)
    files = [SafetensorsFile(p) for p in paths]
    where, found, twice = {}, {}, []
    for f in files:
        for n in f.names():
            if n in where:
                twice.append(n)
            where[n] = f
            found[n] = (f.shape(n), f.dtype_name(n))
    if twice:
        raise WeightsError(source, other=["stored in more than one shard: " + ", ".join(sorted(twice))])
    check_against_manifest(source, found, manifest)
    out = {}
    for n, spec in manifest.items():
        t = _normalise(where[n].tensor(n), spec.kind)
        out[n] = t.to(device) if device is not None else t.clone()
    for f in files:
        f.close()
    return WeightSet(out, source)


def weights_from_tensors(tensors: Mapping[str, torch.Tensor], manifest: Mapping[str, TensorSpec],
                         source: str = "<tensors>") -> WeightSet:
    """The same check for tensors already in memory (random weights made on the device)."""
    names = {torch.bfloat16: "BF16", torch.float16: "F16", torch.float32: "F32", torch.int32: "I32",
             torch.int64: "I64", torch.int16: "I16", torch.int8: "I8", torch.uint8: "U8"}
    found = {n: (tuple(t.shape), names.get(t.dtype, str(t.dtype))) for n, t in tensors.items()}
    check_against_manifest(source, found, manifest)
    return WeightSet({n: _normalise(tensors[n], manifest[n].kind) for n in manifest}, source)
