"""Weights from safetensors, by tensor name.

Files are found as the reference finds them
(crates/vapi-backend-candle/src/backend.rs:115-143): ``model.safetensors.index.json`` lists
shards in its ``weight_map``; otherwise a single ``model.safetensors``.  Every tensor a plan
names is fetched by name and checked against the shape the plan expects; all problems of a
checkpoint are reported together in one :class:`WeightError`.

Run-time dtypes: with ``dtype=bfloat16`` a matrix stored in 16 bits is held as bfloat16, a
matrix stored in 32 bits stays float32 (its products then run in float32); with
``dtype=float32`` everything is float32.  Small vectors are always float32 for the kernels
(widening bfloat16 is exact) and integer tables are int32.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Iterable, List, Sequence, Tuple

import torch

from ..parts.base import TensorSpec

_INT_DTYPES = (torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8, torch.bool)


class WeightError(RuntimeError):
    """A checkpoint that does not fit the model: lists missing, unexpected and misshapen tensors."""

    def __init__(self, where: str, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 other: Sequence[str] = ()):
        self.missing, self.unexpected, self.wrong_shape, self.other = list(missing), list(unexpected), list(wrong_shape), list(other)
        lines = [f"{where}: the checkpoint does not fit the model"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: file has {list(got)}, model wants {list(want)}" for n, got, want in self.wrong_shape))
        for o in self.other:
            lines.append("  " + o)
        super().__init__("\n".join(lines))


def weight_files(model_dir: str) -> List[str]:
    index = os.path.join(model_dir, "model.safetensors.index.json")
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            wm = json.load(f).get("weight_map")
        if not isinstance(wm, dict) or not wm:
            raise WeightError(index, [], [], [], ["the index has an empty weight_map"])
        return [os.path.join(model_dir, n) for n in sorted(set(str(v) for v in wm.values()))]
    if os.path.isfile(single):
        return [single]
    raise WeightError(model_dir, [], [], [], ["no model.safetensors or model.safetensors.index.json"])


def _runtime_dtype(spec: TensorSpec, stored: torch.dtype, dtype: torch.dtype) -> torch.dtype:
    if spec.role == "table" or stored in _INT_DTYPES:
        return torch.int32
    if spec.role == "vector":
        return torch.float32
    if dtype == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32          # stored in 32 bits: stays so
    return dtype


def load_tensors(model_dir: str, specs: Iterable[TensorSpec], dtype: torch.dtype,
                 device: torch.device | str, strict_unexpected: bool = True) -> Dict[str, torch.Tensor]:
    """Read every tensor ``specs`` names, check shapes, convert and move to ``device``."""
    from safetensors import safe_open

    specs = list(specs)
    files = weight_files(model_dir)
    where: Dict[str, str] = {}
    handles = {}
    for path in files:
        if not os.path.isfile(path):
            raise WeightError(model_dir, [], [], [], [f"shard {os.path.basename(path)} named by the index is absent"])
        h = safe_open(path, framework="pt", device="cpu")
        handles[path] = h
        for k in h.keys():
            where[k] = path
    wanted = {s.name: s for s in specs}
    missing = [s.name for s in specs if s.name not in where and not s.optional]
    unexpected = sorted(k for k in where if k not in wanted) if strict_unexpected else []
    wrong = []
    for s in specs:
        if s.name in where:
            got = tuple(handles[where[s.name]].get_slice(s.name).get_shape())
            if got != tuple(s.shape):
                wrong.append((s.name, got, tuple(s.shape)))
    if missing or unexpected or wrong:
        raise WeightError(model_dir, missing, unexpected, wrong)
    out: Dict[str, torch.Tensor] = {}
    for s in specs:
        if s.name not in where:
            continue
        t = handles[where[s.name]].get_tensor(s.name)
        out[s.name] = t.to(_runtime_dtype(s, t.dtype, dtype)).to(device).contiguous()
    return out
