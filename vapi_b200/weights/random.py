"""Random-weights mode: write a model folder from a configuration and a seed.

The folder holds ``config.json`` and ``model.safetensors`` with every tensor the
architecture's plan names, so the ordinary loader path is what reads it back.  Each tensor
is drawn from its own generator, seeded from ``seed`` and the tensor's name, so the values
do not depend on the order of the plan.  Matrices, biases and conv taps are N(0, ``std``)
(0.02, the reference's benches use the same, examples/gemm_bench.rs:26-27); norm weights
are 1, or 1 + 0.1 N(0,1) with ``norm_init="perturbed"`` (what the reference's golden
generator does, tools/gen_lfm2_goldens.py:27-49) so that a test can tell a missing norm
weight from a present one.
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Any, Dict, Optional

import torch

from ..config.model import resolve_architecture


def _gen(seed: int, name: str, device: str = "cpu") -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(((int(seed) & 0xFFFFFFFF) * 1_000_003 + zlib.crc32(name.encode())) & 0x7FFF_FFFF_FFFF_FFFF)
    return g


def random_tensors(plan, seed: int, std: float = 0.02, norm_init: str = "ones",
                   dtype: torch.dtype = torch.float32, device: str = "cpu") -> Dict[str, torch.Tensor]:
    """Every tensor of ``plan``, drawn on ``device`` (the values of a CPU draw and of a CUDA
    draw differ; a folder is always written from a CPU draw)."""
    out: Dict[str, torch.Tensor] = {}
    dev = str(torch.device(device))
    for spec in plan.tensor_specs():
        g = _gen(seed, spec.name, dev)
        if spec.role == "table":
            out[spec.name] = torch.zeros(spec.shape, dtype=torch.int32, device=dev)
            continue
        if spec.init == "ones":
            t = torch.ones(spec.shape, dtype=torch.float32, device=dev)
            if norm_init == "perturbed":
                t = t + 0.1 * torch.randn(spec.shape, generator=g, dtype=torch.float32, device=dev)
        elif spec.init == "zeros":
            t = torch.zeros(spec.shape, dtype=torch.float32, device=dev)
        else:
            t = torch.randn(spec.shape, generator=g, dtype=torch.float32, device=dev).mul_(std)
        out[spec.name] = t.to(dtype).contiguous()
    return out


def write_random_model(out_dir: str, config_json: Dict[str, Any], seed: int, *, std: float = 0.02,
                       norm_init: str = "ones", dtype: torch.dtype = torch.float32,
                       overrides: Optional[Dict[str, torch.Tensor]] = None) -> str:
    """Write ``config.json`` (as given) and ``model.safetensors`` into ``out_dir``.

    ``overrides`` replaces named tensors after the random draw (tests use it to plant a
    value that makes a fault visible)."""
    from safetensors.torch import save_file

    arch = resolve_architecture(config_json)
    plan = arch.plan(arch.parse(config_json))
    tensors = random_tensors(plan, seed, std, norm_init, dtype)
    for k, v in (overrides or {}).items():
        if k not in tensors or tuple(tensors[k].shape) != tuple(v.shape):
            raise KeyError(f"override `{k}` does not match a tensor of the model")
        tensors[k] = v.to(tensors[k].dtype).contiguous()
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config_json, f, indent=1)
    save_file(tensors, os.path.join(out_dir, "model.safetensors"), metadata={"format": "pt"})
    return out_dir
