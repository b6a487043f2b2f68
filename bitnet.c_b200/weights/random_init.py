"""Seeded random weights, and the random-weights mode that writes a model folder.

Values come from a counter-based generator: element ``i`` of the tensor named
``n`` under seed ``s`` is a pure function of ``(s, n, i)``, so tensors can be made
in any order, in pieces, and again later, and always come out the same.  The
reference has no such mode (its models are GGUF files only, src/main.c:110-168).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict

import numpy as np
import torch

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)
_MASK64 = (1 << 64) - 1


def _mix_int(x: int) -> int:
    x &= _MASK64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK64
    return x ^ (x >> 31)


def _mix(x: np.ndarray) -> np.ndarray:
    x = (x ^ (x >> np.uint64(30))) * _M1
    x = (x ^ (x >> np.uint64(27))) * _M2
    return x ^ (x >> np.uint64(31))


def name_key(name: str) -> int:
    """FNV-1a over the tensor's name: the tensor's stream within a seed."""
    h = 0xCBF29CE484222325
    for b in name.encode("utf-8"):
        h = ((h ^ b) * 0x100000001B3) & _MASK64
    return h


def stream_key(seed: int, name: str) -> int:
    return _mix_int(_mix_int(seed) ^ name_key(name))


def standard_normal(seed: int, name: str, count: int, start: int = 0) -> np.ndarray:
    """``count`` standard normal values (float32) of tensor ``name`` from element ``start``."""
    key = np.uint64(stream_key(seed, name))
    with np.errstate(over="ignore"):
        idx = np.arange(start, start + count, dtype=np.uint64)
        h = _mix(key + idx * _GOLDEN)
    u1 = ((h >> np.uint64(40)).astype(np.float64) + 1.0) * (1.0 / 16777216.0)  # (0, 1]
    u2 = ((h >> np.uint64(16)) & np.uint64(0xFFFFFF)).astype(np.float64) * (1.0 / 16777216.0)  # [0, 1)
    z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return z.astype(np.float32)


def random_tensor(seed: int, name: str, shape, mean: float, std: float, dtype: torch.dtype) -> torch.Tensor:
    n = int(np.prod(shape)) if len(shape) else 1
    if std == 0.0:
        return torch.full(tuple(shape), mean, dtype=dtype)
    out = np.empty(n, dtype=np.float32)
    step = 1 << 22
    for s in range(0, n, step):
        c = min(step, n - s)
        out[s:s + c] = standard_normal(seed, name, c, s) * np.float32(std) + np.float32(mean)
    return torch.from_numpy(out).reshape(tuple(shape)).to(dtype)


def write_random_model(folder: str, config: Dict[str, Any], seed: int, dtype: str = "bfloat16",
                       matrix_std: float = 0.02, norm_std: float = 0.1) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` under ``folder``.

    Matrices and the embedding are N(0, matrix_std); norm gains are 1 + N(0, norm_std).
    ``dtype`` is the storage type of the file: ``bfloat16`` or ``float32``.
    """
    from ..config import architecture_of
    from ..engine.model import parameter_table
    from .safetensors_io import write_safetensors

    store = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    arch = architecture_of(config)
    cfg = arch.read_config(config)
    spec = arch.to_spec(cfg)
    os.makedirs(folder, exist_ok=True)

    def tensors():
        for path, p in parameter_table(spec).items():
            name = arch.tensor_name(path)
            if p.init == "ones":
                yield name, random_tensor(seed, name, p.shape, 1.0, norm_std, store)
            elif p.init == "normal":
                yield name, random_tensor(seed, name, p.shape, 0.0, matrix_std, store)
            elif p.init == "zeros":
                yield name, torch.zeros(p.shape, dtype=torch.int32 if p.integer else store)
            else:
                raise ValueError(f"parameter '{path}' has unknown init '{p.init}'")

    write_safetensors(os.path.join(folder, "model.safetensors"), tensors(),
                      metadata={"format": "pt", "seed": str(seed)})
    out = dict(arch.config_to_dict(cfg))
    out["torch_dtype"] = dtype
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(out, f, indent=1)
    return folder
