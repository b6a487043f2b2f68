"""Seeded random weights, and the random-weights mode that writes a model folder.

Values come from a counter-based generator: element ``i`` of the tensor named
``n`` under seed ``s`` is a pure function of ``(s, n, i)``, so tensors can be made
in any order, in pieces, and again later, and always come out the same.  The
reference has no such mode (its models are GGUF files only, src/main.c:110-168).
"""
from __future__ import annotations

import json
import math
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


def _signed(x: int) -> int:
    """The 64-bit pattern ``x`` as a signed integer (torch has no unsigned 64-bit arithmetic;
    signed products and sums wrap to the same bits)."""
    x &= _MASK64
    return x - (1 << 64) if x >> 63 else x


def _lsr(x: torch.Tensor, n: int) -> torch.Tensor:
    """Logical right shift of int64 bit patterns."""
    return (x >> n) & ((1 << (64 - n)) - 1)


def standard_normal_on(device, seed: int, name: str, count: int, start: int = 0) -> torch.Tensor:
    """``standard_normal`` restated in torch, for tensors too large to draw on the host: the same
    function of ``(seed, name, index)``, evaluated on ``device``.  The integer part is bit-exact;
    the float64 logarithm and cosine are the device's, so a value may differ from the host's in
    its last float32 bit now and then."""
    key = _signed(stream_key(seed, name))
    idx = torch.arange(start, start + count, dtype=torch.int64, device=device)
    x = idx * _signed(int(_GOLDEN)) + key
    x = (x ^ _lsr(x, 30)) * _signed(int(_M1))
    x = (x ^ _lsr(x, 27)) * _signed(int(_M2))
    h = x ^ _lsr(x, 31)
    u1 = (_lsr(h, 40).to(torch.float64) + 1.0) * (1.0 / 16777216.0)
    u2 = (_lsr(h, 16) & 0xFFFFFF).to(torch.float64) * (1.0 / 16777216.0)
    z = torch.sqrt(-2.0 * torch.log(u1)) * torch.cos(2.0 * math.pi * u2)
    return z.to(torch.float32)


def random_tensor(seed: int, name: str, shape, mean: float, std: float, dtype: torch.dtype, device=None) -> torch.Tensor:
    """Tensor ``name`` under ``seed``: mean + std * standard normal, computed in float32 and then
    rounded to ``dtype``.  Without ``device`` the values are drawn on the host with NumPy; with one
    they are drawn there (``standard_normal_on``) and the tensor stays there."""
    n = int(np.prod(shape)) if len(shape) else 1
    if std == 0.0:
        return torch.full(tuple(shape), mean, dtype=dtype, device=device)
    if device is not None:
        out_t = torch.empty(n, dtype=dtype, device=device)
        step = 1 << 24
        for s in range(0, n, step):
            c = min(step, n - s)
            out_t[s:s + c] = standard_normal_on(device, seed, name, c, s) * std + mean
        return out_t.reshape(tuple(shape))
    out = np.empty(n, dtype=np.float32)
    step = 1 << 22
    for s in range(0, n, step):
        c = min(step, n - s)
        out[s:s + c] = standard_normal(seed, name, c, s) * np.float32(std) + np.float32(mean)
    return torch.from_numpy(out).reshape(tuple(shape)).to(dtype)


def random_parameters(spec, tensor_name, seed: int, dtype: torch.dtype, matrix_std: float = 0.02,
                      norm_std: float = 0.1, device=None):
    """Yield ``(path, name, tensor)`` for every parameter of a model of ``spec``: matrices and the
    embedding N(0, matrix_std), norm gains 1 + N(0, norm_std), integer tables zero.  The values
    depend on the seed and on the tensor's name in the file only."""
    from ..engine.model import parameter_table
    for path, p in parameter_table(spec).items():
        name = tensor_name(path)
        if p.init == "ones":
            yield path, name, random_tensor(seed, name, p.shape, 1.0, norm_std, dtype, device)
        elif p.init == "normal":
            yield path, name, random_tensor(seed, name, p.shape, 0.0, matrix_std, dtype, device)
        elif p.init == "zeros":
            yield path, name, torch.zeros(p.shape, dtype=torch.int32 if p.integer else dtype, device=device)
        else:
            raise ValueError(f"parameter '{path}' has unknown init '{p.init}'")


def write_random_model(folder: str, config: Dict[str, Any], seed: int, dtype: str = "bfloat16",
                       matrix_std: float = 0.02, norm_std: float = 0.1, device=None) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` under ``folder``.

    Matrices and the embedding are N(0, matrix_std); norm gains are 1 + N(0, norm_std).
    ``dtype`` is the storage type of the file: ``bfloat16`` or ``float32``.  ``device``: draw the
    values there instead of on the host (large models; see ``standard_normal_on``).
    """
    from ..config import architecture_of
    from .safetensors_io import write_safetensors

    store = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    arch = architecture_of(config)
    cfg = arch.read_config(config)
    spec = arch.to_spec(cfg)
    os.makedirs(folder, exist_ok=True)

    def tensors():
        for _path, name, t in random_parameters(spec, arch.tensor_name, seed, store, matrix_std, norm_std, device):
            yield name, t

    write_safetensors(os.path.join(folder, "model.safetensors"), tensors(),
                      metadata={"format": "pt", "seed": str(seed)})
    out = dict(arch.config_to_dict(cfg))
    out["torch_dtype"] = dtype
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(out, f, indent=1)
    return folder
