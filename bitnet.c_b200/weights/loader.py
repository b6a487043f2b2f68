"""Loading a model's tensors from safetensors by name.

The model says which parameters it has and of what shape (``parameter_table``);
the architecture says what each is called in the file.  Everything that does not
fit is collected and reported in one error: tensors the model needs and the
file lacks, tensors the file holds and the model does not know, and tensors of
the wrong shape or kind.  The reference stops at the first missing tensor
(``"Tensor not found" name=...``, src/model.c:1043-1045) and checks rank and
type per tensor (src/model.c:135-187).

Storage types: a tensor stored in bfloat16 stays bfloat16, one stored in 32-bit
floating point stays 32-bit, half precision is converted to the compute type,
integer tables become int32.  With ``dtype=float32`` every floating tensor is
widened to 32-bit so that the whole model runs in true single precision.
"""
from __future__ import annotations

import json
import os
import warnings
from typing import Callable, Dict, List, Mapping

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile


class WeightsError(ValueError):
    """Raised once per load with every problem found; see ``missing``, ``unexpected``, ``mismatched``."""

    def __init__(self, where: str, missing: List[str], unexpected: List[str], mismatched: List[str],
                 other: List[str] = ()):
        self.missing, self.unexpected, self.mismatched, self.other = missing, unexpected, mismatched, list(other)
        lines = [f"weights in '{where}' do not fit the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if mismatched:
            lines.append(f"  wrong shape or type ({len(mismatched)}): " + "; ".join(mismatched))
        for o in self.other:
            lines.append("  " + o)
        super().__init__("\n".join(lines))


def _open_files(model_dir: str) -> List[SafetensorsFile]:
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(single):
        return [SafetensorsFile(single)]
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            weight_map = json.load(f).get("weight_map", {})
        shards = sorted(set(weight_map.values()))
        if not shards:
            raise WeightsError(model_dir, [], [], [], [f"'{index}' names no shard"])
        absent = [s for s in shards if not os.path.isfile(os.path.join(model_dir, s))]
        if absent:
            raise WeightsError(model_dir, [], [], [], [f"'{index}' names shards that are not in the folder: "
                                                       + ", ".join(absent)])
        return [SafetensorsFile(os.path.join(model_dir, s)) for s in shards]
    raise WeightsError(model_dir, [], [], [], ["no model.safetensors and no model.safetensors.index.json"])


def stored_dtype_to_kept(stored: torch.dtype, compute: torch.dtype, integer: bool) -> torch.dtype:
    if integer:
        return torch.int32
    if compute == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def load_weights(model_dir: str, table: Mapping[str, "ParamSpec"], tensor_name: Callable[[str], str],
                 dtype: torch.dtype, device) -> Dict[str, torch.Tensor]:
    """Read every parameter of ``table`` (path -> ParamSpec) and return path -> tensor on ``device``."""
    if not os.path.isdir(model_dir):
        raise WeightsError(model_dir, [], [], [], ["not a folder"])
    try:
        files = _open_files(model_dir)
    except SafetensorsError as e:
        raise WeightsError(model_dir, [], [], [], [str(e)]) from None
    try:
        where: Dict[str, SafetensorsFile] = {}
        dup: List[str] = []
        for f in files:
            for n in f.names():
                if n in where:
                    dup.append(f"tensor '{n}' is stored in two shards")
                where[n] = f
        wanted = {tensor_name(path): path for path in table}
        missing = sorted(n for n, path in wanted.items() if n not in where and not table[path].optional)
        unexpected = sorted(n for n in where if n not in wanted)
        mismatched: List[str] = []
        for n, path in wanted.items():
            if n not in where:
                continue
            e = where[n].entries[n]
            p = table[path]
            is_int = e.dtype in ("I64", "I32", "I16", "I8", "U8", "BOOL")
            if tuple(e.shape) != tuple(p.shape):
                mismatched.append(f"{n}: file has {list(e.shape)}, model needs {list(p.shape)}")
            elif is_int != bool(p.integer):
                mismatched.append(f"{n}: file has {e.dtype}, model needs "
                                  f"{'an integer table' if p.integer else 'floating point'}")
        if missing or unexpected or mismatched or dup:
            raise WeightsError(model_dir, missing, unexpected, mismatched, dup)
        out: Dict[str, torch.Tensor] = {}
        wide: List[str] = []
        for n, path in wanted.items():
            if n not in where:  # an optional tensor that this file does not have
                out[path] = None
                continue
            t = where[n].read(n)
            keep = stored_dtype_to_kept(t.dtype, dtype, bool(table[path].integer))
            if keep == torch.float32 and dtype == torch.bfloat16 and t.dim() >= 2:
                wide.append(n)
            out[path] = t.to(device=device, dtype=keep).contiguous()
        if wide:
            # a tensor stored in 32-bit stays 32-bit; say what that costs instead of doing it silently
            warnings.warn(f"'{model_dir}': {len(wide)} matrices are stored in 32-bit floating point and are kept so "
                          f"in this bfloat16 model (first: {wide[0]}): they take twice the memory and their products "
                          "run in float32 on the slower kernels; store them in bfloat16 to avoid that", stacklevel=2)
        return out
    finally:
        for f in files:
            f.close()
