"""Loads a model folder's tensors into a model, by name, after checking the whole file.

The check compares the names and shapes the model's parts expect with what the file holds and
raises ONE error that lists every missing tensor, every unexpected tensor and every wrong
shape — before anything is copied to the device.  (The reference loads strictly by name,
scripts/generate.py:37, and its tolerant loader lists missing and unexpected keys,
src/common.py:111-125.)

Dtype rule.  In a bfloat16 run, floating-point tensors are kept in bfloat16, except that a
tensor stored in 32-bit stays 32-bit; integer tables become int32.  In a float32 run every
floating-point tensor is widened to float32.  A *matrix* that stays 32-bit in a bfloat16 run sends
its projection through the 32-bit kernel, which is exact and some hundred times slower than the
tensor cores: the loader says so once (a warning), and ``cast_matrices=True`` rounds such matrices
to bfloat16 at load instead, which is what the reference's engine does with its 32-bit parameters
at every projection (torch.autocast, src/engine.py:35).  Vectors (norm weights) stay 32-bit either way.
"""

from __future__ import annotations

import warnings
from pathlib import Path

import torch

from ..parts.base import TensorSpec
from .safetensors_io import ModelFolderTensors

_FLOATS = (torch.float64, torch.float32, torch.float16, torch.bfloat16)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


class WeightsError(ValueError):
    """The tensors of a model folder do not fit the model; ``missing``, ``unexpected`` and
    ``wrong_shape`` hold the details that the message lists."""

    def __init__(self, folder, missing, unexpected, wrong_shape, wrong_kind=()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_kind = list(wrong_shape), list(wrong_kind)
        lines = [f"weights in {folder} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{name} is {list(got)}, expected {list(want)}" for name, got, want in self.wrong_shape))
        if self.wrong_kind:
            lines.append(f"  wrong type ({len(self.wrong_kind)}): " + ", ".join(
                f"{name} is {got}, expected {want}" for name, got, want in self.wrong_kind))
        super().__init__("\n".join(lines))


def check_tensors(folder, specs: dict[str, TensorSpec], have_shapes: dict[str, tuple], have_dtypes: dict[str, torch.dtype]) -> None:
    missing = [n for n, s in specs.items() if n not in have_shapes and not s.optional]
    unexpected = [n for n in have_shapes if n not in specs]
    wrong_shape = [(n, have_shapes[n], s.shape) for n, s in specs.items() if n in have_shapes and tuple(have_shapes[n]) != tuple(s.shape)]
    wrong_kind = []
    for name, spec in specs.items():
        if name not in have_dtypes:
            continue
        dtype = have_dtypes[name]
        if spec.kind == "table" and dtype not in _INTS:
            wrong_kind.append((name, str(dtype), "an integer type"))
        if spec.kind != "table" and dtype not in _FLOATS:
            wrong_kind.append((name, str(dtype), "a floating-point type"))
    if missing or unexpected or wrong_shape or wrong_kind:
        raise WeightsError(folder, missing, unexpected, wrong_shape, wrong_kind)


def stored_dtype_rule(stored: torch.dtype, kind: str, run_dtype: torch.dtype, cast_matrices: bool = False) -> torch.dtype:
    """The dtype a tensor is kept in on the device."""
    if kind == "table":
        return torch.int32
    if run_dtype == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64) and not (cast_matrices and kind == "matrix"):
        return torch.float32
    return torch.bfloat16


def load_weights(model, folder: str | Path, cast_matrices: bool = False) -> None:
    """Checks the folder against ``model.tensor_specs()`` and hands the tensors to the parts."""
    files = ModelFolderTensors(folder)
    specs = model.tensor_specs()
    names = files.names()
    check_tensors(folder, specs, {n: files.shape(n) for n in names}, {n: files.dtype(n) for n in names})
    tensors = {}
    slow = []
    for name, spec in specs.items():
        if name not in files.where:
            continue  # optional and absent
        host = files.tensor(name)
        keep = stored_dtype_rule(host.dtype, spec.kind, model.dtype, cast_matrices)
        if spec.kind == "matrix" and keep == torch.float32 and model.dtype == torch.bfloat16:
            slow.append(name)
        tensors[name] = host.to(device=model.device, dtype=keep)
    if slow:
        warnings.warn(
            f"{len(slow)} matrices of {folder} are stored in 32-bit and stay so in this bfloat16 run ({slow[0]}, ...): "
            "their projections run on the 32-bit kernel, far slower than the tensor cores.  Load with "
            "cast_matrices=True (command line: --cast-matrices) to round them to bfloat16 once, as the reference's "
            "autocast does at every projection.", stacklevel=2)
    model.load(tensors)
