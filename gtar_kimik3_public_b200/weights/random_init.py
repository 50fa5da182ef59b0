"""Random-weights mode: writes a model folder (config.json, model.safetensors) from a
configuration and a seed.

Values: projection matrices and the embedding are N(0, initializer_range) (the reference's
init, src/models/transformer.py:80-84; the narrower init of the residual projections,
:85-87, is a training aid and is not copied); norm weights are 1 + N(0, 0.1) rather than the
reference's ones (src/layers/rmsnorm.py:8) so that a dropped or misplaced norm weight changes
the output.  Matrices are stored in bfloat16 and vectors in float32 unless asked otherwise, so
a float32 run and a bfloat16 run of the folder use the very same values.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

from ..config.base import ModelConfig
from ..registry import architecture
from .safetensors_io import write_safetensors


def random_tensors(specs, seed: int, std: float, matrix_dtype=torch.bfloat16, vector_dtype=torch.float32):
    """One generator, tensors drawn in the order of ``specs`` (optional ones are not written)."""
    gen = torch.Generator().manual_seed(int(seed))
    out = {}
    for name, spec in specs.items():
        if spec.optional:
            continue
        if spec.kind == "table":
            out[name] = torch.randint(0, 2**15, spec.shape, generator=gen, dtype=torch.int32)
        elif spec.kind == "vector":
            out[name] = (1.0 + 0.1 * torch.randn(spec.shape, generator=gen)).to(vector_dtype)
        else:
            # drawn row block by row block so that a 150k x 4k table needs no second full-size buffer
            t = torch.empty(spec.shape, dtype=matrix_dtype)
            rows = spec.shape[0]
            step = max(1, (1 << 24) // max(1, t[0].numel()))
            for start in range(0, rows, step):
                block = torch.randn((min(step, rows - start), *spec.shape[1:]), generator=gen) * std
                t[start:start + block.shape[0]] = block.to(matrix_dtype)
            out[name] = t
    return out


def write_random_model(folder: str | Path, config: ModelConfig, seed: int, std: float | None = None,
                       matrix_dtype=torch.bfloat16, vector_dtype=torch.float32) -> Path:
    """Writes ``folder/config.json`` and ``folder/model.safetensors``; returns the folder."""
    from ..models.model import Model  # local: models imports weights' siblings

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    if std is None:
        std = getattr(config, "initializer_range", None)
        if std is None:
            raise ValueError("the configuration has no initializer_range; pass std")
    arch = architecture(config.ARCH_NAMES[0])
    specs = Model(arch.build_plan(config), config, torch.float32, "cpu").tensor_specs()
    tensors = random_tensors(specs, seed, std, matrix_dtype, vector_dtype)
    (folder / "config.json").write_text(json.dumps(config.to_dict(), indent=2) + "\n")
    write_safetensors(folder / "model.safetensors", tensors, {"format": "pt", "seed": str(seed)})
    return folder


def load_random_weights(model, seed: int, std: float | None = None) -> None:
    """Fills a model with random weights drawn on its own device (no folder in between): for sizes at which
    writing and reading a model folder would take minutes.  The values follow the same rule as
    ``write_random_model`` (matrices N(0, std) in bfloat16, vectors 1 + N(0, 0.1) in float32) but come from the
    device's generator, so they are not the numbers that a folder of the same seed holds."""
    from .loader import stored_dtype_rule

    if std is None:
        std = getattr(model.config, "initializer_range", None)
        if std is None:
            raise ValueError("the configuration has no initializer_range; pass std")
    gen = torch.Generator(device=model.device).manual_seed(int(seed))
    tensors = {}
    for name, spec in model.tensor_specs().items():
        if spec.optional:
            continue
        if spec.kind == "table":
            tensors[name] = torch.randint(0, 2**15, spec.shape, generator=gen, dtype=torch.int32, device=model.device)
        elif spec.kind == "vector":
            keep = stored_dtype_rule(torch.float32, spec.kind, model.dtype)
            tensors[name] = (1.0 + 0.1 * torch.randn(spec.shape, generator=gen, device=model.device)).to(keep)
        else:
            keep = stored_dtype_rule(torch.bfloat16, spec.kind, model.dtype)
            t = torch.empty(spec.shape, dtype=keep, device=model.device)
            rows = spec.shape[0]
            step = max(1, (1 << 26) // max(1, t[0].numel()))
            for start in range(0, rows, step):  # row blocks: no second full-size 32-bit buffer
                n = min(step, rows - start)
                t[start:start + n] = (torch.randn((n, *spec.shape[1:]), generator=gen, device=model.device) * std).to(keep)
            tensors[name] = t
    model.load(tensors)
