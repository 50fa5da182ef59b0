"""Converter: a checkpoint file of the reference's training loop -> a model folder of this library.

The reference saves ``torch.save({"model": state_dict, "optimizer": ..., "loader": ..., "step": ...,
"config": asdict(config)})`` (src/common.py:85-93) and generates from such a file by building the model from
``checkpoint["config"]`` and loading ``checkpoint["model"]`` by name (scripts/generate.py:33-37).  Its tensor
names are the names this library's parts expect, and its flat config dictionary holds this library's
config.json keys, so the conversion is: read the two entries, check them against the architecture, write
``config.json`` and ``model.safetensors``.  The optimizer and loader states are not read.

    python -m gtar_kimik3_public_b200.weights.convert CKPT.pt FOLDER [--arch transformer] [--dtype bfloat16]
        [--max-position-embeddings N]
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

from ..registry import architecture, config_from_dict
from .loader import check_tensors
from .safetensors_io import write_safetensors

_PREFIXES = ("_orig_mod.", "module.")  # what torch.compile and DistributedDataParallel put before a name


def convert_checkpoint(checkpoint_path: str | Path, folder: str | Path, arch: str = "transformer",
                       matrix_dtype: torch.dtype | None = None, extra_config: dict | None = None) -> Path:
    """Writes ``folder/config.json`` and ``folder/model.safetensors`` from the checkpoint; returns the folder.

    ``matrix_dtype``: None keeps every tensor as stored (the reference trains in 32-bit, so the folder is then
    32-bit); ``torch.bfloat16`` rounds the matrices once, which is what the reference's engine does at every
    projection (src/engine.py:35) and what this library's bfloat16 kernels want.  Vectors stay as stored.
    ``extra_config``: keys the checkpoint's config does not carry (``max_position_embeddings``, ``eos_token_id``).
    """
    from ..models.model import Model

    checkpoint = torch.load(str(checkpoint_path), map_location="cpu", weights_only=True)
    for key in ("model", "config"):
        if key not in checkpoint:
            raise ValueError(f"{checkpoint_path} has no {key!r} entry; it holds {sorted(checkpoint)}")
    config = config_from_dict({"arch": arch, **checkpoint["config"], **(extra_config or {})})
    state = {}
    for name, tensor in checkpoint["model"].items():
        for prefix in _PREFIXES:
            while name.startswith(prefix):
                name = name[len(prefix):]
        state[name] = tensor.detach()
    specs = Model(architecture(arch).build_plan(config), config, torch.float32, "cpu").tensor_specs()
    check_tensors(checkpoint_path, specs, {n: tuple(t.shape) for n, t in state.items()}, {n: t.dtype for n, t in state.items()})
    tensors = {}
    for name, spec in specs.items():
        if name not in state:
            continue  # optional and absent
        tensor = state[name].contiguous()
        if matrix_dtype is not None and spec.kind == "matrix":
            tensor = tensor.to(matrix_dtype)
        tensors[name] = tensor.clone()  # a tied head shares its storage with the embedding in the checkpoint
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config.to_dict(), indent=2) + "\n")
    write_safetensors(folder / "model.safetensors", tensors, {"format": "pt", "source": Path(checkpoint_path).name,
                                                             "step": str(checkpoint.get("step", ""))})
    return folder


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description="turn a checkpoint of the reference's training loop into a model folder")
    parser.add_argument("checkpoint")
    parser.add_argument("folder")
    parser.add_argument("--arch", default="transformer")
    parser.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "as-stored"], help="type of the matrices in the folder")
    parser.add_argument("--max-position-embeddings", type=int, default=None)
    parser.add_argument("--eos-token-id", type=int, default=None)
    args = parser.parse_args(argv)
    extra = {k: v for k, v in (("max_position_embeddings", args.max_position_embeddings), ("eos_token_id", args.eos_token_id))
             if v is not None}
    folder = convert_checkpoint(args.checkpoint, args.folder, args.arch,
                                torch.bfloat16 if args.dtype == "bfloat16" else None, extra)
    print(f"wrote {folder}/config.json and {folder}/model.safetensors")
    return 0


if __name__ == "__main__":
    sys.exit(main())
