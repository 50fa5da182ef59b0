"""The Python entry point: load a model folder, generate.

The reference's programming interface is ``Engine(model).generate(input_ids, max_new_tokens,
temperature, top_k, eos_token_id)`` (src/engine.py:22-29); its ``src/generate.py`` is an empty
file.  The option names and meanings are kept: ``temperature`` (0 = greedy), ``top_k`` (None =
off), ``eos_token_id`` (here also a set, ``stop_ids``), ``max_new_tokens``, and the command line's
``seed``.  Prompts are lists of token ids of any lengths; the result is a list of token lists.
"""

from __future__ import annotations

from pathlib import Path
from typing import Sequence

import torch

from .cache import rounded_tokens
from .engine.engine import Engine
from .engine.generation import DeviceChooser, GenerationParams, run_generation
from .models.model import Model
from .registry import architecture, config_from_file
from .sampling.sampler import SamplingParams, choose
from .weights.loader import load_weights

_DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16, torch.bfloat16: torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32, torch.float32: torch.float32,
}


def parse_dtype(name) -> torch.dtype:
    try:
        return _DTYPES[name]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got {name!r}") from None


def load(model_dir: str | Path, dtype="bfloat16", device: str | torch.device = "cuda:0",
         cast_matrices: bool = False) -> Model:
    """Builds the model class that ``model_dir/config.json`` names and loads its safetensors.
    ``cast_matrices``: in a bfloat16 run, round matrices that the file stores in 32-bit to bfloat16
    (by default they stay 32-bit and their projections run on the slow, exact 32-bit kernel)."""
    config = config_from_file(model_dir)
    arch = architecture(config.ARCH_NAMES[0])
    model = Model(arch.build_plan(config), config, parse_dtype(dtype), device)
    load_weights(model, model_dir, cast_matrices=cast_matrices)
    return model


class Generator:
    """A loaded model with a cache, ready to generate: the successor of the reference's ``Engine``."""

    def __init__(self, model: Model, max_tokens: int | None = None, max_batch: int = 64):
        self.model = model
        self.max_batch = max_batch
        if max_tokens is None:
            max_tokens = self.default_max_tokens(model, max_batch)
        self.engine = Engine(model, max_tokens, max_seqs=max_batch)

    @staticmethod
    def default_max_tokens(model: Model, max_batch: int, share_of_free_memory: float = 0.8) -> int:
        """Tokens of cache when the caller names none: ``max_batch`` sequences of the longest context the
        configuration allows, but no more than fits in most of the device memory that is free now (a
        configuration may allow tens of thousands of positions, far more than a batch of them fits)."""
        longest = getattr(model.config, "max_position_embeddings", None) or 4096
        wanted = max_batch * rounded_tokens(longest)
        per_token = model.make_cache(rounded_tokens(1), 1).kv_bytes_per_token()
        if model.device.type != "cuda" or per_token == 0:
            return wanted
        free, _ = torch.cuda.mem_get_info(model.device)
        fits = int(free * share_of_free_memory) // per_token
        if fits < rounded_tokens(1):
            raise RuntimeError(f"no device memory left for a cache: {free} bytes free, {per_token} bytes a token")
        return min(wanted, fits - fits % rounded_tokens(1))

    @torch.no_grad()
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 64, temperature: float = 1.0,
                 top_k: int | None = None, eos_token_id: int | None = None, stop_ids: Sequence[int] = (),
                 seed: int = 42, on_step=None) -> list[list[int]]:
        """``on_step(live, tokens)``, if given, is called after every step once the step's tokens
        have reached the host (``tokens``: one id per live sequence)."""
        stops = set(int(s) for s in stop_ids)
        if eos_token_id is not None:
            stops.add(int(eos_token_id))
        sampling = SamplingParams(temperature=temperature, top_k=top_k, seed=seed)
        params = GenerationParams(max_new_tokens=max_new_tokens, stop_ids=frozenset(stops), max_batch=self.max_batch)
        device = self.model.device

        def chooser(logits, request_indices, steps):
            if sampling.temperature == 0:  # greedy needs no keys
                return choose(logits, sampling, None, None).cpu().tolist()
            keys = torch.tensor([request_indices, steps], dtype=torch.int32)
            if device.type == "cuda":
                keys = keys.pin_memory()
            keys = keys.to(device, non_blocking=True)
            tokens = choose(logits, sampling, keys[0], keys[1])
            return tokens.cpu().tolist()

        def choose_on_device(logits, request_indices, steps):
            if sampling.temperature == 0:
                return choose(logits, sampling, None, None)
            keys = torch.tensor([request_indices, steps], dtype=torch.int32).pin_memory().to(device, non_blocking=True)
            return choose(logits, sampling, keys[0], keys[1])

        def fetch(tokens):
            host = torch.empty(tokens.shape, dtype=tokens.dtype, pin_memory=True)
            host.copy_(tokens, non_blocking=True)
            arrived = torch.cuda.Event()
            arrived.record()

            def wait():
                arrived.synchronize()
                return host.tolist()
            return wait

        def take(tokens, rows):
            return tokens[torch.tensor(rows, dtype=torch.int64, device=tokens.device)]

        ahead = DeviceChooser(choose_on_device, fetch, take) if device.type == "cuda" else None
        outputs = run_generation(self.engine, prompts, params, chooser, on_step=on_step, device_chooser=ahead)
        self.engine.check()
        return outputs


def generate(model: Model, prompts: Sequence[Sequence[int]], max_new_tokens: int = 64, temperature: float = 1.0,
             top_k: int | None = None, eos_token_id: int | None = None, stop_ids: Sequence[int] = (), seed: int = 42,
             max_tokens: int | None = None, max_batch: int | None = None) -> list[list[int]]:
    """One-call form: sizes a cache for these prompts, generates, and lets the cache go."""
    prompts = [list(p) for p in prompts]
    max_batch = max_batch or max(1, min(64, len(prompts)))
    if max_tokens is None:
        longest = sorted((rounded_tokens(len(p) + max_new_tokens) for p in prompts), reverse=True)
        max_tokens = max(rounded_tokens(1), sum(longest[:max_batch]))
    return Generator(model, max_tokens, max_batch).generate(
        prompts, max_new_tokens, temperature, top_k, eos_token_id, stop_ids, seed)
