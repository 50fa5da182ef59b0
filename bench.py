"""Benchmark of the library's flagship step: decoding with the Qwen3-0.6B layer sizes.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  ``value`` is decoded tokens per second at batch 8 after 2,048-token
prompts (device-timed with CUDA events over exactly K decode steps; a step = the model's
forward for one token of every sequence + the greedy token choice, tokens staying on the
device).  ``e2e`` is the same through the Python entry point with host tokens in and out every
step.  ``prefill`` is one 2,048-token prompt in one step; ``points`` holds decoding at batch 1
and 64; ``roofline`` is the decode step's bytes (every weight once + the live requests' keys and
values) over its time, against the measured copy bandwidth.

Weights are random (written as a model folder by the library's random-weights mode and loaded
from there), token ids are seeded uniform-random: there is no network for checkpoints or data.
The library runs on one GPU; with --gpus N > 1 a line says so and the exit code is 2.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# BASELINE.json configs[2]: the Qwen3-0.6B layer sizes (the reference's configs/transformer_0.6B.json
# plus the vocabulary its tokenizer gives).
BENCH_CONFIG = {
    "arch": "transformer",
    "vocab_size": 151936,
    "hidden_size": 1024,
    "intermediate_size": 3072,
    "num_hidden_layers": 28,
    "num_attention_heads": 16,
    "num_key_value_heads": 8,
    "head_dim": 128,
    "rms_norm_eps": 1e-6,
    "rope_theta": 1000000.0,
    "tie_word_embeddings": True,
    "initializer_range": 0.02,
    "max_position_embeddings": 4096,
}
PROMPT_LEN = 2048
PREFILL_TOKENS = 2048
# BASELINE.json configs[3] and configs[4]: the Qwen3-4B and Qwen3-8B layer sizes, measured as extra points
LARGE_CONFIGS = {
    "qwen3_4b": {"arch": "transformer", "vocab_size": 151936, "hidden_size": 2560, "intermediate_size": 9728,
                 "num_hidden_layers": 36, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
                 "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "tie_word_embeddings": True, "initializer_range": 0.02,
                 "max_position_embeddings": 8192},
    "qwen3_8b": {"arch": "transformer", "vocab_size": 151936, "hidden_size": 4096, "intermediate_size": 12288,
                 "num_hidden_layers": 36, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
                 "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "tie_word_embeddings": False, "initializer_range": 0.02,
                 "max_position_embeddings": 4096},
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            raw = json.loads(path.read_text())
            out = dict(FALLBACK_PEAKS)
            for key in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                if isinstance(raw.get(key), (int, float)):
                    out[key] = float(raw[key])
            return out, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, sm_max, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in self.rows:
            if len(row) < 7:
                continue
            try:
                sm.append(float(row[0]))
                sm_max.append(float(row[1]))
            except ValueError:
                continue
            for name, cell in zip(names, row[3:7]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(sm_max) if sm_max else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def step_bytes(batch: int, kv_tokens_each: int, layers: int) -> float:
    """Bytes a decode step has to read, from the sizes alone (both arms print it the same way): every
    bfloat16 matrix once, the 32-bit norm weights, and the live requests' keys and values."""
    c = BENCH_CONFIG
    q_width = c["num_attention_heads"] * c["head_dim"]
    kv_width = c["num_key_value_heads"] * c["head_dim"]
    per_layer = 2 * c["hidden_size"] * (2 * q_width + 2 * kv_width + 3 * c["intermediate_size"])
    per_layer += 4 * (2 * c["hidden_size"] + 2 * c["head_dim"])
    head = 2 * c["vocab_size"] * c["hidden_size"] * (1 if c["tie_word_embeddings"] else 2)
    kv = 2 * 2 * kv_width * layers * kv_tokens_each * batch
    return layers * per_layer + head + 4 * c["hidden_size"] + kv


def config_record(batch: int, layers: int, peak_source: str) -> dict:
    """The ``config`` of the JSON line: every size by name, flat.  Both arms build it here."""
    c = BENCH_CONFIG
    return {
        "model": "transformer (Qwen3-0.6B layer sizes)", "global_batch": batch, "seq_len": PROMPT_LEN,
        "context_length": c["max_position_embeddings"], "parallelism": "single GPU",
        "layers": layers, "layers_full_config": c["num_hidden_layers"], "hidden_size": c["hidden_size"],
        "q_heads": c["num_attention_heads"], "kv_heads": c["num_key_value_heads"], "head_dim": c["head_dim"],
        "intermediate_size": c["intermediate_size"], "vocab_size": c["vocab_size"],
        "tied_embeddings": c["tie_word_embeddings"], "prefill_tokens": PREFILL_TOKENS,
        "l2": "no flush: a step reads %.2f GB, far above the 126 MB L2" % (step_bytes(batch, PROMPT_LEN, layers) / 1e9),
        "peaks": peak_source,
    }


def make_model(dtype: str, layers: int | None = None):
    from gtar_kimik3_public_b200.generate import load
    from gtar_kimik3_public_b200.registry import config_from_dict
    from gtar_kimik3_public_b200.weights import write_random_model

    cfg = dict(BENCH_CONFIG)
    if layers:
        cfg["num_hidden_layers"] = layers
    config = config_from_dict(cfg)
    with tempfile.TemporaryDirectory(prefix="gtar_bench_model_") as folder:
        write_random_model(folder, config, seed=0)
        model = load(folder, dtype, "cuda:0")
    return model, config


def random_prompts(batch: int, length: int, vocab: int, seed: int = 0):
    import torch

    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (batch, length), generator=gen).tolist()


def decode_bytes(model, engine, kv_tokens: int) -> float:
    return model.weight_bytes_per_step() + kv_tokens * engine.cache.kv_bytes_per_token()


def time_decode(model, batch: int, steps: int, warmup: int, sample_clocks: bool = False) -> dict:
    """Device-timed decoding: prompts of PROMPT_LEN in one step, then warm-up and K timed steps."""
    import torch

    from gtar_kimik3_public_b200.cache import rounded_tokens
    from gtar_kimik3_public_b200.engine import Engine, StepEntry
    from gtar_kimik3_public_b200.ops import functional as F
    from gtar_kimik3_public_b200.ops import library

    room = rounded_tokens(PROMPT_LEN + warmup + steps + 1)
    engine = Engine(model, batch * room, max_seqs=batch)
    prompts = random_prompts(batch, PROMPT_LEN, model.vocab_size)
    ids = list(range(batch))
    with torch.no_grad():
        logits = None
        for start in range(0, batch, 8):  # prompts in groups of 8 keep the prefill's activations small
            part = engine.step([StepEntry(i, prompts[i], [PROMPT_LEN - 1]) for i in ids[start:start + 8]])
            logits = part if logits is None else torch.cat([logits, part])
        tokens = F.argmax(logits)
        sampler = ClockSampler() if sample_clocks else None
        if sampler:  # started before the warm-up steps: nvidia-smi needs a moment to deliver its first sample
            sampler.start()
        for _ in range(warmup):
            tokens = F.argmax(engine.decode_on_device(ids, tokens))
        torch.cuda.synchronize()
        launches_before = library.launch_count
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(steps):
            tokens = F.argmax(engine.decode_on_device(ids, tokens))
        end.record()
        torch.cuda.synchronize()
        ms = begin.elapsed_time(end)
        launches = library.launch_count - launches_before
        clocks = sampler.stop() if sampler else None
    kv_tokens = sum(engine.cache.length.values()) - batch * (steps // 2)  # mid-point of the timed region
    result = {
        "tokens_per_s": batch * steps / (ms / 1e3), "ms_per_step": ms / steps, "launches": launches,
        "bytes_per_step": decode_bytes(model, engine, kv_tokens), "clocks": clocks,
    }
    engine.end_all()
    del engine
    torch.cuda.empty_cache()
    return result


def time_e2e(model, batch: int, steps: int, warmup: int) -> dict:
    """The same decode through the Python entry point: host token lists in, host token lists out,
    every step a pinned host-to-device copy of its numbers and a device-to-host read of its tokens."""
    import torch

    from gtar_kimik3_public_b200.cache import rounded_tokens
    from gtar_kimik3_public_b200.generate import Generator

    room = rounded_tokens(PROMPT_LEN + warmup + steps + 2)
    generator = Generator(model, max_tokens=batch * room, max_batch=batch)
    prompts = random_prompts(batch, PROMPT_LEN, model.vocab_size)
    stamps = []

    def on_step(live, tokens):
        stamps.append(time.perf_counter())  # the step's tokens are on the host here

    generator.generate(prompts, max_new_tokens=warmup + steps + 1, temperature=0.0, on_step=on_step)
    torch.cuda.synchronize()
    timed = stamps[warmup:warmup + steps + 1]
    seconds = timed[-1] - timed[0]
    # per step: positions + sequence index + starts + slots + lengths + wanted rows in (the token ids a step
    # chose stay on the device for the next step: the loop runs the device one step ahead of the host),
    # tokens out; a sequence's page-table row follows every 64 steps and is not counted
    h2d = 4 * (5 * batch + 1)
    return {"value": batch * steps / seconds, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * batch}


def time_prefill(model, warmup: int, repeats: int = 7) -> dict:
    import torch

    from gtar_kimik3_public_b200.cache import rounded_tokens
    from gtar_kimik3_public_b200.engine import Engine, StepEntry

    engine = Engine(model, rounded_tokens(PREFILL_TOKENS + 1), max_seqs=1)
    prompt = random_prompts(1, PREFILL_TOKENS, model.vocab_size, seed=1)[0]
    times = []
    with torch.no_grad():
        for i in range(warmup + repeats):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            begin.record()
            engine.step([StepEntry("p", prompt, [PREFILL_TOKENS - 1])])
            end.record()
            torch.cuda.synchronize()
            engine.end(["p"])
            if i >= warmup:
                times.append(begin.elapsed_time(end))
    ms = statistics.median(times)
    c = model.config
    t = PREFILL_TOKENS
    per_layer = 2 * t * c.hidden_size * ((c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim
                                         + c.num_attention_heads * c.head_dim + 3 * c.intermediate_size)
    attention = 4 * c.num_attention_heads * c.head_dim * t * t / 2  # QK^T and PV over the causal half
    flops = len(model.plan.run_list) * (per_layer + attention) + 2 * c.hidden_size * c.vocab_size
    del engine
    torch.cuda.empty_cache()
    return {"value": t / (ms / 1e3), "tokens": t, "ms": ms, "flops": flops}


def prefill_flops(config, layers: int, lengths) -> float:
    """Matrix products of every token, attention over the causal half of each prompt, the head for one row each."""
    c = config
    per_token = 2 * c.hidden_size * ((2 * c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim + 3 * c.intermediate_size)
    attention = sum(4 * c.num_attention_heads * c.head_dim * t * t / 2 for t in lengths)
    return layers * (per_token * sum(lengths) + attention) + 2 * c.hidden_size * c.vocab_size * len(lengths)


def time_large(name: str, peak: dict, steps: int, warmup: int) -> dict:
    """The 4B and 8B workloads: weights drawn on the device (a folder of these sizes would take minutes to write
    and read), the whole number of layers.  4B: eight prompts of unequal lengths (uniform in [256, 4096], seeded) in
    one step, then decode steps.  8B: 64 prompts of 1,024 tokens, then decode steps; and one 2,048-token prompt."""
    import random

    import torch

    from gtar_kimik3_public_b200.cache import rounded_tokens
    from gtar_kimik3_public_b200.engine import Engine, StepEntry
    from gtar_kimik3_public_b200.models.model import Model
    from gtar_kimik3_public_b200.ops import functional as F
    from gtar_kimik3_public_b200.registry import architecture, config_from_dict
    from gtar_kimik3_public_b200.weights import load_random_weights

    config = config_from_dict(LARGE_CONFIGS[name])
    model = Model(architecture(config.ARCH_NAMES[0]).build_plan(config), config, torch.bfloat16, "cuda:0")
    load_random_weights(model, seed=0)
    layers = len(model.plan.run_list)
    rng = random.Random(0)
    if name == "qwen3_4b":
        lengths, steps, group = [rng.randint(256, 4096) for _ in range(8)], min(steps, 256), 8
    else:
        lengths, steps, group = [1024] * 64, min(steps, 64), 8
    batch = len(lengths)
    engine = Engine(model, sum(rounded_tokens(n + warmup + steps + 1) for n in lengths), max_seqs=batch)
    gen = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, config.vocab_size, (n,), generator=gen).tolist() for n in lengths]
    ids = list(range(batch))
    out = {}
    with torch.no_grad():
        logits = None
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        begin.record()
        for start in range(0, batch, group):
            part = engine.step([StepEntry(i, prompts[i], [lengths[i] - 1]) for i in ids[start:start + group]])
            logits = part if logits is None else torch.cat([logits, part])
        end.record()
        torch.cuda.synchronize()
        if name == "qwen3_4b":  # the unequal prompts in one step (launched kernel by kernel: a first appearance of its shape)
            ms = begin.elapsed_time(end)
            out[f"{name}_prefill_unequal_tokens_per_s"] = round(sum(lengths) / (ms / 1e3), 1)
            out[f"{name}_prefill_unequal_frac"] = round(prefill_flops(config, layers, lengths) / (ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4)
        tokens = F.argmax(logits)
        for _ in range(warmup):
            tokens = F.argmax(engine.decode_on_device(ids, tokens))
        torch.cuda.synchronize()
        begin.record()
        for _ in range(steps):
            tokens = F.argmax(engine.decode_on_device(ids, tokens))
        end.record()
        torch.cuda.synchronize()
        ms = begin.elapsed_time(end) / steps
        kv_tokens = sum(engine.cache.length.values()) - batch * (steps // 2)
        step_bytes_read = decode_bytes(model, engine, kv_tokens)
        tag = f"{name}_decode_b{batch}" + ("_unequal" if name == "qwen3_4b" else "")
        out[tag] = round(batch / (ms / 1e3), 1)
        out[tag + "_ms"] = round(ms, 4)
        out[tag + "_hbm_frac"] = round(step_bytes_read / (ms / 1e3) / 1e9 / peak["hbm_gbs"], 4)
        engine.end_all()
        del engine
        torch.cuda.empty_cache()
        if name == "qwen3_8b":
            engine = Engine(model, rounded_tokens(PREFILL_TOKENS + 1), max_seqs=1)
            prompt = torch.randint(0, config.vocab_size, (PREFILL_TOKENS,), generator=gen).tolist()
            times = []
            for i in range(8):  # the first is the shape's first appearance; the median of the other seven
                torch.cuda.synchronize()
                begin.record()
                engine.step([StepEntry("p", prompt, [PREFILL_TOKENS - 1])])
                end.record()
                torch.cuda.synchronize()
                engine.end(["p"])
                times.append(begin.elapsed_time(end))
            ms = statistics.median(times[1:])
            out[f"{name}_prefill_{PREFILL_TOKENS}_tokens_per_s"] = round(PREFILL_TOKENS / (ms / 1e3), 1)
            out[f"{name}_prefill_{PREFILL_TOKENS}_frac"] = round(prefill_flops(config, layers, [PREFILL_TOKENS]) / (ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4)
            del engine
    out[f"{name}_layers"] = layers
    del model
    torch.cuda.empty_cache()
    return out


def run_ours(args) -> dict:
    import torch

    from gtar_kimik3_public_b200.ops.library import require_device

    require_device(torch.device("cuda:0"))
    peak, peak_source = peaks()
    model, config = make_model("bfloat16", args.layers)
    layers_run = len(model.plan.run_list)
    batch = args.batch
    main = time_decode(model, batch, args.steps, args.warmup, sample_clocks=True)
    e2e = time_e2e(model, batch, args.steps, args.warmup)
    prefill = time_prefill(model, max(1, min(args.warmup, 3)))
    points = {}
    for b in (1, 64):
        points[f"decode_b{b}"] = round(time_decode(model, b, min(args.steps, 64), args.warmup)["tokens_per_s"], 1)
    del model
    import gc

    gc.collect()
    torch.cuda.empty_cache()
    if not args.no_large:
        for name in LARGE_CONFIGS:
            points.update(time_large(name, peak, args.steps, args.warmup))
    achieved = main["bytes_per_step"] / (main["ms_per_step"] / 1e3) / 1e9
    prefill_peak = peak["bf16_tflops"] * 1e12
    return {
        "metric": "decode tokens/s (Qwen3-0.6B layer sizes, batch 8, after 2,048-token prompts)",
        "value": round(main["tokens_per_s"], 1),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(main["ms_per_step"], 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: seeded uniform-random token ids, random weights (N(0, 0.02)) of the named architecture",
        "impl": "ours",
        "config": config_record(batch, layers_run, peak_source),
        "e2e": {k: (round(v, 1) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": main["launches"],
        "clocks": main["clocks"],
        "prefill": {"value": round(prefill["value"], 1), "tokens": prefill["tokens"], "ms": round(prefill["ms"], 3),
                    "frac": round(prefill["flops"] / (prefill["ms"] / 1e3) / prefill_peak, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4)},
        "points": points,
    }


def reference_folder() -> Path | None:
    """Where the unmodified reference lies: ``baseline/_ref`` beside this file (a plain copy of the
    reference's folder; it is a folder of scripts that runs from ``sys.path``), or the folder that the
    environment variable GTAR_REFERENCE_DIR names."""
    for folder in (os.environ.get("GTAR_REFERENCE_DIR"), ROOT / "baseline" / "_ref"):
        if folder and (Path(folder) / "src" / "engine.py").exists():
            return Path(folder)
    return None


class ReferenceArm:
    """The reference's own generation, untouched: ``Engine(TransformerForCausalLM).generate`` (src/engine.py:22-46)
    on the model that configs/transformer_0.6B.json describes, with the reference's own random initialisation.
    Nothing of this repository's package is imported here."""

    def __init__(self, folder: Path, device: str, layers: int | None, sizes: dict | None = None):
        import torch

        sys.path.insert(0, str(folder))
        from src.engine import Engine
        from src.models import ARCHITECTURES

        file = json.loads((folder / "configs" / "transformer_0.6B.json").read_text())
        config_class, model_class = ARCHITECTURES[file["arch"]]
        fields = dict(file["model"], vocab_size=BENCH_CONFIG["vocab_size"])
        for key, value in fields.items():  # the reference's file and the benchmark's sizes are the same model
            assert BENCH_CONFIG[key] == value, f"{key}: the reference's config has {value}, the benchmark {BENCH_CONFIG[key]}"
        if layers:
            fields["num_hidden_layers"] = layers
        if sizes:  # only the tests shrink the model (they run this arm on the CPU)
            fields.update(sizes)
        self.torch, self.device, self.fields = torch, device, fields
        torch.manual_seed(0)
        with torch.device(device):
            model = model_class(config_class(**fields))
        self.engine = Engine(model)
        self.eos = fields["vocab_size"] - 1  # the command line always passes a stop token (scripts/generate.py:40,44)

    def generate_seconds(self, prompts, new_tokens: int) -> float:
        """Wall clock of one call of the public API between synchronisations, as the reference times generation
        (scripts/benchmark_speculative.py:107-117): host token ids in, host token ids out."""
        torch = self.torch
        cuda = self.device.startswith("cuda")
        if cuda:
            torch.cuda.synchronize()
        begin = time.perf_counter()
        out = self.engine.generate(prompts, max_new_tokens=new_tokens, temperature=0.0, eos_token_id=self.eos).cpu()
        if cuda:
            torch.cuda.synchronize()
        seconds = time.perf_counter() - begin
        if out.shape[1] != new_tokens:  # every sequence chose the stop token: the run was cut short
            raise RuntimeError(f"the reference stopped after {out.shape[1]} of {new_tokens} tokens")
        return seconds

    def decode(self, batch: int, prompt_len: int, steps: int, warmup: int, repeats: int = 3) -> dict:
        """Seconds per decode step: a call that decodes warm-up + K steps minus a call that decodes warm-up steps,
        so that the prompts' step and the set-up cancel.  (A call for n new tokens runs n - 1 decode steps.)"""
        torch = self.torch
        gen = torch.Generator().manual_seed(0)
        prompts = torch.randint(0, self.fields["vocab_size"] - 1, (batch, prompt_len), generator=gen)
        self.generate_seconds(prompts, warmup + 1)  # untimed: compiles the attention kernel, loads the libraries
        short = [self.generate_seconds(prompts, warmup + 1) for _ in range(repeats)]
        long = [self.generate_seconds(prompts, warmup + steps + 1) for _ in range(repeats)]
        seconds = statistics.median(long) - statistics.median(short)
        return {"tokens_per_s": batch * steps / seconds, "ms_per_step": seconds / steps * 1e3,
                "h2d_bytes_per_step": batch * prompt_len * 8 // steps, "d2h_bytes_per_step": batch * 8}

    def prefill(self, tokens: int, repeats: int = 3) -> float:
        """Milliseconds of one prompt through the public API (one new token: the prompt's step and nothing else)."""
        torch = self.torch
        gen = torch.Generator().manual_seed(1)
        prompt = torch.randint(0, self.fields["vocab_size"] - 1, (1, tokens), generator=gen)
        self.generate_seconds(prompt, 1)
        return statistics.median(self.generate_seconds(prompt, 1) for _ in range(repeats)) * 1e3


def run_reference(args, device: str = "cuda:0", sizes: dict | None = None, prompt_len: int = PROMPT_LEN,
                  prefill_tokens: int = PREFILL_TOKENS, batches: tuple = (1, 64)) -> dict:
    """The reference arm: the same metric on the same configuration from the unmodified reference."""
    folder = reference_folder()
    if folder is None:
        return {"impl": "reference", "unavailable": "no copy of the reference under baseline/_ref (it is not part of "
                                                    "the repository's history) and GTAR_REFERENCE_DIR names none"}
    import torch

    if device.startswith("cuda") and not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "no CUDA device here: the arm is timed on a GPU only"}
    peak, peak_source = peaks()
    try:
        arm = ReferenceArm(folder, device, args.layers, sizes)
        sampler = ClockSampler()
        sampler.start()
        main = arm.decode(args.batch, prompt_len, args.steps, args.warmup)
        clocks = sampler.stop()
        prefill_ms = arm.prefill(prefill_tokens)
        points = {f"decode_b{b}": round(arm.decode(b, prompt_len, min(args.steps, 64), args.warmup, repeats=1)["tokens_per_s"], 1)
                  for b in batches}
    except Exception as error:  # the line says why; the trace goes to standard error
        import traceback

        traceback.print_exc()
        return {"impl": "reference", "unavailable": ("the reference failed here: %s: %s" % (type(error).__name__, error)).replace("\n", " ")[:300]}
    layers = arm.fields["num_hidden_layers"]
    achieved = step_bytes(args.batch, prompt_len + args.warmup + args.steps // 2, layers) / (main["ms_per_step"] / 1e3) / 1e9
    c = BENCH_CONFIG
    t = prefill_tokens
    per_layer = 2 * t * c["hidden_size"] * ((2 * c["num_attention_heads"] + 2 * c["num_key_value_heads"]) * c["head_dim"] + 3 * c["intermediate_size"])
    attention = 4 * c["num_attention_heads"] * c["head_dim"] * t * t / 2
    flops = layers * (per_layer + attention) + 2 * c["hidden_size"] * c["vocab_size"]  # counted as for the own arm: the wanted row only
    rate = round(main["tokens_per_s"], 1)
    return {
        "metric": "decode tokens/s (Qwen3-0.6B layer sizes, batch 8, after 2,048-token prompts)",
        "value": rate, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: seeded uniform-random token ids, random weights of the named architecture (the reference's own init_weights)",
        "impl": "reference",
        "timing": "wall clock around Engine.generate between synchronisations, long call minus short call (the "
                  "reference has no device-timed loop; value and e2e are the same measurement)",
        "config": config_record(args.batch, layers, peak_source),
        "e2e": {"value": rate, "unit": "tokens/s", "h2d_bytes_per_step": main["h2d_bytes_per_step"],
                "d2h_bytes_per_step": main["d2h_bytes_per_step"]},
        "gpu_launches": None,
        "clocks": clocks,
        "prefill": {"value": round(t / (prefill_ms / 1e3), 1), "tokens": t, "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4)},
        "points": points,
    }


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    parser.add_argument("--no-large", action="store_true", help="leave out the points at the 4B and 8B layer sizes")
    args = parser.parse_args()
    if args.impl == "reference":
        if args.warmup < 3:
            args.warmup = 3
        print(json.dumps(run_reference(args)))
        return 0
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported (no distributed path is built)")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    print(json.dumps(run_ours(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
