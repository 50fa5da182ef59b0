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

    from gtar_kimik3_public_b200.engine import Engine, StepEntry
    from gtar_kimik3_public_b200.ops import functional as F
    from gtar_kimik3_public_b200.ops import library

    room = -(-(PROMPT_LEN + warmup + steps + 1) // 64) * 64
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

    from gtar_kimik3_public_b200.generate import Generator

    room = -(-(PROMPT_LEN + warmup + steps + 2) // 64) * 64
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


def time_prefill(model, warmup: int, repeats: int = 3) -> dict:
    import torch

    from gtar_kimik3_public_b200.engine import Engine, StepEntry

    engine = Engine(model, -(-PREFILL_TOKENS // 64) * 64 + 64, max_seqs=1)
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


def run_ours(args) -> dict:
    import torch

    from gtar_kimik3_public_b200.ops.library import require_device

    require_device(torch.device("cuda:0"))
    peak, peak_source = peaks()
    model, config = make_model("bfloat16", args.layers)
    batch = args.batch
    main = time_decode(model, batch, args.steps, args.warmup, sample_clocks=True)
    e2e = time_e2e(model, batch, args.steps, args.warmup)
    prefill = time_prefill(model, max(1, min(args.warmup, 3)))
    points = {}
    for b in (1, 64):
        points[f"decode_b{b}"] = round(time_decode(model, b, min(args.steps, 64), args.warmup)["tokens_per_s"], 1)
    achieved = main["bytes_per_step"] / (main["ms_per_step"] / 1e3) / 1e9
    prefill_peak = peak["bf16_tflops"] * 1e12
    full_layers = BENCH_CONFIG["num_hidden_layers"]
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
        "config": {
            "model": "transformer (Qwen3-0.6B layer sizes)", "global_batch": batch, "seq_len": PROMPT_LEN,
            "context_length": config.max_position_embeddings, "parallelism": "single GPU",
            "layers": len(model.plan.run_list), "layers_full_config": full_layers, "hidden_size": config.hidden_size,
            "q_heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads, "head_dim": config.head_dim,
            "intermediate_size": config.intermediate_size, "vocab_size": config.vocab_size,
            "tied_embeddings": config.tie_word_embeddings, "prefill_tokens": PREFILL_TOKENS,
            "l2": "no flush: a step reads %.2f GB, far above the 126 MB L2" % (main["bytes_per_step"] / 1e9),
            "peaks": peak_source,
        },
        "e2e": {k: (round(v, 1) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": main["launches"],
        "clocks": main["clocks"],
        "prefill": {"value": round(prefill["value"], 1), "tokens": prefill["tokens"], "ms": round(prefill["ms"], 3),
                    "frac": round(prefill["flops"] / (prefill["ms"] / 1e3) / prefill_peak, 4)},
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
    args = parser.parse_args()
    if args.impl == "reference":
        print(json.dumps({
            "impl": "reference",
            "unavailable": "the reference cannot be installed offline: pip reports \"Neither 'setup.py' nor "
                           "'pyproject.toml' found\" (it is a folder of scripts, not a package)",
        }))
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
