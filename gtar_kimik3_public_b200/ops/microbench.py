"""Micro-benchmarks of single kernels at the shapes of a model's step.

    python -m gtar_kimik3_public_b200.ops.microbench --kernel gemm --m 8 --n 4096 --k 1024
    python -m gtar_kimik3_public_b200.ops.microbench --kernel gemv --m 8 --n 4096 --k 1024
    python -m gtar_kimik3_public_b200.ops.microbench --kernel attention_decode --batch 8 --context 2048
    python -m gtar_kimik3_public_b200.ops.microbench --kernel attention_prefill --tokens 2048
    python -m gtar_kimik3_public_b200.ops.microbench --kernel step --batch 8 --context 2048
    python -m gtar_kimik3_public_b200.ops.microbench --kernel decode_layers --batch 8 --context 2048

Each run launches the kernel on fresh inputs (a ring of operand sets larger than the L2 cache, so
that every launch reads from HBM), times it with CUDA events over a graph replay, and prints one
JSON line with microseconds per launch, the bytes or flops the kernel has to move or do, and the
rate they amount to.  The same command line under ``ncu -k regex:<kernel> -c 3`` gives a profile of
exactly that kernel on a case of a few hundred megabytes.
"""

from __future__ import annotations

import argparse
import json

import torch

from . import functional as F

DEV = "cuda:0"


def _time_graph(fn, iters: int) -> float:
    """Microseconds per call of ``fn`` replayed from a CUDA graph (median of ``iters`` replays)."""
    fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    times = []
    for _ in range(iters):
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        graph.replay()
        end.record()
        torch.cuda.synchronize()
        times.append(begin.elapsed_time(end) * 1e3)
    return sorted(times)[len(times) // 2]


def bench_gemm(args) -> dict:
    m, n, k = args.m, args.n, args.k
    ring = max(2, min(64, (256 << 20) // (n * k * 2) + 1))
    weights = [torch.randn(n, k, device=DEV, dtype=torch.bfloat16) * 0.02 for _ in range(ring)]
    x = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    splits = args.splits or F.split_k_for(m, n, k)

    def run():
        for w in weights:
            F.gemm_tc(x, w, torch.bfloat16, swiglu=args.swiglu, splits=splits)

    us = _time_graph(run, args.iters) / ring
    return {"kernel": "gemm_tc", "m": m, "n": n, "k": k, "splits": splits, "swiglu": args.swiglu, "us": round(us, 2),
            "weight_gb_s": round(n * k * 2 / us / 1e3, 1), "tflop_s": round(2 * m * n * k / us / 1e6, 1)}


def bench_gemv(args) -> dict:
    m, n, k = args.m, args.n, args.k
    ring = max(2, min(64, (256 << 20) // (n * k * 2) + 1))
    weights = [torch.randn(n, k, device=DEV, dtype=torch.bfloat16) * 0.02 for _ in range(ring)]
    x = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    before = F.set_pdl(args.pdl)

    def run():
        for w in weights:
            F.gemv(x, w, torch.bfloat16, swiglu=args.swiglu)

    try:
        us = _time_graph(run, args.iters) / ring
    finally:
        F.set_pdl(before)
    return {"kernel": "gemv", "m": m, "n": n, "k": k, "swiglu": args.swiglu, "pdl": args.pdl, "us": round(us, 2),
            "weight_gb_s": round(n * k * 2 / us / 1e3, 1)}


def _paged(batch: int, context: int, n_kv: int, d: int):
    per_seq = -(-context // 64)
    n_pages = batch * per_seq
    k = torch.randn(n_pages, n_kv, 64, d, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(n_pages, n_kv, 64, d, device=DEV, dtype=torch.bfloat16)
    table = torch.randperm(n_pages, device=DEV).to(torch.int32).view(batch, per_seq).contiguous()
    return F.PagedKV(k, v, table)


def bench_attention_decode(args) -> dict:
    b, s, n_q, n_kv, d = args.batch, args.context, args.q_heads, args.kv_heads, args.head_dim
    ring = max(2, min(16, (256 << 20) // (b * s * n_kv * d * 4) + 1))
    caches = [_paged(b, s, n_kv, d) for _ in range(ring)]
    q = torch.randn(b, n_q, d, device=DEV, dtype=torch.bfloat16)
    kv_len = torch.full((b,), s, dtype=torch.int32, device=DEV)
    slots = torch.arange(b, dtype=torch.int32, device=DEV)
    splits = args.splits or F.decode_splits(b, n_kv, s, 64, F.sm_count(), F.decode_cluster_places(d, F.sm_count()))
    if args.dealt_evenly:
        work = F.DecodeWork(torch.device(DEV))
        for kv in caches:
            kv.work = work

    def run():
        for kv in caches:
            if args.dealt_evenly:
                F.attention_decode_flat(q, None, n_q, n_kv, d, None, None, 1.0, None, None, kv, kv_len, slots, s - 1, d**-0.5)
            else:
                F.attention_decode(q, kv, kv_len, slots, d**-0.5, 0, splits)

    us = _time_graph(run, args.iters) / ring
    nbytes = b * s * n_kv * d * 2 * 2
    return {"kernel": "attention_decode", "batch": b, "context": s, "q_heads": n_q, "kv_heads": n_kv, "head_dim": d,
            "splits": "pages dealt evenly" if args.dealt_evenly else splits, "us": round(us, 2),
            "kv_gb_s": round(nbytes / us / 1e3, 1)}


def bench_attention_prefill(args) -> dict:
    t, n_q, n_kv, d = args.tokens, args.q_heads, args.kv_heads, args.head_dim
    kv = _paged(1, t, n_kv, d)
    q = torch.randn(t, n_q, d, device=DEV, dtype=torch.bfloat16)
    cu_q = torch.tensor([0, t], dtype=torch.int32, device=DEV)
    kv_len = torch.tensor([t], dtype=torch.int32, device=DEV)
    slots = torch.zeros(1, dtype=torch.int32, device=DEV)

    def run():
        F.attention_prefill(q, kv, cu_q, kv_len, slots, t, d**-0.5, tensor_cores=args.attention_path)

    before = F.set_attention_prefill_one_tile(args.one_tile)
    stay = F.set_attention_prefill_stay(args.stay)
    try:
        us = _time_graph(run, args.iters)
    finally:
        F.set_attention_prefill_one_tile(before)
        F.set_attention_prefill_stay(stay)
    flops = 4 * n_q * d * t * t / 2
    return {"kernel": "attention_prefill", "path": args.attention_path, "tokens": t, "q_heads": n_q, "kv_heads": n_kv, "head_dim": d,
            "us": round(us, 2), "tflop_s": round(flops / us / 1e6, 1)}


def bench_step(args) -> dict:
    """One decode step of a random model of the Qwen3-0.6B layer sizes, launched kernel by kernel (no
    graph) between cudaProfilerStart/Stop, so that ``ncu --profile-from-start off`` lists exactly
    the step's launches."""
    import tempfile

    from ..engine import Engine, StepEntry
    from ..generate import load
    from ..registry import config_from_dict
    from ..weights import write_random_model

    config = config_from_dict({
        "arch": "transformer", "vocab_size": 151936, "hidden_size": args.hidden, "intermediate_size": args.intermediate,
        "num_hidden_layers": args.layers, "num_attention_heads": args.q_heads, "num_key_value_heads": args.kv_heads,
        "head_dim": args.head_dim, "rms_norm_eps": 1e-6, "rope_theta": 1e6, "tie_word_embeddings": True,
        "initializer_range": 0.02, "max_position_embeddings": 4096,
    })
    with tempfile.TemporaryDirectory(prefix="gtar_microbench_") as folder:
        write_random_model(folder, config, seed=0)
        model = load(folder, "bfloat16", DEV)
    b, s = args.batch, args.context
    engine = Engine(model, b * (s + 64), max_seqs=b, use_graphs=False)
    gen = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, config.vocab_size, (b, s), generator=gen).tolist()
    ids = list(range(b))
    with torch.no_grad():
        tokens = None
        for start in range(0, b, 8):
            logits = engine.step([StepEntry(i, prompts[i], [s - 1]) for i in ids[start:start + 8]])
            part = F.argmax(logits)
            tokens = part if tokens is None else torch.cat([tokens, part])
        for _ in range(2):
            tokens = F.argmax(engine.decode_on_device(ids, tokens))
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        tokens = F.argmax(engine.decode_on_device(ids, tokens))
        end.record()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    return {"kernel": "decode step, kernel by kernel", "batch": b, "context": s, "layers": args.layers,
            "us": round(begin.elapsed_time(end) * 1e3, 1)}


def bench_prefill_step(args) -> dict:
    """One step over ``--batch`` whole prompts of ``--tokens`` tokens of a random model of the given layer sizes,
    launched kernel by kernel between cudaProfilerStart/Stop (after two steps of the same shape that are not listed)."""
    import tempfile

    from ..engine import Engine, StepEntry
    from ..generate import load
    from ..registry import config_from_dict
    from ..weights import write_random_model

    config = config_from_dict({
        "arch": "transformer", "vocab_size": 151936, "hidden_size": args.hidden, "intermediate_size": args.intermediate,
        "num_hidden_layers": args.layers, "num_attention_heads": args.q_heads, "num_key_value_heads": args.kv_heads,
        "head_dim": args.head_dim, "rms_norm_eps": 1e-6, "rope_theta": 1e6, "tie_word_embeddings": True,
        "initializer_range": 0.02, "max_position_embeddings": max(4096, args.tokens),
    })
    with tempfile.TemporaryDirectory(prefix="gtar_microbench_") as folder:
        write_random_model(folder, config, seed=0)
        model = load(folder, "bfloat16", DEV)
    b, s = args.batch, args.tokens
    engine = Engine(model, b * (s + 64), max_seqs=b, use_graphs=False)
    gen = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, config.vocab_size, (b, s), generator=gen).tolist()
    ids = list(range(b))
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.no_grad():
        for turn in range(3):
            if turn == 2:
                torch.cuda.synchronize()
                torch.cuda.profiler.start()
                begin.record()
            engine.step([StepEntry(i, prompts[i], [s - 1]) for i in ids])
            if turn == 2:
                end.record()
                torch.cuda.synchronize()
                torch.cuda.profiler.stop()
            engine.end(ids)
    return {"kernel": "prefill step, kernel by kernel", "batch": b, "tokens": s, "layers": args.layers,
            "us": round(begin.elapsed_time(end) * 1e3, 1)}


def bench_decode_layers(args) -> dict:
    """One decode step through the persistent kernel for all layers, with the kernel's own clock stamps: for every
    stage of a layer in the middle of the model, how long the blocks work on it (from their release out of the barrier
    before it to their arrival at the barrier behind it) and how long the barrier takes once the last block is there."""
    import tempfile

    from ..engine import Engine, StepEntry
    from ..generate import load
    from ..models import persistent_decode
    from ..registry import config_from_dict
    from ..weights import write_random_model

    persistent_decode.ENABLED = True
    config = config_from_dict({
        "arch": "transformer", "vocab_size": 151936, "hidden_size": 1024, "intermediate_size": 3072,
        "num_hidden_layers": args.layers, "num_attention_heads": args.q_heads, "num_key_value_heads": args.kv_heads,
        "head_dim": args.head_dim, "rms_norm_eps": 1e-6, "rope_theta": 1e6, "tie_word_embeddings": True,
        "initializer_range": 0.02, "max_position_embeddings": 4096,
    })
    with tempfile.TemporaryDirectory(prefix="gtar_microbench_") as folder:
        write_random_model(folder, config, seed=0)
        model = load(folder, "bfloat16", DEV)
    b, s, layers = args.batch, args.context, args.layers
    engine = Engine(model, b * (s + 64), max_seqs=b, use_graphs=False)
    gen = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, config.vocab_size, (b, s), generator=gen).tolist()
    ids = list(range(b))
    blocks = F.sm_count(torch.device(DEV))
    with torch.no_grad():
        tokens = F.argmax(engine.step([StepEntry(i, prompts[i], [s - 1]) for i in ids]))
        plan = model.persistent_decode(engine.cache)
        if plan is None:
            raise SystemExit("the persistent kernel does not take this model")
        for _ in range(3):
            tokens = F.argmax(engine.decode_on_device(ids, tokens))
        stamps = torch.zeros(blocks * 5 * layers * 2 + 5 * layers * 8, dtype=torch.int64, device=DEV)
        plan.stamps = stamps
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        tokens = F.argmax(engine.decode_on_device(ids, tokens))
        end.record()
        torch.cuda.synchronize()
        plan.stamps = None
    at = stamps[:blocks * 5 * layers * 2].view(blocks, 5 * layers, 2).cpu()
    layer = layers // 2
    stages = {}
    for index, name in enumerate(("qkv", "attention", "output", "gate_up", "down")):
        o = layer * 5 + index
        if o == 0 or o >= 5 * layers - 1:
            continue
        work = (at[:, o, 0] - at[:, o - 1, 1]).double() / 1e3
        stages[name] = {"work_us_min_median_max": [round(work.min().item(), 2), round(work.median().item(), 2), round(work.max().item(), 2)],
                        "barrier_after_last_arrival_us": round((at[:, o, 1].double().median().item() - at[:, o, 0].max().item()) / 1e3, 2)}
    span = (at[:, 5 * layers - 2, 1].max() - at[:, 0, 0].min()).item() / 1e3
    return {"kernel": "decode_layers (persistent, all layers)", "batch": b, "context": s, "layers": layers,
            "step_us": round(begin.elapsed_time(end) * 1e3, 1), "first_to_last_barrier_us": round(span, 1),
            "stages_of_layer": layer, "stages": stages}


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--kernel", required=True, choices=["gemm", "gemv", "attention_decode", "attention_prefill", "step", "prefill_step", "decode_layers"])
    parser.add_argument("--m", type=int, default=8)
    parser.add_argument("--n", type=int, default=4096)
    parser.add_argument("--k", type=int, default=1024)
    parser.add_argument("--splits", type=int, default=0)
    parser.add_argument("--swiglu", action="store_true")
    parser.add_argument("--dealt-evenly", action="store_true",
                        help="attention_decode: the kernel that cuts the line of all sequences' pages into equal pieces")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=2048)
    parser.add_argument("--tokens", type=int, default=2048)
    parser.add_argument("--q-heads", type=int, default=16)
    parser.add_argument("--kv-heads", type=int, default=8)
    parser.add_argument("--head-dim", type=int, default=128)
    parser.add_argument("--hidden", type=int, default=1024, help="step: the model's width")
    parser.add_argument("--intermediate", type=int, default=3072, help="step: the feed-forward's width")
    parser.add_argument("--attention-path", default="auto", choices=["auto", "tcgen05", "mma"])
    parser.add_argument("--stay", type=int, default=2, choices=[0, 1, 2],
                        help="attention_prefill on tcgen05: blocks that stay and take query tiles from a list: 1 = always, 0 = never, 2 = the library's choice")
    parser.add_argument("--one-tile", type=int, default=1, choices=[0, 1],
                        help="attention_prefill on tcgen05: 1 = a query tile a block, heaviest first (the default), 0 = a heavy and a light tile a block")
    parser.add_argument("--layers", type=int, default=28)
    parser.add_argument("--iters", type=int, default=5)
    parser.add_argument("--pdl", action="store_true", help="gemv: launch with programmatic dependent launch, as a model step does")
    args = parser.parse_args()
    F.require_device(torch.device(DEV))
    result = {"gemm": bench_gemm, "gemv": bench_gemv, "attention_decode": bench_attention_decode,
              "attention_prefill": bench_attention_prefill, "step": bench_step, "prefill_step": bench_prefill_step, "decode_layers": bench_decode_layers}[args.kernel](args)
    F.check_kernel_errors(DEV)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
