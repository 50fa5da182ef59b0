"""Generate from a model folder.  From the repository root:

    python -m gtar_kimik3_public_b200.scripts.generate --model DIR --prompt-ids 1,2,3 \\
        --max-new-tokens 64 --temperature 0.8 --top-k 50 --num-samples 2

The options are the reference's (scripts/generate.py:18-29) where it has them:
``--prompt``, ``--tokenizer``, ``--eos-token``, ``--max-new-tokens`` (64), ``--temperature`` (0.8),
``--top-k`` (50), ``--num-samples`` (1), ``--seed`` (42), with the same meanings and defaults.
``--config``/``--checkpoint`` (a training config and a pickled state dict) are replaced by
``--model`` (a folder with config.json and model.safetensors), or ``--config`` with
``--random-weights`` to write and use a random model of that configuration.  There is no
network here, so ``--tokenizer`` names a local ``tokenizer.json`` (default: the one in the model
folder) and prompts can be given as token ids (``--prompt-ids``, ``--prompt-ids-file``).
"""

from __future__ import annotations

import argparse
import json
import sys
import tempfile
from pathlib import Path


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(description="Generate from a model folder")
    parser.add_argument("--model", help="folder with config.json and model.safetensors")
    parser.add_argument("--config", help="config file for --random-weights (flat, or the reference's nested form)")
    parser.add_argument("--random-weights", action="store_true", help="write a random model of --config and use it")
    parser.add_argument("--seed-weights", type=int, default=0, help="seed of the random weights")
    parser.add_argument("--vocab-size", type=int, default=None, help="vocabulary size if the config file has none")
    parser.add_argument("--checkpoint", help="a checkpoint file of the reference's training loop (its --checkpoint): "
                                             "converted to a model folder first")
    parser.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    parser.add_argument("--cast-matrices", action="store_true",
                        help="bfloat16 run of a folder stored in 32-bit: round its matrices to bfloat16 at load")
    parser.add_argument("--prompt", default=None)
    parser.add_argument("--prompt-ids", default=None, help="comma-separated token ids; several prompts separated by ';'")
    parser.add_argument("--prompt-ids-file", default=None, help="JSON file: a list of token-id lists")
    parser.add_argument("--tokenizer", default=None, help="path of a local tokenizer.json")
    parser.add_argument("--eos-token", default="<|endoftext|>")
    parser.add_argument("--stop-ids", default="", help="comma-separated token ids that end a sequence")
    parser.add_argument("--max-new-tokens", type=int, default=64)
    parser.add_argument("--temperature", type=float, default=0.8)
    parser.add_argument("--top-k", type=int, default=50)
    parser.add_argument("--num-samples", type=int, default=1)
    parser.add_argument("--seed", type=int, default=42)
    parser.add_argument("--device", default="cuda:0")
    return parser


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    from ..generate import generate, load
    from ..registry import config_from_file
    from ..weights.random_init import write_random_model

    scratch = None
    if args.random_weights:
        if not args.config:
            raise SystemExit("--random-weights needs --config")
        overrides = {"vocab_size": args.vocab_size} if args.vocab_size else None
        config = config_from_file(args.config, overrides)
        scratch = tempfile.TemporaryDirectory(prefix="gtar_b200_random_")
        model_dir = write_random_model(scratch.name, config, args.seed_weights)
    elif args.checkpoint:
        from ..weights.convert import convert_checkpoint

        scratch = tempfile.TemporaryDirectory(prefix="gtar_b200_checkpoint_")
        model_dir = convert_checkpoint(args.checkpoint, scratch.name, matrix_dtype=None)
    elif args.model:
        model_dir = Path(args.model)
    else:
        raise SystemExit("give --model DIR, --checkpoint FILE, or --config FILE --random-weights")

    tokenizer = None
    tokenizer_path = Path(args.tokenizer) if args.tokenizer else Path(model_dir) / "tokenizer.json"
    if tokenizer_path.exists():
        from tokenizers import Tokenizer

        tokenizer = Tokenizer.from_file(str(tokenizer_path))

    if args.prompt_ids_file:
        prompts = json.loads(Path(args.prompt_ids_file).read_text())
    elif args.prompt_ids:
        prompts = [[int(t) for t in part.split(",") if t.strip()] for part in args.prompt_ids.split(";")]
    elif args.prompt is not None:
        if tokenizer is None:
            raise SystemExit(f"--prompt needs a tokenizer: {tokenizer_path} does not exist (use --prompt-ids instead)")
        prompts = [tokenizer.encode(args.prompt).ids]
    else:
        raise SystemExit("give --prompt, --prompt-ids or --prompt-ids-file")
    prompts = [p for p in prompts for _ in range(args.num_samples)]

    stop_ids = [int(t) for t in args.stop_ids.split(",") if t.strip()]
    if tokenizer is not None:
        eos = tokenizer.token_to_id(args.eos_token)
        if eos is not None:
            stop_ids.append(eos)

    # a checkpoint is 32-bit: as in the reference's engine its matrices are rounded for a bfloat16 run
    model = load(model_dir, args.dtype, args.device, cast_matrices=args.cast_matrices or bool(args.checkpoint))
    config_eos = getattr(model.config, "eos_token_id", None)
    if config_eos is not None:
        stop_ids.append(config_eos)
    outputs = generate(model, prompts, args.max_new_tokens, args.temperature, args.top_k or None,
                       stop_ids=stop_ids, seed=args.seed)
    for prompt, tokens in zip(prompts, outputs):
        shown = tokens[:-1] if tokens and tokens[-1] in stop_ids else tokens
        if tokenizer is not None:
            print(tokenizer.decode(prompt) + tokenizer.decode(shown))
        else:
            print(",".join(str(t) for t in shown))
        print("---")
    if scratch is not None:
        scratch.cleanup()
    return 0


if __name__ == "__main__":
    sys.exit(main())
