"""Makes tests/golden/*.npz: logits and greedy tokens of the reference's OWN model code
(qtris123/gtar-kimik3-public, src/models/transformer.py + src/engine.py) on two tiny random models,
float32 on the CPU.  Run once, from the repository root, with the reference checkout's path:

    python tests/golden/make_golden.py /path/to/gtar-kimik3-public

The weights come from tests/plain/weights.py::make_weights(cfg, seed) and are loaded into the
reference model with load_state_dict, so the test can regenerate them instead of storing them.
Each request runs alone (the reference takes only rectangular batches, src/engine.py:31).
tests/test_plain_golden.py compares the plain implementation under tests/plain/ with these files.
"""

import sys
from pathlib import Path

import numpy as np
import torch

REPO = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(REPO))

from tests.plain.weights import make_weights  # noqa: E402
from tests.tiny_configs import TINY_A, TINY_B  # noqa: E402


def main(reference_root: str) -> None:
    sys.dont_write_bytecode = True
    sys.path.insert(0, reference_root)
    from src.engine import Engine
    from src.models import ARCHITECTURES

    Config, ForCausalLM = ARCHITECTURES["transformer"]
    fields = set(Config.__dataclass_fields__)
    for tag, cfg, seed, lengths, n_new in (("tiny_a", TINY_A, 0, (5, 17, 32), 16), ("tiny_b", TINY_B, 1, (1, 9, 40), 8)):
        model = ForCausalLM(Config(**{k: v for k, v in cfg.items() if k in fields})).eval()
        weights = make_weights(cfg, seed, std=0.08)
        state = dict(weights)
        if cfg["tie_word_embeddings"]:
            state["lm_head.weight"] = state["model.embed_tokens.weight"]
        model.load_state_dict(state, strict=True)
        gen = torch.Generator().manual_seed(1000 + seed)
        out = {}
        for r, n in enumerate(lengths):
            ids = torch.randint(0, cfg["vocab_size"], (n,), generator=gen)
            with torch.no_grad():
                logits = model(ids[None])[0].float()
                tokens = Engine(model).generate(ids[None], n_new, temperature=0.0)[0]
            out[f"ids_{r}"] = ids.numpy().astype(np.int32)
            out[f"logits_{r}"] = logits.numpy().astype(np.float32)
            out[f"greedy_{r}"] = tokens.numpy().astype(np.int32)
        np.savez_compressed(Path(__file__).parent / f"{tag}.npz", **out)
        print(tag, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1])
