"""Trace replay: feeds given token ids through the model step by step, writes logits.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps come on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step are one batch.  For a step in which something is wanted,
`OUT/<step>.f32` holds the logits at the wanted places, in the order of the entries
and of `want`, as little-endian float32 [wanted, vocab].  After every step the line
`done <step>` is printed.  Nothing is sampled.  The program has no model code of its
own: it loads through the package's loader, keeps pages through its cache manager
and runs its step function (`ModelRunner.step`), the one generation uses.  The
nearest thing in Azimml/shrike is the teacher forcing in tests/test_paged.py:76-98.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np
import torch

PAGE_SIZE = 16
MAX_LIVE = 16


class TraceSession:
    """The replay state: a model, its cache pool, and the live requests' pages."""

    def __init__(self, model_dir, dtype: str, max_tokens: int, device="cuda"):
        from . import models as _models  # noqa: F401
        from .config.registry import load_config
        from .engine.llm_engine import make_ops
        from .engine.runner import TORCH_DTYPES, ModelRunner
        from .weights.loader import load_weights

        self.device = torch.device(device)
        self.config = load_config(model_dir)
        ops = make_ops(dtype, self.device)
        tensors = load_weights(model_dir, self.config, TORCH_DTYPES[dtype], self.device)
        num_pages = max(1, -(-max_tokens // PAGE_SIZE))
        self.max_tokens = max_tokens
        self.runner = ModelRunner(self.config, tensors, ops, self.device, dtype, page_size=PAGE_SIZE,
                                  num_pages=num_pages, max_slots=MAX_LIVE)
        self.live: dict[str, list] = {}  # id -> [RequestCache, tokens fed]

    def step(self, record: dict):
        """Runs one step; returns float32 logits [wanted, vocab] on the host, or None."""
        from .engine.batch import StepEntry

        cache_manager = self.runner.cache
        step, vocab = record.get("step"), self.config.vocab_size
        entries = []
        for item in record.get("entries", []):
            ident, tokens = str(item["id"]), [int(t) for t in item["tokens"]]
            if not tokens:
                continue
            if min(tokens) < 0 or max(tokens) >= vocab:
                raise ValueError(f"step {step}: token ids of {ident!r} lie outside [0, {vocab})")
            if ident not in self.live:
                self.live[ident] = [cache_manager.open(), 0]
            cache, fed = self.live[ident]
            if not cache_manager.can_append(cache, fed, len(tokens)):
                raise RuntimeError(
                    f"step {step}: no pages left for {len(tokens)} tokens of {ident!r} "
                    f"(--max-tokens {self.max_tokens}; free pages {cache_manager.num_free})"
                )
            cache_manager.append(cache, fed, len(tokens))
            entries.append((ident, StepEntry(cache, tokens, fed, [int(w) for w in item.get("want", [])])))
        result = None
        if entries:
            logits = self.runner.step([entry for _, entry in entries])
            if logits.shape[0]:
                result = logits.cpu().numpy()
            for ident, entry in entries:
                self.live[ident][1] += len(entry.tokens)
                cache_manager.advance(self.live[ident][0], self.live[ident][1])
        for ident in record.get("end", []):
            held = self.live.pop(str(ident), None)
            if held is not None:
                cache_manager.free(held[0])
        return result


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at once (each rounded up to 64)")
    args = parser.parse_args(argv)
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    session = TraceSession(args.model, args.dtype, args.max_tokens)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        logits = session.step(record)
        if logits is not None:
            logits.astype("<f4", copy=False).tofile(out_dir / f"{record['step']}.f32")
        else:
            torch.cuda.synchronize()
        print(f"done {record['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
