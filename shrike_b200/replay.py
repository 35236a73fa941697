"""Trace replay: feeds given token ids through the model step by step, writes logits.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N
              [--block-size 16] [--num-blocks B] [--max-live 16]

Steps come on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step are one batch.  For a step in which something is wanted,
`OUT/<step>.f32` holds the logits at the wanted places, in the order of the entries
and of `want`, as little-endian float32 [wanted, vocab].  After every step the line
`done <step>` is printed.  Nothing is sampled.  The program has no model code of its
own: it loads through the package's loader, keeps pages through its cache manager
and runs its step function (`ModelRunner.step`), the one generation uses.  The
nearest thing in Azimml/shrike is the teacher forcing in tests/test_paged.py:76-98,
and the explicit `block_size` and pool size of its engine (shrike/engine/engine.py:42-53)
as its paged tests set them (tests/test_paged.py:22-26).

The pool.  `--block-size` is the number of tokens a page holds.  `--num-blocks` gives
the number of pages outright; without it the pool is made for `--max-tokens`: the most
tokens that live requests hold at any time, each request's count rounded up to a
multiple of 64 (a page size that does not divide 64 gets one page more per live
request).  `--max-live` is the number of requests that may be live at once (state
slots).  The first line of the input may instead be a header,

    {"header": {"block_size": 8, "num_blocks": 20, "max_live": 4}}

whose keys fill what the command line left unset.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

DEFAULT_PAGE_SIZE = 16
DEFAULT_MAX_LIVE = 16


def pages_for(max_tokens: int, page_size: int, max_live: int) -> int:
    """Pages that hold `max_tokens` tokens of live requests, each request's count a multiple of 64."""
    pages = -(-max_tokens // page_size)
    if 64 % page_size:
        pages += max_live   # a request's last page may be part empty although its count is a multiple of 64
    return max(1, pages)


class TraceSession:
    """The replay state: a model, its cache pool, and the live requests' pages."""

    def __init__(self, model_dir, dtype: str, max_tokens: int | None = None, device="cuda",
                 page_size: int | None = None, num_pages: int | None = None, max_live: int | None = None,
                 ops=None):
        from . import models as _models  # noqa: F401
        from .config.registry import load_config
        from .engine.llm_engine import make_ops
        from .engine.runner import TORCH_DTYPES, ModelRunner
        from .weights.loader import load_weights

        page_size = page_size or DEFAULT_PAGE_SIZE
        max_live = max_live or DEFAULT_MAX_LIVE
        if page_size < 1 or max_live < 1:
            raise ValueError("block size and the number of live requests must be positive")
        if num_pages is None:
            if max_tokens is None:
                raise ValueError("the pool needs a size: --max-tokens or --num-blocks")
            num_pages = pages_for(max_tokens, page_size, max_live)
        self.device = torch.device(device)
        self.config = load_config(model_dir)
        if ops is None:
            ops = make_ops(dtype, self.device)
        tensors = load_weights(model_dir, self.config, TORCH_DTYPES[dtype], self.device)
        self.max_tokens = max_tokens
        self.page_size = page_size
        self.runner = ModelRunner(self.config, tensors, ops, self.device, dtype, page_size=page_size,
                                  num_pages=num_pages, max_slots=max_live)
        self.live: dict[str, list] = {}  # id -> [RequestCache, tokens fed]
        # (group, page id) -> the requests that held it, in order: what a test of page reuse reads
        self.page_owners: dict[tuple[int, int], list[str]] = {}

    def _note_pages(self, ident: str, cache) -> None:
        for group, table in enumerate(cache.tables):
            for page in table.view():
                if page >= 0:
                    owners = self.page_owners.setdefault((group, int(page)), [])
                    if not owners or owners[-1] != ident:
                        owners.append(ident)

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
                if not cache_manager.can_open():
                    raise RuntimeError(f"step {step}: {ident!r} would be live request number "
                                       f"{len(self.live) + 1}; raise --max-live")
                self.live[ident] = [cache_manager.open(), 0]
            cache, fed = self.live[ident]
            if not cache_manager.can_append(cache, fed, len(tokens)):
                raise RuntimeError(
                    f"step {step}: no pages left for {len(tokens)} tokens of {ident!r} "
                    f"(pool of {cache_manager.num_pages} pages of {self.page_size}; free {cache_manager.num_free})"
                )
            cache_manager.append(cache, fed, len(tokens))
            self._note_pages(ident, cache)
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


def parse_args(argv=None) -> argparse.Namespace:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, default=None,
                        help="most tokens live requests hold at once (each rounded up to 64); sizes the pool")
    parser.add_argument("--block-size", type=int, default=None, help=f"tokens per page (default {DEFAULT_PAGE_SIZE})")
    parser.add_argument("--num-blocks", type=int, default=None, help="pages in the pool, instead of --max-tokens")
    parser.add_argument("--max-live", type=int, default=None,
                        help=f"requests that may be live at once (default {DEFAULT_MAX_LIVE})")
    args = parser.parse_args(argv)
    return args


def main(argv=None) -> int:
    args = parse_args(argv)
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    session = None
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        header = record.pop("header", None) if session is None else None
        if session is None:
            header = header or {}
            unknown = set(header) - {"block_size", "num_blocks", "max_live", "max_tokens"}
            if unknown:
                raise SystemExit(f"trace_run: unknown header keys {sorted(unknown)}")
            max_tokens = args.max_tokens if args.max_tokens is not None else header.get("max_tokens")
            num_blocks = args.num_blocks if args.num_blocks is not None else header.get("num_blocks")
            if max_tokens is None and num_blocks is None:
                raise SystemExit("trace_run: give --max-tokens or --num-blocks (or a header with one of them)")
            session = TraceSession(
                args.model, args.dtype, max_tokens,
                page_size=args.block_size or header.get("block_size"),
                num_pages=num_blocks, max_live=args.max_live or header.get("max_live"))
            if "step" not in record:
                continue   # the line held the header only
        logits = session.step(record)
        if logits is not None:
            logits.astype("<f4", copy=False).tofile(out_dir / f"{record['step']}.f32")
        else:
            torch.cuda.synchronize()
        print(f"done {record['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
