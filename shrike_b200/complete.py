"""One prompt in, its completion streamed out: the quickest way from a shell to tokens.

    python -m shrike_b200.complete [PROMPT] [--max-tokens 128] [--temperature 0.0]
        --model DIR | --random SHAPE [--seed 0] [--dtype ...] [--num-blocks N] ...

PROMPT is text when the model folder has tokenizer files; otherwise (and always with
`--random`) it is token ids separated by spaces or commas, and ids are printed back.
The completion goes to standard output as it is generated; what the engine needed to
start and the rate achieved go to standard error, so the output can be piped.  The
option names and defaults are those of Azimml/shrike's smoke script
(scripts/chat.py:17-22: positional prompt, --max-tokens 128, --temperature 0.0, --model);
the engine options are the ones the interactive command line takes.
"""

from __future__ import annotations

import argparse
import sys
import time

from .cli import TokenPrinter, add_engine_options, open_engine, run_requests
from .engine.request import SamplingParams

DEFAULT_IDS = "1 2 3 5 8 13 21 34"


def read_prompt(text: str, engine):
    """Text for a tokenizer, or token ids when there is none."""
    if engine.tokenizer is not None:
        return text
    try:
        return [int(field) for field in text.replace(",", " ").split()]
    except ValueError:
        raise SystemExit("this model has no tokenizer: the prompt must be token ids, e.g. \"5 17 3\"") from None


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="shrike_b200_complete", description=__doc__.split("\n\n")[0])
    parser.add_argument("prompt", nargs="?", default=None,
                        help="text, or token ids when the model has no tokenizer")
    parser.add_argument("--max-tokens", type=int, default=128)
    parser.add_argument("--temperature", type=float, default=0.0)
    add_engine_options(parser)
    args = parser.parse_args(argv)

    began = time.perf_counter()
    engine, name = open_engine(args)
    print(f"[{name}: engine up in {time.perf_counter() - began:.1f} s, "
          f"{engine.block_manager.total_pages} KV blocks]", file=sys.stderr, flush=True)
    default = "Explain in two sentences what a paged key/value cache is." if engine.tokenizer is not None else DEFAULT_IDS
    prompt = read_prompt(args.prompt if args.prompt is not None else default, engine)
    try:
        engine.add_request(prompt, SamplingParams(max_new_tokens=args.max_tokens, temperature=args.temperature))
    except ValueError as error:
        print(f"refused: {error}", file=sys.stderr)
        return 2
    printer = TokenPrinter(engine.tokenizer)

    def show(output):
        print(printer.feed(output.token_id), end="", flush=True)

    began = time.perf_counter()
    count, steps = run_requests(engine, show)
    seconds = max(time.perf_counter() - began, 1e-9)
    print()
    print(f"[{count} tokens in {seconds:.2f} s, {count / seconds:.1f} tok/s, {steps} steps]", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
