"""Interactive terminal chat over the in-process engine.

The command names and what they do are Azimml/shrike's (shrike/CLI_SPEC.md, "Slash
commands"; shrike/cli.py:29-52): /help /clear /metrics /reset /temp /max /budget /bench
/system /exit; chat samples at temperature 0.7, top_p 0.9, up to 512 new tokens; every
reply ends with a status line (tokens, seconds, tokens per second, time to the first
token); Ctrl-C during a reply aborts it and gives its pages back, Ctrl-C at the prompt
only prints a hint, Ctrl-D or /exit leaves.  `/spec` and `/cache` are gone with the
features they switched.  The program itself is this package's own: a table of commands,
each with one argument reader and one handler, and a `Console` that owns the
conversation.  A model folder without tokenizer files is served too: a line of
space-separated token ids is the prompt then, and ids are printed back.

    python -m shrike_b200.cli --model DIR | --random SHAPE [--seed 0]
        [--dtype bfloat16|float32] [--block-size 16] [--num-blocks N] [--gpu-mem-util 0.85]
        [--max-tokens-per-step 512] [--max-running 256]

`--random SHAPE` starts without a checkpoint: SHAPE names one of the package's shape
files (`shrike_b200/shapes/`, e.g. qwen2.5-7b, tiny) or is the path of a config.json, and
the weights are drawn on the GPU from `--seed`.
"""

from __future__ import annotations

import argparse
import sys
import time
from dataclasses import dataclass
from typing import Callable

from .engine.request import SamplingParams
from .settings import DEFAULT_MODEL_DIR

CHAT_TEMPERATURE, CHAT_TOP_P, CHAT_MAX_NEW_TOKENS = 0.7, 0.9, 512


def add_engine_options(parser: argparse.ArgumentParser) -> None:
    """The options every entry point of the package shares: where the model comes from and how
    the engine is sized.  The names are the constructor arguments of Azimml/shrike's LLMEngine
    (shrike/engine/engine.py:42-53) with dashes."""
    parser.add_argument("--model", default=None, help=f"model folder (default {DEFAULT_MODEL_DIR})")
    parser.add_argument("--random", default=None, metavar="SHAPE",
                        help="no checkpoint: a named shape or a config.json, filled with random weights")
    parser.add_argument("--seed", type=int, default=0, help="seed of random weights and of sampling")
    parser.add_argument("--dtype", default=None, choices=["bfloat16", "float32"])
    parser.add_argument("--block-size", type=int, default=16)
    parser.add_argument("--num-blocks", type=int, default=None)
    parser.add_argument("--gpu-mem-util", type=float, default=0.85)
    parser.add_argument("--max-tokens-per-step", type=int, default=512)
    parser.add_argument("--max-running", type=int, default=256)
    parser.add_argument("--warm-up", action="store_true",
                        help="run a throw-away step per usual token count before the first request (LLMEngine.warm_up)")


def open_engine(args):
    """The engine the shared options describe, and a name for it."""
    from .engine import llm_engine

    if args.random is not None and args.model is not None:
        raise SystemExit("give --model or --random, not both")
    options = dict(block_size=args.block_size, gpu_mem_util=args.gpu_mem_util,
                   max_tokens_per_step=args.max_tokens_per_step, max_running=args.max_running,
                   num_blocks=args.num_blocks, dtype=args.dtype, seed=args.seed)
    if args.random is not None:
        engine, name = llm_engine.LLMEngine.from_random(args.random, **options), f"random weights, shape {args.random}"
    else:
        name = args.model or DEFAULT_MODEL_DIR
        engine = llm_engine.LLMEngine(name, **options)
    if getattr(args, "warm_up", False):
        engine.warm_up()
    return engine, name


def parse_args(argv=None) -> argparse.Namespace:
    parser = argparse.ArgumentParser(description="Chat with a local model through shrike_b200")
    add_engine_options(parser)
    return parser.parse_args(argv)


# ---- argument readers: text after the command -> value, or ValueError ------------------
def _number(kind, low, inclusive=True):
    def read(text: str):
        value = kind(text)
        if value != value or value == float("inf") or value < low or (value == low and not inclusive):
            raise ValueError(text)
        return value
    return read


def _bench_arguments(text: str):
    fields = text.split()
    if not 1 <= len(fields) <= 2:
        raise ValueError(text)
    count = _number(int, 1)(fields[0])
    tokens = _number(int, 1)(fields[1]) if len(fields) == 2 else 64
    return count, tokens


def _text(text: str) -> str:
    if not text:
        raise ValueError(text)
    return text


@dataclass(frozen=True)
class Command:
    name: str
    signature: str                       # how the argument is shown in /help and in a usage hint
    summary: str
    handler: Callable                    # Console method; gets the read argument when `read` is set
    read: Callable | None = None


class TokenPrinter:
    """Turns a stream of token ids into printable text.  With a tokenizer, ids are held back
    while they decode to half a character (shrike/CLI_SPEC.md, "Behavior"); without one the
    ids themselves are printed."""

    def __init__(self, tokenizer):
        self.tokenizer = tokenizer
        self.held: list[int] = []

    def feed(self, token_id: int) -> str:
        if self.tokenizer is None:
            return f"{token_id} "
        self.held.append(token_id)
        text = self.tokenizer.decode(self.held, skip_special_tokens=True)
        if text.endswith("�"):
            return ""
        self.held.clear()
        return text


def run_requests(engine, on_output=None) -> tuple[int, int]:
    """Steps the engine until it is idle; returns (outputs seen, steps)."""
    outputs = steps = 0
    while engine.has_work:
        for output in engine.step():
            outputs += 1
            if on_output is not None:
                on_output(output)
        steps += 1
    return outputs, steps


class Console:
    """One conversation with one engine: the settings the commands change, and the turns."""

    def __init__(self, engine, write=print, color: bool = False):
        self.engine = engine
        self.write = write
        self.color = color
        self.turns: list[dict] = []          # {role, content[, ids]} as a chat template takes them
        self.temperature = CHAT_TEMPERATURE
        self.max_new_tokens = CHAT_MAX_NEW_TOKENS
        self.commands = {c.name: c for c in (
            Command("/help", "", "this list", Console.show_help),
            Command("/clear", "", "forget the conversation so far", Console.clear),
            Command("/metrics", "", "engine counters: steps, tokens, KV blocks, preemptions", Console.show_metrics),
            Command("/reset", "", "set the counters of /metrics back to zero", Console.reset_metrics),
            Command("/temp", "<float >= 0>", "sampling temperature; 0 decodes greedily", Console.set_temperature,
                    _number(float, 0.0)),
            Command("/max", "<int >= 1>", "most new tokens per reply", Console.set_max_new_tokens, _number(int, 1)),
            Command("/budget", "<int >= 1>", "tokens the scheduler runs per step (chunked prefill)",
                    Console.set_budget, _number(int, 1)),
            Command("/bench", "<requests> [tokens each, default 64]",
                    "run that many identical greedy requests at once and report the throughput",
                    Console.bench, _bench_arguments),
            Command("/system", "<text>", "set or replace the system message", Console.set_system, _text),
            Command("/exit", "", "leave", Console.leave),
        )}

    # ---- dispatch ---------------------------------------------------------------
    def handle(self, line: str) -> bool:
        """One input line.  Returns False when the session is over."""
        line = line.strip()
        if not line:
            return True
        if not line.startswith("/"):
            self.say(line)
            return True
        name, _, rest = line.partition(" ")
        command = self.commands.get(name)
        if command is None:
            self.write(f"{name} is not a command here; /help lists them.")
            return True
        if command.read is None:
            return command.handler(self) is not False
        try:
            value = command.read(rest.strip())
        except (ValueError, OverflowError):
            self.write(f"usage: {command.name} {command.signature}")
            return True
        return command.handler(self, value) is not False

    # ---- commands ---------------------------------------------------------------
    def show_help(self):
        width = max(len(f"{c.name} {c.signature}") for c in self.commands.values())
        for c in self.commands.values():
            self.write(f"  {f'{c.name} {c.signature}':<{width}}  {c.summary}")
        if self.engine.tokenizer is None:
            self.write("This model folder has no tokenizer: a prompt is a line of token ids, e.g. 12 7 105")

    def clear(self):
        self.turns.clear()
        self.write("conversation cleared")

    def show_metrics(self):
        metrics = self.engine.metrics()
        width = max(map(len, metrics))
        for key, value in metrics.items():
            self.write(f"{key:<{width}}  {value}")

    def reset_metrics(self):
        self.engine.reset_stats()
        self.write("counters are back at zero")

    def set_temperature(self, value: float):
        self.temperature = value
        self.write(f"temperature = {value:g}" + (" (greedy)" if value == 0 else ""))

    def set_max_new_tokens(self, value: int):
        self.max_new_tokens = value
        self.write(f"replies stop after {value} new tokens")

    def set_budget(self, value: int):
        self.engine.scheduler.max_tokens_per_step = value
        self.write(f"the scheduler now runs up to {value} tokens per step")

    def set_system(self, text: str):
        if self.engine.tokenizer is None:
            self.write("a system message needs a tokenizer, and this model folder has none")
            return
        replaced = bool(self.turns) and self.turns[0]["role"] == "system"
        if replaced:
            self.turns[0]["content"] = text
        else:
            self.turns.insert(0, {"role": "system", "content": text})
        self.write("system message replaced" if replaced else "system message set")

    def leave(self):
        return False

    def bench(self, arguments):
        """`count` identical greedy requests of fixed length, run together (the `/bench` of
        shrike/cli.py:55-77; the prompt here is 16 fixed token ids, since random-weight folders
        have no tokenizer)."""
        count, tokens = arguments
        vocab = self.engine.config.vocab_size
        prompt = [(7 * i + 3) % vocab for i in range(16)]
        sampling = SamplingParams(max_new_tokens=tokens, temperature=0.0, ignore_eos=True)
        try:
            for _ in range(count):
                self.engine.add_request(prompt, sampling)
        except ValueError as error:
            self.write(f"refused: {error}")
            return
        began = time.perf_counter()
        generated, steps = run_requests(self.engine)
        seconds = max(time.perf_counter() - began, 1e-9)
        self.write(f"{count} requests x {tokens} tokens: {generated} tokens in {seconds:.2f} s, "
                   f"{generated / seconds:.0f} tok/s in all, {generated / seconds / count:.1f} tok/s each, {steps} steps")

    # ---- a turn -----------------------------------------------------------------
    def _prompt_ids(self, line: str):
        """Token ids of the conversation with `line` as the next user turn, and the turn."""
        tokenizer = self.engine.tokenizer
        if tokenizer is not None:
            turn = {"role": "user", "content": line}
            encoded = tokenizer.apply_chat_template(self.turns + [turn], add_generation_prompt=True)
            return list(encoded["input_ids"] if isinstance(encoded, dict) else encoded), turn
        try:
            ids = [int(field) for field in line.split()]
        except ValueError:
            self.write("no tokenizer in this model folder: type token ids separated by spaces, or a /command")
            return None, None
        history = [token for turn in self.turns for token in turn.get("ids", [])]
        return history + ids, {"role": "user", "content": line, "ids": ids}

    def say(self, line: str):
        ids, turn = self._prompt_ids(line)
        if ids is None:
            return
        reply = self.stream(ids)
        if reply is None:
            return
        text, generated = reply
        self.turns.append(turn)
        answer = {"role": "assistant", "content": text}
        if self.engine.tokenizer is None:
            answer["ids"] = generated
        self.turns.append(answer)

    def stream(self, prompt_ids):
        """One request, printed as it is generated.  Returns (text, token ids), or None when
        the request was refused or interrupted (its pages are back in the pool then)."""
        sampling = SamplingParams(max_new_tokens=self.max_new_tokens, temperature=self.temperature, top_p=CHAT_TOP_P)
        try:
            request_id = self.engine.add_request(prompt_ids, sampling, chat=False)
        except ValueError as error:
            self.write(f"refused: {error}")
            return None
        printer = TokenPrinter(self.engine.tokenizer)
        generated: list[int] = []
        pieces: list[str] = []
        began = time.perf_counter()
        first = [None]

        def show(output):
            if output.req_id != request_id:
                return
            if first[0] is None:
                first[0] = time.perf_counter()
            generated.append(output.token_id)
            piece = printer.feed(output.token_id)
            if piece:
                pieces.append(piece)
                print(piece, end="", flush=True)

        try:
            run_requests(self.engine, show)
        except KeyboardInterrupt:
            self.engine.abort(request_id)
            self.write("\n(interrupted; the reply is dropped)")
            return None
        seconds = max(time.perf_counter() - began, 1e-9)
        waited = (first[0] - began) * 1000 if first[0] is not None else 0.0
        status = (f"[{len(generated)} tok | {seconds:.1f} s | {len(generated) / seconds:.0f} tok/s | "
                  f"first token after {waited:.0f} ms]")
        self.write("")
        self.write(f"\033[2m{status}\033[0m" if self.color else status)
        return "".join(pieces), generated


def main(argv=None) -> None:
    args = parse_args(argv)
    try:
        import readline  # noqa: F401  (line editing and history at the prompt)
    except ImportError:
        pass
    color = sys.stdout.isatty()
    began = time.perf_counter()
    print("loading ...", flush=True)
    engine, name = open_engine(args)
    print(f"shrike_b200 ready: {name}, {engine.block_manager.total_pages} KV blocks of "
          f"{engine.block_manager.page_size} tokens, {time.perf_counter() - began:.1f} s to load; /help lists commands")
    console = Console(engine, color=color)
    prompt = "\001\033[1;36m\002shrike_b200> \001\033[0m\002" if color else "shrike_b200> "
    alive = True
    while alive:
        try:
            line = input(prompt)
        except EOFError:
            print()
            break
        except KeyboardInterrupt:
            print("\n(/exit or Ctrl-D leaves)")
            continue
        alive = console.handle(line)


if __name__ == "__main__":
    main()
