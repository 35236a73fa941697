"""Interactive terminal chat over the in-process engine.

The commands and their meanings are those of Azimml/shrike's REPL
(shrike/cli.py:29-52,173-283): /help /clear /metrics /reset /temp /max /budget
/bench /system /exit; chat defaults temperature 0.7, top_p 0.9, 512 new tokens
(cli.py:110,169-170); a status line with tokens, seconds, tokens per second and the
time to the first token after each reply (cli.py:145-150); Ctrl-C aborts the reply
and frees its pages (cli.py:131-143).  `/spec` and `/cache` are gone with the
features they switched.  A model folder without tokenizer files is served too: a
line of space-separated token ids is the prompt then, and ids are printed back.

    python -m shrike_b200.cli --model DIR [--dtype bfloat16|float32] [--block-size 16]
        [--num-blocks N] [--gpu-mem-util 0.85] [--max-tokens-per-step 512] [--max-running 256]
        [--seed 0]
"""

from __future__ import annotations

import argparse
import sys
import time

from .engine.request import SamplingParams
from .settings import DEFAULT_MODEL_DIR

HELP = """Commands:
  /help                Show this help
  /clear               Clear conversation history
  /metrics             Show engine metrics (steps, tokens, blocks, preemptions)
  /reset               Zero the metrics counters (clean measurements)
  /temp <float>        Set temperature; 0 uses greedy decoding
  /max <int>           Set maximum new tokens
  /budget <int>        Set scheduler token budget per step (chunked prefill)
  /bench <n> [tokens]  Fire n concurrent requests (default 64 tokens each)
                       and report aggregate throughput
  /system <text>       Set or replace the system message
  /exit                Quit

Without tokenizer files in the model folder a prompt is a line of token ids: 12 7 105"""


def parse_args(argv=None) -> argparse.Namespace:
    parser = argparse.ArgumentParser(description="Chat with a local model through shrike_b200")
    parser.add_argument("--model", default=DEFAULT_MODEL_DIR)
    parser.add_argument("--dtype", default=None, choices=["bfloat16", "float32"])
    parser.add_argument("--block-size", type=int, default=16)
    parser.add_argument("--num-blocks", type=int, default=None)
    parser.add_argument("--gpu-mem-util", type=float, default=0.85)
    parser.add_argument("--max-tokens-per-step", type=int, default=512)
    parser.add_argument("--max-running", type=int, default=256)
    parser.add_argument("--seed", type=int, default=0)
    return parser.parse_args(argv)


def _dim(text: str, enabled: bool) -> str:
    return f"\033[2m{text}\033[0m" if enabled else text


def run_bench(engine, count: int, tokens: int, out=print) -> None:
    """n identical requests, greedy, fixed length (shrike/cli.py:55-77)."""
    if engine.tokenizer is not None:
        prompt = "Explain why paged memory management helps LLM serving."
    else:
        vocab = engine.config.vocab_size
        prompt = [(7 * i + 3) % vocab for i in range(16)]
    sampling = SamplingParams(max_new_tokens=tokens, temperature=0.0, ignore_eos=True)
    try:
        for _ in range(count):
            engine.add_request(prompt, sampling)
    except ValueError as error:
        out(f"[error] {error}")
        return
    started = time.perf_counter()
    generated = steps = 0
    while engine.has_work:
        generated += len(engine.step())
        steps += 1
    elapsed = time.perf_counter() - started
    out(f"{count} reqs x {tokens} tok -> {generated} tok in {elapsed:.2f}s = {generated / elapsed:.0f} tok/s aggregate "
        f"({generated / elapsed / count:.1f} tok/s per request, {steps} steps)")


def stream_reply(engine, prompt_ids, temperature, max_new_tokens, use_color, out=None):
    """Adds one request and prints its tokens as they come.  Returns the reply text
    (or token ids as text), or None when the request was refused or aborted."""
    out = out or sys.stdout
    started = time.perf_counter()
    first_at = None
    generated: list[int] = []
    pending: list[int] = []
    parts: list[str] = []
    request_id = None
    try:
        sampling = SamplingParams(max_new_tokens=max_new_tokens, temperature=temperature, top_p=0.9)
        try:
            request_id = engine.add_request(prompt_ids, sampling, chat=False)
        except ValueError as error:
            print(f"[error] {error}", file=out)
            return None
        while engine.has_work:
            for output in engine.step():
                if output.req_id != request_id:
                    continue
                if first_at is None:
                    first_at = time.perf_counter()
                generated.append(output.token_id)
                if engine.tokenizer is None:
                    text = f"{output.token_id} "
                else:
                    pending.append(output.token_id)
                    text = engine.tokenizer.decode(pending, skip_special_tokens=True)
                    if text.endswith("�"):  # half a character: wait for the rest
                        continue
                    pending.clear()
                print(text, end="", flush=True, file=out)
                parts.append(text)
    except KeyboardInterrupt:
        if request_id is not None:
            engine.abort(request_id)
        print("\n[aborted]", file=out)
        return None
    elapsed = time.perf_counter() - started
    ttft = (first_at - started) * 1000 if first_at is not None else 0.0
    rate = len(generated) / max(elapsed, 1e-9)
    print(file=out)
    print(_dim(f"⏱ {len(generated)} tok · {elapsed:.1f}s · {rate:.0f} tok/s · TTFT {ttft:.0f}ms", use_color), file=out)
    return "".join(parts)


def encode_turn(engine, messages, line):
    """Token ids for the conversation so far; None (with a message printed) when the line cannot be used."""
    if engine.tokenizer is not None:
        encoded = engine.tokenizer.apply_chat_template(messages, add_generation_prompt=True)
        return list(encoded["input_ids"] if isinstance(encoded, dict) else encoded)
    try:
        ids = [int(field) for field in line.split()]
    except ValueError:
        print("This model folder has no tokenizer: enter token ids separated by spaces, or a /command.")
        return None
    history = [tid for message in messages[:-1] for tid in message.get("ids", [])]
    return history + ids


def main(argv=None) -> None:
    args = parse_args(argv)
    try:
        import readline  # noqa: F401  (line editing at the prompt)
    except ImportError:
        pass
    from .engine.llm_engine import EngineStats, LLMEngine

    use_color = sys.stdout.isatty()
    print(f"Loading {args.model} ...", flush=True)
    started = time.perf_counter()
    engine = LLMEngine(
        args.model, block_size=args.block_size, gpu_mem_util=args.gpu_mem_util,
        max_tokens_per_step=args.max_tokens_per_step, max_running=args.max_running,
        num_blocks=args.num_blocks, dtype=args.dtype, seed=args.seed,
    )
    print(f"shrike_b200 ready · {args.model} · {min(engine.block_manager.num_pages)} KV blocks "
          f"· loaded in {time.perf_counter() - started:.1f}s")

    messages: list[dict] = []
    temperature, max_new_tokens = 0.7, 512
    prompt = "\001\033[1;36m\002shrike> \001\033[0m\002" if use_color else "shrike> "
    while True:
        try:
            line = input(prompt)
        except EOFError:
            print()
            break
        except KeyboardInterrupt:
            print("\nUse /exit to quit.")
            continue
        if not line.strip():
            continue
        if line.startswith("/"):
            command, _, argument = line.strip().partition(" ")
            argument = argument.strip()
            if command == "/exit":
                break
            if command == "/help":
                print(HELP)
            elif command == "/clear":
                messages.clear()
                print("Conversation cleared.")
            elif command == "/metrics":
                metrics = engine.metrics()
                width = max(len(key) for key in metrics)
                for key, value in metrics.items():
                    print(f"{key:<{width}}  {value}")
            elif command == "/reset":
                engine.stats = EngineStats()
                engine.scheduler.num_preemptions = 0
                print("Metrics counters reset.")
            elif command == "/temp":
                try:
                    value = float(argument)
                    if not 0 <= value < float("inf"):
                        raise ValueError
                except ValueError:
                    print("Usage: /temp <non-negative float>")
                else:
                    temperature = value
                    print(f"Temperature set to {temperature:g}.")
            elif command == "/max":
                try:
                    value = int(argument)
                    if value <= 0:
                        raise ValueError
                except ValueError:
                    print("Usage: /max <positive int>")
                else:
                    max_new_tokens = value
                    print(f"Maximum new tokens set to {max_new_tokens}.")
            elif command == "/budget":
                try:
                    value = int(argument)
                    if value < 1:
                        raise ValueError
                except ValueError:
                    print("Usage: /budget <positive int>")
                else:
                    engine.scheduler.max_tokens_per_step = value
                    print(f"Scheduler token budget set to {value} per step.")
            elif command == "/bench":
                fields = argument.split()
                try:
                    count = int(fields[0])
                    tokens = int(fields[1]) if len(fields) > 1 else 64
                    if count < 1 or tokens < 1:
                        raise ValueError
                except (IndexError, ValueError):
                    print("Usage: /bench <num_requests> [tokens_each]")
                else:
                    run_bench(engine, count, tokens)
            elif command == "/system":
                if not argument:
                    print("Usage: /system <text>")
                elif engine.tokenizer is None:
                    print("A system message needs a tokenizer; this model folder has none.")
                elif messages and messages[0]["role"] == "system":
                    messages[0]["content"] = argument
                    print("System message updated.")
                else:
                    messages.insert(0, {"role": "system", "content": argument})
                    print("System message set.")
            else:
                print(f"Unknown command: {command}. Type /help for commands.")
            continue

        messages.append({"role": "user", "content": line})
        prompt_ids = encode_turn(engine, messages, line)
        if prompt_ids is None:
            messages.pop()
            continue
        if engine.tokenizer is None:
            messages[-1]["ids"] = [int(field) for field in line.split()]
        reply = stream_reply(engine, prompt_ids, temperature, max_new_tokens, use_color)
        if reply is None:
            messages.pop()
        elif engine.tokenizer is None:
            messages.append({"role": "assistant", "content": reply, "ids": [int(t) for t in reply.split()]})
        else:
            messages.append({"role": "assistant", "content": reply})


if __name__ == "__main__":
    main()
