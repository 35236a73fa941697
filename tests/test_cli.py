"""The command line on a pipe (shrike CLI_SPEC.md, "Acceptance": it must work without a TTY),
its commands, token-id prompts, the shared engine options, and the one-prompt program."""

import io
import sys

import pytest

import shrike_b200.models  # noqa: F401
from shrike_b200 import cli, complete
from shrike_b200.config import parse_config
from shrike_b200.engine.llm_engine import LLMEngine
from shrike_b200.shapes import known_shapes, shape_config
from shrike_b200.weights import random_tensors
from tests.emulated_ops import EmulatedOps
from tests.tiny_configs import TINY_A

COMMANDS = ("/help", "/clear", "/metrics", "/reset", "/temp", "/max", "/budget", "/bench", "/system", "/exit")


def test_options_keep_the_reference_names():
    args = cli.parse_args(["--model", "some/dir"])
    assert args.model == "some/dir" and args.block_size == 16 and args.max_tokens_per_step == 512
    assert args.max_running == 256 and args.gpu_mem_util == 0.85 and args.dtype is None
    assert args.random is None and args.seed == 0
    args = cli.parse_args(["--random", "tiny", "--seed", "4", "--num-blocks", "12"])
    assert args.random == "tiny" and args.seed == 4 and args.num_blocks == 12 and args.model is None


def test_shapes_are_config_files_of_a_registered_architecture():
    assert {"tiny", "qwen2.5-7b", "qwen2.5-1.5b", "qwen2.5-14b"} <= set(known_shapes())
    for name in known_shapes():
        config = parse_config(shape_config(name))
        assert config.num_layers >= 1 and config.vocab_size > 0
    assert shape_config("7b") == shape_config("qwen2.5-7b")
    with pytest.raises(FileNotFoundError, match="tiny"):
        shape_config("no-such-shape")


def fake_engine(monkeypatch, seen=None):
    config = parse_config(TINY_A)

    def make(model_dir, **kw):
        if seen is not None:
            seen.update(kw, model_dir=model_dir)
        kw = {k: v for k, v in kw.items() if k in ("block_size", "max_tokens_per_step", "max_running", "seed")}
        return LLMEngine(None, num_blocks=32, dtype="float32", device="cpu", config=config,
                         tensors=dict(random_tensors(config, 0)), ops=EmulatedOps(), **kw)

    import shrike_b200.engine.llm_engine as module

    make.from_random = lambda shape, **kw: make(None, shape=shape, **kw)
    monkeypatch.setattr(module, "LLMEngine", make)


def test_repl_on_a_pipe(monkeypatch, capsys):
    fake_engine(monkeypatch)
    lines = ("/help\n/temp 0\n/max 5\n/budget 7\n5 17 3 9\n/metrics\n/bench 3 4\n/temp x\n/temp -1\n/max 0\n"
             "/bench\n/nonsense\nhello\n/system be brief\n/reset\n/metrics\n/clear\n/exit\nnever reached\n")
    monkeypatch.setattr(sys, "stdin", io.StringIO(lines))
    cli.main(["--model", "unused"])
    out = capsys.readouterr().out
    assert "shrike_b200 ready" in out and "KV blocks" in out
    for command in COMMANDS:
        assert command in out                                  # /help lists every command
    assert "temperature = 0 (greedy)" in out and "replies stop after 5 new tokens" in out
    assert "up to 7 tokens per step" in out
    assert "[5 tok |" in out and "first token after" in out    # the reply's status line
    assert "tokens_generated" in out and "kv_blocks_free" in out
    assert "3 requests x 4 tokens: 12 tokens in" in out
    assert out.count("usage: /temp") == 2 and "usage: /max" in out and "usage: /bench" in out
    assert "/nonsense is not a command here" in out
    assert "type token ids" in out and "needs a tokenizer" in out
    assert "counters are back at zero" in out and "conversation cleared" in out
    assert "never reached" not in out
    after_reset = out.split("counters are back at zero")[1]
    assert "tokens_generated    0\n" in after_reset


def test_a_conversation_keeps_its_token_ids(monkeypatch, capsys):
    fake_engine(monkeypatch)
    config = parse_config(TINY_A)
    engine = LLMEngine(None, num_blocks=32, dtype="float32", device="cpu", config=config,
                       tensors=dict(random_tensors(config, 0)), ops=EmulatedOps())
    seen = []
    add = engine.add_request
    engine.add_request = lambda ids, sampling, chat=True: (seen.append(list(ids)), add(ids, sampling, chat))[1]
    console = cli.Console(engine)
    console.handle("/temp 0")
    console.handle("/max 3")
    console.handle("5 17 3")
    console.handle("9 9")
    assert seen[0] == [5, 17, 3]
    first_reply = console.turns[1]["ids"]
    assert len(first_reply) == 3 and seen[1] == [5, 17, 3] + first_reply + [9, 9]
    console.handle("/clear")
    console.handle("4")
    assert seen[2] == [4] and engine.block_manager.whole()


def test_end_of_input_quits(monkeypatch, capsys):
    fake_engine(monkeypatch)
    monkeypatch.setattr(sys, "stdin", io.StringIO(""))
    cli.main(["--model", "unused"])
    assert "ready" in capsys.readouterr().out


def test_random_shape_reaches_the_engine(monkeypatch, capsys):
    seen = {}
    fake_engine(monkeypatch, seen)
    monkeypatch.setattr(sys, "stdin", io.StringIO("/exit\n"))
    cli.main(["--random", "tiny", "--seed", "3", "--num-blocks", "9"])
    assert seen["shape"] == "tiny" and seen["seed"] == 3 and seen["num_blocks"] == 9
    assert "random weights, shape tiny" in capsys.readouterr().out
    with pytest.raises(SystemExit):
        cli.main(["--random", "tiny", "--model", "x"])


def test_one_prompt_program(monkeypatch, capsys):
    fake_engine(monkeypatch)
    assert complete.main(["5, 17 3", "--max-tokens", "4", "--model", "unused"]) == 0
    captured = capsys.readouterr()
    tokens = [int(t) for t in captured.out.split()]
    assert len(tokens) == 4 and all(0 <= t < 256 for t in tokens)
    assert "engine up in" in captured.err and "4 tokens in" in captured.err
    with pytest.raises(SystemExit, match="token ids"):
        complete.main(["hello there", "--model", "unused"])


def test_from_random_builds_an_engine_from_a_shape_file():
    engine = LLMEngine.from_random("tiny", seed=1, dtype="float32", device="cpu", num_blocks=8, ops=EmulatedOps())
    assert engine.config.hidden_size == 192 and engine.seed == 1
    from shrike_b200 import SamplingParams

    out = engine.generate([[1, 2, 3]], SamplingParams(max_new_tokens=2))
    assert len(out[0]) == 2 and engine.block_manager.whole()
