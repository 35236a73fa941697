"""The command line: options, commands on a non-TTY (shrike CLI_SPEC.md:48), token-id prompts."""

import io
import sys

import pytest

import shrike_b200.models  # noqa: F401
from shrike_b200 import cli
from shrike_b200.config import parse_config
from shrike_b200.engine.llm_engine import LLMEngine
from shrike_b200.weights import random_tensors
from tests.emulated_ops import EmulatedOps
from tests.tiny_configs import TINY_A


def test_options_keep_the_reference_names():
    args = cli.parse_args(["--model", "some/dir"])
    assert args.model == "some/dir" and args.block_size == 16 and args.max_tokens_per_step == 512
    assert args.max_running == 256 and args.gpu_mem_util == 0.85 and args.dtype is None
    for command in ("/help", "/clear", "/metrics", "/reset", "/temp", "/max", "/budget", "/bench", "/system", "/exit"):
        assert command in cli.HELP


def fake_engine(monkeypatch):
    config = parse_config(TINY_A)

    def make(model_dir, **kw):
        kw = {k: v for k, v in kw.items() if k in ("block_size", "max_tokens_per_step", "max_running", "seed")}
        return LLMEngine(None, num_blocks=32, dtype="float32", device="cpu", config=config,
                         tensors=dict(random_tensors(config, 0)), ops=EmulatedOps(), **kw)

    import shrike_b200.engine.llm_engine as module

    monkeypatch.setattr(module, "LLMEngine", make)


def test_repl_on_a_pipe(monkeypatch, capsys):
    fake_engine(monkeypatch)
    lines = "/help\n/temp 0\n/max 5\n/budget 7\n5 17 3 9\n/metrics\n/bench 3 4\n/temp x\n/nonsense\nhello\n/reset\n/exit\n"
    monkeypatch.setattr(sys, "stdin", io.StringIO(lines))
    cli.main(["--model", "unused"])
    out = capsys.readouterr().out
    assert "shrike_b200 ready" in out and "KV blocks" in out
    assert "Temperature set to 0." in out and "Maximum new tokens set to 5." in out
    assert "Scheduler token budget set to 7 per step." in out
    assert "5 tok" in out and "TTFT" in out                  # the reply's status line
    assert "tokens_generated" in out and "kv_blocks_free" in out
    assert "3 reqs x 4 tok -> 12 tok" in out
    assert "Usage: /temp" in out and "Unknown command: /nonsense" in out
    assert "enter token ids" in out and "Metrics counters reset." in out


def test_end_of_input_quits(monkeypatch, capsys):
    fake_engine(monkeypatch)
    monkeypatch.setattr(sys, "stdin", io.StringIO(""))
    cli.main(["--model", "unused"])
    assert "ready" in capsys.readouterr().out
