"""The programs under bin/ as a user runs them on the GPU: the interactive command line on a
pipe with a real model folder (shrike CLI_SPEC.md, "Acceptance"), started from a shape without
a folder, and the one-prompt program.  Replies are checked against the plain implementation."""

import os
import subprocess
import sys
from pathlib import Path

import pytest

from tests.helpers import make_model_folder, read_weights
from tests.plain import plain_model as pm
from tests.tiny_configs import TINY

pytestmark = pytest.mark.gpu
BIN = Path(__file__).resolve().parents[1] / "bin"


def run(program, arguments, text=""):
    done = subprocess.run([sys.executable, str(BIN / program), *arguments], input=text, capture_output=True,
                          text=True, timeout=900, env=dict(os.environ, PYTHONUNBUFFERED="1"))
    assert done.returncode == 0, done.stderr[-3000:]
    return done


def test_command_line_on_a_pipe_with_a_model_folder(tmp_path):
    folder = make_model_folder(tmp_path, "A")
    prompt = [5, 17, 3, 9]
    want, margins = pm.greedy_continue(TINY["A"], read_weights(folder), prompt, 6)
    assert min(margins) > 1e-4
    done = run("shrike_b200", ["--model", str(folder), "--num-blocks", "16", "--dtype", "float32"],
               "/temp 0\n/max 6\n5 17 3 9\n/metrics\n/exit\n")
    out = done.stdout
    assert "shrike_b200 ready" in out and "16 KV blocks" in out
    assert " ".join(map(str, want)) in out, out
    assert "[6 tok |" in out
    assert "tokens_generated    6" in out and "kv_blocks_free      16" in out


def test_command_line_from_a_shape_without_a_folder():
    done = run("shrike_b200", ["--random", "tiny", "--seed", "1", "--num-blocks", "32"],
               "/temp 0\n/max 4\n1 2 3\n/bench 5 8\n/exit\n")
    assert "random weights, shape tiny" in done.stdout and "[4 tok |" in done.stdout
    assert "5 requests x 8 tokens: 40 tokens in" in done.stdout


def test_one_prompt_program_streams_the_greedy_continuation(tmp_path):
    folder = make_model_folder(tmp_path, "B")
    prompt = [7, 300, 41, 41, 2]
    want, margins = pm.greedy_continue(TINY["B"], read_weights(folder), prompt, 8)
    assert min(margins) > 1e-4
    done = run("shrike_b200_complete", [" ".join(map(str, prompt)), "--model", str(folder), "--max-tokens", "8",
                                         "--dtype", "float32", "--num-blocks", "8", "--block-size", "8"])
    assert [int(t) for t in done.stdout.split()] == want
    assert "8 tokens in" in done.stderr and "8 KV blocks" in done.stderr
