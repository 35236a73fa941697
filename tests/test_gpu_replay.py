"""Replay on the GPU, every way of cutting, float32 and bfloat16, against the plain
implementation: whole; most in one step and the last 32 tokens one by one; portions
of changing size down to two tokens; mixed, up to four live requests with so few
pages that they are used again (and the pool poisoned with NaN beforehand); long
decoding; the first tokens of a sequence; and the program itself as a subprocess."""

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from tests.gpu_common import TOL, assert_close, replay
from tests.helpers import (
    make_model_folder, mixed_trace, max_live_tokens, plain_logits, portions_trace, random_tokens,
    read_weights, tail_decode_trace, whole_trace, write_trace,
)
from tests.tiny_configs import TINY

pytestmark = pytest.mark.gpu
LENGTHS = [5, 17, 33, 70, 1, 130, 2, 64]
LONG = {"D": [5, 300, 33, 70, 1, 130, 2, 64]}   # tiny D: one request long enough for several key steps of the tensor-core kernel
_cache = {}


def setup(tmp_path_factory, key, dtype):
    if key not in _cache:
        folder = make_model_folder(tmp_path_factory.mktemp(f"model_{key}"), key)
        weights = read_weights(folder)
        requests = {f"r{i}": random_tokens(TINY[key]["vocab_size"], n, 100 + i) for i, n in enumerate(LONG.get(key, LENGTHS))}
        _cache[key] = (folder, weights, requests, {})
    folder, weights, requests, refs = _cache[key]
    if dtype not in refs:
        refs[dtype] = {k: plain_logits(key, weights, t, bf16=(dtype == "bfloat16")) for k, t in requests.items()}
    return folder, requests, refs[dtype]


WAYS = {
    "whole": lambda reqs: whole_trace(reqs),
    "tail32": lambda reqs: tail_decode_trace(reqs, 32),
    "portions": lambda reqs: portions_trace(reqs, [7, 2, 5, 3, 2, 15, 16, 17, 2, 31, 33]),
    "mixed": lambda reqs: mixed_trace(reqs, seed=3),
    "mixed_other_order": lambda reqs: mixed_trace(dict(reversed(list(reqs.items()))), seed=11),
}


# every tiny configuration at the page size it is named with (A 16, B 8, C 16), and two more
# page sizes so that a page's edge falls elsewhere among the same portions: 32, and 24, which
# divides neither 64 nor the portion sizes
MODEL_PAGES = [("A", 16), ("B", 8), ("C", 16), ("B", 32), ("A", 8), ("C", 24), ("D", 16), ("D", 8)]


@pytest.mark.parametrize("way", list(WAYS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key,page", MODEL_PAGES)
def test_replay_matches_plain(tmp_path_factory, key, page, dtype, way):
    folder, requests, want = setup(tmp_path_factory, key, dtype)
    steps = WAYS[way](requests)
    got, session = replay(folder, dtype, steps, poison=way.startswith("mixed"), page_size=page, max_live=4)
    assert session.page_size == page and session.runner.storage.kv[0].shape[3] == page
    assert session.runner.cache.whole(), "pages or slots were not given back"
    for ident in requests:
        assert_close(got[ident], want[ident], TOL[dtype], f"{key} page {page} {dtype} {way} {ident}")


def pages_needed(steps, page):
    """The fewest pages a trace can run on: the most that live requests hold at once."""
    held, worst = {}, 0
    for record in steps:
        for entry in record["entries"]:
            held[entry["id"]] = held.get(entry["id"], 0) + len(entry["tokens"])
        worst = max(worst, sum(-(-n // page) for n in held.values()))
        for ident in record["end"]:
            held.pop(ident, None)
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key,page", [("B", 8), ("A", 16), ("B", 32)])
def test_mixed_replay_reuses_pages(tmp_path_factory, key, page, dtype):
    """The pool holds exactly as many pages as the trace needs at its fullest moment (given
    with --num-blocks), so later requests can only run on pages that earlier ones gave back:
    if `free` stopped returning pages, the replay would run out of them."""
    folder, requests, want = setup(tmp_path_factory, key, dtype)
    steps = mixed_trace(requests, seed=5)
    num_pages = pages_needed(steps, page)
    assert num_pages < sum(-(-len(t) // page) for t in requests.values()), "the trace never frees anything"
    got, session = replay(folder, dtype, steps, num_pages=num_pages, page_size=page, max_live=4, poison=True)
    assert session.runner.cache.num_pages == [num_pages]
    shared = {page_id: owners for page_id, owners in session.page_owners.items() if len(owners) > 1}
    assert shared, "no page was held by more than one request over the trace"
    assert len({owner for owners in shared.values() for owner in owners}) >= 4
    assert session.runner.cache.whole()
    for ident in requests:
        assert_close(got[ident], want[ident], TOL[dtype], f"reuse {key} page {page} {dtype} {ident}")


def test_replay_runs_out_of_pages_when_nothing_is_given_back(tmp_path_factory):
    """The same tight pool with the `end` lists dropped: the replay must say that pages ran out."""
    folder, requests, _ = setup(tmp_path_factory, "B", "float32")
    steps = [dict(record, end=[]) for record in mixed_trace(requests, seed=5)]
    num_pages = pages_needed(mixed_trace(requests, seed=5), 8)
    with pytest.raises(RuntimeError, match="no pages left|raise --max-live"):
        replay(folder, "float32", steps, num_pages=num_pages, page_size=8, max_live=8)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_token_by_token(tmp_path_factory, dtype):
    folder = make_model_folder(tmp_path_factory.mktemp("long"), "C")
    tokens = random_tokens(TINY["C"]["vocab_size"], 300, 9)
    want = plain_logits("C", read_weights(folder), tokens, bf16=(dtype == "bfloat16"))
    steps = [{"step": i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": ["x"] if i == 299 else []}
             for i, t in enumerate(tokens)]
    got, session = replay(folder, dtype, steps, page_size=16)
    assert_close(got["x"], want, TOL[dtype], f"long decode {dtype}")
    assert session.runner.cache.whole()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["A", "B"])
def test_first_tokens_of_a_sequence(tmp_path_factory, key, dtype):
    folder, requests, _ = setup(tmp_path_factory, key, dtype)
    tokens = random_tokens(TINY[key]["vocab_size"], 4, 77)
    want = plain_logits(key, read_weights(folder), tokens, bf16=(dtype == "bfloat16"))
    one_by_one = [{"step": i, "entries": [{"id": "f", "tokens": [t], "want": [0]}], "end": []} for i, t in enumerate(tokens)]
    got, _ = replay(folder, dtype, one_by_one, max_tokens=64)
    assert_close(got["f"], want, TOL[dtype], "first tokens one by one")
    two_two = [{"step": 0, "entries": [{"id": "f", "tokens": tokens[:2], "want": [0, 1]}], "end": []},
               {"step": 1, "entries": [{"id": "f", "tokens": tokens[2:], "want": [0, 1]}], "end": ["f"]}]
    got, _ = replay(folder, dtype, two_two, max_tokens=64)
    assert_close(got["f"], want, TOL[dtype], "first tokens two and two")


def test_wanting_nothing_writes_nothing_and_cutting_is_bitwise_stable_in_float32(tmp_path_factory):
    folder, requests, want = setup(tmp_path_factory, "B", "float32")
    whole, _ = replay(folder, "float32", whole_trace(requests))
    mixed, _ = replay(folder, "float32", mixed_trace(requests, seed=3))
    for ident in requests:
        assert np.array_equal(whole[ident], mixed[ident]), "float32 logits changed with the cutting"


def test_trace_run_program(tmp_path):
    """The program as a user runs it: stdin in, <step>.f32 files and `done` lines out."""
    folder = make_model_folder(tmp_path, "A")
    requests = {"a": random_tokens(256, 21, 1), "b": random_tokens(256, 9, 2)}
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": requests["a"][:14], "want": [0, 13]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": requests["a"][14:15], "want": []},
                                {"id": "b", "tokens": requests["b"], "want": [8]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": requests["a"][15:], "want": [5]}], "end": ["a"]},
    ]
    out = tmp_path / "out"
    program = Path(__file__).resolve().parents[1] / "bin" / "trace_run"
    run = subprocess.run(
        [sys.executable, str(program), "--model", str(folder), "--dtype", "float32", "--out", str(out), "--max-tokens", "128"],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600,
    )
    assert run.returncode == 0, run.stderr[-2000:]
    assert [line for line in run.stdout.splitlines() if line.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert sorted(p.name for p in out.iterdir()) == ["0.f32", "1.f32", "2.f32"]
    weights = read_weights(folder)
    ref_a, ref_b = plain_logits("A", weights, requests["a"]), plain_logits("A", weights, requests["b"])
    step0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, 256)
    step1 = np.fromfile(out / "1.f32", dtype="<f4").reshape(1, 256)
    step2 = np.fromfile(out / "2.f32", dtype="<f4").reshape(1, 256)
    assert_close(step0, ref_a[[0, 13]], TOL["float32"], "step 0")
    assert_close(step1, ref_b[[8]], TOL["float32"], "step 1")
    assert_close(step2, ref_a[[20]], TOL["float32"], "step 2")
