"""The replay session's host side, on the CPU through the stand-in kernels: the pool options
(page size, explicit page count, live requests), page reuse under a pool that is exactly as
large as the trace needs, and what happens when nothing is given back."""

import io
import json
import sys

import numpy as np
import pytest

import shrike_b200.models  # noqa: F401
from shrike_b200 import replay as replay_module
from shrike_b200.replay import TraceSession, pages_for
from tests.emulated_ops import EmulatedOps
from tests.helpers import collect, make_model_folder, mixed_trace, plain_logits, random_tokens, read_weights
from tests.tiny_configs import TINY

LENGTHS = [5, 17, 33, 70, 1, 40, 2, 64]


def pages_needed(steps, page):
    held, worst = {}, 0
    for record in steps:
        for entry in record["entries"]:
            held[entry["id"]] = held.get(entry["id"], 0) + len(entry["tokens"])
        worst = max(worst, sum(-(-n // page) for n in held.values()))
        for ident in record["end"]:
            held.pop(ident, None)
    return worst


def run(folder, steps, **options):
    session = TraceSession(folder, "float32", device="cpu", ops=EmulatedOps(), **options)
    outputs = {}
    for record in steps:
        result = session.step(record)
        if result is not None:
            outputs[record["step"]] = result.copy()
    return collect(steps, outputs), session


def test_pages_for_rounds_as_the_option_says():
    assert pages_for(256, 16, 4) == 16 and pages_for(256, 8, 4) == 32 and pages_for(256, 64, 4) == 4
    assert pages_for(256, 24, 4) == 11 + 4        # 24 does not divide 64: one more page per live request
    assert pages_for(1, 16, 4) == 1


@pytest.mark.parametrize("key,page", [("B", 8), ("A", 16), ("B", 32)])
def test_mixed_replay_on_a_tight_pool_reuses_pages(tmp_path, key, page):
    folder = make_model_folder(tmp_path, key)
    weights = read_weights(folder)
    requests = {f"r{i}": random_tokens(TINY[key]["vocab_size"], n, 100 + i) for i, n in enumerate(LENGTHS)}
    steps = mixed_trace(requests, seed=5)
    num_pages = pages_needed(steps, page)
    assert num_pages < sum(-(-len(t) // page) for t in requests.values())
    got, session = run(folder, steps, page_size=page, num_pages=num_pages, max_live=4)
    assert session.runner.cache.num_pages == [num_pages] and session.runner.cache.whole()
    shared = {ident: owners for ident, owners in session.page_owners.items() if len(owners) > 1}
    assert shared, "no page was held by more than one request"
    assert len({owner for owners in shared.values() for owner in owners}) >= 4
    for ident, tokens in requests.items():
        np.testing.assert_allclose(got[ident], plain_logits(key, weights, tokens), atol=2e-5)


def test_running_out_of_pages_and_of_live_requests_is_said(tmp_path):
    folder = make_model_folder(tmp_path, "A")
    requests = {f"r{i}": random_tokens(256, 20, i) for i in range(3)}
    steps = [{"step": i, "entries": [{"id": ident, "tokens": tokens, "want": []}], "end": []}
             for i, (ident, tokens) in enumerate(requests.items())]
    with pytest.raises(RuntimeError, match="no pages left"):
        run(folder, steps, page_size=16, num_pages=5, max_live=4)
    with pytest.raises(RuntimeError, match="raise --max-live"):
        run(folder, steps, page_size=16, num_pages=16, max_live=2)


def test_header_line_fills_what_the_command_line_left_unset(tmp_path, monkeypatch, capsys):
    folder = make_model_folder(tmp_path, "A")
    seen = {}

    class Recorder(TraceSession):
        def __init__(self, model_dir, dtype, max_tokens=None, **options):
            seen.update(options, max_tokens=max_tokens)
            super().__init__(model_dir, dtype, max_tokens, device="cpu", ops=EmulatedOps(), **options)

    monkeypatch.setattr(replay_module, "TraceSession", Recorder)
    monkeypatch.setattr(replay_module.torch.cuda, "synchronize", lambda: None)
    tokens = random_tokens(256, 11, 3)
    lines = [json.dumps({"header": {"block_size": 8, "num_blocks": 5, "max_live": 2}}),
             json.dumps({"step": 0, "entries": [{"id": "a", "tokens": tokens, "want": [10]}], "end": ["a"]})]
    monkeypatch.setattr(sys, "stdin", io.StringIO("\n".join(lines) + "\n"))
    out = tmp_path / "out"
    assert replay_module.main(["--model", str(folder), "--dtype", "float32", "--out", str(out), "--max-live", "3"]) == 0
    assert seen == dict(page_size=8, num_pages=5, max_live=3, max_tokens=None)
    assert capsys.readouterr().out.split() == ["done", "0"]
    logits = np.fromfile(out / "0.f32", dtype="<f4")
    np.testing.assert_allclose(logits, plain_logits("A", read_weights(folder), tokens)[10], atol=2e-5)
