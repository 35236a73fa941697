"""The plain implementation: against Azimml/shrike's own model code (stored golden
logits), and its own properties."""

import hashlib
from pathlib import Path

import numpy as np
import pytest
import torch

from tests.helpers import make_model_folder, plain_logits, random_tokens, read_weights
from tests.plain import plain_model as pm
from tests.tiny_configs import TINY

GOLDEN = Path(__file__).parent / "golden" / "reference_logits.npz"


def _checksum(weights):
    h = hashlib.sha256()
    for name in sorted(weights):
        h.update(name.encode())
        h.update(weights[name].contiguous().numpy().tobytes())
    return h.hexdigest()


@pytest.mark.parametrize("key,lengths", [("A", [5, 17, 33]), ("B", [1, 9, 40, 70])])
def test_plain_matches_reference_logits(tmp_path, key, lengths):
    golden = np.load(GOLDEN)
    weights = read_weights(make_model_folder(tmp_path, key))
    stored = bytes(golden[f"{key}_checksum"]).decode()
    assert _checksum(weights) == stored, (
        "the random-weights writer no longer reproduces the weights the golden logits were made "
        "from; rerun tests/golden/make_golden.py"
    )
    for index, n in enumerate(lengths):
        ids = random_tokens(TINY[key]["vocab_size"], n, 1000 + index)
        got = plain_logits(key, weights, ids)
        np.testing.assert_allclose(got, golden[f"{key}_{n}"], atol=2e-6, rtol=0)


def test_plain_is_causal(tmp_path):
    weights = read_weights(make_model_folder(tmp_path, "A"))
    ids = random_tokens(256, 40, 7)
    full = plain_logits("A", weights, ids)
    part = plain_logits("A", weights, ids[:23])
    np.testing.assert_allclose(full[:23], part, atol=1e-12)


def test_plain_window_limits_what_a_query_sees():
    torch.manual_seed(0)
    q, k, v = torch.randn(9, 2, 16).double(), torch.randn(9, 1, 16).double(), torch.randn(9, 1, 16).double()
    windowed = pm.causal_attention(q, k, v, window=3)
    last = pm.causal_attention(q[6:9], k[6:9], v[6:9])  # the last query with exactly its 3 keys
    np.testing.assert_allclose(windowed[8].numpy(), last[2].numpy(), atol=1e-12)
    everything = pm.causal_attention(q, k, v, window=None)
    np.testing.assert_allclose(pm.causal_attention(q, k, v, window=100).numpy(), everything.numpy(), atol=0)


def test_plain_order_shares_weights_and_caches(tmp_path):
    weights = read_weights(make_model_folder(tmp_path, "A"))
    ids = random_tokens(256, 12, 3)
    usual = pm.forward(TINY["A"], weights, ids)
    listed = pm.forward(TINY["A"], weights, ids, order=[(0, None), (1, None)])
    assert torch.equal(usual, listed)
    twice = pm.forward(TINY["A"], weights, ids, order=[(0, None), (1, None), (1, None)])
    shared = pm.forward(TINY["A"], weights, ids, order=[(0, None), (1, None), (1, 1)])
    assert not torch.allclose(usual, twice) and not torch.allclose(twice, shared)


def test_plain_rounding_emulation_changes_little(tmp_path):
    weights = read_weights(make_model_folder(tmp_path, "B"))
    ids = random_tokens(384, 30, 3)
    exact = plain_logits("B", weights, ids)
    rounded = plain_logits("B", weights, ids, bf16=True)
    diff = np.abs(exact - rounded).max()
    assert 1e-5 < diff < 5e-2


def test_top_p_keep_follows_the_reference_rule():
    probs = torch.tensor([0.05, 0.5, 0.15, 0.3])
    assert pm.top_p_keep(probs, 0.5).tolist() == [False, True, False, False]
    assert pm.top_p_keep(probs, 0.51).tolist() == [False, True, False, True]
    assert pm.top_p_keep(probs, 1.0).tolist() == [True, True, True, True]
    assert pm.top_p_keep(probs, 1e-9).tolist() == [False, True, False, False]
