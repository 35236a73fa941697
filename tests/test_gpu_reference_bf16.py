"""The bfloat16 engine against what Azimml/shrike itself computes in bfloat16 on the GPU.

Everywhere else the bfloat16 oracle is the plain float64 implementation with rounding at the
engine's own rounding points.  Here the other side is the reference's model code, unmodified
(`QwenForCausalLM.load(dir, device="cuda")` run over whole prompts through its
`NaiveKVBackend`, shrike/models/qwen.py:195-249), on model folders written in bfloat16.  The
reference keeps its residual stream and its logits in bfloat16 and this engine keeps them in
float32, so this is a tolerance test, in the manner of the reference's own check against
another implementation (tests/test_parity.py:29-39,47-52): logits within the suite's bfloat16
tolerance, and the same argmax wherever the top-2 gap is clear of it.  Skipped where the
reference is not installed under baseline/_ref."""

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests.gpu_common import TOL, replay
from tests.helpers import make_model_folder, random_tokens, whole_trace
from tests.tiny_configs import TINY

pytestmark = pytest.mark.gpu
REF = Path(__file__).resolve().parents[1] / "baseline" / "_ref"


def reference_model():
    if not (REF / "shrike" / "models" / "qwen.py").is_file():
        pytest.skip("the reference is not installed under baseline/_ref")
    if str(REF) not in sys.path:
        sys.path.insert(0, str(REF))
    try:
        from shrike.models import qwen
    except Exception as error:  # noqa: BLE001
        pytest.skip(f"baseline/_ref does not import here: {type(error).__name__}: {error}")
    return qwen


@pytest.mark.parametrize("key,page", [("A", 16), ("B", 8)])
def test_engine_bfloat16_logits_match_the_reference_in_bfloat16(tmp_path, key, page):
    qwen = reference_model()
    folder = make_model_folder(tmp_path, key, "bfloat16")
    vocab = TINY[key]["vocab_size"]
    requests = {f"r{i}": random_tokens(vocab, n, 200 + i) for i, n in enumerate((5, 33, 70, 1, 130))}
    model = qwen.QwenForCausalLM.load(str(folder), device="cuda")
    assert next(model.parameters()).dtype == torch.bfloat16
    want = {}
    with torch.inference_mode():
        for ident, tokens in requests.items():
            ids = torch.tensor(tokens, device="cuda")
            out = model(ids, torch.arange(len(tokens), device="cuda"), qwen.NaiveKVBackend(model.cfg))
            want[ident] = out.float().cpu().numpy()
    got, session = replay(folder, "bfloat16", whole_trace(requests), page_size=page)
    assert session.runner.cache.whole()
    atol = TOL["bfloat16"]
    clear = agree = 0
    for ident in requests:
        assert got[ident].shape == want[ident].shape
        assert np.abs(want[ident]).max() > 10 * atol, "the logits are too small for this tolerance to mean anything"
        diff = np.abs(got[ident] - want[ident]).max()
        assert diff <= atol, f"tiny {key} {ident}: engine and reference differ by {diff:.3e} in bfloat16"
        top2 = np.sort(want[ident], axis=-1)[:, -2:]
        rows = (top2[:, 1] - top2[:, 0]) > 2 * atol
        clear += int(rows.sum())
        agree += int((got[ident].argmax(-1)[rows] == want[ident].argmax(-1)[rows]).sum())
    assert clear >= 20 and agree == clear
