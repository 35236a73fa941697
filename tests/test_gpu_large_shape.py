"""The serving shapes: Qwen2.5-7B widths (hidden 3584, 28 / 4 heads of 128, intermediate
18944, vocabulary 152064) with two layers, and Qwen2.5-14B widths (hidden 5120, 40 / 8 heads,
intermediate 13824; rows wider than 4,096 take another form of the norm kernel and the
products other K cuts) with one layer and a short vocabulary, random weights made on the GPU.  A plain
float64 pass of this size is out of reach on the CPU, so the checks are the engine against
itself: float32 logits must not change with the cutting (they are bitwise equal), bfloat16
must agree with float32 within the bfloat16 tolerance, and the tensor-core product for few
tokens must agree with the library product for many."""

import numpy as np
import pytest
import torch

from shrike_b200.config import parse_config
from shrike_b200.engine.batch import StepEntry
from shrike_b200.engine.runner import ModelRunner
from shrike_b200.weights.random_init import random_tensors
from tests.gpu_common import cuda_ops
from tests.helpers import random_tokens

pytestmark = pytest.mark.gpu

SHAPES = {
    "7b": dict(
        architectures=["Qwen2ForCausalLM"], hidden_size=3584, intermediate_size=18944, num_hidden_layers=2,
        num_attention_heads=28, num_key_value_heads=4, head_dim=128, vocab_size=152064, rms_norm_eps=1e-6,
        rope_theta=1000000.0, tie_word_embeddings=False, max_position_embeddings=32768, eos_token_id=151643,
    ),
    "14b": dict(
        architectures=["Qwen2ForCausalLM"], hidden_size=5120, intermediate_size=13824, num_hidden_layers=1,
        num_attention_heads=40, num_key_value_heads=8, head_dim=128, vocab_size=5003, rms_norm_eps=1e-5,
        rope_theta=1000000.0, tie_word_embeddings=True, max_position_embeddings=32768, eos_token_id=5002,
    ),
}
LENGTH = 150


def run(runner, tokens, cuts):
    cache, pos, rows = runner.cache.open(), 0, []
    for n in cuts:
        runner.cache.append(cache, pos, n)
        rows.append(runner.step([StepEntry(cache, tokens[pos:pos + n], pos, list(range(n)))]).cpu().numpy().copy())
        pos += n
    assert pos == len(tokens)
    runner.cache.free(cache)
    assert runner.cache.whole()
    return np.concatenate(rows)


@pytest.fixture(scope="module", params=list(SHAPES))
def logits(request):
    shape = SHAPES[request.param]
    config = parse_config(shape)
    tokens = random_tokens(shape["vocab_size"], LENGTH, 11)
    out = {}
    for dtype, torch_dtype in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
        tensors = random_tensors(config, 5, "cuda", torch.float32)
        tensors = {k: (v.to(torch_dtype) if v.dim() >= 2 else v) for k, v in tensors.items()}
        runner = ModelRunner(config, tensors, cuda_ops(torch_dtype), "cuda", dtype, page_size=16, num_pages=16, max_slots=2)
        del tensors
        out[dtype, "whole"] = run(runner, tokens, [LENGTH])
        out[dtype, "portions"] = run(runner, tokens, [70, 2, 33, 17, 16, 12])
        out[dtype, "tail"] = run(runner, tokens, [LENGTH - 20] + [1] * 20)
        if dtype == "bfloat16":
            runner.ops.check_status()
        del runner
        torch.cuda.empty_cache()
    return out


def test_float32_logits_do_not_depend_on_the_cutting(logits):
    assert np.array_equal(logits["float32", "whole"], logits["float32", "portions"])
    assert np.array_equal(logits["float32", "whole"], logits["float32", "tail"])
    assert np.isfinite(logits["float32", "whole"]).all()


def test_bfloat16_agrees_with_float32_and_with_itself(logits):
    exact = logits["float32", "whole"].astype(np.float64)
    scale = np.abs(exact).max()
    for way in ("whole", "portions", "tail"):
        diff = np.abs(logits["bfloat16", way] - exact).max()
        assert diff <= 2e-2 * max(1.0, scale), f"bfloat16 {way}: {diff:.3e} against a logit scale of {scale:.2f}"
    # portions of at most 64 tokens run on the tensor-core product of this package, the whole
    # prompt on the library's: both must tell the same story, to rounding
    between = np.abs(logits["bfloat16", "whole"] - logits["bfloat16", "portions"]).max()
    assert between <= 2e-2 * max(1.0, scale)
    greedy32 = logits["float32", "whole"].argmax(-1)
    top2 = np.sort(logits["float32", "whole"], axis=-1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > 4e-2 * max(1.0, scale)
    assert (logits["bfloat16", "tail"].argmax(-1)[clear] == greedy32[clear]).all()
