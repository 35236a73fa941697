"""The serving shapes: Qwen2.5-7B widths (hidden 3584, 28 / 4 heads of 128, intermediate
18944, vocabulary 152064) with two layers, and Qwen2.5-14B widths (hidden 5120, 40 / 8 heads,
intermediate 13824; rows wider than 4,096 take another form of the norm kernel and the
products other K cuts) with one layer and a short vocabulary, random weights made on the GPU.

The oracle is the plain implementation (tests/plain/plain_model.py), run in float64 on the GPU:
it is plain torch, and on the CPU a pass at these widths would take minutes.  Compared with it:
one 150-token prompt whole, in portions and with its tail decoded token by token, in float32
(where the logits must moreover be bitwise the same under every cutting) and in bfloat16
(against the oracle with bfloat16 rounding at the engine's rounding points); and decode steps
of 72, 65 and 64 rows, around the batch size at which bfloat16 products change from this
package's tensor-core kernel to the library's."""

import numpy as np
import pytest
import torch

from shrike_b200.config import parse_config
from shrike_b200.engine.batch import StepEntry
from shrike_b200.engine.runner import ModelRunner
from shrike_b200.weights.random_init import random_tensors
from tests.gpu_common import cuda_ops
from tests.helpers import random_tokens
from tests.plain import plain_model as pm

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
# relative to the largest logit: float32 against float64, and bfloat16 against the like-rounded
# float64 oracle (the tiny models' absolute 2e-5 and 2e-2, on logits of order one there)
REL_TOL = {"float32": 1e-4, "bfloat16": 2e-2}
DTYPES = (("float32", torch.float32), ("bfloat16", torch.bfloat16))


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


def oracle(shape, master, tokens, bf16):
    """Float64 logits of the plain implementation on the GPU; `master` holds float32 weights."""
    weights = {k: (v.to(torch.bfloat16) if bf16 and v.dim() >= 2 else v) for k, v in master.items()}
    out = pm.forward(shape, weights, tokens, dtype=torch.float64, rounding=pm.ROUNDING_POINTS if bf16 else ())
    return out.cpu().numpy()


def engine_weights(master, torch_dtype):
    return {k: (v.to(torch_dtype) if v.dim() >= 2 else v.clone()) for k, v in master.items()}


@pytest.fixture(scope="module", params=list(SHAPES))
def served(request):
    shape = SHAPES[request.param]
    config = parse_config(shape)
    master = random_tensors(config, 5, "cuda", torch.float32)
    yield request.param, shape, config, master
    del master
    torch.cuda.empty_cache()


@pytest.fixture(scope="module")
def logits(served):
    name, shape, config, master = served
    tokens = random_tokens(shape["vocab_size"], LENGTH, 11)
    out = {}
    for dtype, torch_dtype in DTYPES:
        runner = ModelRunner(config, engine_weights(master, torch_dtype), cuda_ops(torch_dtype), "cuda", dtype,
                             page_size=16, num_pages=16, max_slots=2)
        out[dtype, "whole"] = run(runner, tokens, [LENGTH])
        out[dtype, "portions"] = run(runner, tokens, [70, 2, 33, 17, 16, 12])
        out[dtype, "tail"] = run(runner, tokens, [LENGTH - 20] + [1] * 20)
        if dtype == "bfloat16":
            runner.ops.check_status()
        del runner
        torch.cuda.empty_cache()
        out[dtype, "plain"] = oracle(shape, master, tokens, dtype == "bfloat16")
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("way", ["whole", "portions", "tail"])
def test_logits_match_the_plain_implementation(logits, dtype, way):
    want = logits[dtype, "plain"]
    scale = max(1.0, float(np.abs(want).max()))
    got = logits[dtype, way]
    assert np.isfinite(got).all()
    diff = np.abs(got - want)
    worst = np.unravel_index(int(diff.argmax()), diff.shape)
    assert diff.max() <= REL_TOL[dtype] * scale, (
        f"{dtype} {way}: |diff| {diff.max():.3e} at token {worst[0]}, logit {worst[1]}; logits reach {scale:.2f}")


def test_float32_logits_do_not_depend_on_the_cutting(logits):
    assert np.array_equal(logits["float32", "whole"], logits["float32", "portions"])
    assert np.array_equal(logits["float32", "whole"], logits["float32", "tail"])


def test_bfloat16_keeps_the_clear_argmaxes_of_the_plain_float64_run(logits):
    exact = logits["float32", "plain"]
    scale = max(1.0, float(np.abs(exact).max()))
    top2 = np.sort(exact, axis=-1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > 4e-2 * scale
    assert clear.sum() >= LENGTH // 4
    for way in ("whole", "portions", "tail"):
        assert (logits["bfloat16", way].argmax(-1)[clear] == exact.argmax(-1)[clear]).all(), way


@pytest.mark.parametrize("dtype,torch_dtype", DTYPES)
def test_decode_steps_of_more_than_64_rows_match_the_plain_implementation(served, dtype, torch_dtype):
    """72 short sequences are fed whole (a few at a time), then decode together: 72 rows, then
    65 after seven have ended, then 64.  Every row of every step against the float64 oracle of
    its own sequence."""
    name, shape, config, master = served
    vocab = shape["vocab_size"]
    lengths = [3 + (7 * i) % 19 for i in range(72)]
    sequences = [random_tokens(vocab, n + 3, 1000 + i) for i, n in enumerate(lengths)]   # prompt + 3 decoded
    runner = ModelRunner(config, engine_weights(master, torch_dtype), cuda_ops(torch_dtype), "cuda", dtype,
                         page_size=16, num_pages=160, max_slots=80)
    caches = [runner.cache.open() for _ in sequences]
    for lo in range(0, 72, 9):   # the prompts, nine sequences a step
        entries = []
        for i in range(lo, lo + 9):
            runner.cache.append(caches[i], 0, lengths[i])
            entries.append(StepEntry(caches[i], sequences[i][:lengths[i]], 0, []))
        runner.step(entries)
    got = {}
    live = list(range(72))
    for step, keep in enumerate((72, 65, 64)):
        live = live[:keep]
        entries = []
        for i in live:
            position = lengths[i] + step
            runner.cache.append(caches[i], position, 1)
            entries.append(StepEntry(caches[i], [sequences[i][position]], position, [0]))
        rows = runner.step(entries).cpu().numpy()
        assert rows.shape == (keep, vocab)
        for row, i in zip(rows, live):
            got[i, step] = row.copy()
    if dtype == "bfloat16":
        assert runner.ops.library_calls > 0, "the 72-row steps were meant to use the library product"
        runner.ops.check_status()
    for cache in caches:
        runner.cache.free(cache)
    assert runner.cache.whole()
    del runner
    torch.cuda.empty_cache()
    worst = 0.0
    for i in range(72):
        want = oracle(shape, master, sequences[i], dtype == "bfloat16")
        scale = max(1.0, float(np.abs(want).max()))
        for step in range(3):
            if (i, step) in got:
                diff = float(np.abs(got[i, step] - want[lengths[i] + step]).max())
                assert diff <= REL_TOL[dtype] * scale, f"{dtype}: sequence {i}, decode step {step}: |diff| {diff:.3e}"
                worst = max(worst, diff / scale)
    assert worst > 0.0 or dtype == "float32"
