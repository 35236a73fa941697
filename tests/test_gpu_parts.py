"""Each part alone on the GPU against its plain formula: norm, attention with
rotary encoding over a paged cache, feed-forward, and the block that arranges them;
plus a model whose run order names a layer twice and shares a cache."""

import numpy as np
import pytest
import torch

import shrike_b200.models  # noqa: F401
from shrike_b200.config import LayerRun, parse_config
from shrike_b200.config.model_config import AttentionSpec, GatedMLPSpec, RMSNormSpec, RotarySpec
from shrike_b200.engine.batch import StepEntry
from shrike_b200.engine.model import Runtime
from shrike_b200.engine.runner import ModelRunner
from shrike_b200.parts import part_class
from shrike_b200.weights import random_tensors
from tests.gpu_common import TOL, assert_close, cuda_ops
from tests.helpers import random_tokens
from tests.plain import plain_model as pm
from tests.tiny_configs import TINY

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_part(dtype):
    spec = RMSNormSpec(width=200, eps=1e-5)
    ops, rt = cuda_ops(DTYPES[dtype]), Runtime(DEV, DTYPES[dtype])
    weight = 1 + 0.1 * rnd(200, seed=1)
    part = part_class("norm", spec.kind)(spec, {"weight": weight.to(DEV)}, ops, rt)
    resid, delta = rnd(5, 200, seed=2).to(DEV), rnd(5, 200, seed=3).to(DEV)
    want = pm.rms_norm((resid + delta).double().cpu(), weight.double(), 1e-5)
    got = part.add_norm(resid, delta)
    assert got.dtype == DTYPES[dtype]
    assert_close(got.float().cpu().numpy(), want.numpy(), 1e-5 if dtype == "float32" else 3e-2, "norm part")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_feed_forward_part(dtype):
    spec = GatedMLPSpec(width=80, intermediate=176, activation="silu")
    ops, rt = cuda_ops(DTYPES[dtype]), Runtime(DEV, DTYPES[dtype])
    tensors = {"gate_proj.weight": rnd(176, 80, seed=1, scale=0.1), "up_proj.weight": rnd(176, 80, seed=2, scale=0.1),
               "down_proj.weight": rnd(80, 176, seed=3, scale=0.1)}
    if dtype == "bfloat16":
        tensors = {k: v.bfloat16() for k, v in tensors.items()}
    part = part_class("feed_forward", spec.kind)(spec, {k: v.to(DEV) for k, v in tensors.items()}, ops, rt)
    x = rnd(9, 80, seed=4).to(DTYPES[dtype])
    w = {f"p.{k}": v.double() for k, v in tensors.items()}
    rounding = pm.Rounder(pm.ROUNDING_POINTS if dtype == "bfloat16" else ())
    want = pm.mlp(x.double(), w, "p", rounding)
    got = part.forward(x.to(DEV), None)
    assert got.dtype == torch.float32
    assert_close(got.cpu().numpy(), want.numpy(), 1e-5 if dtype == "float32" else 1e-2, "feed-forward part")
    with pytest.raises(ValueError, match="activation"):
        part_class("feed_forward", "gated_mlp")(GatedMLPSpec(80, 176, "gelu"), {}, ops, rt)


def test_order_names_a_layer_twice_and_shares_a_cache():
    """Run order [0, 1, 1 again on a cache of its own, 1 reading run 1's cache]."""
    raw = TINY["A"]
    config = parse_config(raw)
    weights = random_tensors(config, 0)
    config.order = [LayerRun(0, 0), LayerRun(1, 1), LayerRun(1, 2), LayerRun(1, 1, writes_cache=False)]
    config.validate()
    ids = random_tokens(256, 45, 8)
    want = pm.forward(raw, weights, ids, order=[(0, None), (1, None), (1, None), (1, 1)]).numpy()
    ops = cuda_ops(torch.float32)
    runner = ModelRunner(config, {k: v.to(DEV) for k, v in weights.items()}, ops, DEV, "float32", page_size=16, num_pages=4, max_slots=2)
    assert len(runner.groups) == 1 and runner.groups[0].cache_ids == (0, 1, 2)
    cache, pos, rows = runner.cache.open(), 0, []
    for n in (20, 1, 1, 2, 21):
        runner.cache.append(cache, pos, n)
        rows.append(runner.step([StepEntry(cache, ids[pos:pos + n], pos, list(range(n)))]).cpu().numpy().copy())
        pos += n
    assert_close(np.concatenate(rows), want, TOL["float32"], "shared layers and caches")
