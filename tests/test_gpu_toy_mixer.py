"""A toy mixer with state of its own, defined here, is registered, built and stepped
through the engine without a change to the package: a running mean over the
sequence, kept per request in a state slot, mixed with attention layers."""

from dataclasses import dataclass, field

import numpy as np
import pytest
import torch

from shrike_b200.config import Architecture, LayerRun, LayerSpec, ModelConfig, TensorNames, parse_config, register_architecture
from shrike_b200.config.model_config import PartSpec
from shrike_b200.engine.batch import StepEntry
from shrike_b200.engine.runner import ModelRunner
from shrike_b200.models.qwen2 import parse_qwen2
from shrike_b200.parts import ParamSpec, StateNeed, register_part
from shrike_b200.weights import random_tensors
from tests.gpu_common import TOL, assert_close, cuda_ops
from tests.helpers import random_tokens
from tests.plain import plain_model as pm
from tests.tiny_configs import TINY_A

pytestmark = pytest.mark.gpu
DEV = "cuda"


@dataclass(frozen=True)
class RunningMeanSpec(PartSpec):
    width: int
    kind: str = field(init=False, default="running_mean")


class RunningMean:
    """out[t] = proj(mean of x[0..t]).  The sum so far is the request's state."""

    @staticmethod
    def parameters(spec):
        return {"proj.weight": ParamSpec((spec.width, spec.width), "matrix")}

    @staticmethod
    def cache_needs(spec):
        return [StateNeed((spec.width,), "float32")]

    def __init__(self, spec, tensors, ops, runtime):
        self.spec, self.ops, self.runtime = spec, ops, runtime
        self.proj = tensors["proj.weight"].contiguous()

    def forward(self, x, ctx, run):
        state = ctx.storage.state[run.cache]
        mean = torch.empty(x.shape, dtype=torch.float32, device=x.device)
        cursor = 0
        for q_len, start, slot in zip(ctx.q_lens, ctx.starts, ctx.slots):
            if start == 0:
                state[slot].zero_()
            sums = torch.cumsum(x[cursor: cursor + q_len].float(), 0) + state[slot]
            state[slot].copy_(sums[-1])
            counts = torch.arange(start + 1, start + q_len + 1, device=x.device, dtype=torch.float32)
            mean[cursor: cursor + q_len] = sums / counts[:, None]
            cursor += q_len
        delta = self.runtime.buffer("mixer_delta", (x.shape[0], self.spec.width), torch.float32)
        self.ops.linear(mean.to(self.runtime.act_dtype), self.proj, delta)
        return delta


def parse_toy(raw):
    base = parse_qwen2(dict(raw, architectures=["Qwen2ForCausalLM"]))
    layers = list(base.layers)
    toy = RunningMeanSpec(width=base.hidden_size)
    layers[1] = LayerSpec(mixer=toy, mixer_norm=layers[1].mixer_norm, feed_forward=layers[1].feed_forward,
                          feed_forward_norm=layers[1].feed_forward_norm)
    base.architecture = "ToyStateForCausalLM"
    base.layers = layers
    base.order = [LayerRun(0, 0), LayerRun(1, 1), LayerRun(2, 2)]
    return base


def toy_names(config):
    prefix = {"mixer": "mix.", "mixer_norm": "ln1.", "feed_forward": "mlp.", "feed_forward_norm": "ln2."}
    return TensorNames("emb.weight", "ln_f.", "head.weight", lambda layer, role: f"h.{layer}.{prefix[role]}")


def plain_toy(raw, w, ids):
    """Whole-sequence oracle built from the plain implementation's parts."""
    sizes = pm.config_sizes(raw)
    rnd = pm.Rounder(())
    w = {k: v.double() for k, v in w.items()}
    n = len(ids)
    cos, sin = pm.rope_tables(torch.arange(n), sizes["head_dim"], sizes["theta"], torch.float64)
    x = w["emb.weight"][torch.tensor(ids)]
    for layer in range(3):
        p = f"h.{layer}"
        a = pm.rms_norm(x, w[f"{p}.ln1.weight"], sizes["eps"])
        if layer == 1:
            mean = torch.cumsum(a, 0) / torch.arange(1, n + 1)[:, None]
            x = x + mean @ w[f"{p}.mix.proj.weight"].T
        else:
            q, k, v = pm.attention_inputs(a, w, f"{p}.mix", sizes, cos, sin, rnd)
            x = x + pm.causal_attention(q, k, v).reshape(n, -1) @ w[f"{p}.mix.o_proj.weight"].T
        m = pm.rms_norm(x, w[f"{p}.ln2.weight"], sizes["eps"])
        x = x + pm.mlp(m, w, f"{p}.mlp", rnd)
    return (pm.rms_norm(x, w["ln_f.weight"], sizes["eps"]) @ w["head.weight"].T).numpy()


def test_toy_mixer_with_state_is_registered_built_and_stepped():
    register_part("mixer", "running_mean", RunningMean)
    register_architecture(Architecture("ToyStateForCausalLM", parse_toy, toy_names))
    raw = dict(TINY_A, architectures=["ToyStateForCausalLM"], num_hidden_layers=3, tie_word_embeddings=False)
    config = parse_config(raw)
    weights = random_tensors(config, 4)
    assert "h.1.mix.proj.weight" in weights and "h.1.mix.q_proj.weight" not in weights
    runner = ModelRunner(config, {k: v.to(DEV) for k, v in weights.items()}, cuda_ops(torch.float32), DEV,
                         "float32", page_size=16, num_pages=12, max_slots=3)
    assert [g.cache_ids for g in runner.groups] == [(0, 2)] and list(runner.storage.state) == [1]
    requests = {name: random_tokens(256, n, seed) for name, n, seed in (("a", 37, 1), ("b", 20, 2), ("c", 9, 3))}
    want = {name: plain_toy(raw, weights, ids) for name, ids in requests.items()}
    caches = {name: runner.cache.open() for name in requests}
    fed = {name: 0 for name in requests}
    got = {name: [] for name in requests}
    plan = [{"a": 16, "b": 1}, {"a": 1, "b": 7, "c": 9}, {"a": 20, "b": 12}]
    for step in plan:
        names = sorted(step, key=lambda nm: step[nm] > 1)
        entries = []
        for name in names:
            n = step[name]
            runner.cache.append(caches[name], fed[name], n)
            entries.append(StepEntry(caches[name], requests[name][fed[name]: fed[name] + n], fed[name], list(range(n))))
        logits = runner.step(entries).cpu().numpy()
        cursor = 0
        for name in names:
            got[name].append(logits[cursor: cursor + step[name]].copy())
            cursor += step[name]
            fed[name] += step[name]
    for name in requests:
        assert_close(np.concatenate(got[name]), want[name], TOL["float32"], f"toy model request {name}")
    # a slot handed to a new request starts from zero again
    slot_of_c = caches["c"].slot
    runner.storage.state[1][slot_of_c].fill_(123.0)   # what a finished request may leave behind
    runner.cache.free(caches["c"])
    again = runner.cache.open()
    assert again.slot == slot_of_c
    runner.cache.append(again, 0, 9)
    redo = runner.step([StepEntry(again, requests["c"], 0, list(range(9)))]).cpu().numpy()
    assert_close(redo, want["c"], TOL["float32"], "state slot reused")
