"""A toy feed-forward with routing, defined here, is registered, built and stepped through
the engine without a change to the package: a float32 router picks one of three small gated
experts per token (top-1, weighted by its softmax probability).  One layer of the model uses
it, the others keep the dense feed-forward: parts are chosen layer by layer.  This is a toy,
not any published architecture."""

from dataclasses import dataclass, field

import numpy as np
import pytest
import torch

from shrike_b200.config import Architecture, LayerRun, LayerSpec, TensorNames, parse_config, register_architecture
from shrike_b200.config.model_config import PartSpec
from shrike_b200.engine.batch import StepEntry
from shrike_b200.engine.runner import ModelRunner
from shrike_b200.models.qwen2 import parse_qwen2
from shrike_b200.parts import ParamSpec, register_part
from shrike_b200.weights import random_tensors
from tests.gpu_common import TOL, assert_close, cuda_ops
from tests.helpers import random_tokens
from tests.plain import plain_model as pm
from tests.tiny_configs import TINY_A

pytestmark = pytest.mark.gpu
DEV = "cuda"
EXPERTS, EXPERT_WIDTH = 3, 48


@dataclass(frozen=True)
class RoutedSpec(PartSpec):
    width: int
    experts: int
    expert_width: int
    kind: str = field(init=False, default="toy_routed")


class RoutedFeedForward:
    """delta[t] = p[t, e] * down_e(silu(gate_e(x[t])) * up_e(x[t])) with e = argmax_e router(x[t]),
    p = softmax(router logits) in float32.  Tokens are gathered per expert and run through the
    package's own product and activation kernels."""

    @staticmethod
    def parameters(spec):
        names = {"router.weight": ParamSpec((spec.experts, spec.width), "matrix")}
        for e in range(spec.experts):
            names[f"experts.{e}.gate.weight"] = ParamSpec((spec.expert_width, spec.width), "matrix")
            names[f"experts.{e}.up.weight"] = ParamSpec((spec.expert_width, spec.width), "matrix")
            names[f"experts.{e}.down.weight"] = ParamSpec((spec.width, spec.expert_width), "matrix")
        return names

    def __init__(self, spec, tensors, ops, runtime):
        self.spec, self.ops, self.runtime = spec, ops, runtime
        self.router = tensors["router.weight"].float().contiguous()     # router logits are formed in 32-bit
        self.gate_up = [torch.cat([tensors[f"experts.{e}.gate.weight"], tensors[f"experts.{e}.up.weight"]]).contiguous()
                        for e in range(spec.experts)]
        self.down = [tensors[f"experts.{e}.down.weight"].contiguous() for e in range(spec.experts)]

    def forward(self, x, ctx):
        spec, ops, rt = self.spec, self.ops, self.runtime
        logits = x.float() @ self.router.T
        probs = torch.softmax(logits, dim=-1)
        choice = logits.argmax(dim=-1)
        delta = torch.zeros(x.shape[0], spec.width, dtype=torch.float32, device=x.device)
        for e in range(spec.experts):
            rows = (choice == e).nonzero().flatten()
            if rows.numel() == 0:
                continue
            picked = x[rows].contiguous()
            gate_up = torch.empty(rows.numel(), 2 * spec.expert_width, dtype=rt.act_dtype, device=x.device)
            ops.linear(picked, self.gate_up[e], gate_up)
            act = torch.empty(rows.numel(), spec.expert_width, dtype=rt.act_dtype, device=x.device)
            ops.silu_mul(gate_up, act)
            out = torch.empty(rows.numel(), spec.width, dtype=torch.float32, device=x.device)
            ops.linear(act, self.down[e], out)
            delta[rows] = out * probs[rows, e][:, None]
        return delta


def parse_toy(raw):
    base = parse_qwen2(dict(raw, architectures=["Qwen2ForCausalLM"]))
    layers = list(base.layers)
    routed = RoutedSpec(width=base.hidden_size, experts=EXPERTS, expert_width=EXPERT_WIDTH)
    layers[1] = LayerSpec(mixer=layers[1].mixer, mixer_norm=layers[1].mixer_norm, feed_forward=routed,
                          feed_forward_norm=layers[1].feed_forward_norm)
    base.architecture = "ToyRoutedForCausalLM"
    base.layers = layers
    base.order = [LayerRun(0, 0), LayerRun(1, 1), LayerRun(2, 2)]
    return base


def toy_names(config):
    prefix = {"mixer": "mix.", "mixer_norm": "ln1.", "feed_forward": "ffn.", "feed_forward_norm": "ln2."}
    return TensorNames("emb.weight", "ln_f.", "head.weight", lambda layer, role: f"h.{layer}.{prefix[role]}")


def plain_toy(raw, w, ids):
    """Whole-sequence oracle built from the plain implementation's parts."""
    sizes = pm.config_sizes(raw)
    rnd = pm.Rounder(())
    w = {k: v.double() for k, v in w.items()}
    n = len(ids)
    cos, sin = pm.rope_tables(torch.arange(n), sizes["head_dim"], sizes["theta"], torch.float64)
    x = w["emb.weight"][torch.tensor(ids)]
    margins, used = [], set()
    for layer in range(3):
        p = f"h.{layer}"
        a = pm.rms_norm(x, w[f"{p}.ln1.weight"], sizes["eps"])
        q, k, v = pm.attention_inputs(a, w, f"{p}.mix", sizes, cos, sin, rnd)
        x = x + pm.causal_attention(q, k, v).reshape(n, -1) @ w[f"{p}.mix.o_proj.weight"].T
        m = pm.rms_norm(x, w[f"{p}.ln2.weight"], sizes["eps"])
        if layer == 1:
            logits = m @ w[f"{p}.ffn.router.weight"].T
            probs = torch.softmax(logits, -1)
            top = torch.sort(logits, -1, descending=True).values
            margins.append((top[:, 0] - top[:, 1]).min().item())
            choice = logits.argmax(-1)
            used |= set(choice.tolist())
            out = torch.zeros_like(x)
            for t in range(n):
                e = int(choice[t])
                g = m[t] @ w[f"{p}.ffn.experts.{e}.gate.weight"].T
                u = m[t] @ w[f"{p}.ffn.experts.{e}.up.weight"].T
                out[t] = probs[t, e] * ((g * torch.sigmoid(g) * u) @ w[f"{p}.ffn.experts.{e}.down.weight"].T)
            x = x + out
        else:
            x = x + pm.mlp(m, w, f"{p}.ffn", rnd)
    return (pm.rms_norm(x, w["ln_f.weight"], sizes["eps"]) @ w["head.weight"].T).numpy(), min(margins), used


def test_toy_feed_forward_with_routing_is_registered_built_and_stepped():
    register_part("feed_forward", "toy_routed", RoutedFeedForward)
    register_architecture(Architecture("ToyRoutedForCausalLM", parse_toy, toy_names))
    raw = dict(TINY_A, architectures=["ToyRoutedForCausalLM"], num_hidden_layers=3, tie_word_embeddings=False)
    config = parse_config(raw)
    weights = random_tensors(config, 6)
    assert "h.1.ffn.router.weight" in weights and "h.1.ffn.gate_proj.weight" not in weights
    assert "h.0.ffn.gate_proj.weight" in weights and f"h.1.ffn.experts.{EXPERTS - 1}.down.weight" in weights
    weights["h.1.ffn.router.weight"] = weights["h.1.ffn.router.weight"] * 40   # clear choices: no near ties
    runner = ModelRunner(config, {k: v.to(DEV) for k, v in weights.items()}, cuda_ops(torch.float32), DEV,
                         "float32", page_size=16, num_pages=12, max_slots=3)
    requests = {name: random_tokens(256, n, seed) for name, n, seed in (("a", 41, 1), ("b", 23, 2), ("c", 10, 3))}
    want, taken = {}, set()
    for name, ids in requests.items():
        want[name], margin, used = plain_toy(raw, weights, ids)
        taken |= used
        assert margin > 1e-3, "a router choice this close could flip between float32 and float64"
    assert len(taken) >= 2, "the test is only worth its name if more than one expert is taken"
    caches = {name: runner.cache.open() for name in requests}
    fed = {name: 0 for name in requests}
    got = {name: [] for name in requests}
    plan = [{"a": 18, "b": 1}, {"a": 1, "b": 9, "c": 10}, {"a": 22, "b": 13}]
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
        assert_close(np.concatenate(got[name]), want[name], TOL["float32"], f"toy routed model request {name}")
