"""A fourth toy, again registered from outside the package: a model whose only memory is
per-request state (no key/value group at all), with an embedding part of its own (scaled
rows) and a mixer whose forward pass reads the step's metadata on the device only
(`ctx.state_slot`, `ctx.seq_start`), so that it may be recorded and replayed as a CUDA graph.
It runs through `LLMEngine.generate` with chunked prompts, with requests preempted on the way
(their state is rebuilt by running the prompt again), on state slots that were left dirty:
the framework zeroes a slot when a request is opened; the mixer never does."""

from dataclasses import dataclass, field

import pytest
import torch

from shrike_b200 import SamplingParams
from shrike_b200.config import Architecture, LayerRun, LayerSpec, ModelConfig, TensorNames, parse_config, register_architecture
from shrike_b200.config.model_config import GatedMLPSpec, PartSpec, RMSNormSpec
from shrike_b200.engine.llm_engine import LLMEngine
from shrike_b200.parts import ParamSpec, StateNeed, register_part
from shrike_b200.weights import random_tensors
from tests.gpu_common import cuda_ops
from tests.helpers import random_tokens
from tests.plain import plain_model as pm

pytestmark = pytest.mark.gpu
DEV = "cuda"


@dataclass(frozen=True)
class ScaledEmbeddingSpec(PartSpec):
    vocab: int
    width: int
    scale: float
    kind: str = field(init=False, default="toy_scaled_embedding")


class ScaledEmbedding:
    capture_safe = True

    @staticmethod
    def parameters(spec):
        return {"weight": ParamSpec((spec.vocab, spec.width), "table")}

    def __init__(self, spec, tensors, ops, runtime):
        self.spec, self.ops, self.runtime = spec, ops, runtime
        self.table = tensors["weight"]

    def forward(self, ctx):
        resid = self.runtime.buffer("resid", (ctx.num_tokens, self.spec.width), torch.float32)
        self.ops.embed(ctx.token_ids, self.table, resid, ctx.previous_tokens)
        return resid.mul_(self.spec.scale)


@dataclass(frozen=True)
class PrefixMeanSpec(PartSpec):
    width: int
    kind: str = field(init=False, default="toy_prefix_mean")


class PrefixMean:
    """out[t] = proj(mean of x[0..t]); the state is the sum so far.  Everything that differs
    between two steps of the same shape (slots, positions) is read on the device."""

    capture_safe = True

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
        slots = ctx.state_slot.long()
        valid = (slots >= 0).unsqueeze(1)                       # padding rows carry slot -1
        held = state[slots.clamp(min=0)] * valid                # [S, W]: the sums before this step
        mean = torch.empty(x.shape, dtype=torch.float32, device=x.device)
        added = torch.zeros_like(held)
        cursor = 0
        for index, q_len in enumerate(ctx.q_lens):              # the batch's shape: the same in every replay
            sums = torch.cumsum(x[cursor: cursor + q_len].float(), 0) + held[index]
            counts = ctx.seq_start[index] + torch.arange(1, q_len + 1, device=x.device)
            mean[cursor: cursor + q_len] = sums / counts.unsqueeze(1)
            added[index] = sums[-1] - held[index]
            cursor += q_len
        state.index_add_(0, slots.clamp(min=0), added * valid)  # padding rows add zero to slot 0
        delta = self.runtime.buffer("mixer_delta", (x.shape[0], self.spec.width), torch.float32)
        self.ops.linear(mean.to(self.runtime.act_dtype), self.proj, delta)
        return delta


def parse_state_only(raw):
    width, layers = raw["hidden_size"], raw["num_hidden_layers"]
    norm = RMSNormSpec(width=width, eps=raw["rms_norm_eps"])
    layer = LayerSpec(mixer=PrefixMeanSpec(width=width), mixer_norm=norm,
                      feed_forward=GatedMLPSpec(width=width, intermediate=raw["intermediate_size"], activation="silu"),
                      feed_forward_norm=norm)
    return ModelConfig(
        architecture="ToyStateOnlyForCausalLM", hidden_size=width, vocab_size=raw["vocab_size"],
        layers=[layer] * layers, order=[LayerRun(i, i) for i in range(layers)], final_norm=norm,
        tie_word_embeddings=True, max_position_embeddings=4096, eos_token_ids=[], dtype="float32", raw=dict(raw),
        embedding=ScaledEmbeddingSpec(vocab=raw["vocab_size"], width=width, scale=raw["embedding_scale"]),
    )


def state_only_names(config):
    prefix = {"mixer": "mix.", "mixer_norm": "ln1.", "feed_forward": "mlp.", "feed_forward_norm": "ln2."}
    return TensorNames("emb.weight", "ln_f.", "head.weight", lambda layer, role: f"h.{layer}.{prefix[role]}")


RAW = dict(architectures=["ToyStateOnlyForCausalLM"], hidden_size=96, intermediate_size=160, num_hidden_layers=2,
           vocab_size=211, rms_norm_eps=1e-5, embedding_scale=96 ** 0.5)


def plain_logits(w, ids):
    """Whole-sequence oracle from the plain implementation's parts, in float64."""
    w = {k: v.double().cpu() for k, v in w.items()}
    n = len(ids)
    x = w["emb.weight"][torch.tensor(ids)] * RAW["embedding_scale"]
    for layer in range(RAW["num_hidden_layers"]):
        p = f"h.{layer}"
        a = pm.rms_norm(x, w[f"{p}.ln1.weight"], RAW["rms_norm_eps"])
        x = x + (torch.cumsum(a, 0) / torch.arange(1, n + 1)[:, None]) @ w[f"{p}.mix.proj.weight"].T
        m = pm.rms_norm(x, w[f"{p}.ln2.weight"], RAW["rms_norm_eps"])
        x = x + pm.mlp(m, w, f"{p}.mlp", pm.Rounder(()))
    return pm.rms_norm(x, w["ln_f.weight"], RAW["rms_norm_eps"]) @ w["emb.weight"].T   # tied head


def plain_greedy(w, prompt, count):
    seq, margins = list(prompt), []
    for _ in range(count):
        row = plain_logits(w, seq)[-1]
        top = torch.topk(row, 2).values
        margins.append(float(top[0] - top[1]))
        seq.append(int(row.argmax()))
    return seq[len(prompt):], margins


def test_state_only_model_generates_through_the_engine_with_preemption():
    register_part("embedding", "toy_scaled_embedding", ScaledEmbedding)
    register_part("mixer", "toy_prefix_mean", PrefixMean)
    register_architecture(Architecture("ToyStateOnlyForCausalLM", parse_state_only, state_only_names))
    config = parse_config(RAW)
    weights = random_tensors(config, 7)
    assert set(weights) >= {"emb.weight", "h.0.mix.proj.weight", "ln_f.weight"} and "head.weight" not in weights
    engine = LLMEngine(None, config=config, tensors={k: v.to(DEV) for k, v in weights.items()}, dtype="float32",
                       max_tokens_per_step=12, max_running=3, gpu_mem_util=0.01)
    runner = engine.runner
    assert runner.groups == [] and runner.storage.kv == [] and sorted(runner.storage.state) == [0, 1]
    assert runner.state_bytes == 2 * 3 * 96 * 4 and runner.capture_safe
    for tensor in runner.storage.state.values():
        tensor.fill_(1e3)   # what earlier requests may have left: a newly opened slot must not see it
    prompts = [random_tokens(211, n, 50 + n) for n in (5, 30, 17, 1, 26)]
    params = SamplingParams(max_new_tokens=10, ignore_eos=True)
    ids = [engine.add_request(prompt, params) for prompt in prompts]
    out = {i: [] for i in ids}
    steps = 0
    while engine.has_work:
        for output in engine.step():
            out[output.req_id].append(output.token_id)
        steps += 1
        if steps in (3, 9, 14):   # as a shortage of pages would: the newest running request starts over
            engine.scheduler.preempt_newest()
    assert engine.scheduler.num_preemptions == 3 and engine.block_manager.whole()
    assert len(runner._graphs) >= 1, "no step of the state-only model was recorded"
    for prompt, i in zip(prompts, ids):
        want, margins = plain_greedy(weights, prompt, 10)
        assert len(out[i]) == 10
        for a, b, margin in zip(out[i], want, margins):
            if a != b:
                assert margin < 1e-4, f"engine {out[i]} against plain {want}"
                break
