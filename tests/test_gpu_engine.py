"""Generation through the Python entry point on the GPU."""

import pytest
import torch

from shrike_b200 import SamplingParams
from shrike_b200.engine.llm_engine import LLMEngine
from tests.helpers import make_model_folder, random_tokens, read_weights
from tests.plain import plain_model as pm
from tests.tiny_configs import PAGE_SIZES, TINY, windows_of

pytestmark = pytest.mark.gpu


def plain_greedy(key, weights, prompt, count, bf16):
    raw = TINY[key]
    if bf16:
        weights = {k: (v.to(torch.bfloat16) if v.dim() >= 2 else v) for k, v in weights.items()}
    return pm.greedy_continue(raw, weights, prompt, count, rounding=pm.ROUNDING_POINTS if bf16 else (),
                              windows=windows_of(raw))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key,lengths,new", [("A", (5, 17, 33), 8), ("C", (3, 40, 29), 8)])
def test_greedy_generation_matches_plain(tmp_path, key, lengths, new, dtype):
    folder = make_model_folder(tmp_path, key)
    weights = read_weights(folder)
    engine = LLMEngine(str(folder), block_size=PAGE_SIZES[key], num_blocks=24, dtype=dtype)
    prompts = [random_tokens(TINY[key]["vocab_size"], n, 30 + n) for n in lengths]
    outs = engine.generate(prompts, SamplingParams(max_new_tokens=new, ignore_eos=True))
    assert engine.block_manager.whole()
    for prompt, out in zip(prompts, outs):
        want, margins = plain_greedy(key, weights, prompt, new, dtype == "bfloat16")
        tie = 1e-4 if dtype == "float32" else 4e-2   # a top-2 gap below twice the logit tolerance is a tie
        for position, (a, b, margin) in enumerate(zip(out, want, margins)):
            if a != b:
                assert margin < tie, f"token {position}: engine {a}, plain {b}, gap {margin}"
                break  # after a tie went the other way the continuations differ


def test_tiny_b_with_few_pages_chunking_and_temperature(tmp_path):
    """Prompts 1/9/40/64/70, 12 tokens each at temperature 0.8, budget 24, page 8, 20
    pages: preemption happens, and every request's tokens equal those it gets alone."""
    folder = make_model_folder(tmp_path, "B")
    prompts = [random_tokens(384, n, 40 + n) for n in (1, 9, 40, 64, 70)]
    params = [SamplingParams(max_new_tokens=12, temperature=0.8, ignore_eos=True, seed=500 + i) for i in range(5)]
    crowded = LLMEngine(str(folder), block_size=8, num_blocks=20, max_tokens_per_step=24, max_running=4, dtype="float32")
    batched = crowded.generate(prompts, params)
    assert crowded.scheduler.num_preemptions >= 1 and crowded.block_manager.whole()
    roomy = LLMEngine(str(folder), block_size=8, num_blocks=64, dtype="float32")
    for prompt, param, want in zip(prompts, params, batched):
        assert roomy.generate([prompt], param)[0] == want
    assert all(len(o) == 12 for o in batched)


def test_engine_refuses_without_kernels_dtype(tmp_path):
    folder = make_model_folder(tmp_path, "A")
    with pytest.raises(ValueError, match="dtype"):
        LLMEngine(str(folder), dtype="float16")


@pytest.mark.parametrize("block_size", [8, 32, 64])
def test_pool_sized_from_free_memory_and_other_page_sizes(tmp_path, block_size):
    """`gpu_mem_util` sizes the pool from free device memory (no explicit num_blocks), and
    generation does not depend on the page size."""
    folder = make_model_folder(tmp_path, "B")
    weights = read_weights(folder)
    engine = LLMEngine(str(folder), block_size=block_size, gpu_mem_util=0.002, dtype="float32")
    assert min(engine.block_manager.num_pages) > 100
    prompts = [random_tokens(384, n, 80 + n) for n in (7, 70, 33)]
    outs = engine.generate(prompts, SamplingParams(max_new_tokens=6, ignore_eos=True))
    assert engine.block_manager.whole()
    for prompt, out in zip(prompts, outs):
        want, margins = plain_greedy("B", weights, prompt, 6, False)
        for a, b, margin in zip(out, want, margins):
            if a != b:
                assert margin < 1e-4
                break


def test_bfloat16_decode_steps_are_replayed_and_match_eager(tmp_path):
    """The captured decode step gives the tokens the eager step gives."""
    folder = make_model_folder(tmp_path, "A")
    prompts = [random_tokens(256, n, 90 + n) for n in (5, 17, 33, 2)]
    params = SamplingParams(max_new_tokens=40, ignore_eos=True)
    captured = LLMEngine(str(folder), num_blocks=32, dtype="bfloat16")
    a = captured.generate(prompts, params)
    assert len(captured.runner._graphs) >= 1, "no decode step was captured"
    eager = LLMEngine(str(folder), num_blocks=32, dtype="bfloat16")
    eager.runner.use_graphs = False
    b = eager.generate(prompts, params)
    assert a == b


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batches_with_portions_are_captured_when_their_shape_repeats(tmp_path, dtype):
    """A long prompt cut into equal portions beside a decoding request: from the third such step
    on the launch sequence is replayed, at other positions and pages than it was captured at;
    the logits are those of the eager steps."""
    import torch

    from shrike_b200.config import load_config
    from shrike_b200.engine.batch import StepEntry
    from shrike_b200.engine.llm_engine import make_ops
    from shrike_b200.engine.runner import ModelRunner
    from shrike_b200.weights import load_weights

    folder = make_model_folder(tmp_path, "C")   # windows on some layers: pages are given back on the way
    config = load_config(str(folder))
    ids = {"long": random_tokens(331, 150, 1), "short": random_tokens(331, 12, 2)}

    def run(capture: bool):
        tensors = load_weights(str(folder), config, getattr(torch, dtype), "cuda")
        runner = ModelRunner(config, tensors, make_ops(dtype, "cuda"), "cuda", dtype, page_size=16, num_pages=24, max_slots=4)
        assert runner.capture_portions
        runner.capture_portions = capture
        caches = {name: runner.cache.open() for name in ids}
        runner.cache.append(caches["short"], 0, 5)
        runner.step([StepEntry(caches["short"], ids["short"][:5], 0, [])])
        fed, short_fed, rows = 0, 5, []
        runner.portion_sightings = 2
        for _ in range(6):   # six steps of the same shape: one decoded token beside a portion of 24
            runner.cache.append(caches["short"], short_fed, 1)
            runner.cache.append(caches["long"], fed, 24)
            logits = runner.step([StepEntry(caches["short"], ids["short"][short_fed: short_fed + 1], short_fed, [0]),
                                  StepEntry(caches["long"], ids["long"][fed: fed + 24], fed, [0, 23])])
            rows.append(logits.float().cpu().clone())
            short_fed += 1
            fed += 24
            runner.cache.advance(caches["long"], fed)
            runner.cache.advance(caches["short"], short_fed)
        return torch.cat(rows), len(runner._graphs)

    captured, graphs = run(True)
    eager, none = run(False)
    assert graphs >= 1 and none == 0
    assert torch.equal(captured, eager) if dtype == "float32" else (captured - eager).abs().max() < 2e-2


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_launching_ahead_gives_the_tokens_of_the_plain_loop_on_the_gpu(tmp_path, dtype):
    """Greedy and sampled requests of different lengths, long enough for the block tables to
    widen (new launch sequences are captured while a step is in flight): the engine that
    launches a step ahead of the host and the one that does not draw the same tokens."""
    folder = make_model_folder(tmp_path, "C")
    prompts = [random_tokens(331, n, 7 + n) for n in (3, 40, 130, 17)]
    params = [SamplingParams(max_new_tokens=m, ignore_eos=True, temperature=t, top_p=p, seed=11)
              for m, t, p in ((160, 0.0, 1.0), (120, 0.9, 0.95), (60, 0.0, 1.0), (150, 1.2, 1.0))]
    outs = []
    for ahead in (True, False):
        engine = LLMEngine(str(folder), num_blocks=120, dtype=dtype, max_running=4)
        engine.launch_ahead = ahead
        outs.append(engine.generate(prompts, params))
        assert engine.block_manager.whole() and not engine.requests
        assert len(engine.runner._graphs) >= 3
        engine.ops.check_status()
    assert outs[0] == outs[1]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_batches_padded_to_a_few_sizes_give_the_same_logits_and_tokens(tmp_path, dtype):
    """Batches of 9 to 17 single tokens run as batches of 16 and 24 (padding rows that store
    nothing): the logits and drawn tokens of the real rows are those of the unpadded batch (in
    float32 bit for bit), the cache is left as the unpadded run leaves it (the next steps agree
    too), and far fewer launch sequences are captured."""
    import torch

    from shrike_b200.config import load_config
    from shrike_b200.engine.batch import StepEntry
    from shrike_b200.engine.llm_engine import make_ops
    from shrike_b200.engine.runner import ModelRunner
    from shrike_b200.weights import load_weights

    folder = make_model_folder(tmp_path, "B")
    config = load_config(str(folder))
    prompts = [random_tokens(384, 3 + 5 * i, 20 + i) for i in range(17)]

    def run(pad: bool):
        tensors = load_weights(str(folder), config, getattr(torch, dtype), "cuda")
        runner = ModelRunner(config, tensors, make_ops(dtype, "cuda"), "cuda", dtype, page_size=8, num_pages=300, max_slots=32)
        assert runner.pad_decode
        runner.pad_decode = pad
        caches, fed = [], []
        for ids in prompts:
            cache = runner.cache.open()
            runner.cache.append(cache, 0, len(ids))
            runner.step([StepEntry(cache, ids, 0, [])])
            caches.append(cache)
            fed.append(len(ids))
        logits, tokens = [], []
        for step, live in enumerate([17, 16, 13, 12, 11, 9, 9, 10, 17, 8, 15]):   # requests pause and come back
            entries = []
            for i in range(live):
                runner.cache.append(caches[i], fed[i], 1)
                entries.append(StepEntry(caches[i], [(31 * step + 7 * i) % 384], fed[i], [0], (0.8 if i % 3 else 0.0, 0.9, 5 + i)))
                fed[i] += 1
            out, drawn = runner.step(entries, sample=True)
            assert out.shape[0] == live and drawn.shape[0] == live
            logits.append(out.float().cpu().clone())
            tokens.append(drawn.cpu().tolist())
        graphs = len(runner._graphs)
        for cache in caches:
            runner.cache.free(cache)
        assert runner.cache.whole()
        return torch.cat(logits), tokens, graphs

    padded, padded_tokens, few = run(True)
    exact, exact_tokens, many = run(False)
    assert few <= 5 and many >= 9   # sizes 8, 16, 24 (times two table widths) against every size that came
    if dtype == "float32":
        assert torch.equal(padded, exact) and padded_tokens == exact_tokens
    else:
        assert (padded - exact).abs().max() < 2e-2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_kernel_that_gave_up_is_seen_before_its_tokens_are_used(tmp_path, dtype):
    """The status word comes to the host in the same copy as a step's tokens.  A code in it (set
    by hand here; on the device a bounded wait that ran out sets it) makes `step` raise before
    anything is appended or handed out, drops the step launched ahead, and clears the word; the
    caller aborts what was running, and the engine serves on."""
    from shrike_b200.ops.cuda_ops import KernelError

    folder = make_model_folder(tmp_path, "A")
    engine = LLMEngine(str(folder), num_blocks=32, dtype=dtype)
    params = SamplingParams(max_new_tokens=20, ignore_eos=True)
    first = engine.generate([random_tokens(256, 9, 1)], params)[0]
    ids = [engine.add_request(random_tokens(256, n, 2 + n), params) for n in (9, 5)]
    for _ in range(4):
        engine.step()
    lengths = {i: engine.requests[i].num_tokens for i in ids}
    engine.ops.status[0] = 2
    with pytest.raises(KernelError, match="MMA issuer"):
        for _ in range(3):   # the word travels with the next step's tokens (or the one launched ahead)
            engine.step()
    assert engine._flight is None and int(engine.ops.status[0]) == 0
    assert all(engine.requests[i].num_tokens <= lengths[i] + 2 for i in ids)
    for i in ids:
        engine.abort(i)
    assert engine.block_manager.whole() and not engine.has_work
    assert engine.generate([random_tokens(256, 9, 1)], params)[0] == first


@pytest.mark.parametrize("shape", ["tiny_c", "d64", "d128"])
def test_layers_issued_by_one_native_call_equal_the_part_by_part_path(tmp_path, shape):
    """A whole layer issued by one native call launches the same kernels with the same arguments
    as the parts do one by one: steps of up to 64 tokens give the same bits.  Longer steps send
    their products to the library through another door (cublasGemmEx instead of torch.mm), which
    may choose another kernel: those are held to the bfloat16 tolerance."""
    import torch

    from shrike_b200.config import parse_config
    from shrike_b200.engine.batch import StepEntry
    from shrike_b200.engine.llm_engine import make_ops
    from shrike_b200.engine.runner import ModelRunner
    from shrike_b200.weights import random_tensors

    raw = {
        "tiny_c": TINY["C"],
        "d64": dict(TINY["B"], hidden_size=448, num_attention_heads=7, num_key_value_heads=1, head_dim=64,
                    intermediate_size=608, vocab_size=1000, num_hidden_layers=2),
        "d128": dict(TINY["B"], hidden_size=512, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                     intermediate_size=1376, vocab_size=777, num_hidden_layers=2),
    }[shape]
    config = parse_config(raw)
    weights = random_tensors(config, 3, "cuda", torch.float32)
    vocab = raw["vocab_size"]
    ids = {"long": random_tokens(vocab, 400, 1), "short": random_tokens(vocab, 40, 2), "third": random_tokens(vocab, 90, 3)}
    plan = [{"long": 200}, {"long": 100, "short": 30}, {"long": 1, "short": 1, "third": 62}, {"long": 3, "short": 1, "third": 2},
            {"long": 1, "short": 1, "third": 1}, {"long": 95, "short": 1, "third": 25}]

    def run(native: bool):
        tensors = {k: (v.to(torch.bfloat16) if v.dim() >= 2 else v.clone()) for k, v in weights.items()}
        ops = make_ops("bfloat16", "cuda")
        ops.native_layers = native
        runner = ModelRunner(config, tensors, ops, "cuda", "bfloat16", page_size=16, num_pages=48, max_slots=4)
        runner.use_graphs = False
        caches = {name: runner.cache.open() for name in ids}
        fed = {name: 0 for name in ids}
        rows = []
        for step in plan:
            entries = []
            for name in sorted(step, key=lambda nm: step[nm] > 1):
                count = step[name]
                runner.cache.append(caches[name], fed[name], count)
                entries.append(StepEntry(caches[name], ids[name][fed[name]: fed[name] + count], fed[name], [0, count - 1]))
                fed[name] += count
            rows.append(runner.step(entries).float().cpu().clone())
            for name in step:
                runner.cache.advance(caches[name], fed[name])
        ops.check_status()
        return rows, ops.launches, ops.library_calls

    native, native_launches, native_library = run(True)
    parts, parts_launches, parts_library = run(False)
    assert (native_launches, native_library) == (parts_launches, parts_library)
    for step, a, b in zip(plan, native, parts):
        if sum(step.values()) <= 64:
            assert torch.equal(a, b), f"step {step}: the two ways of issuing differ"
        else:
            assert (a - b).abs().max() <= 2e-2 * max(1.0, float(b.abs().max())), f"step {step}"


@pytest.mark.parametrize("key", ["A", "C"])
def test_warm_up_leaves_the_engine_as_it_was(tmp_path, key):
    """warm_up() runs throw-away steps (those counts that the step's budget, the window's pool and the
    pool's size allow), gives every page and slot back, counts nothing, and the tokens generated after
    it are those of an engine that never warmed up."""
    folder = make_model_folder(tmp_path, key)
    prompts = [random_tokens(TINY[key]["vocab_size"], n, 70 + n) for n in (7, 45)]
    params = SamplingParams(max_new_tokens=6, ignore_eos=True)
    plain = LLMEngine(str(folder), block_size=PAGE_SIZES[key], num_blocks=24, dtype="bfloat16")
    want = plain.generate(prompts, params)
    warmed = LLMEngine(str(folder), block_size=PAGE_SIZES[key], num_blocks=24, max_tokens_per_step=100, dtype="bfloat16")
    launches = warmed.ops.launches
    seconds = warmed.warm_up(token_counts=(1, 16, 64, 100, 4096))
    assert seconds > 0 and warmed.ops.launches > launches
    assert warmed.block_manager.whole() and warmed.stats.steps == 0 and warmed.stats.tokens_generated == 0
    assert warmed.generate(prompts, params) == want
    warmed.add_request(prompts[0], params)
    with pytest.raises(RuntimeError):
        warmed.warm_up()
