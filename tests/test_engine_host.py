"""The engine loop and the step function's metadata, driven on the CPU through a
stand-in for the kernels (tests/emulated_ops.py).  This checks host logic only:
block tables, slots, positions, wanted rows, preemption and recompute."""

import numpy as np
import pytest
import torch

import shrike_b200.models  # noqa: F401
from shrike_b200 import SamplingParams
from shrike_b200.config import parse_config
from shrike_b200.engine.batch import StepEntry
from shrike_b200.engine.llm_engine import LLMEngine
from shrike_b200.engine.runner import ModelRunner
from shrike_b200.weights import random_tensors
from tests.emulated_ops import EmulatedOps
from tests.helpers import random_tokens
from tests.plain import plain_model as pm
from tests.tiny_configs import PAGE_SIZES, SEEDS, TINY, windows_of


def engine_for(key, **kw):
    config = parse_config(TINY[key])
    weights = random_tensors(config, SEEDS[key])
    options = dict(block_size=PAGE_SIZES[key], dtype="float32", device="cpu", config=config,
                   tensors=dict(weights), ops=EmulatedOps())
    options.update(kw)
    return LLMEngine(None, **options), weights


@pytest.mark.parametrize("key", ["A", "C"])
def test_step_function_matches_plain_under_cutting(key):
    raw = TINY[key]
    config = parse_config(raw)
    weights = random_tensors(config, SEEDS[key])
    ids = random_tokens(raw["vocab_size"], 70, 5)
    want = pm.forward(raw, weights, ids, windows=windows_of(raw)).numpy()
    runner = ModelRunner(config, dict(weights), EmulatedOps(), "cpu", "float32", page_size=16, num_pages=6, max_slots=2)
    cache, pos, rows = runner.cache.open(), 0, []
    for n in [7, 2, 5, 3, 2, 15, 16, 17, 1, 1, 1]:
        runner.cache.append(cache, pos, n)
        rows.append(runner.step([StepEntry(cache, ids[pos:pos + n], pos, list(range(n)))]).clone())
        pos += n
        runner.cache.advance(cache, pos)
    np.testing.assert_allclose(torch.cat(rows).numpy(), want, atol=2e-5)
    runner.cache.free(cache)
    assert runner.cache.whole()


def test_generate_equals_plain_greedy_with_preemption():
    engine, weights = engine_for("B", max_tokens_per_step=24, max_running=4, num_blocks=20)
    prompts = [random_tokens(384, n, 40 + n) for n in (1, 9, 40, 64, 70)]
    outs = engine.generate(prompts, SamplingParams(max_new_tokens=12, ignore_eos=True))
    assert engine.scheduler.num_preemptions >= 1, "the pool was meant to be too small"
    assert engine.block_manager.whole() and not engine.requests
    for prompt, out in zip(prompts, outs):
        want, margins = pm.greedy_continue(TINY["B"], weights, prompt, 12)
        assert min(margins) > 1e-5
        assert out == want
    metrics = engine.metrics()
    assert metrics["tokens_generated"] == 60 and metrics["kv_blocks_free"] == metrics["kv_blocks_total"] == 20


def test_eos_stops_and_ignore_eos_does_not():
    engine, weights = engine_for("A", num_blocks=16)
    prompt = random_tokens(256, 9, 1)
    free_run = engine.generate([prompt], SamplingParams(max_new_tokens=6, ignore_eos=True))[0]
    engine.eos_ids = {free_run[2]}
    first = free_run.index(free_run[2])
    outs = []
    engine.add_request(prompt, SamplingParams(max_new_tokens=6))
    while engine.has_work:
        outs += engine.step()
    assert [o.token_id for o in outs] == free_run[: first + 1]
    assert outs[-1].finished and outs[-1].finish_reason == "stop"
    again = engine.generate([prompt], SamplingParams(max_new_tokens=6, ignore_eos=True))[0]
    assert again == free_run and engine.block_manager.whole()


def test_requests_that_can_never_run_are_refused():
    engine, _ = engine_for("A", num_blocks=4)
    with pytest.raises(ValueError, match="empty prompt"):
        engine.add_request([], SamplingParams())
    with pytest.raises(ValueError, match="could never be scheduled"):
        engine.add_request([1] * 60, SamplingParams(max_new_tokens=10))
    with pytest.raises(ValueError, match="max_position_embeddings"):
        engine.add_request([1, 2], SamplingParams(max_new_tokens=10_000_000))
    with pytest.raises(ValueError, match="token ids"):
        engine.add_request([1, 256], SamplingParams())
    with pytest.raises(ValueError, match="tokenizer"):
        engine.add_request("hello", SamplingParams())
    assert not engine.has_work


def test_sampling_does_not_depend_on_the_batch():
    prompts = [random_tokens(384, n, 70 + n) for n in (3, 11, 26)]
    params = [SamplingParams(max_new_tokens=8, temperature=0.8, ignore_eos=True, seed=100 + i) for i in range(3)]
    together, _ = engine_for("B", num_blocks=32)
    batched = together.generate(prompts, params)
    for prompt, param, want in zip(prompts, params, batched):
        alone, _ = engine_for("B", num_blocks=32, max_tokens_per_step=5)
        assert alone.generate([prompt], param)[0] == want


def test_abort_frees_pages():
    engine, _ = engine_for("A", num_blocks=16)
    rid = engine.add_request(random_tokens(256, 20, 2), SamplingParams(max_new_tokens=50))
    engine.step()
    engine.step()
    engine.abort(rid)
    assert not engine.has_work and engine.block_manager.whole()


def test_single_token_split_rule_keeps_its_bounds():
    from shrike_b200.ops.cuda_ops import CudaOps

    resident = 296
    for tiles in (1, 2, 3, 7, 16, 17, 33, 64, 512, 4096):
        for groups in (1, 2, 4, 8, 16, 32, 33, 64, 100, 256, 1000):
            splits, cluster = CudaOps.single_token_splits(tiles, groups, resident)
            assert cluster in (1, 2, 4, 8) and splits >= 1 and splits % cluster == 0
            assert splits <= max(1, min(tiles, resident // groups)) and splits // cluster <= 32
            if cluster == 8:   # clusters of eight only while they leave a third of the GPU free
                assert groups * 8 * 3 <= resident * 2
    assert CudaOps.single_token_splits(16, 4, resident) == (8, 8)       # one sequence of a 4-kv-head model
    assert CudaOps.single_token_splits(16, 32, resident) == (8, 1)      # eight of them: too full for clusters
    assert CudaOps.single_token_splits(16, 64, resident) == (4, 4)
    assert CudaOps.single_token_splits(16, 256, resident) == (1, 1)
    assert CudaOps.single_token_splits(512, 4, resident) == (72, 8)     # a long context: nine clusters


def _run_script(launch_ahead: bool, pool: int):
    """Requests that arrive, stop on a token, run out of length and are aborted at fixed steps."""
    engine, _ = engine_for("B", max_tokens_per_step=32, max_running=4, num_blocks=pool)
    engine.launch_ahead = launch_ahead
    prompts = [random_tokens(384, n, 70 + n) for n in (5, 12, 30, 3, 17)]
    first = engine.generate([prompts[0]], SamplingParams(max_new_tokens=8, ignore_eos=True))[0]
    engine.eos_ids = {first[4]}   # the first request now stops at its fifth token (or earlier)
    ids = [engine.add_request(prompts[0], SamplingParams(max_new_tokens=20)),
           engine.add_request(prompts[1], SamplingParams(max_new_tokens=9, temperature=0.8, top_p=0.9, seed=3)),
           engine.add_request(prompts[2], SamplingParams(max_new_tokens=25, ignore_eos=True))]
    log, staged_steps, step = [], 0, 0
    mixed_ahead = 0
    while engine.has_work:
        staged_steps += engine._flight is not None
        mixed_ahead += engine._flight is not None and any(n > 1 for _, n in engine._flight[0])
        for out in engine.step():
            log.append((out.req_id - ids[0], out.token_id, out.finished, out.finish_reason))
        step += 1
        if step == 6:
            ids.append(engine.add_request(prompts[3], SamplingParams(max_new_tokens=7, ignore_eos=True)))
        if step == 9:
            engine.abort(ids[2])
        if step == 11:
            ids.append(engine.add_request(prompts[4], SamplingParams(max_new_tokens=5, temperature=1.1, seed=9)))
    assert engine.block_manager.whole() and not engine.requests
    return log, (staged_steps, mixed_ahead), engine.scheduler.num_preemptions


def _by_request(log):
    table = {}
    for req, token, finished, reason in log:
        table.setdefault(req, []).append((token, finished, reason))
    return table


@pytest.mark.parametrize("pool", [40, 8])
def test_launching_the_next_step_ahead_changes_no_token(pool):
    """The engine launches a step before the tokens of the step before it are read back (the
    embedding takes them on the device): in steady decoding, and, where pages are plenty, also
    steps with portions of prompts and newly admitted requests.  Arrivals, a stop token, length
    limits, an abort and (with the small pool) preemption all fall between such steps; every
    request gets the tokens, the end and the reason of the plain loop.  Only the interleaving
    may differ: a request that arrives while a step is in flight joins one step later."""
    plain, (none_ahead, _), _ = _run_script(False, pool)
    ahead, (launched_ahead, with_portions), preemptions = _run_script(True, pool)
    assert none_ahead == 0 and launched_ahead >= 4
    if pool == 40:
        assert with_portions >= 1, "no step with a portion was launched ahead although pages were plenty"
    assert _by_request(ahead) == _by_request(plain)
    assert any(reason == "stop" for *_, reason in plain) and any(reason == "length" for *_, reason in plain)
    if pool == 8:
        assert preemptions >= 1


def test_a_stop_token_while_the_next_step_is_in_flight_drops_that_row_only():
    engine, _ = engine_for("A", num_blocks=24, max_running=4)
    prompts = [random_tokens(256, n, 11 + n) for n in (9, 4, 13)]
    free_run = engine.generate(prompts, SamplingParams(max_new_tokens=10, ignore_eos=True))
    stop = free_run[1][3]                      # the second request's fourth token becomes the stop token
    engine.eos_ids = {stop}
    cut = [run[: run.index(stop) + 1] if stop in run else run for run in free_run]
    got = engine.generate(prompts, SamplingParams(max_new_tokens=10))
    assert got == cut and len(cut[1]) <= 4
    assert engine.block_manager.whole() and not engine.requests
    # whatever was in flight when the last request ended is drained by the next call
    assert engine.generate([prompts[0]], SamplingParams(max_new_tokens=3, ignore_eos=True))[0] == free_run[0][:3]


def test_padding_rows_of_a_decode_batch_store_nothing_and_come_last():
    """A batch of single tokens padded to a fixed size: real rows first and unchanged, padding rows
    are one-token sequences at position 0 over page 0 with slot -1 and state slot -1; batches
    with a portion, or with a row that wants nothing, are never padded."""
    from shrike_b200.engine.batch import BatchBuilder

    engine, _ = engine_for("A", num_blocks=16)
    cache_manager, builder = engine.block_manager, BatchBuilder(16, 1, "cpu", None)
    caches = []
    for length in (20, 3, 17):
        cache = cache_manager.open()
        cache_manager.append(cache, 0, length + 1)
        caches.append((cache, length))
    entries = [StepEntry(c, [7 + i], n, [0], (0.5, 0.9, 11 + i)) for i, (c, n) in enumerate(caches)]
    plain = builder.stage(entries)
    assert (plain.s, plain.r, plain.rows) == (3, 3, 3)
    a = builder.context(plain)
    rows_a = [t.clone() for t in (a.token_ids, a.positions, a.ctx_len, a.state_slot, a.groups[0].slot_mapping,
                                   a.groups[0].block_table, a.sample_temperature, a.sample_seed)]
    padded = builder.stage(entries, pad_to=8)
    assert (padded.n, padded.s, padded.r, padded.rows) == (8, 8, 8, 3)
    b = builder.context(padded)
    rows_b = (b.token_ids, b.positions, b.ctx_len, b.state_slot, b.groups[0].slot_mapping,
              b.groups[0].block_table, b.sample_temperature, b.sample_seed)
    for x, y in zip(rows_a, rows_b):
        assert torch.equal(x, y[:3])
    assert b.token_ids[3:].tolist() == [0] * 5 and b.positions[3:].tolist() == [0] * 5
    assert b.ctx_len[3:].tolist() == [1] * 5 and b.state_slot[3:].tolist() == [-1] * 5
    assert b.groups[0].slot_mapping[3:].tolist() == [-1] * 5
    assert b.groups[0].block_table[3:, 0].tolist() == [0] * 5 and (b.groups[0].block_table[3:, 1:] == -1).all()
    assert b.sample_temperature[3:].tolist() == [0.0] * 5 and b.sample_top_p[3:].tolist() == [1.0] * 5
    assert b.q_start.tolist() == list(range(9)) and b.out_rows.tolist() == list(range(8)) and b.all_single
    silent = entries[:2] + [StepEntry(caches[2][0], [9], caches[2][1], [])]
    assert builder.stage(silent, pad_to=8).s == 3
    cache_manager.append(caches[0][0], 21, 1)
    portion = [StepEntry(caches[0][0], [1, 2], 20, [1])] + entries[1:]
    assert builder.stage(portion, pad_to=8).s == 3
    for cache, _ in caches:
        cache_manager.free(cache)


def test_batch_metadata_carries_each_entrys_first_position_and_pads_with_zero():
    """`seq_start` lies beside `state_slot` in the packed block: a part with state can tell a request's
    first portion from a later one without a host-side list."""
    config = parse_config(TINY["A"])
    runner = ModelRunner(config, dict(random_tensors(config, 0)), EmulatedOps(), "cpu", "float32", page_size=16,
                         num_pages=16, max_slots=4)
    caches = [runner.cache.open() for _ in range(3)]
    starts, counts = [0, 7, 20], [5, 1, 3]
    for cache, start, count in zip(caches, starts, counts):
        runner.cache.append(cache, 0, start + count)
    entries = [StepEntry(cache, [1] * count, start, [count - 1]) for cache, start, count in zip(caches, starts, counts)]
    ctx = runner.builder.build(sorted(entries, key=lambda e: len(e.tokens) > 1))
    assert ctx.seq_start.tolist() == [7, 0, 20] and ctx.state_slot.tolist() == [caches[1].slot, caches[0].slot, caches[2].slot]
    assert ctx.q_start.tolist() == [0, 1, 6, 9] and ctx.ctx_len.tolist() == [8, 5, 23]
    singles = [StepEntry(cache, [1], start + count, [0]) for cache, start, count in zip(caches, starts, counts)]
    for cache, start, count in zip(caches, starts, counts):
        runner.cache.append(cache, start + count, 1)
    staged = runner.builder.stage(singles, pad_to=8)
    padded = runner.builder.context(staged)
    assert padded.seq_start.tolist() == [5, 8, 23, 0, 0, 0, 0, 0] and padded.state_slot.tolist()[3:] == [-1] * 5
    for cache in caches:
        runner.cache.free(cache)
    assert runner.cache.whole()


def test_opening_a_request_zeroes_its_state_before_the_step():
    """The step function clears the state slots of requests opened since the last step; nothing else is touched."""
    from shrike_b200.cache.manager import CacheManager
    from shrike_b200.cache.storage import CacheStorage, state_bytes
    from shrike_b200.parts.base import StateNeed

    needs = {3: StateNeed((4, 2), "float32"), 5: StateNeed((6,), "float32")}
    assert state_bytes(needs, 10) == 10 * (8 + 6) * 4
    manager = CacheManager([], 16, [], 4)
    storage = CacheStorage([], 16, [], needs, 4, torch.float32, "cpu")
    for tensor in storage.state.values():
        tensor.fill_(9.0)
    a = manager.open()
    storage.zero_slots(manager.take_opened())
    assert float(storage.state[3][a.slot].abs().sum()) == 0 and float(storage.state[5][a.slot].abs().sum()) == 0
    others = [s for s in range(4) if s != a.slot]
    assert all(float(storage.state[3][s].min()) == 9.0 for s in others)
    storage.zero_slots(manager.take_opened())   # nothing opened since: nothing cleared
    assert all(float(storage.state[5][s].min()) == 9.0 for s in others)
