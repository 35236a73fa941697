"""Helpers shared by the tests: model folders, traces, comparisons."""

from __future__ import annotations

import json
import random
from pathlib import Path

import numpy as np
import torch

from tests.plain import plain_model as pm
from tests.tiny_configs import SEEDS, TINY, windows_of


def make_model_folder(tmp_path, key: str, dtype: str = "float32") -> Path:
    from shrike_b200 import models  # noqa: F401
    from shrike_b200.weights.random_init import write_model_folder

    return write_model_folder(Path(tmp_path) / f"tiny_{key}_{dtype}", TINY[key], SEEDS[key], dtype)


def read_weights(folder) -> dict:
    """Name -> float32 tensor, read with the `safetensors` package (not the engine's loader)."""
    from safetensors.torch import load_file

    return {k: v for k, v in load_file(str(Path(folder) / "model.safetensors")).items()}


def random_tokens(vocab: int, count: int, seed: int) -> list[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(count)]


def plain_logits(key: str, weights: dict, tokens, bf16: bool = False, **kw) -> np.ndarray:
    raw = TINY[key]
    if bf16:
        weights = {k: (v.to(torch.bfloat16) if v.dim() >= 2 else v) for k, v in weights.items()}
    out = pm.forward(raw, weights, tokens, dtype=torch.float64,
                     rounding=pm.ROUNDING_POINTS if bf16 else (), windows=windows_of(raw), **kw)
    return out.numpy()


# ---- traces --------------------------------------------------------------------
def whole_trace(requests: dict[str, list[int]]) -> list[dict]:
    """Each request alone and whole, one step each; all logits wanted."""
    steps = []
    for index, (ident, tokens) in enumerate(requests.items()):
        steps.append({"step": index, "entries": [{"id": ident, "tokens": tokens, "want": list(range(len(tokens)))}],
                      "end": [ident]})
    return steps


def tail_decode_trace(requests: dict[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of each request in one step, the last `tail` tokens one by one."""
    steps = []
    for ident, tokens in requests.items():
        t = min(tail, len(tokens) - 1)
        head = len(tokens) - t
        steps.append({"step": len(steps), "entries": [{"id": ident, "tokens": tokens[:head], "want": list(range(head))}],
                      "end": [ident] if t == 0 else []})
        for i in range(head, len(tokens)):
            steps.append({"step": len(steps), "entries": [{"id": ident, "tokens": [tokens[i]], "want": [0]}],
                          "end": [ident] if i == len(tokens) - 1 else []})
    return steps


def portions_trace(requests: dict[str, list[int]], sizes) -> list[dict]:
    """Portions of changing size, cycling through `sizes`, one request after the other."""
    steps = []
    for ident, tokens in requests.items():
        pos, turn = 0, 0
        while pos < len(tokens):
            n = min(sizes[turn % len(sizes)], len(tokens) - pos)
            turn += 1
            last = pos + n == len(tokens)
            steps.append({"step": len(steps), "entries": [{"id": ident, "tokens": tokens[pos:pos + n], "want": list(range(n))}],
                          "end": [ident] if last else []})
            pos += n
    return steps


def mixed_trace(requests: dict[str, list[int]], seed: int, max_live: int = 4, prompt_fraction: float = 0.6) -> list[dict]:
    """Up to `max_live` requests at a time; in each step some feed a portion of
    their 'prompt' part, others single tokens, some sit the step out.  Requests are
    admitted as others end, so pages are handed out again."""
    rng = random.Random(seed)
    pending = list(requests.items())
    live: dict[str, list] = {}  # id -> [tokens, fed, prompt_len]
    steps = []
    while pending or live:
        while pending and len(live) < max_live:
            ident, tokens = pending.pop(0)
            live[ident] = [tokens, 0, max(1, int(len(tokens) * prompt_fraction))]
        entries, ended = [], []
        for ident in list(live):
            tokens, fed, prompt_len = live[ident]
            if len(live) > 1 and rng.random() < 0.2:
                continue  # left out of this step
            if fed < prompt_len:
                n = min(prompt_len - fed, rng.choice([2, 3, 5, 7, 15, 16, 17, 33]))
            else:
                n = 1
            n = min(n, len(tokens) - fed)
            entries.append({"id": ident, "tokens": tokens[fed:fed + n], "want": list(range(n))})
            live[ident][1] = fed + n
            if fed + n == len(tokens):
                ended.append(ident)
                del live[ident]
        if entries:
            entries.sort(key=lambda e: len(e["tokens"]) > 1)  # singles first, as the scheduler does
            steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


def collect(steps: list[dict], outputs: dict[int, np.ndarray]) -> dict[str, np.ndarray]:
    """Reassembles per-request [len, vocab] logits from per-step outputs."""
    rows: dict[str, dict[int, np.ndarray]] = {}
    fed: dict[str, int] = {}
    for record in steps:
        out = outputs.get(record["step"])
        cursor = 0
        for entry in record["entries"]:
            ident = entry["id"]
            base = fed.get(ident, 0)
            for w in entry["want"]:
                rows.setdefault(ident, {})[base + w] = out[cursor]
                cursor += 1
            fed[ident] = base + len(entry["tokens"])
    return {ident: np.stack([table[i] for i in sorted(table)]) for ident, table in rows.items()}


def max_live_tokens(steps: list[dict]) -> int:
    """The --max-tokens a trace needs: live requests' tokens, each rounded up to 64."""
    held: dict[str, int] = {}
    worst = 0
    for record in steps:
        for entry in record["entries"]:
            held[entry["id"]] = held.get(entry["id"], 0) + len(entry["tokens"])
        worst = max(worst, sum(-(-n // 64) * 64 for n in held.values()))
        for ident in record["end"]:
            held.pop(ident, None)
    return worst


def write_trace(path, steps):
    Path(path).write_text("".join(json.dumps(s) + "\n" for s in steps))
