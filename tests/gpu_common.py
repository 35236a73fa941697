"""Shared by the GPU tests: tolerances and a replay runner."""

from __future__ import annotations

import numpy as np
import torch

from tests.helpers import collect, max_live_tokens

# Absolute tolerances on logits of order one, fixed before the first GPU run:
# float32 against the float64 plain implementation, and bfloat16 against the plain
# implementation with bfloat16 rounding at the engine's rounding points.
TOL = {"float32": 2e-5, "bfloat16": 2e-2}


def replay(folder, dtype, steps, max_tokens=None, poison=False, page_size=None, num_pages=None, max_live=None):
    """Runs a trace in-process through the replay program's session; returns
    per-request logits and the session."""
    from shrike_b200.replay import TraceSession

    if num_pages is None and max_tokens is None:
        max_tokens = max_live_tokens(steps)
    session = TraceSession(folder, dtype, max_tokens, page_size=page_size, num_pages=num_pages, max_live=max_live)
    if poison:  # whatever is read from a page before it was written shows as NaN
        for pool in session.runner.storage.kv:
            pool.fill_(float("nan"))
    outputs = {}
    for record in steps:
        result = session.step(record)
        if result is not None:
            outputs[record["step"]] = result.copy()
    return collect(steps, outputs), session


def assert_close(got: np.ndarray, want: np.ndarray, tol: float, what: str = ""):
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite values"
    diff = np.abs(got.astype(np.float64) - want)
    if diff.max() > tol:
        row = int(np.argmax(diff.max(axis=-1))) if diff.ndim > 1 else int(np.argmax(diff))
        raise AssertionError(f"{what}: max |diff| {diff.max():.3e} > {tol:.1e}; first bad row {np.argmax(diff.max(axis=-1) > tol) if diff.ndim > 1 else row}, worst row {row}")


def cuda_ops(dtype):
    from shrike_b200.ops.cuda_ops import CudaOps

    return CudaOps(dtype, "cuda")
