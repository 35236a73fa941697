"""Weights from a model folder, by tensor name.

What Azimml/shrike does (shrike/models/qwen.py:202-214): every `*.safetensors` in
the folder in sorted order, merged; a tied model without `lm_head.weight` aliases
the embedding; every tensor is cast to the model dtype; a strict load rejects
missing and unexpected names.  Here the check is explicit and says everything at
once: missing names, unexpected names and wrong shapes in one `WeightError`.

Kept precision: 16-bit floating tensors stay 16-bit (bfloat16) when the engine
runs bfloat16; a tensor stored in 32-bit stays 32-bit, except matrices and tables
(two or more dimensions), which feed the tensor cores and are cast to the engine
dtype; integer tensors become int32.  In float32 everything floating is float32.
"""

from __future__ import annotations

from pathlib import Path

import torch

from ..config.model_config import ModelConfig
from .expected import expected_tensors, tensor_names
from .safetensors_io import SafetensorsFile


class WeightError(RuntimeError):
    """Lists missing tensors, unexpected tensors and wrong shapes."""

    def __init__(self, folder, missing, unexpected, wrong_shape, duplicates=()):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)
        self.duplicates = sorted(duplicates)
        lines = [f"weights under {str(folder)!r} do not fit the configuration:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{name} expected {list(want)} got {list(got)}" for name, want, got in self.wrong_shape))
        if self.duplicates:
            lines.append(f"  in more than one file ({len(self.duplicates)}): " + ", ".join(self.duplicates))
        super().__init__("\n".join(lines))


def kept_dtype(stored: torch.dtype, ndim: int, engine_dtype: torch.dtype) -> torch.dtype:
    if not stored.is_floating_point:
        return torch.int32
    if engine_dtype == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64) and ndim < 2:
        return torch.float32
    return engine_dtype


def open_shards(model_dir) -> list[SafetensorsFile]:
    shards = sorted(Path(model_dir).glob("*.safetensors"))
    if not shards:
        raise FileNotFoundError(
            f"no *.safetensors under {str(model_dir)!r}; the model folder needs config.json "
            "and its weight files"
        )
    return [SafetensorsFile(path) for path in shards]


def load_weights(model_dir, config: ModelConfig, engine_dtype: torch.dtype, device) -> dict[str, torch.Tensor]:
    """name -> tensor on `device`; raises WeightError unless the folder fits."""
    expected = expected_tensors(config)
    head = tensor_names(config).lm_head
    where: dict[str, SafetensorsFile] = {}
    duplicates = []
    for shard in open_shards(model_dir):
        for name in shard.names():
            if name in where:
                duplicates.append(name)
            where[name] = shard

    missing = [name for name in expected if name not in where]
    if getattr(config.head, "tied", config.tie_word_embeddings) and head in missing:
        missing.remove(head)
    unexpected = [name for name in where if name not in expected]
    wrong = [
        (name, expected[name].shape, where[name].shape(name))
        for name in expected
        if name in where and tuple(where[name].shape(name)) != tuple(expected[name].shape)
    ]
    if missing or unexpected or wrong or duplicates:
        raise WeightError(model_dir, missing, unexpected, wrong, duplicates)

    tensors: dict[str, torch.Tensor] = {}
    for name in expected:
        if name not in where:
            continue
        view = where[name].tensor(name)
        target = kept_dtype(view.dtype, view.dim(), engine_dtype)
        tensors[name] = view.to(device=device, dtype=target, copy=True)
    if head not in tensors:   # tied and left out of the file: the same tensor under both names
        tensors[head] = tensors[tensor_names(config).embedding]
    return tensors
