"""Random weights from a configuration and a seed.

Azimml/shrike always loads a real snapshot; this mode exists so that tests and
benchmarks need no network.  Matrices and tables are N(0, 0.02), biases N(0, 0.02),
norm weights 1 + N(0, 0.1).  Each tensor has its own stream, seeded from the seed
and the tensor's name, so a tensor's values do not depend on which others exist.

    python -m shrike_b200.weights.random_init --config config.json --seed 0 --out DIR
"""

from __future__ import annotations

import argparse
import json
import zlib
from pathlib import Path

import torch

from ..config.registry import parse_config
from .expected import expected_tensors, tensor_names
from .safetensors_io import write_safetensors

_TORCH_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _tensor_seed(seed: int, name: str) -> int:
    return (int(seed) * 0x9E3779B1 + zlib.crc32(name.encode())) & 0x7FFFFFFFFFFFFFFF


def random_tensor(name: str, spec, seed: int, device="cpu", dtype=torch.float32) -> torch.Tensor:
    generator = torch.Generator(device=device)
    generator.manual_seed(_tensor_seed(seed, name))
    values = torch.randn(spec.shape, generator=generator, device=device, dtype=torch.float32)
    if spec.init == "norm":
        values = 1.0 + 0.1 * values
    else:
        values = 0.02 * values
    return values.to(dtype)


def random_tensors(config, seed: int, device="cpu", dtype=torch.float32) -> dict[str, torch.Tensor]:
    """name -> tensor; a tied model gets no separate LM head."""
    head = tensor_names(config).lm_head
    tensors = {}
    for name, spec in expected_tensors(config).items():
        if name == head and getattr(config.head, "tied", config.tie_word_embeddings):
            continue
        tensors[name] = random_tensor(name, spec, seed, device, dtype)
    return tensors


def write_model_folder(out_dir, raw_config: dict, seed: int, dtype: str = "float32") -> Path:
    """Writes `config.json` and `model.safetensors`; returns the folder."""
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    raw = dict(raw_config)
    raw["torch_dtype"] = dtype
    config = parse_config(raw)
    tensors = random_tensors(config, seed, "cpu", _TORCH_DTYPES[dtype])
    (out / "config.json").write_text(json.dumps(raw, indent=2) + "\n")
    write_safetensors(out / "model.safetensors", tensors, {"format": "pt", "seed": seed})
    return out


def main(argv=None) -> None:
    parser = argparse.ArgumentParser(description="Write a model folder with random weights")
    parser.add_argument("--config", required=True, help="a config.json of the architecture")
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--dtype", default="float32", choices=sorted(_TORCH_DTYPES))
    parser.add_argument("--out", required=True)
    args = parser.parse_args(argv)
    raw = json.loads(Path(args.config).read_text())
    folder = write_model_folder(args.out, raw, args.seed, args.dtype)
    print(f"wrote {folder}/config.json and model.safetensors (seed {args.seed}, {args.dtype})")


if __name__ == "__main__":
    main()
