"""Makes tests/golden/reference_logits.npz from Azimml/shrike's own model code.

Run once, on the CPU, from the repository root:

    python tests/golden/make_golden.py /path/to/shrike

It writes tiny model folders with this package's random-weights writer, loads them
with the reference's `QwenForCausalLM.load(dir, device="cpu")` in float32, runs
whole sequences through its `NaiveKVBackend` (shrike/models/qwen.py:218-249) and
stores the logits with a checksum of the weights.  `tests/test_plain.py` then
checks the plain implementation against these numbers.  Only configurations the
reference can express are included (tiny A and B; it has no key window).
"""

import hashlib
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from tests.helpers import make_model_folder, random_tokens, read_weights  # noqa: E402
from tests.tiny_configs import TINY  # noqa: E402

LENGTHS = {"A": [5, 17, 33], "B": [1, 9, 40, 70]}


def weights_checksum(weights: dict) -> str:
    h = hashlib.sha256()
    for name in sorted(weights):
        h.update(name.encode())
        h.update(weights[name].contiguous().numpy().tobytes())
    return h.hexdigest()


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <checkout of Azimml/shrike>")
    reference = sys.argv[1]
    sys.path.insert(0, reference)
    from shrike.models.qwen import NaiveKVBackend, QwenForCausalLM

    arrays = {}
    with tempfile.TemporaryDirectory() as tmp:
        for key, lengths in LENGTHS.items():
            folder = make_model_folder(tmp, key)
            model = QwenForCausalLM.load(str(folder), device="cpu")
            arrays[f"{key}_checksum"] = np.frombuffer(weights_checksum(read_weights(folder)).encode(), dtype=np.uint8)
            for index, n in enumerate(lengths):
                ids = random_tokens(TINY[key]["vocab_size"], n, 1000 + index)
                with torch.inference_mode():
                    logits = model(torch.tensor(ids), torch.arange(n), NaiveKVBackend(model.cfg))
                arrays[f"{key}_{n}"] = logits.numpy().astype(np.float32)
    out = Path(__file__).with_name("reference_logits.npz")
    np.savez_compressed(out, **arrays)
    print("wrote", out, {k: v.shape for k, v in arrays.items()})


if __name__ == "__main__":
    main()
