"""Model sizes as data: one config.json per named shape, for random-weights runs.

A "shape" is a config.json of a registered architecture without a checkpoint behind it.
`--random NAME` on the command line, the one-prompt program and the benchmark read the
file `NAME.json` of this folder (or any path to a config.json, or to a folder holding
one) and fill the model with seeded random weights.  No size lives in code: the engine
reads these files exactly as it reads a checkpoint's config.json.  Azimml/shrike has no
such mode (it always opens a downloaded snapshot, shrike/config.py:21-29).
"""

from __future__ import annotations

import json
from pathlib import Path

FOLDER = Path(__file__).resolve().parent


def known_shapes() -> list[str]:
    return sorted(path.stem for path in FOLDER.glob("*.json"))


def shape_config(name_or_path: str) -> dict:
    """The raw config.json dictionary of a named shape, a config.json file or a model folder."""
    text = str(name_or_path)
    for candidate in (FOLDER / f"{text}.json", FOLDER / f"qwen2.5-{text}.json", Path(text), Path(text) / "config.json"):
        if candidate.is_file():
            return json.loads(candidate.read_text())
    raise FileNotFoundError(
        f"no shape {text!r}: give one of {', '.join(known_shapes())}, or the path of a config.json")
