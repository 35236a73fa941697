"""Settings shared by the entry points.

`DEFAULT_MODEL_DIR` is the folder the command line opens when `--model` is not
given; the environment variable `SHRIKE_B200_MODEL_DIR` overrides it, as
`SHRIKE_MODEL_DIR` does in Azimml/shrike (shrike/config.py:29).
"""

import os

DEFAULT_MODEL_DIR: str = os.environ.get("SHRIKE_B200_MODEL_DIR", "models_cache/qwen2.5-0.5b-instruct")
