"""shrike_b200: a single-GPU inference engine for the Qwen2 dense decoder on B200.

Paged key/value cache, continuous batching with chunked prefill, hand-written
sm_100a kernels.  `SamplingParams` is re-exported here because it is light (no
torch import, as in Azimml/shrike's shrike/__init__.py:13-22); `LLMEngine` lives in
`shrike_b200.engine.llm_engine`.
"""

from .engine.request import SamplingParams

__version__ = "0.1.0"
__all__ = ["SamplingParams", "__version__"]
