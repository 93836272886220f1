"""purhie_b200: a small, whole LLM inference engine for one NVIDIA B200 (sm_100a).

Model folder (config.json + safetensors, or seeded random weights) -> tokens, for the Qwen3 dense
decoder, built from parts: typed configuration and registry (:mod:`.config`), weights by name
(:mod:`.weights`), layers composed from mixer / feed-forward / norm / position encoding
(:mod:`.parts`), a paged cache manager (:mod:`.cache`), one step function and a scheduler
(:mod:`.engine`), sampling (:mod:`.sampling`) and hand-written CUDA kernels (:mod:`.csrc`).
"""
from . import config as config            # registers the architectures

__version__ = "0.1.0"
