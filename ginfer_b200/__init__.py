"""ginfer_b200: a small, whole LLM inference engine for one B200 (sm_100a).

Token ids in, token ids out: typed configuration and an architecture registry, safetensors
loading and random weights, layers put together from parts, a paged cache manager with
per-request state slots, one step function over mixed batches, a continuous-batching scheduler,
greedy and temperature sampling, hand-written CUDA kernels, a true 32-bit path, and trace replay.
"""
__version__ = "0.1.0"

from . import architectures  # noqa: F401  (registers the known architectures)
