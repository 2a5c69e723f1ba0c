"""nanospec_b200: a small, whole, single-GPU inference engine for the Llama 3 dense decoder
on NVIDIA B200 (sm_100a): typed configuration and registry, safetensors weights, layers
assembled from parts, a paged cache manager, one step function for mixed batches, a
continuous-batching scheduler, sampling, trace replay, and hand-written CUDA kernels."""

from .config import EngineConfig, LlamaConfig
from .weights import load_model, random_model, write_random_model

__all__ = ["EngineConfig", "LlamaConfig", "load_model", "random_model", "write_random_model"]
__version__ = "0.1.0"
