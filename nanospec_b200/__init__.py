"""nanospec_b200: a small, whole, single-GPU inference engine for the Llama 3 dense decoder
on NVIDIA B200 (sm_100a): typed configuration and registry, safetensors weights, layers
assembled from parts, a paged cache manager, one step function for mixed batches, a
continuous-batching scheduler, sampling, trace replay, and hand-written CUDA kernels.

    from nanospec_b200 import Engine, EngineConfig, SamplingParams, load_model
    model = load_model("path/to/folder", device="cuda", dtype=torch.bfloat16)
    engine = Engine(model, EngineConfig(num_blocks=4096, block_size=16))
    outputs = engine.generate([[1, 2, 3]], SamplingParams(max_tokens=32))
"""

from .config import EngineConfig, LlamaConfig
from .engine import Engine, Request, SamplingParams
from .weights import load_model, random_model, write_random_model

__all__ = ["Engine", "EngineConfig", "LlamaConfig", "Request", "SamplingParams", "load_model", "random_model",
           "write_random_model"]
__version__ = "0.1.0"
