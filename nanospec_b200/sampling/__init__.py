"""Token choice: greedy, temperature, top-k and top-p, as the reference samples
(spec/sampling.py:24-42; engine/engine.py:385-402).  The work is done by one CUDA kernel
(csrc/sampling.cu) over float32 logits; this package holds its options and its Python face."""

from ..engine.scheduler import SamplingParams, TokenInfo
from ..ops import sample_rows

__all__ = ["SamplingParams", "TokenInfo", "sample_rows"]
