from . import llama  # registers LlamaForCausalLM

__all__ = ["llama"]
