"""A B200-native inference engine for Gemma 1: from a model folder to generated tokens on one GPU."""
__version__ = "0.1.0"

from .sampling.params import SamplingParams

__all__ = ["LLM", "SamplingParams", "RequestOutput"]


def __getattr__(name):
    if name in ("LLM", "RequestOutput"):
        from . import llm
        return getattr(llm, name)
    raise AttributeError(f"module 'wllm_b200' has no attribute {name!r}")
