"""B200-native LLM serving engine (sm_100a) with the capabilities of mini-SGLang's RDNA4 fork."""
from .core import SamplingParams

__version__ = "0.1.0"


def __getattr__(name):
    if name == "LLM":
        from .llm import LLM

        return LLM
    raise AttributeError(name)


__all__ = ["LLM", "SamplingParams", "__version__"]
