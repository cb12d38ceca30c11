"""Recursive self-aggregation (RSA) on top of the chat API (python/minisgl/rsa/core.py:427,
config.py:157-228): N parallel rollouts, T rounds in which each rollout is rewritten from K
sampled peers, and a final selection."""
from .core import RSAParams, run_rsa

__all__ = ["RSAParams", "run_rsa"]
