"""Benchmark helpers: kernel micro-benchmarks (``kernels.py``) and an OpenAI-API load client
(``client.py``), the counterparts of python/minisgl/benchmark/perf.py and client.py."""
