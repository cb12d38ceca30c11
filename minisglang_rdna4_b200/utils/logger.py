"""Process-wide logging with rank-aware helpers.

Behaviour follows python/minisgl/utils/logger.py: one stream handler, a per-process suffix
(for example ``dp0|tp1``) and ``info_rank0`` / ``warning_rank0`` helpers that stay quiet on
every rank but the first.
"""
from __future__ import annotations

import logging
import os
import sys
from typing import Optional

_SUFFIX: str = ""
_CONFIGURED = False


class _RankLogger(logging.LoggerAdapter):
    def process(self, msg, kwargs):
        return (f"[{_SUFFIX}] {msg}" if _SUFFIX else msg), kwargs

    @staticmethod
    def _is_rank0() -> bool:
        from ..parallel.info import try_get_tp_info

        info = try_get_tp_info()
        return info is None or info.rank == 0

    def info_rank0(self, msg, *args, **kwargs):
        if self._is_rank0():
            self.info(msg, *args, **kwargs)

    def warning_rank0(self, msg, *args, **kwargs):
        if self._is_rank0():
            self.warning(msg, *args, **kwargs)

    def debug_rank0(self, msg, *args, **kwargs):
        if self._is_rank0():
            self.debug(msg, *args, **kwargs)


def init_logger(name: str, suffix: Optional[str] = None) -> _RankLogger:
    global _SUFFIX, _CONFIGURED
    if suffix is not None:
        _SUFFIX = suffix
    if not _CONFIGURED:
        level = os.environ.get("MSGL_LOG_LEVEL", os.environ.get("LOG_LEVEL", "INFO")).upper()
        handler = logging.StreamHandler(sys.stderr)
        handler.setFormatter(
            logging.Formatter("%(asctime)s %(levelname).1s %(name)s: %(message)s", "%H:%M:%S")
        )
        root = logging.getLogger("msgl")
        root.handlers[:] = [handler]
        root.setLevel(getattr(logging, level, logging.INFO))
        root.propagate = False
        _CONFIGURED = True
    short = name.replace("minisglang_rdna4_b200", "msgl")
    if not short.startswith("msgl"):
        short = "msgl." + short
    return _RankLogger(logging.getLogger(short), {})
