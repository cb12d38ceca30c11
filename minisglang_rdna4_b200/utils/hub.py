"""Model paths that name a hub repository instead of a directory
(python/minisgl/utils/hf.py ``download_hf_weight`` / ``cached_load_hf_config``).

``resolve_model_path`` leaves directories and the built-in benchmark shapes alone. Anything that looks like
``owner/name`` is looked up in the local hub cache first (no network needed for a model that was fetched
before); only then is a download attempted, config / tokenizer / safetensors files only. ``HF_HUB_OFFLINE=1``
or ``MSGL_HUB_OFFLINE=1`` forbids the attempt. A failure says what was tried instead of surfacing later as a
missing ``config.json``.
"""
from __future__ import annotations

import os
import re
from typing import Optional

_REPO = re.compile(r"^[A-Za-z0-9][\w.\-]*/[\w.\-]+$")
PATTERNS = ["*.json", "*.safetensors", "*.model", "*.txt", "*.jinja", "tokenizer*"]


def looks_like_repo(name: str) -> bool:
    return bool(name) and not os.path.exists(name) and bool(_REPO.match(name))


def resolve_model_path(name: Optional[str], revision: Optional[str] = None) -> Optional[str]:
    if not name or os.path.isdir(name) or not looks_like_repo(name):
        return name
    from ..models.config import NAMED_CONFIGS

    if name in NAMED_CONFIGS:
        return name
    try:
        from huggingface_hub import snapshot_download
    except ImportError as exc:               # pragma: no cover - the package ships with transformers
        raise FileNotFoundError(f"{name!r} is not a directory and huggingface_hub is not installed") from exc
    try:
        return snapshot_download(name, revision=revision, allow_patterns=PATTERNS, local_files_only=True)
    except Exception:
        pass
    from ..env import ENV

    if os.environ.get("HF_HUB_OFFLINE") == "1" or ENV.HUB_OFFLINE.value:
        raise FileNotFoundError(f"{name!r} is not a directory, is not in the local hub cache, and downloads are off")
    try:
        return snapshot_download(name, revision=revision, allow_patterns=PATTERNS)
    except Exception as exc:
        raise FileNotFoundError(f"{name!r} is not a directory, is not in the local hub cache, and could not be "
                                f"downloaded ({type(exc).__name__}: {exc})") from exc
