"""Side files of a Hugging Face checkpoint directory (python/minisgl/utils/hf.py:45-256):
``generation_config.json`` (the author's stop tokens and sampling defaults), chat templates
shipped next to the tokenizer, and the served model's chat-template override. Local
directories only: nothing here talks to the hub.
"""
from __future__ import annotations

import functools
import json
import os
from typing import Any, Dict, Iterable, List, Optional

_SAMPLING_KEYS = ("temperature", "top_p", "top_k", "min_p", "repetition_penalty")


def _read_json(path: str) -> Dict[str, Any]:
    try:
        with open(path, encoding="utf-8") as fh:
            data = json.load(fh)
        return data if isinstance(data, dict) else {}
    except (OSError, ValueError):
        return {}


@functools.lru_cache(maxsize=32)
def load_generation_config(model_path: str) -> Dict[str, Any]:
    """``generation_config.json`` as a dict ({} when absent or unreadable)."""
    if not model_path or not os.path.isdir(model_path):
        return {}
    return _read_json(os.path.join(model_path, "generation_config.json"))


def sampling_defaults(model_path: str) -> Dict[str, float]:
    """The sampling parameters the model's author recommends; applied to requests that leave
    them unset (a checkpoint served with top_p = 1, top_k = -1 when its card says 0.95 / 64
    samples from the whole distribution)."""
    gen = load_generation_config(model_path)
    if gen.get("do_sample") is False:
        return {"temperature": 0.0}
    return {k: gen[k] for k in _SAMPLING_KEYS if isinstance(gen.get(k), (int, float))}


def resolve_stop_token_ids(model_path: str, tokenizer: Any = None, config_eos: Iterable[int] = ()) -> List[int]:
    """Every end-of-generation id, in a stable order and without duplicates: the list in
    ``generation_config.json`` (int or list: the serving list, e.g. three ids for Llama-3 and
    GLM-4 chat models), the tokenizer's single ``eos_token_id``, the model config's. A chat model
    whose turns end with a token other than the tokenizer's EOS never stops unless all of them
    count."""
    ids: List[int] = []

    def add(v) -> None:
        for t in v if isinstance(v, (list, tuple)) else [v]:
            if isinstance(t, int) and not isinstance(t, bool) and t >= 0 and t not in ids:
                ids.append(t)

    add(load_generation_config(model_path).get("eos_token_id"))
    add(getattr(tokenizer, "eos_token_id", None))
    add(list(config_eos))
    return ids


def side_chat_template(model_path: str) -> Optional[str]:
    """A template shipped as ``chat_template.json`` ({"chat_template": ...}) or ``chat_template.jinja``."""
    if not model_path or not os.path.isdir(model_path):
        return None
    tpl = _read_json(os.path.join(model_path, "chat_template.json")).get("chat_template")
    if isinstance(tpl, str) and tpl:
        return tpl
    try:
        with open(os.path.join(model_path, "chat_template.jinja"), encoding="utf-8") as fh:
            return fh.read() or None
    except OSError:
        return None


def chat_template_override(model_path: str) -> Optional[str]:
    """``MSGL_CHAT_TEMPLATE`` (a file path or a literal Jinja string) applies to the tokenizer of
    ``MSGL_CHAT_TEMPLATE_MODEL`` only, so every process that loads the served tokenizer gets the
    same template while drafters' and calibrators' tokenizers stay untouched."""
    from ..env import ENV

    spec, model = ENV.CHAT_TEMPLATE.value, ENV.CHAT_TEMPLATE_MODEL.value
    if not spec or model != model_path:
        return None
    if os.path.isfile(spec):
        with open(spec, encoding="utf-8") as fh:
            return fh.read()
    return spec


def apply_chat_template_sources(tokenizer: Any, model_path: str) -> Any:
    """Give the tokenizer the template it should use: the override, else its own, else a side file."""
    tpl = chat_template_override(model_path)
    if tpl is None and not getattr(tokenizer, "chat_template", None):
        tpl = side_chat_template(model_path)
    if tpl is not None:
        try:
            tokenizer.chat_template = tpl
        except AttributeError:
            pass
    return tokenizer
