"""Built-in byte-level tokenizer for runs without a Hugging Face tokenizer on disk (named
benchmark shapes, tests): ids 0..255 are bytes, followed by a few special tokens. It offers
the small slice of the ``transformers`` tokenizer API that the workers use."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence


class ByteTokenizer:
    bos_token_id = 256
    eos_token_id = 257
    pad_token_id = 258
    vocab_size = 260
    chat_template = "byte-chatml"

    def __init__(self, eos_token_id: Optional[int] = None) -> None:
        if eos_token_id is not None:
            self.eos_token_id = eos_token_id

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        ids = list(text.encode("utf-8"))
        return ([self.bos_token_id] + ids) if add_special_tokens else ids

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        data = bytes(i for i in ids if 0 <= i < 256)
        return data.decode("utf-8", errors="replace")

    def convert_ids_to_tokens(self, ids: Sequence[int]) -> List[str]:
        return [chr(i) if i < 256 else f"<|{i}|>" for i in ids]

    def apply_chat_template(self, messages: List[Dict[str, Any]], tokenize: bool = False,
                            add_generation_prompt: bool = True, **kwargs: Any):
        parts = []
        for m in messages:
            content = m.get("content") or ""
            if isinstance(content, list):
                content = "".join(p.get("text", "") for p in content if isinstance(p, dict))
            parts.append(f"<|im_start|>{m.get('role', 'user')}\n{content}<|im_end|>\n")
        if add_generation_prompt:
            parts.append("<|im_start|>assistant\n")
        text = "".join(parts)
        return self.encode(text) if tokenize else text


def load_tokenizer(model_path: str):
    """Hugging Face tokenizer when ``model_path`` has one, else the byte tokenizer."""
    import os

    if model_path and os.path.isdir(model_path) and any(
            os.path.exists(os.path.join(model_path, f)) for f in ("tokenizer.json", "tokenizer_config.json",
                                                                  "tokenizer.model")):
        from transformers import AutoTokenizer

        from ..utils.hf import apply_chat_template_sources

        return apply_chat_template_sources(AutoTokenizer.from_pretrained(model_path), model_path)
    return ByteTokenizer()
