from .detokenize import DetokenizeManager
from .simple import ByteTokenizer, load_tokenizer
from .tokenize import TokenizeManager

__all__ = ["DetokenizeManager", "ByteTokenizer", "load_tokenizer", "TokenizeManager"]
