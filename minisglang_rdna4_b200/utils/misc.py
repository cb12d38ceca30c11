"""Integer helpers, a name registry and NVTX range helpers."""
from __future__ import annotations

import contextlib
import functools
from typing import Callable, Dict, Generic, Iterator, List, TypeVar

T = TypeVar("T")


class Unset:
    """Sentinel type for "argument not given" where None is a meaningful value."""

    _inst = None

    def __new__(cls):
        if cls._inst is None:
            cls._inst = super().__new__(cls)
        return cls._inst

    def __repr__(self) -> str:
        return "UNSET"

    def __bool__(self) -> bool:
        return False


UNSET = Unset()


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


def align_ceil(a: int, b: int) -> int:
    return cdiv(a, b) * b


def align_down(a: int, b: int) -> int:
    return (a // b) * b


def next_pow2(n: int) -> int:
    return 1 if n <= 1 else 1 << (n - 1).bit_length()


def div_even(a: int, b: int, allow_replicate: bool = False) -> int:
    """``a / b`` where the division must be exact. With ``allow_replicate`` a smaller ``a``
    that divides ``b`` yields 1: that is how KV heads are replicated when there are fewer of
    them than tensor-parallel ranks (python/minisgl/utils/misc.py:20)."""
    if allow_replicate and a < b:
        if b % a != 0:
            raise ValueError(f"{b} ranks cannot replicate {a} heads evenly")
        return 1
    if a % b != 0:
        raise ValueError(f"{a} is not divisible by {b}")
    return a // b


def call_if_main(name: str) -> Callable[[Callable[[], None]], Callable[[], None]]:
    def deco(fn: Callable[[], None]) -> Callable[[], None]:
        if name == "__main__":
            fn()
        return fn

    return deco


class Registry(Generic[T]):
    """String → object table with a decorator form; duplicate names are an error."""

    def __init__(self, kind: str) -> None:
        self.kind = kind
        self._items: Dict[str, T] = {}

    def register(self, *names: str) -> Callable[[T], T]:
        def deco(obj: T) -> T:
            for name in names:
                if name in self._items:
                    raise KeyError(f"{self.kind} {name!r} registered twice")
                self._items[name] = obj
            return obj

        return deco

    def __getitem__(self, name: str) -> T:
        try:
            return self._items[name]
        except KeyError:
            raise KeyError(
                f"unknown {self.kind} {name!r}; known: {', '.join(sorted(self._items))}"
            ) from None

    def __contains__(self, name: str) -> bool:
        return name in self._items

    def names(self) -> List[str]:
        return sorted(self._items)


@contextlib.contextmanager
def nvtx_range(name: str) -> Iterator[None]:
    """NVTX range when CUDA is up, otherwise nothing. The reference decorates layers with
    ``nvtx_annotate`` (python/minisgl/utils/torch_utils.py:23)."""
    import torch

    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


def nvtx_annotate(name: str):
    def deco(fn):
        @functools.wraps(fn)
        def wrapped(*args, **kwargs):
            with nvtx_range(name):
                return fn(*args, **kwargs)

        return wrapped

    return deco
