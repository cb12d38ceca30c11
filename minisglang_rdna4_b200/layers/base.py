"""Minimal module system: tensors are parameters, ``BaseOP`` attributes are children.

Same state-dict protocol as python/minisgl/layers/base.py:92 — names are dotted attribute
paths, lists of ops are indexed (``layers.3.mlp.down_proj.weight``) — without autograd.
``post_load`` runs after the checkpoint has been copied in and is where a layer repacks
weights into the layout its kernels want.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Iterator, List, Tuple

import torch


class BaseOP:
    # attribute names that are tensors but not checkpoint parameters
    _non_persistent: Tuple[str, ...] = ()

    def _children(self) -> Iterator[Tuple[str, "BaseOP"]]:
        for name, value in vars(self).items():
            if name.startswith("_"):
                continue
            if isinstance(value, BaseOP):
                yield name, value
            elif isinstance(value, (list, tuple)) and value and all(isinstance(v, BaseOP) for v in value):
                for i, child in enumerate(value):
                    yield f"{name}.{i}", child

    def _params(self) -> Iterator[Tuple[str, torch.Tensor]]:
        for name, value in vars(self).items():
            if name.startswith("_") or name in self._non_persistent:
                continue
            if isinstance(value, torch.Tensor):
                yield name, value

    def named_parameters(self, prefix: str = "") -> Iterator[Tuple[str, torch.Tensor, "BaseOP", str]]:
        for name, tensor in self._params():
            yield prefix + name, tensor, self, name
        for cname, child in self._children():
            yield from child.named_parameters(prefix + cname + ".")

    def state_dict(self) -> Dict[str, torch.Tensor]:
        return {name: tensor for name, tensor, _, _ in self.named_parameters()}

    def load_state_dict(self, state: Dict[str, torch.Tensor], strict: bool = True) -> List[str]:
        """Copy ``state`` in (replacing meta tensors). Returns the names that were missing."""
        missing: List[str] = []
        used = set()
        for name, tensor, owner, attr in self.named_parameters():
            src = state.get(name)
            if src is None:
                missing.append(name)
                continue
            used.add(name)
            if tuple(src.shape) != tuple(tensor.shape):
                raise ValueError(f"{name}: checkpoint shape {tuple(src.shape)} != model {tuple(tensor.shape)}")
            if tensor.device.type == "meta":
                setattr(owner, attr, src.to(tensor.dtype))
            else:
                tensor.copy_(src)
        if strict:
            extra = sorted(set(state) - used)
            if missing or extra:
                raise KeyError(f"state dict mismatch: missing={missing[:8]} unexpected={extra[:8]}")
        return missing

    def apply_to_tensors(self, fn: Callable[[torch.Tensor], torch.Tensor]) -> "BaseOP":
        for name, value in list(vars(self).items()):
            if isinstance(value, torch.Tensor):
                setattr(self, name, fn(value))
        for _, child in self._children():
            child.apply_to_tensors(fn)
        return self

    def to(self, device: Any) -> "BaseOP":
        return self.apply_to_tensors(lambda t: t.to(device))

    def modules(self) -> Iterator["BaseOP"]:
        yield self
        for _, child in self._children():
            yield from child.modules()

    def post_load(self) -> None:
        """Hook: convert loaded checkpoint tensors to kernel layouts. Children first."""
        for _, child in self._children():
            child.post_load()
        self._post_load_self()

    def _post_load_self(self) -> None:
        return None
