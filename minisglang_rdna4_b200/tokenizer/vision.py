"""Image preprocessing for multimodal prompts (python/minisgl/tokenizer/vision.py:48-140).

An image (an encoded file, a PIL image or a tensor) becomes a ``[3, S, S]`` uint8 tensor: RGB,
resized to the tower's square input with bilinear resampling. Normalisation to ``[-1, 1]`` happens
on the device next to the tower. In the prompt every image is one run of ``tokens_per_image``
placeholder tokens between a begin and an end marker; ``expand_placeholders`` turns each begin
marker the chat template emitted into that run.
"""
from __future__ import annotations

import base64
import io
from typing import List, Sequence, Union

import torch


class VisionPreprocessor:
    def __init__(self, image_size: int, tokens_per_image: int, image_token_id: int, boi_token_id: int,
                 eoi_token_id: int) -> None:
        self.image_size, self.tokens_per_image = int(image_size), int(tokens_per_image)
        self.image_token_id, self.boi_token_id, self.eoi_token_id = int(image_token_id), int(boi_token_id), int(eoi_token_id)

    @classmethod
    def from_vision_config(cls, vc) -> "VisionPreprocessor":
        return cls(vc.image_size, vc.tokens_per_image, vc.image_token_id, vc.boi_token_id, vc.eoi_token_id)

    # ---- pixels ----
    def load(self, image) -> torch.Tensor:
        """``image``: bytes of an encoded file, a ``data:`` URL, a PIL image, or a ``[3, H, W]`` /
        ``[H, W, 3]`` uint8 tensor."""
        from PIL import Image
        import numpy as np

        if isinstance(image, str):
            if not image.startswith("data:"):
                raise ValueError("only data: URLs are accepted for images (this server fetches nothing)")
            image = base64.b64decode(image.split(",", 1)[1])
        if isinstance(image, (bytes, bytearray)):
            image = Image.open(io.BytesIO(image))
        if isinstance(image, torch.Tensor):
            t = image
            if t.dim() == 3 and t.shape[0] == 3:
                t = t.permute(1, 2, 0)
            image = Image.fromarray(t.to(torch.uint8).cpu().numpy())
        image = image.convert("RGB").resize((self.image_size, self.image_size), Image.BILINEAR)
        return torch.from_numpy(np.asarray(image).copy()).permute(2, 0, 1).contiguous()

    def batch(self, images: Sequence) -> torch.Tensor:
        return torch.stack([self.load(im) for im in images])

    # ---- tokens ----
    def expand_placeholders(self, ids: Sequence[int], n_images: int) -> List[int]:
        """Every begin-of-image marker becomes ``begin, placeholder x tokens_per_image, end``."""
        out: List[int] = []
        seen = 0
        run = [self.image_token_id] * self.tokens_per_image
        for t in ids:
            if int(t) == self.boi_token_id:
                out += [self.boi_token_id] + run + [self.eoi_token_id]
                seen += 1
            else:
                out.append(int(t))
        if seen != n_images:
            raise ValueError(f"the prompt has {seen} image marker(s) for {n_images} image(s)")
        return out
