"""SigLIP vision encoder and the Gemma-3 multimodal projector
(python/minisgl/models/gemma4_vision.py, python/minisgl/tokenizer/vision.py:48-140: the reference's
vision path is Gemma-4's; this is the same role for Gemma-3 checkpoints).

An image of ``image_size x image_size`` pixels is cut into ``patch x patch`` patches, each embedded
by one linear map (a stride-``patch`` convolution) plus a learned position embedding; ``layers``
pre-norm transformer blocks with full (bidirectional) attention and a tanh-GELU MLP follow, then
a final layer norm. The projector averages ``k x k`` neighbouring patch features down to
``tokens_per_image`` positions, applies a ``(1 + w)`` RMS norm and maps to the text width. The
result replaces the embeddings of the image's placeholder tokens in the prompt.

The tower is a few percent of a request's prefill work and runs once per image, replicated on
every tensor-parallel rank, through library GEMMs and ``scaled_dot_product_attention``; weights
are kept under their checkpoint names.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch
import torch.nn.functional as F


@dataclass
class VisionConfig:
    hidden_size: int
    intermediate_size: int
    num_layers: int
    num_heads: int
    image_size: int
    patch_size: int
    layer_norm_eps: float = 1e-6
    tokens_per_image: int = 256
    text_hidden: int = 0
    rms_norm_eps: float = 1e-6
    image_token_id: int = -1
    boi_token_id: int = -1
    eoi_token_id: int = -1

    @classmethod
    def from_hf(cls, cfg: dict) -> Optional["VisionConfig"]:
        v = cfg.get("vision_config")
        if not v or "text_config" not in cfg:
            return None
        t = cfg["text_config"]
        return cls(hidden_size=int(v["hidden_size"]), intermediate_size=int(v["intermediate_size"]),
                   num_layers=int(v["num_hidden_layers"]), num_heads=int(v["num_attention_heads"]),
                   image_size=int(v["image_size"]), patch_size=int(v["patch_size"]),
                   layer_norm_eps=float(v.get("layer_norm_eps", 1e-6)),
                   tokens_per_image=int(cfg.get("mm_tokens_per_image", 256)), text_hidden=int(t["hidden_size"]),
                   rms_norm_eps=float(t.get("rms_norm_eps", 1e-6)),
                   image_token_id=int(cfg.get("image_token_index", cfg.get("image_token_id", -1))),
                   boi_token_id=int(cfg.get("boi_token_index", cfg.get("boi_token_id", -1))),
                   eoi_token_id=int(cfg.get("eoi_token_index", cfg.get("eoi_token_id", -1))))

    @property
    def patches_per_side(self) -> int:
        return self.image_size // self.patch_size


_PREFIXES = ("model.vision_tower.", "vision_tower.", "model.multi_modal_projector.", "multi_modal_projector.")


class VisionTower:
    def __init__(self, cfg: VisionConfig, dtype, device) -> None:
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        self.w: Dict[str, torch.Tensor] = {}

    # ---- weights ----
    def load(self, path: str) -> int:
        from .weight import iter_safetensors

        for name, t in iter_safetensors(path):
            for lead in _PREFIXES:
                if name.startswith(lead):
                    key = ("proj." if "multi_modal_projector" in lead else "") + name[len(lead):]
                    self.w[key] = t.to(self.device, self.dtype)
                    break
        need = ["vision_model.embeddings.patch_embedding.weight", "proj.mm_input_projection_weight"]
        missing = [k for k in need if k not in self.w]
        if missing:
            raise KeyError(f"the checkpoint has no vision tower ({missing[0]} not found)")
        return len(self.w)

    def init_dummy(self, seed: int) -> None:
        c = self.cfg
        g = torch.Generator().manual_seed(seed)

        def rnd(*shape, std=0.02):
            return (torch.randn(*shape, generator=g) * std).to(self.device, self.dtype)

        d, i = c.hidden_size, c.intermediate_size
        self.w["vision_model.embeddings.patch_embedding.weight"] = rnd(d, 3, c.patch_size, c.patch_size)
        self.w["vision_model.embeddings.patch_embedding.bias"] = rnd(d)
        self.w["vision_model.embeddings.position_embedding.weight"] = rnd(c.patches_per_side ** 2, d)
        for l in range(c.num_layers):
            p = f"vision_model.encoder.layers.{l}."
            for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
                self.w[p + f"self_attn.{n}.weight"], self.w[p + f"self_attn.{n}.bias"] = rnd(d, d), rnd(d)
            self.w[p + "mlp.fc1.weight"], self.w[p + "mlp.fc1.bias"] = rnd(i, d), rnd(i)
            self.w[p + "mlp.fc2.weight"], self.w[p + "mlp.fc2.bias"] = rnd(d, i), rnd(d)
            for n in ("layer_norm1", "layer_norm2"):
                self.w[p + n + ".weight"] = torch.ones(d, dtype=self.dtype, device=self.device)
                self.w[p + n + ".bias"] = torch.zeros(d, dtype=self.dtype, device=self.device)
        self.w["vision_model.post_layernorm.weight"] = torch.ones(d, dtype=self.dtype, device=self.device)
        self.w["vision_model.post_layernorm.bias"] = torch.zeros(d, dtype=self.dtype, device=self.device)
        self.w["proj.mm_input_projection_weight"] = rnd(d, c.text_hidden)
        self.w["proj.mm_soft_emb_norm.weight"] = torch.zeros(d, dtype=self.dtype, device=self.device)

    # ---- compute ----
    def encode(self, pixels: torch.Tensor) -> torch.Tensor:
        """``pixels`` ``[B, 3, S, S]`` normalised → ``[B, patches, hidden]``."""
        c, w = self.cfg, self.w
        x = F.conv2d(pixels.to(self.device, self.dtype), w["vision_model.embeddings.patch_embedding.weight"],
                     w.get("vision_model.embeddings.patch_embedding.bias"), stride=c.patch_size)
        x = x.flatten(2).transpose(1, 2) + w["vision_model.embeddings.position_embedding.weight"][None]
        b, n, d = x.shape
        h = c.num_heads
        for l in range(c.num_layers):
            p = f"vision_model.encoder.layers.{l}."
            y = F.layer_norm(x, (d,), w[p + "layer_norm1.weight"], w[p + "layer_norm1.bias"], c.layer_norm_eps)
            q = F.linear(y, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.q_proj.bias"])
            k = F.linear(y, w[p + "self_attn.k_proj.weight"], w[p + "self_attn.k_proj.bias"])
            v = F.linear(y, w[p + "self_attn.v_proj.weight"], w[p + "self_attn.v_proj.bias"])
            q, k, v = (t.view(b, n, h, d // h).transpose(1, 2) for t in (q, k, v))
            a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(b, n, d)
            x = x + F.linear(a, w[p + "self_attn.out_proj.weight"], w[p + "self_attn.out_proj.bias"])
            y = F.layer_norm(x, (d,), w[p + "layer_norm2.weight"], w[p + "layer_norm2.bias"], c.layer_norm_eps)
            y = F.gelu(F.linear(y, w[p + "mlp.fc1.weight"], w[p + "mlp.fc1.bias"]), approximate="tanh")
            x = x + F.linear(y, w[p + "mlp.fc2.weight"], w[p + "mlp.fc2.bias"])
        return F.layer_norm(x, (d,), w["vision_model.post_layernorm.weight"], w["vision_model.post_layernorm.bias"],
                            c.layer_norm_eps)

    def project(self, feats: torch.Tensor) -> torch.Tensor:
        """``[B, patches, hidden]`` → ``[B, tokens_per_image, text_hidden]``."""
        c, w = self.cfg, self.w
        b, n, d = feats.shape
        side = c.patches_per_side
        out_side = int(round(c.tokens_per_image ** 0.5))
        x = feats.transpose(1, 2).reshape(b, d, side, side)
        x = F.avg_pool2d(x, kernel_size=side // out_side, stride=side // out_side).flatten(2).transpose(1, 2)
        xf = x.float()
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + c.rms_norm_eps)
        xf = xf * (1.0 + w["proj.mm_soft_emb_norm.weight"].float())
        return torch.matmul(xf.to(self.dtype), w["proj.mm_input_projection_weight"])

    def image_embeddings(self, pixels: torch.Tensor) -> torch.Tensor:
        """``[B, 3, S, S]`` → ``[B * tokens_per_image, text_hidden]`` in prompt order."""
        out = self.project(self.encode(pixels))
        return out.reshape(-1, out.shape[-1])
