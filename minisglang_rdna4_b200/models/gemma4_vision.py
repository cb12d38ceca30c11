"""Gemma-4 vision tower and its projector into the text model (python/minisgl/models/gemma4_vision.py:1-225).

An image is cut into ``patch x patch`` pixel patches (flattened row, column, channel); each patch is
projected and gets the sum of two learned position rows, one for its column and one for its row. The
encoder layers are the text model's layer in miniature (sandwich norms, GeGLU, weighted q/k norms and a
weight-less v norm, softmax scale 1, attention in both directions) with a two-dimensional rotary embedding:
the first half of every head rotates with the patch's column, the second half with its row. The patch grid
is averaged ``k x k`` into soft tokens, scaled by sqrt(hidden), optionally standardised, RMS-normalised
without a weight and projected to the text width.

Images are resized to one square whose patch grid gives the configured number of soft tokens; the
published preprocessor keeps the aspect ratio and so yields a varying token count per image, which this
pipeline (one token run length per model) does not. The tower itself takes any grid.

Tensor ops and library GEMMs, replicated on every rank, once per image at admission (like the
Gemma-3 tower in ``siglip.py``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch
import torch.nn.functional as F


@dataclass
class Gemma4VisionConfig:
    hidden_size: int
    intermediate_size: int
    num_layers: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    patch_size: int
    pooling: int
    position_rows: int
    rope_theta: float
    rms_norm_eps: float
    clipped: bool
    standardize: bool
    text_hidden: int
    image_size: int            # side of the square every image is resized to
    tokens_per_image: int
    image_token_id: int = -1
    boi_token_id: int = -1
    eoi_token_id: int = -1
    kind: str = "gemma4"

    @classmethod
    def from_hf(cls, cfg: dict) -> Optional["Gemma4VisionConfig"]:
        v = cfg.get("vision_config")
        if not v or "text_config" not in cfg:
            return None
        heads = int(v["num_attention_heads"])
        pool, patch = int(v.get("pooling_kernel_size", 3)), int(v.get("patch_size", 16))
        budget = int(cfg.get("vision_soft_tokens_per_image") or v.get("default_output_length") or 280)
        side = max(1, int(budget ** 0.5))                     # soft tokens per side of the square grid
        rope = v.get("rope_parameters") or {}
        return cls(hidden_size=int(v["hidden_size"]), intermediate_size=int(v["intermediate_size"]),
                   num_layers=int(v["num_hidden_layers"]), num_heads=heads,
                   num_kv_heads=int(v.get("num_key_value_heads") or heads),
                   head_dim=int(v.get("head_dim") or int(v["hidden_size"]) // heads), patch_size=patch, pooling=pool,
                   position_rows=int(v.get("position_embedding_size", 10240)),
                   rope_theta=float(rope.get("rope_theta", 100.0)), rms_norm_eps=float(v.get("rms_norm_eps", 1e-6)),
                   clipped=bool(v.get("use_clipped_linears", False)), standardize=bool(v.get("standardize", False)),
                   text_hidden=int(cfg["text_config"]["hidden_size"]), image_size=side * pool * patch,
                   tokens_per_image=side * side, image_token_id=int(cfg.get("image_token_id", -1)),
                   boi_token_id=int(cfg.get("boi_token_id", -1)), eoi_token_id=int(cfg.get("eoi_token_id", -1)))


_LEADS = (("model.vision_tower.", ""), ("vision_tower.", ""), ("model.embed_vision.", "embed."), ("embed_vision.", "embed."))


def _rms(x: torch.Tensor, eps: float, w: Optional[torch.Tensor] = None) -> torch.Tensor:
    xf = x.float()
    xf = xf * torch.pow(xf.pow(2).mean(-1, keepdim=True) + eps, -0.5)
    if w is not None:
        xf = xf * w.float()
    return xf.to(x.dtype)


class Gemma4VisionTower:
    def __init__(self, cfg: Gemma4VisionConfig, dtype, device) -> None:
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        self.w: Dict[str, torch.Tensor] = {}

    # ---- weights ----
    def load(self, path: str) -> int:
        from .weight import iter_safetensors

        for name, t in iter_safetensors(path):
            for lead, to in _LEADS:
                if name.startswith(lead):
                    self.w[to + name[len(lead):]] = t.to(self.device, self.dtype if t.is_floating_point() else t.dtype)
                    break
        for key in ("patch_embedder.input_proj.weight", "embed.embedding_projection.weight"):
            if key not in self.w:
                raise KeyError(f"the checkpoint has no vision tower ({key} not found)")
        return len(self.w)

    def init_dummy(self, seed: int) -> None:
        c = self.cfg
        g = torch.Generator().manual_seed(seed)
        rnd = lambda *shape: (torch.randn(*shape, generator=g) * 0.02).to(self.device, self.dtype)
        one = lambda n: torch.ones(n, dtype=self.dtype, device=self.device)
        d, i, hd = c.hidden_size, c.intermediate_size, c.head_dim
        self.w["patch_embedder.input_proj.weight"] = rnd(d, 3 * c.patch_size ** 2)
        self.w["patch_embedder.position_embedding_table"] = rnd(2, c.position_rows, d)
        for l in range(c.num_layers):
            p = f"encoder.layers.{l}."
            self.w[p + "self_attn.q_proj.linear.weight"] = rnd(c.num_heads * hd, d)
            self.w[p + "self_attn.k_proj.linear.weight"] = rnd(c.num_kv_heads * hd, d)
            self.w[p + "self_attn.v_proj.linear.weight"] = rnd(c.num_kv_heads * hd, d)
            self.w[p + "self_attn.o_proj.linear.weight"] = rnd(d, c.num_heads * hd)
            self.w[p + "self_attn.q_norm.weight"], self.w[p + "self_attn.k_norm.weight"] = one(hd), one(hd)
            self.w[p + "mlp.gate_proj.linear.weight"], self.w[p + "mlp.up_proj.linear.weight"] = rnd(i, d), rnd(i, d)
            self.w[p + "mlp.down_proj.linear.weight"] = rnd(d, i)
            for n in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm",
                      "post_feedforward_layernorm"):
                self.w[p + n + ".weight"] = one(d)
        self.w["embed.embedding_projection.weight"] = rnd(c.text_hidden, d)

    # ---- compute ----
    def _linear(self, x: torch.Tensor, name: str) -> torch.Tensor:
        w = self.w
        if self.cfg.clipped and (name + ".input_min") in w:
            x = torch.clamp(x, w[name + ".input_min"], w[name + ".input_max"])
        y = F.linear(x, w[name + ".linear.weight"])
        if self.cfg.clipped and (name + ".output_min") in w:
            y = torch.clamp(y, w[name + ".output_min"], w[name + ".output_max"])
        return y

    def _rope(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        """``x`` ``[B, N, H, D]``; ``cos`` / ``sin`` ``[N, D]``: the halves of D rotate independently
        (columns, rows), each as NeoX-style halves of its own."""
        half = x.shape[-1] // 2
        out = []
        for part in (slice(0, half), slice(half, 2 * half)):
            xp, c, s = x[..., part], cos[None, :, None, part], sin[None, :, None, part]
            q = half // 2
            rot = torch.cat([-xp[..., q:], xp[..., :q]], dim=-1)
            out.append(xp * c + rot * s)
        return torch.cat(out, dim=-1)

    def encode(self, pixels: torch.Tensor) -> torch.Tensor:
        """``pixels`` ``[B, 3, S, S]`` in ``[-1, 1]`` → pooled soft tokens ``[B, tokens, hidden]``."""
        c, w = self.cfg, self.w
        b, _, hgt, wid = pixels.shape
        ps, k = c.patch_size, c.pooling
        gh, gw = hgt // ps, wid // ps
        x = pixels.to(self.device, self.dtype).reshape(b, 3, gh, ps, gw, ps).permute(0, 2, 4, 3, 5, 1)
        x = F.linear(x.reshape(b, gh * gw, ps * ps * 3), w["patch_embedder.input_proj.weight"])
        col = torch.arange(gw, device=self.device).repeat(gh)              # x of every patch, row-major
        row = torch.arange(gh, device=self.device).repeat_interleave(gw)
        table = w["patch_embedder.position_embedding_table"]
        x = x + (table[0][col] + table[1][row])[None]
        hd = c.head_dim
        quarter = hd // 2                                                    # channels per spatial axis
        inv = 1.0 / (c.rope_theta ** (torch.arange(0, quarter, 2, device=self.device).float() / quarter))
        ang = [torch.cat([p.float()[:, None] * inv[None], p.float()[:, None] * inv[None]], -1) for p in (col, row)]
        cos = torch.cat([a.cos() for a in ang], -1).to(self.dtype)
        sin = torch.cat([a.sin() for a in ang], -1).to(self.dtype)
        n = gh * gw
        for l in range(c.num_layers):
            p = f"encoder.layers.{l}."
            y = _rms(x, c.rms_norm_eps, w[p + "input_layernorm.weight"])
            q = self._linear(y, p + "self_attn.q_proj").view(b, n, c.num_heads, hd)
            kk = self._linear(y, p + "self_attn.k_proj").view(b, n, c.num_kv_heads, hd)
            v = self._linear(y, p + "self_attn.v_proj").view(b, n, c.num_kv_heads, hd)
            q = self._rope(_rms(q, c.rms_norm_eps, w[p + "self_attn.q_norm.weight"]), cos, sin)
            kk = self._rope(_rms(kk, c.rms_norm_eps, w[p + "self_attn.k_norm.weight"]), cos, sin)
            v = _rms(v, c.rms_norm_eps)
            rep = c.num_heads // c.num_kv_heads
            kk, v = kk.repeat_interleave(rep, dim=2), v.repeat_interleave(rep, dim=2)
            a = F.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), v.transpose(1, 2), scale=1.0)
            a = self._linear(a.transpose(1, 2).reshape(b, n, c.num_heads * hd), p + "self_attn.o_proj")
            x = x + _rms(a, c.rms_norm_eps, w[p + "post_attention_layernorm.weight"])
            y = _rms(x, c.rms_norm_eps, w[p + "pre_feedforward_layernorm.weight"])
            y = F.gelu(self._linear(y, p + "mlp.gate_proj"), approximate="tanh") * self._linear(y, p + "mlp.up_proj")
            x = x + _rms(self._linear(y, p + "mlp.down_proj"), c.rms_norm_eps, w[p + "post_feedforward_layernorm.weight"])
        d = x.shape[-1]
        if k > 1:
            x = F.avg_pool2d(x.float().transpose(1, 2).reshape(b, d, gh, gw), kernel_size=k, stride=k)
            x = x.flatten(2).transpose(1, 2).to(self.dtype)
        x = x * (float(d) ** 0.5)
        if c.standardize and "std_bias" in w:
            x = (x - w["std_bias"]) * w["std_scale"]
        return x

    def project(self, feats: torch.Tensor) -> torch.Tensor:
        return F.linear(_rms(feats, self.cfg.rms_norm_eps), self.w["embed.embedding_projection.weight"])

    def image_embeddings(self, pixels: torch.Tensor) -> torch.Tensor:
        """``[B, 3, S, S]`` → ``[B * tokens_per_image, text_hidden]`` in prompt order."""
        out = self.project(self.encode(pixels))
        return out.reshape(-1, out.shape[-1])
