"""Gemma-2 / Gemma-3 style text decoder: sandwich norms, GeGLU, (1 + w) RMSNorm weights,
scaled embeddings, a query scale that is not ``head_dim ** -0.5``, optional QK-norm, and
alternating sliding-window / global attention layers with their own RoPE base.

The reference serves this family with ``gemma4.py`` (python/minisgl/models/gemma4.py:1-510).
Every block output is normalised *before* it joins the residual stream, so the tensor-parallel
sum cannot be folded into an add + norm the way the Llama-style layer does it: the row-parallel
projections finish their all-reduce, the post-norm runs on the sum, then the add.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..core import get_global_ctx
from ..layers import (
    AttentionLayer, BaseOP, GatedActivation, MergedColumnParallelLinear, ParallelLMHead, QKVParallelLinear,
    RMSNorm, RowParallelLinear, VocabParallelEmbedding,
)
from ..parallel.comm import get_comm
from ..parallel.info import get_tp_info
from ..utils import div_even
from .config import ModelConfig, RotaryConfig
from .transformer import _scheme


class GemmaAttention(BaseOP):
    _non_persistent = ("_qk_w",)

    def __init__(self, cfg: ModelConfig, layer_id: int, dtype, device, prefix: str) -> None:
        tp = get_tp_info().size
        self.qkv_proj = QKVParallelLinear(cfg.hidden_size, cfg.head_dim, cfg.num_qo_heads, cfg.num_kv_heads, dtype,
                                          device, _scheme(cfg, prefix + ".qkv_proj"), bias=cfg.attention_bias)
        self.o_proj = RowParallelLinear(cfg.num_qo_heads * cfg.head_dim, cfg.hidden_size, dtype, device,
                                        _scheme(cfg, prefix + ".o_proj"), bias=cfg.attention_bias)
        self._qk_norm = cfg.qk_norm
        if cfg.qk_norm:
            self.q_norm = RMSNorm(cfg.head_dim, cfg.rms_norm_eps, dtype, device, plus_one=True)
            self.k_norm = RMSNorm(cfg.head_dim, cfg.rms_norm_eps, dtype, device, plus_one=True)
        sliding = bool(cfg.sliding_window) and cfg.layer_types is not None and \
            cfg.layer_types[layer_id] == "sliding_attention"
        rotary = cfg.rotary_config
        if sliding and cfg.rope_local_base_freq:
            rotary = RotaryConfig(head_dim=rotary.head_dim, rotary_dim=rotary.rotary_dim,
                                  max_position=rotary.max_position, base=float(cfg.rope_local_base_freq),
                                  scaling=None)
        scalar = cfg.query_pre_attn_scalar or cfg.head_dim
        self.attn = AttentionLayer(layer_id, div_even(cfg.num_qo_heads, tp), div_even(cfg.num_kv_heads, tp, True),
                                   cfg.head_dim, rotary, cfg.rms_norm_eps, dtype, device,
                                   window=int(cfg.sliding_window) if sliding else 0, scale=float(scalar) ** -0.5)
        self._qk_w = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        qkv = self.qkv_proj.forward(x)
        if self._qk_norm:
            if self._qk_w is None:  # the fused kernel multiplies by its weight as given: fold the + 1 in
                self._qk_w = ((self.q_norm.weight.float() + 1).to(self.q_norm.weight.dtype),
                              (self.k_norm.weight.float() + 1).to(self.k_norm.weight.dtype))
            o = self.attn.forward(qkv, self._qk_w[0], self._qk_w[1])
        else:
            o = self.attn.forward(qkv)
        return self.o_proj.forward(o, reduce=True)


class GemmaMLP(BaseOP):
    def __init__(self, cfg: ModelConfig, dtype, device, prefix: str) -> None:
        self.gate_up_proj = MergedColumnParallelLinear(cfg.hidden_size, [cfg.intermediate_size] * 2, dtype, device,
                                                       _scheme(cfg, prefix + ".gate_up_proj"))
        self.down_proj = RowParallelLinear(cfg.intermediate_size, cfg.hidden_size, dtype, device,
                                           _scheme(cfg, prefix + ".down_proj"))
        self._act = GatedActivation(cfg.hidden_act if cfg.hidden_act != "silu" else "gelu_pytorch_tanh")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = self._act(self.gate_up_proj.forward(x), quant=self.down_proj.wants_act_quant)
        return self.down_proj.forward(h, reduce=True)


class GemmaDecoderLayer(BaseOP):
    def __init__(self, cfg: ModelConfig, layer_id: int, dtype, device) -> None:
        prefix = f"model.layers.{layer_id}"
        norm = lambda: RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, plus_one=True)
        self.input_layernorm = norm()
        self.self_attn = GemmaAttention(cfg, layer_id, dtype, device, prefix + ".self_attn")
        self.post_attention_layernorm = norm()
        self.pre_feedforward_layernorm = norm()
        self.mlp = GemmaMLP(cfg, dtype, device, prefix + ".mlp")
        self.post_feedforward_layernorm = norm()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        a = self.self_attn.forward(self.input_layernorm.forward(x))
        x = x + self.post_attention_layernorm.forward(a)
        m = self.mlp.forward(self.pre_feedforward_layernorm.forward(x))
        return x + self.post_feedforward_layernorm.forward(m)


class GemmaBody(BaseOP):
    def __init__(self, cfg: ModelConfig, dtype, device) -> None:
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, dtype, device)
        self.layers = [GemmaDecoderLayer(cfg, i, dtype, device) for i in range(cfg.num_layers)]
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, plus_one=True)


class GemmaForCausalLM(BaseOP):
    def __init__(self, cfg: ModelConfig, dtype: torch.dtype, device) -> None:
        self._cfg = cfg
        self.model = GemmaBody(cfg, dtype, device)
        self.lm_head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, dtype, device,
                                      tied=self.model.embed_tokens if cfg.tie_word_embeddings else None)
        self._embed_scale = float(cfg.hidden_size) ** 0.5
        self._embed_scale_dtype = None
        self._embed_scale_rounded = self._embed_scale

    @property
    def config(self) -> ModelConfig:
        return self._cfg

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        get_comm().row_shard_ok = False
        get_comm().split_k_ok = False
        ctx = get_global_ctx()
        capture = ctx.batch.capture_layers
        x = self.model.embed_tokens.forward(input_ids)
        # the scale is rounded to the activation dtype first, as the published implementation does
        # (a Python scalar: nothing is copied to the device, so the step stays graph-capturable)
        if self._embed_scale_dtype != x.dtype:
            self._embed_scale_rounded = float(torch.tensor(self._embed_scale, dtype=x.dtype))
            self._embed_scale_dtype = x.dtype
        x = x * self._embed_scale_rounded
        if ctx.batch.mm_rows is not None:
            # image placeholder rows take the projected vision features as they are (not scaled)
            x = x.index_copy(0, ctx.batch.mm_rows, ctx.batch.mm_values.to(x.dtype))
        seen = {}
        for i, layer in enumerate(self.model.layers):
            if capture is not None and i in capture:
                seen[i] = x
            x = layer.forward(x)
        if capture is not None:
            ctx.aux_hidden = [seen[i] for i in capture]
        return self.model.norm.forward(x)

    def init_dummy(self, seed: int, std: float = 0.02, gen_device: str = "cpu") -> None:
        gen = torch.Generator(device=gen_device)
        gen.manual_seed(seed)
        for mod in self.modules():
            if mod is self:
                continue
            fn = getattr(mod, "init_dummy", None)
            if fn is not None:
                fn(gen, std)
        for mod in self.modules():
            if isinstance(mod, RMSNorm):  # (1 + w) convention: the neutral weight is zero
                mod.weight = torch.zeros_like(mod.weight)
