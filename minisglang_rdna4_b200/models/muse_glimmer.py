"""Muse-Glimmer text decoder (python/minisgl/models/muse_glimmer.py:1-289): a dense sliding-window /
global hybrid with Gemma-style sandwich norms. What sets it apart from the Gemma layer:

* the embedding output is RMS-normalised without a weight (no sqrt(hidden) multiplier);
* the four norms of a layer are ``(1 + w)``, the two on a sub-layer's output with an epsilon of their own;
  the final norm is plain ``w``;
* queries and keys are RMS-normalised per head without a weight before the rotary embedding; the factor the
  published model multiplies the queries with afterwards is part of the softmax scale here;
* layers whose entry of ``layer_rope_theta`` is 0 (the global ones in the released model) have no positional
  encoding at all;
* a sigmoid gate per channel of the attention output, projected from the layer's normalised input;
* logits are multiplied by ``output_multiplier`` before the soft cap (folded into the returned hidden
  state: the head is linear).

Text only: the vision tower of the checkpoint is not loaded.
"""
from __future__ import annotations

import torch

from ..core import get_global_ctx
from ..layers import (
    AttentionLayer, BaseOP, ColumnParallelLinear, ParallelLMHead, QKVParallelLinear, RMSNorm, RowParallelLinear,
    VocabParallelEmbedding,
)
from .. import ops
from ..parallel.comm import get_comm
from ..parallel.info import get_tp_info
from ..utils import div_even
from .config import ModelConfig, RotaryConfig
from .transformer import GatedMLP, _scheme


class MuseAttention(BaseOP):
    _non_persistent = ("_unit",)

    def __init__(self, cfg: ModelConfig, layer_id: int, dtype, device, prefix: str) -> None:
        tp = get_tp_info().size
        d = cfg.head_dim
        self.qkv_proj = QKVParallelLinear(cfg.hidden_size, d, cfg.num_qo_heads, cfg.num_kv_heads, dtype, device,
                                          _scheme(cfg, prefix + ".qkv_proj"))
        self.gate_proj = ColumnParallelLinear(cfg.hidden_size, cfg.num_qo_heads * d, dtype, device,
                                              _scheme(cfg, prefix + ".gate_proj"))
        self.o_proj = RowParallelLinear(cfg.num_qo_heads * d, cfg.hidden_size, dtype, device,
                                        _scheme(cfg, prefix + ".o_proj"))
        sliding = bool(cfg.sliding_window) and cfg.layer_types[layer_id] == "sliding_attention"
        theta = cfg.layer_rope_theta[layer_id] if cfg.layer_rope_theta else cfg.rotary_config.base
        base = cfg.rotary_config
        rotary = RotaryConfig(head_dim=d, rotary_dim=base.rotary_dim if theta else 0, max_position=base.max_position,
                              base=float(theta or base.base), scaling=base.scaling if theta else None)
        self.attn = AttentionLayer(layer_id, div_even(cfg.num_qo_heads, tp), div_even(cfg.num_kv_heads, tp, True), d,
                                   rotary, cfg.rms_norm_eps, dtype, device,
                                   window=int(cfg.sliding_window) if sliding else 0,
                                   scale=float(cfg.qk_scale_factor or 1.0) * d ** -0.5)
        self._unit = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        qkv = self.qkv_proj.forward(x)
        if self._unit is None:
            self._unit = torch.ones((self.attn._d,), dtype=qkv.dtype, device=qkv.device)
        o = self.attn.forward(qkv, self._unit, self._unit)
        o = o * torch.sigmoid(self.gate_proj.forward(x).float()).to(o.dtype)
        return self.o_proj.forward(o, reduce=True)


class MuseDecoderLayer(BaseOP):
    def __init__(self, cfg: ModelConfig, layer_id: int, dtype, device) -> None:
        prefix = f"model.layers.{layer_id}"
        eps_post = cfg.post_norm_eps if cfg.post_norm_eps is not None else cfg.rms_norm_eps
        norm = lambda eps: RMSNorm(cfg.hidden_size, eps, dtype, device, plus_one=True)
        self.input_layernorm = norm(cfg.rms_norm_eps)
        self.self_attn = MuseAttention(cfg, layer_id, dtype, device, prefix + ".self_attn")
        self.post_attention_layernorm = norm(eps_post)
        self.pre_feedforward_layernorm = norm(cfg.rms_norm_eps)
        self.mlp = GatedMLP(cfg, cfg.intermediate_size, dtype, device, prefix + ".mlp")
        self.post_feedforward_layernorm = norm(eps_post)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        a = self.self_attn.forward(self.input_layernorm.forward(x))
        x = x + self.post_attention_layernorm.forward(a)
        m = self.mlp.forward(self.pre_feedforward_layernorm.forward(x))
        if get_tp_info().size > 1:
            m = get_comm().all_reduce(m)
        return x + self.post_feedforward_layernorm.forward(m)


class MuseBody(BaseOP):
    def __init__(self, cfg: ModelConfig, dtype, device) -> None:
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, dtype, device)
        self.layers = [MuseDecoderLayer(cfg, i, dtype, device) for i in range(cfg.num_layers)]
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)


class MuseGlimmerForConditionalGeneration(BaseOP):
    _non_persistent = ("_unit",)

    def __init__(self, cfg: ModelConfig, dtype: torch.dtype, device) -> None:
        self._cfg = cfg
        self.model = MuseBody(cfg, dtype, device)
        self.lm_head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, dtype, device,
                                      tied=self.model.embed_tokens if cfg.tie_word_embeddings else None)
        self._unit = None

    @property
    def config(self) -> ModelConfig:
        return self._cfg

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        get_comm().row_shard_ok = False
        get_comm().split_k_ok = False
        ctx = get_global_ctx()
        capture = ctx.batch.capture_layers
        x = self.model.embed_tokens.forward(input_ids)
        if self._unit is None:
            self._unit = torch.ones((x.shape[-1],), dtype=x.dtype, device=x.device)
        x = ops.rms_norm(x, self._unit, self._cfg.rms_norm_eps)
        seen = {}
        for i, layer in enumerate(self.model.layers):
            if capture is not None and i in capture:
                seen[i] = x
            x = layer.forward(x)
        x = self.model.norm.forward(x)
        if capture is not None:
            seen[len(self.model.layers)] = x
            ctx.aux_hidden = [seen[i] for i in capture]
        if self._cfg.output_multiplier is not None:
            x = x * float(self._cfg.output_multiplier)
        return x

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
            if isinstance(mod, RMSNorm):
                mod.weight = torch.zeros_like(mod.weight) if mod._plus_one else torch.ones_like(mod.weight)
