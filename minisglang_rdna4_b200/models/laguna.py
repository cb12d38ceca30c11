"""Laguna decoder (python/minisgl/models/laguna.py:1-382): a sliding-window / global hybrid with a
mixture of experts.

* attention: a query-head count per layer (``num_attention_heads_per_layer``), weighted q/k norms, the
  global layers' rotary table (YaRN over part of the head) or the sliding layers' own, the window on the
  sliding layers, and a gate per head (softplus of a projection of the layer's normalised input) on the
  attention output before the output projection;
* layers: pre-norm residual; the first ``first_k_dense_replace`` MLPs are dense SwiGLU, the others route
  with sigmoid scores (selection by score + correction bias, weights from the plain scores, renormalised,
  times ``routed_scaling_factor``) and add an always-on shared expert.
"""
from __future__ import annotations

import torch

from ..core import get_global_ctx
from ..layers import (
    AttentionLayer, BaseOP, ColumnParallelLinear, ParallelLMHead, QKVParallelLinear, RMSNorm, RowParallelLinear,
    VocabParallelEmbedding,
)
from ..layers.moe import MoELayer
from ..parallel.comm import get_comm
from ..parallel.info import get_tp_info
from ..utils import div_even
from .config import ModelConfig
from .transformer import GatedMLP, _scheme


class LagunaAttention(BaseOP):
    def __init__(self, cfg: ModelConfig, layer_id: int, dtype, device, prefix: str) -> None:
        tp = get_tp_info().size
        d = cfg.head_dim
        heads = cfg.attn_head_counts[layer_id] if cfg.attn_head_counts else cfg.num_qo_heads
        sliding = bool(cfg.sliding_window) and cfg.layer_types is not None and \
            cfg.layer_types[layer_id] == "sliding_attention"
        self.qkv_proj = QKVParallelLinear(cfg.hidden_size, d, heads, cfg.num_kv_heads, dtype, device,
                                          _scheme(cfg, prefix + ".qkv_proj"))
        self.g_proj = ColumnParallelLinear(cfg.hidden_size, heads, dtype, device, _scheme(cfg, prefix + ".g_proj"))
        self.q_norm = RMSNorm(d, cfg.rms_norm_eps, dtype, device)
        self.k_norm = RMSNorm(d, cfg.rms_norm_eps, dtype, device)
        self.o_proj = RowParallelLinear(heads * d, cfg.hidden_size, dtype, device, _scheme(cfg, prefix + ".o_proj"))
        rotary = (cfg.sliding_rotary or cfg.rotary_config) if sliding else cfg.rotary_config
        self._heads, self._d = div_even(heads, tp), d
        self.attn = AttentionLayer(layer_id, self._heads, div_even(cfg.num_kv_heads, tp, True), d, rotary,
                                   cfg.rms_norm_eps, dtype, device, window=int(cfg.sliding_window) if sliding else 0)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        o = self.attn.forward(self.qkv_proj.forward(x), self.q_norm.weight, self.k_norm.weight)
        gate = torch.nn.functional.softplus(self.g_proj.forward(x).float()).to(o.dtype)
        o = (o.view(-1, self._heads, self._d) * gate.unsqueeze(-1)).reshape(-1, self._heads * self._d)
        return self.o_proj.forward(o, reduce=True)


class LagunaMoEBlock(BaseOP):
    def __init__(self, cfg: ModelConfig, dtype, device, prefix: str) -> None:
        self.experts = MoELayer(cfg.hidden_size, cfg.moe_intermediate_size, cfg.num_experts, cfg.num_experts_per_tok,
                                cfg.norm_topk_prob, dtype, device, "sigmoid", cfg.routed_scaling_factor,
                                _scheme(cfg, prefix + ".experts"), selection_bias=True)
        self.shared_expert = GatedMLP(cfg, cfg.shared_expert_intermediate_size, dtype, device, prefix + ".shared_expert")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.experts.forward(x)
        if self.experts.needs_tp_reduce:
            y = get_comm().all_reduce(y)
        s = self.shared_expert.forward(x)
        if get_tp_info().size > 1:
            s = get_comm().all_reduce(s)
        return y + s


class LagunaDecoderLayer(BaseOP):
    def __init__(self, cfg: ModelConfig, layer_id: int, dtype, device) -> None:
        prefix = f"model.layers.{layer_id}"
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.self_attn = LagunaAttention(cfg, layer_id, dtype, device, prefix + ".self_attn")
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self._is_moe = cfg.layer_is_moe(layer_id)
        if self._is_moe:
            self.mlp = LagunaMoEBlock(cfg, dtype, device, prefix + ".mlp")
        else:
            self.mlp = GatedMLP(cfg, cfg.intermediate_size, dtype, device, prefix + ".mlp")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = x + self.self_attn.forward(self.input_layernorm.forward(x))
        m = self.mlp.forward(self.post_attention_layernorm.forward(x))
        if not self._is_moe and get_tp_info().size > 1:
            m = get_comm().all_reduce(m)
        return x + m


class LagunaBody(BaseOP):
    def __init__(self, cfg: ModelConfig, dtype, device) -> None:
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, dtype, device)
        self.layers = [LagunaDecoderLayer(cfg, i, dtype, device) for i in range(cfg.num_layers)]
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)


class LagunaForCausalLM(BaseOP):
    def __init__(self, cfg: ModelConfig, dtype: torch.dtype, device) -> None:
        self._cfg = cfg
        self.model = LagunaBody(cfg, dtype, device)
        self.lm_head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, dtype, device,
                                      tied=self.model.embed_tokens if cfg.tie_word_embeddings else None)

    @property
    def config(self) -> ModelConfig:
        return self._cfg

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        get_comm().row_shard_ok = False
        get_comm().split_k_ok = False
        ctx = get_global_ctx()
        capture = ctx.batch.capture_layers
        x = self.model.embed_tokens.forward(input_ids)
        seen = {}
        for i, layer in enumerate(self.model.layers):
            if capture is not None and i in capture:
                seen[i] = x
            x = layer.forward(x)
        x = self.model.norm.forward(x)
        if capture is not None:
            seen[len(self.model.layers)] = x
            ctx.aux_hidden = [seen[i] for i in capture]
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
                mod.weight = torch.ones_like(mod.weight)
