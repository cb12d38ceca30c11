"""Decoder-only transformer covering the Llama, Mistral, Qwen2, Qwen3 dense families and the
Qwen2-MoE / Qwen3-MoE families. Parameter names follow the Hugging Face checkpoints after
the q/k/v and gate/up merges (``model.layers.N.self_attn.qkv_proj.weight`` …), like the
reference's per-family files (python/minisgl/models/llama.py:60-82, qwen3.py, qwen3_moe.py,
models/utils.py:97-232).

Residual handling: every block hands its *unreduced* tensor-parallel partial sum to the next
RMSNorm, which performs all-reduce + residual add + norm in one fused op. With quantised
linears the norm and the gated activation also emit the per-token e4m3 pair the next GEMM
consumes.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from ..core import get_global_ctx
from ..layers import (
    AttentionLayer, BaseOP, GatedActivation, MergedColumnParallelLinear, MoELayer, ParallelLMHead,
    QKVParallelLinear, RMSNorm, RowParallelLinear, VocabParallelEmbedding,
)
from ..layers import tp_overlap
from ..parallel.comm import get_comm
from ..parallel.info import get_tp_info
from ..utils import div_even
from .config import ModelConfig


def _scheme(cfg: ModelConfig, name: str):
    return cfg.quant.for_module(name) if cfg.quant is not None else None


class SelfAttention(BaseOP):
    def __init__(self, cfg: ModelConfig, layer_id: int, dtype, device, prefix: str) -> None:
        tp = get_tp_info().size
        self.qkv_proj = QKVParallelLinear(
            cfg.hidden_size, cfg.head_dim, cfg.num_qo_heads, cfg.num_kv_heads, dtype, device,
            _scheme(cfg, prefix + ".qkv_proj"), bias=cfg.attention_bias,
        )
        # the output projection has a bias where the family's attention_bias covers it (Llama, Qwen3); Qwen2 and
        # GLM-4.5 put biases on q / k / v only
        self.o_proj = RowParallelLinear(
            cfg.num_qo_heads * cfg.head_dim, cfg.hidden_size, dtype, device,
            _scheme(cfg, prefix + ".o_proj"),
            bias=bool(cfg.attention_bias) and cfg.model_type not in ("qwen2", "qwen2_moe", "glm4_moe"),
        )
        if cfg.qk_norm:
            self.q_norm = RMSNorm(cfg.head_dim, cfg.rms_norm_eps, dtype, device)
            self.k_norm = RMSNorm(cfg.head_dim, cfg.rms_norm_eps, dtype, device)
        window = 0
        if cfg.sliding_window and cfg.layer_types and cfg.layer_types[layer_id] == "sliding_attention":
            window = int(cfg.sliding_window)
        elif cfg.sliding_window and cfg.model_type == "mistral":
            window = int(cfg.sliding_window)
        self.attn = AttentionLayer(
            layer_id, div_even(cfg.num_qo_heads, tp), div_even(cfg.num_kv_heads, tp, True),
            cfg.head_dim, cfg.rotary_config, cfg.rms_norm_eps, dtype, device, window=window,
        )
        self._qk_norm = cfg.qk_norm

    def forward(self, x):
        qkv = self.qkv_proj.forward(x)
        if self._qk_norm:
            o = self.attn.forward(qkv, self.q_norm.weight, self.k_norm.weight)
        else:
            o = self.attn.forward(qkv)
        return self.o_proj.forward(o)  # partial sum


class GatedMLP(BaseOP):
    def __init__(self, cfg: ModelConfig, inter: int, dtype, device, prefix: str) -> None:
        self.gate_up_proj = MergedColumnParallelLinear(
            cfg.hidden_size, [inter, inter], dtype, device, _scheme(cfg, prefix + ".gate_up_proj"),
            bias=cfg.mlp_bias,
        )
        self.down_proj = RowParallelLinear(
            inter, cfg.hidden_size, dtype, device, _scheme(cfg, prefix + ".down_proj"), bias=cfg.mlp_bias,
        )
        self._act = GatedActivation(cfg.hidden_act)

    def forward(self, x):
        h = self.gate_up_proj.forward(x)
        h = self._act(h, quant=self.down_proj.wants_act_quant)
        return self.down_proj.forward(h)  # partial sum


class SparseMoEBlock(BaseOP):
    def __init__(self, cfg: ModelConfig, dtype, device, prefix: str) -> None:
        self.experts = MoELayer(
            cfg.hidden_size, cfg.moe_intermediate_size, cfg.num_experts, cfg.num_experts_per_tok,
            cfg.norm_topk_prob, dtype, device, cfg.scoring_func, cfg.routed_scaling_factor,
            _scheme(cfg, prefix + ".experts"),
        )
        self._shared_gate = cfg.shared_expert_gate
        if cfg.shared_expert_intermediate_size > 0:
            self.shared_expert = GatedMLP(cfg, cfg.shared_expert_intermediate_size, dtype, device,
                                          prefix + ".shared_expert")
            if cfg.shared_expert_gate:
                self.shared_expert_gate = torch.empty((1, cfg.hidden_size), dtype=dtype, device=device)
        self._has_shared = cfg.shared_expert_intermediate_size > 0

    def forward(self, x: torch.Tensor) -> Tuple[torch.Tensor, bool]:
        """Returns ``(y, partial)``: ``partial`` tells whether ``y`` still needs the TP sum."""
        if self.experts.needs_tp_reduce and tp_overlap.applies(x.shape[0]):
            # a large prefill step: reduce finished row chunks while the experts run on the next ones
            return tp_overlap.chunked_all_reduce(self._partial_rows, x), False
        return self._partial_rows(x), self.experts.needs_tp_reduce

    def _partial_rows(self, x: torch.Tensor) -> torch.Tensor:
        y = self.experts.forward(x)
        partial = self.experts.needs_tp_reduce
        if self._has_shared:
            s = self.shared_expert.forward(x)
            if self._shared_gate:
                g = torch.sigmoid(x.float() @ self.shared_expert_gate.float().t()).to(x.dtype)
                s = s * g
            if get_tp_info().size > 1 and not partial:
                s = get_comm().all_reduce(s)
            y = y + s
        return y

    def init_dummy(self, gen, std=0.02) -> None:
        if self._has_shared and self._shared_gate:
            self.shared_expert_gate = torch.zeros_like(self.shared_expert_gate)


class DecoderLayer(BaseOP):
    def __init__(self, cfg: ModelConfig, layer_id: int, dtype, device, prefix: Optional[str] = None) -> None:
        # ``prefix``: the layer's name in the checkpoint when that is not its place in the decoder
        # (the next-token head's layer), for the quantisation scheme lookup
        prefix = prefix or f"model.layers.{layer_id}"
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.self_attn = SelfAttention(cfg, layer_id, dtype, device, prefix + ".self_attn")
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self._is_moe = cfg.layer_is_moe(layer_id)
        # GLM-4.5-style experts: sigmoid scores with a selection bias, group-limited routing, shared experts
        # (the block of models/glm4_moe_lite.py, which sums over the tensor-parallel ranks itself)
        self._glm_moe = self._is_moe and cfg.model_type == "glm4_moe"
        if self._glm_moe:
            from .glm4_moe_lite import GlmMoEBlock

            self.mlp = GlmMoEBlock(cfg, dtype, device, prefix + ".mlp")
        elif self._is_moe:
            self.mlp = SparseMoEBlock(cfg, dtype, device, prefix + ".mlp")
        else:
            self.mlp = GatedMLP(cfg, cfg.intermediate_size, dtype, device, prefix + ".mlp")

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor], partial: bool):
        h, residual = self.input_layernorm.forward_fused(
            x, residual, partial=partial, quant=self.self_attn.qkv_proj.wants_act_quant, to_gemm=True)
        h = self.self_attn.forward(h)
        if self._is_moe:
            h, residual = self.post_attention_layernorm.forward_fused(h, residual, partial=True)
            if self._glm_moe:
                return self.mlp.forward(h), residual, False
            h, part = self.mlp.forward(h)
            return h, residual, part
        h, residual = self.post_attention_layernorm.forward_fused(
            h, residual, partial=True, quant=self.mlp.gate_up_proj.wants_act_quant, to_gemm=True)
        h = self.mlp.forward(h)
        return h, residual, True


class TransformerBody(BaseOP):
    def __init__(self, cfg: ModelConfig, dtype, device) -> None:
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, dtype, device)
        self.layers: List[DecoderLayer] = [DecoderLayer(cfg, i, dtype, device) for i in range(cfg.num_layers)]
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)


class CausalLM(BaseOP):
    """``forward`` returns the final normed hidden states ``[T, H]``; the engine picks the
    rows it needs and calls ``lm_head``."""

    def __init__(self, cfg: ModelConfig, dtype: torch.dtype, device) -> None:
        self._cfg = cfg
        self.model = TransformerBody(cfg, dtype, device)
        self.lm_head = ParallelLMHead(
            cfg.vocab_size, cfg.hidden_size, dtype, device,
            tied=self.model.embed_tokens if cfg.tie_word_embeddings else None,
        )

    @property
    def config(self) -> ModelConfig:
        return self._cfg

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        ctx = get_global_ctx()
        capture = ctx.batch.capture_layers
        x = self.model.embed_tokens.forward(input_ids)
        residual: Optional[torch.Tensor] = None
        partial = False
        # the row-sharded prefill path needs every row-parallel output of the pass to end in a
        # fused add + norm: dense layers only, no hidden-state capture
        comm = get_comm()
        comm.row_shard_ok = capture is None and not any(l._is_moe for l in self.model.layers)
        comm.split_k_ok = False
        if comm.row_shard_ok and comm.size == 1 and input_ids.is_cuda and ctx.batch.is_decode and not ctx.batch.spec_verify:
            from ..ops import cuda as K

            comm.split_k_ok = K.SPLIT_K_DECODE
        seen = {}
        for i, layer in enumerate(self.model.layers):
            if capture is not None and i in capture:
                # hidden state entering layer i = residual + pending block output
                seen[i] = self._materialise(x, residual, partial)
            x, residual, partial = layer.forward(x, residual, partial)
        out, _ = self.model.norm.forward_fused(x, residual, partial=partial)
        if capture is not None:
            seen[len(self.model.layers)] = out      # "layer" num_layers: the final hidden state (the next-token head's input)
            ctx.aux_hidden = [seen[i] for i in capture]
        return out

    @staticmethod
    def _materialise(x, residual, partial):
        if partial:
            x = get_comm().all_reduce(x.clone())
        return x if residual is None else (x.float() + residual.float()).to(x.dtype)

    def init_dummy(self, seed: int, std: float = 0.02, gen_device: str = "cpu") -> None:
        """Random-init every parameter (``--dummy-weight``): N(0, std) linears and embeddings,
        unit norms. The stream of random numbers depends on the seed and on the visit order."""
        gen = torch.Generator(device=gen_device)
        gen.manual_seed(seed)
        for mod in self.modules():
            if mod is self:
                continue
            fn = getattr(mod, "init_dummy", None)
            if fn is not None:
                fn(gen, std)
