"""Qwen3.5 / Qwen3-Next text decoder: a hybrid of gated-delta-net (linear attention) layers and
gated full-attention layers, dense or mixture-of-experts MLP
(python/minisgl/models/qwen3_5.py:1-718, python/minisgl/models/qwen3_5_moe.py,
python/minisgl/gdn/layer.py:186-760).

* every ``full_attention`` layer (one in four by default): GQA with per-head QK RMSNorm, rotary
  embedding on the first quarter of the head dimension, and a per-head sigmoid gate of the
  attention output that comes out of the same projection as the queries;
* every ``linear_attention`` layer: projections to q / k / v (+ output gate z and the two gate
  scalars a, b per value head) → depthwise causal convolution with SiLU → gated delta rule with a
  recurrent ``[Dk, Dv]`` state per value head → gated RMSNorm → output projection;
* RMSNorm weights are stored as ``w - 1``.

The recurrent and convolution states live in ``ctx.gdn_state`` (one slot per request row); the
scheduler passes the slots and whether each request already has a state in
``batch.gdn_slots`` / ``batch.gdn_has_state``.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from ..core import get_global_ctx
from ..layers import (
    AttentionLayer, BaseOP, ColumnParallelLinear, ParallelLMHead, QKVParallelLinear, RMSNorm, ReplicatedLinear,
    RowParallelLinear, VocabParallelEmbedding,
)
from ..parallel.comm import get_comm
from ..parallel.info import get_tp_info
from ..utils import div_even
from .config import ModelConfig
from .transformer import GatedMLP, SparseMoEBlock, _scheme


class GatedAttention(BaseOP):
    _non_persistent = ("_qk_w",)

    def __init__(self, cfg: ModelConfig, layer_id: int, attn_id: int, dtype, device, prefix: str) -> None:
        tp = get_tp_info().size
        self.qkv_proj = QKVParallelLinear(cfg.hidden_size, cfg.head_dim, cfg.num_qo_heads, cfg.num_kv_heads, dtype,
                                          device, _scheme(cfg, prefix + ".qkv_proj"), bias=cfg.attention_bias)
        # the gate half of the checkpoint's q_proj (rows [q_h ‖ gate_h] per head are split at load time)
        self.gate_proj = ColumnParallelLinear(cfg.hidden_size, cfg.num_qo_heads * cfg.head_dim, dtype, device,
                                              _scheme(cfg, prefix + ".gate_proj"), bias=cfg.attention_bias)
        self.o_proj = RowParallelLinear(cfg.num_qo_heads * cfg.head_dim, cfg.hidden_size, dtype, device,
                                        _scheme(cfg, prefix + ".o_proj"), bias=cfg.attention_bias)
        self.q_norm = RMSNorm(cfg.head_dim, cfg.rms_norm_eps, dtype, device, plus_one=True)
        self.k_norm = RMSNorm(cfg.head_dim, cfg.rms_norm_eps, dtype, device, plus_one=True)
        # K/V pages exist for the attention layers only: the pool is indexed by attn_id
        self.attn = AttentionLayer(attn_id, div_even(cfg.num_qo_heads, tp), div_even(cfg.num_kv_heads, tp, True),
                                   cfg.head_dim, cfg.rotary_config, cfg.rms_norm_eps, dtype, device)
        self._qk_w = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        qkv = self.qkv_proj.forward(x)
        gate = self.gate_proj.forward(x)
        if self._qk_w is None:  # the fused kernel multiplies by its weight as given: fold the + 1 in
            self._qk_w = ((self.q_norm.weight.float() + 1).to(self.q_norm.weight.dtype),
                          (self.k_norm.weight.float() + 1).to(self.k_norm.weight.dtype))
        o = self.attn.forward(qkv, self._qk_w[0], self._qk_w[1])
        o = o * torch.sigmoid(gate.float()).to(o.dtype)
        return self.o_proj.forward(o, reduce=True)


class GatedDeltaNet(BaseOP):
    def __init__(self, cfg: ModelConfig, gdn_id: int, dtype, device, prefix: str) -> None:
        # tensor parallelism: key and value heads are split evenly over the ranks (a value head stays with
        # its key head), every rank keeps the state of its own heads, the output projection sums
        tp = get_tp_info().size
        self._gdn_id = gdn_id
        self._hk, self._hv = div_even(cfg.linear_num_key_heads, tp), div_even(cfg.linear_num_value_heads, tp)
        self._dk, self._dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        self._key_dim, self._value_dim = self._hk * self._dk, self._hv * self._dv
        self._conv_dim = 2 * self._key_dim + self._value_dim
        self._eps = cfg.rms_norm_eps
        kw = cfg.linear_conv_kernel_dim
        # one projection for q ‖ k ‖ v ‖ z ‖ b ‖ a (the checkpoint's four in_proj_* matrices stacked);
        # the output width is padded to a multiple of 8 columns for the GEMM
        n = self._conv_dim + self._value_dim + 2 * self._hv
        self._n_proj = n
        self.in_proj = ReplicatedLinear(cfg.hidden_size, (n + 7) // 8 * 8, dtype, device,
                                        _scheme(cfg, prefix + ".in_proj"))
        self.conv1d_weight = torch.empty((self._conv_dim, kw), dtype=dtype, device=device)
        self.dt_bias = torch.empty((self._hv,), dtype=torch.float32, device=device)
        self.A_log = torch.empty((self._hv,), dtype=torch.float32, device=device)
        self.norm_weight = torch.empty((self._dv,), dtype=dtype, device=device)
        self.out_proj = RowParallelLinear(cfg.linear_num_value_heads * self._dv, cfg.hidden_size, dtype, device,
                                          _scheme(cfg, prefix + ".out_proj"))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ctx = get_global_ctx()
        batch = ctx.batch
        proj = self.in_proj.forward(x)                                  # [T, q‖k‖v‖z‖b‖a (+pad)]
        if ctx.recurrent_journal is not None:
            ctx.recurrent_journal.append((self, proj))
        vd = self._value_dim
        o = self._mix(proj, batch.attn_metadata.cu_q, batch.gdn_slots, batch.gdn_has_state)
        return self.out_proj.forward(o.reshape(o.shape[0], vd), reduce=True)

    def _mix(self, proj: torch.Tensor, cu_q, slots, has_state) -> torch.Tensor:
        """Convolution → delta rule → gated norm over the projected rows; advances the two states."""
        st = get_global_ctx().gdn_state
        c, vd, hv = self._conv_dim, self._value_dim, self._hv
        qkv = ops.gdn_conv1d(proj[:, :c], self.conv1d_weight, st.conv_state(self._gdn_id), cu_q, slots, has_state)
        z = proj[:, c:c + vd]
        b = proj[:, c + vd:c + vd + hv]
        a = proj[:, c + vd + hv:c + vd + 2 * hv]
        o = ops.gdn_recurrent(qkv, a, b, self.A_log, self.dt_bias, st.ssm_state(self._gdn_id), cu_q,
                              slots, has_state, self._hk, self._hv, self._dk, self._dv)
        return ops.rms_norm_gated(o, z, self.norm_weight, self._eps)

    def replay(self, proj: torch.Tensor, cu_q, slots, has_state) -> None:
        """Re-advance the (restored) states over the kept rows of a verify step."""
        self._mix(proj, cu_q, slots, has_state)

    def init_dummy(self, gen: torch.Generator, std: float = 0.02) -> None:
        self.conv1d_weight = (torch.randn(self.conv1d_weight.shape, generator=gen, device=gen.device) * 0.3).to(
            self.conv1d_weight.device, self.conv1d_weight.dtype)
        self.dt_bias = torch.ones_like(self.dt_bias)
        a = torch.empty(self.A_log.shape, device=gen.device).uniform_(1.0, 16.0, generator=gen)
        self.A_log = torch.log(a).to(self.A_log.device, torch.float32)
        self.norm_weight = torch.ones_like(self.norm_weight)


class HybridDecoderLayer(BaseOP):
    def __init__(self, cfg: ModelConfig, layer_id: int, attn_id: int, gdn_id: int, dtype, device,
                 prefix: Optional[str] = None) -> None:
        # ``prefix``: the layer's name in the checkpoint when that is not its place in the decoder
        # (the next-token head's layer), for the quantisation scheme lookup
        prefix = prefix or f"model.layers.{layer_id}"
        self._linear = cfg.layer_types[layer_id] == "linear_attention"
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, plus_one=True)
        if self._linear:
            self.linear_attn = GatedDeltaNet(cfg, gdn_id, dtype, device, prefix + ".linear_attn")
        else:
            self.self_attn = GatedAttention(cfg, layer_id, attn_id, dtype, device, prefix + ".self_attn")
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, plus_one=True)
        self._is_moe = cfg.layer_is_moe(layer_id)
        if self._is_moe:
            self.mlp = SparseMoEBlock(cfg, dtype, device, prefix + ".mlp")
        else:
            self.mlp = GatedMLP(cfg, cfg.intermediate_size, dtype, device, prefix + ".mlp")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = self.input_layernorm.forward(x)
        h = self.linear_attn.forward(h) if self._linear else self.self_attn.forward(h)
        x = x + h
        h = self.post_attention_layernorm.forward(x)
        if self._is_moe:
            m, partial = self.mlp.forward(h)
            if partial:
                m = get_comm().all_reduce(m)
        else:
            m = self.mlp.forward(h)
            if get_tp_info().size > 1:
                m = get_comm().all_reduce(m)
        return x + m


class HybridBody(BaseOP):
    def __init__(self, cfg: ModelConfig, dtype, device) -> None:
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, dtype, device)
        self.layers: List[HybridDecoderLayer] = []
        attn_id = gdn_id = 0
        for i in range(cfg.num_layers):
            linear = cfg.layer_types[i] == "linear_attention"
            self.layers.append(HybridDecoderLayer(cfg, i, attn_id, gdn_id, dtype, device))
            if linear:
                gdn_id += 1
            else:
                attn_id += 1
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device, plus_one=True)


class Qwen3_5ForCausalLM(BaseOP):
    def __init__(self, cfg: ModelConfig, dtype: torch.dtype, device) -> None:
        self._cfg = cfg
        self.model = HybridBody(cfg, dtype, device)
        self.lm_head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, dtype, device,
                                      tied=self.model.embed_tokens if cfg.tie_word_embeddings else None)

    @property
    def config(self) -> ModelConfig:
        return self._cfg

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        comm = get_comm()
        comm.row_shard_ok = False
        comm.split_k_ok = False
        ctx = get_global_ctx()
        capture = ctx.batch.capture_layers
        x = self.model.embed_tokens.forward(input_ids)
        seen = {}
        for i, layer in enumerate(self.model.layers):
            if capture is not None and i in capture:
                seen[i] = x
            x = layer.forward(x)
        out = self.model.norm.forward(x)
        if capture is not None:
            seen[len(self.model.layers)] = out      # "layer" num_layers: the final hidden state (the MTP head's input)
            ctx.aux_hidden = [seen[i] for i in capture]
        return out

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
