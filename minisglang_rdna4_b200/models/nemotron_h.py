"""Nemotron-H: a hybrid of Mamba-2 state-space mixers, grouped-query attention without positional
embedding, and squared-ReLU MLPs or mixture-of-experts blocks; one mixer per layer, pre-norm and
residual around each (python/minisgl/models/nemotron_h.py, python/minisgl/mamba2/).

* ``mamba`` layers: one projection to ``z ‖ x ‖ B ‖ C ‖ dt``; depthwise causal convolution with bias and
  SiLU over ``x ‖ B ‖ C``; the selective state-space recurrence with a ``[head_dim, state]`` matrix per
  head and request; ``w * norm_group(y * silu(z))``; output projection;
* ``attention`` layers: plain GQA, no rotary embedding, no QK norm;
* ``mlp`` layers: ``down(relu(up x)^2)``;
* ``moe`` layers: sigmoid router with a selection bias and group-limited choice, non-gated
  squared-ReLU experts (optionally behind a latent projection), plus a shared non-gated MLP.

The recurrent and convolution states live in ``ctx.gdn_state`` (one slot per request row, the same
cache the gated-delta-net family uses); K/V pages exist for the attention layers only.
"""
from __future__ import annotations

from typing import List

import torch

from .. import ops
from ..core import get_global_ctx
from ..layers import (
    AttentionLayer, BaseOP, ColumnParallelLinear, ParallelLMHead, QKVParallelLinear, RMSNorm, ReplicatedLinear,
    RowParallelLinear, VocabParallelEmbedding,
)
from ..layers.moe import MoELayer
from ..parallel.comm import get_comm
from ..parallel.info import get_tp_info
from ..utils import div_even
from .config import ModelConfig
from .transformer import _scheme


class Mamba2Mixer(BaseOP):
    def __init__(self, cfg: ModelConfig, state_id: int, dtype, device, prefix: str) -> None:
        # tensor parallelism: heads and B / C groups are split evenly over the ranks (the grouped norm never
        # crosses a group), every rank keeps the state of its own heads, the output projection sums
        tp = get_tp_info().size
        self._state_id = state_id
        self._h, self._p, self._n, self._g = (div_even(cfg.mamba_num_heads, tp), cfg.mamba_head_dim,
                                              cfg.ssm_state_size, div_even(cfg.mamba_n_groups, tp))
        self._inter = self._h * self._p
        self._conv_dim = self._inter + 2 * self._g * self._n
        self._eps = cfg.rms_norm_eps
        self._dt_min = cfg.time_step_min
        n = self._inter + self._conv_dim + self._h                      # z ‖ x ‖ B ‖ C ‖ dt
        self._n_proj = n
        self.in_proj = ReplicatedLinear(cfg.hidden_size, (n + 7) // 8 * 8, dtype, device,
                                        _scheme(cfg, prefix + ".in_proj"), bias=cfg.mamba_proj_bias)
        kw = cfg.linear_conv_kernel_dim
        self.conv1d_weight = torch.empty((self._conv_dim, kw), dtype=dtype, device=device)
        self.conv1d_bias = torch.empty((self._conv_dim,), dtype=dtype, device=device) if cfg.mamba_conv_bias else None
        self.dt_bias = torch.empty((self._h,), dtype=torch.float32, device=device)
        self.A_log = torch.empty((self._h,), dtype=torch.float32, device=device)
        self.D = torch.empty((self._h,), dtype=torch.float32, device=device)
        self.norm_weight = torch.empty((self._inter,), dtype=dtype, device=device)
        self.out_proj = RowParallelLinear(cfg.mamba_num_heads * self._p, cfg.hidden_size, dtype, device,
                                          _scheme(cfg, prefix + ".out_proj"), bias=cfg.mamba_proj_bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ctx = get_global_ctx()
        batch = ctx.batch
        proj = self.in_proj.forward(x)
        if ctx.recurrent_journal is not None:
            ctx.recurrent_journal.append((self, proj))
        y = self._mix(proj, batch.attn_metadata.cu_q, batch.gdn_slots, batch.gdn_has_state)
        return self.out_proj.forward(y, reduce=True)

    def _mix(self, proj: torch.Tensor, cu_q, slots, has_state) -> torch.Tensor:
        """Convolution → selective scan → grouped gated norm over the projected rows; advances the two states."""
        st = get_global_ctx().gdn_state
        i, c, h = self._inter, self._conv_dim, self._h
        z = proj[:, :i]
        xbc = ops.gdn_conv1d(proj[:, i:i + c], self.conv1d_weight, st.conv_state(self._state_id), cu_q,
                             slots, has_state, self.conv1d_bias)
        dt = proj[:, i + c:i + c + h]
        y = ops.mamba2_scan(xbc, dt, self.A_log, self.D, self.dt_bias, st.ssm_state(self._state_id), cu_q,
                            slots, has_state, self._h, self._g, self._p, self._n, self._dt_min)
        return ops.rms_norm_gate_first(y.reshape(y.shape[0], i), z, self.norm_weight, self._eps, i // self._g)

    def replay(self, proj: torch.Tensor, cu_q, slots, has_state) -> None:
        """Re-advance the (restored) states over the kept rows of a verify step."""
        self._mix(proj, cu_q, slots, has_state)

    def init_dummy(self, gen: torch.Generator, std: float = 0.02) -> None:
        self.conv1d_weight = (torch.randn(self.conv1d_weight.shape, generator=gen, device=gen.device) * 0.3).to(
            self.conv1d_weight.device, self.conv1d_weight.dtype)
        if self.conv1d_bias is not None:
            self.conv1d_bias = torch.zeros_like(self.conv1d_bias)
        self.dt_bias = torch.ones_like(self.dt_bias)
        a = torch.empty(self.A_log.shape, device=gen.device).uniform_(1.0, 16.0, generator=gen)
        self.A_log = torch.log(a).to(self.A_log.device, torch.float32)
        self.D = torch.ones_like(self.D)
        self.norm_weight = torch.ones_like(self.norm_weight)


class PlainAttention(BaseOP):
    def __init__(self, cfg: ModelConfig, attn_id: int, dtype, device, prefix: str) -> None:
        tp = get_tp_info().size
        self.qkv_proj = QKVParallelLinear(cfg.hidden_size, cfg.head_dim, cfg.num_qo_heads, cfg.num_kv_heads, dtype,
                                          device, _scheme(cfg, prefix + ".qkv_proj"), bias=cfg.attention_bias)
        self.o_proj = RowParallelLinear(cfg.num_qo_heads * cfg.head_dim, cfg.hidden_size, dtype, device,
                                        _scheme(cfg, prefix + ".o_proj"), bias=cfg.attention_bias)
        # the K/V pool is indexed by attn_id: only attention layers own pages
        self.attn = AttentionLayer(attn_id, div_even(cfg.num_qo_heads, tp), div_even(cfg.num_kv_heads, tp, True),
                                   cfg.head_dim, cfg.rotary_config, cfg.rms_norm_eps, dtype, device)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.o_proj.forward(self.attn.forward(self.qkv_proj.forward(x)), reduce=True)


class Relu2MLP(BaseOP):
    def __init__(self, cfg: ModelConfig, inter: int, dtype, device, prefix: str) -> None:
        self.up_proj = ColumnParallelLinear(cfg.hidden_size, inter, dtype, device, _scheme(cfg, prefix + ".up_proj"),
                                            bias=cfg.mlp_bias)
        self.down_proj = RowParallelLinear(inter, cfg.hidden_size, dtype, device, _scheme(cfg, prefix + ".down_proj"),
                                           bias=cfg.mlp_bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down_proj.forward(ops.relu2(self.up_proj.forward(x)), reduce=True)


class NemotronMoE(BaseOP):
    def __init__(self, cfg: ModelConfig, dtype, device, prefix: str) -> None:
        latent = cfg.moe_latent_size
        self.experts = MoELayer(
            cfg.hidden_size, cfg.moe_intermediate_size, cfg.num_experts, cfg.num_experts_per_tok, cfg.norm_topk_prob,
            dtype, device, "sigmoid", cfg.routed_scaling_factor, None, n_group=cfg.n_group,
            topk_group=cfg.topk_group, selection_bias=True, gated=False, act="relu2", expert_input=latent,
        )
        self._latent = latent is not None
        if self._latent:
            self.fc1_latent_proj = ReplicatedLinear(cfg.hidden_size, latent, dtype, device, None, bias=cfg.mlp_bias)
            self.fc2_latent_proj = ReplicatedLinear(latent, cfg.hidden_size, dtype, device, None, bias=cfg.mlp_bias)
        self.shared_experts = Relu2MLP(cfg, cfg.shared_expert_intermediate_size, dtype, device,
                                       prefix + ".shared_experts")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self._latent:
            y = self.experts.forward(x, self.fc1_latent_proj.forward(x))
        else:
            y = self.experts.forward(x)
        if self.experts.needs_tp_reduce:
            y = get_comm().all_reduce(y)
        if self._latent:
            y = self.fc2_latent_proj.forward(y)
        return y + self.shared_experts.forward(x)


class NemotronBlock(BaseOP):
    def __init__(self, cfg: ModelConfig, layer_id: int, attn_id: int, state_id: int, dtype, device) -> None:
        prefix = f"model.layers.{layer_id}.mixer"
        self._kind = cfg.layer_types[layer_id]
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        if self._kind == "mamba":
            self.mixer = Mamba2Mixer(cfg, state_id, dtype, device, prefix)
        elif self._kind == "attention":
            self.mixer = PlainAttention(cfg, attn_id, dtype, device, prefix)
        elif self._kind == "moe":
            self.mixer = NemotronMoE(cfg, dtype, device, prefix)
        elif self._kind == "mlp":
            self.mixer = Relu2MLP(cfg, cfg.intermediate_size, dtype, device, prefix)
        else:
            raise ValueError(f"unknown Nemotron-H layer type {self._kind!r}")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x + self.mixer.forward(self.norm.forward(x))


class NemotronBody(BaseOP):
    def __init__(self, cfg: ModelConfig, dtype, device) -> None:
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, dtype, device)
        self.layers: List[NemotronBlock] = []
        attn_id = state_id = 0
        for i, kind in enumerate(cfg.layer_types):
            self.layers.append(NemotronBlock(cfg, i, attn_id, state_id, dtype, device))
            attn_id += kind == "attention"
            state_id += kind == "mamba"
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)


class NemotronHForCausalLM(BaseOP):
    def __init__(self, cfg: ModelConfig, dtype: torch.dtype, device) -> None:
        self._cfg = cfg
        self.model = NemotronBody(cfg, dtype, device)
        self.lm_head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, dtype, device,
                                      tied=self.model.embed_tokens if cfg.tie_word_embeddings else None)

    @property
    def config(self) -> ModelConfig:
        return self._cfg

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        comm = get_comm()
        comm.row_shard_ok = False
        comm.split_k_ok = False
        x = self.model.embed_tokens.forward(input_ids)
        for layer in self.model.layers:
            x = layer.forward(x)
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
