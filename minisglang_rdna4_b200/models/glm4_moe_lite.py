"""GLM-4.x MoE "lite" / DeepSeek-V2-style decoder: multi-head latent attention (MLA) and a
mixture-of-experts MLP with sigmoid scores, a selection bias, group-limited routing and shared
experts (python/minisgl/models/glm4_moe_lite.py:1-655, python/minisgl/attention/mla.py:35-161).

Attention. Queries come from a low-rank pair ``q_a_proj → RMSNorm → q_b_proj`` (or one ``q_proj``);
keys and values from a shared latent: ``kv_a_proj_with_mqa`` yields ``kv_lora_rank`` latent channels
plus one rotary key of ``qk_rope_head_dim`` channels shared by all heads, and ``kv_b_proj`` expands
the normalised latent into a per-head non-rotary key part and a value. A head's key is
``[k_nope_h ‖ rope(k_rot)]`` and its query ``[q_nope_h ‖ rope(q_rot_h)]``.

This implementation runs the *materialised* form: the per-head keys and values are built for the
step's tokens and stored in the ordinary paged K/V pool (head width = ``qk_nope + qk_rope`` = 256 =
``v_head_dim`` for GLM-4.7-Flash; where the value heads are narrower or the width is not one the
kernels are built for, as with DeepSeek-V2/V3's 192 key and 128 value channels, queries, keys and
values are zero-padded to a common width, which changes no dot product), so every attention kernel
of the engine (prefill, extend, decode, verify) serves the family unchanged. The head layout is
permuted to ``[rope ‖ nope]`` for both queries and keys, which leaves every dot product unchanged
and puts the rotary channels where the fused RoPE + store kernel expects them (the first
``rotary_dim`` channels). The latent-cache ("absorbed") decode form of the reference's ``mla_hip``
kernels, which keeps ``kv_lora_rank + qk_rope`` channels per token instead of
``2 * heads * 256``, is not built.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..core import get_global_ctx
from ..layers import (
    AttentionLayer, BaseOP, ColumnParallelLinear, ParallelLMHead, RMSNorm, ReplicatedLinear, RowParallelLinear,
    VocabParallelEmbedding,
)
from ..layers.moe import MoELayer
from ..parallel.comm import get_comm
from ..parallel.info import get_tp_info
from ..utils import div_even
from .config import ModelConfig, RotaryConfig
from .transformer import GatedMLP, _scheme


def _mscale(scale: float, m: float) -> float:
    import math

    return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0


class LatentAttention(BaseOP):
    def __init__(self, cfg: ModelConfig, layer_id: int, dtype, device, prefix: str) -> None:
        tp = get_tp_info().size
        self._h = div_even(cfg.num_qo_heads, tp)
        self._nope, self._rope, self._vd = int(cfg.qk_nope_head_dim), int(cfg.qk_rope_head_dim), int(cfg.v_head_dim)
        self._d = self._nope + self._rope
        # width of a head in the K/V pool: keys / queries (nope + rope channels) and values zero-padded to it
        self._pd = int(cfg.head_dim)
        if self._pd < max(self._d, self._vd):
            raise ValueError(f"pool head width {self._pd} below the latent-attention head ({self._d}, {self._vd})")
        self._lora = int(cfg.kv_lora_rank)
        if cfg.q_lora_rank:
            self.q_a_proj = ReplicatedLinear(cfg.hidden_size, int(cfg.q_lora_rank), dtype, device,
                                             _scheme(cfg, prefix + ".q_a_proj"), bias=cfg.attention_bias)
            self.q_a_layernorm = RMSNorm(int(cfg.q_lora_rank), 1e-6, dtype, device)
            self.q_b_proj = ColumnParallelLinear(int(cfg.q_lora_rank), cfg.num_qo_heads * self._d, dtype, device,
                                                 _scheme(cfg, prefix + ".q_b_proj"))
        else:
            self.q_proj = ColumnParallelLinear(cfg.hidden_size, cfg.num_qo_heads * self._d, dtype, device,
                                               _scheme(cfg, prefix + ".q_proj"))
        self._q_lora = bool(cfg.q_lora_rank)
        self.kv_a_proj_with_mqa = ReplicatedLinear(cfg.hidden_size, self._lora + self._rope, dtype, device,
                                                   _scheme(cfg, prefix + ".kv_a_proj_with_mqa"),
                                                   bias=cfg.attention_bias)
        self.kv_a_layernorm = RMSNorm(self._lora, 1e-6, dtype, device)
        self.kv_b_proj = ColumnParallelLinear(self._lora, cfg.num_qo_heads * (self._nope + self._vd), dtype, device,
                                              _scheme(cfg, prefix + ".kv_b_proj"))
        self.o_proj = RowParallelLinear(cfg.num_qo_heads * self._vd, cfg.hidden_size, dtype, device,
                                        _scheme(cfg, prefix + ".o_proj"), bias=cfg.attention_bias)
        scale = self._d ** -0.5
        sc = cfg.rotary_config.scaling or {}
        if sc.get("rope_type", sc.get("type", "default")) not in ("default", None) and sc.get("mscale_all_dim"):
            m = _mscale(float(sc.get("factor", 1.0)), float(sc["mscale_all_dim"]))
            scale = scale * m * m
        self.attn = AttentionLayer(layer_id, self._h, self._h, self._pd, cfg.rotary_config, cfg.rms_norm_eps, dtype,
                                   device, scale=scale)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        t = x.shape[0]
        h, nope, rope, d = self._h, self._nope, self._rope, self._d
        if self._q_lora:
            q = self.q_b_proj.forward(self.q_a_layernorm.forward(self.q_a_proj.forward(x)))
        else:
            q = self.q_proj.forward(x)
        q = q.view(t, h, d)
        ckv = self.kv_a_proj_with_mqa.forward(x)
        latent, k_rot = ckv[:, : self._lora], ckv[:, self._lora:]
        if getattr(get_global_ctx().kv_cache, "latent", False):
            return self._forward_absorbed(q, latent, k_rot)
        kv = self.kv_b_proj.forward(self.kv_a_layernorm.forward(latent.contiguous())).view(t, h, nope + self._vd)
        # [rope ‖ nope] layout for q and k (the same permutation on both sides of every dot product)
        pd, vd = self._pd, self._vd
        padded = pd != d or pd != vd
        qkv = (torch.zeros if padded else torch.empty)((t, 3 * h, pd), dtype=x.dtype, device=x.device)
        qkv[:, :h, :rope] = q[:, :, nope:]
        qkv[:, :h, rope:d] = q[:, :, :nope]
        qkv[:, h:2 * h, :rope] = k_rot[:, None, :]
        qkv[:, h:2 * h, rope:d] = kv[:, :, :nope]
        qkv[:, 2 * h:, :vd] = kv[:, :, nope:]
        o = self.attn.forward(qkv.view(t, 3 * h * pd))
        if pd != vd:                               # the padding channels of the value heads come back as zeros
            o = o.view(t, h, pd)[:, :, :vd].reshape(t, h * vd)
        return self.o_proj.forward(o, reduce=True)


    def _forward_absorbed(self, q: torch.Tensor, latent: torch.Tensor, k_rot: torch.Tensor) -> torch.Tensor:
        """The pool holds the normalised latent and the shared rotary key of every token
        (``kvcache/mla_pool.py``); queries go into the latent space through the key half of ``kv_b_proj``,
        the attended latents come back through its value half."""
        from ..layers.rotary import get_rope_cache
        from ..ops import ref

        ctx = get_global_ctx()
        batch, md, pool = ctx.batch, ctx.batch.attn_metadata, ctx.kv_cache
        t, h, nope, rope, vd, lora = q.shape[0], self._h, self._nope, self._rope, self._vd, self._lora
        w = getattr(self.kv_b_proj, "weight", None)
        if w is None or w.dtype not in (torch.float32, torch.bfloat16, torch.float16) or w.shape[1] != lora:
            raise NotImplementedError("the latent pool needs kv_b_proj in a 16- or 32-bit dense form")
        w = w.view(h, nope + vd, lora)
        rot_cfg = self.attn._rotary
        cos_sin = get_rope_cache(rot_cfg, q.device)
        q_rot, k_rot = ref.qk_norm_rope(q[:, :, nope:].reshape(t, h * rope), k_rot.contiguous(), None, None,
                                        batch.positions, cos_sin, rope, rope, 0.0, rot_cfg.interleaved)
        layer = self.attn._kv_index
        pool.store(layer, self.kv_a_layernorm.forward(latent.contiguous()), k_rot, batch.out_loc)
        q_lat = torch.einsum("thn,hnl->thl", q[:, :, :nope].float(), w[:, :nope].float()).to(q.dtype)
        o_lat = ref.mla_attention(q_lat, q_rot.view(t, h, rope), pool.rows(layer), md.block_table, md.cu_q,
                                  md.seq_lens, self.attn._scale, lora)
        o = torch.einsum("thl,hvl->thv", o_lat.float(), w[:, nope:].float()).to(q.dtype)
        return self.o_proj.forward(o.reshape(t, h * vd), reduce=True)


class GlmMoEBlock(BaseOP):
    def __init__(self, cfg: ModelConfig, dtype, device, prefix: str) -> None:
        self.experts = MoELayer(
            cfg.hidden_size, cfg.moe_intermediate_size, cfg.num_experts, cfg.num_experts_per_tok, cfg.norm_topk_prob,
            dtype, device, cfg.scoring_func, cfg.routed_scaling_factor, _scheme(cfg, prefix + ".experts"),
            # DeepSeek-V2 scores with a softmax and has no selection bias; V3 / GLM use sigmoid scores and one
            n_group=cfg.n_group, topk_group=cfg.topk_group, selection_bias=cfg.scoring_func == "sigmoid",
        )
        self._shared = cfg.n_shared_experts > 0
        if self._shared:
            self.shared_experts = GatedMLP(cfg, cfg.moe_intermediate_size * cfg.n_shared_experts, dtype, device,
                                           prefix + ".shared_experts")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.experts.forward(x)
        if self.experts.needs_tp_reduce:
            y = get_comm().all_reduce(y)
        if self._shared:
            s = self.shared_experts.forward(x)
            if get_tp_info().size > 1:
                s = get_comm().all_reduce(s)
            y = y + s
        return y


class GlmDecoderLayer(BaseOP):
    def __init__(self, cfg: ModelConfig, layer_id: int, dtype, device, prefix: Optional[str] = None) -> None:
        # ``prefix``: the layer's name in the checkpoint when that is not its place in the decoder
        # (the next-token head's layer), for the quantisation scheme lookup
        prefix = prefix or f"model.layers.{layer_id}"
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.self_attn = LatentAttention(cfg, layer_id, dtype, device, prefix + ".self_attn")
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self._is_moe = cfg.layer_is_moe(layer_id)
        if self._is_moe:
            self.mlp = GlmMoEBlock(cfg, dtype, device, prefix + ".mlp")
        else:
            self.mlp = GatedMLP(cfg, cfg.intermediate_size, dtype, device, prefix + ".mlp")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = x + self.self_attn.forward(self.input_layernorm.forward(x))
        h = self.post_attention_layernorm.forward(x)
        if self._is_moe:
            m = self.mlp.forward(h)
        else:
            m = self.mlp.forward(h)
            if get_tp_info().size > 1:
                m = get_comm().all_reduce(m)
        return x + m


class GlmBody(BaseOP):
    def __init__(self, cfg: ModelConfig, dtype, device) -> None:
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, dtype, device)
        self.layers: List[GlmDecoderLayer] = [GlmDecoderLayer(cfg, i, dtype, device) for i in range(cfg.num_layers)]
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)


class Glm4MoeLiteForCausalLM(BaseOP):
    def __init__(self, cfg: ModelConfig, dtype: torch.dtype, device) -> None:
        self._cfg = cfg
        self.model = GlmBody(cfg, dtype, device)
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
            seen[len(self.model.layers)] = out      # "layer" num_layers: the final hidden state (the next-token head's input)
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
