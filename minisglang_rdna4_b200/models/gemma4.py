"""Gemma-4 text decoder (python/minisgl/models/gemma4.py:1-510).

What it adds to the Gemma-3 layer (sandwich norms, GeGLU, scaled embeddings, sliding / global layers):

* global layers with their own head width (``global_head_dim``) and, with ``attention_k_eq_v``, their own
  K/V head count and no value projection: the key projection's output, before its norm and rotary
  embedding, is the value. Values are RMS-normalised without a weight; queries and keys with one;
  the softmax scale is 1;
* "proportional" rotary embedding on the global layers: pairs ``(i, i + width / 2)`` over the whole head,
  the first ``partial_rotary_factor`` of them rotating, the others at angle zero (a table, ``ops.ref``);
* the last ``num_kv_shared_layers`` layers keep no K/V: each reads the pool rows of the last earlier layer
  of its kind (``AttentionLayer._kv_donor``) and only projects queries. Their MLP can be twice as wide;
* per-layer input embeddings: a second embedding table of ``layers x hidden_size_per_layer_input`` columns
  plus a projection of the first one, gated into every layer after its MLP;
* a scalar per layer on the layer's output;
* optionally a mixture-of-experts block beside the dense MLP (router on the un-normalised stream with its
  own scale vector and a scale per expert, GELU-gated experts); both results are normalised and summed.

Norm weights are plain (not ``1 + w``). Every layer type has its own (kv heads, head width), so the K/V
pool carries a geometry per layer (``kvcache/mha_pool.py``) or, with the sliding-window pool, one per pool.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..core import get_global_ctx
from ..layers import (
    AttentionLayer, BaseOP, ColumnParallelLinear, GatedActivation, MergedColumnParallelLinear, ParallelLMHead,
    RMSNorm, ReplicatedLinear, RowParallelLinear, VocabParallelEmbedding,
)
from ..layers.moe import MoELayer
from ..parallel.comm import get_comm
from ..parallel.info import get_tp_info
from ..utils import div_even
from .config import ModelConfig, RotaryConfig
from .transformer import _scheme


def _ones(n: int, like: torch.Tensor) -> torch.Tensor:
    return torch.ones((n,), dtype=like.dtype, device=like.device)


class Gemma4Attention(BaseOP):
    _non_persistent = ("_unit",)

    def __init__(self, cfg: ModelConfig, layer_id: int, dtype, device, prefix: str) -> None:
        tp = get_tp_info().size
        sliding = cfg.layer_types[layer_id] == "sliding_attention"
        kv_heads, d = cfg.attn_geometry(layer_id)
        if kv_heads % tp:
            raise NotImplementedError(f"{kv_heads} K/V heads do not split over {tp} tensor-parallel ranks")
        self._d, self._hq, self._hk = d, div_even(cfg.num_qo_heads, tp), kv_heads // tp
        self._donor = cfg.kv_donor(layer_id)
        self._k_eq_v = cfg.attention_k_eq_v and not sliding
        self.q_proj = ColumnParallelLinear(cfg.hidden_size, cfg.num_qo_heads * d, dtype, device,
                                           _scheme(cfg, prefix + ".q_proj"), bias=cfg.attention_bias)
        self.q_norm = RMSNorm(d, cfg.rms_norm_eps, dtype, device)
        if self._donor is None:
            self.k_proj = ColumnParallelLinear(cfg.hidden_size, kv_heads * d, dtype, device,
                                               _scheme(cfg, prefix + ".k_proj"), bias=cfg.attention_bias)
            self.k_norm = RMSNorm(d, cfg.rms_norm_eps, dtype, device)
            if not self._k_eq_v:
                self.v_proj = ColumnParallelLinear(cfg.hidden_size, kv_heads * d, dtype, device,
                                                   _scheme(cfg, prefix + ".v_proj"), bias=cfg.attention_bias)
        self.o_proj = RowParallelLinear(cfg.num_qo_heads * d, cfg.hidden_size, dtype, device,
                                        _scheme(cfg, prefix + ".o_proj"), bias=cfg.attention_bias)
        if sliding:
            rotary = RotaryConfig(head_dim=d, rotary_dim=d, max_position=cfg.rotary_config.max_position,
                                  base=float(cfg.rope_local_base_freq or 10000.0), scaling=None)
        else:
            rotary = cfg.rotary_config
        self.attn = AttentionLayer(layer_id, self._hq, self._hk, d, rotary, cfg.rms_norm_eps, dtype, device,
                                   window=int(cfg.sliding_window) if sliding else 0, scale=1.0)
        self.attn._kv_donor = self._donor
        self._eps = cfg.rms_norm_eps
        self._unit = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        q = self.q_proj.forward(x)
        if self._donor is not None:
            o = self.attn.forward(q, self.q_norm.weight)
            return self.o_proj.forward(o, reduce=True)
        k = self.k_proj.forward(x)
        v = k if self._k_eq_v else self.v_proj.forward(x)
        if self._unit is None:
            self._unit = _ones(self._d, v)
        t = v.shape[0]
        v = ops.rms_norm(v.reshape(t * self._hk, self._d), self._unit, self._eps).view(t, self._hk * self._d)
        o = self.attn.forward(torch.cat([q, k, v], dim=-1), self.q_norm.weight, self.k_norm.weight)
        return self.o_proj.forward(o, reduce=True)


class Gemma4MLP(BaseOP):
    def __init__(self, cfg: ModelConfig, inter: int, dtype, device, prefix: str) -> None:
        self.gate_up_proj = MergedColumnParallelLinear(cfg.hidden_size, [inter] * 2, dtype, device,
                                                       _scheme(cfg, prefix + ".gate_up_proj"))
        self.down_proj = RowParallelLinear(inter, cfg.hidden_size, dtype, device, _scheme(cfg, prefix + ".down_proj"))
        self._act = GatedActivation(cfg.hidden_act)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = self._act(self.gate_up_proj.forward(x), quant=self.down_proj.wants_act_quant)
        return self.down_proj.forward(h, reduce=True)


class Gemma4Router(BaseOP):
    """Scores on the RMS-normalised (no weight) stream times a learned vector and ``hidden ** -0.5``; soft-max
    over all experts, top-k, renormalised, then a learned scale per chosen expert. The projection itself
    is the expert layer's ``gate`` (the loader puts ``router.proj.weight`` there)."""
    _non_persistent = ("_unit",)

    def __init__(self, cfg: ModelConfig, dtype, device) -> None:
        self.scale = torch.empty((cfg.hidden_size,), dtype=dtype, device=device)
        self.per_expert_scale = torch.empty((cfg.num_experts,), dtype=dtype, device=device)
        self._root, self._eps, self._k = float(cfg.hidden_size) ** -0.5, cfg.rms_norm_eps, cfg.num_experts_per_tok
        self._unit = None

    def forward(self, x: torch.Tensor, proj) -> tuple:
        if self._unit is None:
            self._unit = _ones(x.shape[-1], x)
        r = ops.rms_norm(x, self._unit, self._eps) * self.scale * self._root
        probs = torch.softmax(proj.forward(r).float(), dim=-1)
        w, ids = torch.topk(probs, self._k, dim=-1)
        w = w / w.sum(-1, keepdim=True)
        w = w * self.per_expert_scale.float()[ids]
        return w.to(x.dtype), ids.to(torch.int32)

    def init_dummy(self, gen: torch.Generator, std: float = 0.02) -> None:
        self.scale = torch.ones_like(self.scale)
        self.per_expert_scale = torch.ones_like(self.per_expert_scale)


class Gemma4DecoderLayer(BaseOP):
    def __init__(self, cfg: ModelConfig, layer_id: int, dtype, device) -> None:
        prefix = f"model.layers.{layer_id}"
        norm = lambda: RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.input_layernorm = norm()
        self.self_attn = Gemma4Attention(cfg, layer_id, dtype, device, prefix + ".self_attn")
        self.post_attention_layernorm = norm()
        self.pre_feedforward_layernorm = norm()
        shared = cfg.kv_donor(layer_id) is not None
        inter = cfg.intermediate_size * (2 if cfg.use_double_wide_mlp and shared else 1)
        self.mlp = Gemma4MLP(cfg, inter, dtype, device, prefix + ".mlp")
        self.post_feedforward_layernorm = norm()
        self.layer_scalar = torch.ones((1,), dtype=dtype, device=device)
        self._ple = int(cfg.hidden_size_per_layer_input)
        if self._ple:
            self.per_layer_input_gate = ReplicatedLinear(cfg.hidden_size, self._ple, dtype, device,
                                                         _scheme(cfg, prefix + ".per_layer_input_gate"))
            self.per_layer_projection = ReplicatedLinear(self._ple, cfg.hidden_size, dtype, device,
                                                         _scheme(cfg, prefix + ".per_layer_projection"))
            self.post_per_layer_input_norm = norm()
        self._moe = bool(cfg.enable_moe_block)
        if self._moe:
            self.router = Gemma4Router(cfg, dtype, device)
            self.experts = MoELayer(cfg.hidden_size, cfg.moe_intermediate_size, cfg.num_experts,
                                    cfg.num_experts_per_tok, True, dtype, device,
                                    scheme=_scheme(cfg, prefix + ".experts"), act=cfg.hidden_act)
            self.post_feedforward_layernorm_1 = norm()
            self.post_feedforward_layernorm_2 = norm()
            self.pre_feedforward_layernorm_2 = norm()
        self._tanh = cfg.hidden_act != "gelu"

    def forward(self, x: torch.Tensor, per_layer_input: Optional[torch.Tensor]) -> torch.Tensor:
        a = self.self_attn.forward(self.input_layernorm.forward(x))
        x = x + self.post_attention_layernorm.forward(a)
        m = self.mlp.forward(self.pre_feedforward_layernorm.forward(x))
        if self._moe:
            w, ids = self.router.forward(x, self.experts.gate)
            e = self.experts.local_experts(self.pre_feedforward_layernorm_2.forward(x), w, ids)
            if self.experts._ep is not None or get_tp_info().size > 1:
                e = get_comm().all_reduce(e)
            m = self.post_feedforward_layernorm_1.forward(m) + self.post_feedforward_layernorm_2.forward(e)
        x = x + self.post_feedforward_layernorm.forward(m)
        if self._ple:
            g = torch.nn.functional.gelu(self.per_layer_input_gate.forward(x),
                                         approximate="tanh" if self._tanh else "none")
            p = self.per_layer_projection.forward(g * per_layer_input)
            x = x + self.post_per_layer_input_norm.forward(p)
        return x * self.layer_scalar

    def init_dummy(self, gen: torch.Generator, std: float = 0.02) -> None:
        self.layer_scalar = torch.ones_like(self.layer_scalar)


class Gemma4Body(BaseOP):
    def __init__(self, cfg: ModelConfig, dtype, device) -> None:
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, dtype, device)
        self.layers = [Gemma4DecoderLayer(cfg, i, dtype, device) for i in range(cfg.num_layers)]
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        ple = int(cfg.hidden_size_per_layer_input)
        if ple:
            self.embed_tokens_per_layer = VocabParallelEmbedding(cfg.vocab_size_per_layer_input or cfg.vocab_size,
                                                                 cfg.num_layers * ple, dtype, device)
            self.per_layer_model_projection = ReplicatedLinear(cfg.hidden_size, cfg.num_layers * ple, dtype, device,
                                                               _scheme(cfg, "model.per_layer_model_projection"))
            self.per_layer_projection_norm = RMSNorm(ple, cfg.rms_norm_eps, dtype, device)


def _rounded(value: float, dtype) -> float:
    """The published implementation keeps its embedding scales in the activation dtype."""
    return float(torch.tensor(value, dtype=dtype))


class Gemma4ForCausalLM(BaseOP):
    def __init__(self, cfg: ModelConfig, dtype: torch.dtype, device) -> None:
        self._cfg = cfg
        self.model = Gemma4Body(cfg, dtype, device)
        self.lm_head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, dtype, device,
                                      tied=self.model.embed_tokens if cfg.tie_word_embeddings else None)
        self._ple = int(cfg.hidden_size_per_layer_input)
        self._scales = None

    @property
    def config(self) -> ModelConfig:
        return self._cfg

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        get_comm().row_shard_ok = False
        get_comm().split_k_ok = False
        ctx = get_global_ctx()
        cfg, body = self._cfg, self.model
        capture = ctx.batch.capture_layers
        x = body.embed_tokens.forward(input_ids)
        if self._scales is None or self._scales[0] != x.dtype:
            self._scales = (x.dtype, _rounded(float(cfg.hidden_size) ** 0.5, x.dtype),
                            _rounded(float(max(self._ple, 1)) ** 0.5, x.dtype))
        x = x * self._scales[1]
        if ctx.batch.mm_rows is not None:
            # image placeholder rows take the projected vision features as they are (not scaled)
            x = x.index_copy(0, ctx.batch.mm_rows, ctx.batch.mm_values.to(x.dtype))
        x = self._condition(x, ctx.batch)
        per_layer = None
        if self._ple:
            t, n = x.shape[0], cfg.num_layers
            ids = input_ids
            limit = cfg.vocab_size_per_layer_input or cfg.vocab_size
            # image placeholder rows (ids past the vocabulary) and ids the second table does not have read the
            # padding token's row, as the published model does for soft tokens
            ids = torch.where(ids < min(limit, cfg.vocab_size), ids, torch.full_like(ids, cfg.pad_token_id))
            tok = body.embed_tokens_per_layer.forward(ids) * self._scales[2]
            proj = body.per_layer_model_projection.forward(x) * (float(cfg.hidden_size) ** -0.5)
            proj = body.per_layer_projection_norm.forward(proj.reshape(t * n, self._ple)).view(t, n, self._ple)
            per_layer = (proj + tok.view(t, n, self._ple)) * (2.0 ** -0.5)
        seen = {}
        for i, layer in enumerate(body.layers):
            if capture is not None and i in capture:
                seen[i] = x
            x = layer.forward(x, per_layer[:, i] if per_layer is not None else None)
        x = body.norm.forward(x)
        if capture is not None:
            seen[len(body.layers)] = x
            ctx.aux_hidden = [seen[i] for i in capture]
        return x

    def _condition(self, x: torch.Tensor, batch) -> torch.Tensor:
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


class SelfConditioning(BaseOP):
    """The block a denoising step puts between the embedding and the first layer
    (python/minisgl/models/diffusion_gemma.py:68-100): a dense GeGLU MLP of the decoder's width over the
    normalised signal of the previous step, added to the embedding; the sum is RMS-normalised without a
    weight on every denoising step, the first one (signal zero: the MLP contributes exactly zero) included."""
    _non_persistent = ("_unit",)

    def __init__(self, cfg: ModelConfig, dtype, device) -> None:
        prefix = "model.self_conditioning"
        self.gate_up_proj = MergedColumnParallelLinear(cfg.hidden_size, [cfg.intermediate_size] * 2, dtype, device,
                                                       _scheme(cfg, prefix + ".gate_up_proj"))
        self.down_proj = RowParallelLinear(cfg.intermediate_size, cfg.hidden_size, dtype, device,
                                           _scheme(cfg, prefix + ".down_proj"))
        self.pre_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self._act = GatedActivation(cfg.hidden_act)
        self._eps = cfg.rms_norm_eps
        self._unit = None

    def forward(self, embeds: torch.Tensor, signal: Optional[torch.Tensor]) -> torch.Tensor:
        if signal is not None:
            h = self._act(self.gate_up_proj.forward(self.pre_norm.forward(signal.to(embeds.dtype))))
            embeds = embeds + self.down_proj.forward(h, reduce=True)
        if self._unit is None:
            self._unit = _ones(embeds.shape[-1], embeds)
        return ops.rms_norm(embeds, self._unit, self._eps)


class DiffusionGemmaForBlockDiffusion(Gemma4ForCausalLM):
    """Block diffusion on the Gemma-4 stack (python/minisgl/models/diffusion_gemma.py:103-250). The
    checkpoint's encoder and decoder are one set of weights: the causal pass that writes K/V is the inherited
    forward; a denoising step (``batch.canvas_signal`` set by the diffusion loop) differs only in the
    self-conditioning block on its input and in the batch's attention mask."""

    def __init__(self, cfg: ModelConfig, dtype: torch.dtype, device) -> None:
        super().__init__(cfg, dtype, device)
        self.model.self_conditioning = SelfConditioning(cfg, dtype, device)
        self.self_conditioning_width = cfg.hidden_size

    def _condition(self, x: torch.Tensor, batch) -> torch.Tensor:
        signal = batch.canvas_signal
        if signal is None:
            return x
        return self.model.self_conditioning.forward(x, signal if signal.numel() else None)

    def soft_embedding(self, probs: torch.Tensor) -> torch.Tensor:
        """What a canvas row carries into its next denoising step: its predicted distribution times the
        embedding table, scaled like an embedding. ``probs`` ``[rows, vocab]`` fp32; each rank contracts
        its slice of the vocabulary and the partial sums are added."""
        emb = self.model.embed_tokens
        w = emb.weight[: emb._len]
        local = probs[:, emb._start: emb._start + emb._len].to(w.dtype) @ w
        if emb._tp.size > 1:
            local = get_comm().all_reduce(local)
        return local * _rounded(float(self._cfg.hidden_size) ** 0.5, w.dtype)
