"""Model hyper-parameters, normalised from a Hugging Face ``config.json``.

Covers the dense Llama/Mistral/Qwen2/Qwen3 families, the Qwen2/Qwen3 MoE families, MLA
(DeepSeek/GLM-lite style latent attention) and sliding-window fields. The reference does the
same normalisation in python/minisgl/models/config.py:144-1273.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, replace
from typing import Any, Dict, List, Optional, Tuple

from ..quant.config import QuantConfig


@dataclass(frozen=True)
class RotaryConfig:
    head_dim: int
    rotary_dim: int
    max_position: int
    base: float
    scaling: Optional[Dict[str, Any]] = None  # llama3 / yarn / linear / dynamic parameters
    interleaved: bool = False                 # GPT-J pairing (x0,x1) instead of NeoX halves

    def key(self) -> Tuple:
        return (
            self.head_dim,
            self.rotary_dim,
            self.max_position,
            self.base,
            json.dumps(self.scaling, sort_keys=True) if self.scaling else None,
            self.interleaved,
        )


@dataclass(frozen=True)
class ModelConfig:
    num_layers: int
    num_qo_heads: int
    num_kv_heads: int
    head_dim: int
    hidden_size: int
    vocab_size: int
    intermediate_size: int
    rms_norm_eps: float
    rotary_config: RotaryConfig
    hidden_act: str = "silu"
    tie_word_embeddings: bool = False
    model_type: str = "llama"
    architectures: Tuple[str, ...] = ("LlamaForCausalLM",)
    attention_bias: bool = False
    mlp_bias: bool = False
    qk_norm: bool = False
    # mixture of experts
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    shared_expert_intermediate_size: int = 0
    shared_expert_gate: bool = False
    decoder_sparse_step: int = 1
    mlp_only_layers: Tuple[int, ...] = ()
    first_k_dense_replace: int = 0
    n_shared_experts: int = 0
    routed_scaling_factor: float = 1.0
    scoring_func: str = "softmax"
    n_group: int = 1
    topk_group: int = 1
    # latent attention
    kv_lora_rank: Optional[int] = None
    q_lora_rank: Optional[int] = None
    qk_nope_head_dim: Optional[int] = None
    qk_rope_head_dim: Optional[int] = None
    v_head_dim: Optional[int] = None
    # gated delta net (linear-attention layers of the Qwen3.5 / Qwen3-Next hybrid family)
    linear_num_key_heads: int = 0
    linear_num_value_heads: int = 0
    linear_key_head_dim: int = 0
    linear_value_head_dim: int = 0
    linear_conv_kernel_dim: int = 4
    # Mamba-2 mixers (Nemotron-H hybrid family): layer_types entries "mamba" / "attention" / "moe" / "mlp"
    mamba_num_heads: int = 0
    mamba_head_dim: int = 0
    ssm_state_size: int = 0
    mamba_n_groups: int = 1
    mamba_conv_bias: bool = True
    mamba_proj_bias: bool = False
    time_step_min: float = 0.0
    moe_latent_size: Optional[int] = None
    mlp_hidden_act: str = "silu"          # "relu2": non-gated squared-ReLU MLPs and experts
    attn_output_gate: bool = False        # q_proj also emits a per-head sigmoid gate of the attention output
    norm_plus_one: bool = False           # RMSNorm weights are stored as (w - 1)
    # misc
    sliding_window: Optional[int] = None
    layer_types: Optional[Tuple[str, ...]] = None
    final_logit_softcapping: Optional[float] = None
    # Gemma family
    query_pre_attn_scalar: Optional[float] = None   # attention scale = this ** -0.5 (default head_dim)
    rope_local_base_freq: Optional[float] = None    # RoPE base of the sliding-window layers
    # Gemma-4: global layers with their own head width / K/V head count, keys reused as values, the last
    # layers reading the K/V of an earlier layer of their kind, per-layer input embeddings
    global_head_dim: Optional[int] = None
    num_global_kv_heads: Optional[int] = None
    attention_k_eq_v: bool = False
    num_kv_shared_layers: int = 0
    hidden_size_per_layer_input: int = 0
    vocab_size_per_layer_input: int = 0
    use_double_wide_mlp: bool = False
    enable_moe_block: bool = False
    num_nextn_predict_layers: int = 0
    mtp_num_hidden_layers: int = 0            # Qwen3.5 / Qwen3-Next: decoder layers stored under mtp.*
    canvas_length: int = 0                    # block-diffusion models: tokens written per block
    vision: Any = None                        # models.siglip.VisionConfig of a multimodal checkpoint
    # Muse-Glimmer: the two post-norms of a layer have an epsilon of their own, layers whose rotary base is 0
    # have no positional encoding, logits are multiplied before the soft cap, queries are scaled after their norm
    # Laguna: a query-head count per layer and a rotary table of their own for the sliding layers
    attn_head_counts: Optional[Tuple[int, ...]] = None
    sliding_rotary: Optional[RotaryConfig] = None
    post_norm_eps: Optional[float] = None
    layer_rope_theta: Optional[Tuple[float, ...]] = None
    output_multiplier: Optional[float] = None
    qk_scale_factor: Optional[float] = None
    image_bidirectional: bool = True          # the tokens of one image see each other in both directions in the prefill
    pad_token_id: int = 0
    mask_token_id: Optional[int] = None       # absorbing-state diffusion models
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"
    max_position_embeddings: int = 32768
    quant: Optional[QuantConfig] = None
    # EAGLE3 draft head fields
    draft_vocab_size: Optional[int] = None
    eagle_aux_layers: Optional[Tuple[int, ...]] = None

    # ---- derived ----
    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def is_mla(self) -> bool:
        return self.kv_lora_rank is not None

    @property
    def is_recurrent(self) -> bool:
        """Some layers keep a recurrent state per request instead of K/V pages."""
        return bool(self.layer_types) and any(t in ("linear_attention", "mamba") for t in self.layer_types)

    @property
    def num_linear_layers(self) -> int:
        """Layers with a recurrent state (gated delta net or Mamba-2)."""
        return sum(1 for t in (self.layer_types or ()) if t in ("linear_attention", "mamba"))

    @property
    def num_kv_layers(self) -> int:
        """Layers that keep K/V pages."""
        if self.model_type == "nemotron_h":
            return sum(1 for t in (self.layer_types or ()) if t == "attention")
        return self.num_layers - self.num_linear_layers - self.num_kv_shared_layers

    @property
    def swa_layers(self) -> Tuple[int, ...]:
        """Decoder layers whose attention only looks at the last ``sliding_window`` positions (of those
        that keep K/V of their own)."""
        if not self.sliding_window or self.is_recurrent:
            return ()
        if self.layer_types:
            own = self.num_layers - self.num_kv_shared_layers
            return tuple(i for i, t in enumerate(self.layer_types[:own]) if t == "sliding_attention")
        return tuple(range(self.num_layers)) if self.model_type == "mistral" else ()

    def kv_donor(self, layer: int) -> Optional[int]:
        """The earlier layer whose K/V ``layer`` reads instead of keeping its own: the last layer of the
        same kind before the shared range (Gemma-4). ``None`` for a layer with K/V of its own."""
        first = self.num_layers - self.num_kv_shared_layers
        if not self.num_kv_shared_layers or layer < first:
            return None
        kind = self.layer_types[layer]
        return max(i for i in range(first) if self.layer_types[i] == kind)

    def attn_geometry(self, layer: int) -> Tuple[int, int]:
        """``(kv heads, head width)`` of a layer's attention."""
        if self.global_head_dim and self.layer_types and self.layer_types[layer] != "sliding_attention":
            heads = self.num_global_kv_heads if (self.attention_k_eq_v and self.num_global_kv_heads) \
                else self.num_kv_heads
            return int(heads), int(self.global_head_dim)
        return self.num_kv_heads, self.head_dim

    @property
    def mixed_kv_geometry(self) -> bool:
        return len({self.attn_geometry(i) for i in range(self.num_kv_layers)}) > 1 if self.global_head_dim else False

    @property
    def recurrent_geometry(self) -> Tuple[int, int, int, int]:
        """``(conv channels, heads, rows, cols)`` of one recurrent layer's state: a convolution window
        over ``conv channels`` inputs and a ``[heads, rows, cols]`` fp32 state matrix per request."""
        if self.mamba_num_heads:
            inter = self.mamba_num_heads * self.mamba_head_dim
            return (inter + 2 * self.mamba_n_groups * self.ssm_state_size, self.mamba_num_heads, self.mamba_head_dim,
                    self.ssm_state_size)
        return (2 * self.linear_num_key_heads * self.linear_key_head_dim
                + self.linear_num_value_heads * self.linear_value_head_dim,
                self.linear_num_value_heads, self.linear_key_head_dim, self.linear_value_head_dim)

    @property
    def q_size(self) -> int:
        return self.num_qo_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    def layer_is_moe(self, layer: int) -> bool:
        if not self.is_moe or layer in self.mlp_only_layers:
            return False
        if layer < self.first_k_dense_replace:
            return False
        return (layer + 1) % max(self.decoder_sparse_step, 1) == 0

    def with_quant(self, quant: Optional[QuantConfig]) -> "ModelConfig":
        return replace(self, quant=quant)

    def param_count(self) -> int:
        """Parameter count of the unquantised model (used for memory planning)."""
        h, v = self.hidden_size, self.vocab_size
        attn = h * (self.q_size + 2 * self.kv_size) + self.q_size * h
        total = v * h * (1 if self.tie_word_embeddings else 2)
        for layer in range(self.num_layers):
            total += attn + 2 * h
            if self.layer_is_moe(layer):
                total += self.num_experts * 3 * h * self.moe_intermediate_size + h * self.num_experts
                total += 3 * h * self.shared_expert_intermediate_size
            else:
                total += 3 * h * self.intermediate_size
        return total

    # ---- construction ----
    @staticmethod
    def from_hf(cfg: Any) -> "ModelConfig":
        """Build from a dict, a ``transformers`` config object or a path to ``config.json``."""
        if isinstance(cfg, (str, os.PathLike)):
            path = os.fspath(cfg)
            if os.path.isdir(path):
                path = os.path.join(path, "config.json")
            with open(path) as fh:
                cfg = json.load(fh)
        if not isinstance(cfg, dict):
            cfg = cfg.to_dict()
        vision = None
        if "text_config" in cfg and isinstance(cfg["text_config"], dict):
            if str(cfg.get("model_type", "")).startswith("gemma3") and cfg.get("vision_config"):
                from .siglip import VisionConfig

                vision = VisionConfig.from_hf(cfg)
            elif str(cfg.get("model_type", "")) in ("gemma4", "diffusion_gemma") and cfg.get("vision_config"):
                from .gemma4_vision import Gemma4VisionConfig

                vision = Gemma4VisionConfig.from_hf(cfg)
            inner = dict(cfg["text_config"])
            for key in ("quantization_config", "architectures", "torch_dtype", "tie_word_embeddings", "canvas_length",
                        "mask_token_id"):
                if key in cfg and key not in inner:
                    inner[key] = cfg[key]
            cfg = inner
        g = cfg.get
        model_type = g("model_type", "llama")
        archs = tuple(g("architectures") or _default_arch(model_type))
        heads = int(g("num_attention_heads"))
        hidden = int(g("hidden_size"))
        head_dim = int(g("head_dim") or hidden // heads)
        kv_heads = int(g("num_key_value_heads") or heads)
        max_pos = int(g("max_position_embeddings", 32768))
        rope_params = g("rope_parameters") or {}
        scaling = g("rope_scaling") or ({k: v for k, v in rope_params.items() if k != "rope_theta"} or None)
        if scaling and scaling.get("rope_type", scaling.get("type", "default")) in ("default", None):
            scaling = None
        theta = float(g("rope_theta") or rope_params.get("rope_theta") or 10000.0)
        partial = float(g("partial_rotary_factor") or rope_params.get("partial_rotary_factor") or 1.0)
        rope_dim = int(g("qk_rope_head_dim") or 0) or int(head_dim * partial)
        rotary = RotaryConfig(
            head_dim=head_dim, rotary_dim=rope_dim, max_position=max_pos, base=theta, scaling=scaling
        )
        eos = g("eos_token_id")
        eos_ids = tuple(eos) if isinstance(eos, (list, tuple)) else (() if eos is None else (int(eos),))
        num_experts = int(g("num_experts") or g("num_local_experts") or g("n_routed_experts") or 0)
        quant = QuantConfig.from_hf(g("quantization_config")) if g("quantization_config") else None
        layer_types = g("layer_types")
        gdn_family = model_type in ("qwen3_5", "qwen3_5_text", "qwen3_5_moe", "qwen3_5_moe_text", "qwen3_next")
        qk_norm = (model_type in ("qwen3", "qwen3_moe", "gemma3", "gemma3_text") or gdn_family
                   or bool(g("use_qk_norm", False)))
        if gdn_family:
            if layer_types is None:
                every = int(g("full_attention_interval") or 4)
                layer_types = ["linear_attention" if (i + 1) % every else "full_attention"
                               for i in range(int(g("num_hidden_layers")))]
            if partial == 1.0 and "partial_rotary_factor" not in cfg and "partial_rotary_factor" not in rope_params:
                rope_dim = head_dim // 4
                rotary = RotaryConfig(head_dim=head_dim, rotary_dim=rope_dim, max_position=max_pos, base=theta,
                                      scaling=scaling)
            if archs and not any(a.startswith("Qwen3_5") or a.startswith("Qwen3Next") for a in archs):
                archs = ("Qwen3_5ForCausalLM",)
        if layer_types is None and model_type in ("gemma3", "gemma3_text") and g("sliding_window_pattern"):
            pat = int(g("sliding_window_pattern"))
            layer_types = ["full_attention" if (i + 1) % pat == 0 else "sliding_attention"
                           for i in range(int(g("num_hidden_layers")))]
        if layer_types is None and model_type == "gemma2":
            layer_types = ["sliding_attention" if i % 2 == 0 else "full_attention"
                           for i in range(int(g("num_hidden_layers")))]
        sliding_rotary = None
        local_theta = g("rope_local_base_freq")
        if local_theta is None and isinstance(rope_params.get("sliding_attention"), dict):
            local_theta = rope_params["sliding_attention"].get("rope_theta")
        muse = model_type in ("muse_glimmer", "muse_glimmer_text")
        if muse:
            cfg = dict(cfg, hidden_act=g("hidden_act") or g("hidden_activation") or "silu")
            g = cfg.get
        gemma4 = model_type in ("gemma4", "gemma4_text", "diffusion_gemma", "diffusion_gemma_text")
        if model_type.startswith("diffusion_gemma") and "attention_k_eq_v" not in cfg:
            # the block-diffusion variant's config does not carry the field; its global layers have no
            # value projection all the same
            cfg = dict(cfg, attention_k_eq_v=True)
            g = cfg.get
        if isinstance(rope_params.get("full_attention"), dict):  # per-layer-type RoPE tables
            full = rope_params["full_attention"]
            theta = float(full.get("rope_theta", theta))
            scaling = {k: v for k, v in full.items() if k != "rope_theta"} or None
            if scaling and scaling.get("rope_type", "default") in ("default", None):
                scaling = None
            g_dim = int(g("global_head_dim") or head_dim) if gemma4 else head_dim
            if full.get("partial_rotary_factor") and not gemma4:
                rope_dim = int(head_dim * float(full["partial_rotary_factor"]))
            rotary = RotaryConfig(head_dim=g_dim, rotary_dim=g_dim if gemma4 else rope_dim, max_position=max_pos,
                                  base=theta, scaling=scaling)
            sub = rope_params.get("sliding_attention")
            if isinstance(sub, dict) and model_type == "laguna":
                sub_scaling = {k: v for k, v in sub.items() if k != "rope_theta"} or None
                if sub_scaling and sub_scaling.get("rope_type", "default") in ("default", None):
                    sub_scaling = None
                sliding_rotary = RotaryConfig(head_dim=head_dim,
                                              rotary_dim=int(head_dim * float(sub.get("partial_rotary_factor") or 1.0)),
                                              max_position=max_pos, base=float(sub.get("rope_theta", theta)),
                                              scaling=sub_scaling)
        if gemma4:
            if layer_types is None:
                layer_types = ["sliding_attention" if (i + 1) % 6 else "full_attention"
                               for i in range(int(g("num_hidden_layers")))]
            layer_types = list(layer_types)
            layer_types[-1] = "full_attention"
            cfg = dict(cfg, hidden_act=g("hidden_activation", "gelu_pytorch_tanh"),
                       num_experts_per_tok=g("top_k_experts"), tie_word_embeddings=g("tie_word_embeddings", True),
                       num_experts=g("num_experts") if g("enable_moe_block") else 0)
            g = cfg.get
            num_experts = int(g("num_experts") or 0)
        if g("kv_lora_rank"):
            # latent attention: the pool holds materialised per-head keys of qk_nope + qk_rope channels;
            # the rotary part is GPT-J interleaved unless the checkpoint says otherwise
            # (where the value head is narrower than that, or the width is not one the attention kernels
            # are built for, keys, queries and values are zero-padded to a common width: DeepSeek-V2/V3's
            # 128 + 64 key channels and 128 value channels are stored 256 wide)
            head_dim = max(int(g("qk_nope_head_dim")) + int(g("qk_rope_head_dim")), int(g("v_head_dim") or 0))
            if head_dim > 64 and head_dim not in (128, 256):
                head_dim = 128 if head_dim < 128 else 256 if head_dim < 256 else head_dim
            kv_heads = heads
            rotary = RotaryConfig(head_dim=head_dim, rotary_dim=int(g("qk_rope_head_dim")), max_position=max_pos,
                                  base=theta, scaling=scaling, interleaved=bool(g("rope_interleave", True)))
            if g("mlp_layer_types") and not g("first_k_dense_replace"):
                dense = [i for i, t in enumerate(g("mlp_layer_types")) if t != "sparse"]
                cfg = dict(cfg, mlp_only_layers=dense)
                g = cfg.get
        attn_bias = bool(g("attention_bias", model_type in ("qwen2", "qwen2_moe")))
        if model_type == "nemotron_h":
            # one mixer per layer: M = Mamba-2, * = attention, E = mixture of experts, - = MLP; no rotary embedding
            pattern = g("hybrid_override_pattern")
            names = {"M": "mamba", "*": "attention", "E": "moe", "-": "mlp"}
            layer_types = list(g("layers_block_type") or g("layer_types") or [names[ch] for ch in (pattern or "")])
            if not layer_types:
                raise ValueError("nemotron_h config without layers_block_type / hybrid_override_pattern")
            rotary = RotaryConfig(head_dim=head_dim, rotary_dim=0, max_position=max_pos, base=theta)
            cfg = dict(cfg, num_hidden_layers=len(layer_types), rms_norm_eps=g("layer_norm_epsilon", g("rms_norm_eps", 1e-5)),
                       shared_expert_intermediate_size=g("moe_shared_expert_intermediate_size") or 0,
                       scoring_func="sigmoid")
            g = cfg.get
        return ModelConfig(
            num_layers=int(g("num_hidden_layers")),
            num_qo_heads=heads,
            num_kv_heads=kv_heads,
            head_dim=head_dim,
            hidden_size=hidden,
            vocab_size=int(g("vocab_size")),
            intermediate_size=int(g("intermediate_size") or 0),
            rms_norm_eps=float(g("rms_norm_eps", 1e-6)),
            rotary_config=rotary,
            hidden_act=g("hidden_act", "silu"),
            tie_word_embeddings=bool(g("tie_word_embeddings", False)),
            model_type=model_type,
            architectures=archs,
            attention_bias=attn_bias,
            mlp_bias=bool(g("mlp_bias", False)),
            qk_norm=qk_norm,
            num_experts=num_experts,
            num_experts_per_tok=int(g("num_experts_per_tok") or 0),
            # Mixtral's experts have the width its config calls intermediate_size
            moe_intermediate_size=int(g("moe_intermediate_size") or (g("intermediate_size") if model_type == "mixtral" else 0) or 0),
            norm_topk_prob=bool(g("norm_topk_prob", True)),
            shared_expert_intermediate_size=int(g("shared_expert_intermediate_size") or 0),
            # a sigmoid gate on the shared expert's output: Qwen2-MoE and the Qwen3.5 / Qwen3-Next MoE blocks
            shared_expert_gate=model_type in ("qwen2_moe", "qwen3_5_moe", "qwen3_5_moe_text", "qwen3_next"),
            decoder_sparse_step=int(g("decoder_sparse_step") or 1),
            mlp_only_layers=tuple(g("mlp_only_layers") or ()),
            first_k_dense_replace=int(g("first_k_dense_replace") or 0),
            n_shared_experts=int(g("n_shared_experts") or 0),
            routed_scaling_factor=float(g("routed_scaling_factor") or 1.0),
            scoring_func=g("scoring_func", "sigmoid" if model_type in ("glm4_moe_lite", "glm4_moe", "deepseek_v3", "laguna")
                           else "softmax"),
            # DeepSeek-V2's plain "greedy" top-k ignores the routing groups its config still lists
            n_group=1 if g("topk_method") == "greedy" else int(g("n_group") or 1),
            topk_group=int(g("topk_group") or 1),
            kv_lora_rank=g("kv_lora_rank"),
            q_lora_rank=g("q_lora_rank"),
            qk_nope_head_dim=g("qk_nope_head_dim"),
            qk_rope_head_dim=g("qk_rope_head_dim"),
            v_head_dim=g("v_head_dim"),
            linear_num_key_heads=int(g("linear_num_key_heads") or 0),
            linear_num_value_heads=int(g("linear_num_value_heads") or 0),
            linear_key_head_dim=int(g("linear_key_head_dim") or 0),
            linear_value_head_dim=int(g("linear_value_head_dim") or 0),
            linear_conv_kernel_dim=int(g("linear_conv_kernel_dim") or g("conv_kernel") or g("mamba_d_conv") or 4),
            mamba_num_heads=int(g("mamba_num_heads") or 0),
            mamba_head_dim=int(g("mamba_head_dim") or 0),
            ssm_state_size=int(g("ssm_state_size") or 0),
            mamba_n_groups=int(g("n_groups") or g("mamba_n_groups") or 1),
            mamba_conv_bias=bool(g("use_conv_bias", g("mamba_conv_bias", True))),
            mamba_proj_bias=bool(g("mamba_proj_bias", g("use_bias", False))),
            time_step_min=float(g("time_step_min") or g("mamba_dt_min") or 0.0) if model_type == "nemotron_h" else 0.0,
            moe_latent_size=g("moe_latent_size"),
            mlp_hidden_act=g("mlp_hidden_act", "silu"),
            attn_output_gate=gdn_family,
            norm_plus_one=gdn_family,
            sliding_window=g("sliding_window") if g("use_sliding_window", True) else None,
            layer_types=tuple(layer_types) if layer_types else None,
            final_logit_softcapping=g("final_logit_softcapping"),
            query_pre_attn_scalar=g("query_pre_attn_scalar"),
            rope_local_base_freq=float(local_theta) if local_theta else None,
            global_head_dim=int(g("global_head_dim") or 0) or None if gemma4 else None,
            num_global_kv_heads=g("num_global_key_value_heads") if gemma4 else None,
            attention_k_eq_v=bool(g("attention_k_eq_v", False)) if gemma4 else False,
            num_kv_shared_layers=int(g("num_kv_shared_layers") or 0) if gemma4 else 0,
            hidden_size_per_layer_input=int(g("hidden_size_per_layer_input") or 0) if gemma4 else 0,
            vocab_size_per_layer_input=int(g("vocab_size_per_layer_input") or 0) if gemma4 else 0,
            use_double_wide_mlp=bool(g("use_double_wide_mlp", False)) if gemma4 else False,
            enable_moe_block=bool(g("enable_moe_block", False)) if gemma4 else False,
            num_nextn_predict_layers=int(g("num_nextn_predict_layers") or 0),
            mtp_num_hidden_layers=int(g("mtp_num_hidden_layers") or 0),
            canvas_length=int(g("canvas_length") or g("block_length") or 0),
            vision=vision,
            attn_head_counts=tuple(int(h) for h in g("num_attention_heads_per_layer")) if g("num_attention_heads_per_layer") else None,
            sliding_rotary=sliding_rotary,
            post_norm_eps=g("post_norm_eps") if muse else None,
            layer_rope_theta=tuple(float(x) for x in g("layer_rope_theta")) if muse and g("layer_rope_theta") else None,
            output_multiplier=g("output_multiplier") if muse else None,
            qk_scale_factor=float(g("qk_scale_factor") or 3.87) if muse else None,
            image_bidirectional=(g("use_bidirectional_attention") == "vision") if gemma4 else True,
            pad_token_id=int(g("pad_token_id") or 0),
            mask_token_id=g("mask_token_id"),
            eos_token_ids=eos_ids,
            bos_token_id=g("bos_token_id"),
            torch_dtype=str(g("torch_dtype") or g("dtype") or "bfloat16").replace("torch.", ""),
            max_position_embeddings=max_pos,
            quant=quant,
            draft_vocab_size=g("draft_vocab_size"),
            eagle_aux_layers=tuple(g("eagle_aux_hidden_state_layer_ids") or ()) or None,
        )


def _default_arch(model_type: str) -> List[str]:
    return {
        "llama": ["LlamaForCausalLM"],
        "mistral": ["MistralForCausalLM"],
        "mixtral": ["MixtralForCausalLM"],
        "qwen2": ["Qwen2ForCausalLM"],
        "qwen2_moe": ["Qwen2MoeForCausalLM"],
        "qwen3": ["Qwen3ForCausalLM"],
        "qwen3_moe": ["Qwen3MoeForCausalLM"],
        "gemma2": ["Gemma2ForCausalLM"],
        "gemma3": ["Gemma3ForCausalLM"],
        "gemma3_text": ["Gemma3ForCausalLM"],
        "gemma4": ["Gemma4ForCausalLM"],
        "gemma4_text": ["Gemma4ForCausalLM"],
        "laguna": ["LagunaForCausalLM"],
        "muse_glimmer": ["MuseGlimmerForConditionalGeneration"],
        "muse_glimmer_text": ["MuseGlimmerForConditionalGeneration"],
        "diffusion_gemma": ["DiffusionGemmaForBlockDiffusion"],
        "diffusion_gemma_text": ["DiffusionGemmaForBlockDiffusion"],
        "glm4_moe_lite": ["Glm4MoeLiteForCausalLM"],
        "glm4_moe": ["Glm4MoeForCausalLM"],
        "deepseek_v2": ["DeepseekV2ForCausalLM"],
        "deepseek_v3": ["DeepseekV3ForCausalLM"],
        "qwen3_5": ["Qwen3_5ForCausalLM"],
        "qwen3_5_text": ["Qwen3_5ForCausalLM"],
        "qwen3_5_moe": ["Qwen3_5MoeForCausalLM"],
        "qwen3_5_moe_text": ["Qwen3_5MoeForCausalLM"],
        "qwen3_next": ["Qwen3NextForCausalLM"],
        "nemotron_h": ["NemotronHForCausalLM"],
    }.get(model_type, ["LlamaForCausalLM"])


# --------------------------------------------------------------------------------------------
# Named shapes used by the benchmark configurations (random-init, no checkpoint on disk).
# --------------------------------------------------------------------------------------------
def _rot(head_dim: int, theta: float, max_pos: int = 40960) -> RotaryConfig:
    return RotaryConfig(head_dim=head_dim, rotary_dim=head_dim, max_position=max_pos, base=theta)


def tiny_llama_config() -> ModelConfig:
    """2 layers, hidden 256, 4 q / 2 kv heads of 64, SwiGLU 512, vocab 1024 (CPU oracle run)."""
    return ModelConfig(
        num_layers=2, num_qo_heads=4, num_kv_heads=2, head_dim=64, hidden_size=256,
        vocab_size=1024, intermediate_size=512, rms_norm_eps=1e-6,
        rotary_config=_rot(64, 1e6, 4096), model_type="llama", torch_dtype="float32",
        max_position_embeddings=4096,
    )


def qwen3_4b_config(quant: Optional[QuantConfig] = None) -> ModelConfig:
    return ModelConfig(
        num_layers=36, num_qo_heads=32, num_kv_heads=8, head_dim=128, hidden_size=2560,
        vocab_size=151936, intermediate_size=9728, rms_norm_eps=1e-6,
        rotary_config=_rot(128, 1e6), model_type="qwen3",
        architectures=("Qwen3ForCausalLM",), qk_norm=True, tie_word_embeddings=True,
        max_position_embeddings=40960, quant=quant,
    )


def qwen3_8b_config(quant: Optional[QuantConfig] = None) -> ModelConfig:
    return ModelConfig(
        num_layers=36, num_qo_heads=32, num_kv_heads=8, head_dim=128, hidden_size=4096,
        vocab_size=151936, intermediate_size=12288, rms_norm_eps=1e-6,
        rotary_config=_rot(128, 1e6), model_type="qwen3",
        architectures=("Qwen3ForCausalLM",), qk_norm=True, max_position_embeddings=40960,
        quant=quant,
    )


def qwen3_30b_a3b_config(quant: Optional[QuantConfig] = None) -> ModelConfig:
    return ModelConfig(
        num_layers=48, num_qo_heads=32, num_kv_heads=4, head_dim=128, hidden_size=2048,
        vocab_size=151936, intermediate_size=6144, rms_norm_eps=1e-6,
        rotary_config=_rot(128, 1e6), model_type="qwen3_moe",
        architectures=("Qwen3MoeForCausalLM",), qk_norm=True, num_experts=128,
        num_experts_per_tok=8, moe_intermediate_size=768, norm_topk_prob=True,
        max_position_embeddings=40960, quant=quant,
    )


def llama3_70b_config(quant: Optional[QuantConfig] = None) -> ModelConfig:
    return ModelConfig(
        num_layers=80, num_qo_heads=64, num_kv_heads=8, head_dim=128, hidden_size=8192,
        vocab_size=128256, intermediate_size=28672, rms_norm_eps=1e-5,
        rotary_config=_rot(128, 5e5, 8192), model_type="llama",
        architectures=("LlamaForCausalLM",), max_position_embeddings=8192, quant=quant,
    )


NAMED_CONFIGS = {
    "tiny-llama": tiny_llama_config,
    "qwen3-4b": qwen3_4b_config,
    "qwen3-8b": qwen3_8b_config,
    "qwen3-30b-a3b": qwen3_30b_a3b_config,
    "llama3-70b": llama3_70b_config,
}
