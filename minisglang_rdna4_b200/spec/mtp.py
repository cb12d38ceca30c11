"""Multi-token-prediction head of the target checkpoint as the draft model
(python/minisgl/spec/mtp.py:25-364, python/minisgl/models/qwen3_5.py MTP module).

Qwen3.5 / Qwen3-Next checkpoints carry one extra decoder layer under ``mtp.*`` that predicts the
token after next:

    x      = fc([norm_e(embed(token at p+1)) ‖ norm_h(hidden at p)])
    h      = decoder_layer(x)                      (gated full attention + the model's MLP / MoE)
    hidden = norm(h) ;  draft token at p+2 = argmax(lm_head(hidden))

``hidden at p`` is the target's final (normalised) hidden state for positions the target has run
and the head's own ``hidden`` for positions it is extrapolating. Embedding and LM head are the
target's. The layer is built from the target's own layer class, so it is sharded over the
tensor-parallel ranks and quantised exactly like the decoder; all ranks run the proposer in step on
identical inputs. Its self-attention needs the causal context, not just the draft chain: K/V of
the last ``WINDOW`` positions live in a per-request ring (python/minisgl/spec/mtp.py:98-140).

GLM-4.x MoE / DeepSeek-V3 checkpoints store the head as decoder layer ``model.layers.<num_layers>``
with ``enorm``, ``hnorm``, ``eh_proj`` and ``shared_head.{norm, head}``: the same fusion, a latent-
attention layer, and the state handed to the next extrapolation step is the layer's output before
``shared_head.norm`` (``GlmMTPDraft``).

``MTPProposer`` reuses the chain-drafting logic of the EAGLE3 proposer (features after every prefill
and verify forward, K - 1 single-row extrapolation steps); the speculative step is the
host-driven one.
"""
from __future__ import annotations

from dataclasses import replace
from typing import Dict, Iterator, List, Sequence, Tuple

import torch

from ..layers import BaseOP, RMSNorm, ReplicatedLinear
from ..layers.rotary import get_rope_cache
from ..models.config import ModelConfig
from ..ops import ref
from ..parallel.comm import get_comm
from ..parallel.info import get_tp_info
from ..utils import div_even
from .eagle3 import WINDOW, Eagle3Proposer


class _Layers(BaseOP):
    """``model.layers.0`` of a one-layer decoder: the names the checkpoint loader expects."""

    def __init__(self, layer: BaseOP) -> None:
        self.layers = [layer]


class _OneLayerModel(BaseOP):
    def __init__(self, layer: BaseOP) -> None:
        self.model = _Layers(layer)


def mtp_layer_config(cfg: ModelConfig) -> ModelConfig:
    """The target's config cut down to the one full-attention layer of the head; the MLP kind
    (dense or experts) follows the decoder's last layer."""
    moe = cfg.layer_is_moe(cfg.num_layers - 1)
    return replace(cfg, num_layers=1, layer_types=("full_attention",), mlp_only_layers=() if moe else (0,),
                   first_k_dense_replace=0, decoder_sparse_step=1)


def _ring_attention(q, k, v, ring, positions, scale, dtype):
    """``q [n, hq, d]``, ``k, v [n, hk, d]`` (rotary applied) for ``n`` consecutive positions of one
    request: writes K/V into the ring (slot = position % WINDOW) and attends causally over the last
    ``WINDOW`` positions. Returns ``[n, hq * dv]``."""
    n, hq, d = q.shape
    hk = k.shape[1]
    kr, vr = ring
    pos = positions.long()
    kr[pos % WINDOW] = k.float()
    vr[pos % WINDOW] = v.float()
    last = int(pos[-1])
    span = torch.arange(max(0, last - WINDOW + 1), last + 1, device=q.device)
    kk = kr[span % WINDOW].permute(1, 0, 2)                       # [hk, S, d]
    vv = vr[span % WINDOW].permute(1, 0, 2)
    g = hq // hk
    qq = q.float().view(n, hk, g, d).permute(1, 2, 0, 3)          # [hk, g, n, d]
    s = torch.einsum("hgqd,hkd->hgqk", qq, kk) * scale
    s = s.masked_fill((span[None, :] > pos[:, None])[None, None], float("-inf"))
    o = torch.einsum("hgqk,hkd->hgqd", torch.softmax(s, -1), vv)
    return o.permute(2, 0, 1, 3).reshape(n, hq * vv.shape[-1]).to(dtype)


class _MTPBase(BaseOP):
    """State and plumbing shared by the two checkpoint layouts."""

    def _setup(self, cfg: ModelConfig, dtype, device, target, ring_heads: int, ring_dim: int) -> None:
        self._cfg = cfg
        self._dtype, self._device = dtype, torch.device(device)
        self._target = target
        self._ring_shape = (WINDOW, ring_heads, ring_dim)
        self._rings: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        self._cos_sin = None

    def ring(self, uid: int) -> Tuple[torch.Tensor, torch.Tensor]:
        r = self._rings.get(uid)
        if r is None:
            r = (torch.zeros(self._ring_shape, dtype=torch.float32, device=self._device),
                 torch.zeros(self._ring_shape, dtype=torch.float32, device=self._device))
            self._rings[uid] = r
        return r

    def drop(self, uid: int) -> None:
        self._rings.pop(uid, None)

    def init_dummy(self, seed: int, std: float = 0.02) -> None:
        gen = torch.Generator(device="cpu").manual_seed(seed)
        for mod in self.modules():
            if mod is self:
                continue
            fn = getattr(mod, "init_dummy", None)
            if fn is not None:
                fn(gen, std)
        if self._cfg.norm_plus_one:
            for mod in self.modules():
                if isinstance(mod, RMSNorm):        # (1 + w) convention: the neutral weight is zero
                    mod.weight = torch.zeros_like(mod.weight)

    def fuse_features(self, aux: Sequence[torch.Tensor]) -> torch.Tensor:
        return aux[-1]

    def to_target(self, draft_ids: torch.Tensor) -> torch.Tensor:
        return draft_ids

    def _mlp(self, layer, h: torch.Tensor) -> torch.Tensor:
        out = layer.mlp.forward(h)
        if isinstance(out, tuple):                  # (y, still needs the tensor-parallel sum)
            m, partial = out
            return get_comm().all_reduce(m) if partial else m
        if not layer._is_moe and get_tp_info().size > 1:
            out = get_comm().all_reduce(out)
        return out


class MTPDraft(_MTPBase):
    """Qwen3.5 / Qwen3-Next ``mtp.*``."""

    def __init__(self, cfg: ModelConfig, dtype, device, target) -> None:
        from ..models.qwen3_5 import HybridDecoderLayer

        tp = get_tp_info().size
        self._hq, self._hk = div_even(cfg.num_qo_heads, tp), div_even(cfg.num_kv_heads, tp, True)
        self._setup(cfg, dtype, device, target, self._hk, cfg.head_dim)
        h = cfg.hidden_size
        self.pre_fc_norm_embedding = RMSNorm(h, cfg.rms_norm_eps, dtype, device, plus_one=True)
        self.pre_fc_norm_hidden = RMSNorm(h, cfg.rms_norm_eps, dtype, device, plus_one=True)
        self.fc = ReplicatedLinear(2 * h, h, dtype, device)
        self._lcfg = mtp_layer_config(cfg)
        self.layer = HybridDecoderLayer(self._lcfg, 0, 0, 0, dtype, device, prefix="mtp.layers.0")
        self.norm = RMSNorm(h, cfg.rms_norm_eps, dtype, device, plus_one=True)
        self._qk_w = None

    def _attention(self, uid: int, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        cfg = self._cfg
        attn = self.layer.self_attn
        hq, hk, d = self._hq, self._hk, cfg.head_dim
        if self._cos_sin is None:
            self._cos_sin = get_rope_cache(cfg.rotary_config, x.device)
        if self._qk_w is None:
            self._qk_w = ((attn.q_norm.weight.float() + 1).to(self._dtype), (attn.k_norm.weight.float() + 1).to(self._dtype))
        qkv = attn.qkv_proj.forward(x)
        gate = attn.gate_proj.forward(x)
        q, k, v = qkv.split([hq * d, hk * d, hk * d], dim=-1)
        q, k = ref.qk_norm_rope(q, k, self._qk_w[0], self._qk_w[1], positions, self._cos_sin, d,
                                cfg.rotary_config.rotary_dim, cfg.rms_norm_eps, cfg.rotary_config.interleaved)
        n = x.shape[0]
        o = _ring_attention(q.view(n, hq, d), k.view(n, hk, d), v.view(n, hk, d), self.ring(uid), positions,
                            d ** -0.5, self._dtype)
        o = o * torch.sigmoid(gate.float()).to(self._dtype)
        return attn.o_proj.forward(o, reduce=True)

    def forward_rows(self, uid: int, embeds: torch.Tensor, features: torch.Tensor, positions: torch.Tensor
                     ) -> Tuple[torch.Tensor, torch.Tensor]:
        """``n`` consecutive rows of one request: row i pairs the hidden state of position
        ``positions[i]`` with the embedding of the token after it. Returns ``(hidden [n, H],
        logits of the last row [1, vocab])``; the ring receives the rows' K/V."""
        layer = self.layer
        x = self.fc.forward(torch.cat([self.pre_fc_norm_embedding.forward(embeds.to(self._dtype)),
                                       self.pre_fc_norm_hidden.forward(features.to(self._dtype))], dim=-1))
        x = x + self._attention(uid, layer.input_layernorm.forward(x), positions)
        m = self._mlp(layer, layer.post_attention_layernorm.forward(x))
        hidden = self.norm.forward(x + m)
        return hidden, self._target.lm_head.forward(hidden[-1:])


class _SharedHead(BaseOP):
    def __init__(self, cfg: ModelConfig, dtype, device) -> None:
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)


class GlmMTPDraft(_MTPBase):
    """GLM-4.x MoE / DeepSeek-V3 next-token layer ``model.layers.<num_layers>``."""

    def __init__(self, cfg: ModelConfig, dtype, device, target) -> None:
        from ..models.glm4_moe_lite import GlmDecoderLayer

        self._lcfg = replace(cfg, num_layers=1, first_k_dense_replace=0, mlp_only_layers=(), decoder_sparse_step=1)
        self.layer = GlmDecoderLayer(self._lcfg, 0, dtype, device, prefix=f"model.layers.{cfg.num_layers}")
        attn = self.layer.self_attn
        self._setup(cfg, dtype, device, target, attn._h, attn._d)
        h = cfg.hidden_size
        self.enorm = RMSNorm(h, cfg.rms_norm_eps, dtype, device)
        self.hnorm = RMSNorm(h, cfg.rms_norm_eps, dtype, device)
        self.eh_proj = ReplicatedLinear(2 * h, h, dtype, device)
        self.shared_head = _SharedHead(cfg, dtype, device)

    def _attention(self, uid: int, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        cfg = self._cfg
        a = self.layer.self_attn
        t = x.shape[0]
        h, nope, rope, d = a._h, a._nope, a._rope, a._d
        if self._cos_sin is None:
            self._cos_sin = get_rope_cache(cfg.rotary_config, x.device)
        q = a.q_b_proj.forward(a.q_a_layernorm.forward(a.q_a_proj.forward(x))) if a._q_lora else a.q_proj.forward(x)
        q = q.view(t, h, d)
        ckv = a.kv_a_proj_with_mqa.forward(x)
        latent, k_rot = ckv[:, : a._lora], ckv[:, a._lora:]
        kv = a.kv_b_proj.forward(a.kv_a_layernorm.forward(latent.contiguous())).view(t, h, nope + a._vd)
        # [rope ‖ nope] per head, as the decoder's layers lay their heads out: the rotary channels come first
        qp = torch.cat([q[:, :, nope:], q[:, :, :nope]], dim=-1).reshape(t, h * d)
        kp = torch.cat([k_rot[:, None, :].expand(t, h, rope), kv[:, :, :nope]], dim=-1).reshape(t, h * d)
        qp, kp = ref.qk_norm_rope(qp, kp, None, None, positions, self._cos_sin, d, cfg.rotary_config.rotary_dim,
                                  cfg.rms_norm_eps, cfg.rotary_config.interleaved)
        v = kv[:, :, nope:]
        if a._vd < d:                              # one ring shape for K and V: narrower values are zero-padded
            v = torch.cat([v, v.new_zeros((t, h, d - a._vd))], dim=-1)
        o = _ring_attention(qp.view(t, h, d), kp.view(t, h, d), v, self.ring(uid), positions, a.attn._scale, self._dtype)
        if a._vd < d:
            o = o.view(t, h, d)[:, :, : a._vd].reshape(t, h * a._vd)
        return a.o_proj.forward(o, reduce=True)

    def forward_rows(self, uid: int, embeds: torch.Tensor, features: torch.Tensor, positions: torch.Tensor
                     ) -> Tuple[torch.Tensor, torch.Tensor]:
        """As ``MTPDraft.forward_rows``; the returned hidden state is the layer's output before
        ``shared_head.norm`` (what the next extrapolation step is fed), the logits use the norm."""
        layer = self.layer
        x = self.eh_proj.forward(torch.cat([self.enorm.forward(embeds.to(self._dtype)),
                                            self.hnorm.forward(features.to(self._dtype))], dim=-1))
        x = x + self._attention(uid, layer.input_layernorm.forward(x), positions)
        hidden = x + self._mlp(layer, layer.post_attention_layernorm.forward(x))
        return hidden, self._target.lm_head.forward(self.shared_head.norm.forward(hidden[-1:]))


class Glm4MoeMTPDraft(GlmMTPDraft):
    """GLM-4.5 / 4.6: the same ``model.layers.<num_layers>`` layout around an ordinary grouped-query
    attention layer (q / k / v biases, optional QK norm, partial rotary embedding) and the GLM expert block."""

    def __init__(self, cfg: ModelConfig, dtype, device, target) -> None:
        from ..models.transformer import DecoderLayer

        self._lcfg = replace(cfg, num_layers=1, first_k_dense_replace=0, mlp_only_layers=(), decoder_sparse_step=1,
                             layer_types=None)
        self.layer = DecoderLayer(self._lcfg, 0, dtype, device, prefix=f"model.layers.{cfg.num_layers}")
        tp = get_tp_info().size
        self._hq, self._hk = div_even(cfg.num_qo_heads, tp), div_even(cfg.num_kv_heads, tp, True)
        self._setup(cfg, dtype, device, target, self._hk, cfg.head_dim)
        h = cfg.hidden_size
        self.enorm = RMSNorm(h, cfg.rms_norm_eps, dtype, device)
        self.hnorm = RMSNorm(h, cfg.rms_norm_eps, dtype, device)
        self.eh_proj = ReplicatedLinear(2 * h, h, dtype, device)
        self.shared_head = _SharedHead(cfg, dtype, device)

    def _attention(self, uid: int, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        cfg = self._cfg
        attn = self.layer.self_attn
        hq, hk, d = self._hq, self._hk, cfg.head_dim
        if self._cos_sin is None:
            self._cos_sin = get_rope_cache(cfg.rotary_config, x.device)
        q, k, v = attn.qkv_proj.forward(x).split([hq * d, hk * d, hk * d], dim=-1)
        qw, kw = (attn.q_norm.weight, attn.k_norm.weight) if cfg.qk_norm else (None, None)
        q, k = ref.qk_norm_rope(q, k, qw, kw, positions, self._cos_sin, d, cfg.rotary_config.rotary_dim,
                                cfg.rms_norm_eps, cfg.rotary_config.interleaved)
        n = x.shape[0]
        o = _ring_attention(q.view(n, hq, d), k.view(n, hk, d), v.reshape(n, hk, d), self.ring(uid), positions,
                            d ** -0.5, self._dtype)
        return attn.o_proj.forward(o, reduce=True)


def mtp_tensors(path: str, next_layer: int) -> Iterator[Tuple[str, torch.Tensor]]:
    """The head's tensors of a checkpoint directory: ``mtp.*`` (Qwen layout) or
    ``model.layers.<next_layer>.*`` (GLM / DeepSeek layout); the decoder layer's own tensors come
    out under the names of ``model.layers.0``."""
    from ..models.weight import iter_safetensors

    glm = f"model.layers.{next_layer}."
    own_glm = ("enorm.", "hnorm.", "eh_proj.", "shared_head.", "embed_tokens.")
    for name, t in iter_safetensors(path):
        for lead in ("model.language_model.", "language_model."):
            if name.startswith(lead):
                name = ("model." if lead.startswith("model.") else "") + name[len(lead):]
        if name.startswith("model.mtp."):
            name = name[len("model."):]
        if name.startswith("mtp.layers.0."):
            yield "model.layers.0." + name[len("mtp.layers.0."):], t
        elif name.startswith("mtp."):
            yield name, t
        elif name.startswith(glm):
            tail = name[len(glm):]
            yield ("nextn." + tail if tail.startswith(own_glm) else "model.layers.0." + tail), t


def load_mtp(draft: _MTPBase, path: str) -> int:
    """Fill the head from the target's checkpoint directory. Returns the number of tensors used."""
    from ..models.weight import load_weights

    if isinstance(draft, GlmMTPDraft):
        own = {"nextn.eh_proj.weight": (draft.eh_proj, "weight"), "nextn.enorm.weight": (draft.enorm, "weight"),
               "nextn.hnorm.weight": (draft.hnorm, "weight"),
               "nextn.shared_head.norm.weight": (draft.shared_head.norm, "weight")}
    else:
        own = {"mtp.fc.weight": (draft.fc, "weight"), "mtp.norm.weight": (draft.norm, "weight"),
               "mtp.pre_fc_norm_embedding.weight": (draft.pre_fc_norm_embedding, "weight"),
               "mtp.pre_fc_norm_hidden.weight": (draft.pre_fc_norm_hidden, "weight")}
    layer_tensors: List[Tuple[str, torch.Tensor]] = []
    used = 0
    for name, t in mtp_tensors(path, draft._cfg.num_layers):
        if name in own:
            mod, attr = own[name]
            cur = getattr(mod, attr)
            if tuple(cur.shape) != tuple(t.shape):
                raise ValueError(f"{name}: checkpoint shape {tuple(t.shape)} != head {tuple(cur.shape)}")
            setattr(mod, attr, t.to(draft._device, cur.dtype).contiguous())
            used += 1
        elif name.startswith("model.layers.0."):
            layer_tensors.append((name, t))
        # nextn.embed_tokens / nextn.shared_head.head: copies of the target's embedding and LM head, which are used instead
    if layer_tensors:
        load_weights(_OneLayerModel(draft.layer), path, draft._lcfg, draft._device, tensors=iter(layer_tensors))
        used += len(layer_tensors)
    return used


class MTPProposer(Eagle3Proposer):
    """Chain drafting with the checkpoint's own next-token head."""

    name = "mtp"
    device_step_ok = False          # the captured device step is built around the EAGLE3 head's layout

    def __init__(self, config, scheduler) -> None:
        from .base import Proposer

        Proposer.__init__(self, config.spec_num_draft)
        self.tree_width = 1
        eng = scheduler.engine
        self.engine = eng
        cfg = eng.model_config
        # the head reads the target's final hidden state: "layer" num_layers of the capture list
        self.aux_layers = [cfg.num_layers]
        if cfg.mtp_num_hidden_layers:
            kind = MTPDraft
        else:
            kind = GlmMTPDraft if getattr(cfg, "kv_lora_rank", 0) else Glm4MoeMTPDraft
        self.draft = kind(cfg, eng.dtype, eng.device, eng.model)
        path = config.model_path
        used = 0
        if path and not getattr(config, "use_dummy_weight", False):
            used = load_mtp(self.draft, path)
        if used == 0:
            self.draft.init_dummy(config.seed + 17)
        self.loaded_tensors = used
        self.last_feature: Dict[int, torch.Tensor] = {}
        self.last_pos: Dict[int, int] = {}
