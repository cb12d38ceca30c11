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


class MTPDraft(BaseOP):
    def __init__(self, cfg: ModelConfig, dtype, device, target) -> None:
        from ..models.qwen3_5 import HybridDecoderLayer

        self._cfg = cfg
        self._dtype, self._device = dtype, torch.device(device)
        self._target = target
        h = cfg.hidden_size
        self.pre_fc_norm_embedding = RMSNorm(h, cfg.rms_norm_eps, dtype, device, plus_one=True)
        self.pre_fc_norm_hidden = RMSNorm(h, cfg.rms_norm_eps, dtype, device, plus_one=True)
        self.fc = ReplicatedLinear(2 * h, h, dtype, device)
        self._lcfg = mtp_layer_config(cfg)
        self.layer = HybridDecoderLayer(self._lcfg, 0, 0, 0, dtype, device)
        self.norm = RMSNorm(h, cfg.rms_norm_eps, dtype, device, plus_one=True)
        tp = get_tp_info().size
        self._hq, self._hk = div_even(cfg.num_qo_heads, tp), div_even(cfg.num_kv_heads, tp, True)
        self._rings: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        self._cos_sin = None
        self._qk_w = None

    # ---- state ----
    def ring(self, uid: int) -> Tuple[torch.Tensor, torch.Tensor]:
        r = self._rings.get(uid)
        if r is None:
            shape = (WINDOW, self._hk, self._cfg.head_dim)
            r = (torch.zeros(shape, dtype=torch.float32, device=self._device),
                 torch.zeros(shape, dtype=torch.float32, device=self._device))
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
        for mod in self.modules():
            if isinstance(mod, RMSNorm):            # (1 + w) convention: the neutral weight is zero
                mod.weight = torch.zeros_like(mod.weight)

    # ---- compute ----
    def fuse_features(self, aux: Sequence[torch.Tensor]) -> torch.Tensor:
        return aux[-1]

    def to_target(self, draft_ids: torch.Tensor) -> torch.Tensor:
        return draft_ids

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
                                cfg.rotary_config.rotary_dim, cfg.rms_norm_eps)
        n = x.shape[0]
        kr, vr = self.ring(uid)
        pos = positions.long()
        kr[pos % WINDOW] = k.float().view(n, hk, d)
        vr[pos % WINDOW] = v.float().view(n, hk, d)
        last = int(pos[-1])
        lo = max(0, last - WINDOW + 1)
        span = torch.arange(lo, last + 1, device=x.device)
        kk = kr[span % WINDOW].permute(1, 0, 2)                       # [hk, S, d]
        vv = vr[span % WINDOW].permute(1, 0, 2)
        g = hq // hk
        qq = q.float().view(n, hk, g, d).permute(1, 2, 0, 3)          # [hk, g, n, d]
        s = torch.einsum("hgqd,hkd->hgqk", qq, kk) * d ** -0.5
        s = s.masked_fill((span[None, :] > pos[:, None])[None, None], float("-inf"))
        o = torch.einsum("hgqk,hkd->hgqd", torch.softmax(s, -1), vv).permute(2, 0, 1, 3).reshape(n, hq * d)
        o = o.to(self._dtype) * torch.sigmoid(gate.float()).to(self._dtype)
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
        h = layer.post_attention_layernorm.forward(x)
        if layer._is_moe:
            m, partial = layer.mlp.forward(h)
            if partial:
                m = get_comm().all_reduce(m)
        else:
            m = layer.mlp.forward(h)
            if get_tp_info().size > 1:
                m = get_comm().all_reduce(m)
        hidden = self.norm.forward(x + m)
        return hidden, self._target.lm_head.forward(hidden[-1:])


def mtp_tensors(path: str) -> Iterator[Tuple[str, torch.Tensor]]:
    """The checkpoint's ``mtp.*`` tensors; the decoder layer's under the names of ``model.layers.0``."""
    from ..models.weight import iter_safetensors

    for name, t in iter_safetensors(path):
        for lead in ("model.language_model.", "language_model."):
            if name.startswith(lead):
                name = name[len(lead):]
        if name.startswith("model.mtp."):
            name = name[len("model."):]
        if not name.startswith("mtp."):
            continue
        if name.startswith("mtp.layers.0."):
            yield "model.layers.0." + name[len("mtp.layers.0."):], t
        else:
            yield name, t


def load_mtp(draft: MTPDraft, path: str) -> int:
    """Fill the head from the target's checkpoint directory. Returns the number of tensors used."""
    from ..models.weight import load_weights

    own = {"mtp.fc.weight": (draft.fc, "weight"), "mtp.norm.weight": (draft.norm, "weight"),
           "mtp.pre_fc_norm_embedding.weight": (draft.pre_fc_norm_embedding, "weight"),
           "mtp.pre_fc_norm_hidden.weight": (draft.pre_fc_norm_hidden, "weight")}
    layer_tensors: List[Tuple[str, torch.Tensor]] = []
    used = 0
    for name, t in mtp_tensors(path):
        if name in own:
            mod, attr = own[name]
            cur = getattr(mod, attr)
            if tuple(cur.shape) != tuple(t.shape):
                raise ValueError(f"{name}: checkpoint shape {tuple(t.shape)} != head {tuple(cur.shape)}")
            setattr(mod, attr, t.to(draft._device, cur.dtype).contiguous())
            used += 1
        elif name.startswith("model.layers.0."):
            layer_tensors.append((name, t))
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
        self.draft = MTPDraft(cfg, eng.dtype, eng.device, eng.model)
        path = config.model_path
        used = 0
        if path and not getattr(config, "use_dummy_weight", False):
            used = load_mtp(self.draft, path)
        if used == 0:
            self.draft.init_dummy(config.seed + 17)
        self.loaded_tensors = used
        self.last_feature: Dict[int, torch.Tensor] = {}
        self.last_pos: Dict[int, int] = {}
