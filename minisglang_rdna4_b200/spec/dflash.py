"""DFlash: a block-diffusion draft model (python/minisgl/models/dflash.py:1-901,
python/minisgl/spec/dflash.py:230-1777; the tied-vocabulary checkpoint dialect).

A few standard decoder layers (grouped-query attention with per-head q/k norms, SwiGLU) that propose a
whole block in ONE forward instead of token by token:

    context  = hidden_norm(fc([target hidden states of the chosen layers, concatenated]))   per position
    block    = embed([confirmed token, mask, mask, ...])                                     B rows
    layer:     Q from the block; K, V from [context ‖ block]; attention in both directions
    drafts   = argmax(lm_head(norm(block)))[1:]                                              B - 1 tokens

The context rows' K/V depend only on target hidden states of committed positions, so each position is
projected once per layer and kept (a list per request, trimmed to ``WINDOW`` positions). Embedding and LM
head are the target's. Verification is the ordinary chain verification, so a drafted token can only
change the acceptance rate, never the output.

Host-driven, tensor ops; the drafter is replicated on every tensor-parallel rank (its logits come from the
target's sharded head). Not built: the checkpoint dialects with a pruned vocabulary, a Markov or confidence
head, gated (Laguna) or convolutional (CCA) trunks, per-layer causal / windowed masks, captured graphs.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import ops
from ..core import Req
from ..layers import BaseOP, RMSNorm, ReplicatedLinear
from ..layers.rotary import get_rope_cache
from ..models.config import RotaryConfig
from ..ops import ref
from .base import Proposer

WINDOW = 2048          # context positions kept per request


def is_dflash(path: Optional[str]) -> bool:
    if not path or not os.path.isfile(os.path.join(path, "config.json")):
        return False
    with open(os.path.join(path, "config.json")) as fh:
        raw = json.load(fh)
    return bool(raw.get("dflash_config")) or "DFlash" in "".join(raw.get("architectures") or [])


class _Attn(BaseOP):
    def __init__(self, hidden, heads, kv_heads, d, eps, dtype, device) -> None:
        self.q_proj = ReplicatedLinear(hidden, heads * d, dtype, device)
        self.k_proj = ReplicatedLinear(hidden, kv_heads * d, dtype, device)
        self.v_proj = ReplicatedLinear(hidden, kv_heads * d, dtype, device)
        self.o_proj = ReplicatedLinear(heads * d, hidden, dtype, device)
        self.q_norm = RMSNorm(d, eps, dtype, device)
        self.k_norm = RMSNorm(d, eps, dtype, device)


class _MLP(BaseOP):
    def __init__(self, hidden, inter, dtype, device) -> None:
        self.gate_proj = ReplicatedLinear(hidden, inter, dtype, device)
        self.up_proj = ReplicatedLinear(hidden, inter, dtype, device)
        self.down_proj = ReplicatedLinear(inter, hidden, dtype, device)


class _Layer(BaseOP):
    def __init__(self, hidden, inter, heads, kv_heads, d, eps, dtype, device) -> None:
        self.input_layernorm = RMSNorm(hidden, eps, dtype, device)
        self.self_attn = _Attn(hidden, heads, kv_heads, d, eps, dtype, device)
        self.post_attention_layernorm = RMSNorm(hidden, eps, dtype, device)
        self.mlp = _MLP(hidden, inter, dtype, device)


class DFlashDraft(BaseOP):
    def __init__(self, raw: dict, num_aux: int, dtype, device) -> None:
        g = raw.get
        hidden, heads = int(g("hidden_size")), int(g("num_attention_heads"))
        self.hidden, self.heads, self.kv_heads = hidden, heads, int(g("num_key_value_heads") or heads)
        self.d = int(g("head_dim") or hidden // heads)
        self.eps = float(g("rms_norm_eps", 1e-6))
        rp = g("rope_parameters") or g("rope_scaling") or {}
        theta = float(rp.get("rope_theta") or g("rope_theta") or 1e6)
        scaling = {k: v for k, v in rp.items() if k != "rope_theta"} or None
        if scaling and scaling.get("rope_type", scaling.get("type", "default")) in ("default", None):
            scaling = None
        self.rotary = RotaryConfig(head_dim=self.d, rotary_dim=self.d,
                                   max_position=int(g("max_position_embeddings", 32768)), base=theta, scaling=scaling)
        self.fc = ReplicatedLinear(num_aux * hidden, hidden, dtype, device)
        self.hidden_norm = RMSNorm(hidden, self.eps, dtype, device)
        self.layers = [_Layer(hidden, int(g("intermediate_size")), heads, self.kv_heads, self.d, self.eps, dtype, device)
                       for _ in range(int(g("num_hidden_layers")))]
        self.norm = RMSNorm(hidden, self.eps, dtype, device)
        self._cos_sin = None
        self._device = torch.device(device)

    def _table(self) -> torch.Tensor:
        if self._cos_sin is None:
            self._cos_sin = get_rope_cache(self.rotary, self._device)
        return self._cos_sin

    def project_context(self, aux_rows: Sequence[torch.Tensor], positions: torch.Tensor
                        ) -> List[Tuple[torch.Tensor, torch.Tensor]]:
        """Per layer ``(K [m, kv heads, d] with rotary applied, V [m, kv heads, d])`` of ``m`` committed
        positions whose target hidden states are ``aux_rows`` (one ``[m, hidden]`` per chosen layer)."""
        ctx = self.hidden_norm.forward(self.fc.forward(torch.cat([a.to(self.fc.weight.dtype) for a in aux_rows], -1)))
        m = ctx.shape[0]
        out = []
        for layer in self.layers:
            a = layer.self_attn
            k, v = a.k_proj.forward(ctx), a.v_proj.forward(ctx)
            _, k = ref.qk_norm_rope(k[:, : self.d], k, a.k_norm.weight, a.k_norm.weight, positions, self._table(),
                                    self.d, self.d, self.eps, False)
            out.append((k.view(m, self.kv_heads, self.d).float(), v.view(m, self.kv_heads, self.d).float()))
        return out

    def denoise(self, block: torch.Tensor, positions: torch.Tensor, context: List[Tuple[torch.Tensor, torch.Tensor]]
                ) -> torch.Tensor:
        """``block`` ``[B, hidden]`` embeddings of ``[confirmed token, mask, ...]`` → ``[B, hidden]`` (normed)."""
        x = block
        b, h, hk, d = x.shape[0], self.heads, self.kv_heads, self.d
        for layer, (k_ctx, v_ctx) in zip(self.layers, context):
            a = layer.self_attn
            y = layer.input_layernorm.forward(x)
            q, k = ref.qk_norm_rope(a.q_proj.forward(y), a.k_proj.forward(y), a.q_norm.weight, a.k_norm.weight,
                                    positions, self._table(), d, d, self.eps, False)
            kk = torch.cat([k_ctx, k.view(b, hk, d).float()]).permute(1, 0, 2)               # [hk, S, d]
            vv = torch.cat([v_ctx, a.v_proj.forward(y).view(b, hk, d).float()]).permute(1, 0, 2)
            qq = q.view(b, hk, h // hk, d).float().permute(1, 2, 0, 3)                       # [hk, g, B, d]
            s = torch.einsum("hgqd,hkd->hgqk", qq, kk) * d ** -0.5
            o = torch.einsum("hgqk,hkd->hgqd", torch.softmax(s, -1), vv).permute(2, 0, 1, 3).reshape(b, h * d)
            x = x + a.o_proj.forward(o.to(x.dtype))
            y = layer.post_attention_layernorm.forward(x)
            m = layer.mlp
            x = x + m.down_proj.forward(ops.silu_and_mul(torch.cat([m.gate_proj.forward(y), m.up_proj.forward(y)], -1)))
        return self.norm.forward(x)

    def init_dummy(self, seed: int, std: float = 0.05) -> None:
        gen = torch.Generator(device="cpu")
        gen.manual_seed(seed)
        for mod in self.modules():
            fn = getattr(mod, "init_dummy", None)
            if fn is not None and mod is not self:
                fn(gen, std)
        for mod in self.modules():
            if isinstance(mod, RMSNorm):
                mod.weight = torch.ones_like(mod.weight)


class DFlashProposer(Proposer):
    name = "dflash"
    device_step_ok = False

    def __init__(self, config, scheduler) -> None:
        super().__init__(config.spec_num_draft)
        self.tree_width = 1
        eng = scheduler.engine
        self.engine = eng
        path = config.spec_draft_model_path
        with open(os.path.join(path, "config.json")) as fh:
            raw = json.load(fh)
        dfc = dict(raw.get("dflash_config") or {})
        merged = dict(raw, **(raw.get("transformer_layer_config") or {}))
        if int(merged["hidden_size"]) != eng.model_config.hidden_size:
            raise ValueError("the drafter borrows the target's embedding and head: hidden sizes must match")
        if 0 < int(raw.get("draft_vocab_size") or 0) < eng.model_config.vocab_size:
            raise NotImplementedError("DFlash checkpoints with a pruned vocabulary")
        ids = dfc.get("target_layer_ids") or raw.get("target_layer_ids") or raw.get("aux_hidden_state_layer_ids")
        if not ids:
            raise ValueError("the DFlash checkpoint names no target layers to read hidden states from")
        # the drafter reads the OUTPUT of those target layers: entry j + 1 of the capture list is the input of
        # layer j + 1 (the last layer's output comes back after the final norm)
        self.aux_layers = [int(i) + 1 for i in ids]
        self.block = int(dfc.get("block_size") or raw.get("block_size") or 0) or self.num_draft + 1
        mask = dfc.get("mask_token_id", raw.get("mask_token_id"))
        if mask is None:
            raise ValueError("the DFlash checkpoint names no mask token")
        self.mask_token_id = int(mask)
        self.draft = DFlashDraft(merged, len(self.aux_layers), eng.dtype, eng.device)
        if getattr(config, "use_dummy_weight", False) or not any(f.endswith(".safetensors") for f in os.listdir(path)):
            self.draft.init_dummy(config.seed + 17)
        else:
            from ..models.weight import load_weights

            load_weights(self.draft, path, eng.model_config, eng.device)
        self._ctx: Dict[int, List[Tuple[torch.Tensor, torch.Tensor]]] = {}
        self._len: Dict[int, int] = {}
        self._tok: Dict[int, int] = {}

    @property
    def capture_layers(self) -> List[int]:
        return self.aux_layers

    def on_features(self, req: Req, aux_rows: Sequence[torch.Tensor], first_pos: int, tokens_next: torch.Tensor
                    ) -> None:
        n = aux_rows[0].shape[0]
        if n == 0:
            return
        dev = self.engine.device
        pos = torch.arange(first_pos, first_pos + n, device=dev, dtype=torch.int32)
        new = self.draft.project_context(aux_rows, pos)
        old = self._ctx.get(req.uid)
        if old is None or self._len.get(req.uid) != first_pos:
            old = None                                      # not a continuation: start over from these rows
        self._ctx[req.uid] = [(torch.cat([o[0], k])[-WINDOW:], torch.cat([o[1], v])[-WINDOW:]) if old is not None
                              else (k[-WINDOW:], v[-WINDOW:]) for o, (k, v) in zip(old or new, new)]
        self._len[req.uid] = first_pos + n
        self._tok[req.uid] = int(tokens_next[n - 1])

    def propose(self, reqs: Sequence[Req]) -> List[List[int]]:
        out: List[List[int]] = [[] for _ in reqs]
        eng, dev = self.engine, self.engine.device
        for i, r in enumerate(reqs):
            k = min(self.budget(r), self.block - 1)
            if k <= 0 or r.uid not in self._ctx:
                continue
            start = self._len[r.uid]
            ids = torch.full((self.block,), self.mask_token_id, dtype=torch.int32, device=dev)
            ids[0] = self._tok[r.uid]
            pos = torch.arange(start, start + self.block, device=dev, dtype=torch.int32)
            hidden = self.draft.denoise(eng.model.model.embed_tokens.forward(ids), pos, self._ctx[r.uid])
            logits = eng.model.lm_head.forward(hidden[1:k + 1])
            out[i] = logits.float().argmax(-1).tolist()
        return out

    def on_finish(self, req: Req) -> None:
        for d in (self._ctx, self._len, self._tok):
            d.pop(req.uid, None)
