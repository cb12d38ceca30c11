"""EAGLE3-style draft head and its proposer (python/minisgl/spec/draft_model.py:23-357,
python/minisgl/models/glm_eagle3.py:45-201).

The draft is one decoder layer whose attention input is ``[norm(embed(token)) ‖ norm(feature)]``
(2·hidden wide). ``feature`` is ``fc([h_a ‖ h_b ‖ h_c])`` of three target-layer hidden states for
positions the target has already run, and the draft's own previous output for positions it is
extrapolating. Row *i* pairs the feature of position *i* with the token at position *i+1* and
predicts the token at *i+2*. Draft tokens are indices into a reduced vocabulary mapped back
with ``target = draft + d2t[draft]``. Draft K/V live in a per-request ring of ``WINDOW``
positions (python/minisgl/spec/draft_model.py:189).

Checkpoint tensors (13 weights + 2 maps): ``fc, midlayer.{input_layernorm, hidden_norm,
self_attn.{q,k,v,o}_proj, post_attention_layernorm, mlp.{gate,up,down}_proj}, norm, lm_head,
d2t, t2d``. The MTP variant shares the code with one feature layer (the last) and no ``fc``.

The draft is small and replicated on every tensor-parallel rank. Its projections run on the
same GEMM kernels as the target; its ring attention is plain PyTorch (a few rows per step).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import ops
from ..core import Req
from ..layers import BaseOP, RMSNorm, ReplicatedLinear
from ..layers.rotary import get_rope_cache
from ..models.config import ModelConfig
from ..ops import ref
from .base import Proposer

WINDOW = 512


def default_aux_layers(num_layers: int) -> Tuple[int, int, int]:
    """1-based layers {2, L/2, L-3} minus one (python/minisgl/spec/draft_model.py:118-123)."""
    return (1, num_layers // 2 - 1, num_layers - 4)


class _DraftAttention(BaseOP):
    def __init__(self, cfg: ModelConfig, dtype, device) -> None:
        h, d = cfg.hidden_size, cfg.head_dim
        self.qkv_proj = ReplicatedLinear(2 * h, (cfg.num_qo_heads + 2 * cfg.num_kv_heads) * d, dtype, device)
        self.o_proj = ReplicatedLinear(cfg.num_qo_heads * d, h, dtype, device)


class _DraftMLP(BaseOP):
    def __init__(self, cfg: ModelConfig, dtype, device) -> None:
        self.gate_up_proj = ReplicatedLinear(cfg.hidden_size, 2 * cfg.intermediate_size, dtype, device)
        self.down_proj = ReplicatedLinear(cfg.intermediate_size, cfg.hidden_size, dtype, device)


class _DraftLayer(BaseOP):
    def __init__(self, cfg: ModelConfig, dtype, device) -> None:
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.hidden_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.self_attn = _DraftAttention(cfg, dtype, device)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.mlp = _DraftMLP(cfg, dtype, device)


class Eagle3Draft(BaseOP):
    def __init__(self, cfg: ModelConfig, dtype, device, draft_vocab: Optional[int] = None, num_features: int = 3
                 ) -> None:
        self._cfg = cfg
        self._dtype, self._device = dtype, torch.device(device)
        self._nf = num_features
        self._draft_vocab = draft_vocab or cfg.vocab_size
        if num_features > 1:
            self.fc = ReplicatedLinear(num_features * cfg.hidden_size, cfg.hidden_size, dtype, device)
        self.midlayer = _DraftLayer(cfg, dtype, device)
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.lm_head = ReplicatedLinear(cfg.hidden_size, self._draft_vocab, dtype, device)
        self.d2t = torch.zeros(self._draft_vocab, dtype=torch.int64, device=device)
        self.t2d = torch.ones(cfg.vocab_size, dtype=torch.bool, device=device)
        self._cos_sin: Optional[torch.Tensor] = None
        hk, d = cfg.num_kv_heads, cfg.head_dim
        self._rings: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        self._ring_shape = (WINDOW, hk, d)

    # ---- state ----
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
        self.d2t.zero_()

    # ---- compute ----
    def fuse_features(self, aux: Sequence[torch.Tensor]) -> torch.Tensor:
        if self._nf == 1:
            return aux[-1]
        return self.fc.forward(torch.cat(list(aux), dim=-1).to(self._dtype))

    def forward_rows(self, uid: int, embeds: torch.Tensor, features: torch.Tensor, positions: torch.Tensor
                     ) -> Tuple[torch.Tensor, torch.Tensor]:
        """Run the draft layer on ``n`` consecutive rows of one request. Returns
        ``(hidden [n, H], logits [n, draft_vocab])``; the ring receives the rows' K/V."""
        cfg = self._cfg
        hq, hk, d = cfg.num_qo_heads, cfg.num_kv_heads, cfg.head_dim
        if self._cos_sin is None:
            self._cos_sin = get_rope_cache(cfg.rotary_config, embeds.device)
        layer = self.midlayer
        x = torch.cat([layer.input_layernorm.forward(embeds), layer.hidden_norm.forward(features)], dim=-1)
        qkv = layer.self_attn.qkv_proj.forward(x)
        q, k, v = qkv.split([hq * d, hk * d, hk * d], dim=-1)
        q, k = ref.qk_norm_rope(q, k, None, None, positions, self._cos_sin, d, cfg.rotary_config.rotary_dim, 0.0)
        n = embeds.shape[0]
        kr, vr = self.ring(uid)
        pos = positions.long()
        kr[pos % WINDOW] = k.float().view(n, hk, d)
        vr[pos % WINDOW] = v.float().view(n, hk, d)
        last = int(pos[-1])
        lo = max(0, last - WINDOW + 1)
        span = torch.arange(lo, last + 1, device=embeds.device)
        kk = kr[span % WINDOW].permute(1, 0, 2)                       # [hk, S, d]
        vv = vr[span % WINDOW].permute(1, 0, 2)
        g = hq // hk
        qq = q.float().view(n, hk, g, d).permute(1, 2, 0, 3)          # [hk, g, n, d]
        s = torch.einsum("hgqd,hkd->hgqk", qq, kk) * d ** -0.5
        mask = span[None, :] > pos[:, None]
        s = s.masked_fill(mask[None, None], float("-inf"))
        o = torch.einsum("hgqk,hkd->hgqd", torch.softmax(s, -1), vv).permute(2, 0, 1, 3).reshape(n, hq * d)
        h = features.float() + layer.self_attn.o_proj.forward(o.to(self._dtype)).float()
        m = layer.mlp.down_proj.forward(ops.silu_and_mul(layer.mlp.gate_up_proj.forward(
            layer.post_attention_layernorm.forward(h.to(self._dtype)))))
        h = (h + m.float()).to(self._dtype)
        logits = self.lm_head.forward(self.norm.forward(h))
        return h, logits

    def to_target(self, draft_ids: torch.Tensor) -> torch.Tensor:
        return draft_ids + self.d2t[draft_ids]


def load_eagle3(draft: Eagle3Draft, path: str) -> None:
    """Load the 13 weights and 2 maps of an EAGLE3 checkpoint directory."""
    from ..models.weight import iter_safetensors

    cfg = draft._cfg
    parts: Dict[str, Dict[str, torch.Tensor]] = {}
    dev = draft._device
    for name, t in iter_safetensors(path):
        if name == "d2t":
            draft.d2t = t.to(dev, torch.int64)
        elif name == "t2d":
            draft.t2d = t.to(dev, torch.bool)
        elif name == "fc.weight":
            draft.fc.weight = t.to(dev, draft._dtype)
        elif name == "norm.weight":
            draft.norm.weight = t.to(dev, draft._dtype)
        elif name == "lm_head.weight":
            draft.lm_head.weight = t.to(dev, draft._dtype)
        elif name.startswith("midlayer."):
            sub = name[len("midlayer."):]
            if ".q_proj." in sub or ".k_proj." in sub or ".v_proj." in sub:
                parts.setdefault("qkv", {})[sub.split(".")[1]] = t
            elif ".gate_proj." in sub or ".up_proj." in sub:
                parts.setdefault("gate_up", {})[sub.split(".")[1]] = t
            else:
                owner = draft.midlayer
                keys = sub.split(".")
                for kk in keys[:-1]:
                    owner = getattr(owner, kk)
                setattr(owner, keys[-1], t.to(dev, draft._dtype))
    qkv = parts.get("qkv", {})
    if qkv:
        draft.midlayer.self_attn.qkv_proj.weight = torch.cat(
            [qkv["q_proj"], qkv["k_proj"], qkv["v_proj"]]).to(dev, draft._dtype)
    gu = parts.get("gate_up", {})
    if gu:
        draft.midlayer.mlp.gate_up_proj.weight = torch.cat([gu["gate_proj"], gu["up_proj"]]).to(dev, draft._dtype)
    assert cfg.hidden_size == draft.norm.weight.shape[0]


class Eagle3Proposer(Proposer):
    """Chain drafting with the EAGLE3 head. The scheduler hands over the target's auxiliary
    hidden states after every prefill and verify forward (``on_features``)."""

    name = "eagle3"
    max_batch = 64

    def __init__(self, config, scheduler, mtp: bool = False) -> None:
        super().__init__(config.spec_num_draft)
        # candidates per depth of the verify tree (1 = a chain); used by the device step only
        self.tree_width = max(1, int(getattr(config, "spec_tree_width", 1) or 1))
        eng = scheduler.engine
        self.engine = eng
        cfg = eng.model_config
        self.aux_layers = list(cfg.eagle_aux_layers or default_aux_layers(cfg.num_layers)) if not mtp \
            else [cfg.num_layers - 1]
        self.aux_layers = [min(max(a, 0), cfg.num_layers - 1) for a in self.aux_layers]
        self.draft = Eagle3Draft(cfg, eng.dtype, eng.device, cfg.draft_vocab_size, num_features=len(self.aux_layers))
        if config.spec_draft_model_path:
            load_eagle3(self.draft, config.spec_draft_model_path)
        else:
            self.draft.init_dummy(config.seed + 17)
        # per request: feature of the last committed position and the draft state to continue from
        self.last_feature: Dict[int, torch.Tensor] = {}
        self.last_pos: Dict[int, int] = {}

    # ---- hooks ----
    @property
    def capture_layers(self) -> List[int]:
        return self.aux_layers

    def _embed(self, ids: torch.Tensor) -> torch.Tensor:
        return self.engine.model.model.embed_tokens.forward(ids.to(torch.int32))

    def on_features(self, req: Req, aux_rows: Sequence[torch.Tensor], first_pos: int, tokens_next: torch.Tensor
                    ) -> None:
        """``aux_rows[j]`` ``[n, H]``: target hidden states of positions ``first_pos .. first_pos+n-1``;
        ``tokens_next[i]`` is the token at position ``first_pos + i + 1``. Extends the draft KV
        with those rows and remembers the output hidden of the last one."""
        n = aux_rows[0].shape[0]
        if n == 0:
            return
        feat = self.draft.fuse_features(aux_rows)
        emb = self._embed(tokens_next.to(self.engine.device))
        pos = torch.arange(first_pos, first_pos + n, device=self.engine.device, dtype=torch.int32)
        hidden, logits = self.draft.forward_rows(req.uid, emb, feat, pos)
        self.last_feature[req.uid] = hidden[-1:].clone()
        self.last_pos[req.uid] = first_pos + n - 1
        self._first_logits = getattr(self, "_first_logits", {})
        self._first_logits[req.uid] = logits[-1:].clone()

    def propose(self, reqs: Sequence[Req]) -> List[List[int]]:
        out: List[List[int]] = []
        dev = self.engine.device
        for r in reqs:
            k = self.budget(r)
            logits = getattr(self, "_first_logits", {}).get(r.uid)
            if k == 0 or logits is None:
                out.append([])
                continue
            toks: List[int] = []
            hidden = self.last_feature[r.uid]
            pos = self.last_pos[r.uid]
            for j in range(k):
                d_id = logits.float().argmax(-1)
                t_id = self.draft.to_target(d_id)
                toks.append(int(t_id))
                if j == k - 1:
                    break
                pos += 1
                hidden, logits = self.draft.forward_rows(
                    r.uid, self._embed(t_id), hidden, torch.tensor([pos], device=dev, dtype=torch.int32))
            out.append(toks)
        return out

    def on_finish(self, req: Req) -> None:
        self.draft.drop(req.uid)
        self.last_feature.pop(req.uid, None)
        self.last_pos.pop(req.uid, None)
        getattr(self, "_first_logits", {}).pop(req.uid, None)
