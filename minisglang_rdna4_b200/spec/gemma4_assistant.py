"""Gemma-4 assistant drafter: a small decoder that keeps no K/V of its own
(python/minisgl/models/gemma4_assistant.py:1-164, python/minisgl/spec/gemma4_assistant.py:1-260).

Every layer projects queries only and attends over the TARGET's paged K/V: sliding layers over the
target's last sliding layer that keeps K/V, full layers over its last such full layer, with that layer's
rotary table, head width and softmax scale. One draft step:

    x    = pre_projection([target_embedding(token) ‖ seed])
    x    = layers(x)                      (query-only attention, sandwich norms, GeGLU MLP, layer scalar)
    d    = norm(x);  next token = argmax(lm_head(d));  next seed = post_projection(d)

Step 0 takes the confirmed token and the target's final hidden state of the position before it; step j
takes draft j-1 and the previous step's seed. All steps query from the last position the target has
processed, over the same keys, so a chain needs no draft-side cache, roll-back or clean-up.

Host-driven, through tensor ops and the engine's linear layers; the target it serves (Gemma-4) runs on the
CPU oracle path only, and so does this.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..core import Req
from ..layers import (
    AttentionLayer, BaseOP, ColumnParallelLinear, GatedActivation, MergedColumnParallelLinear, ParallelLMHead,
    RMSNorm, ReplicatedLinear, RowParallelLinear, VocabParallelEmbedding,
)
from ..layers.rotary import get_rope_cache
from ..models.config import ModelConfig
from ..parallel.info import get_tp_info
from ..utils import cdiv, div_even
from .base import Proposer


def is_gemma4_assistant(path: Optional[str]) -> bool:
    if not path or not os.path.isfile(os.path.join(path, "config.json")):
        return False
    with open(os.path.join(path, "config.json")) as fh:
        return json.load(fh).get("model_type") == "gemma4_assistant"


class _Attn(BaseOP):
    def __init__(self, cfg: ModelConfig, head_dim: int, dtype, device) -> None:
        self.q_proj = ColumnParallelLinear(cfg.hidden_size, cfg.num_qo_heads * head_dim, dtype, device)
        self.q_norm = RMSNorm(head_dim, cfg.rms_norm_eps, dtype, device)
        self.o_proj = RowParallelLinear(cfg.num_qo_heads * head_dim, cfg.hidden_size, dtype, device)


class _MLP(BaseOP):
    def __init__(self, cfg: ModelConfig, dtype, device) -> None:
        self.gate_up_proj = MergedColumnParallelLinear(cfg.hidden_size, [cfg.intermediate_size] * 2, dtype, device)
        self.down_proj = RowParallelLinear(cfg.intermediate_size, cfg.hidden_size, dtype, device)


class _Layer(BaseOP):
    def __init__(self, cfg: ModelConfig, head_dim: int, dtype, device) -> None:
        norm = lambda: RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.input_layernorm = norm()
        self.self_attn = _Attn(cfg, head_dim, dtype, device)
        self.post_attention_layernorm = norm()
        self.pre_feedforward_layernorm = norm()
        self.mlp = _MLP(cfg, dtype, device)
        self.post_feedforward_layernorm = norm()
        self.layer_scalar = torch.ones((1,), dtype=dtype, device=device)
        self._d = head_dim
        self._heads = div_even(cfg.num_qo_heads, get_tp_info().size)
        self._eps = cfg.rms_norm_eps
        self._act = GatedActivation(cfg.hidden_act)

    def forward(self, x: torch.Tensor, tgt: "_Target", pos, block_table, cu_q, seq_lens) -> torch.Tensor:
        q = self.self_attn.q_proj.forward(self.input_layernorm.forward(x))
        q = ops.q_norm_rope(q, self.self_attn.q_norm.weight, pos, tgt.cos_sin, self._heads, self._d, tgt.rotary_dim,
                            self._eps, False)
        o = ops.paged_attention(q, tgt.pool.k_cache(tgt.kv_index), tgt.pool.v_cache(tgt.kv_index), block_table, cu_q,
                                seq_lens, tgt.scale, causal=True, window=tgt.window, max_q=1,
                                max_kv=int(block_table.shape[1]) * tgt.pool.page_size, decode=True)
        a = self.self_attn.o_proj.forward(o.reshape(x.shape[0], self._heads * self._d), reduce=True)
        x = x + self.post_attention_layernorm.forward(a)
        h = self._act(self.mlp.gate_up_proj.forward(self.pre_feedforward_layernorm.forward(x)))
        x = x + self.post_feedforward_layernorm.forward(self.mlp.down_proj.forward(h, reduce=True))
        return x * self.layer_scalar

    def init_dummy(self, gen: torch.Generator, std: float = 0.02) -> None:
        self.layer_scalar = torch.ones_like(self.layer_scalar)


class _Target:
    """Where one kind of drafter layer reads K/V: the target layer's pool row, rotary table, window, scale."""

    def __init__(self, layer: AttentionLayer, pool, device) -> None:
        self.pool, self.kv_index = pool, layer._kv_index
        self.cos_sin = get_rope_cache(layer._rotary, device)
        self.rotary_dim = layer._rotary.rotary_dim
        self.window, self.scale, self.head_dim = layer._window, layer._scale, layer._d


class _Body(BaseOP):
    def __init__(self, cfg: ModelConfig, head_dims: List[int], dtype, device) -> None:
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, dtype, device)
        self.layers = [_Layer(cfg, d, dtype, device) for d in head_dims]
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)


class Gemma4AssistantDraft(BaseOP):
    def __init__(self, cfg: ModelConfig, backbone: int, dtype, device) -> None:
        self._cfg = cfg
        self.layer_types = list(cfg.layer_types)
        dims = [int(cfg.head_dim) if t == "sliding_attention" else int(cfg.global_head_dim or cfg.head_dim)
                for t in self.layer_types]
        self.model = _Body(cfg, dims, dtype, device)
        self.pre_projection = ReplicatedLinear(2 * backbone, cfg.hidden_size, dtype, device)
        self.post_projection = ReplicatedLinear(cfg.hidden_size, backbone, dtype, device)
        self.lm_head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, dtype, device, tied=self.model.embed_tokens)
        self.backbone = backbone

    def step(self, embed, seed, pos, targets: Dict[str, _Target], block_table, cu_q, seq_lens):
        """``embed`` ``[n, backbone]``: the target's scaled embedding of the input tokens. Returns the
        fp32 logits of this rank's vocabulary shard gathered to the full vocabulary and the next seed."""
        x = self.pre_projection.forward(torch.cat([embed, seed.to(embed.dtype)], dim=-1))
        for kind, layer in zip(self.layer_types, self.model.layers):
            x = layer.forward(x, targets[kind], pos, block_table, cu_q, seq_lens)
        d = self.model.norm.forward(x)
        return self.lm_head.forward(d), self.post_projection.forward(d)

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


class Gemma4AssistantProposer(Proposer):
    name = "gemma4_assistant"
    device_step_ok = False

    def __init__(self, config, scheduler) -> None:
        super().__init__(config.spec_num_draft)
        self.tree_width = 1
        eng = scheduler.engine
        self.engine, self.sched = eng, scheduler
        path = config.spec_draft_model_path
        with open(os.path.join(path, "config.json")) as fh:
            raw = json.load(fh)
        text = dict(raw.get("text_config") or raw)
        text.setdefault("model_type", "gemma4_text")
        if text["model_type"] == "gemma4_assistant":
            text["model_type"] = "gemma4_text"
        if raw.get("use_ordered_embeddings"):
            raise NotImplementedError("assistant checkpoints with ordered embeddings (centroid logits)")
        cfg = ModelConfig.from_hf(text)
        backbone = int(raw.get("backbone_hidden_size") or eng.model_config.hidden_size)
        if backbone != eng.model_config.hidden_size:
            raise ValueError(f"the drafter was trained for a {backbone}-wide target, this one is "
                             f"{eng.model_config.hidden_size} wide")
        if eng.swa is not None:
            raise NotImplementedError("the assistant drafter reads the single K/V pool; turn MSGL_SWA_POOL off")
        self.draft = Gemma4AssistantDraft(cfg, backbone, eng.dtype, eng.device)
        if getattr(config, "use_dummy_weight", False) or not any(f.endswith(".safetensors") for f in os.listdir(path)):
            self.draft.init_dummy(config.seed + 17)
        else:
            from ..models.weight import load_weights

            load_weights(self.draft, path, cfg, eng.device)
        # the target layers the two kinds read: the last of each kind that keeps K/V of its own
        tmc = eng.model_config
        mods = {m._layer_id: m for m in eng.model.modules() if isinstance(m, AttentionLayer)}
        self.targets: Dict[str, _Target] = {}
        for kind in set(self.draft.layer_types):
            own = [i for i in range(tmc.num_layers) if tmc.layer_types[i] == kind and tmc.kv_donor(i) is None]
            if not own:
                raise ValueError(f"the target has no {kind} layer to read K/V from")
            layer = mods[own[-1]]
            want = cfg.head_dim if kind == "sliding_attention" else (cfg.global_head_dim or cfg.head_dim)
            if layer._d != want:
                raise ValueError(f"{kind}: drafter heads are {want} wide, the target's {layer._d}")
            self.targets[kind] = _Target(layer, eng.kv_cache, eng.device)
        self.aux_layers = [tmc.num_layers]            # the target's final normed hidden state
        self._seed: Dict[int, torch.Tensor] = {}
        self._len: Dict[int, int] = {}
        self._tok: Dict[int, int] = {}
        self._scale = float(torch.tensor(float(tmc.hidden_size) ** 0.5, dtype=eng.dtype))

    @property
    def capture_layers(self) -> List[int]:
        return self.aux_layers

    def on_features(self, req: Req, aux_rows: Sequence[torch.Tensor], first_pos: int, tokens_next: torch.Tensor
                    ) -> None:
        n = aux_rows[0].shape[0]
        if n == 0:
            return
        self._seed[req.uid] = aux_rows[0][-1:].clone()
        self._len[req.uid] = first_pos + n              # positions of this request that have K/V
        self._tok[req.uid] = int(tokens_next[n - 1])

    def propose(self, reqs: Sequence[Req]) -> List[List[int]]:
        out: List[List[int]] = [[] for _ in reqs]
        rows = [i for i, r in enumerate(reqs) if self.budget(r) > 0 and r.uid in self._seed]
        if not rows:
            return out
        eng, dev = self.engine, self.engine.device
        ps = eng.page_size
        lens = [self._len[reqs[i].uid] for i in rows]
        width = cdiv(max(lens), ps)
        table = np.stack([self.sched.cache.page_table[reqs[i].table_idx, :width] for i in rows]).astype(np.int32)
        block_table = torch.from_numpy(table).to(dev)
        seq_lens = torch.tensor(lens, dtype=torch.int32, device=dev)
        cu_q = torch.arange(len(rows) + 1, dtype=torch.int32, device=dev)
        pos = (seq_lens - 1).to(torch.int32)
        tok = torch.tensor([self._tok[reqs[i].uid] for i in rows], dtype=torch.int32, device=dev)
        seed = torch.cat([self._seed[reqs[i].uid] for i in rows])
        budget = [self.budget(reqs[i]) for i in rows]
        embed = eng.model.model.embed_tokens
        for j in range(max(budget)):
            logits, seed = self.draft.step(embed.forward(tok) * self._scale, seed, pos, self.targets, block_table,
                                           cu_q, seq_lens)
            tok = logits.float().argmax(-1).to(torch.int32)
            for i, t, k in zip(rows, tok.tolist(), budget):
                if j < k:
                    out[i].append(int(t))
        return out

    def on_finish(self, req: Req) -> None:
        for d in (self._seed, self._len, self._tok):
            d.pop(req.uid, None)
