"""The speculative decode step on the GPU kernel path.

One step = propose → verify → accept → commit → draft update, all on the device, captured as one
CUDA graph per batch bucket, with a single host→device copy of the step's tables before it and a
single device→host copy of the acceptance record after it. The reference builds the same pieces
from several graphs and torch ops (python/minisgl/engine/graph.py:692-1100 verify graphs,
python/minisgl/spec/capture.py:82 propose graph, python/minisgl/spec/draft_attn.py:36 draft KV
through the decode kernel, python/minisgl/spec/accept_gpu.py:110-330 acceptance on the device).

Shapes are fixed: every request feeds ``W = 1 + K`` rows (its last committed token and K draft
tokens that sit behind it in the token pool); a request with fewer drafts has trailing rows that
write their K/V to the scratch page and are ignored by the acceptance kernel. Because the
target's rows of a verify step and of every other verify step run the same kernels with the same
reduction order, greedy output is bit-identical to what the same engine produces with a proposer
that never drafts.

EAGLE3 / MTP draft head, batched (``BatchedDraft``): one decoder layer over all requests per draft
position. Its K/V live in a one-layer paged pool that shares the target's page table, so draft
position p of a request uses the same page and offset as the target's position p and prefix-cache
hits carry their draft K/V with them. The hidden state the chain starts from is kept per request
slot on the device.

Order inside the step for a request whose committed tokens end at position c:

1. propose: ``d_1 = argmax head(hidden[slot])``; for i = 1 .. K-1 the draft layer runs the row
   (previous output, ``d_i``) at draft position ``c + i - 1`` and yields ``d_{i+1}``; ``d_i`` is written
   to pool position ``c + i``.
2. verify: the target runs rows ``c .. c + K``; auxiliary hidden states of the feature layers are kept.
3. accept: ``n`` tokens stand (``spec_accept_kernel``), are written to positions ``c + 1 .. c + n``
   and reported in the record; ``sel_row = b * W + n - 1``.
4. draft update: the draft layer runs all W rows (feature of position ``c + j``, token at ``c + j + 1``),
   which rewrites the draft K/V of positions ``c .. c + K`` (the ones past ``c + n - 1`` are rewritten by
   later steps before anything reads them); the output of row ``sel_row`` becomes ``hidden[slot]``.

Tree verification (``tree_width`` T > 1, draft head only; python/minisgl/engine/graph.py:950,
python/minisgl/spec/ddtree.py): the tree has a fixed shape, so it is captured like the chain. At
every depth the head's best token continues the chain and its next T - 1 candidates become
siblings without children. A request then feeds ``R = 1 + K * T`` verify rows: the root, the chain
(rows 1 .. K, K/V at their sequence positions, exactly as in the chain step), then the siblings,
whose K/V go to scratch slots ``c + K + 1 ..`` of the same request. Rows see the committed prefix,
the root and their ancestors through a constant ``[R, R]`` additive mask over the last R K/V
positions. ``spec_accept_tree_kernel`` follows the target's prediction down the tree; when a sibling
is accepted its K/V is moved to its sequence position in every layer (``spec_kv_compact_kernel``)
and its features replace the chain row's in the draft update. The draft chain costs the same K
layer runs as without a tree; the price of the tree is the wider verify forward.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..core import Batch
from ..kvcache.mha_pool import MHAKVCache
from ..layers.rotary import get_rope_cache
from ..utils import cdiv, init_logger

logger = init_logger(__name__)

BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64)


def _bind():
    from ..ops._lib import bind, c_i, c_ll, c_p

    bind("msgl_spec_accept", c_i, [c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_p])
    bind("msgl_spec_write_draft", c_i, [c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_p])
    bind("msgl_spec_kv_compact", c_i, [c_p, c_p, c_i, c_ll, c_i, c_i, c_i, c_i, c_p])
    bind("msgl_spec_accept_tree", c_i, [c_p] * 12 + [c_p, c_i, c_i, c_i, c_i, c_i, c_p])


class BatchedDraft:
    """The EAGLE3 / MTP head of ``spec.eagle3.Eagle3Draft`` run over all requests at once on the
    engine's kernels, with a paged K/V pool of its own."""

    def __init__(self, draft, engine) -> None:
        self.m = draft
        cfg = draft._cfg
        self.cfg = cfg
        self.hq, self.hk, self.d = cfg.num_qo_heads, cfg.num_kv_heads, cfg.head_dim
        self.scale = self.d ** -0.5
        self.pool = MHAKVCache(1, engine.num_pages, engine.page_size, self.hk, self.d, engine.dtype, engine.device)
        self.cos_sin = get_rope_cache(cfg.rotary_config, engine.device)
        self.embed = engine.model.model.embed_tokens
        self.hidden = torch.zeros((engine.num_slots, cfg.hidden_size), dtype=engine.dtype, device=engine.device)
        self.eps = cfg.rms_norm_eps

    def layer(self, emb, feat, positions, out_loc, block_table, cu_q, seq_lens, max_q: int, max_kv: int):
        """Rows ``(embedding of the next token, feature)`` → the layer's output hidden states. K/V of
        the rows go to ``out_loc`` of the draft pool."""
        L = self.m.midlayer
        x = torch.cat([L.input_layernorm.forward(emb), L.hidden_norm.forward(feat)], dim=-1)
        qkv = L.self_attn.qkv_proj.forward(x)
        q = ops.qk_norm_rope_store(qkv, None, None, positions, self.cos_sin, self.hq, self.hk, self.d,
                                   self.cfg.rotary_config.rotary_dim, self.eps, self.pool.k_cache(0),
                                   self.pool.v_cache(0), out_loc, None, None, self.cfg.rotary_config.interleaved)
        o = ops.paged_attention(q, self.pool.k_cache(0), self.pool.v_cache(0), block_table, cu_q, seq_lens,
                                self.scale, causal=True, max_q=max_q, max_kv=max_kv, decode=(max_q == 1), splits=1)
        h = feat + L.self_attn.o_proj.forward(o.reshape(o.shape[0], self.hq * self.d))
        mlp = L.mlp.down_proj.forward(ops.silu_and_mul(L.mlp.gate_up_proj.forward(
            L.post_attention_layernorm.forward(h))))
        return h + mlp

    def head_topk(self, h, width: int) -> torch.Tensor:
        """The ``width`` highest-scoring draft-vocabulary ids per row, best first, int32 ``[rows, width]``."""
        logits = ops.gemm(self.m.norm.forward(h), self.m.lm_head.weight, None, torch.float32)
        return torch.topk(logits, width, dim=-1).indices.to(torch.int32)

    def head_ids(self, h) -> torch.Tensor:
        """Arg-max of the draft head (reduced vocabulary), int32."""
        logits = ops.gemm(self.m.norm.forward(h), self.m.lm_head.weight, None, torch.float32)
        return ops.argmax(logits)

    def features(self, aux: Sequence[torch.Tensor]) -> torch.Tensor:
        return self.m.fuse_features(aux)


class DeviceSpecRunner:
    def __init__(self, engine, num_draft: int, draft=None, capture_layers: Optional[List[int]] = None,
                 max_batch: int = 64, tree_width: int = 1) -> None:
        _bind()
        self.engine = engine
        self.K = int(num_draft)
        self.W = self.K + 1
        # tree verification needs candidates per depth, which only the draft head provides
        self.T = int(tree_width) if (draft is not None and tree_width > 1) else 1
        self.R = 1 + self.K * self.T                      # verify rows per request (== W for a chain)
        self.draft = BatchedDraft(draft, engine) if draft is not None else None
        self.capture_layers = list(capture_layers) if capture_layers else None
        eng = engine
        self.max_bs = int(min(max_batch, eng.config.max_running_req))
        self.buckets = [b for b in BUCKETS if b <= self.max_bs]
        if self.max_bs not in self.buckets:
            self.buckets.append(self.max_bs)
        self.P = eng.max_pages_per_seq
        B, W, K, P, R = self.max_bs, self.W, self.K, self.P, self.R
        # one int32 arena: a single H2D copy fills every table of the step
        fields = [("token_idx", B * R), ("positions", B * R), ("out_loc", B * R), ("seq_lens", B),
                  ("u_tok_idx", B * W), ("u_positions", B * W), ("u_out_loc", B * W), ("u_seq_lens", B),
                  ("block_table", B * P), ("first_idx", B), ("num_draft", B), ("max_emit", B), ("flags", B),
                  ("slots", B), ("stage_idx", B * K), ("stage_tok", B * K),
                  ("c_tok_idx", max(K - 1, 1) * B), ("c_dst_idx", K * B), ("c_positions", max(K - 1, 1) * B),
                  ("c_out_loc", max(K - 1, 1) * B), ("c_seq_lens", max(K - 1, 1) * B)]
        self.offsets: Dict[str, tuple] = {}
        off = 0
        for name, n in fields:
            self.offsets[name] = (off, n)
            off += n
        self.arena_len = off
        dev = eng.device
        self.arena = torch.zeros(off, dtype=torch.int32, device=dev)
        self._pinned = [torch.zeros(off, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._pin_events = [None, None]
        self._pin_pos = 0
        self.cu_q_verify = (torch.arange(B + 1, dtype=torch.int32, device=dev) * R).contiguous()
        self.cu_q_update = (torch.arange(B + 1, dtype=torch.int32, device=dev) * W).contiguous()
        self.tree_mask = None
        if self.T > 1:
            T = self.T
            vis = torch.full((R, R), float("-inf"))
            vis[:, 0] = 0.0                                             # the root (last committed token)
            for d in range(1, K + 1):
                vis[d, 1:d + 1] = 0.0                                   # chain node: chain nodes 1 .. d
                for sb in range(T - 1):
                    row = K + (d - 1) * (T - 1) + sb + 1
                    vis[row, 1:d] = 0.0                                 # sibling: the chain above it and itself
                    vis[row, row] = 0.0
            self.tree_mask = vis.repeat(B, 1).contiguous().to(dev)      # one [R, R] block per request
            self.sib_tok = torch.zeros((K, B, T - 1), dtype=torch.int32, device=dev)
            self.no_dst = torch.full((B * (T - 1),), -1, dtype=torch.int32, device=dev)
            self.feat_row = torch.zeros(B * W, dtype=torch.int32, device=dev)
            self.moves = torch.full((B * 2,), -1, dtype=torch.int32, device=dev)
        self.cu_q_decode = torch.arange(B + 1, dtype=torch.int32, device=dev)
        self.record = torch.zeros(B * (W + 2), dtype=torch.int32, device=dev)
        self.sel_row = torch.zeros(B, dtype=torch.int32, device=dev)
        self._rec_host = [torch.zeros(B * (W + 2), dtype=torch.int32).pin_memory() for _ in range(2)]
        eos = sorted(eng.model_config.eos_token_ids)[:8]
        self._eos = (ctypes.c_int * 8)(*(eos + [-1] * (8 - len(eos))))
        self._n_eos = len(eos)
        self.graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        self.pool = None
        self.replays = 0
        self.eager_steps = 0

    # ------------------------------------------------------------------ views
    def view(self, name: str, bs: Optional[int] = None) -> torch.Tensor:
        off, n = self.offsets[name]
        return self.arena[off:off + n]

    def _v(self, name: str, rows: int, cols: int = 1) -> torch.Tensor:
        off, _ = self.offsets[name]
        return self.arena[off:off + rows * cols]

    # ------------------------------------------------------------------ the step body (eager or captured)
    def body(self, bs: int) -> None:
        from ..ops import cuda as Kc
        from ..ops._lib import check, lib

        eng, W, K, P, R, T = self.engine, self.W, self.K, self.P, self.R, self.T
        tree = T > 1
        L = lib()
        st = Kc._stream()
        pool_flat = eng.token_pool.view(-1)
        slots = self._v("slots", bs).long()
        bt = self._v("block_table", bs, P).view(bs, P)
        msl = eng.max_seq_len
        d = self.draft
        if d is None:
            # drafts proposed on the host: put them behind the requests' last tokens
            pool_flat[self._v("stage_idx", bs * K).long()] = self._v("stage_tok", bs * K)
        else:
            # ---- propose: chain of K draft tokens from the per-slot hidden state
            h = d.hidden[slots]
            c_dst = self.view("c_dst_idx").view(K, -1)

            def emit(h_rows, depth):
                """Write the head's best token behind the chain (and its runners-up to the sibling table)."""
                if tree:
                    top = d.head_topk(h_rows, T)
                    best, sib = top[:, 0].contiguous(), top[:, 1:].contiguous()
                    check(L.msgl_spec_write_draft(sib.data_ptr(), d.m.d2t.data_ptr(), self.no_dst.data_ptr(),
                                                  pool_flat.data_ptr(), self.sib_tok[depth].data_ptr(), bs * (T - 1),
                                                  d.m._draft_vocab, st), "spec_write_draft")
                else:
                    best = d.head_ids(h_rows)
                check(L.msgl_spec_write_draft(best.data_ptr(), d.m.d2t.data_ptr(), c_dst[depth, :bs].data_ptr(),
                                              pool_flat.data_ptr(), None, bs, d.m._draft_vocab, st), "spec_write_draft")

            emit(h, 0)
            if K > 1:
                c_tok = self.view("c_tok_idx").view(K - 1, -1)
                c_pos = self.view("c_positions").view(K - 1, -1)
                c_loc = self.view("c_out_loc").view(K - 1, -1)
                c_len = self.view("c_seq_lens").view(K - 1, -1)
                for i in range(1, K):
                    emb = d.embed.forward(pool_flat[c_tok[i - 1, :bs].long()])
                    h = d.layer(emb, h, c_pos[i - 1, :bs], c_loc[i - 1, :bs], bt, self.cu_q_decode[:bs + 1],
                                c_len[i - 1, :bs], 1, msl)
                    emit(h, i)
        # ---- verify: R rows per request through the target
        tok_idx = self._v("token_idx", bs * R)
        batch = Batch(reqs=[], phase="decode")
        batch.spec_verify = True
        batch.capture_layers = self.capture_layers
        batch.positions = self._v("positions", bs * R)
        batch.out_loc = self._v("out_loc", bs * R)
        batch.input_ids = pool_flat[tok_idx.long()]
        if tree:
            # sibling rows take their tokens from the sibling table ([K, B, T - 1] -> per request, depth-major)
            batch.input_ids.view(bs, R)[:, W:] = self.sib_tok[:, :bs].permute(1, 0, 2).reshape(bs, K * (T - 1))
        seq_lens = self._v("seq_lens", bs)
        cu_q = self.cu_q_verify[:bs + 1]
        eng.ctx.attn_backend.prepare_metadata(batch, bt, cu_q, seq_lens, R, msl, causal=True,
                                              mask=self.tree_mask[:bs * R] if tree else None,
                                              mask_window=R if tree else 0)
        prev = Kc.gemm_pair_mode(1)   # verify rows never leave the single-CTA GEMM (one code path for all steps)
        try:
            with eng.ctx.forward_batch(batch):
                hidden = eng.model.forward(batch.input_ids)
                target = eng.model.lm_head.forward_argmax(hidden)
        finally:
            Kc.gemm_pair_mode(prev)
        aux = eng.ctx.aux_hidden
        eng.ctx.aux_hidden = None
        # ---- accept + commit
        if tree:
            check(L.msgl_spec_accept_tree(
                target.data_ptr(), pool_flat.data_ptr(), self._v("first_idx", bs).data_ptr(),
                self._v("num_draft", bs).data_ptr(), self._v("max_emit", bs).data_ptr(), self._v("flags", bs).data_ptr(),
                self.sib_tok.data_ptr(), batch.out_loc.data_ptr(), self.record.data_ptr(), self.sel_row.data_ptr(),
                self.feat_row.data_ptr(), self.moves.data_ptr(), self._eos, self._n_eos, bs, K, T, self.max_bs, st),
                "spec_accept_tree")
            Kc._count("spec_accept", "spec_accept_tree_kernel")
            # an accepted sibling's K/V goes from its scratch slot to its sequence position, in every layer
            buf = eng.kv_cache._buf
            _, layers, pages_p1, hk, ps, hd = buf.shape
            check(L.msgl_spec_kv_compact(buf.data_ptr(), self.moves.data_ptr(), bs,
                                         pages_p1 * hk * ps * hd * buf.element_size(), 2 * layers, hk, ps,
                                         hd * buf.element_size(), st), "spec_kv_compact")
            Kc._count("spec_kv_compact", "spec_kv_compact_kernel")
        else:
            check(L.msgl_spec_accept(target.data_ptr(), pool_flat.data_ptr(), self._v("first_idx", bs).data_ptr(),
                                     self._v("num_draft", bs).data_ptr(), self._v("max_emit", bs).data_ptr(),
                                     self._v("flags", bs).data_ptr(), self.record.data_ptr(), self.sel_row.data_ptr(),
                                     self._eos, self._n_eos, bs, W, st), "spec_accept")
            Kc._count("spec_accept", "spec_accept_kernel")
        if d is not None:
            # ---- draft update over the accepted path's rows (feature of position p, token at p + 1)
            feat = d.features(aux)
            if tree:
                feat = feat[self.feat_row[:bs * W].long()]
                u_tok = self._v("u_tok_idx", bs * W)
                emb = d.embed.forward(pool_flat[(u_tok + 1).long()])
                hx = d.layer(emb, feat, self._v("u_positions", bs * W), self._v("u_out_loc", bs * W), bt,
                             self.cu_q_update[:bs + 1], self._v("u_seq_lens", bs), W, msl)
            else:
                emb = d.embed.forward(pool_flat[(tok_idx + 1).long()])
                hx = d.layer(emb, feat, batch.positions, batch.out_loc, bt, cu_q, seq_lens, W, msl)
            d.hidden[slots] = hx[self.sel_row[:bs].long()]

    # ------------------------------------------------------------------ prefill feed
    def feed_prefill(self, batch: Batch, token_idx: torch.Tensor, slots_np: np.ndarray, cu_q_np: np.ndarray) -> None:
        """After a target prefill step with captured feature layers: run the draft layer over the
        same rows (same positions, K/V slots and attention tables) and keep the output of every
        request's last row as its chain state."""
        d = self.draft
        eng = self.engine
        aux = eng.ctx.aux_hidden
        eng.ctx.aux_hidden = None
        if d is None or not aux:
            return
        md = batch.attn_metadata
        pool_flat = eng.token_pool.view(-1)
        t = int(cu_q_np[-1])
        feat = d.features([a[:t] for a in aux])
        limit = pool_flat.numel() - 1
        emb = d.embed.forward(pool_flat[(token_idx[:t].long() + 1).clamp_max(limit)])
        hx = d.layer(emb, feat, batch.positions[:t], batch.out_loc[:t], md.block_table, md.cu_q, md.seq_lens,
                     md.max_q, md.max_kv)
        last = torch.from_numpy((cu_q_np[1:] - 1).astype(np.int64)).to(eng.device, non_blocking=True)
        d.hidden[torch.from_numpy(slots_np.astype(np.int64)).to(eng.device, non_blocking=True)] = hx[last]

    # ------------------------------------------------------------------ graphs
    def capture(self) -> None:
        eng = self.engine
        if eng.device.type != "cuda" or eng.config.cuda_graph_max_bs == -1:
            return
        from ..env import ENV

        if ENV.DISABLE_GRAPH.value:
            return
        self._fill_dummy(self.max_bs)
        stream = eng.stream or torch.cuda.current_stream()
        torch.cuda.synchronize()
        with torch.cuda.stream(stream):
            for bs in sorted(self.buckets, reverse=True):
                for _ in range(2):
                    self.body(bs)
                stream.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, pool=self.pool, stream=stream):
                    self.body(bs)
                if self.pool is None:
                    self.pool = g.pool()
                self.graphs[bs] = g
        torch.cuda.synchronize()
        logger.info_rank0("captured %d speculative-step graphs (width %d, buckets up to %d)", len(self.graphs),
                          self.W, self.max_bs)

    def _fill_dummy(self, bs: int) -> None:
        """Tables of a step made of padding requests only (dummy slot, scratch page)."""
        host = self._dummy_tables(bs)
        self.arena.copy_(torch.from_numpy(host))

    def _dummy_tables(self, bs: int) -> np.ndarray:
        eng, W, K, P = self.engine, self.W, self.K, self.P
        host = np.zeros(self.arena_len, dtype=np.int32)
        self.pack(host, [], [], bs)
        return host

    # ------------------------------------------------------------------ host side: tables of one step
    def bucket_of(self, bs: int) -> int:
        for b in self.buckets:
            if b >= bs:
                return b
        raise ValueError(bs)

    def pack(self, host: np.ndarray, rows: List[dict], staged: List[List[int]], bucket: int) -> None:
        """Fill ``host`` (arena layout) for ``rows`` = per request dict(slot, c, k, max_emit, ignore_eos,
        alloc_end, pages) padded to ``bucket`` requests."""
        eng, W, K, P = self.engine, self.W, self.K, self.P
        ps, msl = eng.page_size, eng.max_seq_len
        dummy_slot = eng.num_slots - 1
        dummy_page = eng.kv_cache.dummy_page
        B = self.max_bs

        def put(name, arr):
            off, n = self.offsets[name]
            a = np.asarray(arr, dtype=np.int32).reshape(-1)
            host[off:off + a.size] = a

        n = len(rows)
        slot = np.full(bucket, dummy_slot, dtype=np.int64)
        c = np.zeros(bucket, dtype=np.int64)
        k = np.zeros(bucket, dtype=np.int64)
        alloc_end = np.zeros(bucket, dtype=np.int64)
        max_emit = np.ones(bucket, dtype=np.int64)
        flags = np.ones(bucket, dtype=np.int64)
        bt = np.full((bucket, P), dummy_page, dtype=np.int32)
        for i, r in enumerate(rows):
            slot[i], c[i], k[i] = r["slot"], r["c"], r["k"]
            alloc_end[i], max_emit[i], flags[i] = r["alloc_end"], r["max_emit"], 1 if r["ignore_eos"] else 0
            pages = r["pages"]
            bt[i, :len(pages)] = pages
        j = np.arange(W, dtype=np.int64)[None, :]
        pos = c[:, None] + j                                   # [bucket, W]
        live = pos < alloc_end[:, None]
        pos_c = np.minimum(pos, msl - 1)
        page = np.take_along_axis(bt.astype(np.int64), np.minimum(pos_c // ps, P - 1), axis=1)
        loc = np.where(live, page * ps + pos_c % ps, dummy_page * ps + (j % ps))
        tok = slot[:, None] * msl + np.minimum(pos, msl - 2)
        if self.T == 1:
            put("token_idx", tok)
            put("positions", pos_c)
            put("out_loc", loc)
            put("seq_lens", np.minimum(c + W, msl))
        else:
            T, R = self.T, self.R
            put("u_tok_idx", tok)
            put("u_positions", pos_c)
            put("u_out_loc", loc)
            put("u_seq_lens", np.minimum(c + W, msl))
            # sibling i (depth-major): position of its depth, K/V at scratch position c + K + 1 + i
            i_s = np.arange(K * (T - 1), dtype=np.int64)[None, :]
            s_pos = np.minimum(c[:, None] + i_s // (T - 1) + 1, msl - 1)
            s_at = c[:, None] + K + 1 + i_s
            s_live = s_at < alloc_end[:, None]
            s_at_c = np.minimum(s_at, msl - 1)
            s_page = np.take_along_axis(bt.astype(np.int64), np.minimum(s_at_c // ps, P - 1), axis=1)
            s_loc = np.where(s_live, s_page * ps + s_at_c % ps, dummy_page * ps + (i_s % ps))
            put("token_idx", np.concatenate([tok, np.full_like(s_pos, dummy_slot * msl)], axis=1))
            put("positions", np.concatenate([pos_c, s_pos], axis=1))
            put("out_loc", np.concatenate([loc, s_loc], axis=1))
            put("seq_lens", np.minimum(c + R, msl))
        off, _ = self.offsets["block_table"]
        host[off:off + bucket * P] = bt.reshape(-1)
        put("first_idx", slot * msl + np.minimum(c + 1, msl - 1))
        put("num_draft", k)
        put("max_emit", max_emit)
        put("flags", flags)
        put("slots", slot)
        # host-proposed drafts (unused entries point at the dummy slot's row)
        s_idx = np.full((bucket, K), dummy_slot * msl, dtype=np.int64)
        s_tok = np.zeros((bucket, K), dtype=np.int64)
        for i, dr in enumerate(staged):
            for jj, t in enumerate(dr[:K]):
                s_idx[i, jj] = slot[i] * msl + c[i] + 1 + jj
                s_tok[i, jj] = t
        put("stage_idx", s_idx)
        put("stage_tok", s_tok)
        # chain step i (1 .. K-1): input token d_i at pool position c + i, draft position c + i - 1
        steps = np.arange(1, max(K, 2), dtype=np.int64)[:, None]          # [K-1, 1]
        cpos = c[None, :] + steps - 1                                        # [K-1, bucket]
        clive = cpos < alloc_end[None, :]
        cpos_c = np.minimum(cpos, msl - 1)
        cpage = bt.astype(np.int64)[np.arange(bucket)[None, :], np.minimum(cpos_c // ps, P - 1)]
        cloc = np.where(clive, cpage * ps + cpos_c % ps, dummy_page * ps)

        def put2(name, arr):   # [steps, bucket] into a [steps, max_bs] table
            off, n_ = self.offsets[name]
            rows_ = arr.shape[0]
            view = host[off:off + rows_ * B].reshape(rows_, B)
            view[:, :bucket] = arr

        put2("c_tok_idx", slot[None, :] * msl + np.minimum(c[None, :] + steps, msl - 1))
        put2("c_positions", cpos_c)
        put2("c_out_loc", cloc)
        put2("c_seq_lens", np.minimum(cpos_c + 1, msl))
        dsteps = np.arange(K, dtype=np.int64)[:, None]                       # draft i+1 goes to position c + 1 + i
        dpos = c[None, :] + 1 + dsteps
        dst = np.where((dpos < msl) & (slot[None, :] != dummy_slot), slot[None, :] * msl + np.minimum(dpos, msl - 1), -1)
        put2("c_dst_idx", dst)

    def run(self, rows: List[dict], staged: List[List[int]]) -> np.ndarray:
        """Executes one step for ``rows`` and returns the acceptance record ``[len(rows), W + 2]``
        (count, EOS flag, emitted tokens)."""
        eng = self.engine
        bs = len(rows)
        graph_ok = bool(self.graphs) and bs <= self.max_bs
        bucket = self.bucket_of(bs) if graph_ok else bs
        pin = self._pin_pos % 2
        self._pin_pos += 1
        ev = self._pin_events[pin]
        if ev is not None:
            ev.synchronize()
        host = self._pinned[pin].numpy()
        self.pack(host, rows, staged, bucket)
        self.arena.copy_(self._pinned[pin], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._pin_events[pin] = ev
        eng.h2d_bytes += 4 * self.arena_len
        if graph_ok:
            self.graphs[bucket].replay()
            self.replays += 1
        else:
            self.body(bucket)
            self.eager_steps += 1
        n = bs * (self.W + 2)
        rec = self._rec_host[pin]
        rec[:n].copy_(self.record[:n], non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        done.synchronize()
        eng.d2h_bytes += 4 * n
        return rec[:n].numpy().reshape(bs, self.W + 2).copy()
