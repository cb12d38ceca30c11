"""CUDA-graph capture and replay of the decode step.

One graph per batch-size bucket ``[1,2,4,8,12,16,24,32] + range(48, max+1, 16) + [max]``
(python/minisgl/engine/graph.py:169-212). A decode batch is padded on the host to the next
bucket with rows that read the dummy request's token and write the dummy KV page
(python/minisgl/engine/graph.py:473-479), copied into static device buffers, and the graph
(token gather → all layers → LM head) is launched with one ``cudaGraphLaunch``. Sampling runs
after the graph on the static logits buffer.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np
import torch

from ..core import Batch
from ..env import ENV
from ..utils import init_logger

logger = init_logger(__name__)


def graph_buckets(max_bs: int) -> List[int]:
    base = [b for b in (1, 2, 4, 8, 12, 16, 24, 32) if b <= max_bs]
    base += list(range(48, max_bs + 1, 16))
    if max_bs not in base:
        base.append(max_bs)
    return sorted(set(base))


class GraphRunner:
    def __init__(self, engine) -> None:
        self.engine = engine
        cfg = engine.config
        want = cfg.cuda_graph_max_bs or ENV.GRAPH_MAX_BS.value or min(cfg.max_running_req, 256)
        self.max_bs = int(min(want, cfg.max_running_req))
        self.buckets = graph_buckets(self.max_bs) if self.max_bs > 0 else []
        dev = engine.device
        n, p = self.max_bs, engine.max_pages_per_seq
        self.token_idx = torch.zeros(n, dtype=torch.int32, device=dev)
        self.positions = torch.zeros(n, dtype=torch.int32, device=dev)
        self.out_loc = torch.zeros(n, dtype=torch.int32, device=dev)
        self.seq_lens = torch.ones(n, dtype=torch.int32, device=dev)
        self.cu_q = torch.arange(n + 1, dtype=torch.int32, device=dev)
        self.block_table = torch.full((max(n, 1), p), engine.kv_cache.dummy_page, dtype=torch.int32, device=dev)
        self.graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        self.logits: Dict[int, torch.Tensor] = {}
        self.kernels_per_graph: Dict[int, int] = {}
        self.pool = None
        self.replays = 0
        from ..utils.tracing import GraphTimer

        self.timer = GraphTimer()
        if self.buckets:
            self._capture_all()

    def can_run(self, bs: int) -> bool:
        return bool(self.graphs) and bs <= self.max_bs

    def bucket_of(self, bs: int) -> int:
        for b in self.buckets:
            if b >= bs:
                return b
        raise ValueError(bs)

    # ------------------------------------------------------------------ capture
    def _run_model(self, bs: int) -> torch.Tensor:
        eng = self.engine
        batch = Batch(reqs=[], phase="decode")
        batch.positions = self.positions[:bs]
        batch.out_loc = self.out_loc[:bs]
        batch.input_ids = eng.token_pool.view(-1)[self.token_idx[:bs].long()]
        if eng.gdn_state is not None:
            batch.gdn_slots = (self.token_idx[:bs] // eng.max_seq_len).to(torch.int32)
            batch.gdn_has_state = torch.ones(bs, dtype=torch.int32, device=eng.device)
        if eng.swa is not None:
            # inside the graph: derived from the static inputs and the device copy of the pool's page table
            batch.swa_out_loc, batch.swa_block_table = eng.swa_arrays(
                self.token_idx[:bs], self.positions[:bs], self.cu_q[: bs + 1], self.block_table.shape[1])
        eng.ctx.attn_backend.prepare_metadata(
            batch, self.block_table[:bs], self.cu_q[: bs + 1], self.seq_lens[:bs], 1, eng.max_seq_len)
        with eng.ctx.forward_batch(batch):
            hidden = eng.model.forward(batch.input_ids)
            # the vocabulary shard only: gathering (or the shard arg-max) happens after the replay
            return eng.model.lm_head.forward_local(hidden)

    def _capture_all(self) -> None:
        from ..ops import cuda as K

        eng = self.engine
        ep = getattr(eng.ctx, "ep", None)
        if ep is not None and hasattr(ep, "static_bound"):
            # Expert-parallel replicas run their warm-up forwards together (each one exchanges rows
            # with every peer), under the row bound of the largest bucket. All replicas have the same
            # bucket list, so they stay in step; the barrier removes the boot skew first.
            import torch.distributed as dist

            ep.static_bound = self.max_bs
            ep.common_tokens = None
            dist.barrier(group=eng.dp_cpu_group)
        dummy_slot = eng.kv_cache.dummy_page * eng.page_size
        self.out_loc.fill_(dummy_slot)
        self.token_idx.fill_((eng.num_slots - 1) * eng.max_seq_len)
        torch.cuda.synchronize()
        stream = eng.stream or torch.cuda.current_stream()
        with torch.cuda.stream(stream):
            for bs in sorted(self.buckets, reverse=True):
                for _ in range(2):  # warm-up: lazy attribute setup, descriptor caches, allocator
                    self._run_model(bs)
                stream.synchronize()
                before = K.LAUNCHES
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, pool=self.pool, stream=stream):
                    self.logits[bs] = self._run_model(bs)
                if self.pool is None:
                    self.pool = g.pool()
                self.graphs[bs] = g
                self.kernels_per_graph[bs] = K.LAUNCHES - before
        torch.cuda.synchronize()
        logger.info_rank0("captured %d decode graphs (buckets up to %d)", len(self.graphs), self.max_bs)

    # ------------------------------------------------------------------ replay
    def pad_plan_arrays(self, bs: int, bucket: int, token_idx: np.ndarray, positions: np.ndarray,
                        out_loc: np.ndarray, seq_lens: np.ndarray):
        """Host-side padding rows: dummy token, position 0, dummy KV slot, length 1."""
        pad = bucket - bs
        if pad == 0:
            return token_idx, positions, out_loc, seq_lens
        eng = self.engine
        d_tok = np.full(pad, (eng.num_slots - 1) * eng.max_seq_len, dtype=np.int32)
        d_pos = np.zeros(pad, dtype=np.int32)
        d_loc = np.full(pad, eng.kv_cache.dummy_page * eng.page_size, dtype=np.int32)
        d_len = np.ones(pad, dtype=np.int32)
        return (np.concatenate([token_idx, d_tok]), np.concatenate([positions, d_pos]),
                np.concatenate([out_loc, d_loc]), np.concatenate([seq_lens, d_len]))

    def replay(self, bs: int, token_idx: torch.Tensor, positions: torch.Tensor, out_loc: torch.Tensor,
               seq_lens: torch.Tensor, block_table: torch.Tensor) -> torch.Tensor:
        """Inputs are device tensors already padded to the bucket (``block_table`` is
        ``[bucket, n_pages]``)."""
        from ..ops import cuda as K

        bucket = token_idx.numel()
        self.token_idx[:bucket].copy_(token_idx)
        self.positions[:bucket].copy_(positions)
        self.out_loc[:bucket].copy_(out_loc)
        self.seq_lens[:bucket].copy_(seq_lens)
        self.block_table[:bucket, : block_table.shape[1]].copy_(block_table)
        tok = self.timer.begin(bucket)
        self.graphs[bucket].replay()
        self.timer.end(tok)
        K.LAUNCHES += self.kernels_per_graph[bucket]
        self.replays += 1
        return self.logits[bucket][:bs]
