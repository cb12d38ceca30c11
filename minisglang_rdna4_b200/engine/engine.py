"""Per-rank engine: owns the model, the KV pool, the token pool, the attention backend, the
sampler and the CUDA graphs, and runs one forward step for the scheduler.

Boot order follows python/minisgl/engine/engine.py:217-845: rank info → device/stream →
communication → model on the target device → weights (checkpoint or random) → post-load
repack → KV sizing (min over ranks) → pools → attention backend → sampler → graph capture.

Host→device traffic of a step is one pinned int32 staging buffer (gather indices, positions,
KV slots, lengths, block table, sample rows); device→host traffic is the sampled ids.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from datetime import timedelta
from typing import List, Optional

import numpy as np
import torch
import torch.distributed as dist

from ..attention import create_attention_backend
from ..config import EngineConfig
from ..core import Batch, Context, set_global_ctx
from ..env import ENV
from ..kvcache import MHAKVCache
from ..models import create_model
from ..models.config import NAMED_CONFIGS, ModelConfig
from ..parallel import comm as comm_mod
from ..parallel.info import set_dp_info, set_ep, set_tp_info
from ..utils import cdiv, div_even, init_logger
from .sample import BatchSamplingArgs, SampleOutput, Sampler

logger = init_logger(__name__)


@dataclass
class StepPlan:
    """Host-side description of one forward step (all int32 NumPy arrays)."""

    token_idx: np.ndarray      # [T] flat index into the token pool of every input token
    positions: np.ndarray      # [T]
    out_loc: np.ndarray        # [T] KV slot of every input token
    cu_q: np.ndarray           # [B+1]
    seq_lens: np.ndarray       # [B]
    block_table: np.ndarray    # [B, P]
    sample_rows: np.ndarray    # [S] rows of the packed hidden states that are sampled
    write_idx: np.ndarray      # [S] flat token-pool index receiving each sampled token
    max_q: int = 1
    max_kv: int = 1

    @property
    def num_tokens(self) -> int:
        return int(self.token_idx.shape[0])

    @property
    def h2d_bytes(self) -> int:
        return 4 * (3 * self.token_idx.size + self.cu_q.size + self.seq_lens.size
                    + self.block_table.size + self.sample_rows.size + self.write_idx.size)


@dataclass
class ForwardOutput:
    tokens_gpu: torch.Tensor
    tokens_cpu: torch.Tensor
    event: Optional["torch.cuda.Event"]
    sample: Optional[SampleOutput] = None
    logits: Optional[torch.Tensor] = None

    def wait(self) -> torch.Tensor:
        if self.event is not None:
            self.event.synchronize()
        return self.tokens_cpu


def _resolve_dtype(cfg: EngineConfig, model_cfg: ModelConfig, device: str) -> torch.dtype:
    name = cfg.dtype
    if name == "auto":
        name = "fp32" if device == "cpu" else model_cfg.torch_dtype
    table = {"fp16": torch.float16, "float16": torch.float16, "half": torch.float16,
             "bf16": torch.bfloat16, "bfloat16": torch.bfloat16,
             "fp32": torch.float32, "float32": torch.float32, "float": torch.float32}
    dt = table[name]
    if device == "cuda" and dt == torch.float32:
        dt = torch.bfloat16
    return dt


def resolve_model_config(cfg: EngineConfig) -> ModelConfig:
    if cfg.model_config is not None:
        mc = cfg.model_config
    elif cfg.model_path in NAMED_CONFIGS:
        mc = NAMED_CONFIGS[cfg.model_path]()
    else:
        mc = ModelConfig.from_hf(cfg.model_path)
        # the serving list of stop tokens lives in generation_config.json; config.json often names
        # only one of them
        from dataclasses import replace

        from ..utils.hf import resolve_stop_token_ids

        stops = resolve_stop_token_ids(cfg.model_path, None, mc.eos_token_ids)
        if tuple(stops) != tuple(mc.eos_token_ids):
            mc = replace(mc, eos_token_ids=tuple(stops))
    if cfg.quantization and mc.quant is None:
        from ..quant.config import QuantConfig

        qc = {
            "mxfp4": {"quant_method": "mxfp4"},
            "fp8": {"quant_method": "compressed-tensors", "config_groups": {"g": {
                "weights": {"num_bits": 8, "type": "float", "strategy": "channel"}, "targets": ["Linear"]}},
                "ignore": ["lm_head"]},
            "fp8_block": {"quant_method": "fp8", "weight_block_size": [128, 128]},
            "nvfp4": {"quant_method": "compressed-tensors", "format": "nvfp4-pack-quantized", "config_groups": {"g": {
                "weights": {"num_bits": 4, "type": "float", "group_size": 16}, "targets": ["Linear"]}},
                "ignore": ["lm_head"]},
            "int4": {"quant_method": "gptq", "bits": 4, "group_size": 128, "sym": True},
        }[cfg.quantization]
        mc = mc.with_quant(QuantConfig.from_hf(qc))
    return mc


class Engine:
    def __init__(self, config: EngineConfig) -> None:
        from ..weights import BootTimeline, MemoryLedger

        self.config = config
        self.boot = BootTimeline()
        self.ledger = MemoryLedger()
        set_tp_info(config.tp_rank, config.tp_size)
        set_dp_info(config.dp_rank, config.dp_size)
        set_ep(config.enable_ep, over_tp=(config.dp_size == 1))
        dev_kind = config.resolve_device()
        if dev_kind == "cuda":
            local = int(os.environ.get("LOCAL_RANK", config.device_id)) if "LOCAL_RANK" in os.environ else config.device_id
            self.device = torch.device("cuda", local)
            torch.cuda.set_device(self.device)
            self.stream = torch.cuda.Stream(self.device)
        else:
            self.device = torch.device("cpu")
            self.stream = None
        self.model_config = resolve_model_config(config)
        self.dtype = _resolve_dtype(config, self.model_config, dev_kind)
        self.cpu_group: Optional[dist.ProcessGroup] = None
        self.tp_group: Optional[dist.ProcessGroup] = None
        self.dp_group: Optional[dist.ProcessGroup] = None
        self.dp_cpu_group: Optional[dist.ProcessGroup] = None
        self._init_communication()
        self.boot.mark("process groups")
        if dev_kind == "cuda":
            self.ledger.capacity = int(torch.cuda.get_device_properties(self.device).total_memory)

        free_before = self._free_memory()
        self.model = create_model(self.model_config, self.dtype, self.device)
        if config.use_dummy_weight or not config.model_path or config.model_path in NAMED_CONFIGS:
            gen_dev = "cuda" if dev_kind == "cuda" else "cpu"
            self.model.init_dummy(config.seed, gen_device=gen_dev)
        else:
            from ..models.weight import load_weights

            baked_dir = ENV.BAKED_DIR.value
            loaded = None
            if baked_dir:
                # Stage B: this rank's weights as an earlier boot left them after loading, streamed from
                # one flat file; Stage A (below) when there is no file for this configuration yet
                from ..parallel.info import ep_enabled
                from ..weights import bake

                rank = config.tp_rank + config.tp_size * getattr(config, "dp_rank", 0)
                mark = bake.fingerprint(self.model_config, config.model_path, self.dtype, config.tp_rank,
                                        config.tp_size, ep=f"{ep_enabled()}:{getattr(config, 'dp_rank', 0)}/"
                                                           f"{getattr(config, 'dp_size', 1)}")
                loaded = bake.load_bake(self.model, baked_dir, rank, mark, self.device,
                                        verify=ENV.BAKED_VERIFY.value)
                if loaded is not None:
                    logger.info_rank0("weights from the baked file in %s (%.2f GiB)", baked_dir, loaded / 2 ** 30)
            if loaded is None:
                load_weights(self.model, config.model_path, self.model_config, self.device)
                if baked_dir:
                    n = bake.write_bake(self.model, baked_dir, rank, mark)
                    logger.info_rank0("baked this rank's weights into %s (%.2f GiB)", baked_dir, n / 2 ** 30)
            self.baked_bytes = loaded
        self._configure_expert_tier()
        self.model.post_load()
        # vision tower of a multimodal checkpoint: replicated on every rank, runs once per image at admission
        self.vision = None
        if self.model_config.vision is not None:
            if getattr(self.model_config.vision, "kind", "") == "gemma4":
                from ..models.gemma4_vision import Gemma4VisionTower as VisionTower
            else:
                from ..models.siglip import VisionTower

            self.vision = VisionTower(self.model_config.vision, self.dtype, self.device)
            if config.use_dummy_weight or not config.model_path or config.model_path in NAMED_CONFIGS:
                self.vision.init_dummy(config.seed + 29)
            else:
                try:
                    self.vision.load(config.model_path)
                except KeyError as exc:
                    logger.warning("%s: serving the text decoder only", exc)
                    self.vision = None
        if dev_kind == "cuda":
            torch.cuda.synchronize()
            torch.cuda.empty_cache()
        self.model_bytes = max(free_before - self._free_memory(), 0)
        self.ledger.add("weights", self.model_bytes)
        self.boot.mark("weights (load + post-load)")

        # ---- KV pool ----
        mc = self.model_config
        self.page_size = config.page_size
        self.kv_heads_local = div_even(mc.num_kv_heads, config.tp_size, allow_replicate=True)
        self.q_heads_local = div_even(mc.num_qo_heads, config.tp_size)
        kv_fp8 = config.kv_cache_dtype == "fp8" or (config.kv_cache_dtype == "auto" and (
            ENV.KV_FP8.value or (mc.quant is not None and mc.quant.kv_cache_fp8)))
        self.kv_calibrating = bool(ENV.KV_FP8_CALIBRATE.value)
        self.kv_fp8 = bool(kv_fp8) and not self.kv_calibrating
        # sliding-window layers in a pool of their own (MSGL_SWA_POOL): the layers are re-numbered per pool
        self.swa = None
        self.swa_kv_cache = None
        self._swa_layers = 0
        self.kv_layers = mc.num_kv_layers          # hybrid models keep K/V pages for their attention layers only
        if ENV.SWA_POOL.value and mc.swa_layers:
            if config.spec_algorithm != "none" and getattr(config, "spec_tree_width", 1) > 1:
                # a tree's attention mask replaces the window rule of the sliding layers
                raise ValueError("the sliding-window pool (MSGL_SWA_POOL) does not work with tree verification; "
                                 "use a draft chain (spec tree width 1)")
            from ..layers.attention import AttentionLayer

            n_global = n_swa = 0
            for mod in self.model.modules():
                if isinstance(mod, AttentionLayer) and mod._kv_donor is None:
                    if mod._window > 0:
                        mod._swa, mod._kv_index = True, n_swa
                        n_swa += 1
                    else:
                        mod._swa, mod._kv_index = False, n_global
                        n_global += 1
            self._swa_layers = n_swa
            self.kv_layers = max(n_global, 1)      # a model without global layers keeps a one-layer main pool
            self._swa_window = int(mc.sliding_window)
            # pages a request can hold (its window, the page being written, one partly outside the window),
            # for every request slot, plus the pages of one prefill step
            self._swa_pages = ((config.max_running_req + 1) * (cdiv(self._swa_window, self.page_size) + 3)
                               + cdiv(getattr(config, "max_extend_tokens", 8192), self.page_size))
            # windows kept for prefix reuse pin pages of this pool: room for them on top
            itemsize_ = 1 if self.kv_fp8 else torch.empty((), dtype=self.dtype).element_size()
            page_bytes = self.page_size * MHAKVCache.token_bytes(n_swa, self.kv_heads_local, mc.head_dim, itemsize_)
            self._swa_page_bytes = page_bytes
            if config.cache_type == "radix" and ENV.RECURRENT_SNAPSHOT_MIB.value > 0:
                self._swa_pages += (ENV.RECURRENT_SNAPSHOT_MIB.value << 20) // max(page_bytes, 1)
        # layers that read an earlier layer's K/V take that layer's pool and row
        if mc.num_kv_shared_layers:
            from ..layers.attention import AttentionLayer

            by_id = {m._layer_id: m for m in self.model.modules() if isinstance(m, AttentionLayer)}
            for m in by_id.values():
                if m._kv_donor is not None:
                    m._swa, m._kv_index = by_id[m._kv_donor]._swa, by_id[m._kv_donor]._kv_index
        # (kv heads, head width) of the main pool and, with two pools, of the sliding-window one
        tp_ = config.tp_size
        geoms = [mc.attn_geometry(i) for i in range(mc.num_kv_layers)] if mc.global_head_dim else None
        self._main_geometry = None
        self._swa_geometry = (self.kv_heads_local, mc.head_dim)
        if geoms:
            local = [(div_even(h, tp_, allow_replicate=True), d) for h, d in geoms]
            if self._swa_layers:
                swa_set = set(mc.swa_layers)
                self._main_geometry = [g_ for i, g_ in enumerate(local) if i not in swa_set] or [local[0]]
                self._swa_geometry = next(g_ for i, g_ in enumerate(local) if i in swa_set)
            else:
                self._main_geometry = local
            widths = {d for _, d in local}
            if self.device.type == "cuda" and (len(set(self._main_geometry)) > 1 or not widths <= {64, 128, 256}):
                raise NotImplementedError(
                    f"attention head widths {sorted(widths)}: the attention kernels are built for 64 / 128 / 256 "
                    "and one geometry per pool; this model runs on the CPU oracle path only")
        # latent-attention models can keep the compressed latent per token instead of per-head K/V
        # (MSGL_MLA_LATENT): absorbed attention through tensor ops, eager steps, no draft verification
        self.mla_latent = bool(ENV.MLA_LATENT.value and mc.is_mla)
        if self.mla_latent:
            if self.kv_fp8 or self.kv_calibrating:
                raise ValueError("the latent pool (MSGL_MLA_LATENT) is 16-bit only")
            if config.spec_algorithm != "none":
                raise ValueError("the latent pool (MSGL_MLA_LATENT) does not verify drafts; turn speculation off")
        self.num_pages = self._determine_num_pages()
        self.max_seq_len = self._resolve_max_seq_len()
        self.max_pages_per_seq = cdiv(self.max_seq_len, self.page_size)
        if self.mla_latent:
            from ..kvcache.mla_pool import MLALatentCache

            self.kv_cache = MLALatentCache(self.kv_layers, self.num_pages, self.page_size, int(mc.kv_lora_rank),
                                           int(mc.qk_rope_head_dim), self.dtype, self.device)
            logger.info_rank0("latent K/V pool: %d values per token and layer (per-head K/V would take %d)",
                              self.kv_cache.width, 2 * self.kv_heads_local * mc.head_dim)
        else:
            self.kv_cache = MHAKVCache(
                self.kv_layers, self.num_pages, self.page_size, self.kv_heads_local, mc.head_dim,
                self.dtype, self.device, fp8=self.kv_fp8, geometry=self._main_geometry,
            )
        if self.kv_fp8:
            from ..kvcache.fp8_scales import resolve_kv_scales

            ks, vs, source = resolve_kv_scales(config.model_path, mc.num_kv_layers if self._swa_layers else self.kv_layers,
                                               mc.num_kv_heads, config.tp_rank, config.tp_size)
            self._kv_scales = (ks, vs)
            if self._swa_layers:                   # the scales of the layers that stay in the main pool
                keep = [i for i in range(mc.num_kv_layers) if i not in set(mc.swa_layers)] or [0]
                ks, vs = ks[keep], vs[keep]
            self.kv_cache.set_scales(ks, vs)
            logger.info_rank0("fp8 KV scales: %s", source)
        if self.kv_calibrating:
            self.kv_cache.start_calibration()
            logger.info_rank0("fp8 KV calibration run: 16-bit pool, eager steps")
        self.ledger.add("kv pool", self.kv_cache._buf.numel() * self.kv_cache._buf.element_size())
        if self._swa_layers:
            from ..kvcache.swa_pages import SwaPages

            self.swa_kv_cache = MHAKVCache(self._swa_layers, self._swa_pages, self.page_size, self._swa_geometry[0],
                                           self._swa_geometry[1], self.dtype, self.device, fp8=self.kv_fp8)
            if self.kv_fp8:
                ids = list(mc.swa_layers)
                self.swa_kv_cache.set_scales(self._kv_scales[0][ids], self._kv_scales[1][ids])
            self.swa = SwaPages(config.max_running_req + 1, self.max_pages_per_seq, self._swa_pages, self.page_size,
                                self._swa_window, self.device)
            assert self.swa.dummy == self.swa_kv_cache.dummy_page
            self.swa.page_nbytes = self._swa_page_bytes
            self.ledger.add("sliding-window kv pool",
                            self.swa_kv_cache._buf.numel() * self.swa_kv_cache._buf.element_size())
            logger.info_rank0("sliding-window K/V pool: %d layers x %d pages (window %d), main pool %d layers",
                              self._swa_layers, self._swa_pages, self._swa_window, self.kv_layers)
        self.boot.mark("kv pool")
        # slot max_running_req is the dummy request used to pad graph batches
        self.num_slots = config.max_running_req + 1
        self.token_pool = torch.zeros((self.num_slots, self.max_seq_len), dtype=torch.int32, device=self.device)
        self.ctx = Context(page_size=self.page_size)
        self.ctx.kv_cache = self.kv_cache
        self.ctx.swa_kv_cache = self.swa_kv_cache
        self.gdn_state = None
        if mc.is_recurrent:
            from ..kvcache.gdn_state import GDNStateCache

            conv_dim, st_heads, st_rows, st_cols = mc.recurrent_geometry
            conv_dim, st_heads = conv_dim // config.tp_size, st_heads // config.tp_size   # this rank's heads
            self.gdn_state = GDNStateCache(mc.num_linear_layers, self.num_slots, conv_dim, mc.linear_conv_kernel_dim,
                                           st_heads, st_rows, st_cols, self.dtype, self.device)
            self.ledger.add("recurrent state", self.gdn_state.conv.numel() * self.gdn_state.conv.element_size()
                            + self.gdn_state.ssm.numel() * 4)
        self.ctx.gdn_state = self.gdn_state
        if self.gdn_state is not None and dev_kind == "cuda":
            self.gdn_state.stream = self.stream
        self.ctx.attn_backend = create_attention_backend(
            config.attention_backend, self.q_heads_local, self.kv_heads_local, mc.head_dim, self.device,
            max_batch=config.max_running_req, max_seq_len=self.max_seq_len,
            single_split=config.spec_algorithm != "none",
        )
        self.ctx.comm = comm_mod.get_comm()
        self._spec_exact = config.spec_algorithm != "none" and dev_kind == "cuda"
        if self._spec_exact:
            # greedy speculative decoding must reproduce plain decoding bit for bit: verify rows
            # (many per request) and decode rows have to take the same GEMM code path, so K is
            # never split and verify steps never switch to the CTA-pair kernel
            from ..ops import cuda as K

            K.SPLIT_K = False
            K.SPLIT_K_DECODE = False
        if config.enable_ep and config.dp_size > 1:
            from ..parallel.ep import EPContext, FusedEPContext

            self.ctx.ep = None
            from ..layers.moe import MoELayer as _MoeCls

            if (dev_kind == "cuda" and mc.is_moe and not ENV.DISABLE_FUSED_COMM.value
                    and not _MoeCls.offload_slots):
                try:
                    kinds = {m._quant_kind or "bf16" for m in self.model.modules() if isinstance(m, _MoeCls)}
                    kind = kinds.pop() if len(kinds) == 1 else "bf16"
                    # regions for the largest step (a full prefill chunk) as long as they stay within
                    # MSGL_EP_REGION_GIB per rank; the 16-bit return rows dominate: 2 bytes x hidden
                    # x top_k x ranks per token
                    per_token = mc.hidden_size * mc.num_experts_per_tok * config.dp_size * 3 + 64
                    fit = int((ENV.EP_REGION_GIB.value << 30) // per_token)
                    want = max(config.max_running_req, config.max_extend_tokens)
                    self.ctx.ep = FusedEPContext(
                        self.dp_group, self.dp_cpu_group, config.dp_rank, config.dp_size, self.device,
                        mc.hidden_size, mc.num_experts_per_tok, mc.num_experts // config.dp_size,
                        max_tokens=max(min(want, fit), min(config.max_running_req, 512)), kind=kind)
                    self.ledger.add("expert exchange regions", self.ctx.ep.region_bytes)
                except Exception as exc:
                    logger.warning("fused expert-parallel exchange unavailable (%s); using NCCL", exc)
            if self.ctx.ep is None:
                self.ctx.ep = EPContext(self.dp_group, config.dp_rank, config.dp_size)
        set_global_ctx(self.ctx)
        self.sampler = Sampler(self.device, mc.vocab_size, mc.final_logit_softcapping, seed=config.seed)
        self._staging_cap = 0
        self._ring = 4
        self._ring_pos = 0
        self._out_pos = 0
        self._out_ring = [None] * self._ring
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.steps = 0
        self.graph_runner = None
        # Replicas that exchange expert rows every layer can only capture their decode step when
        # the exchange itself is capturable (the peer-memory kernels with device-resident sequence
        # numbers, under a fixed row bound); the NCCL gather / reduce form pins the agreed row count
        # and runs eagerly.
        from ..parallel.ep import FusedEPContext as _FusedEP

        ep_replicas = config.enable_ep and config.dp_size > 1 and not isinstance(self.ctx.ep, _FusedEP)
        from ..layers.moe import MoELayer as _Moe

        host_tier = _Moe.offload_slots > 0   # expert residency is decided on the host every step
        if dev_kind == "cuda":
            from ..ops import cuda as K

            K.set_pdl(ENV.PDL.value)
            # model parameters never change while kernels run, unless experts are paged in from the
            # host tier: only then must a GEMM wait for the stream before it reads its weights
            K.gemm_static_weights((2 if ENV.GEMM_L2_AHEAD.value else 1) if (ENV.PDL.value and not host_tier) else 0)
        if (dev_kind == "cuda" and not ENV.DISABLE_GRAPH.value and not self.kv_calibrating and (config.cuda_graph_max_bs or 0) >= 0
                and not ep_replicas and not host_tier and not self.mla_latent):
            from .graph import GraphRunner

            before = self._free_memory()
            self.graph_runner = GraphRunner(self)
            self.ledger.add("cuda graphs", max(before - self._free_memory(), 0))
            self.boot.mark("graph capture")
        logger.info_rank0("%s", self.ledger.report())
        logger.info_rank0("%s", self.boot.render())
        logger.info_rank0(
            "engine ready: %s, %d pages x %d tokens, max_seq_len %d, dtype %s, kv %s",
            mc.model_type, self.num_pages, self.page_size, self.max_seq_len, self.dtype,
            "fp8" if self.kv_fp8 else str(self.dtype))

    # ------------------------------------------------------------------ boot helpers
    def _init_communication(self) -> None:
        cfg = self.config
        comm = comm_mod.reset_comm()
        world = cfg.tp_size * cfg.dp_size
        if world == 1:
            return
        timeout = timedelta(seconds=cfg.distributed_timeout)
        backend = "nccl" if self.device.type == "cuda" else "gloo"
        if not dist.is_initialized():
            if "RANK" in os.environ and "MASTER_ADDR" in os.environ:
                dist.init_process_group(backend, timeout=timeout,
                                        device_id=self.device if backend == "nccl" else None)
            else:
                dist.init_process_group(backend, init_method=cfg.world_addr, rank=cfg.global_rank,
                                        world_size=world, timeout=timeout,
                                        device_id=self.device if backend == "nccl" else None)
        # one TP group per replica; every rank must create all of them
        for r in range(cfg.dp_size):
            ranks = list(range(r * cfg.tp_size, (r + 1) * cfg.tp_size))
            g = dist.new_group(ranks, backend=backend, timeout=timeout)
            c = dist.new_group(ranks, backend="gloo", timeout=timeout)
            if r == cfg.dp_rank:
                self.tp_group, self.cpu_group = g, c
        if cfg.dp_size > 1:
            for t in range(cfg.tp_size):
                ranks = [r * cfg.tp_size + t for r in range(cfg.dp_size)]
                g = dist.new_group(ranks, backend=backend, timeout=timeout)
                c = dist.new_group(ranks, backend="gloo", timeout=timeout)
                if t == cfg.tp_rank:
                    self.dp_group, self.dp_cpu_group = g, c
        if cfg.tp_size > 1:
            comm.register(comm_mod.TorchCollectives(self.tp_group))
            if self.device.type == "cuda" and not ENV.DISABLE_FUSED_COMM.value:
                try:
                    from ..parallel.symm import SymmetricCollectives

                    symm = SymmetricCollectives(self.tp_group, self.cpu_group, self.device, cfg.tp_rank, cfg.tp_size)
                    comm.register(symm)
                    if not ENV.DISABLE_ROW_SHARD.value and not self.model_config.is_moe:
                        # prefill chunks: GEMM -> reduce-scatter -> add + norm -> all-gather -> GEMM
                        symm.enable_row_shard(int(getattr(cfg, "max_extend_tokens", 8192)),
                                              self.model_config.hidden_size)
                except Exception as exc:  # falls back to the NCCL data plane, loudly
                    logger.warning("symmetric-memory collectives unavailable (%s); using NCCL only", exc)

    def _configure_expert_tier(self) -> None:
        """``--expert-cache-gb G``: keep only as many experts per MoE layer on the device as fit in
        G GiB in total; the rest stay in pinned host memory (python/minisgl/server/args.py:199-249)."""
        from ..layers.moe import MoELayer

        from ..weights import ExpertGeometry, TierBudgets, resolve_plan
        from ..weights.host_capacity import check_pinned

        cfg, mc = self.config, self.model_config
        MoELayer.offload_slots = 0
        self.offload_plan = None
        if cfg.expert_cache_gb <= 0 or not mc.is_moe:
            return
        itemsize = torch.empty((), dtype=self.dtype).element_size()
        layers = sum(1 for i in range(mc.num_layers) if mc.layer_is_moe(i))
        geo = ExpertGeometry(layers, mc.num_experts, mc.num_experts_per_tok,
                             3 * mc.hidden_size * mc.moe_intermediate_size * itemsize)
        MoELayer.offload_host_experts, MoELayer.offload_disk_dir, MoELayer._tier_seq = 0, "", 0
        host_bytes = int(cfg.expert_host_gb * (1 << 30)) if cfg.expert_host_gb > 0 else None
        plan = resolve_plan(geo, TierBudgets(device_bytes=int(cfg.expert_cache_gb * (1 << 30)), host_bytes=host_bytes,
                                             disk=bool(cfg.expert_disk_dir)))
        if self.cpu_group is not None and cfg.tp_size > 1:
            # every rank must have resolved the same placement before anything is pinned
            from ..weights.plan import check_agreement

            digests = [None] * cfg.tp_size
            dist.all_gather_object(digests, plan.digest, group=self.cpu_group)
            check_agreement(digests)
        if plan.offloaded and self.device.type == "cuda":
            check_pinned(plan.host_bytes)
        self.offload_plan = plan
        MoELayer.offload_slots = plan.layers[0].device_slots if plan.offloaded else 0
        if plan.offloaded and plan.layers[0].disk_experts > 0:
            MoELayer.offload_host_experts = plan.layers[0].host_experts
            MoELayer.offload_disk_dir = os.path.join(cfg.expert_disk_dir, f"rank{cfg.tp_rank}")
        for note in plan.notes:
            logger.info_rank0("offload plan: %s", note)
        logger.info_rank0("host expert tier: %d of %d experts resident per layer (plan %s, %.2f GiB pinned)",
                          plan.layers[0].device_slots, mc.num_experts, plan.digest, plan.host_bytes / (1 << 30))

    def _free_memory(self) -> int:
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
            return torch.cuda.mem_get_info(self.device)[0]
        return 0

    def _determine_num_pages(self) -> int:
        """Pages that fit in ``memory_ratio`` of the device after the model, minus room for
        activations and graphs; the minimum over tensor-parallel ranks is used
        (python/minisgl/engine/engine.py:1828-2093)."""
        cfg, mc = self.config, self.model_config
        if cfg.num_page_override is not None:
            return int(cfg.num_page_override)
        itemsize = 1 if self.kv_fp8 else torch.empty((), dtype=self.dtype).element_size()
        per_page = MHAKVCache.token_bytes(self.kv_layers, self.kv_heads_local, mc.head_dim,
                                          itemsize) * self.page_size
        if self._main_geometry:
            per_page = MHAKVCache.token_bytes(self.kv_layers, 1, max(h * d for h, d in self._main_geometry),
                                              itemsize) * self.page_size
        if self.mla_latent:
            from ..kvcache.mla_pool import MLALatentCache

            per_page = MLALatentCache.token_bytes(self.kv_layers, int(mc.kv_lora_rank), int(mc.qk_rope_head_dim),
                                                  itemsize) * self.page_size
        if cfg.spec_algorithm in ("eagle3", "mtp"):
            # the draft head keeps one 16-bit, unsharded layer of K/V on the same page table
            per_page += MHAKVCache.token_bytes(1, mc.num_kv_heads, mc.head_dim, 2) * self.page_size
        if self.device.type != "cuda":
            return 2048
        free, total = torch.cuda.mem_get_info(self.device)
        # activation reserve: the widest intermediates of one prefill chunk
        chunk = getattr(cfg, "max_extend_tokens", 8192)
        widest = max(2 * mc.intermediate_size // cfg.tp_size, mc.q_size + 2 * mc.kv_size, mc.hidden_size * 4)
        act_reserve = chunk * widest * 2 * 4 + (2 << 30)
        budget = int(total * cfg.memory_ratio) - (total - free) - act_reserve
        if self._swa_layers:
            budget -= (self._swa_pages + 1) * self.page_size * MHAKVCache.token_bytes(
                self._swa_layers, self.kv_heads_local, mc.head_dim, itemsize)
        if mc.is_recurrent:
            from ..kvcache.gdn_state import GDNStateCache

            conv_dim, st_heads, st_rows, st_cols = mc.recurrent_geometry
            conv_dim, st_heads = conv_dim // cfg.tp_size, st_heads // cfg.tp_size
            budget -= (cfg.max_running_req + 1) * GDNStateCache.slot_bytes(
                mc.num_linear_layers, conv_dim, mc.linear_conv_kernel_dim, st_heads, st_rows, st_cols, 2)
        pages = budget // per_page
        if self.cpu_group is not None:
            t = torch.tensor([pages], dtype=torch.int64)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.cpu_group)
            pages = int(t.item())
        if pages < 16:
            raise RuntimeError(f"not enough memory for the KV cache ({pages} pages)")
        return int(pages)

    def _resolve_max_seq_len(self) -> int:
        cfg, mc = self.config, self.model_config
        limit = cfg.max_seq_len_override or mc.max_position_embeddings
        limit = min(limit, mc.rotary_config.max_position, self.num_pages * self.page_size)
        return int(limit // self.page_size * self.page_size) or self.page_size

    # ------------------------------------------------------------------ step
    def _stage(self, plan: StepPlan):
        """Pack the plan into one pinned buffer and start a single H2D copy; returns device
        views in plan order. The pinned side is a ring: with overlapped scheduling the host
        fills the plan of step n+1 while the copy of step n may still be queued behind
        kernels, so a slot is reused only after the event recorded behind its copy."""
        parts = [plan.token_idx, plan.positions, plan.out_loc, plan.cu_q, plan.seq_lens,
                 plan.block_table.reshape(-1), plan.sample_rows, plan.write_idx]
        total = sum(int(p.size) for p in parts)
        cuda = self.device.type == "cuda"
        if total > self._staging_cap:
            if cuda:
                torch.cuda.synchronize(self.device)
            self._staging_cap = max(total * 2, 1 << 16)
            self._staging_ring = [
                torch.empty(self._staging_cap, dtype=torch.int32, pin_memory=cuda) for _ in range(self._ring)]
            self._staging_dev_ring = [
                torch.empty(self._staging_cap, dtype=torch.int32, device=self.device) for _ in range(self._ring)]
            self._staging_events = [None] * self._ring
        slot = self._ring_pos % self._ring
        self._ring_pos += 1
        ev = self._staging_events[slot]
        if ev is not None:
            ev.synchronize()
        host = self._staging_ring[slot]
        host_np = host.numpy()
        off, views = 0, []
        for p in parts:
            n = int(p.size)
            host_np[off : off + n] = p.reshape(-1)
            views.append((off, n))
            off += n
        if cuda:
            dev = self._staging_dev_ring[slot]
            dev[:total].copy_(host[:total], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            self._staging_events[slot] = ev
            src = dev
        else:
            src = host.clone()
        self.h2d_bytes += 4 * total
        out = [src[o : o + n] for o, n in views]
        out[5] = out[5].view(plan.block_table.shape)
        return out

    def swa_arrays(self, token_idx: torch.Tensor, positions: torch.Tensor, cu_q: torch.Tensor, n_pages: int):
        """K/V slot of every row and block table of every request in the sliding-window pool, from the
        device copy of that pool's page table (rows of the padding request map to the dummy page)."""
        ps = self.page_size
        table = self.swa.table_dev
        row_slot = (token_idx // self.max_seq_len).long()
        pos = positions.long()
        out_loc = (table[row_slot, pos // ps].long() * ps + pos % ps).to(torch.int32)
        req_slot = row_slot[cu_q[:-1].long()]
        return out_loc, table[req_slot, :n_pages].contiguous()

    def _out_buffer(self, n: int) -> torch.Tensor:
        """Pinned landing buffer for the sampled ids of one step (ring, see ``_stage``)."""
        slot = self._out_pos % self._ring
        self._out_pos += 1
        buf = self._out_ring[slot]
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(n, 64), dtype=torch.int32, pin_memory=self.device.type == "cuda")
            self._out_ring[slot] = buf
        return buf[:n]

    def forward_batch(self, batch: Batch, plan: StepPlan, args: BatchSamplingArgs,
                      return_logits: bool = False) -> ForwardOutput:
        """Run one step: gather ids, model forward, LM head on the sampled rows, sample, write
        the new ids back into the token pool and start their device→host copy."""
        if self.stream is not None:
            with torch.cuda.stream(self.stream):
                return self._forward_impl(batch, plan, args, return_logits)
        return self._forward_impl(batch, plan, args, return_logits)

    def _forward_impl(self, batch, plan, args, return_logits) -> ForwardOutput:
        if self._spec_exact and batch.spec_verify:
            from ..ops import cuda as K

            prev = K.gemm_pair_mode(1)
            try:
                return self._forward_step(batch, plan, args, return_logits)
            finally:
                K.gemm_pair_mode(prev)
        return self._forward_step(batch, plan, args, return_logits)

    def _forward_step(self, batch, plan, args, return_logits) -> ForwardOutput:
        n_sample = int(plan.sample_rows.size)
        bs = batch.size
        use_graph = (self.graph_runner is not None and batch.is_decode and not batch.spec_verify
                     and plan.max_q == 1 and self.graph_runner.can_run(bs)
                     and batch.capture_layers is None and n_sample == bs)
        ep = self.ctx.ep
        if use_graph and ep is not None and hasattr(ep, "static_bound"):
            # the captured exchange works under the row bound of the largest bucket: a step in which
            # some replica sends more rows than that (a prefill chunk elsewhere) runs eagerly, as
            # does every step once the exchange fell back to NCCL
            common = ep.common_tokens
            use_graph = ep.healthy and common is not None and common <= self.graph_runner.max_bs
        if use_graph:
            gr = self.graph_runner
            bucket = gr.bucket_of(bs)
            if bucket != bs:
                tok, pos, loc, lens = gr.pad_plan_arrays(bs, bucket, plan.token_idx, plan.positions,
                                                         plan.out_loc, plan.seq_lens)
                bt = np.full((bucket, plan.block_table.shape[1]), self.kv_cache.dummy_page, dtype=np.int32)
                bt[:bs] = plan.block_table
                plan = StepPlan(tok, pos, loc, plan.cu_q, lens, bt, plan.sample_rows, plan.write_idx,
                                plan.max_q, plan.max_kv)
        elif self._row_shard_rows(int(plan.token_idx.size)):
            # Tensor-parallel prefill: the fused reduce-scatter / all-gather GEMMs move rows in
            # blocks of 128, so the step is padded with rows that belong to no request (dummy
            # token, dummy KV slot; attention never looks at them, nothing samples them).
            t = int(plan.token_idx.size)
            pad = (-t) % 128
            if pad:
                d_tok = np.full(pad, (self.num_slots - 1) * self.max_seq_len, dtype=np.int32)
                d_loc = np.full(pad, self.kv_cache.dummy_page * self.page_size, dtype=np.int32)
                plan = StepPlan(np.concatenate([plan.token_idx, d_tok]),
                                np.concatenate([plan.positions, np.zeros(pad, dtype=np.int32)]),
                                np.concatenate([plan.out_loc, d_loc]), plan.cu_q, plan.seq_lens, plan.block_table,
                                plan.sample_rows, plan.write_idx, plan.max_q, plan.max_kv)
        if ENV.CHECK_BOUNDS.value:
            self._check_plan_bounds(plan)
            self._bounds_steps = getattr(self, "_bounds_steps", 0) + 1
            if self._bounds_steps % 64 == 0:
                self.check_device_bounds()
        token_idx, positions, out_loc, cu_q, seq_lens, block_table, sample_rows, write_idx = self._stage(plan)
        batch.positions = positions
        batch.out_loc = out_loc
        batch.token_idx = token_idx
        batch.host_cu_q = plan.cu_q
        if self.gdn_state is not None and not use_graph:
            # state slot of every request (its row of the token pool) and whether it already has a
            # state: a request whose step starts at position 0 begins from zeros
            first = cu_q[:-1].long()
            batch.gdn_slots = (token_idx[first] // self.max_seq_len).to(torch.int32)
            batch.gdn_has_state = (positions[first] > 0).to(torch.int32)
        if self.swa is not None:
            self.swa.flush()                       # page changes noted by the scheduler, ahead of this step
            if not use_graph:
                batch.swa_out_loc, batch.swa_block_table = self.swa_arrays(token_idx, positions, cu_q,
                                                                           block_table.shape[1])
        if use_graph:
            logits = self.graph_runner.replay(bs, token_idx, positions, out_loc, seq_lens, block_table)
        else:
            batch.input_ids = self.token_pool.view(-1)[token_idx.long()]
            self.ctx.attn_backend.prepare_metadata(
                batch, block_table, cu_q, seq_lens, plan.max_q, plan.max_kv,
                causal=True, mask=batch.tree_mask, host_cu_q=plan.cu_q, host_seq_lens=plan.seq_lens,
                mask_window=batch.mask_window, mask_swa=batch.tree_mask_swa)
            with self.ctx.forward_batch(batch):
                hidden = self.model.forward(batch.input_ids)
                if n_sample == 0:
                    logits = None
                else:
                    rows = hidden if n_sample == hidden.shape[0] else hidden[sample_rows.long()]
                    logits = self.model.lm_head.forward_local(rows)
        self.steps += 1
        if n_sample == 0:
            empty = torch.empty(0, dtype=torch.int32)
            return ForwardOutput(empty.to(self.device), empty, None)
        if batch.spec_verify:
            # the verify step decides acceptance itself from the logits of every row
            empty = torch.empty(0, dtype=torch.int32)
            return ForwardOutput(empty.to(self.device), empty, None, None, self.model.lm_head.gather(logits))
        head = self.model.lm_head
        if (self.config.tp_size > 1 and args.greedy and not return_logits and args.logprobs == 0
                and args.bitmask is None and args.penalty_rows is None and not self.sampler.softcap
                and not ENV.SANITIZE_LOGITS.value):
            # plain greedy under tensor parallelism: shard arg-max + exchange of (max, index) pairs
            # instead of gathering rows x vocabulary fp32 logits on every rank
            # every rank picks the winner from the same exchanged (max, index) pairs in rank order:
            # the ids are identical by construction and need no further agreement
            sample = SampleOutput(head.argmax_from_local(logits))
            tokens = sample.tokens
        else:
            logits = head.gather(logits)
            sample = self.sampler.sample(logits, args)
            tokens = self._agree_tokens(sample.tokens)
        self.token_pool.view(-1)[write_idx.long()] = tokens
        host = self._out_buffer(n_sample)
        event = None
        if self.device.type == "cuda":
            host.copy_(tokens, non_blocking=True)
            event = torch.cuda.Event()
            event.record()
            host_out = host
        else:
            host_out = tokens.clone()
        self.d2h_bytes += 4 * n_sample
        return ForwardOutput(tokens, host_out, event, sample, logits if return_logits else None)

    def _check_plan_bounds(self, plan: StepPlan) -> None:
        """``MSGL_CHECK_BOUNDS=1``: every index a kernel will dereference is range-checked on the
        host first, so a scheduler bug shows up as an exception naming the array instead of as a
        device fault (the reference builds its kernels with bounds checks for the same purpose)."""
        pool = self.num_slots * self.max_seq_len
        slots = (self.kv_cache.dummy_page + 1) * self.page_size
        checks = [("token_idx", plan.token_idx, pool), ("write_idx", plan.write_idx, pool),
                  ("out_loc", plan.out_loc, slots), ("block_table", plan.block_table, self.kv_cache.dummy_page + 1),
                  ("sample_rows", plan.sample_rows, max(int(plan.token_idx.size), 1)),
                  ("positions", plan.positions, self.max_seq_len)]
        for name, arr, hi in checks:
            if arr.size and (int(arr.min()) < 0 or int(arr.max()) >= hi):
                raise IndexError(f"step plan: {name} outside [0, {hi}): min {int(arr.min())} max {int(arr.max())}")
        if int(plan.cu_q[-1]) > int(plan.token_idx.size) or np.any(np.diff(plan.cu_q) < 0):
            raise IndexError("step plan: cu_q is not a prefix sum within the token rows")

    def _row_shard_rows(self, tokens: int) -> bool:
        """Whether a step of ``tokens`` rows takes the row-sharded tensor-parallel path."""
        if self.config.tp_size == 1 or self.model_config.is_moe:
            return False
        for impl in comm_mod.get_comm().impls:
            rs = getattr(impl, "row_shard", None)
            if rs is not None:
                return impl.max_rows < tokens <= rs.max_rows
        return False

    def _agree_tokens(self, tokens: torch.Tensor) -> torch.Tensor:
        """All tensor-parallel ranks adopt rank 0's ids
        (python/minisgl/engine/sample.py:252-277)."""
        if self.config.tp_size == 1 or self.tp_group is None:
            return tokens
        dist.broadcast(tokens, src=self.config.dp_rank * self.config.tp_size, group=self.tp_group)
        return tokens

    def check_device_bounds(self) -> None:
        """``MSGL_CHECK_BOUNDS=1`` on a GPU: collect what the bounds-checking kernel build recorded
        (out-of-range indices that the kernels skipped) and re-read the guard zones around the
        kernels' workspaces; anything found is an error naming the source line or the workspace."""
        if self.device.type != "cuda":
            return
        from ..ops import cuda as K

        found = K.bounds_report() + [f"workspace overrun: {n}" for n in K.verify_workspaces()]
        if found:
            raise RuntimeError("device-side bounds check: " + "; ".join(found))

    def finish_kv_calibration(self, path: Optional[str] = None, margin: float = 1.0):
        """End a calibration run (``MSGL_KV_FP8_CALIBRATE=1``): per-(layer, kv head) descales from the
        recorded amax, heads of all tensor-parallel ranks put back in checkpoint order, written as the
        side-car ``kv_scales.safetensors`` that an fp8-KV engine picks up at boot
        (python/minisgl/kvcache/mha_pool.py:207-270, tools/kv_fp8_calibrate.py). Returns
        ``(k_scale, v_scale)`` with the full head count."""
        k, v = self.kv_cache.finish_calibration(margin)
        cfg = self.config
        total = self.model_config.num_kv_heads
        if cfg.tp_size > 1 and self.cpu_group is not None:
            parts: List = [None] * cfg.tp_size
            dist.all_gather_object(parts, (k, v), group=self.cpu_group)
            # with fewer kv heads than ranks a head is replicated on tp_size // total neighbouring ranks
            step = max(cfg.tp_size // total, 1)
            k = torch.cat([parts[r][0] for r in range(0, cfg.tp_size, step)], dim=1)
            v = torch.cat([parts[r][1] for r in range(0, cfg.tp_size, step)], dim=1)
        if path is None and cfg.model_path and os.path.isdir(cfg.model_path):
            path = os.path.join(cfg.model_path, "kv_scales.safetensors")
        if path is not None and cfg.tp_rank == 0:
            from safetensors.torch import save_file

            save_file({"k_scale": k.contiguous(), "v_scale": v.contiguous()}, path)
            logger.info_rank0("fp8 KV scales written to %s (k %.4g..%.4g, v %.4g..%.4g)", path, float(k.min()),
                              float(k.max()), float(v.min()), float(v.max()))
        return k, v

    def shutdown(self) -> None:
        """Release what would keep a process-group teardown waiting: captured graphs (they hold
        NCCL kernels), peer-memory mappings, then meet the other ranks at a CPU barrier."""
        import gc

        if ENV.CHECK_BOUNDS.value:
            self.check_device_bounds()
        set_global_ctx(None)
        if self.graph_runner is not None:
            self.graph_runner.graphs.clear()
            self.graph_runner.logits.clear()
            self.graph_runner = None
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        for impl in comm_mod.get_comm().impls:
            close = getattr(impl, "close", None)
            if close is not None:
                try:
                    close()
                except Exception:
                    pass
        ep = getattr(self.ctx, "ep", None)
        if ep is not None and hasattr(ep, "close"):
            try:
                ep.close()
            except Exception:
                pass
        comm_mod.reset_comm()
        gc.collect()
        if dist.is_initialized() and self.config.world_size > 1:
            try:
                dist.barrier(group=self.cpu_group if self.cpu_group is not None else self.dp_cpu_group)
            except Exception:
                pass
