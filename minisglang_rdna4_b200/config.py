"""Typed configuration tree: ``EngineConfig`` ⊂ ``SchedulerConfig`` ⊂ ``ServerArgs``.

Field names and defaults follow the reference's public surface
(python/minisgl/engine/config.py:136-283, python/minisgl/scheduler/config.py:14-57,
python/minisgl/server/args.py:85-542) so that a launch line written for it keeps working.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field, replace
from typing import Any, Dict, Optional

from .models.config import ModelConfig


@dataclass(frozen=True)
class EngineConfig:
    model_path: str = ""
    dtype: str = "auto"                      # auto | fp16 | bf16 | fp32
    tp_size: int = 1
    tp_rank: int = 0
    dp_size: int = 1
    dp_rank: int = 0
    enable_ep: bool = False
    max_running_req: int = 256
    max_seq_len_override: Optional[int] = None
    distributed_timeout: float = 60.0
    memory_ratio: float = 0.9
    use_dummy_weight: bool = False
    use_pynccl: bool = True
    cuda_graph_max_bs: Optional[int] = None
    num_page_override: Optional[int] = None
    page_size: int = 16
    attention_backend: str = "auto"          # accepted for compatibility; there is one backend
    moe_backend: str = "auto"
    model_source: str = "huggingface"
    cache_type: str = "radix"                # radix | naive
    kv_cache_dtype: str = "auto"             # auto | bf16 | fp8
    quantization: Optional[str] = None       # force a scheme for dummy weights: mxfp4|nvfp4|fp8|fp8_block|int4
    device: str = "auto"                     # auto | cuda | cpu
    seed: int = 0
    # speculative decode
    spec_algorithm: str = "none"             # none | ngram | eagle3 | mtp | dflash | tidar
    spec_draft_model_path: Optional[str] = None
    spec_num_draft: int = 4
    spec_ngram_max: int = 3
    spec_ngram_min: int = 1
    spec_tree_width: int = 1
    # block-diffusion models: entries that override the checkpoint's generation_config.json schedule
    diffusion_overrides: Optional[dict] = None
    # expert offload tiers
    weight_offload_gb: float = 0.0
    expert_cache_gb: float = 0.0
    expert_host_gb: float = 0.0       # pinned host budget of the expert tier (0 = every expert pinned)
    expert_disk_dir: str = ""         # flat expert files for what the pinned budget cannot hold
    # when set, overrides the config read from model_path (named shapes, tests)
    model_config: Optional[ModelConfig] = None
    base_port: int = 2333

    @property
    def world_size(self) -> int:
        return self.tp_size * self.dp_size

    @property
    def global_rank(self) -> int:
        return self.dp_rank * self.tp_size + self.tp_rank

    @property
    def device_id(self) -> int:
        return self.dp_rank * self.tp_size + self.tp_rank

    @property
    def distributed_addr(self) -> str:
        """Rendezvous of one replica's TP group (python/minisgl/engine/config.py:279-283)."""
        return f"tcp://127.0.0.1:{self.base_port + self.dp_rank}"

    @property
    def world_addr(self) -> str:
        return f"tcp://127.0.0.1:{self.base_port + 64}"

    def resolve_device(self) -> str:
        if self.device != "auto":
            return self.device
        import torch

        return "cuda" if torch.cuda.is_available() else "cpu"


@dataclass(frozen=True)
class SchedulerConfig(EngineConfig):
    max_extend_tokens: int = 8192
    offline_mode: bool = False
    disable_overlap: bool = False
    _unique: str = ""

    def _suffix(self) -> str:
        uniq = self._unique or f"pid={os.getpid()}"
        return f".{uniq}" + (f".dp={self.dp_rank}" if self.dp_size > 1 else "")

    # ZMQ endpoints (python/minisgl/scheduler/config.py:28-49)
    @property
    def zmq_backend_addr(self) -> str:      # tokenizer -> scheduler rank 0 of this replica
        return f"ipc:///tmp/msgl_0{self._suffix()}"

    @property
    def zmq_detokenizer_addr(self) -> str:  # scheduler -> detokenizer
        uniq = self._unique or f"pid={os.getpid()}"
        return f"ipc:///tmp/msgl_1.{uniq}"

    @property
    def zmq_scheduler_broadcast_addr(self) -> str:  # rank 0 -> other TP ranks
        return f"ipc:///tmp/msgl_2{self._suffix()}"

    @property
    def backend_create_detokenizer_link(self) -> bool:
        return self.tp_rank == 0


@dataclass(frozen=True)
class ServerArgs(SchedulerConfig):
    host: str = "127.0.0.1"
    port: int = 1919
    served_model_name: Optional[str] = None
    num_tokenizer: int = 0
    shell_mode: bool = False
    chat_template: Optional[str] = None
    chat_template_kwargs: Optional[Dict[str, Any]] = None
    reasoning_parser: str = "auto"
    # recursive self-aggregation defaults (rsa.RSAParams) of requests that ask for it with ``rsa: true``,
    # and whether ``reasoning_effort`` alone switches it on through the effort ladder
    rsa: Optional[Any] = None
    rsa_effort_ladder: bool = False

    @property
    def zmq_frontend_addr(self) -> str:     # detokenizer -> frontend
        uniq = self._unique or f"pid={os.getpid()}"
        return f"ipc:///tmp/msgl_3.{uniq}"

    @property
    def zmq_tokenizer_addr(self) -> str:    # frontend -> tokenizer
        uniq = self._unique or f"pid={os.getpid()}"
        return f"ipc:///tmp/msgl_4.{uniq}"

    def backend_addr_of(self, dp_rank: int) -> str:
        return replace(self, dp_rank=dp_rank).zmq_backend_addr

    @property
    def share_tokenizer(self) -> bool:
        return self.num_tokenizer == 0

    @property
    def model_name(self) -> str:
        return self.served_model_name or os.path.basename(self.model_path.rstrip("/")) or "model"
