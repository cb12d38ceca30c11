"""Typed environment-variable registry.

Every tunable that is read from the process environment is declared here exactly once,
with a type, a default and a one-line description. The reference reads seven variables
through a typed singleton (python/minisgl/env.py:58-87) and about 260 more through ad hoc
``os.environ`` lookups scattered over the tree; this build keeps one registry so that
``python -m minisglang_rdna4_b200 --print-env`` can list every knob.

Names use the ``MSGL_`` prefix. For drop-in use, a variable that is not set under
``MSGL_X`` is also looked up as ``MINISGL_X`` (the reference's prefix).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Generic, TypeVar

T = TypeVar("T")

_TRUE = {"1", "true", "yes", "on", "y", "t"}
_FALSE = {"0", "false", "no", "off", "n", "f", ""}


def _parse_bool(text: str) -> bool:
    low = text.strip().lower()
    if low in _TRUE:
        return True
    if low in _FALSE:
        return False
    raise ValueError(f"not a boolean: {text!r}")


def _parse_int(text: str) -> int:
    return int(text.strip(), 0)


def _parse_float(text: str) -> float:
    return float(text.strip())


def _parse_str(text: str) -> str:
    return text


@dataclass
class EnvVar(Generic[T]):
    """One declared variable. ``value`` re-reads the environment on each access so tests
    can monkeypatch ``os.environ`` without resetting a cache."""

    name: str
    default: T
    parser: Callable[[str], T]
    doc: str = ""

    def raw(self) -> str | None:
        for prefix in ("MSGL_", "MINISGL_"):
            text = os.environ.get(prefix + self.name)
            if text is not None:
                return text
        return None

    @property
    def value(self) -> T:
        text = self.raw()
        if text is None or text.strip() == "":
            # An empty string means "unset" (python/minisgl/kvcache/_envutil.py tolerates the
            # same: compose files export VAR= for knobs that are switched off).
            return self.default
        try:
            return self.parser(text)
        except ValueError as exc:  # pragma: no cover - message path
            raise ValueError(f"environment variable {self.name}: {exc}") from None

    def __bool__(self) -> bool:
        return bool(self.value)


class EnvRegistry:
    """Attribute-style access to the declared variables: ``ENV.KV_FP8.value``."""

    def __init__(self) -> None:
        self._vars: Dict[str, EnvVar[Any]] = {}

    def _add(self, var: EnvVar[Any]) -> EnvVar[Any]:
        if var.name in self._vars:
            raise KeyError(f"duplicate env declaration {var.name}")
        self._vars[var.name] = var
        setattr(self, var.name, var)
        return var

    def flag(self, name: str, default: bool = False, doc: str = "") -> EnvVar[bool]:
        return self._add(EnvVar(name, default, _parse_bool, doc))

    def int(self, name: str, default: int, doc: str = "") -> EnvVar[int]:
        return self._add(EnvVar(name, default, _parse_int, doc))

    def float(self, name: str, default: float, doc: str = "") -> EnvVar[float]:
        return self._add(EnvVar(name, default, _parse_float, doc))

    def str(self, name: str, default: str = "", doc: str = "") -> EnvVar[str]:
        return self._add(EnvVar(name, default, _parse_str, doc))

    def items(self):
        return sorted(self._vars.items())

    def describe(self) -> str:
        lines = []
        for name, var in self.items():
            lines.append(f"MSGL_{name:<28} = {var.value!r:<12} (default {var.default!r})  {var.doc}")
        return "\n".join(lines)


ENV = EnvRegistry()

# --- engine -------------------------------------------------------------------------------
ENV.flag("KV_FP8", False, "store the paged KV pool as e4m3 with per-(layer,head) scales")
ENV.flag("KV_FP8_CALIBRATE", False, "calibration run: 16-bit KV pool, eager steps, running |max| per (layer, kv head) "
         "of every stored row; Engine.finish_kv_calibration writes the kv_scales side-car")
ENV.flag("DISABLE_OVERLAP", False, "run the synchronous scheduler loop instead of the overlapped one")
ENV.flag("GEMM_SPLIT_K", False, "experimental: GEMMs with at most 256 rows split K over several SMs (measured slower than full-K tiles; breaks chunk-size invariance)")
ENV.flag("DISABLE_GRAPH", False, "never capture CUDA graphs (eager decode)")
ENV.int("GRAPH_MAX_BS", 0, "largest decode batch captured as a CUDA graph (0 = auto)")
ENV.int("EXIT_AFTER_STEPS", 0, "stop the scheduler loop after this many forward steps (0 = never)")
ENV.flag("SANITIZE_LOGITS", False, "replace NaN/Inf logits before sampling and count them")
ENV.flag("CHECK_BOUNDS", False, "validate every step's token / KV-slot / page ids on the host before they reach a "
         "kernel; on a GPU also load the bounds-checking kernel build (indices checked on the device, recorded and "
         "skipped) and put guard zones around the kernels' workspaces")
ENV.flag("DISPATCH_LEDGER", False, "log once per op which sm_100a kernel served it")
ENV.str("PROFILE", "", "path of a torch.profiler chrome trace to write around the profiled steps")
ENV.int("PROFILE_SKIP", 8, "forward steps to skip before the profiler window opens")
ENV.int("PROFILE_STEPS", 8, "forward steps inside the profiler window")
ENV.flag("HOSTPROF", False, "print a host-side stage breakdown of the scheduler loop")
ENV.flag("GRAPH_TIMING", False, "time every graph replay with CUDA events")
ENV.flag("DISABLE_SPLIT_K_DECODE", False, "decode-phase o_proj / down_proj keep K in one range instead of handing split-K planes to the next add + norm")
ENV.flag("DISABLE_TC_PREFILL", False, "prefill attention on the general (warp-level MMA) kernel instead of the tcgen05 one")
# --- distributed --------------------------------------------------------------------------
ENV.int("PYNCCL_MAX_BUFFER_SIZE", 1 << 30, "upper bound of the registered all-reduce staging buffer")
ENV.flag("DISABLE_FUSED_COMM", False, "route every collective through NCCL (the baseline data plane)")
ENV.flag("TP_OVERLAP", False, "prefill steps of MoE layers under tensor parallelism reduce their output row chunk by row chunk "
         "on a second stream, under the experts of the next chunk")
ENV.int("TP_OVERLAP_MIN_ROWS", 1024, "smallest step (rows) that takes the chunked overlap")
ENV.int("TP_OVERLAP_CHUNKS", 4, "row chunks of an overlapped step")
ENV.flag("DISABLE_ROW_SHARD", False, "prefill chunks use all-reduce instead of the fused reduce-scatter / all-gather GEMMs")
ENV.flag("PDL", True, "programmatic dependent launch: a kernel's prologue overlaps the tail of the kernel ahead of it")
ENV.int("EP_REGION_GIB", 6, "per-rank budget of the expert-parallel exchange regions (sets the largest fused step)")
ENV.str("NVLS", "auto", "decode all-reduce by in-switch reduction (multimem): auto = from 8 ranks up (measured slower than peer "
        "stores at 2 and 4 ranks), on, off")
ENV.int("SYMM_HEAP_MIB", 256, "size of the per-rank symmetric peer-memory heap")
ENV.int("ONESHOT_AR_MAX_KIB", 512, "messages up to this size use the one-shot all-reduce; larger ones go to the row-sharded GEMM fusion or to NCCL")
ENV.int("RECURRENT_SNAPSHOT_MIB", 2048, "memory for recurrent-state snapshots (prefix reuse of hybrid models); 0 = no "
        "prefix reuse for models with recurrent layers")
ENV.int("RECURRENT_SNAPSHOT_TOKENS", 512, "a running request's recurrent state is kept every this many tokens")
ENV.int("RECURRENT_SNAPSHOT_HOST_MIB", 0, "keep recurrent-state snapshots in this much page-locked host memory instead of device memory (0 = on the device)")
ENV.flag("IMAGE_BIDIRECTIONAL", True, "the placeholder tokens of one image attend to each other in both directions during the prefill (as the published Gemma-3 does); off = causal")
ENV.flag("STATE_DIGEST", False, "log exact per-layer digests of the K/V and recurrent state every prefill leaves behind (diagnostic; slow)")
ENV.str("BAKED_DIR", "", "directory of baked checkpoints: a rank's weights as they stand after loading, streamed back on later "
        "boots instead of parsing, slicing and merging the checkpoint again (written on the first boot)")
ENV.flag("BAKED_VERIFY", False, "check every baked tensor's checksum while loading")
ENV.flag("HUB_OFFLINE", False, "a model path that names a hub repository is looked up in the local hub cache only (no download)")
ENV.flag("MLA_LATENT", False, "latent-attention models keep the compressed latent and the shared rotary key per token instead of "
         "per-head keys and values (absorbed attention through tensor ops, eager steps only: a capacity mode, not a fast one)")
ENV.flag("SWA_POOL", False, "sliding-window layers keep their K/V in a pool of their own whose pages are handed back as they "
         "leave the window (long contexts cost the full-attention layers only)")
ENV.int("THINK_LOOP_PERIOD", 64, "longest repeated block (tokens) the reasoning-loop detector looks for; 0 = off")
ENV.int("THINK_LOOP_SPAN", 48, "a reasoning loop is reported once this many consecutive tokens repeat")
ENV.int("THINK_LOOP_REPS", 3, "... and the block has repeated this many times")
ENV.int("TOOLCALL_RUNAWAY_LIMIT", 8192, "tokens one open tool call may run for before the request is ended; 0 = off")
ENV.int("TOOLCALL_CONT_LIMIT", 49152, "a final assistant message that ends inside an unclosed tool-call block of at least this many characters is refused (0 = no check)")
ENV.flag("GEMM_L2_AHEAD", False, "decode-sized and grouped GEMMs request a work item's whole weight stream into L2 one "
         "item ahead (dense decode: before they wait for the kernel ahead of them; needs MSGL_PDL)")
ENV.int("COMM_HEALTH_STEPS", 8, "the tensor-parallel ranks agree on the collectives' status word every this many steps")
ENV.int("COMM_WAIT_US", 500_000, "bound of every device-side flag wait, in microseconds")
# --- speculative decode -------------------------------------------------------------------
ENV.flag("SPEC_SAMPLED", False, "verify drafts by rejection sampling instead of greedy prefix match")
ENV.int("SPEC_MAX_BS", 0, "largest batch that still runs a speculative step (0 = per-algorithm default)")
ENV.flag("SPEC_HOST_STEP", False, "run the speculative step through the host-driven path even on a GPU")
ENV.flag("SPEC_ADAPTIVE_WIDTH", True, "choose the verify width from the running acceptance rate")
# --- quantization -------------------------------------------------------------------------
ENV.flag("MOE_W4A16", False, "run int4/fp4 expert weights against 16-bit activations")
ENV.flag("FORCE_BF16_DEQUANT", False, "dequantise quantised checkpoints to bf16 at load (debug)")
# --- server -------------------------------------------------------------------------------
ENV.flag("METRICS", True, "collect Prometheus metrics")
ENV.int("DEFAULT_MAX_TOKENS", 1024, "max_tokens applied to a request that gives none")
ENV.str("SHELL_SYSTEM_PROMPT", "", "system prompt of the interactive shell")
ENV.flag("LOG_REQUESTS", False, "log one line per admitted and finished request")
ENV.str("CHAT_TEMPLATE", "", "chat template of the served model: a file path or a literal Jinja string")
ENV.str("CHAT_TEMPLATE_MODEL", "", "model path the CHAT_TEMPLATE override applies to")
# --- measurement --------------------------------------------------------------------------
ENV.flag("GHOST_ORACLE", False, "count what an unbounded prefix cache would have reused (measure-only)")
ENV.str("GHOST_ORACLE_DIR", "", "directory where the prefix-reuse oracle keeps its state across restarts")


def env_int(name: str, default: int) -> int:
    """Read an undeclared integer knob, treating an empty string as unset."""
    for prefix in ("MSGL_", "MINISGL_"):
        text = os.environ.get(prefix + name)
        if text is not None and text.strip() != "":
            return int(text, 0)
    return default


__all__ = ["ENV", "EnvVar", "EnvRegistry", "env_int"]
