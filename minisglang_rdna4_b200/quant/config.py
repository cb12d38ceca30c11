"""Quantisation scheme description parsed from a checkpoint's ``quantization_config``.

Accepted producers: AWQ, GPTQ, compressed-tensors (int4 pack-quantized, MXFP4, NVFP4, fp8
per-channel, fp8 block), ModelOpt and Quark; ModelOpt and Quark descriptions are rewritten to
the compressed-tensors vocabulary first. Mirrors the decision table of
python/minisgl/quant/config.py:52-143 (ModelOpt), :228-290 (Quark), :294-622 (from_hf).
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field, replace
from typing import Any, Dict, List, Optional, Tuple

# Canonical scheme names (what the linear methods dispatch on)
SCHEME_NONE = "none"
SCHEME_INT4 = "int4"            # group-wise int4 weights, optional zero point (AWQ/GPTQ/CT)
SCHEME_MXFP4 = "mxfp4"          # e2m1 weights, UE8M0 scale per 32
SCHEME_NVFP4 = "nvfp4"          # e2m1 weights, e4m3 scale per 16, fp32 global scale
SCHEME_FP8_CHANNEL = "fp8_channel"  # e4m3 weights, one scale per output channel, W8A8
SCHEME_FP8_BLOCK = "fp8_block"      # e4m3 weights, 128x128 weight blocks, 1x128 act groups
SCHEME_FP8_TENSOR = "fp8_tensor"    # e4m3 weights, one scale per tensor


@dataclass(frozen=True)
class QuantScheme:
    name: str = SCHEME_NONE
    bits: int = 16
    group_size: int = 0
    symmetric: bool = True
    # tensor-naming dialect of the checkpoint: awq | gptq | ct
    fmt: str = "ct"
    block: Tuple[int, int] = (0, 0)
    act_dynamic: bool = True
    global_scale_divides: bool = False  # CT NVFP4 stores 448*6/amax (divide); ModelOpt stores amax/(448*6)

    @property
    def quantized(self) -> bool:
        return self.name != SCHEME_NONE


@dataclass(frozen=True)
class QuantConfig:
    method: str                                   # producer string as found in the checkpoint
    default: QuantScheme
    ignore: Tuple[str, ...] = ()
    # (targets, scheme) for mixed precision; targets are regex ("re:...") or substrings
    groups: Tuple[Tuple[Tuple[str, ...], QuantScheme], ...] = ()
    kv_cache_fp8: bool = False

    # ---- per-module lookup ----
    def for_module(self, name: str) -> QuantScheme:
        """Scheme that applies to the linear module called ``name``
        (python/minisgl/quant/config.py:446-483)."""
        if _matches_any(name, self.ignore):
            return QuantScheme()
        for targets, scheme in self.groups:
            if _matches_any(name, targets, class_name="Linear"):
                return scheme
        if self.groups:
            # explicit groups but none matched: unquantised
            only_generic = all(t == ("Linear",) for t, _ in self.groups)
            return self.default if only_generic else QuantScheme()
        return self.default

    # ---- parsing ----
    @staticmethod
    def from_hf(qc: Optional[Dict[str, Any]]) -> Optional["QuantConfig"]:
        if not qc:
            return None
        method = str(qc.get("quant_method", "")).lower()
        if method in ("modelopt", "modelopt_fp8", "modelopt_fp4") or "quant_algo" in qc or "quantization" in qc:
            qc = _rewrite_modelopt(qc)
            method = "compressed-tensors"
            producer = "modelopt"
        elif method == "quark":
            qc = _rewrite_quark(qc)
            method = "compressed-tensors"
            producer = "quark"
        else:
            producer = method
        if method == "awq":
            bits = int(qc.get("bits", qc.get("w_bit", 4)))
            if bits != 4:
                raise ValueError(f"AWQ with {bits} bits is not supported")
            scheme = QuantScheme(
                SCHEME_INT4, 4, int(qc.get("group_size", qc.get("q_group_size", 128))),
                symmetric=not bool(qc.get("zero_point", True)), fmt="awq",
            )
            ignore = tuple(qc.get("modules_to_not_convert") or ())
            return QuantConfig(producer, scheme, ignore)
        if method == "gptq":
            if qc.get("desc_act"):
                raise ValueError("GPTQ checkpoints with desc_act=true are not supported")
            bits = int(qc.get("bits", 4))
            if bits != 4:
                raise ValueError(f"GPTQ with {bits} bits is not supported")
            scheme = QuantScheme(
                SCHEME_INT4, 4, int(qc.get("group_size", 128)), symmetric=bool(qc.get("sym", True)), fmt="gptq"
            )
            return QuantConfig(producer, scheme, tuple(qc.get("modules_to_not_convert") or ()))
        if method in ("compressed-tensors", "compressed_tensors"):
            return _from_compressed_tensors(qc, producer)
        if method == "fp8":
            block = qc.get("weight_block_size")
            if block:
                scheme = QuantScheme(SCHEME_FP8_BLOCK, 8, 0, fmt="ct", block=(int(block[0]), int(block[1])))
            else:
                scheme = QuantScheme(SCHEME_FP8_TENSOR, 8, 0, fmt="ct")
            return QuantConfig(producer, scheme, tuple(qc.get("modules_to_not_convert") or ()))
        if method == "mxfp4":
            return QuantConfig(producer, QuantScheme(SCHEME_MXFP4, 4, 32, fmt="ct"),
                               tuple(qc.get("modules_to_not_convert") or ()))
        raise ValueError(f"unsupported quantization method {method!r}")


def _matches_any(name: str, patterns, class_name: Optional[str] = None) -> bool:
    for pat in patterns:
        if pat.startswith("re:"):
            if re.match(pat[3:], name):
                return True
        elif class_name is not None and pat == class_name:
            return True
        elif pat == name or name.endswith("." + pat) or pat in name:
            return True
    return False


def _scheme_from_ct_group(group: Dict[str, Any], fmt_hint: Optional[str]) -> QuantScheme:
    w = group.get("weights") or {}
    a = group.get("input_activations") or {}
    fmt = (group.get("format") or fmt_hint or "").lower()
    bits = int(w.get("num_bits", 16))
    wtype = str(w.get("type", "int")).lower()
    strategy = str(w.get("strategy", "channel")).lower()
    gsz = int(w.get("group_size") or 0)
    sym = bool(w.get("symmetric", True))
    dyn = bool(a.get("dynamic", True)) if a else True
    if wtype == "float" and bits == 4:
        if "mxfp4" in fmt or gsz == 32 or str(w.get("scale_dtype", "")).lower() in ("uint8", "e8m0"):
            return QuantScheme(SCHEME_MXFP4, 4, gsz or 32, fmt="ct", act_dynamic=dyn)
        return QuantScheme(SCHEME_NVFP4, 4, gsz or 16, fmt="ct", act_dynamic=dyn,
                           global_scale_divides=not bool(group.get("_modelopt", False)))
    if wtype == "float" and bits == 8:
        if strategy == "block":
            bs = w.get("block_structure") or [128, 128]
            if isinstance(bs, str):
                bs = [int(x) for x in bs.lower().split("x")]
            return QuantScheme(SCHEME_FP8_BLOCK, 8, 0, fmt="ct", block=(int(bs[0]), int(bs[1])), act_dynamic=dyn)
        if strategy == "tensor":
            return QuantScheme(SCHEME_FP8_TENSOR, 8, 0, fmt="ct", act_dynamic=dyn)
        return QuantScheme(SCHEME_FP8_CHANNEL, 8, 0, fmt="ct", act_dynamic=dyn)
    if wtype == "int" and bits == 4:
        return QuantScheme(SCHEME_INT4, 4, gsz or 32, symmetric=sym, fmt="ct", act_dynamic=dyn)
    if bits >= 16:
        return QuantScheme()
    raise ValueError(f"unsupported compressed-tensors weights: type={wtype} bits={bits} strategy={strategy}")


def _from_compressed_tensors(qc: Dict[str, Any], producer: str) -> QuantConfig:
    fmt = qc.get("format")
    groups_raw = qc.get("config_groups") or {}
    groups: List[Tuple[Tuple[str, ...], QuantScheme]] = []
    for _, group in sorted(groups_raw.items()):
        scheme = _scheme_from_ct_group(group, fmt)
        targets = tuple(group.get("targets") or ("Linear",))
        groups.append((targets, scheme))
    if not groups:
        raise ValueError("compressed-tensors config has no config_groups")
    default = groups[0][1]
    kv = qc.get("kv_cache_scheme") or {}
    kv_fp8 = bool(kv) and int(kv.get("num_bits", 16)) == 8
    ignore = tuple(qc.get("ignore") or ())
    if len(groups) == 1 and groups[0][0] == ("Linear",):
        return QuantConfig(producer, default, ignore, (), kv_fp8)
    return QuantConfig(producer, default, ignore, tuple(groups), kv_fp8)


def _rewrite_modelopt(qc: Dict[str, Any]) -> Dict[str, Any]:
    """ModelOpt ``hf_quant_config`` → compressed-tensors vocabulary."""
    q = qc.get("quantization", qc)
    algo = str(q.get("quant_algo", "")).upper()
    ignore = list(q.get("exclude_modules") or q.get("ignore") or [])
    ignore = [("re:" + i.replace(".", r"\.").replace("*", ".*")) if "*" in i else i for i in ignore]
    kv_algo = str(q.get("kv_cache_quant_algo") or "").upper()
    out: Dict[str, Any] = {"quant_method": "compressed-tensors", "ignore": ignore}
    if kv_algo.startswith("FP8"):
        out["kv_cache_scheme"] = {"num_bits": 8, "type": "float"}
    if algo in ("NVFP4", "NVFP4_AWQ"):
        group = {"weights": {"num_bits": 4, "type": "float", "group_size": int(q.get("group_size", 16)),
                             "strategy": "tensor_group"},
                 "input_activations": {"num_bits": 4, "type": "float", "dynamic": False},
                 "format": "nvfp4-pack-quantized", "targets": ["Linear"], "_modelopt": True}
    elif algo in ("FP8", "FP8_PER_TENSOR"):
        group = {"weights": {"num_bits": 8, "type": "float", "strategy": "tensor"},
                 "input_activations": {"num_bits": 8, "type": "float", "dynamic": False},
                 "format": "float-quantized", "targets": ["Linear"]}
    elif algo == "FP8_PER_CHANNEL_PER_TOKEN":
        group = {"weights": {"num_bits": 8, "type": "float", "strategy": "channel"},
                 "input_activations": {"num_bits": 8, "type": "float", "dynamic": True, "strategy": "token"},
                 "format": "float-quantized", "targets": ["Linear"]}
    elif algo in ("FP8_PB_WO", "FP8_BLOCK"):
        group = {"weights": {"num_bits": 8, "type": "float", "strategy": "block", "block_structure": [128, 128]},
                 "format": "float-quantized", "targets": ["Linear"]}
    else:
        raise ValueError(f"unsupported ModelOpt quant_algo {algo!r}")
    out["config_groups"] = {"group_0": group}
    out["format"] = group["format"]
    return out


def _rewrite_quark(qc: Dict[str, Any]) -> Dict[str, Any]:
    """AMD Quark export → compressed-tensors vocabulary (fp4+e8m0 → MXFP4, fp4+e4m3 → NVFP4,
    fp8_e4m3 → float-quantized)."""
    g = qc.get("global_quant_config") or {}
    w = g.get("weight") or {}
    if isinstance(w, list):
        w = w[0]
    dtype = str(w.get("dtype", "")).lower()
    scale = str(w.get("scale_format", w.get("scale_type", ""))).lower()
    gsz = int(w.get("group_size") or 0)
    export = qc.get("export") or {}
    pack = str(export.get("pack_method", "reorder")).lower()
    if pack != "reorder":
        raise ValueError(f"unsupported Quark pack_method {pack!r}")
    ignore = list(qc.get("exclude") or [])
    ignore = [("re:" + i.replace(".", r"\.").replace("*", ".*")) if "*" in i else i for i in ignore]
    if dtype in ("fp4", "mxfp4", "float4") and ("e8m0" in scale or gsz == 32):
        group = {"weights": {"num_bits": 4, "type": "float", "group_size": gsz or 32, "scale_dtype": "e8m0"},
                 "format": "mxfp4-pack-quantized", "targets": ["Linear"]}
    elif dtype in ("fp4", "float4"):
        group = {"weights": {"num_bits": 4, "type": "float", "group_size": gsz or 16},
                 "format": "nvfp4-pack-quantized", "targets": ["Linear"], "_modelopt": True}
    elif dtype in ("fp8_e4m3", "fp8", "float8_e4m3fn"):
        qs = str(w.get("qscheme", "per_channel")).lower()
        group = {"weights": {"num_bits": 8, "type": "float",
                             "strategy": "tensor" if "tensor" in qs else "channel"},
                 "format": "float-quantized", "targets": ["Linear"]}
    else:
        raise ValueError(f"unsupported Quark weight dtype {dtype!r}")
    out = {"quant_method": "compressed-tensors", "ignore": ignore,
           "config_groups": {"group_0": group}, "format": group["format"]}
    kv = g.get("kv_cache") or qc.get("kv_cache_quant_config")
    if kv:
        out["kv_cache_scheme"] = {"num_bits": 8, "type": "float"}
    return out
