"""Streaming safetensors loader.

Reads ``*.safetensors`` shard by shard and fills the model's parameters directly, applying on
the fly what the reference's generic loader applies (python/minisgl/models/weight.py:3077-3218):

* tensor-parallel sharding: q/k/v/gate/up along the output dimension, o/down along the input
  dimension (the packed dimension of AWQ/GPTQ tensors follows the same logical dimension);
  KV heads are replicated when there are fewer of them than ranks; embedding and LM-head rows
  are sharded as ``ceil(V / tp)``;
* merges: ``q_proj, k_proj, v_proj → qkv_proj`` and ``gate_proj, up_proj → gate_up_proj``;
* expert stacking ``…experts.<i>.<proj> → w13 / w2`` with the expert-parallel filter;
* dropped tensors: vision towers, multi-token-prediction layers beyond ``num_layers``,
  ``g_idx``, rotary ``inv_freq`` buffers.

Quantised expert tensors (fp8 block / channel) are expanded to 16-bit while stacking.
"""
from __future__ import annotations

import glob
import json
import os
import re
from typing import Dict, Iterator, List, Optional, Tuple

import torch

from ..layers.linear import (
    MergedColumnParallelLinear, QKVParallelLinear, RowParallelLinear, _LinearBase,
)
from ..layers.embedding import ParallelLMHead, VocabParallelEmbedding
from ..layers.moe import MoELayer
from ..parallel.info import ep_enabled, get_ep_info, get_tp_info
from ..utils import init_logger
from .config import ModelConfig

logger = init_logger(__name__)

_DROP = re.compile(r"(rotary_emb\.inv_freq|\.g_idx$|^visual\.|vision_tower|vision_model|multi_modal_projector)")
_QKV = {"q_proj": 0, "k_proj": 1, "v_proj": 2}
_GATE_UP = {"gate_proj": 0, "up_proj": 1}
_EXPERT = re.compile(r"^(.*\.mlp)\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.(.+)$")


def iter_safetensors(path: str) -> Iterator[Tuple[str, torch.Tensor]]:
    from safetensors import safe_open

    files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no .safetensors files under {path}")
    for fname in files:
        if os.path.basename(fname).startswith("kv_scales"):
            continue
        with safe_open(fname, framework="pt", device="cpu") as fh:
            for name in fh.keys():
                yield name, fh.get_tensor(name)


def _slice(t: torch.Tensor, dim: int, index: int, parts: int) -> torch.Tensor:
    size = t.shape[dim]
    if size % parts != 0:
        raise ValueError(f"cannot split dimension {dim} of size {size} into {parts} shards")
    step = size // parts
    return t.narrow(dim, index * step, step)


class _Collector:
    """Accumulates the pieces of one merged / stacked parameter until it is complete."""

    def __init__(self, n_parts: int) -> None:
        self.parts: Dict[int, torch.Tensor] = {}
        self.n = n_parts

    def add(self, idx: int, t: torch.Tensor) -> bool:
        self.parts[idx] = t
        return len(self.parts) == self.n

    def cat(self, dim: int) -> torch.Tensor:
        return torch.cat([self.parts[i] for i in range(self.n)], dim=dim)


def load_weights(model, path: str, cfg: ModelConfig, device, tensors: Optional[Iterator] = None) -> None:
    tp = get_tp_info()
    ep = get_ep_info() if ep_enabled() else None
    modules: Dict[str, object] = {}

    def walk(obj, prefix: str) -> None:
        modules[prefix.rstrip(".")] = obj
        for cname, child in obj._children():
            walk(child, prefix + cname + ".")

    walk(model, "")
    pending: Dict[str, _Collector] = {}
    expert_buf: Dict[Tuple[str, int, str], Dict[str, torch.Tensor]] = {}
    loaded = set()

    def assign(owner, attr: str, value: torch.Tensor, full_name: str) -> None:
        cur = getattr(owner, attr)
        if tuple(cur.shape) != tuple(value.shape):
            raise ValueError(f"{full_name}: checkpoint shape {tuple(value.shape)} != model {tuple(cur.shape)}")
        setattr(owner, attr, value.to(device=device, dtype=cur.dtype).contiguous())
        loaded.add(full_name)

    def shard_linear(mod: _LinearBase, suffix: str, t: torch.Tensor, which: str, part: Optional[int]) -> torch.Tensor:
        dims = mod._method.shard_dims().get(suffix)
        if suffix == "bias":
            dims = (0, -1)
        if dims is None:
            return t
        n_dim, k_dim = dims
        if which == "col":
            if n_dim < 0 or t.dim() <= n_dim or t.shape[n_dim] == 1:
                return t
            if isinstance(mod, QKVParallelLinear) and part in (1, 2) and cfg.num_kv_heads < tp.size:
                group = tp.size // cfg.num_kv_heads
                return _slice(t, n_dim, tp.rank // group, cfg.num_kv_heads)
            return _slice(t, n_dim, tp.rank, tp.size)
        if which == "row":
            if k_dim < 0 or t.dim() <= k_dim or t.shape[k_dim] == 1:
                return t
            return _slice(t, k_dim, tp.rank, tp.size)
        return t

    def shard_segments(t: torch.Tensor, sizes) -> torch.Tensor:
        """Rows of ``t`` are consecutive segments of ``sizes`` rows (q | k | v ..., one per head group);
        this rank's equal share of every segment, concatenated in the same order."""
        if tp.size == 1:
            return t
        parts, off = [], 0
        for n in sizes:
            per = n // tp.size
            parts.append(t[off + tp.rank * per: off + (tp.rank + 1) * per])
            off += n
        return torch.cat(parts)

    def vocab_shard(t: torch.Tensor, per_rank: int) -> torch.Tensor:
        start = tp.rank * per_rank
        rows = t[start : start + per_rank]
        if rows.shape[0] < per_rank:
            pad = torch.zeros((per_rank - rows.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype)
            rows = torch.cat([rows, pad])
        return rows

    stream = tensors if tensors is not None else iter_safetensors(path)
    for name, tensor in stream:
        if _DROP.search(name):
            continue
        if ".block_sparse_moe." in name:
            # Mixtral: experts under block_sparse_moe with w1 / w3 / w2 for gate / up / down
            name = name.replace(".block_sparse_moe.", ".mlp.")
            for short, full in ((".w1.", ".gate_proj."), (".w3.", ".up_proj."), (".w2.", ".down_proj.")):
                name = name.replace(short, full)
        # the text decoder of a multimodal checkpoint: language_model.model.*, model.language_model.* or
        # model.language_model.model.* depending on the exporting version
        for lead in ("model.language_model.", "language_model."):
            if name.startswith(lead):
                rest = name[len(lead):]
                name = rest if rest.startswith(("model.", "lm_head.")) else "model." + rest
                break
        if name.startswith("model.visual."):
            continue
        # block-diffusion Gemma: encoder and decoder share every weight and the checkpoint keeps the decoder's
        # names; the encoder side only has loose copies of the layer scalars
        if name.startswith("model.encoder."):
            continue
        if name.startswith("model.decoder."):
            name = "model." + name[len("model.decoder."):]
        # ---- Nemotron-H (Mamba-2 hybrid): backbone.* names, one "mixer" per layer
        if cfg.model_type == "nemotron_h":
            if name.startswith("backbone."):
                name = "model." + name[len("backbone."):]
            name = {"model.embeddings.weight": "model.embed_tokens.weight", "model.norm_f.weight": "model.norm.weight"
                    }.get(name, name)
            if ".mixer." in name:
                block, _, tail = name.partition(".mixer.")
                mixer = modules.get(block + ".mixer")
                if mixer is None:
                    continue
                m_inter = cfg.mamba_num_heads * cfg.mamba_head_dim
                m_gn = cfg.mamba_n_groups * cfg.ssm_state_size
                if tail == "conv1d.weight":
                    assign(mixer, "conv1d_weight",
                           shard_segments(tensor.reshape(tensor.shape[0], -1), [m_inter, m_gn, m_gn]),
                           block + ".mixer.conv1d_weight")
                    continue
                if tail == "conv1d.bias":
                    assign(mixer, "conv1d_bias", shard_segments(tensor, [m_inter, m_gn, m_gn]),
                           block + ".mixer.conv1d_bias")
                    continue
                if tail == "norm.weight":
                    assign(mixer, "norm_weight", shard_segments(tensor, [m_inter]), block + ".mixer.norm_weight")
                    continue
                if tail in ("dt_bias", "A_log", "D"):
                    assign(mixer, tail, shard_segments(tensor.float(), [cfg.mamba_num_heads]), block + ".mixer." + tail)
                    continue
                if tail in ("in_proj.weight", "in_proj.bias") and hasattr(mixer, "in_proj"):
                    tensor = shard_segments(tensor, [m_inter, m_inter, m_gn, m_gn, cfg.mamba_num_heads])
                    rows = getattr(mixer.in_proj, tail.split(".")[1]).shape[0]
                    if tensor.shape[0] < rows:      # the projection is padded to a multiple of 8 output columns
                        pad = torch.zeros((rows - tensor.shape[0],) + tuple(tensor.shape[1:]), dtype=tensor.dtype)
                        tensor = torch.cat([tensor, pad])
                    assign(mixer.in_proj, tail.split(".")[1], tensor, block + ".mixer." + tail)
                    continue
                if tail in ("experts.up_proj", "experts.down_proj") and tensor.dim() == 3:
                    moe = mixer.experts
                    t3 = tensor[moe._e_start:moe._e_start + moe._e_local]
                    if moe._ep is None and tp.size > 1:       # intermediate dimension split over the ranks
                        t3 = _slice(t3, 1 if tail.endswith("up_proj") else 2, tp.rank, tp.size)
                    assign(moe, "w13" if tail.endswith("up_proj") else "w2", t3,
                           block + ".mixer.experts." + ("w13" if tail.endswith("up_proj") else "w2"))
                    continue
                if tail == "gate.weight" and hasattr(mixer, "experts"):
                    assign(mixer.experts.gate, "weight", tensor, block + ".mixer.experts.gate.weight")
                    continue
                if tail == "gate.e_score_correction_bias" and hasattr(mixer, "experts"):
                    assign(mixer.experts, "e_score_correction_bias", tensor.float(),
                           block + ".mixer.experts.e_score_correction_bias")
                    continue
        # ---- gated delta net (Qwen3.5 / Qwen3-Next linear-attention layers)
        if ".linear_attn." in name:
            block, _, tail = name.partition(".linear_attn.")
            gdn = modules.get(block + ".linear_attn")
            if gdn is None:
                continue
            if tail in ("in_proj_qkvz.weight", "in_proj_ba.weight"):
                # Qwen3-Next stores the projections grouped per key head: [q ‖ k ‖ v of its value heads ‖ z of
                # them] and [b ‖ a of its value heads]; regroup into the per-kind blocks the layer uses
                hk_, dk_, dv_ = cfg.linear_num_key_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
                r_ = cfg.linear_num_value_heads // hk_
                w = tensor.view(hk_, -1, tensor.shape[-1])
                if tail == "in_proj_qkvz.weight":
                    q_, k_, v_, z_ = w.split([dk_, dk_, r_ * dv_, r_ * dv_], dim=1)
                    flat = lambda t_: t_.reshape(-1, tensor.shape[-1])          # noqa: E731
                    pieces = {0: torch.cat([flat(q_), flat(k_), flat(v_)]), 1: flat(z_)}
                else:
                    b_, a_ = w.split([r_, r_], dim=1)
                    pieces = {2: b_.reshape(-1, tensor.shape[-1]), 3: a_.reshape(-1, tensor.shape[-1])}
            elif tail in ("in_proj_qkv.weight", "in_proj_z.weight", "in_proj_b.weight", "in_proj_a.weight"):
                pieces = {("in_proj_qkv.weight", "in_proj_z.weight", "in_proj_b.weight", "in_proj_a.weight").index(tail):
                          tensor}
            else:
                pieces = None
            if pieces is not None:
                key = block + ".linear_attn.in_proj.weight"
                qk, vv, hv = cfg.linear_num_key_heads * cfg.linear_key_head_dim, \
                    cfg.linear_num_value_heads * cfg.linear_value_head_dim, cfg.linear_num_value_heads
                for part, piece in pieces.items():
                    piece = shard_segments(piece.contiguous(), ([qk, qk, vv], [vv], [hv], [hv])[part])
                    col = pending.setdefault(key, _Collector(4))
                    if col.add(part, piece):
                        w = col.cat(0)
                        rows = gdn.in_proj.weight.shape[0]
                        if w.shape[0] < rows:   # the projection is padded to a multiple of 8 output columns
                            w = torch.cat([w, w.new_zeros((rows - w.shape[0], w.shape[1]))])
                        assign(gdn.in_proj, "weight", w, key)
                        del pending[key]
            elif tail == "conv1d.weight":
                qk = cfg.linear_num_key_heads * cfg.linear_key_head_dim
                vv = cfg.linear_num_value_heads * cfg.linear_value_head_dim
                assign(gdn, "conv1d_weight", shard_segments(tensor.reshape(tensor.shape[0], -1), [qk, qk, vv]),
                       block + ".linear_attn.conv1d_weight")
            elif tail == "norm.weight":
                assign(gdn, "norm_weight", tensor, block + ".linear_attn.norm_weight")
            elif tail in ("dt_bias", "A_log"):
                assign(gdn, tail, shard_segments(tensor.float(), [cfg.linear_num_value_heads]),
                       block + ".linear_attn." + tail)
            elif tail == "out_proj.weight":
                assign(gdn.out_proj, "weight", shard_linear(gdn.out_proj, "weight", tensor, "row", None), name)
            continue
        if cfg.attn_output_gate and name.endswith(".self_attn.q_proj.weight"):
            # rows are [q_h ‖ gate_h] per head: the query half joins the merged q/k/v projection, the
            # gate half becomes a projection of its own
            attn = modules.get(name[: -len(".q_proj.weight")])
            d = cfg.head_dim
            t4 = tensor.view(cfg.num_qo_heads, 2, d, tensor.shape[-1])
            gate = t4[:, 1].reshape(cfg.num_qo_heads * d, -1)
            tensor = t4[:, 0].reshape(cfg.num_qo_heads * d, -1).contiguous()
            if attn is not None and hasattr(attn, "gate_proj"):
                assign(attn.gate_proj, "weight", shard_linear(attn.gate_proj, "weight", gate, "col", None),
                       name[: -len(".q_proj.weight")] + ".gate_proj.weight")
        m = re.match(r"^model\.layers\.(\d+)\.", name)
        if m and int(m.group(1)) >= cfg.num_layers:
            continue  # MTP / next-n layers stored after the decoder
        if name.startswith("mtp."):
            continue
        # ---- experts
        em = _EXPERT.match(name)
        if em:
            block, eidx, proj, suffix = em.group(1), int(em.group(2)), em.group(3), em.group(4)
            moe: MoELayer = modules.get(block + ".experts")  # type: ignore[assignment]
            if moe is None:
                continue
            lo, hi = moe._e_start, moe._e_start + moe._e_local
            if not (lo <= eidx < hi):
                continue  # expert-parallel filter
            expert_buf.setdefault((block, eidx, proj), {})[suffix] = tensor
            continue
        if name.endswith(".mlp.gate.e_score_correction_bias"):
            moe = modules.get(name[: -len(".gate.e_score_correction_bias")] + ".experts")
            if moe is not None and hasattr(moe, "e_score_correction_bias"):
                assign(moe, "e_score_correction_bias", tensor.float(),
                       name[: -len(".gate.e_score_correction_bias")] + ".experts.e_score_correction_bias")
            continue
        if name.endswith(".router.proj.weight") and (name[: -len(".router.proj.weight")] + ".experts") in modules:
            # Gemma-4: the router's projection is the expert layer's gate
            moe = modules[name[: -len(".router.proj.weight")] + ".experts"]
            assign(moe.gate, "weight", tensor, name[: -len(".router.proj.weight")] + ".experts.gate.weight")
            continue
        if name == "model.embed_tokens_per_layer.weight" and hasattr(model.model, "embed_tokens_per_layer"):
            emb = model.model.embed_tokens_per_layer
            assign(emb, "weight", vocab_shard(tensor, emb._per_rank), name)
            continue
        if name.endswith((".experts.gate_up_proj", ".experts.down_proj")) and tensor.dim() == 3:
            # expert stacks stored fused: [E, 2I, H] (gate rows then up rows) and [E, H, I]
            moe = modules.get(name.rsplit(".", 1)[0])
            if moe is None:
                continue
            lo, hi = moe._e_start, moe._e_start + moe._e_local
            t3 = tensor[lo:hi]
            if name.endswith("gate_up_proj"):
                if moe._ep is None and tp.size > 1:
                    gate, up = t3.chunk(2, dim=1)
                    t3 = torch.cat([_slice(gate, 1, tp.rank, tp.size), _slice(up, 1, tp.rank, tp.size)], dim=1)
                assign(moe, "w13", t3, name.rsplit(".", 1)[0] + ".w13")
            else:
                if moe._ep is None and tp.size > 1:
                    t3 = _slice(t3, 2, tp.rank, tp.size)
                assign(moe, "w2", t3, name.rsplit(".", 1)[0] + ".w2")
            continue
        if name.endswith(".mlp.gate.weight") and (name[: -len(".gate.weight")] + ".experts") in modules:
            moe = modules[name[: -len(".gate.weight")] + ".experts"]
            assign(moe.gate, "weight", tensor, name[: -len(".gate.weight")] + ".experts.gate.weight")
            continue
        if name.endswith(".mlp.shared_expert_gate.weight"):
            blk = modules.get(name[: -len(".shared_expert_gate.weight")])
            if blk is not None and hasattr(blk, "shared_expert_gate"):
                assign(blk, "shared_expert_gate", tensor, name[: -len(".weight")])
            continue
        # ---- embeddings / head
        if name == "model.embed_tokens.weight":
            emb: VocabParallelEmbedding = model.model.embed_tokens
            assign(emb, "weight", vocab_shard(tensor, emb._per_rank), name)
            continue
        if name == "lm_head.weight":
            head: ParallelLMHead = model.lm_head
            if head._tied is None:
                assign(head, "weight", vocab_shard(tensor, head._per_rank), name)
            continue
        # ---- linear projections (possibly merged)
        parent, _, leaf = name.rpartition(".")
        gp, _, proj = parent.rpartition(".")
        # suffixes with a dot ("weight_scale_inv" has none, fine)
        merged_name = gp + (".qkv_proj" if proj in _QKV else ".gate_up_proj")
        if (proj in _QKV or proj in _GATE_UP) and (merged_name in modules or parent not in modules):
            mod = modules.get(merged_name)
            if mod is None:
                continue
            part = _QKV[proj] if proj in _QKV else _GATE_UP[proj]
            n_parts = 3 if proj in _QKV else 2
            piece = shard_linear(mod, leaf, tensor, "col", part)
            key = merged_name + "." + leaf
            col = pending.setdefault(key, _Collector(n_parts))
            if col.add(part, piece):
                dims = mod._method.shard_dims().get(leaf, (0, -1))
                n_dim = dims[0] if dims[0] >= 0 else 0
                if piece.dim() == 0 or (piece.dim() >= 1 and leaf.endswith("global_scale") and piece.numel() == 1):
                    # one scalar per sub-projection: expand to per-channel
                    sizes = [mod._q_local * mod._head_dim, mod._kv_local * mod._head_dim,
                             mod._kv_local * mod._head_dim] if proj in _QKV else mod._parts
                    value = torch.cat([col.parts[i].reshape(1).expand(sizes[i]) for i in range(n_parts)])
                else:
                    value = col.cat(n_dim)
                assign(mod, leaf, value, key)
                del pending[key]
            continue
        mod = modules.get(parent)
        if mod is None:
            logger.debug_rank0("skipping unexpected tensor %s", name)
            continue
        if isinstance(mod, RowParallelLinear):
            assign(mod, leaf, shard_linear(mod, leaf, tensor, "row", None), name)
        elif isinstance(mod, _LinearBase) and not isinstance(mod, (MergedColumnParallelLinear, QKVParallelLinear)):
            which = "none" if type(mod).__name__ == "ReplicatedLinear" else "col"
            assign(mod, leaf, shard_linear(mod, leaf, tensor, which, None), name)
        elif hasattr(mod, leaf):
            assign(mod, leaf, tensor, name)

    # ---- stack experts
    by_block: Dict[str, List[Tuple[int, str]]] = {}
    for (block, eidx, proj) in expert_buf:
        by_block.setdefault(block, []).append((eidx, proj))
    for block, _items in by_block.items():
        moe = modules[block + ".experts"]
        scheme = cfg.quant.for_module(block + ".experts.0.gate_proj") if cfg.quant is not None else None
        inter = moe._i_local
        first = expert_buf[(block, moe._e_start, "gate_proj")]
        kind = getattr(moe, "_quant_kind", None)
        raw_ok = (kind in ("fp8_block", "fp8_channel") and first.get("weight") is not None
                  and first["weight"].dtype == torch.float8_e4m3fn
                  and ("weight_scale_inv" in first if kind == "fp8_block" else "weight_scale" in first))
        if raw_ok:
            # keep the checkpoint's e4m3 values and scales: [E, 2I, H] + scales, [E, H, I] + scales
            sname = "weight_scale_inv" if kind == "fp8_block" else "weight_scale"
            qs13, ss13, qs2, ss2 = [], [], [], []
            for local in range(moe._e_local):
                e = moe._e_start + local
                parts = {p: expert_buf[(block, e, p)] for p in ("gate_proj", "up_proj", "down_proj")}
                gq, uq, dq = (parts[p]["weight"] for p in ("gate_proj", "up_proj", "down_proj"))
                gs, us, ds = (parts[p][sname].float() for p in ("gate_proj", "up_proj", "down_proj"))
                if kind == "fp8_channel":
                    gs, us, ds = gs.reshape(-1), us.reshape(-1), ds.reshape(-1)
                if moe._ep is None and tp.size > 1:
                    gq, uq = _slice(gq, 0, tp.rank, tp.size), _slice(uq, 0, tp.rank, tp.size)
                    dq = _slice(dq, 1, tp.rank, tp.size)
                    gs, us = _slice(gs, 0, tp.rank, tp.size), _slice(us, 0, tp.rank, tp.size)
                    if kind == "fp8_block":
                        ds = _slice(ds, 1, tp.rank, tp.size)
                qs13.append(torch.cat([gq, uq], 0))
                ss13.append(torch.cat([gs, us], 0))
                qs2.append(dq)
                ss2.append(ds)
            moe._raw_fp8 = (torch.stack(qs13), torch.stack(ss13), torch.stack(qs2), torch.stack(ss2))
            moe.w13 = torch.empty((0,) + tuple(moe.w13.shape[1:]), dtype=moe.w13.dtype, device=device)
            moe.w2 = torch.empty((0,) + tuple(moe.w2.shape[1:]), dtype=moe.w2.dtype, device=device)
            loaded.add(block + ".experts.w13")
            loaded.add(block + ".experts.w2")
            continue
        w13 = torch.empty(moe.w13.shape, dtype=moe.w13.dtype)
        w2 = torch.empty(moe.w2.shape, dtype=moe.w2.dtype)
        for local in range(moe._e_local):
            e = moe._e_start + local
            gate = _expert_dense(expert_buf[(block, e, "gate_proj")], scheme)
            up = _expert_dense(expert_buf[(block, e, "up_proj")], scheme)
            down = _expert_dense(expert_buf[(block, e, "down_proj")], scheme)
            if moe._ep is None and tp.size > 1:
                gate, up = _slice(gate, 0, tp.rank, tp.size), _slice(up, 0, tp.rank, tp.size)
                down = _slice(down, 1, tp.rank, tp.size)
            w13[local, :inter] = gate
            w13[local, inter:] = up
            w2[local] = down
        moe.w13 = w13.to(device)
        moe.w2 = w2.to(device)
        loaded.add(block + ".experts.w13")
        loaded.add(block + ".experts.w2")
    if pending:
        raise KeyError(f"incomplete merged parameters: {sorted(pending)[:6]}")
    # anything still on the meta device or uninitialised that the checkpoint did not provide
    missing = [n for n, t, _, _ in model.named_parameters() if n not in loaded and not n.endswith("bias")]
    still = [n for n in missing if not _optional(n)]
    if still:
        raise KeyError(f"checkpoint is missing parameters: {still[:8]} (+{max(len(still) - 8, 0)} more)")
    for n, t, owner, attr in model.named_parameters():
        if n not in loaded and n.endswith("bias"):
            setattr(owner, attr, torch.zeros_like(t))  # all-zero biases are dropped by exporters


def _optional(name: str) -> bool:
    return name.endswith(("weight_zero_point", "qzeros"))


def _expert_dense(parts: Dict[str, torch.Tensor], scheme) -> torch.Tensor:
    """One expert projection as a 16/32-bit ``(N, K)`` matrix."""
    w = parts.get("weight")
    if w is None:
        if "weight_packed" in parts and scheme is not None and scheme.name == "mxfp4":
            from ..ops.ref import dequant_mxfp4

            return dequant_mxfp4(parts["weight_packed"], parts["weight_scale"])
        raise KeyError(f"unsupported expert tensor set {sorted(parts)}")
    if w.dtype == torch.float8_e4m3fn:
        wf = w.float()
        if "weight_scale_inv" in parts:
            s = parts["weight_scale_inv"].float()
            bn, bk = -(-w.shape[0] // s.shape[0]), -(-w.shape[1] // s.shape[1])
            s = s.repeat_interleave(bn, 0).repeat_interleave(bk, 1)[: w.shape[0], : w.shape[1]]
            return wf * s
        if "weight_scale" in parts:
            return wf * parts["weight_scale"].float().reshape(-1, 1)
        return wf
    return w


def save_dummy_checkpoint(model, path: str, cfg_dict: dict) -> None:
    """Write a model's parameters in the Hugging Face layout (tests and tooling): splits the
    merged projections back into q/k/v and gate/up and unstacks experts. Tensor-parallel size
    must be 1."""
    from safetensors.torch import save_file

    assert get_tp_info().size == 1
    os.makedirs(path, exist_ok=True)
    cfg = model.config
    out: Dict[str, torch.Tensor] = {}
    qs, ks = cfg.num_qo_heads * cfg.head_dim, cfg.num_kv_heads * cfg.head_dim
    for name, t, owner, attr in model.named_parameters():
        t = t.detach().cpu()
        if ".qkv_proj." in name:
            dims = owner._method.shard_dims().get(attr, (0, -1)) if attr != "bias" else (0, -1)
            nd = max(dims[0], 0)
            unit = t.shape[nd] // (cfg.num_qo_heads + 2 * cfg.num_kv_heads)
            sizes = [cfg.num_qo_heads * unit, cfg.num_kv_heads * unit, cfg.num_kv_heads * unit]
            for proj, piece in zip(("q_proj", "k_proj", "v_proj"), t.split(sizes, nd)):
                out[name.replace("qkv_proj", proj)] = piece.contiguous()
        elif ".gate_up_proj." in name:
            dims = owner._method.shard_dims().get(attr, (0, -1)) if attr != "bias" else (0, -1)
            nd = max(dims[0], 0)
            g, u = t.chunk(2, nd)
            out[name.replace("gate_up_proj", "gate_proj")] = g.contiguous()
            out[name.replace("gate_up_proj", "up_proj")] = u.contiguous()
        elif name.endswith(".experts.w13"):
            base = name[: -len(".w13")]
            for e in range(t.shape[0]):
                g, u = t[e].chunk(2, 0)
                out[f"{base}.{e}.gate_proj.weight"] = g.contiguous()
                out[f"{base}.{e}.up_proj.weight"] = u.contiguous()
        elif name.endswith(".experts.w2"):
            base = name[: -len(".w2")]
            for e in range(t.shape[0]):
                out[f"{base}.{e}.down_proj.weight"] = t[e].contiguous()
        elif name.endswith(".experts.gate.weight"):
            out[name.replace(".experts.gate.weight", ".gate.weight")] = t
        elif name.endswith(".shared_expert_gate"):
            out[name + ".weight"] = t
        else:
            out[name] = t
    save_file(out, os.path.join(path, "model.safetensors"))
    with open(os.path.join(path, "config.json"), "w") as fh:
        json.dump(cfg_dict, fh)
