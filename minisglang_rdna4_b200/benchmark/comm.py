"""Multi-GPU micro-benchmarks of the fused compute + collective kernels.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        -m minisglang_rdna4_b200.benchmark.comm {allreduce|row_shard|ep} [options]

One rank per GPU. Every number is a CUDA-event time on the launching stream after warm-up,
reduced with MAX over the ranks (the slowest rank is the step time); rank 0 prints one JSON line
per case with the NVLink bytes the case must move and the fraction of the link roofline
(770 GB/s per direction per GPU, the measured peer-copy figure) it reaches.

* ``allreduce``: decode-sized all-reduce + residual add + RMSNorm + e4m3 producer
  (``comm.cu::ar_oneshot_kernel``, peer-store form and in-switch ``multimem`` form) against
  ``torch.distributed.all_reduce`` followed by the norm kernel; timed inside a CUDA graph.
* ``row_shard``: prefill-sized row-parallel GEMM → reduce-scatter push → owner-side add + norm +
  quantise → all-gather stores → column-parallel GEMM that waits per 128-row block
  (``gemm_pair_kernel`` rs_* / a_ready, ``rs_norm_ag_kernel``) against GEMM + NCCL all-reduce + norm.
* ``ep``: expert-parallel dispatch → grouped expert GEMMs → return → combine (``ep_a2a.cu``) for
  the three expert kinds, against the bytes that cross NVLink.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

LINK_GBS = 770.0


def _setup():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    cpu = dist.new_group(list(range(world)), backend="gloo")
    return rank, world, dev, cpu


def _max_over_ranks(ms: float, dev) -> float:
    t = torch.tensor([ms], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def time_eager(fn, dev, iters=20, warmup=5) -> float:
    """Microseconds per call, max over ranks."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return _max_over_ranks(s.elapsed_time(e) / iters, dev) * 1e3


def time_in_graph(fn, dev, per_graph=10, replays=5) -> float:
    """Microseconds per call when ``per_graph`` calls are captured in one CUDA graph (the decode
    step runs these kernels from a graph), max over ranks."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            for _ in range(per_graph):
                fn()
        g.replay()
        side.synchronize()
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(side)
        for _ in range(replays):
            g.replay()
        e.record(side)
        side.synchronize()
    return _max_over_ranks(s.elapsed_time(e) / (per_graph * replays), dev) * 1e3


def _emit(rank, **kw) -> None:
    if rank == 0:
        print(json.dumps(kw), flush=True)


def bench_allreduce(a) -> None:
    rank, world, dev, cpu = _setup()
    from ..ops import cuda as K
    from ..parallel.symm import SymmetricCollectives

    comm = SymmetricCollectives(dist.group.WORLD, cpu, dev, rank, world, max_rows=512, max_hidden=max(a.hidden, 4096))
    form = "in-switch (multimem)" if comm.nvls is not None else "peer stores"
    w = torch.ones(a.hidden, device=dev).bfloat16()
    for rows in a.rows:
        x = torch.randn(rows, a.hidden, device=dev).bfloat16()
        res = torch.zeros(rows, a.hidden, device=dev).bfloat16()
        fused = time_in_graph(lambda: comm.fused_allreduce_add_rmsnorm(x, res, w, 1e-6, quant=True), dev)

        def nccl():
            y = x.clone()
            dist.all_reduce(y)
            K.rms_norm_quant(y, w, 1e-6, res)

        base = time_in_graph(nccl, dev)
        msg = rows * a.hidden * 2
        # bytes one rank must receive: every peer's rows (peer stores) or one reduced row set (in-switch)
        link_bytes = msg if comm.nvls is not None else msg * (world - 1)
        roof = link_bytes / LINK_GBS / 1e3
        _emit(rank, op="allreduce_add_norm_quant", form=form, ranks=world, rows=rows, hidden=a.hidden, fused_us=fused,
              nccl_plus_norm_us=base, link_bytes_per_rank=link_bytes, link_roofline_us=roof, frac_of_link_roofline=roof / fused)
    healthy = comm.check_health()
    _emit(rank, op="allreduce", healthy=bool(healthy))
    dist.barrier()
    comm.close()
    dist.destroy_process_group()


def bench_row_shard(a) -> None:
    rank, world, dev, cpu = _setup()
    from ..ops import cuda as K
    from ..parallel.symm import SymmetricCollectives
    from ..quant import mxfp4

    m, h, inter = a.m, a.hidden, a.inter
    comm = SymmetricCollectives(dist.group.WORLD, cpu, dev, rank, world, max_rows=512, max_hidden=max(h, 4096))
    comm.enable_row_shard(m, h)
    rs = comm.row_shard

    def packed(n, k):
        p, sf = mxfp4.quantize_mxfp4(torch.randn(n, k, device=dev) * 0.02)
        return p, mxfp4.pack_sf_atoms(sf)

    res = torch.randn(m, h, device=dev).bfloat16()
    nw = torch.ones(h, device=dev).bfloat16()
    peak = json.load(open(os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                                       "MEASURED_PEAKS.json")))["bf16_tflops"] if a.peaks else 1662.9
    for name, kfull in (("o_proj", a.attn_width), ("down_proj", inter)):
        k = kfull // world
        xq, xs = K.per_token_quant_fp8(torch.randn(m, k, device=dev).bfloat16())
        wp, wa = packed(h, k)

        def fused():
            plan = rs.begin(m, torch.bfloat16)
            K.set_next_gemm_tp(rs.gemm_args(plan))
            K.gemm_w4a8_mxfp4(xq, xs, wp, wa)
            rs.finish(plan, res, nw, 1e-6, True)

        def nccl():
            y = K.gemm_w4a8_mxfp4(xq, xs, wp, wa, bn=256)
            dist.all_reduce(y)
            K.rms_norm_quant(y, nw, 1e-6, res)

        t_f, t_n = time_eager(fused, dev), time_eager(nccl, dev)
        t_g = time_eager(lambda: K.gemm_w4a8_mxfp4(xq, xs, wp, wa, bn=256), dev)
        frac = (world - 1) / world
        link = frac * m * h * 2 + frac * m * h          # 16-bit partial rows out, e4m3 result rows in
        flops = 2.0 * m * h * k
        roof = max(link / LINK_GBS / 1e3, flops / (peak * 1e6))
        _emit(rank, op="gemm_rs_norm_ag", layer=name, ranks=world, m=m, n=h, k=k, fused_us=t_f, gemm_nccl_norm_us=t_n,
              local_gemm_us=t_g, link_bytes_per_rank=link, roofline_us=roof, frac_of_roofline=roof / t_f)
    _emit(rank, op="row_shard", gemm_status=K.gemm_status(), healthy=bool(comm.check_health()))
    dist.barrier()
    comm.close()
    dist.destroy_process_group()


def bench_ep(a) -> None:
    rank, world, dev, cpu = _setup()
    from ..ops import ref
    from ..parallel.ep import FusedEPContext

    e, h, inter, k = a.experts, a.hidden, a.inter, a.top_k
    e_local = e // world

    class Experts:
        def __init__(self, kind):
            self.kind = kind
            w13 = torch.randn(e_local, 2 * inter, h, device=dev) * 0.05
            w2 = torch.randn(e_local, h, inter, device=dev) * 0.05
            if kind == "bf16":
                self.weights = (w13.bfloat16(), w2.bfloat16())
            elif kind == "fp8_block":
                def enc(wt):
                    ee, n, kk = wt.shape
                    b = wt.view(ee, n // 128, 128, kk // 128, 128)
                    sc = b.abs().amax((2, 4)).clamp_min(1e-8) / 448.0
                    return (b / sc[:, :, None, :, None]).reshape(ee, n, kk).to(torch.float8_e4m3fn), sc.float()
                self.weights = enc(w13) + enc(w2)
            else:
                def enc(wt):
                    sc = wt.abs().amax(-1).clamp_min(1e-8) / 448.0
                    return (wt / sc[..., None]).to(torch.float8_e4m3fn), sc.float()
                self.weights = enc(w13) + enc(w2)

        def expert_weights(self):
            return self.kind, self.weights

    for kind in a.kinds:
        moe = Experts(kind)
        ctx = FusedEPContext(dist.group.WORLD, cpu, rank, world, dev, h, k, e_local, max_tokens=max(a.tokens), kind=kind)
        for n in a.tokens:
            g = torch.Generator().manual_seed(17 * n + rank)
            x = torch.randn(n, h, generator=g).bfloat16().to(dev)
            tw, ids = ref.moe_route(torch.randn(n, e, generator=g), k, True)
            tw, ids = tw.to(dev), ids.to(dev)
            ctx.common_tokens = n
            t = time_eager(lambda: ctx.dispatch_compute_combine(moe, x, tw, ids), dev, iters=a.iters)
            pairs_out = n * k * (world - 1) / world                # pairs that leave this rank, on average
            row_out = h * (2 if kind == "bf16" else 1) + (h // 128 * 4 if kind == "fp8_block" else 4 if kind != "bf16" else 0)
            link = pairs_out * (row_out + 8) + pairs_out * h * 2    # dispatch rows (+ id, weight), bf16 rows back
            flops = 2.0 * n * k * 3 * h * inter
            _emit(rank, op="ep_dispatch_experts_combine", kind=kind, ranks=world, tokens_per_rank=n, hidden=h, inter=inter,
                  experts=e, top_k=k, us=t, link_bytes_per_rank_each_way=link / 2,
                  link_roofline_us=link / 2 / LINK_GBS / 1e3, expert_tflops_per_rank=flops / t / 1e6)
        del ctx
    dist.barrier()
    dist.destroy_process_group()


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="op", required=True)
    p = sub.add_parser("allreduce")
    p.add_argument("--hidden", type=int, default=2560)
    p.add_argument("--rows", type=int, nargs="+", default=[1, 16, 64, 256, 512])
    p = sub.add_parser("row_shard")
    p.add_argument("--m", type=int, default=8192)
    p.add_argument("--hidden", type=int, default=2560)
    p.add_argument("--inter", type=int, default=9728)
    p.add_argument("--attn-width", type=int, default=4096)
    p.add_argument("--peaks", action="store_true", help="read the bf16 peak from MEASURED_PEAKS.json at the repository root")
    p = sub.add_parser("ep")
    p.add_argument("--hidden", type=int, default=2048)
    p.add_argument("--inter", type=int, default=768)
    p.add_argument("--experts", type=int, default=128)
    p.add_argument("--top-k", type=int, default=8)
    p.add_argument("--tokens", type=int, nargs="+", default=[64, 512, 4096])
    p.add_argument("--kinds", nargs="+", default=["bf16", "fp8_channel", "fp8_block"])
    p.add_argument("--iters", type=int, default=10)
    a = ap.parse_args(argv)
    {"allreduce": bench_allreduce, "row_shard": bench_row_shard, "ep": bench_ep}[a.op](a)


if __name__ == "__main__":
    main()
