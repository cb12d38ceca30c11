"""Single-kernel micro-benchmarks with CUDA-event timing and roofline fractions.

``python -m minisglang_rdna4_b200.benchmark.kernels <op> [shape flags]`` runs one op a few times
(L2 is flushed between timed iterations by writing a 256 MiB buffer) and prints one JSON line
with the median time, achieved TFLOP/s or GB/s and the fraction of the measured peaks
(``MEASURED_PEAKS.json`` at the repository root when present). The same command line is what
the ``ncu`` summaries under ``profiles/`` were captured with.

ops: gemm (--kind bf16|w8a8|mxfp4), attn_decode, attn_prefill, rms_norm, silu_quant, rope_store,
     moe
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def timeit(fn, iters: int, warmup: int = 3, flush=None) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2]


def _library_attention(a, q, pool, bt, cu, sl, ks, q_len, kv_len, kv_bytes, flops, hbm, tf, ours, flush) -> dict:
    """The same attention problem through flashinfer: its paged wrappers (``flashinfer``) or the
    TensorRT-LLM generation kernels it ships (``flashinfer-trtllm``). The library gets this GPU's own
    tensors only. Reports the time, the same roofline fractions and the largest difference to our output;
    an arm that cannot run here says why instead."""
    res = {"lib": a.lib}
    try:
        import flashinfer

        hq, hk, d, ps = a.heads, a.kv_heads, a.head_dim, a.page_size
        b = sl.numel()
        kc, vc = pool[0, 0], pool[1, 0]                      # [pages, hk, ps, d] = flashinfer's "HND" layout
        ws = torch.zeros(256 << 20, dtype=torch.uint8, device="cuda")
        scale = d ** -0.5
        kscale = float(ks[0]) if ks is not None else 1.0
        if a.lib == "flashinfer-trtllm":
            if q_len == 1:
                run = lambda: flashinfer.decode.trtllm_batch_decode_with_kv_cache(
                    q, (kc, vc), ws, bt, sl, kv_len, bmm1_scale=scale * kscale, bmm2_scale=kscale, kv_layout="HND")
            else:
                cu_kv = torch.zeros(b + 1, dtype=torch.int32, device="cuda")
                cu_kv[1:] = sl.cumsum(0)
                run = lambda: flashinfer.prefill.trtllm_batch_context_with_kv_cache(
                    q, (kc, vc), ws, bt, sl, q_len, kv_len, scale * kscale, kscale, b, cu, cu_kv, kv_layout="HND")
        else:
            pages = (sl + ps - 1) // ps
            indptr = torch.zeros(b + 1, dtype=torch.int32, device="cuda")
            indptr[1:] = pages.cumsum(0)
            indices = torch.cat([bt[i, :int(pages[i])] for i in range(b)]).to(torch.int32)
            last = ((sl - 1) % ps + 1).to(torch.int32)
            if q_len == 1:
                w = flashinfer.BatchDecodeWithPagedKVCacheWrapper(ws, "HND", use_tensor_cores=True)
                w.plan(indptr, indices, last, hq, hk, d, ps, q_data_type=q.dtype, kv_data_type=kc.dtype, sm_scale=scale)
            else:
                w = flashinfer.BatchPrefillWithPagedKVCacheWrapper(ws, "HND")
                w.plan(cu, indptr, indices, last, hq, hk, d, ps, causal=True, q_data_type=q.dtype,
                       kv_data_type=kc.dtype, sm_scale=scale)
            kw = dict(k_scale=kscale, v_scale=kscale) if ks is not None else {}
            run = lambda: w.run(q, (kc, vc), **kw)
        got = run()
        torch.cuda.synchronize()
        ms = timeit(run, a.iters, a.warmup, flush)
        res.update(us=ms * 1e3, kv_gbs=kv_bytes / ms / 1e6, tflops=flops / ms / 1e9, frac_of_hbm=kv_bytes / ms / 1e6 / hbm,
                   frac_of_bf16_peak=flops / ms / 1e9 / tf,
                   max_abs_diff_to_ours=float((got.float().view(-1) - ours.float().view(-1)).abs().max()))
    except Exception as exc:                                   # missing cubins, no JIT toolchain, unsupported shape
        res["unavailable"] = f"{type(exc).__name__}: {str(exc)[:300]}"
    return res


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["gemm", "attn_decode", "attn_prefill", "rms_norm", "silu_quant", "rope_store", "moe"])
    ap.add_argument("--kind", default="mxfp4", choices=["bf16", "w8a8", "mxfp4", "int4", "fp8_block"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=6144)
    ap.add_argument("--k", type=int, default=2560)
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--ctx", type=int, default=1400)
    ap.add_argument("--ctx-min", type=int, default=0, help="decode: context lengths uniform in [ctx-min, ctx]")
    ap.add_argument("--order", default="random", choices=["random", "desc", "asc"],
                    help="decode with --ctx-min: order of the requests in the batch by context length")
    ap.add_argument("--seqs", type=int, default=6)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--splits", type=int, default=1)
    ap.add_argument("--stages", type=int, default=0, help="attn_decode with fp8 KV: stages of the TMA ring (2-4)")
    ap.add_argument("--general", action="store_true", help="attn_prefill: the warp-level MMA kernel instead of the tcgen05 one")
    ap.add_argument("--kv", default="fp8", choices=["fp8", "bf16"])
    ap.add_argument("--lib", default="", choices=["", "flashinfer", "flashinfer-trtllm"],
                    help="attn_decode / attn_prefill: also time the library kernel on the same inputs (the reference's "
                         "attention backends on this GPU: python/minisgl/attention/fi.py, trtllm.py:53-90)")
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    a = ap.parse_args(argv)

    from ..ops import cuda as K
    from ..ops import ref
    from ..quant import mxfp4

    hbm, tf, src = _peaks()
    flush = None if a.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    out = {"op": a.op, "peaks": src}
    if a.op == "gemm":
        m, n, k = a.m, a.n, a.k
        x = torch.randn(m, k, device="cuda").bfloat16()
        w = torch.randn(n, k, device="cuda") * 0.02
        if a.kind == "bf16":
            wb = w.bfloat16()
            fn = lambda: K.gemm(x, wb, bn=a.bn)
            wbytes = n * k * 2 + m * k * 2
        elif a.kind == "w8a8":
            ws = w.abs().amax(-1) / 448
            wq = (w / ws[:, None]).to(torch.float8_e4m3fn)
            xq, xs = K.per_token_quant_fp8(x)
            fn = lambda: K.gemm_w8a8(xq, xs, wq, ws.float(), bn=a.bn)
            wbytes = n * k + m * k
        elif a.kind == "int4":
            # 4-bit-resident W4A16 (group 128, asymmetric): codes + fp32 scale / zero per group
            g = 128
            codes = torch.randint(0, 16, (n, k), device="cuda", dtype=torch.uint8)
            pk = (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()
            sc = (torch.rand(k // g, n, device="cuda") * 0.01 + 0.001).float()
            zp = torch.full((k // g, n), 8.0, device="cuda")
            fn = lambda: K.gemm_w4a16(x, pk, sc, zp, None, g)
            wbytes = n * k // 2 + 2 * (k // g) * n * 4 + m * k * 2
        elif a.kind == "fp8_block":
            wq = w.to(torch.float8_e4m3fn)
            ws = torch.rand((n + 127) // 128, (k + 127) // 128, device="cuda") * 0.01 + 0.001
            xq, xs = K.per_group_quant_fp8(x, 128)
            fn = lambda: K.gemm_fp8_block(xq, xs, wq, ws)
            wbytes = n * k + m * k
        else:
            packed, sf = mxfp4.quantize_mxfp4(w)
            atoms = mxfp4.pack_sf_atoms(sf)
            xq, xs = K.per_token_quant_fp8(x)
            fn = lambda: K.gemm_w4a8_mxfp4(xq, xs, packed, atoms, bn=a.bn)
            wbytes = n * k // 2 + n * k // 32 + m * k
        del w
        ms = timeit(fn, a.iters, a.warmup, flush)
        flops = 2.0 * m * n * k
        byts = wbytes + m * n * 2
        out.update(kind=a.kind, m=m, n=n, k=k, us=ms * 1e3, tflops=flops / ms / 1e9, gbs=byts / ms / 1e6,
                   frac_of_bf16_peak=flops / ms / 1e9 / tf, frac_of_hbm=byts / ms / 1e6 / hbm)
        assert K.gemm_status() == 0
        if a.kind == "int4":
            assert K.gemm_w4a16_status() == 0
    elif a.op in ("attn_decode", "attn_prefill"):
        hq, hk, d, ps = a.heads, a.kv_heads, a.head_dim, a.page_size
        dt = torch.float8_e4m3fn if a.kv == "fp8" else torch.bfloat16
        if a.op == "attn_decode":
            b, q_len, kv_len = a.batch, 1, a.ctx
        else:
            b, q_len, kv_len = a.seqs, a.ctx, a.ctx
        npg = -(-kv_len // ps)
        pool = (torch.randn(2, 1, b * npg + 1, hk, ps, d, device="cuda") * 4).to(dt)
        bt = torch.arange(b * npg, device="cuda", dtype=torch.int32).view(b, npg)
        cu = torch.arange(b + 1, device="cuda", dtype=torch.int32) * q_len
        sl = torch.full((b,), kv_len, device="cuda", dtype=torch.int32)
        if a.op == "attn_decode" and a.ctx_min > 0:
            g = torch.Generator().manual_seed(0)
            lens = torch.randint(a.ctx_min, kv_len + 1, (b,), generator=g)
            if a.order != "random":
                lens = lens.sort(descending=a.order == "desc").values
            sl = lens.to("cuda", torch.int32)
        q = torch.randn(b * q_len, hq, d, device="cuda").bfloat16()
        ks = torch.ones(hk, device="cuda") / 8 if a.kv == "fp8" else None
        if a.stages:
            K.decode_attention_stages(a.stages)
        plan = None
        if q_len > 1 and not a.general:
            plan = K.PrefillPlan(cu.cpu().numpy(), sl.cpu().numpy(), q.device)  # once per step, as the engine does
        fn = lambda: K.paged_attention(q, pool[0, 0], pool[1, 0], bt, cu, sl, d ** -0.5, k_scale=ks, v_scale=ks,
                                       max_q=q_len, max_kv=kv_len, decode=q_len == 1, splits=a.splits, plan=plan,
                                       tc=plan is not None)
        ms = timeit(fn, a.iters, a.warmup, flush)
        kv_bytes = int(sl.sum()) * hk * d * 2 * pool.element_size()
        flops = 4.0 * b * hq * d * (kv_len * q_len if q_len == 1 else kv_len * kv_len / 2)
        out.update(batch=b, q_len=q_len, kv_len=kv_len, kv=a.kv, splits=a.splits, us=ms * 1e3,
                   kernel=K.LEDGER.get("prefill_attention", K.LEDGER.get("paged_attention")),
                   kv_gbs=kv_bytes / ms / 1e6, tflops=flops / ms / 1e9, frac_of_hbm=kv_bytes / ms / 1e6 / hbm,
                   frac_of_bf16_peak=flops / ms / 1e9 / tf)
        assert K.attn_status() == 0
        if a.lib:
            out["library"] = _library_attention(a, q, pool, bt, cu, sl, ks, q_len, kv_len, kv_bytes, flops, hbm, tf,
                                                fn(), flush)
    elif a.op == "rms_norm":
        x = torch.randn(a.m, a.k, device="cuda").bfloat16()
        r = torch.randn(a.m, a.k, device="cuda").bfloat16()
        w = torch.ones(a.k, device="cuda").bfloat16()
        ms = timeit(lambda: K.rms_norm_quant(x, w, 1e-6, r), a.iters, a.warmup, flush)
        byts = a.m * a.k * (2 + 2 + 2 + 1)
        out.update(m=a.m, hidden=a.k, us=ms * 1e3, gbs=byts / ms / 1e6, frac_of_hbm=byts / ms / 1e6 / hbm)
    elif a.op == "silu_quant":
        g = torch.randn(a.m, 2 * a.k, device="cuda").bfloat16()
        ms = timeit(lambda: K.silu_and_mul_quant(g), a.iters, a.warmup, flush)
        byts = a.m * a.k * 5
        out.update(m=a.m, inter=a.k, us=ms * 1e3, gbs=byts / ms / 1e6, frac_of_hbm=byts / ms / 1e6 / hbm)
    elif a.op == "rope_store":
        hq, hk, d = a.heads, a.kv_heads, a.head_dim
        qkv = torch.randn(a.m, (hq + 2 * hk) * d, device="cuda").bfloat16()
        pool = torch.zeros(2, 1, a.m // 16 + 2, hk, 16, d, device="cuda", dtype=torch.float8_e4m3fn)
        pos = torch.arange(a.m, device="cuda", dtype=torch.int32) % 4096
        loc = torch.arange(a.m, device="cuda", dtype=torch.int32)
        cs = ref.build_cos_sin_cache(d, 4096, 1e6).cuda()
        w = torch.ones(d, device="cuda").bfloat16()
        ks = torch.ones(hk, device="cuda")
        ms = timeit(lambda: K.qk_norm_rope_store(qkv, w, w, pos, cs, hq, hk, d, d, 1e-6, pool[0, 0], pool[1, 0], loc,
                                                 ks, ks), a.iters, a.warmup, flush)
        byts = a.m * ((hq + 2 * hk) * d * 2 + hq * d * 2 + 2 * hk * d)
        out.update(m=a.m, us=ms * 1e3, gbs=byts / ms / 1e6, frac_of_hbm=byts / ms / 1e6 / hbm)
    elif a.op == "moe":
        from ..ops import moe_kernels as MK

        h, inter, e, k = a.k, a.n, a.experts, a.top_k
        x = torch.randn(a.m, h, device="cuda").bfloat16()
        w13 = (torch.randn(e, 2 * inter, h, device="cuda") * 0.02).bfloat16()
        w2 = (torch.randn(e, h, inter, device="cuda") * 0.02).bfloat16()
        logits = torch.randn(a.m, e, device="cuda")
        tw, ids = MK.moe_route(logits, k, True)
        ms = timeit(lambda: MK.moe_forward(x, w13, w2, tw, ids), a.iters, a.warmup, flush)
        flops = 2.0 * a.m * k * 3 * h * inter
        out.update(m=a.m, hidden=h, inter=inter, experts=e, top_k=k, us=ms * 1e3, tflops=flops / ms / 1e9,
                   frac_of_bf16_peak=flops / ms / 1e9 / tf)
        assert K.gemm_status() == 0
    print(json.dumps(out))


if __name__ == "__main__":
    main()
