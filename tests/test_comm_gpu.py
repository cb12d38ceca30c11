"""Peer-memory collectives: numerics against an fp32 reference on 2 GPUs (child processes, one
per GPU), CUDA-graph replay, a lagging rank, and the bounded wait (one GPU: a flag that nothing
sets runs out and is reported, nothing hangs)."""
import ctypes
import os

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    import time

    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    cpu = dist.new_group(list(range(world)), backend="gloo")
    from minisglang_rdna4_b200.ops import ref
    from minisglang_rdna4_b200.parallel.symm import SymmetricCollectives

    comm = SymmetricCollectives(dist.group.WORLD, cpu, dev, rank, world, max_rows=256, max_hidden=4096)
    ok = True
    msgs = []
    nvls = os.environ.get("MSGL_NVLS") == "on"
    if nvls and comm.nvls is None:
        # no NVLink multicast on this machine: nothing to test in this mode
        dist.barrier()
        q.put((rank, True, ["multicast unavailable"]))
        comm.close()
        dist.destroy_process_group()
        return
    for rows, hidden in [(1, 256), (7, 2560), (256, 4096), (33, 1024)]:
        for it in range(3):
            g = torch.Generator(device="cpu").manual_seed(100 * rows + it)
            parts = [torch.randn(rows, hidden, generator=g).bfloat16() for _ in range(world)]
            res0 = torch.randn(rows, hidden, generator=g).bfloat16()
            w = (1 + 0.1 * torch.randn(hidden, generator=g)).bfloat16()
            x = parts[rank].to(dev)
            res = res0.clone().to(dev)
            if rank == 1 and it == 1:
                time.sleep(0.05)  # a lagging rank must not break the flag protocol
            out = comm.fused_allreduce_add_rmsnorm(x, res, w.to(dev), 1e-6)
            total = sum(p.float() for p in parts)
            want_res = (total + res0.float()).bfloat16()
            want = ref.rms_norm(want_res, w, 1e-6)
            # the switch rounds the sum to 16 bits before the residual is added; the push form adds in fp32
            res_ok = (float((res.cpu().float() - want_res.float()).abs().max()) <= 0.07) if nvls \
                else torch.equal(res.cpu(), want_res)
            if not res_ok:
                ok = False
                msgs.append(f"residual mismatch rows={rows} hidden={hidden} it={it}")
            if float((out.cpu().float() - want.float()).abs().max()) > (0.12 if nvls else 0.05):
                ok = False
                msgs.append(f"norm mismatch rows={rows} hidden={hidden} it={it}")
            # quantised variant and plain all-reduce
            res2 = res0.clone().to(dev)
            qv, sc = comm.fused_allreduce_add_rmsnorm(x, res2, w.to(dev), 1e-6, quant=True)
            deq = qv.float().cpu() * sc.cpu()[:, None]
            if float((deq - want.float()).abs().max()) > 0.15 * float(want.float().abs().max()):
                ok = False
                msgs.append(f"quant mismatch rows={rows} hidden={hidden}")
            y = x.clone()
            comm.all_reduce(y)
            if (float((y.cpu().float() - total).abs().max()) > 0.07) if nvls else \
                    (not torch.equal(y.cpu(), total.bfloat16())):
                ok = False
                msgs.append(f"all_reduce mismatch rows={rows} hidden={hidden}")
    # vocabulary-parallel arg-max: shard logits -> global greedy ids, ties to the lowest index
    for rows, shard in [(1, 1000), (37, 4096), (256, 19000)]:
        g = torch.Generator(device="cpu").manual_seed(rows)
        full = torch.randn(rows, shard * world, generator=g)
        full[0, 5] = full[0, shard + 7] = 50.0  # a tie across ranks
        mine = torch.zeros(rows, shard + 24)     # padded leading dimension
        mine[:, :shard] = full[:, rank * shard:(rank + 1) * shard]
        got = comm.vocab_argmax(mine.to(dev), shard, rank * shard)
        for _ in range(2):  # the sequence counters must survive repeated calls
            got = comm.vocab_argmax(mine.to(dev), shard, rank * shard)
        if got is None or not torch.equal(got.cpu().long(), full.argmax(-1)):
            ok = False
            msgs.append(f"vocab argmax mismatch rows={rows}")
    # every rank must hold bit-identical results (rank-ordered reduction)
    x = torch.randn(64, 2560, device=dev).bfloat16()
    res = torch.zeros(64, 2560, device=dev).bfloat16()
    w = torch.ones(2560, device=dev).bfloat16()
    out = comm.fused_allreduce_add_rmsnorm(x, res, w, 1e-6)
    gathered = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(gathered, out)
    if not all(torch.equal(gathered[0], t) for t in gathered):
        ok = False
        msgs.append("ranks disagree bitwise")
    # CUDA graph: the sequence counters live on the device, so a replay needs no host state
    static_x = torch.randn(16, 2560, device=dev).bfloat16()
    static_res = torch.zeros(16, 2560, device=dev).bfloat16()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        comm.fused_allreduce_add_rmsnorm(static_x, static_res, w, 1e-6)
        s.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            static_out = comm.fused_allreduce_add_rmsnorm(static_x, static_res, w, 1e-6)
        for _ in range(3):
            static_res.zero_()
            graph.replay()
        s.synchronize()
    tot = static_x.clone()
    dist.all_reduce(tot)
    want = ref.rms_norm(tot, w, 1e-6)
    if float((static_out.float() - want.float()).abs().max()) > 0.05:
        ok = False
        msgs.append("graph replay mismatch")
    torch.cuda.synchronize()
    if not comm.check_health():
        ok = False
        msgs.append("a device wait timed out")
    dist.barrier()
    q.put((rank, ok, msgs))
    comm.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_allreduce(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run_ranks(_worker, world, 23000, {"MSGL_NVLS": "off"})


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_allreduce_in_switch_reduction(world):
    """The same fused all-reduce + add + norm (+ e4m3) with the sum formed inside the NVSwitch
    (multimem.ld_reduce over a multicast-bound buffer), including the graph replay and the lagging
    rank. All ranks exit normally with nothing in flight."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run_ranks(_worker, world, 24000, {"MSGL_NVLS": "on"})


def test_bounded_wait_reports_and_returns():
    """One GPU plays rank 0 of a 2-rank group whose peer never arrives: the flag wait runs out
    after 2 ms, the status word says which peer was missing, and the context stays usable."""
    from minisglang_rdna4_b200.ops._lib import lib
    from minisglang_rdna4_b200.parallel import symm  # noqa: F401  (registers the signatures)

    L = lib()
    rows, hidden, max_rows, max_hidden = 4, 256, 8, 256
    flag_bytes = 2 * max_rows * 4
    nbytes = 256 + 2 * 2 * max_rows * max_hidden * 2
    a, b = L.msgl_symm_alloc(nbytes), L.msgl_symm_alloc(nbytes)
    assert a and b
    PtrArr = ctypes.c_void_p * 2
    flags = PtrArr(a, b)
    slots = PtrArr(a + 256, b + 256)
    seq = torch.zeros(max_rows, dtype=torch.int32, device="cuda")
    x = torch.ones(rows, hidden, device="cuda").bfloat16()
    out = torch.empty_like(x)
    L.msgl_comm_status(1)
    rc = L.msgl_ar_oneshot(x.data_ptr(), None, None, out.data_ptr(), None, None, slots, flags, seq.data_ptr(),
                           0, 2, rows, hidden, max_rows, max_hidden, 0.0, 0, 2000, 0,
                           torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert L.msgl_comm_status(1) == 301          # waited for peer 1
    assert L.msgl_comm_status(0) == 0            # cleared
    # the context still works
    assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0
    assert flag_bytes > 0
    L.msgl_symm_free(a)
    L.msgl_symm_free(b)


def _explain(ref, moe, x, tw, ids, got, want, tol, e_local):
    """Which tokens are off, and how much of each routed expert's contribution the result holds
    (least-squares coefficient per (token, k) pair: 1 = present, 0 = missing) plus the share of the
    result that no contribution of this step explains."""
    scale = max(float(want.abs().max()), 1e-6)
    out = []
    for t in range(x.shape[0]):
        if float((got[t] - want[t]).abs().max()) / scale <= tol:
            continue
        parts = torch.stack([ref.moe_forward(x[t:t + 1], moe.dense[0], moe.dense[1], tw[t:t + 1, j:j + 1],
                                             ids[t:t + 1, j:j + 1]).float()[0] for j in range(ids.shape[1])], 1)
        coef = torch.linalg.lstsq(parts, got[t][:, None]).solution[:, 0]
        rest = float((got[t] - parts @ coef).norm() / got[t].norm().clamp_min(1e-9))
        owners = [int(v) // e_local for v in ids[t].tolist()]
        out.append(f"token {t} owners {owners} held {[round(float(c), 2) for c in coef]} foreign {rest:.2f}")
    return " | ".join(out[:6])


def _ep_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    import time

    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    cpu = dist.new_group(list(range(world)), backend="gloo")
    from minisglang_rdna4_b200.ops import ref
    from minisglang_rdna4_b200.parallel.ep import FusedEPContext

    e, h, inter, k = 16, 256, 128, 4
    e_local = e // world
    g = torch.Generator().manual_seed(5)
    w13 = (torch.randn(e, 2 * inter, h, generator=g) * 0.05)
    w2 = (torch.randn(e, h, inter, generator=g) * 0.05)

    def blocks(wt):  # [E, N, K] -> e4m3, [E, N/128, K/128] scales, de-quantised copy
        ee, n, kk = wt.shape
        b = wt.view(ee, n // 128, 128, kk // 128, 128)
        sc = b.abs().amax((2, 4)).clamp_min(1e-8) / 448.0
        qv = (b / sc[:, :, None, :, None]).reshape(ee, n, kk).to(torch.float8_e4m3fn)
        deq = qv.float() * sc.repeat_interleave(128, 1).repeat_interleave(128, 2)
        return qv, sc.float(), deq.bfloat16()

    def channels(wt):
        sc = wt.abs().amax(-1).clamp_min(1e-8) / 448.0
        qv = (wt / sc[..., None]).to(torch.float8_e4m3fn)
        return qv, sc.float(), (qv.float() * sc[..., None]).bfloat16()

    mine = slice(rank * e_local, (rank + 1) * e_local)

    class Moe:
        def __init__(self, kind):
            self.kind = kind
            if kind == "bf16":
                self.dense = (w13.bfloat16(), w2.bfloat16())
                self.weights = tuple(t[mine].contiguous().to(dev) for t in self.dense)
            else:
                enc = blocks if kind == "fp8_block" else channels
                q13, s13, d13 = enc(w13)
                q2, s2, d2 = enc(w2)
                self.dense = (d13, d2)
                self.weights = tuple(t[mine].contiguous().to(dev) for t in (q13, s13, q2, s2))

        def expert_weights(self):
            return self.kind, self.weights

    ok, msgs = True, []
    for kind, tol in (("bf16", 0.05), ("fp8_block", 0.12), ("fp8_channel", 0.12)):
        moe = Moe(kind)
        ctx = FusedEPContext(dist.group.WORLD, cpu, rank, world, dev, h, k, e_local, max_tokens=64, kind=kind)
        sizes = [1, 17, 64, 5]
        cases = []
        for it, n in enumerate(sizes):   # inputs and the CPU oracle first: it must not delay a rank between steps
            gi = torch.Generator().manual_seed(100 * it + rank)
            x = torch.randn(n, h, generator=gi).bfloat16()
            logits = torch.randn(n, e, generator=gi)
            tw, ids = ref.moe_route(logits, k, True)
            cases.append((x, tw, ids, ref.moe_forward(x, moe.dense[0], moe.dense[1], tw, ids)))
        for it, (x, tw, ids, want) in enumerate(cases):
            n = x.shape[0]
            ctx.common_tokens = 64 if it % 2 == 0 else 32 if n <= 32 else 64   # the agreed bound of the step
            # the replicas enter a step together (the lock-step loop's host agreement); the device waits
            # are bounded at half a second, which is for a slow peer, not for eight oracle runs sharing the cores
            dist.barrier(group=cpu)
            if rank == world - 1 and it == 1:
                time.sleep(0.05)  # a lagging rank: the peers' waits must simply take longer
            got = ctx.dispatch_compute_combine(moe, x.to(dev), tw.to(dev), ids.to(dev))
            err = float((got.cpu().float() - want.float()).abs().max()) / max(float(want.float().abs().max()), 1e-6)
            if err > tol:
                ok = False
                msgs.append(f"{kind} iteration {it}: relative err {err:.3f}; " + _explain(
                    ref, moe, x, tw, ids, got.cpu().float(), want.float(), tol, e_local))
        # a captured decode step: the exchange replays from device-resident sequence numbers
        ctx.common_tokens = None
        ctx.static_bound = 32
        n = 8 + rank
        gi = torch.Generator().manual_seed(900 + rank)
        x = torch.randn(n, h, generator=gi).bfloat16()
        tw, ids = ref.moe_route(torch.randn(n, e, generator=gi), k, True)
        sx, sw, si = x.to(dev), tw.to(dev), ids.to(dev)
        want = ref.moe_forward(x, moe.dense[0], moe.dense[1], tw, ids)
        s = torch.cuda.Stream()
        dist.barrier(group=cpu)
        with torch.cuda.stream(s):
            ctx.dispatch_compute_combine(moe, sx, sw, si)
            s.synchronize()
            dist.barrier(group=cpu)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=s):
                static_out = ctx.dispatch_compute_combine(moe, sx, sw, si)
            dist.barrier(group=cpu)
            for _ in range(3):
                graph.replay()
            s.synchronize()
        err = float((static_out.cpu().float() - want.float()).abs().max()) / float(want.float().abs().max())
        if err > tol:
            ok = False
            msgs.append(f"{kind} graph replay: relative err {err:.3f}")
        torch.cuda.synchronize()
        if ctx.fused_calls != len(sizes) + 2 or not ctx.check_health():
            ok = False
            msgs.append(f"{kind}: fused_calls={ctx.fused_calls} healthy={ctx.healthy}")
        dist.barrier()
        ctx.close()
    q.put((rank, ok, msgs))
    dist.destroy_process_group()


def _run_ranks(worker, world, port_base, env=None):
    for k, v in (env or {}).items():
        os.environ[k] = v
    try:
        return _run_ranks_inner(worker, world, port_base)
    finally:
        for k in (env or {}):
            os.environ.pop(k, None)


def _run_ranks_inner(worker, world, port_base):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = port_base + os.getpid() % 900 + world
    procs = [ctx.Process(target=worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=420) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    bad = [f"rank {rank} of {world}: {msgs}" for rank, ok, msgs in sorted(results) if not ok]
    assert not bad, "\n".join(bad)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_expert_parallel_exchange(world):
    """Dispatch (16-bit rows, or e4m3 rows with per-token / per-128 scales for fp8 expert stacks),
    owner-side grouped GEMMs, return and gate-weighted combine over peer memory on 2 / 4 / 8 GPUs
    against the fp32 expert oracle, with a lagging rank and a CUDA-graph replay."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run_ranks(_ep_worker, world, 21000)


def _row_shard_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    import math
    import time

    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    cpu = dist.new_group(list(range(world)), backend="gloo")
    from minisglang_rdna4_b200.ops import cuda as K
    from minisglang_rdna4_b200.ops import ref
    from minisglang_rdna4_b200.parallel.symm import SymmetricCollectives
    from minisglang_rdna4_b200.quant.method import ActQ

    comm = SymmetricCollectives(dist.group.WORLD, cpu, dev, rank, world, max_rows=256, max_hidden=4096)
    hidden, k_local, n2 = 1024, 768, 1536
    comm.enable_row_shard(2048, hidden)
    ok, msgs = True, []
    for it, rows in enumerate([512, 2048, 1152, 384]):
        g = torch.Generator(device="cpu").manual_seed(7 * rows + it)
        a_parts = [torch.randn(rows, k_local, generator=g).bfloat16() for _ in range(world)]
        w_parts = [(torch.randn(hidden, k_local, generator=g) / math.sqrt(k_local * world)).bfloat16()
                   for _ in range(world)]
        res0 = torch.randn(rows, hidden, generator=g).bfloat16()
        nw = (1 + 0.1 * torch.randn(hidden, generator=g)).bfloat16()
        w2 = torch.randn(n2, hidden, generator=g) / math.sqrt(hidden)
        w2s = w2.abs().amax(-1) / 448
        w2q = (w2 / w2s[:, None]).to(torch.float8_e4m3fn)
        # fp32 reference of the whole chain
        partials = [(a_parts[r].float() @ w_parts[r].float().t()).bfloat16() for r in range(world)]
        total = sum(p.float() for p in partials)
        want_res = (total + res0.float()).bfloat16()
        want_norm = ref.rms_norm(want_res, nw, 1e-6).float()
        want_y = want_norm @ (w2q.float() * w2s[:, None]).t()

        a = a_parts[rank].to(dev)
        w = w_parts[rank].to(dev)
        res = res0.clone().to(dev)
        if rank == 1 and it == 1:
            time.sleep(0.05)  # a lagging rank: the peers' waits must simply take longer
        for quant in (True, False):
            res.copy_(res0)
            plan = comm.rs_begin(rows, hidden, torch.bfloat16)
            if plan is None:
                ok = False
                msgs.append(f"no plan for rows={rows}")
                break
            K.set_next_gemm_tp(comm.row_shard.gemm_args(plan))
            assert K.gemm(a, w) is None  # nothing is written locally
            qv, sc, ready = comm.row_shard.finish(plan, res, nw.to(dev), 1e-6, quant)
            torch.cuda.synchronize()
            own = torch.arange(rows).view(-1, 128)[rank::world].reshape(-1)  # blocks rank, rank + world, ...
            # the partials come out of a tensor-core GEMM: equal to the fp32 reference up to bf16 rounding
            if own.numel() and float((res.cpu()[own].float() - want_res[own].float()).abs().max()) > 0.05:
                ok = False
                msgs.append(f"owned residual rows differ rows={rows} quant={quant}")
            if quant:
                # all-gather -> GEMM: the consumer waits for the rows block by block
                K.set_next_gemm_tp(ready.gemm_args())
                y = K.gemm_w8a8(qv, sc, w2q.to(dev), w2s.float().to(dev))
                err = float((y.float().cpu() - want_y).abs().max()) / float(want_y.abs().max())
                if err > 0.08:
                    ok = False
                    msgs.append(f"gathered GEMM mismatch rows={rows} err={err:.3f}")
            else:
                comm.wait_ready(ready)
                torch.cuda.synchronize()
                if float((qv.float().cpu() - want_norm).abs().max()) > 0.06:
                    ok = False
                    msgs.append(f"gathered norm mismatch rows={rows}")
            dist.barrier()
    torch.cuda.synchronize()
    if K.gemm_status() != 0:
        ok = False
        msgs.append("a GEMM wait timed out")
    if not comm.check_health():
        ok = False
        msgs.append("a device wait timed out")
    dist.barrier()
    q.put((rank, ok, msgs))
    comm.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_gemm_reduce_scatter_norm_allgather_gemm(world):
    """Row-parallel GEMM whose epilogue pushes partial rows to their owners, the owner-side
    reduce + residual add + RMSNorm (+ e4m3) that stores into every rank, and a column-parallel
    GEMM that waits for the gathered rows per 128-row block, against an fp32 reference, on
    2 / 4 / 8 GPUs."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run_ranks(_row_shard_worker, world, 25000)
