"""Numerics of every sm_100a kernel against the fp32 PyTorch restatement of the same op."""
import math
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from minisglang_rdna4_b200.ops import cuda

    return cuda


def _ref():
    from minisglang_rdna4_b200.ops import ref

    return ref


def _close(a, b, rtol, atol, what=""):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    bad = err > tol
    assert not bool(bad.any()), f"{what}: {int(bad.sum())}/{bad.numel()} off, max err {float(err.max()):.4g}"


# ------------------------------------------------------------------------------------------ elementwise
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_embedding(K, dtype):
    w = torch.randn(1000, 256, device="cuda").to(dtype)
    ids = torch.randint(0, 1000, (77,), device="cuda", dtype=torch.int32)
    assert torch.equal(K.embedding(ids, w), w[ids.long()])
    out = K.embedding(ids, w[:300], 100, 300)
    assert torch.equal(out, _ref().embedding(ids, w[:300], 100, 300))


@pytest.mark.parametrize("hidden", [256, 2560, 8192])
@pytest.mark.parametrize("rows", [1, 7, 300])
def test_rms_norm_family(K, hidden, rows):
    R = _ref()
    torch.manual_seed(hidden + rows)
    x = torch.randn(rows, hidden, device="cuda").bfloat16()
    res = torch.randn(rows, hidden, device="cuda").bfloat16()
    w = (1 + 0.1 * torch.randn(hidden, device="cuda")).bfloat16()
    _close(K.rms_norm(x, w, 1e-6), R.rms_norm(x, w, 1e-6), 1e-2, 1e-2, "rms_norm")
    r1, r2 = res.clone(), res.clone()
    y1 = K.rms_norm_add(x, r1, w, 1e-6)
    y2 = R.rms_norm_add(x, r2, w, 1e-6)
    assert torch.equal(r1, r2)
    _close(y1, y2, 1e-2, 1e-2, "rms_norm_add")
    r1, r2 = res.clone(), res.clone()
    q1, s1 = K.rms_norm_quant(x, w, 1e-6, r1)
    q2, s2 = R.per_token_quant_fp8(R.rms_norm_add(x, r2, w, 1e-6))
    assert torch.equal(r1, r2)
    _close(s1, s2, 1e-2, 0, "scale")
    # a bf16 rounding flip before the quantiser moves a value by one e4m3 step (12.5 % at most)
    _close(q1.float() * s1[:, None], q2.float() * s2[:, None], 0.14, 0.02, "rms_norm_add_quant")
    assert float((q1.float() != q2.float()).float().sum()) <= max(4.0, 0.01 * q1.numel())


def test_act_and_quant(K):
    R = _ref()
    x = torch.randn(130, 2 * 9728, device="cuda").bfloat16()
    _close(K.act_and_mul(x), R.silu_and_mul(x), 1e-2, 1e-2, "silu_and_mul")
    _close(K.act_and_mul(x, "gelu_tanh"), R.gelu_and_mul(x, True), 1e-2, 1e-2, "gelu_tanh")
    q, s = K.silu_and_mul_quant(x)
    q2, s2 = R.per_token_quant_fp8(R.silu_and_mul(x))
    _close(s, s2, 1e-2, 0, "scale")
    _close(q.float() * s[:, None], q2.float() * s2[:, None], 0.14, 0.02, "silu_quant")
    y = torch.randn(33, 4096, device="cuda").bfloat16()
    q, s = K.per_token_quant_fp8(y)
    q2, s2 = R.per_token_quant_fp8(y)
    _close(s, s2, 1e-6, 0, "token scale")
    assert float((q.float() != q2.float()).float().mean()) < 0.01
    q, s = K.per_group_quant_fp8(y, 128)
    q2, s2 = R.per_group_quant_fp8(y, 128)
    _close(s, s2, 1e-6, 0, "group scale")


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("qk_norm", [False, True])
def test_qk_norm_rope_store(K, fp8, qk_norm):
    R = _ref()
    t, hq, hk, d, ps, pages = 37, 8, 2, 128, 16, 12
    qkv = torch.randn(t, (hq + 2 * hk) * d, device="cuda").bfloat16()
    qw = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16() if qk_norm else None
    kw = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16() if qk_norm else None
    pos = torch.randint(0, 500, (t,), device="cuda", dtype=torch.int32)
    cs = R.build_cos_sin_cache(d, 512, 1e6).cuda()
    loc = torch.randperm(pages * ps, device="cuda")[:t].to(torch.int32)
    dt = torch.float8_e4m3fn if fp8 else torch.bfloat16
    pool1 = torch.zeros(2, 1, pages + 1, hk, ps, d, device="cuda", dtype=dt)
    pool2 = torch.zeros_like(pool1)
    ks = (0.5 + torch.rand(hk, device="cuda")) / 40 if fp8 else None
    vs = (0.5 + torch.rand(hk, device="cuda")) / 40 if fp8 else None
    q1 = K.qk_norm_rope_store(qkv, qw, kw, pos, cs, hq, hk, d, d, 1e-6, pool1[0, 0], pool1[1, 0], loc, ks, vs)
    q, k, v = qkv.split([hq * d, hk * d, hk * d], -1)
    q2, k2 = R.qk_norm_rope(q, k, qw, kw, pos, cs, d, d, 1e-6)
    R.store_kv(k2, v, pool2[0, 0], pool2[1, 0], loc, ks, vs)
    _close(q1.view(t, -1), q2, 2e-2, 2e-2, "q")
    if fp8:
        diff = (pool1.float() - pool2.float()).abs()
        assert float((diff > 0).float().mean()) < 0.02  # rounding-boundary flips only
    else:
        _close(pool1, pool2, 2e-2, 2e-2, "kv")
    # stand-alone store
    pool3 = torch.zeros_like(pool1)
    K.store_kv(k2.contiguous(), v.contiguous(), pool3[0, 0], pool3[1, 0], loc, ks, vs)
    assert torch.equal(pool3[1].view(torch.uint8) if fp8 else pool3[1], pool2[1].view(torch.uint8) if fp8 else pool2[1])


# ------------------------------------------------------------------------------------------ GEMM
@pytest.mark.parametrize("m,n,k", [(1, 256, 128), (5, 512, 320), (128, 256, 256), (300, 1024, 2560), (2048, 6144, 2560)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gemm_16bit(K, m, n, k, dtype):
    x = torch.randn(m, k, device="cuda").to(dtype)
    w = (torch.randn(n, k, device="cuda") / math.sqrt(k)).to(dtype)
    for bn in (0, 32, 64, 128, 256):
        y = K.gemm(x, w, bn=bn)
        assert K.gemm_status() == 0
        _close(y, x.float() @ w.float().t(), 2e-2, 2e-2, f"gemm bn={bn}")
    bias = torch.randn(n, device="cuda").to(dtype)
    for bn in (0, 128, 256):
        y32 = K.gemm(x, w, out_dtype=torch.float32, bn=bn)
        _close(y32, x.float() @ w.float().t(), 1e-3, 1e-3, f"gemm f32 out bn={bn}")
        _close(K.gemm(x, w, bias, bn=bn), x.float() @ w.float().t() + bias.float(), 2e-2, 2e-2, f"bias bn={bn}")
    assert K.gemm_status() == 0


@pytest.mark.parametrize("m,n,k", [(640, 1024, 2560), (257, 6144, 512), (4096, 2560, 9728)])
def test_gemm_pair_kernel_matches_single_cta(K, m, n, k):
    """The 256 x 256 CTA-pair tiles and the 128-wide single-CTA tiles accumulate every output
    over the same K order in fp32, so the two kernels agree to the last bit."""
    x = torch.randn(m, k, device="cuda").bfloat16()
    w = (torch.randn(n, k, device="cuda") / math.sqrt(k)).bfloat16()
    single = K.gemm(x, w, bn=128)
    pair = K.gemm(x, w, bn=256)
    assert K.gemm_status() == 0
    _close(pair, x.float() @ w.float().t(), 2e-2, 2e-2, "pair vs fp32")
    assert torch.equal(pair, single)
    prev = K.gemm_pair_mode(1)
    try:
        assert torch.equal(K.gemm(x, w), single)
    finally:
        K.gemm_pair_mode(prev)


def test_gemm_m_invariance(K):
    x = torch.randn(64, 2560, device="cuda").bfloat16()
    w = (torch.randn(4096, 2560, device="cuda") / 50).bfloat16()
    full = K.gemm(x, w)
    for m in (1, 5, 17):
        assert torch.equal(K.gemm(x[:m].contiguous(), w), full[:m])


@pytest.mark.parametrize("m,n,k", [(1, 256, 128), (7, 512, 384), (256, 2560, 4096), (1000, 1024, 2560)])
def test_gemm_w8a8(K, m, n, k):
    R = _ref()
    x = torch.randn(m, k, device="cuda").bfloat16()
    w = torch.randn(n, k, device="cuda") / math.sqrt(k)
    ws = w.abs().amax(-1) / 448
    wq = (w / ws[:, None]).to(torch.float8_e4m3fn)
    xq, xs = K.per_token_quant_fp8(x)
    for bn in (0, 32, 64, 128, 256):
        y = K.gemm_w8a8(xq, xs, wq, ws.float(), bn=bn)
        assert K.gemm_status() == 0
        _close(y, R.gemm_w8a8(xq, xs, wq, ws), 2e-2, 2e-2, f"w8a8 bn={bn}")


@pytest.mark.parametrize("m,n,k", [(1, 128, 128), (9, 256, 256), (256, 2560, 4096), (700, 6144, 2560), (64, 320, 1024),
                                   (2100, 2560, 9728)])
def test_gemm_w4a8_mxfp4(K, m, n, k):
    R = _ref()
    from minisglang_rdna4_b200.quant import mxfp4

    x = torch.randn(m, k, device="cuda").bfloat16()
    w = torch.randn(n, k, device="cuda") * 0.02
    packed, sf = mxfp4.quantize_mxfp4(w)
    atoms = mxfp4.pack_sf_atoms(sf)
    assert torch.equal(mxfp4.unpack_sf_atoms(atoms, n, k // 32), sf)
    xq, xs = K.per_token_quant_fp8(x)
    want = R.gemm_w4a8_mxfp4(xq, xs, packed, sf)
    for bn in (128, 64, 0, 256):
        y = K.gemm_w4a8_mxfp4(xq, xs, packed, atoms, bn=bn)
        assert K.gemm_status() == 0
        _close(y, want, 2e-2, 2e-2, f"mxfp4 bn={bn}")


# ------------------------------------------------------------------------------------------ attention
def _attn_case(K, fp8, b, q_lens, kv_lens, hq, hk, d, ps, causal=True, window=0, mask=False, dtype=torch.bfloat16,
               splits=None, tc=None):
    R = _ref()
    torch.manual_seed(0)
    pages = sum(-(-n // ps) for n in kv_lens) + 3
    dt = torch.float8_e4m3fn if fp8 else dtype
    pool = (torch.randn(2, 1, pages + 1, hk, ps, d, device="cuda") * (8 if fp8 else 1)).to(dt)
    perm = torch.randperm(pages, device="cuda").to(torch.int32)
    maxp = max(-(-n // ps) for n in kv_lens)
    bt = torch.zeros(b, maxp, dtype=torch.int32, device="cuda")
    off = 0
    for i, n in enumerate(kv_lens):
        np_ = -(-n // ps)
        bt[i, :np_] = perm[off : off + np_]
        off += np_
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device="cuda")
    sl = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
    t = int(cu[-1])
    q = torch.randn(t, hq, d, device="cuda").to(dtype)
    ks = (0.5 + torch.rand(hk, device="cuda")) / 8 if fp8 else None
    vs = (0.5 + torch.rand(hk, device="cuda")) / 8 if fp8 else None
    m = None
    if mask:
        m = torch.where(torch.rand(t, max(kv_lens), device="cuda") < 0.7, 0.0, float("-inf")).float()
        m[:, 0] = 0.0
    scale = d ** -0.5
    out = K.paged_attention(q, pool[0, 0], pool[1, 0], bt, cu, sl, scale, causal=causal, window=window, mask=m,
                            k_scale=ks, v_scale=vs, max_q=max(q_lens), max_kv=max(kv_lens), splits=splits, tc=tc)
    assert K.attn_status() == 0
    want = R.paged_attention(q, pool[0, 0], pool[1, 0], bt, cu, sl, scale, causal, window, m, ks, vs)
    _close(out, want, 3e-2, 3e-2, f"attention fp8={fp8}")


@pytest.mark.parametrize("fp8", [False, True])
def test_attention_decode(K, fp8):
    _attn_case(K, fp8, 5, [1] * 5, [1, 17, 64, 333, 1500], 8, 2, 128, 16)
    _attn_case(K, fp8, 3, [1] * 3, [700, 65, 2048], 32, 8, 128, 16, splits=4)
    _attn_case(K, fp8, 2, [1] * 2, [100, 257], 8, 1, 128, 64, splits=2)


@pytest.mark.parametrize("fp8", [False, True])
def test_attention_prefill_and_extend(K, fp8):
    _attn_case(K, fp8, 3, [5, 130, 64], [5, 130, 64], 8, 2, 128, 16)           # pure prefill
    _attn_case(K, fp8, 3, [7, 33, 100], [200, 33, 1000], 16, 4, 128, 16)       # extend over a cached prefix
    _attn_case(K, fp8, 2, [40, 9], [300, 90], 8, 8, 128, 32, window=64)        # sliding window, MHA
    _attn_case(K, fp8, 2, [5, 5], [77, 300], 8, 2, 128, 16, mask=True)         # tree-mask verify
    _attn_case(K, fp8, 2, [20, 12], [20, 50], 8, 2, 128, 16, causal=False)     # bidirectional


@pytest.mark.parametrize("fp8", [False, True])
def test_attention_decode_kernels_agree(K, fp8):
    """The transposed decode kernel and the general kernel are two code paths for the same math."""
    try:
        K.force_general_decode_attention(True)
        _attn_case(K, fp8, 4, [1] * 4, [50, 700, 64, 1333], 32, 8, 128, 16)
        _attn_case(K, fp8, 3, [1] * 3, [300, 20, 901], 8, 1, 128, 16, splits=3)     # group of 8
        _attn_case(K, fp8, 2, [1] * 2, [400, 100], 8, 2, 128, 16, window=128)
    finally:
        K.force_general_decode_attention(False)
    _attn_case(K, fp8, 3, [1] * 3, [300, 20, 901], 8, 1, 128, 16, splits=3)
    _attn_case(K, fp8, 2, [1] * 2, [400, 100], 8, 2, 128, 16, window=128)
    _attn_case(K, fp8, 2, [1] * 2, [400, 100], 16, 16, 128, 16)                     # MHA, group of 1


def test_attention_head_dim_64_and_fp16(K):
    _attn_case(K, False, 2, [9, 1], [40, 200], 4, 2, 64, 16)
    _attn_case(K, False, 2, [9, 1], [40, 200], 8, 2, 128, 16, dtype=torch.float16)


# ------------------------------------------------------------------------------------------ sampling
def test_argmax_and_sampling(K):
    R = _ref()
    logits = torch.randn(9, 151936, device="cuda")
    assert torch.equal(K.argmax(logits), logits.argmax(-1).int())
    sub = logits[:, :1000]  # strided rows
    assert torch.equal(K.argmax(sub), sub.argmax(-1).int())
    # sampling: the kept set must match the reference's and the draw must follow the distribution
    lg = torch.randn(4, 4096, device="cuda") * 3
    temps = torch.tensor([0.0, 0.7, 1.0, 1.3], device="cuda")
    top_k = torch.tensor([0, 20, 0, 50], device="cuda", dtype=torch.int32)
    top_p = torch.tensor([1.0, 1.0, 0.9, 0.8], device="cuda")
    counts = torch.zeros(4, 4096, device="cuda")
    n = 400
    for i in range(n):
        u = torch.rand(4, device="cuda")
        tok = K.sample(lg, temps, top_k, top_p, None, uniform=u)
        counts[torch.arange(4), tok.long()] += 1
    assert int(counts[0].argmax()) == int(lg[0].argmax()) and counts[0].max() == n
    probs = torch.softmax(lg / temps.clamp_min(1e-6)[:, None], -1)
    sp, si = probs.sort(-1, descending=True)
    for r in (1, 2, 3):
        keep = torch.ones(4096, dtype=torch.bool, device="cuda")
        if top_k[r] > 0:
            keep &= torch.arange(4096, device="cuda") < top_k[r]
        keep &= (sp[r].cumsum(0) - sp[r]) <= top_p[r]
        allowed = torch.zeros(4096, dtype=torch.bool, device="cuda")
        allowed[si[r][keep]] = True
        assert counts[r][~allowed].sum() == 0, f"row {r} drew a filtered token"
        assert counts[r][si[r][0]] > 0


# ------------------------------------------------------------------------------------------ MoE
@pytest.mark.parametrize("tokens,E,k", [(1, 8, 2), (37, 64, 4), (300, 128, 8)])
def test_moe_route_and_forward(K, tokens, E, k):
    R = _ref()
    from minisglang_rdna4_b200.ops import moe_kernels as MK

    h, inter = 256, 128
    logits = torch.randn(tokens, E, device="cuda")
    w, ids = MK.moe_route(logits, k, True)
    w2_, ids2 = R.moe_route(logits, k, True)
    assert torch.equal(ids.sort(-1).values, ids2.sort(-1).values)
    _close(w.sort(-1).values, w2_.sort(-1).values, 1e-4, 1e-6, "route weights")
    ws, _ = MK.moe_route(logits, k, False, scoring="sigmoid", scale=2.5)
    wr, _ = R.moe_route(logits, k, False, "sigmoid", None, 2.5)
    _close(ws.sort(-1).values, wr.sort(-1).values, 1e-4, 1e-6, "sigmoid weights")
    # selection bias: experts chosen by score + bias, weighted by the score; per-expert counts
    bias = torch.randn(E, device="cuda") * 0.3
    counts = torch.empty(E, dtype=torch.int32, device="cuda")
    wb, ib = MK.moe_route(logits, k, True, scoring="sigmoid", scale=1.8, bias=bias, counts=counts)
    wbr, ibr = R.moe_route(logits, k, True, "sigmoid", bias, 1.8)
    assert torch.equal(ib.sort(-1).values, ibr.sort(-1).values)
    _close(wb.sort(-1).values, wbr.sort(-1).values, 1e-4, 1e-6, "biased route weights")
    assert torch.equal(counts.long(), torch.bincount(ib.reshape(-1).long(), minlength=E))
    x = torch.randn(tokens, h, device="cuda").bfloat16()
    w13 = (torch.randn(E, 2 * inter, h, device="cuda") * 0.05).bfloat16()
    w2 = (torch.randn(E, h, inter, device="cuda") * 0.05).bfloat16()
    got = MK.moe_forward(x, w13, w2, w, ids)
    assert K.gemm_status() == 0
    want = R.moe_forward(x, w13, w2, w, ids)
    _close(got, want, 3e-2, 3e-2, "moe_forward")
    # expert-parallel slice: only experts [E/2, E) are local
    half = E // 2
    got_ep = MK.moe_forward(x, w13[half:].contiguous(), w2[half:].contiguous(), w, ids, expert_offset=half)
    want_ep = R.moe_forward(x, w13[half:], w2[half:], w, ids, expert_offset=half)
    _close(got_ep, want_ep, 3e-2, 3e-2, "moe_forward ep")


def test_moe_forward_w4a8_mxfp4(K):
    """Expert MLPs with e2m1 weights and e4m3 activations (grouped block-scaled GEMMs) against the
    16-bit expert path run on the de-quantised weights."""
    from minisglang_rdna4_b200.ops import moe_kernels as MK
    from minisglang_rdna4_b200.quant import mxfp4

    R = _ref()
    torch.manual_seed(0)
    tokens, E, k, h, inter = 150, 16, 4, 512, 256
    x = torch.randn(tokens, h, device="cuda").bfloat16()
    logits = torch.randn(tokens, E, device="cuda").bfloat16()
    w, ids = MK.moe_route(logits, k, True)

    def enc(wt):
        e, n, kk = wt.shape
        packed, sf = mxfp4.quantize_mxfp4(wt.reshape(e * n, kk))
        deq = mxfp4.dequant_mxfp4(packed, sf).view(e, n, kk).bfloat16()
        atoms = torch.stack([mxfp4.pack_sf_atoms(sf[i * n:(i + 1) * n]) for i in range(e)]).contiguous()
        return packed.view(e, n, kk // 2).contiguous(), atoms, deq

    p13, a13, d13 = enc(torch.randn(E, 2 * inter, h, device="cuda") * 0.05)
    p2, a2, d2 = enc(torch.randn(E, h, inter, device="cuda") * 0.05)
    got = MK.moe_forward_w4a8(x, p13, a13, p2, a2, w, ids)
    assert K.gemm_status() == 0
    want = R.moe_forward(x, d13, d2, w, ids)
    err = float((got.float() - want.float()).abs().max()) / float(want.float().abs().max())
    assert err < 0.08, err


@pytest.mark.parametrize("n,k", [(2560, 4096), (2560, 9728), (1024, 2048)])
def test_gemm_split_k_small_m(K, n, k, monkeypatch):
    """Small-M GEMMs whose tiles would leave most SMs idle split K over several CTAs. The plan
    depends on (N, K) only, so a row's result is the same at every M up to 256, and the sum of the
    K ranges is taken in a fixed order (repeatable bit for bit)."""
    R = _ref()
    from minisglang_rdna4_b200.ops._lib import lib
    from minisglang_rdna4_b200.quant import mxfp4

    splits = lib().msgl_gemm_splitk_plan(3, n, k)
    x = torch.randn(200, k, device="cuda").bfloat16()
    w = torch.randn(n, k, device="cuda") * 0.02
    packed, sf = mxfp4.quantize_mxfp4(w)
    atoms = mxfp4.pack_sf_atoms(sf)
    xq, xs = K.per_token_quant_fp8(x)
    want = R.gemm_w4a8_mxfp4(xq, xs, packed, sf)
    monkeypatch.setattr(K, "SPLIT_K", True)               # off by default (experimental)
    y = K.gemm_w4a8_mxfp4(xq, xs, packed, atoms)          # split-K when the plan says so
    assert K.gemm_status() == 0
    _close(y, want, 2e-2, 2e-2, f"split-k mxfp4 (splits={splits})")
    assert torch.equal(y, K.gemm_w4a8_mxfp4(xq, xs, packed, atoms))            # repeatable
    for m in (1, 7, 130):
        assert torch.equal(K.gemm_w4a8_mxfp4(xq[:m].contiguous(), xs[:m].contiguous(), packed, atoms), y[:m])
    xb = torch.randn(96, k, device="cuda").bfloat16()
    wb = w.bfloat16()
    bias = torch.randn(n, device="cuda").bfloat16()
    _close(K.gemm(xb, wb, bias), xb.float() @ wb.float().t() + bias.float(), 2e-2, 2e-2, "split-k bf16 + bias")
    _close(K.gemm(xb, wb, out_dtype=torch.float32), xb.float() @ wb.float().t(), 2e-3, 2e-3, "split-k f32 out")
    assert K.gemm_status() == 0


@pytest.mark.parametrize("m", [5, 200, 700])
def test_gemm_w4a8_mxfp4_k_not_multiple_of_128(K, m):
    """A row-parallel shard can leave K = 1216 (9.5 blocks of 128): the 4-bit rows are padded with
    zero codes to whole blocks, the activation keeps its own K and TMA zero-fills its last block."""
    R = _ref()
    from minisglang_rdna4_b200.quant import mxfp4

    n, k = 2560, 1216
    x = torch.randn(m, k, device="cuda").bfloat16()
    w = torch.randn(n, k, device="cuda") * 0.02
    packed, sf = mxfp4.quantize_mxfp4(w)
    atoms = mxfp4.pack_sf_atoms(sf)
    padded = torch.nn.functional.pad(packed, (0, (1280 - k) // 2))
    xq, xs = K.per_token_quant_fp8(x)
    want = R.gemm_w4a8_mxfp4(xq, xs, packed, sf)
    for bn in (0, 128, 256):
        y = K.gemm_w4a8_mxfp4(xq, xs, padded, atoms, bn=bn)
        assert K.gemm_status() == 0
        _close(y, want, 2e-2, 2e-2, f"mxfp4 K=1216 bn={bn}")


@pytest.mark.parametrize("fp8", [False, True])
def test_attention_prefill_tcgen05(K, fp8):
    """The tensor-core prefill kernel (gather to a dense scratch + tcgen05 QK^T / PV) against the fp32
    reference on ragged prefill / extend batches, against the general kernel, and bit for bit
    against itself when a prompt is processed in two chunks."""
    K.LEDGER.pop("prefill_attention", None)
    _attn_case(K, fp8, 3, [5, 130, 64], [5, 130, 64], 8, 2, 128, 16, tc=True)
    assert K.LEDGER.get("prefill_attention") == "attn_prefill_tc_kernel"
    _attn_case(K, fp8, 3, [7, 33, 100], [200, 33, 1000], 16, 4, 128, 16, tc=True)
    _attn_case(K, fp8, 4, [1365, 257, 128, 1], [1365, 300, 128, 513], 32, 8, 128, 16, tc=True)
    _attn_case(K, fp8, 2, [300, 40], [300, 700], 8, 4, 128, 64, dtype=torch.float16, tc=True)

    torch.manual_seed(1)
    hq, hk, d, ps, n, cut = 8, 2, 128, 16, 700, 300
    dt = torch.float8_e4m3fn if fp8 else torch.bfloat16
    pages = -(-n // ps)
    pool = (torch.randn(2, 1, pages + 1, hk, ps, d, device="cuda") * (8 if fp8 else 1)).to(dt)
    bt = torch.randperm(pages, device="cuda").to(torch.int32).view(1, pages)
    q = torch.randn(n, hq, d, device="cuda").bfloat16()
    ks = (0.5 + torch.rand(hk, device="cuda")) / 8 if fp8 else None
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    run = lambda qq, ql, kl, **kw: K.paged_attention(qq, pool[0, 0], pool[1, 0], bt, i32([0, ql]), i32([kl]),
                                                     d ** -0.5, k_scale=ks, v_scale=ks, max_q=ql, max_kv=kl, **kw)
    whole = run(q, n, n, tc=True)
    first = run(q[:cut].contiguous(), cut, cut, tc=True)
    second = run(q[cut:].contiguous(), n - cut, n, tc=True)
    assert torch.equal(whole[:cut], first) and torch.equal(whole[cut:], second)
    general = run(q, n, n, tc=False)
    _close(whole, general, 3e-2, 3e-2, "tcgen05 vs general prefill kernel")
    assert K.attn_status() == 0


@pytest.mark.parametrize("n,k", [(2560, 9728), (2560, 4096)])
def test_gemm_split_k_planes_feed_the_fused_norm(K, n, k):
    """Decode-step row-parallel projections: the GEMM leaves its K ranges as fp32 planes (bias in
    plane 0) and the following residual-add + RMSNorm (+ e4m3 producer) sums them in ascending
    order. Against the fp32 reference of GEMM -> add -> norm, repeatable, and the same rows at
    every M."""
    R = _ref()
    from minisglang_rdna4_b200.ops._lib import lib
    from minisglang_rdna4_b200.quant import mxfp4

    assert lib().msgl_gemm_splitk_plan(3, n, k) > 1
    torch.manual_seed(0)
    m = 200
    x = torch.randn(m, k, device="cuda").bfloat16()
    w = torch.randn(n, k, device="cuda") * 0.02
    packed, sf = mxfp4.quantize_mxfp4(w)
    atoms = mxfp4.pack_sf_atoms(sf)
    xq, xs = K.per_token_quant_fp8(x)
    bias = torch.randn(n, device="cuda").bfloat16()
    res0 = torch.randn(m, n, device="cuda").bfloat16()
    nw = (1 + 0.1 * torch.randn(n, device="cuda")).bfloat16()

    K.set_next_gemm_planes(True)
    part = K.gemm_w4a8_mxfp4(xq, xs, packed, atoms, bias=bias)
    assert isinstance(part, K.SplitPartial) and part.planes.shape[1:] == (m, n)
    assert isinstance(K.gemm_w4a8_mxfp4(xq, xs, packed, atoms), torch.Tensor)      # the request is used up
    want_y = R.gemm_w4a8_mxfp4(xq, xs, packed, sf).float() + bias.float()
    _close(part.materialise(), want_y, 2e-2, 2e-2, "sum of the split-k planes")

    res = res0.clone()
    normed = K.rms_norm_planes(part, res, nw, 1e-6)
    want_res = (want_y.bfloat16().float() + res0.float())
    _close(res, want_res, 3e-2, 3e-2, "residual after planes add")
    want_norm = R.rms_norm(want_res.bfloat16(), nw, 1e-6)
    _close(normed, want_norm, 4e-2, 4e-2, "norm of planes + residual")
    res_q = res0.clone()
    q, s = K.rms_norm_planes(part, res_q, nw, 1e-6, quant=True)
    assert torch.equal(res_q, res)
    _close(q.float() * s[:, None], want_norm.float(), 8e-2, 8e-2, "quantised norm of planes + residual")

    for mm in (1, 130):
        K.set_next_gemm_planes(True)
        sub = K.gemm_w4a8_mxfp4(xq[:mm].contiguous(), xs[:mm].contiguous(), packed, atoms, bias=bias)
        assert torch.equal(sub.planes, part.planes[:, :mm])
    assert K.gemm_status() == 0


# ------------------------------------------------------------------------------------------ block-scaled fp8
def _quant_blocks(w, bn=128, bk=128):
    n, k = w.shape
    npad, kpad = -(-n // bn) * bn, -(-k // bk) * bk
    wp = torch.zeros(npad, kpad, device=w.device)
    wp[:n, :k] = w
    blocks = wp.view(npad // bn, bn, kpad // bk, bk)
    scale = blocks.abs().amax((1, 3)).clamp_min(1e-8) / 448.0
    q = (blocks / scale[:, None, :, None]).view(npad, kpad)[:n, :k].to(torch.float8_e4m3fn).contiguous()
    return q, scale.float().contiguous()


@pytest.mark.parametrize("m,n,k", [(1, 384, 768), (130, 2048, 512), (300, 1536, 2048), (257, 136, 384)])
def test_gemm_fp8_block(K, m, n, k):
    """128 x 128 weight blocks times 1 x 128 activation groups against the fp32 restatement; a
    row's result does not depend on how many rows are multiplied with it."""
    R = _ref()
    torch.manual_seed(m + n + k)
    x = torch.randn(m, k, device="cuda").bfloat16()
    # groups with very different magnitudes make the per-block promotion matter
    x[:, : k // 2] *= 8.0
    w = torch.randn(n, k, device="cuda") * 0.05
    w[: n // 2] *= 4.0
    wq, ws = _quant_blocks(w)
    xq, xs = K.per_group_quant_fp8(x, 128)
    got = K.gemm_fp8_block(xq, xs, wq, ws, torch.bfloat16)
    assert K.gemm_fp8_block_status() == 0
    want = R.gemm_fp8_block(xq, xs, wq, ws, 128, torch.float32)
    _close(got, want, 1e-2, 1e-2 * float(want.abs().max()), "gemm_fp8_block")
    got32 = K.gemm_fp8_block(xq, xs, wq, ws, torch.float32)
    _close(got32, want, 2e-3, 2e-3 * float(want.abs().max()), "gemm_fp8_block fp32")
    one = K.gemm_fp8_block(xq[-1:].contiguous(), xs[-1:].contiguous(), wq, ws, torch.float32)
    assert torch.equal(one[0], got32[-1])


def test_moe_forward_fp8_kinds(K):
    """Expert MLPs on block-scaled and per-channel fp8 expert stacks (grouped GEMMs), with experts
    that receive no token and experts whose rows do not fill a tile, against the 16-bit expert path
    on the de-quantised weights."""
    from minisglang_rdna4_b200.ops import moe_kernels as MK

    R = _ref()
    torch.manual_seed(3)
    tokens, E, k, h, inter = 150, 16, 4, 512, 256
    x = torch.randn(tokens, h, device="cuda").bfloat16()
    logits = torch.randn(tokens, E, device="cuda")
    logits[:, 5] = -1e9      # expert 5 never selected
    logits[:3, 7] = 1e9      # and expert 7 by few rows only
    logits[3:, 7] = -1e9
    w, ids = MK.moe_route(logits, k, True)
    w13 = torch.randn(E, 2 * inter, h, device="cuda") * 0.05
    w2 = torch.randn(E, h, inter, device="cuda") * 0.05

    def blk(wt):
        qs, ss = zip(*[_quant_blocks(wt[e]) for e in range(wt.shape[0])])
        q, s = torch.stack(qs).contiguous(), torch.stack(ss).contiguous()
        deq = q.float() * s.repeat_interleave(128, 1).repeat_interleave(128, 2)
        return q, s, deq.bfloat16()

    def chan(wt):
        s = wt.abs().amax(-1).clamp_min(1e-8) / 448.0
        q = (wt / s[..., None]).to(torch.float8_e4m3fn).contiguous()
        return q, s.float().contiguous(), (q.float() * s[..., None]).bfloat16()

    for kind, enc in (("fp8_block", blk), ("fp8_channel", chan)):
        q13, s13, d13 = enc(w13)
        q2, s2, d2 = enc(w2)
        got = MK.moe_forward_quant(kind, x, (q13, s13, q2, s2), w, ids)
        assert K.gemm_status() == 0 and K.gemm_fp8_block_status() == 0
        want = R.moe_forward(x, d13, d2, w, ids)
        err = float((got.float() - want.float()).abs().max()) / float(want.float().abs().max())
        assert err < 0.06, (kind, err)
    # the fused SiLU·mul + 1 x 128 quantiser against the two-step form
    hcur = torch.randn(77, 2 * inter, device="cuda").bfloat16()
    q, s = K.silu_and_mul_quant_group(hcur)
    q0, s0 = K.per_group_quant_fp8(K.act_and_mul(hcur), 128)
    _close(s, s0, 1e-3, 0, "group scales")
    _close(q.float() * s.repeat_interleave(128, 1), q0.float() * s0.repeat_interleave(128, 1), 0.13, 1e-3, "group q")


def test_spec_accept_kernel_matches_the_host_rules(K):
    """On-device acceptance, EOS / length truncation and commit against ``spec.accept``."""
    import ctypes

    from minisglang_rdna4_b200.ops._lib import check, lib
    from minisglang_rdna4_b200.spec.accept import accept_greedy, eos_truncate
    from minisglang_rdna4_b200.spec.device import _bind

    _bind()
    g = torch.Generator().manual_seed(0)
    B, W, msl = 37, 5, 64
    pool = torch.randint(0, 50, (B + 1, msl), generator=g, dtype=torch.int32)
    target = torch.randint(0, 6, (B, W), generator=g, dtype=torch.int32)
    c = torch.randint(3, 40, (B,), generator=g)
    k = torch.randint(0, W, (B,), generator=g)
    max_emit = torch.randint(1, 7, (B,), generator=g)
    ignore = torch.randint(0, 2, (B,), generator=g)
    for b in range(B):  # make some drafts stand
        good = int(torch.randint(0, W, (1,), generator=g))
        pool[b, c[b] + 1: c[b] + 1 + good] = target[b, :good]
    eos = [3, 4]
    want_pool = pool.clone()
    want = []
    for b in range(B):
        drafts = pool[b, c[b] + 1: c[b] + 1 + int(k[b])].tolist()
        em = accept_greedy(target[b].tolist(), drafts)
        em = em[: max(1, min(len(em), int(max_emit[b])))]
        em, hit = eos_truncate(em, set(eos), bool(ignore[b]))
        want.append((len(em), int(hit), em))
        want_pool[b, c[b] + 1: c[b] + 1 + len(em)] = torch.tensor(em, dtype=torch.int32)
    dev = "cuda"
    d_pool = pool.to(dev)
    rec = torch.zeros(B * (W + 2), dtype=torch.int32, device=dev)
    sel = torch.zeros(B, dtype=torch.int32, device=dev)
    first = (torch.arange(B) * msl + c + 1).to(torch.int32).to(dev)
    eos_arr = (ctypes.c_int * 8)(*(eos + [-1] * 6))
    d_target, d_k = target.to(dev), k.to(torch.int32).to(dev)
    d_emit, d_flags = max_emit.to(torch.int32).to(dev), ignore.to(torch.int32).to(dev)
    check(lib().msgl_spec_accept(d_target.data_ptr(), d_pool.data_ptr(), first.data_ptr(), d_k.data_ptr(),
                                 d_emit.data_ptr(), d_flags.data_ptr(), rec.data_ptr(), sel.data_ptr(), eos_arr,
                                 2, B, W, torch.cuda.current_stream().cuda_stream), "spec_accept")
    torch.cuda.synchronize()
    rec = rec.cpu().view(B, W + 2)
    for b, (n, hit, em) in enumerate(want):
        assert int(rec[b, 0]) == n and int(rec[b, 1]) == hit and rec[b, 2:2 + n].tolist() == em, b
        assert int(sel[b]) == b * W + n - 1
    assert torch.equal(d_pool.cpu(), want_pool)


def test_spec_accept_tree_kernel_follows_the_target_down_the_tree(K):
    """Tree acceptance (chain + siblings per depth): emitted tokens, EOS / length truncation, commit,
    the K/V move of an accepted sibling and the feature rows of the draft update, against a plain
    restatement of the rule."""
    import ctypes

    from minisglang_rdna4_b200.ops._lib import check, lib
    from minisglang_rdna4_b200.spec.device import _bind

    _bind()
    g = torch.Generator().manual_seed(1)
    B, Kd, T, msl, Bmax = 41, 3, 4, 64, 48
    R = 1 + Kd * T
    pool = torch.randint(0, 50, (B + 1, msl), generator=g, dtype=torch.int32)
    target = torch.randint(0, 7, (B, R), generator=g, dtype=torch.int32)
    sib = torch.randint(0, 7, (Kd, Bmax, T - 1), generator=g, dtype=torch.int32)
    c = torch.randint(3, 40, (B,), generator=g)
    k = torch.where(torch.rand(B, generator=g) < 0.2, 0, Kd)
    max_emit = torch.randint(1, 7, (B,), generator=g)
    ignore = torch.randint(0, 2, (B,), generator=g)
    out_loc = torch.randint(0, 10_000, (B, R), generator=g, dtype=torch.int32)
    eos = [5]
    for b in range(B):     # some chain drafts stand: draft at depth d is the prediction of the node above it
        good = int(torch.randint(0, Kd + 1, (1,), generator=g))
        for d in range(1, good + 1):
            pool[b, c[b] + d] = target[b, d - 1]
    want_pool = pool.clone()
    want = []
    for b in range(B):
        em, hit, cur, mv, frow = [], 0, 0, (-1, -1), [b * R + j for j in range(Kd + 1)]
        limit = max(int(max_emit[b]), 1)
        for d in range(1, Kd + 2):
            p = int(target[b, cur])
            em.append(p)
            if not ignore[b] and p in eos:
                hit = 1
                break
            if len(em) >= limit or d > int(k[b]):
                break
            if int(pool[b, c[b] + d]) == p:
                cur = d
                continue
            cands = sib[d - 1, b].tolist()
            if p not in cands:
                break
            row = Kd + (d - 1) * (T - 1) + cands.index(p) + 1
            mv = (int(out_loc[b, row]), int(out_loc[b, d]))
            frow[d] = b * R + row
            p2 = int(target[b, row])
            em.append(p2)
            if not ignore[b] and p2 in eos:
                hit = 1
            break
        want.append((em, hit, mv, frow))
        want_pool[b, c[b] + 1: c[b] + 1 + len(em)] = torch.tensor(em, dtype=torch.int32)
    dev = "cuda"
    d_pool = pool.to(dev)
    rec = torch.zeros(B * (Kd + 3), dtype=torch.int32, device=dev)
    sel = torch.zeros(B, dtype=torch.int32, device=dev)
    frow_d = torch.zeros(B * (Kd + 1), dtype=torch.int32, device=dev)
    moves = torch.zeros(B * 2, dtype=torch.int32, device=dev)
    first = (torch.arange(B) * msl + c + 1).to(torch.int32).to(dev)
    eos_arr = (ctypes.c_int * 8)(*(eos + [-1] * 7))
    keep = [target.to(dev), k.to(torch.int32).to(dev), max_emit.to(torch.int32).to(dev), ignore.to(torch.int32).to(dev),
            sib.to(dev), out_loc.to(dev)]
    check(lib().msgl_spec_accept_tree(keep[0].data_ptr(), d_pool.data_ptr(), first.data_ptr(), keep[1].data_ptr(),
                                      keep[2].data_ptr(), keep[3].data_ptr(), keep[4].data_ptr(), keep[5].data_ptr(),
                                      rec.data_ptr(), sel.data_ptr(), frow_d.data_ptr(), moves.data_ptr(), eos_arr, 1, B,
                                      Kd, T, Bmax, torch.cuda.current_stream().cuda_stream), "spec_accept_tree")
    torch.cuda.synchronize()
    rec = rec.cpu().view(B, Kd + 3)
    accepted_sibling = 0
    for b, (em, hit, mv, frow) in enumerate(want):
        n = len(em)
        assert int(rec[b, 0]) == n and int(rec[b, 1]) == hit and rec[b, 2:2 + n].tolist() == em, (b, rec[b], em)
        assert int(sel[b]) == b * (Kd + 1) + n - 1
        assert tuple(moves.cpu()[2 * b:2 * b + 2].tolist()) == mv, b
        assert frow_d.cpu()[b * (Kd + 1):(b + 1) * (Kd + 1)].tolist() == frow, b
        accepted_sibling += mv[0] >= 0
    assert accepted_sibling >= 3                       # the case this kernel exists for did occur
    assert torch.equal(d_pool.cpu(), want_pool)


def test_windowed_tree_mask_equals_the_full_mask(K):
    """A mask that covers only the last R K/V positions of each request gives the same result as the
    full-length additive mask with zeros in front of it, and as the fp32 restatement."""
    from minisglang_rdna4_b200.ops import ref

    torch.manual_seed(5)
    hq, hk, d, ps, R = 8, 2, 128, 16, 9
    kv_lens = [40, 9, 133, 77]
    b = len(kv_lens)
    pages = sum(-(-n // ps) for n in kv_lens)
    pool = torch.randn(2, 1, pages + 1, hk, ps, d, device="cuda").bfloat16()
    maxp = max(-(-n // ps) for n in kv_lens)
    bt = torch.zeros(b, maxp, dtype=torch.int32, device="cuda")
    off = 0
    for i, n in enumerate(kv_lens):
        np_ = -(-n // ps)
        bt[i, :np_] = torch.arange(off, off + np_, dtype=torch.int32)
        off += np_
    cu = (torch.arange(b + 1, dtype=torch.int32, device="cuda") * R).contiguous()
    sl = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
    q = torch.randn(b * R, hq, d, device="cuda").bfloat16()
    vis = torch.where(torch.rand(R, R) < 0.5, 0.0, float("-inf"))
    vis[:, 0] = 0.0
    win = vis.repeat(b, 1).contiguous().cuda()
    full = torch.zeros(b * R, max(kv_lens), device="cuda")
    for i, n in enumerate(kv_lens):
        full[i * R:(i + 1) * R, n - R:n] = vis.cuda()
        full[i * R:(i + 1) * R, n:] = float("-inf")
    args = (q, pool[0, 0], pool[1, 0], bt, cu, sl, d ** -0.5)
    a = K.paged_attention(*args, mask=win, mask_window=R, max_q=R, max_kv=max(kv_lens), splits=1)
    f = K.paged_attention(*args, mask=full, max_q=R, max_kv=max(kv_lens), splits=1)
    assert K.attn_status() == 0
    assert torch.equal(a, f)
    o = ref.paged_attention(*args, True, 0, win, None, None, R)
    _close(a.float().cpu(), o.float().cpu(), 2e-2, 2e-2, "windowed mask vs oracle")


def test_attention_head_dim_256(K):
    """256-wide heads (the Qwen3.5 full-attention layers): prefill, extend, decode and a split decode."""
    _attn_case(K, False, 2, [70, 9], [70, 200], 8, 2, 256, 16)
    _attn_case(K, False, 3, [1] * 3, [40, 333, 1200], 8, 2, 256, 16)
    _attn_case(K, False, 2, [1] * 2, [700, 2048], 16, 4, 256, 16, splits=4)


# ------------------------------------------------------------------------------------------ gated delta net
@pytest.mark.parametrize("d", [64, 128])
def test_gated_delta_net_kernels(K, d):
    """Causal convolution with a rolling state, the recurrent gated delta rule with its state matrix
    per (request, head), and the gated RMSNorm against their fp32 restatements: packed sequences of
    different lengths, a request that continues from a stored state, slots in any order."""
    R = _ref()
    torch.manual_seed(d)
    hk, hv, kw = 2, 4, 4
    dk = dv = d
    lens = [1, 37, 130, 1]
    t = sum(lens)
    cdim = 2 * hk * dk + hv * dv
    ncol = cdim + hv * dv + 2 * hv
    proj = (torch.randn(t, (ncol + 7) // 8 * 8, device="cuda") * 0.7).bfloat16()
    w = (torch.randn(cdim, kw, device="cuda") * 0.4).bfloat16()
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    slots = torch.tensor([3, 0, 5, 1], dtype=torch.int32, device="cuda")
    has = torch.tensor([1, 0, 1, 0], dtype=torch.int32, device="cuda")
    conv0 = (torch.randn(6, cdim, kw - 1, device="cuda") * 0.5).bfloat16()
    ssm0 = torch.randn(6, hv, dk, dv, device="cuda") * 0.1
    a_log = torch.log(torch.empty(hv, device="cuda").uniform_(1, 8))
    dt_bias = torch.randn(hv, device="cuda") * 0.3
    # GPU
    conv_g, ssm_g = conv0.clone(), ssm0.clone()
    qkv = K.gdn_conv1d(proj[:, :cdim], w, conv_g, cu, slots, has)
    z = proj[:, cdim:cdim + hv * dv]
    b = proj[:, cdim + hv * dv:cdim + hv * dv + hv]
    a = proj[:, cdim + hv * dv + hv:cdim + hv * dv + 2 * hv]
    o = K.gdn_recurrent(qkv, a, b, a_log, dt_bias, ssm_g, cu, slots, has, hk, hv, dk, dv)
    nw = (1 + 0.1 * torch.randn(dv, device="cuda")).bfloat16()
    y = K.rms_norm_gated(o, z, nw, 1e-6)
    torch.cuda.synchronize()
    # fp32 restatement on the CPU
    conv_c, ssm_c = conv0.cpu().clone(), ssm0.cpu().clone()
    pc = proj.cpu()
    qkv_c = R.causal_conv1d(pc[:, :cdim], w.cpu(), conv_c, cu.cpu(), slots.cpu(), has.cpu())
    _close(qkv.cpu(), qkv_c, 2e-2, 2e-2, "conv1d")
    assert torch.equal(conv_g.cpu()[[3, 0, 5, 1]], conv_c[[3, 0, 5, 1]])
    assert torch.equal(conv_g.cpu()[[2, 4]], conv0.cpu()[[2, 4]])        # untouched slots
    g_c, beta_c = R.gdn_gates(pc[:, cdim + hv * dv + hv:cdim + hv * dv + 2 * hv], pc[:, cdim + hv * dv:cdim + hv * dv + hv],
                              a_log.cpu(), dt_bias.cpu())
    q_c, k_c, v_c = qkv.cpu().split([hk * dk, hk * dk, hv * dv], dim=-1)
    o_c = R.gdn_recurrent(q_c.reshape(t, hk, dk), k_c.reshape(t, hk, dk), v_c.reshape(t, hv, dv), g_c, beta_c, ssm_c,
                          cu.cpu(), slots.cpu(), has.cpu())
    _close(o.cpu(), o_c, 3e-2, 3e-2 * float(o_c.float().abs().max()), "delta rule output")
    _close(ssm_g.cpu(), ssm_c, 1e-3, 1e-3 * float(ssm_c.abs().max()), "recurrent state")
    y_c = R.rms_norm_gated(o.cpu(), pc[:, cdim:cdim + hv * dv].reshape(t, hv, dv), nw.cpu(), 1e-6)
    _close(y.cpu(), y_c, 2e-2, 2e-2, "gated norm")


def test_mamba2_kernels_match_the_oracle(K):
    """Convolution with bias, selective scan (fresh and continued states, grouped B / C), gate-first
    grouped norm and squared ReLU against their fp32 restatements."""
    from minisglang_rdna4_b200.ops import ref as R

    torch.manual_seed(3)
    for h, p, n, g in ((16, 64, 128, 4), (4, 32, 16, 2), (8, 64, 64, 8)):
        inter, cdim = h * p, h * p + 2 * g * n
        lens = [5, 1, 37, 12]
        t, b = sum(lens), len(lens)
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
        slots = torch.tensor([3, 0, 5, 1], dtype=torch.int32, device="cuda")
        has = torch.tensor([0, 1, 1, 0], dtype=torch.int32, device="cuda")
        proj = (torch.randn(t, inter + cdim + h, device="cuda") * 0.5).bfloat16()
        w = (torch.randn(cdim, 4, device="cuda") * 0.3).bfloat16()
        bias = (torch.randn(cdim, device="cuda") * 0.1).bfloat16()
        conv = (torch.randn(6, cdim, 3, device="cuda") * 0.5).bfloat16()
        ssm = torch.randn(6, h, p, n, device="cuda") * 0.3
        a_log = torch.log(torch.empty(h, device="cuda").uniform_(1, 8))
        dsk, dtb = torch.randn(h, device="cuda"), torch.randn(h, device="cuda") * 0.5
        nw = (1 + 0.1 * torch.randn(inter, device="cuda")).bfloat16()
        conv_c, ssm_c = conv.cpu().clone(), ssm.cpu().clone()
        xbc = K.gdn_conv1d(proj[:, inter:inter + cdim], w, conv, cu, slots, has, bias)
        dt = proj[:, inter + cdim:]
        y = K.mamba2_scan(xbc, dt, a_log, dsk, dtb, ssm, cu, slots, has, h, g, p, n, 0.001)
        o = K.rms_norm_gate_first(y.reshape(t, inter), proj[:, :inter], nw, 1e-5, inter // g)
        torch.cuda.synchronize()
        pc = proj.cpu()
        xbc_c = R.causal_conv1d(pc[:, inter:inter + cdim].contiguous(), w.cpu(), conv_c, cu.cpu(), slots.cpu(),
                                has.cpu(), bias.cpu())
        _close(xbc.cpu(), xbc_c, 2e-2, 2e-2, "conv with bias")
        assert torch.equal(conv.cpu(), conv_c)
        xs, bb, cc = xbc.cpu().split([inter, g * n, g * n], dim=-1)     # the kernel's own conv output as input
        y_c = R.mamba2_scan(xs.reshape(t, h, p), pc[:, inter + cdim:], bb.reshape(t, g, n), cc.reshape(t, g, n),
                            a_log.cpu(), dsk.cpu(), dtb.cpu(), ssm_c, cu.cpu(), slots.cpu(), has.cpu(), 0.001)
        _close(y.cpu(), y_c, 3e-2, 3e-2 * float(y_c.float().abs().max()), f"scan output {h, p, n}")
        _close(ssm.cpu(), ssm_c, 1e-3, 1e-3 * float(ssm_c.abs().max()), "scan state")
        o_c = R.rms_norm_gate_first(y.cpu().reshape(t, inter), pc[:, :inter], nw.cpu(), 1e-5, inter // g)
        _close(o.cpu(), o_c, 2e-2, 2e-2, "gate-first norm")
    x = torch.randn(33, 256, device="cuda").bfloat16()
    assert torch.equal(K.relu2(x).cpu(), R.relu2(x.cpu()))


# ------------------------------------------------------------------------------------------ 4-bit-resident GEMM
@pytest.mark.parametrize("m,n,k,group", [(1, 256, 256, 128), (77, 1032, 512, 32), (300, 384, 1024, 64)])
def test_gemm_w4a16_int4_dialects(K, m, n, k, group):
    """AWQ, GPTQ and compressed-tensors int4 checkpoints through the GEMM that keeps the codes 4-bit
    in memory, against the fp32 product with the de-quantised weights; the in-kernel expansion equals
    the load-time expansion bit for bit, so a row does not depend on the batch it is multiplied in."""
    from minisglang_rdna4_b200.quant import int4 as I

    torch.manual_seed(m + n)
    w = torch.randn(n, k) * 0.05
    c, s, z = I.quantize_int4(w, group)
    z = torch.randint(5, 12, z.shape).float()          # asymmetric zero points
    x = torch.randn(m, k, device="cuda").bfloat16()
    dense = I.dequant_int4(c, s, z)
    want = x.float().cpu() @ dense.t()
    checks = []
    qw, sc, qz = I.pack_awq(c, s, z)
    checks.append(("awq", I.awq_to_canonical(qw, sc, qz)))
    qw, sc, qz = I.pack_gptq(c, s, z)
    checks.append(("gptq", I.gptq_to_canonical(qw, sc, qz, symmetric=False)))
    packed, sc = I.pack_ct(c, s, twos=True)
    checks.append(("ct", I.ct_to_canonical(packed, sc, None, "twos")))
    for name, (cc, ss, zz) in checks:
        if name == "ct":
            ref_dense = I.dequant_int4(cc, ss, zz)
            ref = x.float().cpu() @ ref_dense.t()
        else:
            assert torch.equal(cc, c)
            ref_dense, ref = I.dequant_int4(cc, ss, zz), want
        pk = (cc[:, 0::2] | (cc[:, 1::2] << 4)).to(torch.uint8).contiguous().cuda()
        got = K.gemm_w4a16(x, pk, ss.float().t().contiguous().cuda(), zz.float().t().contiguous().cuda(), None, group)
        assert K.gemm_w4a16_status() == 0
        _close(got.cpu(), ref, 2e-2, 2e-2 * float(ref.abs().max()), f"w4a16 {name}")
        expanded = K.gemm(x, ref_dense.bfloat16().cuda())
        assert torch.equal(got, expanded), name           # same numerics as the expanded weights
        one = K.gemm_w4a16(x[-1:].contiguous(), pk, ss.float().t().contiguous().cuda(),
                           zz.float().t().contiguous().cuda(), None, group)
        assert torch.equal(one[0], got[-1])
        if m > K.W4_EXPAND_ROWS:
            # above the row threshold the weights are expanded once into a scratch matrix; the
            # tile-by-tile expansion gives the same bits
            keep, K.W4_EXPAND_ROWS = K.W4_EXPAND_ROWS, 1 << 30
            try:
                tiled = K.gemm_w4a16(x, pk, ss.float().t().contiguous().cuda(), zz.float().t().contiguous().cuda(), None,
                                     group)
            finally:
                K.W4_EXPAND_ROWS = keep
            assert torch.equal(tiled, got), name


@pytest.mark.parametrize("m,n,k", [(3, 256, 128), (200, 1032, 512)])
def test_gemm_w4a16_nvfp4(K, m, n, k):
    from minisglang_rdna4_b200.quant import nvfp4 as NV

    torch.manual_seed(n)
    w = torch.randn(n, k) * 0.05
    packed, blk, glob = NV.quantize_nvfp4(w)
    glob = glob * (0.5 + torch.rand(n))                   # per-channel factors
    dense = NV.dequant_nvfp4(packed, blk, glob)
    x = torch.randn(m, k, device="cuda").bfloat16()
    got = K.gemm_w4a16(x, packed.cuda(), blk.view(torch.uint8).t().contiguous().cuda(), None, glob.float().cuda(), 16,
                       True)
    assert K.gemm_w4a16_status() == 0
    want = x.float().cpu() @ dense.float().t()
    _close(got.cpu(), want, 2e-2, 2e-2 * float(want.abs().max()), "w4a16 nvfp4")
    assert torch.equal(got, K.gemm(x, dense.bfloat16().cuda()))


# ------------------------------------------------------------------------------------------ bounds-checking build
_BOUNDS_CHILD = r"""
import torch
from minisglang_rdna4_b200.ops import cuda as K, ref
from minisglang_rdna4_b200.ops._lib import lib
assert K.bounds_checks_enabled(), "the bounds-checking library was not loaded"
hq, hk, d, ps, pages, t = 4, 2, 128, 16, 8, 6
torch.manual_seed(0)
qkv = torch.randn(t, (hq + 2 * hk) * d, device="cuda").bfloat16()
pool = torch.zeros(2, 1, pages + 1, hk, ps, d, device="cuda").bfloat16()
cos_sin = torch.randn(64, d, device="cuda")
pos = torch.tensor([0, 1, 2, 3, 4, 99999], dtype=torch.int32, device="cuda")        # one position past the table
loc = torch.tensor([0, 1, 2, 3, 10 ** 6, 5], dtype=torch.int32, device="cuda")      # one slot past the pool
assert K.bounds_report() == []
q = K.qk_norm_rope_store(qkv, None, None, pos, cos_sin, hq, hk, d, d, 1e-6, pool[0, 0], pool[1, 0], loc, None, None, False)
rep = K.bounds_report()
assert len(rep) >= 2 and all(r.startswith("rope_kv.cu:") for r in rep), rep
assert any("value 99999 limit 64" in r for r in rep) and any("value 1000000" in r for r in rep), rep
assert K.bounds_report() == []                                  # the report clears the rings
# the kernel skipped the bad store and clamped the bad position: the context is alive and the good rows are right
good = K.qk_norm_rope_store(qkv[:4].contiguous(), None, None, pos[:4].contiguous(), cos_sin, hq, hk, d, d, 1e-6,
                            pool[0, 0], pool[1, 0], loc[:4].contiguous(), None, None, False)
torch.cuda.synchronize()
assert torch.equal(good, q[:4]) and K.bounds_report() == []
# guard zones around a workspace: intact after use, and a write past the end is named
ws = K.workspace("probe", 1024, torch.float32, torch.device("cuda"))
ws.fill_(1.0)
assert K.verify_workspaces() == []
full, g = K._GUARDED["probe@cuda"]
full[g + 1024] = 7.0                                            # inside our own allocation: the upper guard zone
assert K.verify_workspaces() == ["probe@cuda"]
print("BOUNDS-OK")
"""


def test_bounds_checking_build_records_and_skips():
    """The -DMSGL_CHECK_BOUNDS library records an out-of-range position and KV slot with the source
    line, skips the access, and leaves the context usable; workspaces carry guard zones."""
    import subprocess
    import sys

    from minisglang_rdna4_b200.ops import _lib

    if not os.path.exists(_lib.CHECKED_LIB_PATH):
        from minisglang_rdna4_b200 import build

        build.build_cuda(checked=True)
    env = dict(os.environ, MSGL_CHECK_BOUNDS="1")
    out = subprocess.run([sys.executable, "-c", _BOUNDS_CHILD], capture_output=True, text=True, env=env, timeout=600,
                         cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert out.returncode == 0 and "BOUNDS-OK" in out.stdout, out.stdout[-2000:] + out.stderr[-4000:]
