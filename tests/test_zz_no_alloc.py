"""The allocation-free attention entry point, called through its exported C symbol.

Some embedders of this library may not request device memory once they are running (no
cudaMalloc from their call sites). For them ``msgl_paged_attention_noalloc`` keeps the split-KV
partials in an array built into the library. This test drives that symbol directly with ctypes
and checks, on two calls in a row with different inputs, that it returns what the regular entry
point returns when it is given a workspace tensor, and what the fp32 restatement of the op gives.

The file name sorts last on purpose: if this test fails, a run that stops at the first failure
has already run everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

c_p, c_i, c_ll, c_f = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def _case(seed, fp8):
    torch.manual_seed(seed)
    hq, hk, d, ps = 8, 2, 128, 16
    kv_lens = [700 + 37 * seed, 65, 1300, 256]
    b = len(kv_lens)
    pages = sum(-(-n // ps) for n in kv_lens) + 2
    dt = torch.float8_e4m3fn if fp8 else torch.bfloat16
    pool = (torch.randn(2, 1, pages + 1, hk, ps, d, device="cuda") * (6 if fp8 else 1)).to(dt)
    perm = torch.randperm(pages, device="cuda").to(torch.int32)
    maxp = max(-(-n // ps) for n in kv_lens)
    bt = torch.zeros(b, maxp, dtype=torch.int32, device="cuda")
    off = 0
    for i, n in enumerate(kv_lens):
        np_ = -(-n // ps)
        bt[i, :np_] = perm[off:off + np_]
        off += np_
    cu = torch.arange(b + 1, dtype=torch.int32, device="cuda")
    sl = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
    q = torch.randn(b, hq, d, device="cuda").bfloat16()
    ks = (0.5 + torch.rand(hk, device="cuda")) / 8 if fp8 else None
    vs = (0.5 + torch.rand(hk, device="cuda")) / 8 if fp8 else None
    return dict(q=q, pool=pool, bt=bt, cu=cu, sl=sl, ks=ks, vs=vs, hq=hq, hk=hk, d=d, ps=ps, pages=pages,
                max_kv=max(kv_lens), b=b)


def _noalloc(fn, K, c, splits):
    desc, layer, layers = K._kv_map(c["pool"][0, 0])
    out = torch.empty_like(c["q"])
    p = lambda t: None if t is None else t.data_ptr()
    fp8 = c["pool"].dtype == torch.float8_e4m3fn
    rc = fn(desc.ctypes.data, p(c["q"]), p(out), p(c["bt"]), c["bt"].stride(0), p(c["cu"]), p(c["sl"]), p(c["ks"]),
            p(c["vs"]), None, 0, c["b"], c["q"].shape[0], 1, c["hq"], c["hk"], c["d"], c["ps"], c["pages"], layer,
            layers, int(fp8), 1, 0, splits, c["d"] ** -0.5, 0, torch.cuda.current_stream().cuda_stream)
    return rc, out


def test_noalloc_entry_point_matches_regular_entry_point():
    from minisglang_rdna4_b200.ops import cuda as K
    from minisglang_rdna4_b200.ops._lib import lib

    fn = lib().msgl_paged_attention_noalloc          # the exported C symbol itself
    fn.restype = c_i
    fn.argtypes = [c_p, c_p, c_p, c_p, c_i, c_p, c_p, c_p, c_p, c_p, c_ll,
                   c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_f, c_i, c_p]
    for call, (seed, fp8, splits) in enumerate([(1, True, 4), (2, False, 3)]):   # two calls in a row
        c = _case(seed, fp8)
        want = K.paged_attention(c["q"], c["pool"][0, 0], c["pool"][1, 0], c["bt"], c["cu"], c["sl"], c["d"] ** -0.5,
                                 k_scale=c["ks"], v_scale=c["vs"], max_q=1, max_kv=c["max_kv"], decode=True,
                                 splits=splits)
        rc, got = _noalloc(fn, K, c, splits)
        torch.cuda.synchronize()
        assert rc == 0, lib().msgl_last_error()
        assert K.attn_status() == 0
        err = (got.float() - want.float()).abs().max().item()
        assert err <= 3e-2 * max(1.0, want.float().abs().max().item()), f"call {call}: max err {err}"
        # and against the fp32 restatement of the op itself
        from minisglang_rdna4_b200.ops import ref

        oracle = ref.paged_attention(c["q"], c["pool"][0, 0], c["pool"][1, 0], c["bt"], c["cu"], c["sl"],
                                     c["d"] ** -0.5, True, 0, None, c["ks"], c["vs"])
        err = (got.float() - oracle.float()).abs().max().item()
        assert err <= 3e-2 * max(1.0, oracle.float().abs().max().item()), f"call {call}: max err vs oracle {err}"
    # a request that cannot fit the built-in scratch is refused with a message, not run
    c = _case(3, False)
    big_q = torch.randn(4096, c["hq"], c["d"], device="cuda").bfloat16()
    c2 = dict(c, q=big_q, b=4)
    rc, _ = _noalloc(fn, K, c2, 16)
    assert rc == 1 and b"built-in scratch" in lib().msgl_last_error()
