"""Host-side tables of the tensor-core prefill attention kernel (ops/cuda.py::PrefillPlan)."""
import numpy as np

from minisglang_rdna4_b200.ops.cuda import PrefillPlan


def _tables(plan):
    t = plan.tables.numpy()
    items = t[:plan.off_blk].reshape(-1, 8)
    return items, t[plan.off_blk:plan.off_req], t[plan.off_req:].reshape(-1, 2)


def test_items_cover_every_query_row_once_and_see_the_right_kv_blocks():
    rng = np.random.default_rng(0)
    q_lens = np.array([5, 130, 64, 1, 700, 128, 257])
    prefix = np.array([0, 200, 0, 512, 37, 128, 0])
    kv = q_lens + prefix
    cu_q = np.concatenate([[0], np.cumsum(q_lens)])
    plan = PrefillPlan(cu_q, kv, "cpu")
    items, blk_req, req_info = _tables(plan)

    assert plan.n_items == int(np.sum((q_lens + 127) // 128)) == items.shape[0]
    assert plan.t_pad == int(np.sum((kv + 127) // 128 * 128)) == blk_req.size * 128
    seen = np.zeros(int(cu_q[-1]), dtype=np.int32)
    for row0, rows, pos0, kv_off, n_blocks, req, _, _ in items:
        assert 1 <= rows <= 128 and kv_off % 128 == 0
        seen[row0:row0 + rows] += 1
        local = row0 - cu_q[req]                       # first row of the tile within its request
        assert local % 128 == 0 and pos0 == prefix[req] + local
        last_pos = pos0 + rows - 1                     # the tile's last row attends to keys 0..last_pos
        assert n_blocks == last_pos // 128 + 1 and n_blocks * 128 <= (kv[req] + 127) // 128 * 128
        assert tuple(req_info[req]) == (kv_off, kv[req])
    assert (seen == 1).all()
    assert (np.diff(items[:, 4]) <= 0).all()           # heaviest tiles first
    # every 128-row block of the scratch belongs to the request whose range covers it
    for b, r in enumerate(blk_req):
        off, n = req_info[r]
        assert off <= b * 128 < off + (n + 127) // 128 * 128
    del rng


def test_empty_and_single_token_steps():
    plan = PrefillPlan(np.array([0, 1]), np.array([1]), "cpu")
    items, blk_req, req_info = _tables(plan)
    assert items.tolist() == [[0, 1, 0, 0, 1, 0, 0, 0]] and blk_req.tolist() == [0] and req_info.tolist() == [[0, 1]]
    plan = PrefillPlan(np.array([0]), np.zeros(0, dtype=np.int64), "cpu")
    assert plan.n_items == 0 and plan.t_pad == 0


def test_short_extends_over_long_prefixes_stay_on_the_general_kernel():
    from minisglang_rdna4_b200.ops.cuda import tc_prefill_pays

    assert tc_prefill_pays(8192, 9600)            # a prefill chunk
    assert tc_prefill_pays(96, 256)               # a small chunk of a chunked prefill
    assert tc_prefill_pays(8192, 4 * 32768)       # last chunk of a 32k prompt
    assert tc_prefill_pays(5, 128)                # a tiny prompt
    assert not tc_prefill_pays(100, 32 * 1024)    # a new chat turn over a 32k history
    assert not tc_prefill_pays(16 * 32, 32 * 32768)
