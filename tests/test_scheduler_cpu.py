import torch

from minisglang_rdna4_b200 import SamplingParams
from minisglang_rdna4_b200.core import ChunkedReq, Req
from minisglang_rdna4_b200.llm import LLM
from minisglang_rdna4_b200.models.config import tiny_llama_config
from minisglang_rdna4_b200.scheduler import CacheManager, DecodeManager, PrefillManager, TableManager
from minisglang_rdna4_b200.scheduler.prefill import MIN_CHUNK, SHORT_REQ_RESERVE


def _mgr(pages=64, ps=16, slots=8):
    cache = CacheManager(pages, ps, slots + 1, 64)
    table = TableManager(slots)
    dec = DecodeManager(ps)
    return PrefillManager(cache, table, dec), cache, table, dec


def test_chunking_leaves_budget_for_short_requests():
    pre, cache, table, dec = _mgr(pages=512)
    long = torch.arange(3000, dtype=torch.int32)
    short = torch.arange(7, dtype=torch.int32) + 5000
    pre.add_one_req(1, long, SamplingParams(max_tokens=4))
    pre.add_one_req(2, short, SamplingParams(max_tokens=4))
    batch, adder = pre.schedule_next_batch(1024)
    # the long prompt is cut short of the budget and the scheduler stops behind it (FIFO head)
    assert isinstance(batch.reqs[0], ChunkedReq)
    assert batch.reqs[0].extend_len == 1024 - SHORT_REQ_RESERVE >= MIN_CHUNK
    assert len(batch.reqs) == 1 and pre.pending[0].chunked is batch.reqs[0]
    # a lone long prompt keeps the whole budget
    pre2, *_ = _mgr(pages=512)
    pre2.add_one_req(1, long, SamplingParams(max_tokens=4))
    b2, _ = pre2.schedule_next_batch(1024)
    assert b2.reqs[0].extend_len == 1024


def test_admission_respects_kv_capacity_and_inflight_reservation():
    pre, cache, table, dec = _mgr(pages=8, ps=16)   # 128 tokens
    pre.add_one_req(1, torch.arange(60, dtype=torch.int32), SamplingParams(max_tokens=20))
    pre.add_one_req(2, torch.arange(60, dtype=torch.int32) + 100, SamplingParams(max_tokens=20))
    batch, _ = pre.schedule_next_batch(4096)
    assert [r.uid for r in batch.reqs] == [1]      # 80 + 80 > 128: the second waits
    assert len(pre.pending) == 1


def test_finish_returns_every_page():
    cfg = tiny_llama_config()
    llm = LLM(model_config=cfg, use_dummy_weight=True, device="cpu", page_size=16, max_running_req=4,
              num_page_override=64, cache_type="naive")
    outs = llm.generate([list(range(20)), list(range(50))], SamplingParams(max_tokens=5, ignore_eos=True))
    assert [len(o.token_ids) for o in outs] == [5, 5]
    assert llm.cache.free_pages == 64 and llm.table.available_size == 4


def test_overlong_prompt_gets_an_error_reply_not_a_crash():
    cfg = tiny_llama_config()
    llm = LLM(model_config=cfg, use_dummy_weight=True, device="cpu", page_size=16, max_running_req=4,
              num_page_override=16, max_seq_len_override=128)
    outs = llm.generate([list(range(300)), list(range(10))], SamplingParams(max_tokens=3, ignore_eos=True))
    assert outs[0].error is not None and outs[0].finish_reason == "error"
    assert len(outs[1].token_ids) == 3


def test_eos_stops_generation_and_sampling_params_apply():
    cfg = tiny_llama_config()
    llm = LLM(model_config=cfg, use_dummy_weight=True, device="cpu", page_size=16, max_running_req=4,
              num_page_override=64)
    base = llm.generate([list(range(30))], SamplingParams(max_tokens=6, ignore_eos=True))[0].token_ids
    llm.eos_ids = {base[2]}
    first = base.index(base[2])
    out = llm.generate([list(range(30))], SamplingParams(max_tokens=6))[0]
    assert out.token_ids == base[: first + 1] and out.finish_reason == "stop"
    # temperature sampling with a seed-free generator still returns max_tokens tokens
    llm.eos_ids = set()
    out = llm.generate([list(range(30))], SamplingParams(max_tokens=6, temperature=0.8, top_k=5, top_p=0.9))[0]
    assert len(out.token_ids) == 6
    # logprobs are returned and are valid log-probabilities
    out = llm.generate([list(range(30))], SamplingParams(max_tokens=3, logprobs=2, ignore_eos=True))[0]
    assert len(out.logprobs) == 3 and all(lp <= 0 for lp in out.logprobs)


def test_penalties_change_the_greedy_path():
    from minisglang_rdna4_b200.engine.sample import apply_penalties

    logits = torch.zeros(2, 10)
    logits[:, 3] = 1.0
    rows = torch.tensor([1])
    toks = torch.tensor([[3, 3, -1]])
    out = apply_penalties(logits, rows, toks, torch.tensor([0.5]), torch.tensor([0.4]))
    assert out[0, 3] == 1.0 and abs(float(out[1, 3]) - (1.0 - 0.5 - 0.8)) < 1e-6


def test_tracing_hooks(monkeypatch, tmp_path):
    """The opt-in tracing knobs: host stage breakdown, profiler window, plan bounds check."""
    import numpy as np

    from minisglang_rdna4_b200.utils.tracing import GraphTimer, HostStages, StepProfiler

    monkeypatch.setenv("MSGL_HOSTPROF", "1")
    hs = HostStages()
    with hs.stage("schedule"):
        pass
    with hs.stage("schedule"):
        pass
    hs.tick()
    assert hs.count["schedule"] == 2 and "schedule=" in hs.summary()
    monkeypatch.delenv("MSGL_HOSTPROF")
    assert not HostStages().enabled and not GraphTimer().enabled

    trace = tmp_path / "trace.json"
    monkeypatch.setenv("MSGL_PROFILE", str(trace))
    monkeypatch.setenv("MSGL_PROFILE_SKIP", "1")
    monkeypatch.setenv("MSGL_PROFILE_STEPS", "2")
    prof = StepProfiler()
    for step in range(5):
        prof.on_step(step)
        np.zeros(4).sum()
    prof.close()
    assert trace.exists() and trace.stat().st_size > 0


def test_a_chunked_prompt_keeps_its_reservation_against_requests_behind_it():
    """A prompt prefilled in pieces still owes pages for the rest of its prompt and its output.
    A short request queued behind it must wait instead of taking that room (which would end in
    an out-of-pages error inside the step planner)."""
    pre, cache, table, dec = _mgr(pages=8, ps=16)   # 128 tokens
    pre.add_one_req(1, torch.arange(90, dtype=torch.int32), SamplingParams(max_tokens=20))
    pre.add_one_req(2, torch.arange(10, dtype=torch.int32) + 500, SamplingParams(max_tokens=10))
    batch, _ = pre.schedule_next_batch(64)
    assert isinstance(batch.reqs[0], ChunkedReq) and len(batch.reqs) == 1
    # the step planner takes the pages of the first chunk
    cache.page_table[batch.reqs[0].table_idx, :4] = cache._take(4)
    batch.reqs[0].cached_len = batch.reqs[0].device_len
    batch, _ = pre.schedule_next_batch(64)
    assert [r.uid for r in batch.reqs] == [1] and not isinstance(batch.reqs[0], ChunkedReq)
    assert [p.uid for p in pre.pending] == [2]     # 26 + 20 owed by request 1, 20 wanted: 66 > 64 free
    # end to end on a pool that holds one of them at a time: both finish, nothing raises
    llm = LLM(model_config=tiny_llama_config(), use_dummy_weight=True, device="cpu", page_size=16, max_running_req=4,
              num_page_override=8, max_extend_tokens=64, cache_type="naive")
    outs = llm.generate([list(range(90)), list(range(500, 510))], SamplingParams(max_tokens=20, ignore_eos=True))
    assert [len(o.token_ids) for o in outs] == [20, 20]


def test_prefill_budget_shrinks_under_memory_pressure():
    """The activation guard: with little free device memory the prefill step shrinks in whole pages,
    never below 1024 tokens, and is the configured chunk again once memory is back."""
    from minisglang_rdna4_b200 import LLM
    from minisglang_rdna4_b200.models.config import tiny_llama_config

    llm = LLM(model_config=tiny_llama_config(), use_dummy_weight=True, device="cpu", page_size=16, max_running_req=4,
              num_page_override=64, max_extend_tokens=8192)
    try:
        assert llm._prefill_budget_now() == 8192                     # no device: the guard stays out of the way
        llm.prefill.add_one_req(0, torch.arange(40, dtype=torch.int32), SamplingParams(max_tokens=1))
        mc = llm.engine.model_config
        per_token = max(2 * mc.intermediate_size, mc.q_size + 2 * mc.kv_size, mc.hidden_size * 4) * 8
        llm._free_device_bytes = lambda: (1 << 30) + 3000 * per_token
        assert llm._prefill_budget_now() == 3000 // 16 * 16
        llm._free_device_bytes = lambda: (1 << 30) + 100 * per_token
        assert llm._prefill_budget_now() == 1024                      # the floor
        llm._free_device_bytes = lambda: 64 << 30
        assert llm._prefill_budget_now() == 8192
    finally:
        llm.shutdown()
