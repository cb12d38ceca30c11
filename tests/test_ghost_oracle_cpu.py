import torch

from minisglang_rdna4_b200.kvcache.ghost_oracle import GhostPrefixOracle, oracle_path


def test_oracle_counts_what_an_unbounded_cache_would_reuse(tmp_path, monkeypatch):
    o = GhostPrefixOracle(page_size=4)
    a = list(range(100, 120))                      # 5 pages
    assert o.observe(a, 0) == 0                    # nothing seen before
    assert o.observe(a[:12] + [7] * 8, 8) == 12    # shares 3 pages; the live cache reused 2 of them
    assert o.observe([1, 2, 3], 0) == 0            # shorter than a page
    c = o.counters()
    assert c["requests"] == 3 and c["prompt_tokens"] == 43 and c["actual_tokens"] == 8
    assert c["potential_tokens"] == 12 and c["gap_evict_tokens"] == 4
    # a page in the middle of a different prefix does not count: the hash is chained
    assert o.observe([9, 9, 9, 9] + a[4:12], 0) == 0
    assert "lost to eviction" in o.report()

    monkeypatch.setenv("MSGL_GHOST_ORACLE_DIR", str(tmp_path))
    path = oracle_path("org/model-7b", dp_rank=1)
    assert path.endswith("ghost-org_model-7b-dp1.json")
    o.save(path)
    again = GhostPrefixOracle.load(path, page_size=4)
    assert again.counters()["prompt_tokens"] == o.counters()["prompt_tokens"]
    assert again.observe(a, 0) == 20               # the remembered prefixes survive a restart
    assert GhostPrefixOracle.load(path, page_size=16).requests == 0   # other page size: start over

    small = GhostPrefixOracle(page_size=4, capacity=3)
    small.observe(a, 0)
    assert small.counters()["remembered_pages"] == 3 and small.observe(a, 0) == 0   # the first pages were forgotten


def test_cache_manager_feeds_the_oracle(monkeypatch):
    monkeypatch.setenv("MSGL_GHOST_ORACLE", "1")
    from minisglang_rdna4_b200.scheduler.cache import CacheManager

    cm = CacheManager(num_pages=32, page_size=4, num_slots=4, max_pages_per_seq=8)
    assert cm.ghost is not None
    ids = torch.arange(50, 67, dtype=torch.int32)
    cm.match_req(ids)
    cm.match_req(ids)
    c = cm.ghost.counters()
    # nothing was inserted into the radix tree, so the live cache reused nothing, but the second
    # prompt's 4 whole pages had been seen
    assert c["requests"] == 2 and c["actual_tokens"] == 0 and c["potential_tokens"] == 16
