import numpy as np
import pytest
import torch

from minisglang_rdna4_b200.kvcache import RadixPrefixCache
from minisglang_rdna4_b200.ops import host


def _ids(*xs):
    return torch.tensor(xs, dtype=torch.int32)


def test_match_is_page_aligned_and_splits_nodes():
    c = RadixPrefixCache(page_size=4)
    a = torch.arange(0, 16, dtype=torch.int32)
    assert c.insert_prefix(a, torch.tensor([10, 11, 12, 13], dtype=torch.int32)) == 0
    h, pages = c.match_prefix(torch.arange(0, 11, dtype=torch.int32))   # 11 tokens -> 8 matched
    assert h.cached_len == 8 and pages.tolist() == [10, 11]
    b = torch.cat([a[:8], torch.tensor([99, 98, 97, 96], dtype=torch.int32)])
    assert c.insert_prefix(b, torch.tensor([10, 11, 20], dtype=torch.int32)) == 8
    h2, p2 = c.match_prefix(b)
    assert h2.cached_len == 12 and p2.tolist() == [10, 11, 20]
    c.check_integrity()
    assert c.size_info.evictable_pages == 5


def test_lock_protects_and_eviction_is_lru():
    c = RadixPrefixCache(page_size=2)
    c.insert_prefix(_ids(1, 2, 3, 4), _ids(0, 1))
    c.insert_prefix(_ids(5, 6, 7, 8), _ids(2, 3))
    h, _ = c.match_prefix(_ids(1, 2, 3, 4))
    c.lock_handle(h)
    assert c.size_info.protected_pages == 2 and c.size_info.evictable_pages == 2
    with pytest.raises(RuntimeError):
        c.evict(3)
    freed = c.evict(2)
    assert sorted(freed.tolist()) == [2, 3]
    c.lock_handle(h, unlock=True)
    assert c.size_info.evictable_pages == 2
    # touching a branch makes it most recently used
    c.insert_prefix(_ids(9, 9, 9, 9), _ids(4, 5))
    c.match_prefix(_ids(1, 2, 3, 4))
    assert sorted(c.evict(2).tolist()) == [4, 5]
    c.check_integrity()


def test_parent_becomes_evictable_leaf():
    c = RadixPrefixCache(page_size=2)
    c.insert_prefix(_ids(1, 2, 3, 4), _ids(0, 1))
    c.insert_prefix(_ids(1, 2, 7, 8), _ids(0, 2))   # splits after page 0
    assert c.size_info.evictable_pages == 3
    freed = c.evict(3)
    assert sorted(freed.tolist()) == [0, 1, 2]
    assert c.size_info.total_pages == 0
    c.check_integrity()


def test_random_ops_keep_invariants():
    rng = np.random.default_rng(0)
    c = RadixPrefixCache(page_size=4)
    next_page = 0
    for _ in range(300):
        n = int(rng.integers(4, 40))
        ids = torch.from_numpy(rng.integers(0, 3, size=n).astype(np.int32))
        h, pages = c.match_prefix(ids)
        want = n // 4
        have = len(pages)
        new = torch.arange(next_page, next_page + want - have, dtype=torch.int32)
        next_page += want - have
        already = c.insert_prefix(ids, torch.cat([pages, new]))
        assert already >= h.cached_len
        if rng.random() < 0.3 and c.size_info.evictable_pages:
            c.evict(int(rng.integers(1, c.size_info.evictable_pages + 1)))
        c.check_integrity()


def test_native_prefix_compare_matches_numpy():
    assert host.host_lib() is not None, "host library must be built"
    rng = np.random.default_rng(1)
    for n in (64, 65, 1000):
        a = rng.integers(0, 100, size=n).astype(np.int32)
        b = a.copy()
        for cut in (0, 1, n // 2, n - 1, n):
            bb = b.copy()
            if cut < n:
                bb[cut] += 1
            assert host.common_prefix_len(a, bb, n) == host.common_prefix_len_numpy(a, bb, n) == min(cut, n)
