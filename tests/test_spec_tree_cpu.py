"""Draft-tree geometry: the tree-verify forward (additive mask) must reproduce, at every node, what
a plain causal forward over that node's root-to-node path computes."""
import pytest
import torch

from minisglang_rdna4_b200.spec.tree import (TokenTree, accept_greedy_tree, apply_moves, compaction_moves,
                                             tree_mask, verify_rows)


def test_tree_from_paths_shares_prefixes_and_bounds_nodes():
    t = TokenTree.from_paths(9, [[1, 2, 3], [1, 2, 4], [1, 5], [6]])
    assert t.tokens == [9, 1, 2, 3, 4, 5, 6] and t.parent == [-1, 0, 1, 2, 2, 1, 0]
    assert t.depth == [0, 1, 2, 3, 3, 2, 1] and t.children(1) == [2, 5] and t.ancestors(4) == [4, 2, 1, 0]
    assert len(TokenTree.from_paths(9, [[1, 2, 3], [4, 5, 6]], max_nodes=4)) == 4
    assert TokenTree.chain(9, [1, 2]).parent == [-1, 0, 1]
    with pytest.raises(ValueError):
        TokenTree([1, 2], [-1, 1])


def test_rows_mask_acceptance_and_compaction():
    t = TokenTree.from_paths(9, [[1, 2, 3], [1, 2, 4], [1, 5], [6]])
    toks, pos, slots = verify_rows(t, prefix_len=10)
    assert toks == t.tokens and pos == [10, 11, 12, 13, 13, 12, 11] and slots == list(range(10, 17))
    m = tree_mask(t, 10, 20)
    assert m.shape == (7, 20) and (m[:, :10] == 0).all() and (m[:, 17:] == float("-inf")).all()
    assert (m[4, 10:17] == 0).tolist() == [True, True, True, False, True, False, False]   # root, 1, 2, itself

    # the target wants 1 after the root, 2 after node 1, 4 after node 2, then 8 (no such child)
    target = [1, 2, 4, 0, 8, 0, 0]
    emitted, path = accept_greedy_tree(t, target)
    assert emitted == [1, 2, 4, 8] and path == [0, 1, 2, 4]
    assert accept_greedy_tree(t, [7, 0, 0, 0, 0, 0, 0]) == ([7], [0])                       # nothing accepted: bonus only
    moves = compaction_moves(path, 10)
    assert moves == [(14, 13)]
    k = torch.arange(20.0).view(20, 1).clone()
    v = -k.clone()
    apply_moves(k, v, moves)
    assert k[13].item() == 14.0 and v[13].item() == -14.0 and k[12].item() == 12.0


def test_masked_tree_attention_equals_causal_attention_over_each_path():
    torch.manual_seed(0)
    d, prefix = 16, 5
    t = TokenTree.from_paths(9, [[1, 2, 3], [1, 2, 4], [1, 5], [6]])
    n = len(t)
    kp, vp = torch.randn(prefix, d), torch.randn(prefix, d)            # committed prefix
    q, kn, vn = torch.randn(n, d), torch.randn(n, d), torch.randn(n, d)  # one row per node
    k_all, v_all = torch.cat([kp, kn]), torch.cat([vp, vn])
    scores = q @ k_all.t() / d ** 0.5 + tree_mask(t, prefix, prefix + n)
    got = torch.softmax(scores, -1) @ v_all
    for i in range(n):
        anc = sorted(t.ancestors(i))
        k_path = torch.cat([kp, kn[anc]])
        v_path = torch.cat([vp, vn[anc]])
        want = torch.softmax(q[i] @ k_path.t() / d ** 0.5, -1) @ v_path
        assert torch.allclose(got[i], want, atol=1e-6), i
