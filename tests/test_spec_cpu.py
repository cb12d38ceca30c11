"""Speculative decoding on the CPU oracle path: greedy output must be bit-identical to plain
decoding, whatever the proposer suggests."""
import numpy as np
import torch

from minisglang_rdna4_b200 import SamplingParams
from minisglang_rdna4_b200.llm import LLM
from minisglang_rdna4_b200.models.config import tiny_llama_config
from minisglang_rdna4_b200.spec import (
    AdaptiveWidth, accept_greedy, accept_greedy_device, accept_rejection_sampling, eos_truncate, ngram_lookup,
)
from minisglang_rdna4_b200.spec.base import Proposer


def test_ngram_lookup_prefers_longest_and_most_recent():
    toks = np.array([1, 2, 3, 9, 9, 1, 2, 3, 7, 8, 5, 1, 2, 3], dtype=np.int32)
    assert ngram_lookup(toks, 2, 3, 1) == [7, 8]          # most recent earlier "1 2 3"
    assert ngram_lookup(np.array([4, 5, 6], dtype=np.int32), 3, 3, 1) == []
    assert ngram_lookup(np.array([5, 1, 5], dtype=np.int32), 4, 3, 1) == [1, 5]
    assert ngram_lookup(toks, 0, 3, 1) == []


def test_accept_rules():
    assert accept_greedy([5, 6, 7, 8], [5, 6, 9]) == [5, 6, 7]
    assert accept_greedy([5, 6, 7, 8], [5, 6, 7]) == [5, 6, 7, 8]   # bonus token
    assert accept_greedy([4], []) == [4]
    assert accept_greedy([1, 2], [9]) == [1]
    target = torch.tensor([5, 6, 7, 8, 1, 2, 4], dtype=torch.int32)
    drafts = torch.tensor([[5, 6, 9], [9, -1, -1], [-1, -1, -1]], dtype=torch.int32)
    cu = torch.tensor([0, 4, 6, 7], dtype=torch.int32)
    n, tgt = accept_greedy_device(target, drafts, cu, torch.tensor([3, 1, 0]))
    assert n.tolist() == [3, 1, 1] and tgt[0, :3].tolist() == [5, 6, 7] and tgt[2, 0] == 4
    assert eos_truncate([3, 9, 4], {9}, False) == ([3, 9], True)
    assert eos_truncate([3, 9, 4], {9}, True) == ([3, 9, 4], False)
    w = AdaptiveWidth(4)
    for _ in range(20):
        w.update(0.0)
    assert w.choose() == 1
    for _ in range(20):
        w.update(4.0)
    assert w.choose() == 4


def test_rejection_sampling_preserves_the_target_distribution():
    g = torch.Generator().manual_seed(0)
    p = torch.tensor([[0.7, 0.2, 0.1], [0.1, 0.1, 0.8]])
    counts = torch.zeros(3)
    for _ in range(4000):
        out = accept_rejection_sampling(p, None, [1], generator=g)   # the proposer always says token 1
        counts[out[0]] += 1
    freq = counts / counts.sum()
    assert torch.allclose(freq, p[0], atol=0.03)


class _Oracle(Proposer):
    """Proposes the true continuation for even uids and garbage for odd ones."""

    name = "oracle"

    def __init__(self, k, truth):
        super().__init__(k)
        self.truth = truth

    def propose(self, reqs):
        out = []
        for r in reqs:
            k = self.budget(r)
            done = r.num_generated
            good = self.truth[r.uid][done:done + k]
            out.append(list(good) if r.uid % 2 == 0 else [(t + 1) % 1000 for t in good])
        return out


def _llm(**kw):
    return LLM(model_config=tiny_llama_config(), use_dummy_weight=True, device="cpu", page_size=16,
               max_running_req=8, num_page_override=256, seed=0, **kw)


def test_spec_decode_is_bit_exact_with_plain_greedy():
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (20, 33, 47, 64)]
    # a repetitive prompt so the n-gram proposer has something to find
    prompts.append([1, 2, 3, 4, 5, 6, 7, 8] * 6)
    sp = SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True)
    plain = _llm()
    want = [o.token_ids for o in plain.generate(prompts, sp)]
    ngram = _llm(spec_algorithm="ngram", spec_num_draft=4)
    got = [o.token_ids for o in ngram.generate(prompts, sp)]
    assert got == want
    assert ngram.stats["spec_steps"] > 0 and ngram.stats["spec_emitted"] >= ngram.stats["spec_steps"]
    ngram.cache.check_integrity()
    assert ngram.table.available_size == 8
    # an oracle proposer: accepted drafts shorten the run, rejected ones never change the output
    oracle = _llm(spec_algorithm="ngram", spec_num_draft=3)
    oracle.proposer = _Oracle(3, {i: w for i, w in enumerate(want)})
    got2 = [o.token_ids for o in oracle.generate(prompts, sp)]
    assert got2 == want
    assert oracle.stats["spec_accepted"] > 0
    assert oracle.stats["spec_steps"] < plain.stats["steps"]


def test_spec_decode_respects_eos_and_max_tokens():
    g = torch.Generator().manual_seed(6)
    prompt = torch.randint(0, 1024, (30,), generator=g).tolist()
    base = _llm().generate([prompt], SamplingParams(max_tokens=10, ignore_eos=True))[0].token_ids
    spec = _llm(spec_algorithm="ngram", spec_num_draft=4)
    spec.proposer = _Oracle(4, {0: base})
    spec.eos_ids = {base[4]}
    out = spec.generate([prompt], SamplingParams(max_tokens=10))[0]
    assert out.token_ids == base[: base.index(base[4]) + 1] and out.finish_reason == "stop"
    spec2 = _llm(spec_algorithm="ngram", spec_num_draft=4)
    spec2.proposer = _Oracle(4, {0: base})
    out = spec2.generate([prompt], SamplingParams(max_tokens=7, ignore_eos=True))[0]
    assert out.token_ids == base[:7] and out.finish_reason == "length"


def test_eagle3_draft_is_exact_and_a_distilled_head_gets_accepted():
    """Greedy output with the EAGLE3 proposer equals plain greedy decoding whatever the draft
    predicts; a draft whose LM head is the target's own head on an identity-like layer agrees with
    the target often enough to shorten the run."""
    g = torch.Generator().manual_seed(8)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (18, 40)]
    sp = SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True)
    want = [o.token_ids for o in _llm().generate(prompts, sp)]
    spec = _llm(spec_algorithm="eagle3", spec_num_draft=3)
    got = [o.token_ids for o in spec.generate(prompts, sp)]
    assert got == want
    assert spec.stats["spec_steps"] > 0 and spec.stats["spec_drafted"] > 0
    spec.cache.check_integrity()
    # chunked prefill feeds the draft in pieces (carry of the chunk-boundary row)
    spec2 = _llm(spec_algorithm="eagle3", spec_num_draft=3, max_extend_tokens=16)
    got2 = [o.token_ids for o in spec2.generate(prompts, sp)]
    assert got2 == want
    # MTP variant: one feature layer, no fc
    mtp = _llm(spec_algorithm="mtp", spec_num_draft=2)
    assert [o.token_ids for o in mtp.generate(prompts, sp)] == want


from minisglang_rdna4_b200.spec.ngram import NgramProposer  # noqa: E402


class _TreeOracle(NgramProposer):
    """Two candidates per request: a wrong continuation first, the true one second, so that the
    accepted path runs through a non-first branch and its K/V has to be moved."""

    def __init__(self, k, answers):
        super().__init__(k, tree_width=2)
        self.answers = answers

    def propose_paths(self, reqs):
        out = []
        for r in reqs:
            done = r.num_generated
            good = self.answers[r.uid][done: done + self.budget(r)]
            bad = [(t + 1) % 1000 for t in good]
            out.append([list(bad), list(good)] if good else [])
        return out


def test_tree_verification_is_exact_and_follows_the_right_branch():
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (20, 33, 47)]
    prompts.append([1, 2, 3, 4, 5, 6, 7, 8] * 6)
    sp = SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True)
    plain = _llm()
    want = [o.token_ids for o in plain.generate(prompts, sp)]
    tree = _llm(spec_algorithm="ngram", spec_num_draft=4, spec_tree_width=3)
    got = [o.token_ids for o in tree.generate(prompts, sp)]
    assert got == want and tree.stats["spec_steps"] > 0
    tree.cache.check_integrity()
    oracle = _llm(spec_algorithm="ngram", spec_num_draft=3, spec_tree_width=2)
    oracle.proposer = _TreeOracle(3, {i: w for i, w in enumerate(want)})
    got2 = [o.token_ids for o in oracle.generate(prompts, sp)]
    assert got2 == want
    assert oracle.stats["spec_accepted"] > 0 and oracle.stats["spec_steps"] < plain.stats["steps"]
    # with max_tokens / eos cut-offs
    short = _llm(spec_algorithm="ngram", spec_num_draft=3, spec_tree_width=2)
    short.proposer = _TreeOracle(3, {0: want[0]})
    out = short.generate([prompts[0]], SamplingParams(max_tokens=7, ignore_eos=True))[0]
    assert out.token_ids == want[0][:7] and out.finish_reason == "length"


def test_sampled_and_constrained_requests_leave_the_speculative_path():
    """A request with temperature > 0 is not silently made greedy by the verify arg-max, and a
    grammar holds with a proposer configured: both decode through the normal sampler."""
    import json

    from minisglang_rdna4_b200.models.config import ModelConfig, RotaryConfig
    from minisglang_rdna4_b200.tokenizer import ByteTokenizer

    g = torch.Generator().manual_seed(11)
    prompt = torch.randint(0, 1024, (24,), generator=g).tolist()
    greedy = _llm().generate([prompt], SamplingParams(max_tokens=24, ignore_eos=True))[0].token_ids
    spec = _llm(spec_algorithm="ngram", spec_num_draft=4)
    spec.proposer = _Oracle(4, {0: greedy, 1: greedy})
    hot = spec.generate([prompt], SamplingParams(temperature=1.5, max_tokens=24, ignore_eos=True))[0].token_ids
    assert hot != greedy                       # sampled, not the verify arg-max
    assert spec.stats["spec_steps"] == 0       # never took a speculative step
    again = spec.generate([prompt], SamplingParams(max_tokens=24, ignore_eos=True))[0].token_ids
    assert again == greedy and spec.stats["spec_steps"] > 0

    cfg = ModelConfig(num_layers=1, num_qo_heads=2, num_kv_heads=1, head_dim=32, hidden_size=64, vocab_size=260,
                      intermediate_size=128, rms_norm_eps=1e-6, rotary_config=RotaryConfig(32, 32, 512, 1e4),
                      model_type="llama", torch_dtype="float32", max_position_embeddings=512, eos_token_ids=(257,))
    llm = LLM(model_config=cfg, use_dummy_weight=True, device="cpu", page_size=16, max_running_req=4,
              num_page_override=64, seed=3, spec_algorithm="ngram", spec_num_draft=3)
    schema = json.dumps({"type": "object", "properties": {"a": {"type": "integer"}, "b": {"type": "boolean"}},
                         "required": ["a", "b"], "additionalProperties": False})
    out = llm.generate([list(b"give me json:")], SamplingParams(max_tokens=60, grammar=schema, temperature=0.8,
                                                              top_k=40))[0]
    obj = json.loads(ByteTokenizer().decode(out.token_ids))
    assert isinstance(obj["a"], int) and isinstance(obj["b"], bool) and llm.stats["spec_steps"] == 0


def test_sampled_verification_is_reproducible_and_rank_independent(monkeypatch):
    """With MSGL_SPEC_SAMPLED a plain-temperature request keeps drafts by rejection sampling. The
    uniforms come from a generator tied to the seed, the request and its length, not from the
    process-wide generator: two engines (as two tensor-parallel ranks would be, each with its own
    global generator state) emit the same tokens, and another seed gives another sample."""
    monkeypatch.setenv("MSGL_SPEC_SAMPLED", "1")
    g = torch.Generator().manual_seed(11)
    prompt = torch.randint(0, 1024, (24,), generator=g).tolist()
    greedy = _llm().generate([prompt], SamplingParams(max_tokens=24, ignore_eos=True))[0].token_ids
    outs = []
    for seed, noise in ((5, 1), (5, 2), (6, 3), (None, 4), (None, 5)):
        torch.manual_seed(noise)                       # the global generator differs between "ranks"
        spec = _llm(spec_algorithm="ngram", spec_num_draft=4)
        spec.proposer = _Oracle(4, {0: greedy})
        outs.append(spec.generate([prompt], SamplingParams(temperature=1.2, max_tokens=24, ignore_eos=True, seed=seed)
                                  )[0].token_ids)
        assert spec.stats["spec_steps"] > 0
    assert outs[0] == outs[1] and outs[0] != outs[2]
    assert outs[3] == outs[4]                          # unseeded: tied to the engine seed and the request id
