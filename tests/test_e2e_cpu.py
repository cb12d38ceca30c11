"""Tiny-Llama plumbing run on CPU fp32: scheduler + radix cache + paged KV must reproduce a
straight (no cache, no paging) transformer's greedy tokens."""
import torch

from minisglang_rdna4_b200 import SamplingParams
from minisglang_rdna4_b200.llm import LLM
from minisglang_rdna4_b200.models.config import tiny_llama_config
from minisglang_rdna4_b200.ops import ref


def _dense_greedy(model, cfg, prompt, n_new):
    """Recompute the whole sequence every step with plain attention."""
    ids = list(prompt)
    body = model.model
    cos_sin = ref.build_cos_sin_cache(cfg.head_dim, 4096, cfg.rotary_config.base)
    out = []
    for _ in range(n_new):
        t = len(ids)
        x = body.embed_tokens.weight[torch.tensor(ids)]
        pos = torch.arange(t)
        for layer in body.layers:
            h = ref.rms_norm(x, layer.input_layernorm.weight, cfg.rms_norm_eps)
            qkv = h @ layer.self_attn.qkv_proj.weight.t()
            qs, ks = cfg.num_qo_heads * cfg.head_dim, cfg.num_kv_heads * cfg.head_dim
            q, k, v = qkv.split([qs, ks, ks], -1)
            q, k = ref.qk_norm_rope(q, k, None, None, pos, cos_sin, cfg.head_dim, cfg.head_dim, 1e-6)
            q = q.view(t, cfg.num_qo_heads, cfg.head_dim).transpose(0, 1)
            k = k.view(t, cfg.num_kv_heads, cfg.head_dim).transpose(0, 1).repeat_interleave(2, 0)
            v = v.view(t, cfg.num_kv_heads, cfg.head_dim).transpose(0, 1).repeat_interleave(2, 0)
            s = (q @ k.transpose(1, 2)) * cfg.head_dim ** -0.5
            s = s.masked_fill(torch.triu(torch.ones(t, t, dtype=torch.bool), 1), float("-inf"))
            o = (torch.softmax(s, -1) @ v).transpose(0, 1).reshape(t, -1)
            x = x + o @ layer.self_attn.o_proj.weight.t()
            h = ref.rms_norm(x, layer.post_attention_layernorm.weight, cfg.rms_norm_eps)
            gu = h @ layer.mlp.gate_up_proj.weight.t()
            x = x + ref.silu_and_mul(gu) @ layer.mlp.down_proj.weight.t()
        h = ref.rms_norm(x[-1:], body.norm.weight, cfg.rms_norm_eps)
        tok = int((h @ model.lm_head.weight.t()).argmax(-1))
        out.append(tok)
        ids.append(tok)
    return out


def test_tiny_llama_matches_dense_oracle_and_hits_prefix_cache():
    cfg = tiny_llama_config()
    llm = LLM(model_config=cfg, use_dummy_weight=True, device="cpu", page_size=16,
              max_running_req=8, num_page_override=256, max_extend_tokens=96, seed=0)
    g = torch.Generator().manual_seed(1)
    shared = torch.randint(0, cfg.vocab_size, (32,), generator=g).tolist()
    prompts = []
    for i in range(8):
        n = int(torch.randint(32, 129, (1,), generator=g))
        body = torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist()
        prompts.append(shared + body[: max(n - 32, 1)] if i < 4 else body)
    sp = SamplingParams(temperature=0.0, max_tokens=32, ignore_eos=True)
    # first pass caches the shared prefix; second pass must hit it
    first = llm.generate(prompts[:1], sp)
    outs = llm.generate(prompts, sp)
    assert sum(o.cached_tokens for o in outs[:4]) >= 4 * 32
    assert llm.cache.prefix_hit_tokens >= 4 * 32
    for p, o in zip(prompts, outs):
        assert len(o.token_ids) == 32 and o.finish_reason == "length"
    for idx in (0, 3, 5):
        want = _dense_greedy(llm.engine.model, cfg, prompts[idx], 32)
        assert outs[idx].token_ids == want, idx
    assert first[0].token_ids == outs[0].token_ids
    llm.cache.check_integrity()
    # every page is either free or owned by the prefix cache once all requests are done
    info = llm.cache.prefix_cache.size_info
    assert llm.cache.free_pages + info.total_pages == llm.cache.num_pages
    assert info.protected_pages == 0


def test_a_seeded_request_is_reproducible_whatever_it_is_batched_with():
    """``seed`` pins a sampled request's draws to (seed, token index): alone or beside other
    requests it generates the same tokens; without a seed two runs differ."""
    from minisglang_rdna4_b200 import LLM, SamplingParams
    from minisglang_rdna4_b200.models.config import tiny_llama_config

    llm = LLM(model_config=tiny_llama_config(), use_dummy_weight=True, device="cpu", page_size=16, max_running_req=8,
              num_page_override=128, seed=0)
    try:
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (12, 30, 7)]
        sp = SamplingParams(temperature=1.5, max_tokens=12, ignore_eos=True, seed=1234)
        free = SamplingParams(temperature=1.5, max_tokens=12, ignore_eos=True)
        alone = llm.generate([prompts[0]], sp)[0].token_ids
        again = llm.generate([prompts[0]], sp)[0].token_ids
        mixed = llm.generate([prompts[1], prompts[0], prompts[2]], [free, sp, free])[1].token_ids
        assert alone == again == mixed
        other = llm.generate([prompts[0]], SamplingParams(temperature=1.5, max_tokens=12, ignore_eos=True, seed=99))
        assert other[0].token_ids != alone
        a, b = llm.generate([prompts[0]], free)[0].token_ids, llm.generate([prompts[0]], free)[0].token_ids
        assert a != b
    finally:
        llm.shutdown()


def test_state_digests_separate_the_reused_span_from_the_computed_one(monkeypatch):
    """MSGL_STATE_DIGEST: after every prefill step the K/V the request holds is hashed per layer and
    per segment of 256 positions. The same prompt prefilled twice gives the same digests; a value
    changed in one page of one layer is named by layer and segment."""
    import numpy as np

    from minisglang_rdna4_b200.kvcache import state_digest

    monkeypatch.setenv("MSGL_STATE_DIGEST", "1")
    g = torch.Generator().manual_seed(7)
    prompt = torch.randint(0, 500, (300,), generator=g).tolist()
    llm = LLM(model_config=tiny_llama_config(), use_dummy_weight=True, device="cpu", page_size=16, max_running_req=8,
              num_page_override=256, seed=0)
    llm.generate([prompt], SamplingParams(max_tokens=2, ignore_eos=True))
    first = llm.last_state_digests[0]
    layers = llm.engine.kv_cache.num_layers
    assert set(first) == {("kv", l, s) for l in range(layers) for s in (0, 1)}        # 300 positions: two segments
    llm.generate([prompt], SamplingParams(max_tokens=2, ignore_eos=True))            # prefix-cache hit this time
    second = llm.last_state_digests[1]
    assert llm.cache.prefix_hit_tokens >= 288
    # segment 0 (positions 0..255) lies inside the 288 reused positions: handed over unchanged. Segment 1 also
    # holds the 12 positions this prefill computed itself, as a 12-row step instead of a 300-row one, whose
    # last bits may differ: a difference may only be there
    assert all(first[k] == second[k] for k in first if k[2] == 0)
    diff = state_digest.first_difference(first, second)
    assert diff is None or diff[2] == 1
    # direct use: flip one K value of layer 1 at position 270 and name it
    pool = llm.engine.kv_cache
    pages = np.arange(19, dtype=np.int64)
    before = state_digest.kv_digests(pool, pages, 300)
    ps = pool.page_size
    pool.k_cache(1)[270 // ps, 0, 270 % ps, 0] += 1.0
    after = state_digest.kv_digests(pool, pages, 300)
    assert state_digest.first_difference(before, after) == ("kv", 1, 1)
    llm.shutdown()
