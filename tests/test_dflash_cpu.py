"""The DFlash block drafter: speculative decoding stays exact, and the proposed blocks equal a restatement of
the published forward over the hidden states the Hugging Face target produces."""
import json
import os
import tempfile

import pytest
import torch
import torch.nn.functional as F

transformers = pytest.importorskip("transformers")

H, HEADS, KV, D, INTER, LAYERS, BLOCK, MASK, AUX = 64, 4, 2, 16, 96, 2, 5, 199, [0, 2]
THETA = 10000.0


def _target(tmp):
    from transformers import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(vocab_size=200, hidden_size=H, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=512, eos_token_id=198, bos_token_id=None,
                      pad_token_id=None, tie_word_embeddings=False)
    torch.manual_seed(0)
    hf = LlamaForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for _, p in hf.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn_like(p) * 0.08)
    hf.save_pretrained(tmp, safe_serialization=True)
    return hf


def _drafter(tmp):
    from safetensors.torch import save_file

    g = torch.Generator().manual_seed(3)
    rnd = lambda *s: torch.randn(*s, generator=g) * 0.12
    w = {"fc.weight": rnd(H, len(AUX) * H), "hidden_norm.weight": 1.0 + rnd(H), "norm.weight": 1.0 + rnd(H)}
    for i in range(LAYERS):
        p = f"layers.{i}."
        w[p + "input_layernorm.weight"], w[p + "post_attention_layernorm.weight"] = 1.0 + rnd(H), 1.0 + rnd(H)
        w[p + "self_attn.q_proj.weight"], w[p + "self_attn.o_proj.weight"] = rnd(HEADS * D, H), rnd(H, HEADS * D)
        w[p + "self_attn.k_proj.weight"], w[p + "self_attn.v_proj.weight"] = rnd(KV * D, H), rnd(KV * D, H)
        w[p + "self_attn.q_norm.weight"], w[p + "self_attn.k_norm.weight"] = 1.0 + rnd(D), 1.0 + rnd(D)
        w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"] = rnd(INTER, H), rnd(INTER, H)
        w[p + "mlp.down_proj.weight"] = rnd(H, INTER)
    os.makedirs(tmp, exist_ok=True)
    save_file({k: v.contiguous() for k, v in w.items()}, os.path.join(tmp, "model.safetensors"))
    json.dump({"architectures": ["DFlashDraftModel"], "hidden_size": H, "num_hidden_layers": LAYERS,
               "num_attention_heads": HEADS, "num_key_value_heads": KV, "head_dim": D, "intermediate_size": INTER,
               "rms_norm_eps": 1e-6, "rope_theta": THETA, "max_position_embeddings": 512,
               "dflash_config": {"block_size": BLOCK, "mask_token_id": MASK, "target_layer_ids": AUX}},
              open(os.path.join(tmp, "config.json"), "w"))
    return w


def _restate(hf, w, ids, k):
    """Drafts for a request whose first ``len(ids) - 1`` tokens are committed in the target and whose last
    token is the confirmed one."""
    rms = lambda x, wt: (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6)) * wt
    L = len(ids) - 1
    with torch.no_grad():
        hs = hf.model(torch.tensor([ids[:L]]), output_hidden_states=True).hidden_states
        ctx = rms(torch.cat([hs[j + 1][0] for j in AUX], -1) @ w["fc.weight"].t(), w["hidden_norm.weight"])
        x = hf.model.embed_tokens(torch.tensor([ids[L]] + [MASK] * (BLOCK - 1)))
        inv = 1.0 / (THETA ** (torch.arange(0, D, 2).float() / D))

        def rope(z, pos):
            ang = pos.float()[:, None] * inv[None]
            cos, sin = torch.cat([ang.cos(), ang.cos()], -1)[:, None], torch.cat([ang.sin(), ang.sin()], -1)[:, None]
            return z * cos + torch.cat([-z[..., D // 2:], z[..., : D // 2]], -1) * sin

        ctx_pos, blk_pos = torch.arange(L), torch.arange(L, L + BLOCK)
        for i in range(LAYERS):
            p = f"layers.{i}."
            y = rms(x, w[p + "input_layernorm.weight"])
            q = rope(rms((y @ w[p + "self_attn.q_proj.weight"].t()).view(BLOCK, HEADS, D), w[p + "self_attn.q_norm.weight"]), blk_pos)
            both = torch.cat([ctx, y])
            kk = rope(rms((both @ w[p + "self_attn.k_proj.weight"].t()).view(-1, KV, D), w[p + "self_attn.k_norm.weight"]),
                      torch.cat([ctx_pos, blk_pos]))
            vv = (both @ w[p + "self_attn.v_proj.weight"].t()).view(-1, KV, D)
            kk, vv = kk.repeat_interleave(HEADS // KV, 1), vv.repeat_interleave(HEADS // KV, 1)
            s = torch.einsum("qhd,khd->hqk", q, kk) / D ** 0.5
            o = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), vv).reshape(BLOCK, -1)
            x = x + o @ w[p + "self_attn.o_proj.weight"].t()
            y = rms(x, w[p + "post_attention_layernorm.weight"])
            x = x + (F.silu(y @ w[p + "mlp.gate_proj.weight"].t()) * (y @ w[p + "mlp.up_proj.weight"].t())) \
                @ w[p + "mlp.down_proj.weight"].t()
        logits = hf.lm_head(rms(x, w["norm.weight"]))
    return logits[1:k + 1].argmax(-1).tolist()


def test_dflash_block_drafter():
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM
    from minisglang_rdna4_b200.spec.dflash import DFlashProposer

    with tempfile.TemporaryDirectory() as tmp:
        hf = _target(tmp)
        w = _drafter(os.path.join(tmp, "drafter"))
        g = torch.Generator().manual_seed(4)
        prompts = [torch.randint(0, 190, (n,), generator=g).tolist() for n in (6, 41)]
        want = [hf.generate(torch.tensor([p]), max_new_tokens=9, do_sample=False)[0, len(p):].tolist() for p in prompts]
        llm = LLM(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64,
                  max_extend_tokens=16, spec_algorithm="dflash", spec_num_draft=4,
                  spec_draft_model_path=os.path.join(tmp, "drafter"))
        prop = llm.proposer
        assert isinstance(prop, DFlashProposer) and prop.block == BLOCK and prop.capture_layers == [1, 3]
        seen = []
        inner = prop.propose

        def spy(reqs):
            out = inner(reqs)
            for r, d in zip(reqs, out):
                if d:
                    seen.append((r.input_ids[: prop._len[r.uid] + 1].tolist(), list(d)))
            return out

        prop.propose = spy
        got = [o.token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=9, ignore_eos=True))]
        llm.shutdown()
    assert got == want
    assert len(seen) >= 4
    for ids, drafts in seen[:6]:
        assert drafts == _restate(hf, w, ids, len(drafts)), len(ids)


def test_tidar_self_drafting():
    """The target drafts for itself: one causal forward over [confirmed token, mask x k]; the arg-max at the
    mask rows are the drafts. Output equals plain greedy decoding; the drafts equal a Hugging Face forward over
    the same rows; the drafting forward leaves lengths and page accounting untouched."""
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM
    from minisglang_rdna4_b200.spec.tidar import TiDARProposer

    with tempfile.TemporaryDirectory() as tmp:
        hf = _target(tmp)
        json.dump({"mask_token_id": MASK, "block_size": 3}, open(os.path.join(tmp, "tidar_config.json"), "w"))
        g = torch.Generator().manual_seed(4)
        prompts = [torch.randint(0, 190, (n,), generator=g).tolist() for n in (6, 41)]
        want = [hf.generate(torch.tensor([p]), max_new_tokens=9, do_sample=False)[0, len(p):].tolist() for p in prompts]
        llm = LLM(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64,
                  max_extend_tokens=16, spec_algorithm="tidar", spec_num_draft=4)
        prop = llm.proposer
        assert isinstance(prop, TiDARProposer) and prop.block == 3 and prop.mask_token_id == MASK
        seen = []
        inner = prop.propose

        def spy(reqs):
            before = [(r.cached_len, r.device_len) for r in reqs]
            out = inner(reqs)
            assert before == [(r.cached_len, r.device_len) for r in reqs]
            for r, d in zip(reqs, out):
                if d:
                    seen.append((r.input_ids[: r.device_len].tolist(), list(d)))
            return out

        prop.propose = spy
        got = [o.token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=9, ignore_eos=True))]
        llm.cache.check_integrity()
        llm.shutdown()
    assert got == want
    assert len(seen) >= 4 and max(len(d) for _, d in seen) == 3
    for ids, drafts in seen[:6]:
        k = len(drafts)
        with torch.no_grad():
            logits = hf(torch.tensor([ids + [MASK] * k])).logits[0]
        assert drafts == logits[len(ids):len(ids) + k].argmax(-1).tolist(), len(ids)


def test_draft_tree_keeps_the_most_probable_prefixes():
    """Best-first enumeration against brute force: the kept prefixes are the highest-scoring ones under the
    product of the per-position distributions, each after its parent."""
    import itertools

    from minisglang_rdna4_b200.spec.ddtree import build_draft_paths

    g = torch.Generator().manual_seed(0)
    logp = torch.log_softmax(torch.randn(4, 3, generator=g) * 2, -1).sort(-1, descending=True).values
    ids = torch.arange(12).view(4, 3) + 100
    every = []
    for d in range(1, 5):
        for ranks in itertools.product(range(3), repeat=d):
            every.append((sum(float(logp[i, r]) for i, r in enumerate(ranks)), [int(ids[i, r]) for i, r in enumerate(ranks)]))
    every.sort(key=lambda t: -t[0])
    for budget in (1, 5, 17):
        got = build_draft_paths(logp.tolist(), ids.tolist(), budget)
        assert len(got) == budget and sorted(map(tuple, got)) == sorted(tuple(p) for _, p in every[:budget])
        for i, p in enumerate(got):
            assert len(p) == 1 or p[:-1] in got[:i]
    assert build_draft_paths([], [], 4) == [] and build_draft_paths(logp.tolist(), ids.tolist(), 0) == []


def test_tidar_with_a_draft_tree():
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    with tempfile.TemporaryDirectory() as tmp:
        hf = _target(tmp)
        json.dump({"mask_token_id": MASK, "block_size": 3}, open(os.path.join(tmp, "tidar_config.json"), "w"))
        g = torch.Generator().manual_seed(4)
        prompts = [torch.randint(0, 190, (n,), generator=g).tolist() for n in (6, 41)]
        want = [hf.generate(torch.tensor([p]), max_new_tokens=9, do_sample=False)[0, len(p):].tolist() for p in prompts]
        llm = LLM(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64,
                  max_extend_tokens=16, spec_algorithm="tidar", spec_num_draft=3, spec_tree_width=2)
        assert llm.proposer.tree_width == 2
        got = [o.token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=9, ignore_eos=True))]
        assert llm.stats["spec_drafted"] > 0
        llm.cache.check_integrity()
        llm.shutdown()
    assert got == want


@pytest.mark.parametrize("algo", ["dflash", "tidar"])
def test_block_drafters_on_two_tensor_parallel_ranks(algo):
    """Both ranks run the (replicated) drafter or the self-drafting forward and reach the same drafts; tokens
    equal the target's greedy decoding."""
    import multiprocessing as mp

    from test_tp_cpu import _worker

    with tempfile.TemporaryDirectory() as tmp:
        hf = _target(tmp)
        json.dump({"mask_token_id": MASK, "block_size": 3}, open(os.path.join(tmp, "tidar_config.json"), "w"))
        _drafter(os.path.join(tmp, "drafter"))
        g = torch.Generator().manual_seed(5)
        prompts = [torch.randint(0, 190, (n,), generator=g).tolist() for n in (7, 30)]
        want = [hf.generate(torch.tensor([p]), max_new_tokens=6, do_sample=False)[0, len(p):].tolist() for p in prompts]
        extra = {"spec_algorithm": algo, "spec_num_draft": 3}
        if algo == "dflash":
            extra["spec_draft_model_path"] = os.path.join(tmp, "drafter")
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        port = 19100 + (os.getpid() % 1500) + (5 if algo == "tidar" else 0)
        procs = [ctx.Process(target=_worker, args=(r, 2, port, tmp, prompts, q, False, extra)) for r in range(2)]
        for p in procs:
            p.start()
        got = q.get(timeout=240)
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    assert got == want
