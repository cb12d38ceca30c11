"""Block-diffusion decoding: the denoising rules against plain restatements, and the engine's
encode → denoise → commit loop against a dense Hugging Face forward with explicit masks."""
import json
import tempfile

import pytest
import torch

from minisglang_rdna4_b200.diffusion import Canvas, DenoiseConfig, entropy_bound_accept

transformers = pytest.importorskip("transformers")


def test_entropy_bound_accepts_the_longest_low_entropy_prefix():
    h = torch.tensor([0.5, 0.05, 2.0, 0.2, 0.1])
    # ascending: .05 .1 .2 .5 2.0 ; sums without the own entry: 0 .05 .15 .35 .85
    assert entropy_bound_accept(h, 0.3).tolist() == [False, True, False, True, True]
    assert entropy_bound_accept(h, 0.0).tolist() == [False, True, False, False, False]   # the lowest always passes
    assert entropy_bound_accept(h, 10.0).all()


def test_uniform_state_rule_step_by_step():
    """One step of the uniform-state rule restated with torch.distributions: same entropies, same
    accepted set, the sampled token where accepted and fresh noise elsewhere, the arg-max canvas as
    the candidate, the temperature falling from t_max towards t_min, early exit only when the arg-max
    canvas stood still and the mean entropy is low."""
    cfg = DenoiseConfig("entropy_bound", block=6, vocab_size=50, max_steps=4, t_min=0.4, t_max=0.8,
                        entropy_bound=0.5, confidence_threshold=0.05, stability_threshold=1)
    assert cfg.temperature(4) == pytest.approx(0.8) and cfg.temperature(1) == pytest.approx(0.5)
    g = torch.Generator().manual_seed(3)
    st = Canvas(cfg, 6, "cpu", g)
    first = st.tokens.clone()
    assert first.min() >= 0 and first.max() < 50 and st.steps_left == 4
    logits = torch.randn(6, 50, generator=torch.Generator().manual_seed(5)) * 3
    logits[0, 7] += 30.0                                       # a confident position
    g2 = torch.Generator().manual_seed(3)
    torch.randint(0, 50, (6,), generator=g2)                   # the initial canvas
    dist = torch.distributions.Categorical(logits=logits / 0.8)
    want_h = dist.entropy()
    st.advance(logits)
    p = torch.softmax(logits / 0.8 - (logits / 0.8).logsumexp(-1, keepdim=True), -1)
    drawn = torch.multinomial(p, 1, generator=g2).squeeze(-1)
    fresh = torch.randint(0, 50, (6,), generator=g2)
    acc = entropy_bound_accept(want_h, 0.5)
    assert acc[0] and not acc.all()
    assert torch.equal(st.tokens, torch.where(acc, drawn, fresh))
    assert torch.equal(st.emit, logits.argmax(-1)) and st.emit[0] == 7
    assert st.steps_left == 3 and not st.finished
    assert st.mean_entropy == pytest.approx(float(want_h.mean()), rel=1e-6)
    # confident everywhere and standing still: the second such step ends the block early
    sharp = torch.full((6, 50), -20.0)
    sharp[torch.arange(6), torch.arange(6)] = 20.0
    st.advance(sharp)
    assert not st.finished                                      # the arg-max canvas just changed
    st.advance(sharp)
    assert st.finished and st.steps_left == 1 and st.emit.tolist() == list(range(6))


def test_absorbing_state_rule_fills_confident_positions_first_and_finishes_in_time():
    cfg = DenoiseConfig("mask_confidence", block=4, vocab_size=20, max_steps=3, mask_token_id=19, unmask_threshold=0.9)
    st = Canvas(cfg, 4, "cpu", torch.Generator().manual_seed(0))
    assert st.tokens.tolist() == [19] * 4
    logits = torch.zeros(4, 20)
    logits[0, 3] = 10.0                 # confident
    logits[1, 4] = 1.0
    logits[2, 5] = 2.0
    logits[3, 19] = 9.0                 # the mask token itself is never proposed
    logits[3, 6] = 0.5
    st.advance(logits)                  # 4 masked, 3 steps: at least 2 are filled; position 0 by confidence
    assert st.tokens[0] == 3 and int((st.tokens == 19).sum()) == 2
    assert st.emit.tolist()[:3] == [3, 4, 5] and st.emit[3] == 6
    st.advance(logits)
    st.advance(logits)
    assert st.finished and st.tokens.tolist() == [3, 4, 5, 6]


def _tiny_llama(tmp, gen_cfg, extra_cfg):
    from transformers import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(vocab_size=200, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=16, max_position_embeddings=256, rms_norm_eps=1e-6,
                      tie_word_embeddings=False, eos_token_id=198, bos_token_id=None, pad_token_id=None)
    cfg._attn_implementation = "eager"
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn_like(p) * 0.2)
    model.save_pretrained(tmp, safe_serialization=True)
    c = json.load(open(f"{tmp}/config.json"))
    c.update(extra_cfg)
    json.dump(c, open(f"{tmp}/config.json", "w"))
    json.dump(gen_cfg, open(f"{tmp}/generation_config.json", "w"))
    return model


def _dense_block_decode(hf, prompt, cfg, max_tokens, eos):
    """Restatement without paging: every forward runs over the whole sequence with an explicit mask
    (committed text causal, canvas rows see everything); greedy absorbing-state rule."""
    ids = list(prompt)
    out = []
    while len(out) < max_tokens:
        n = min(cfg.block, max_tokens - len(out))
        st = Canvas(cfg, n, "cpu", torch.Generator().manual_seed(0))
        while not st.finished:
            seq = torch.tensor([ids + st.tokens.tolist()])
            t, c = seq.shape[1], len(ids)
            mask = torch.full((t, t), float("-inf")).triu(1)
            mask[c:, :] = 0.0
            with torch.no_grad():
                logits = hf(seq, attention_mask=mask[None, None]).logits[0, c:]
            st.advance(logits.float())
        block = st.emit.tolist()
        for tok in block:
            out.append(tok)
            ids.append(tok)
            if tok == eos or len(out) >= max_tokens:
                break
        if out and out[-1] == eos:
            break
    return out


def test_engine_block_diffusion_equals_a_dense_restatement():
    """Greedy absorbing-state decoding through the engine (chunked prompt encode without sampling,
    canvas rows through the verification attention path with a zero mask over the block, commit, causal
    re-encode of the committed block, a shorter last block) equals full-sequence forwards with explicit
    masks, request by request, in one batch."""
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    gen_cfg = {"max_denoising_steps": 3, "confidence_threshold": 0.6, "mask_token_id": 199,
               "sampler_config": {"_cls_name": "MaskConfidenceSamplerConfig"}}
    with tempfile.TemporaryDirectory() as tmp:
        hf = _tiny_llama(tmp, gen_cfg, {"canvas_length": 5, "mask_token_id": 199})
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, 190, (n,), generator=g).tolist() for n in (7, 33, 18)]
        llm = LLM(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64,
                  max_extend_tokens=24)
        assert llm.diffusion is not None and llm.diffusion.cfg.kind == "mask_confidence"
        cfg = llm.diffusion.cfg
        sp = [SamplingParams(max_tokens=m, ignore_eos=True) for m in (12, 10, 7)]
        outs = llm.generate(prompts, sp)
        got = [o.token_ids for o in outs]
        assert [len(x) for x in got] == [12, 10, 7]
        assert llm.stats["blocks"] == 3 + 2 + 2 and llm.stats["denoise_steps"] > 0
        assert all(1 <= s <= 3 for s in llm.diffusion.steps_per_block)
        llm.cache.check_integrity()
        llm.shutdown()
        for p, m, have in zip(prompts, (12, 10, 7), got):
            assert have == _dense_block_decode(hf, p, cfg, m, eos=-1), (len(p), m)


def test_uniform_state_decoding_is_reproducible_per_seed():
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    gen_cfg = {"max_denoising_steps": 6, "t_min": 0.3, "t_max": 0.9, "confidence_threshold": 0.2,
               "stability_threshold": 1, "sampler_config": {"_cls_name": "EntropyBoundSamplerConfig", "entropy_bound": 0.4}}
    with tempfile.TemporaryDirectory() as tmp:
        _tiny_llama(tmp, gen_cfg, {"canvas_length": 6})
        prompts = [[5, 6, 7, 8, 9, 10, 11], list(range(20, 45))]
        kw = dict(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64)
        runs = []
        for seed in (11, 11, 12):
            llm = LLM(**kw)
            assert llm.diffusion.cfg.kind == "entropy_bound"
            outs = llm.generate(prompts, SamplingParams(max_tokens=15, ignore_eos=True, seed=seed))
            runs.append([o.token_ids for o in outs])
            assert all(len(o.token_ids) == 15 for o in outs)
            llm.shutdown()
        assert runs[0] == runs[1]
        assert runs[0] != runs[2]
