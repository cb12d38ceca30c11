"""Gemma-3 style decoder against the published implementation (``transformers``) on CPU fp32:
a tiny random-init checkpoint is written by ``transformers``, loaded through this package's
weight loader, and the greedy continuations must agree token for token. Covers sandwich norms,
(1 + w) norm weights, GeGLU, the embedding scale, QK-norm, the custom query scale and the
sliding / global layer pattern with two RoPE bases."""
import pytest
import torch

from minisglang_rdna4_b200 import SamplingParams
from minisglang_rdna4_b200.llm import LLM

transformers = pytest.importorskip("transformers")


def _tiny_gemma3(tmp_path):
    try:
        from transformers import Gemma3ForCausalLM, Gemma3TextConfig
    except ImportError:
        pytest.skip("this transformers build has no Gemma3")
    cfg = Gemma3TextConfig(
        vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=4, num_attention_heads=4,
        num_key_value_heads=2, head_dim=64, max_position_embeddings=512, rms_norm_eps=1e-6, sliding_window=16,
        query_pre_attn_scalar=48, rope_theta=1e6, rope_local_base_freq=1e4, sliding_window_pattern=2,
        layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"],
        tie_word_embeddings=True, attention_bias=False, final_logit_softcapping=None, attn_logit_softcapping=None,
        pad_token_id=0, bos_token_id=2, eos_token_id=1, torch_dtype="float32",
    )
    torch.manual_seed(0)
    model = Gemma3ForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for name, p in model.named_parameters():
            if "norm" in name:
                p.copy_(0.1 * torch.randn_like(p))  # exercise the (1 + w) convention
    model.save_pretrained(tmp_path, safe_serialization=True)
    return model, cfg


def test_gemma3_matches_transformers_greedy(tmp_path):
    hf, cfg = _tiny_gemma3(tmp_path)
    llm = LLM(model_path=str(tmp_path), device="cpu", page_size=16, max_running_req=4, num_page_override=128,
              max_extend_tokens=64, seed=0, dtype="float32")
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(3, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 40, 23)]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    for prompt, out in zip(prompts, outs):
        ids = torch.tensor([prompt])
        with torch.no_grad():
            want = hf.generate(ids, max_new_tokens=12, do_sample=False, eos_token_id=None, pad_token_id=0)[0, len(prompt):]
        assert out.token_ids == want.tolist(), (out.token_ids, want.tolist())


def test_sliding_window_layers_in_a_pool_of_their_own(tmp_path, monkeypatch):
    """``MSGL_SWA_POOL=1``: the sliding-window layers keep their K/V in a second pool whose pages go
    back to its free list as they leave the window. Outputs equal the one-pool engine and the
    reference implementation; a request never holds more than window / page + 3 pages there, however long
    its context; every page is back when the requests are done."""
    hf, cfg = _tiny_gemma3(tmp_path)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(3, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 150, 23, 77)]
    sp = SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True)
    kw = dict(model_path=str(tmp_path), device="cpu", page_size=16, max_running_req=4, num_page_override=128,
              max_extend_tokens=48, seed=0, dtype="float32")
    plain = LLM(**kw)
    want = [o.token_ids for o in plain.generate(prompts, sp)]
    assert plain.engine.swa is None
    plain.shutdown()
    monkeypatch.setenv("MSGL_SWA_POOL", "1")
    llm = LLM(**kw)
    eng = llm.engine
    assert eng.swa is not None and eng.kv_layers == 2 and eng.swa_kv_cache.num_layers == 2
    assert type(llm.cache.prefix_cache).__name__ == "SnapshotRadixCache"
    got = [o.token_ids for o in llm.generate(prompts, sp)]
    assert got == want
    eng.swa.check()
    # what is still held are the windows kept for prefix reuse (two pages each at window 16, page 16)
    assert eng.swa.in_use == int((eng.swa.refs[: eng.swa.num_pages] > 0).sum()) <= 2 * eng.swa.num_snapshots
    # window 16, page 16: two pages of window, the page being written, one prefill chunk of 48 tokens
    assert eng.swa.peak_in_use <= 4 * (1 + 3) + 3, eng.swa.peak_in_use
    ids = torch.tensor([prompts[1]])
    with torch.no_grad():
        ref = hf.generate(ids, max_new_tokens=40, do_sample=False, eos_token_id=None, pad_token_id=0)[0, len(prompts[1]):]
    assert got[1] == ref.tolist()
    # prefix reuse: a follow-up that extends the 150-token prompt (and its answer) starts from a kept window
    follow = prompts[1] + got[1][:20] + [7, 8, 9]
    again = llm.generate([follow], sp)[0]
    assert again.cached_tokens >= 96, again.cached_tokens
    eng.swa.check()
    llm.shutdown()
    monkeypatch.setenv("MSGL_SWA_POOL", "0")
    plain = LLM(**kw)
    assert plain.generate([follow], sp)[0].token_ids == again.token_ids
    plain.shutdown()
    monkeypatch.setenv("MSGL_SWA_POOL", "1")
    monkeypatch.setenv("MSGL_RECURRENT_SNAPSHOT_MIB", "0")           # no kept windows: no reuse, nothing retained
    bare = LLM(**kw)
    assert type(bare.cache.prefix_cache).__name__ == "NaivePrefixCache"
    assert [o.token_ids for o in bare.generate(prompts[:2], sp)] == want[:2]
    assert bare.engine.swa.in_use == 0
    bare.shutdown()
    # a draft chain works with the pool (verify rows take pages like any other rows); a tree does not
    rep = [prompts[0][:6] * 8, prompts[2]]
    monkeypatch.setenv("MSGL_SWA_POOL", "0")
    ref_llm = LLM(**kw)
    want_rep = [o.token_ids for o in ref_llm.generate(rep, sp)]
    ref_llm.shutdown()
    monkeypatch.setenv("MSGL_SWA_POOL", "1")
    spec = LLM(spec_algorithm="ngram", spec_num_draft=3, **kw)
    assert [o.token_ids for o in spec.generate(rep, sp)] == want_rep
    assert spec.stats["spec_drafted"] > 0
    spec.engine.swa.check()
    spec.shutdown()
    with pytest.raises(ValueError, match="tree verification"):
        LLM(spec_algorithm="ngram", spec_num_draft=2, spec_tree_width=3, **kw)


def test_multimodal_gemma3_checkpoint_serves_its_text_decoder(tmp_path):
    """A ``Gemma3ForConditionalGeneration`` checkpoint (nested ``text_config``, tensors under
    ``model.language_model.*``, a vision tower and projector that are skipped) loads as the text
    decoder and generates what the Hugging Face model generates from token ids."""
    try:
        from transformers import Gemma3Config, Gemma3ForConditionalGeneration
    except ImportError:
        pytest.skip("this transformers build has no Gemma3 multimodal model")
    tc = dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=4, num_attention_heads=4,
              num_key_value_heads=2, head_dim=64, max_position_embeddings=512, rms_norm_eps=1e-6, sliding_window=16,
              query_pre_attn_scalar=48, rope_theta=1e6, rope_local_base_freq=1e4,
              layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"],
              tie_word_embeddings=True, pad_token_id=0, bos_token_id=2, eos_token_id=1)
    vc = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2, image_size=28, patch_size=14)
    cfg = Gemma3Config(text_config=tc, vision_config=vc, mm_tokens_per_image=4, image_token_index=500,
                       boi_token_index=501, eoi_token_index=502)
    torch.manual_seed(0)
    hf = Gemma3ForConditionalGeneration(cfg).float().eval()
    with torch.no_grad():
        for name, p in hf.named_parameters():
            if "norm" in name:
                p.copy_(0.1 * torch.randn_like(p))
    hf.save_pretrained(tmp_path, safe_serialization=True)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(3, 490, (n,), generator=g).tolist() for n in (9, 40)]
    want = [hf.generate(input_ids=torch.tensor([p]), max_new_tokens=8, do_sample=False, eos_token_id=None,
                        pad_token_id=0)[0, len(p):].tolist() for p in prompts]
    llm = LLM(model_path=str(tmp_path), device="cpu", page_size=16, max_running_req=4, num_page_override=64,
              max_extend_tokens=32, dtype="float32")
    got = [o.token_ids for o in llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))]
    llm.shutdown()
    assert got == want
