"""Every decoder family served through ``models/transformer.py`` and ``models/gemma.py`` against the
Hugging Face implementation of a tiny random checkpoint of that family, on the CPU oracle path:
the checkpoint goes through this package's loader (q/k/v and gate/up merges, expert stacking, tied
heads), prompts longer than a prefill chunk exercise the chunked path, and greedy continuations
must agree token for token."""
import tempfile

import pytest
import torch

T = pytest.importorskip("transformers")

COMMON = dict(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4,
              num_key_value_heads=2, max_position_embeddings=512, rms_norm_eps=1e-6, tie_word_embeddings=False,
              eos_token_id=299, bos_token_id=None, pad_token_id=None)
MOE = dict(moe_intermediate_size=32, num_experts=8, num_experts_per_tok=2, decoder_sparse_step=1, mlp_only_layers=[])
FAMILIES = {
    "llama": ("LlamaConfig", "LlamaForCausalLM", dict(head_dim=16)),
    "llama_biases": ("LlamaConfig", "LlamaForCausalLM", dict(head_dim=16, attention_bias=True, mlp_bias=True)),
    "llama_tied": ("LlamaConfig", "LlamaForCausalLM", dict(head_dim=16, tie_word_embeddings=True)),
    "mistral": ("MistralConfig", "MistralForCausalLM", dict(sliding_window=16, head_dim=16)),        # window < context
    "qwen2": ("Qwen2Config", "Qwen2ForCausalLM", dict()),                                           # q/k/v biases
    "qwen3": ("Qwen3Config", "Qwen3ForCausalLM", dict(head_dim=32)),                                # per-head QK norm
    "qwen2_moe": ("Qwen2MoeConfig", "Qwen2MoeForCausalLM",
                  dict(shared_expert_intermediate_size=48, norm_topk_prob=False, **MOE)),           # gated shared expert
    "qwen3_moe": ("Qwen3MoeConfig", "Qwen3MoeForCausalLM", dict(head_dim=32, norm_topk_prob=True, **MOE)),
    # experts on every second layer, one of those forced dense
    "qwen3_moe_mixed": ("Qwen3MoeConfig", "Qwen3MoeForCausalLM",
                        dict(head_dim=32, norm_topk_prob=False, num_hidden_layers=4,
                             **{**MOE, "decoder_sparse_step": 2, "mlp_only_layers": [1]})),
    "qwen2_window": ("Qwen2Config", "Qwen2ForCausalLM",
                     dict(use_sliding_window=True, sliding_window=16, max_window_layers=2, num_hidden_layers=4)),
    "gemma2": ("Gemma2Config", "Gemma2ForCausalLM",
               dict(head_dim=16, sliding_window=16, query_pre_attn_scalar=16, final_logit_softcapping=30.0,
                    attn_logit_softcapping=50.0, tie_word_embeddings=True)),
    "mixtral": ("MixtralConfig", "MixtralForCausalLM",
                dict(head_dim=16, intermediate_size=96, num_local_experts=8, num_experts_per_tok=2, sliding_window=None)),
    # GLM-4.5: partial rotary embedding, q/k/v biases, optional QK norm, sigmoid routing with a selection bias,
    # routing groups, a shared expert, a dense first layer
    "glm4_moe": ("Glm4MoeConfig", "Glm4MoeForCausalLM",
                 dict(head_dim=32, moe_intermediate_size=32, n_shared_experts=1, n_routed_experts=8,
                      routed_scaling_factor=1.7, n_group=2, topk_group=1, num_experts_per_tok=2, first_k_dense_replace=1,
                      use_qk_norm=True, attention_bias=True)),
}


@pytest.mark.parametrize("family", sorted(FAMILIES))
def test_family_matches_transformers(family):
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    cfg_name, model_name, extra = FAMILIES[family]
    if not hasattr(T, cfg_name):
        pytest.skip(f"this transformers build has no {cfg_name}")
    cfg = getattr(T, cfg_name)(**{**COMMON, **extra})
    torch.manual_seed(0)
    hf = getattr(T, model_name)(cfg).float().eval()
    with torch.no_grad():
        for name, p in hf.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn_like(p) * 0.1)
            elif "bias" in name:
                p.copy_(torch.randn_like(p) * 0.1)
            elif "norm" in name:                  # away from the neutral weight (zero for the (1 + w) families)
                p.copy_(0.1 * torch.randn_like(p) + (0.0 if family.startswith("gemma") else 1.0))
        for name, b in hf.named_buffers():
            if "e_score_correction_bias" in name:
                b.copy_(torch.randn_like(b) * 0.1)
    with tempfile.TemporaryDirectory() as tmp:
        hf.save_pretrained(tmp, safe_serialization=True)
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(3, 298, (n,), generator=g).tolist() for n in (5, 41, 23)]
        want = [hf.generate(torch.tensor([p]), max_new_tokens=10, do_sample=False, eos_token_id=None,
                            pad_token_id=0)[0, len(p):].tolist() for p in prompts]
        llm = LLM(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64,
                  max_extend_tokens=32)
        got = [o.token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=10, ignore_eos=True))]
        llm.shutdown()
    assert got == want


ROPE = {
    "llama3": dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                   original_max_position_embeddings=64, rope_theta=10000.0),
    "yarn": dict(rope_type="yarn", factor=4.0, original_max_position_embeddings=64, rope_theta=10000.0),
    "linear": dict(rope_type="linear", factor=2.0, rope_theta=10000.0),
}


@pytest.mark.parametrize("kind", sorted(ROPE))
def test_rope_scaling_matches_transformers(kind):
    """Long-context rotary scalings (Llama-3 frequency bands, YaRN with its attention factor, linear
    position interpolation) with prompts well past the original context length."""
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    cfg = T.LlamaConfig(**{**COMMON, "num_hidden_layers": 2, "head_dim": 16, "max_position_embeddings": 256},
                        rope_parameters=ROPE[kind])
    torch.manual_seed(0)
    hf = T.LlamaForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for _, p in hf.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn_like(p) * 0.1)
    with tempfile.TemporaryDirectory() as tmp:
        hf.save_pretrained(tmp, safe_serialization=True)
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(3, 298, (n,), generator=g).tolist() for n in (5, 150, 90)]
        want = [hf.generate(torch.tensor([p]), max_new_tokens=10, do_sample=False, eos_token_id=None,
                            pad_token_id=0)[0, len(p):].tolist() for p in prompts]
        llm = LLM(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64,
                  max_extend_tokens=64)
        got = [o.token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=10, ignore_eos=True))]
        llm.shutdown()
    assert got == want


def test_all_sliding_model_with_the_window_pool(monkeypatch):
    """Mistral (every layer has the window): with MSGL_SWA_POOL all K/V live in the recycled pool, the main
    pool keeps one unused layer; contexts several windows long still match the Hugging Face model."""
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    cfg = T.MistralConfig(**{**COMMON, "head_dim": 16, "sliding_window": 16})
    torch.manual_seed(0)
    hf = T.MistralForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for _, p in hf.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn_like(p) * 0.1)
    monkeypatch.setenv("MSGL_SWA_POOL", "1")
    with tempfile.TemporaryDirectory() as tmp:
        hf.save_pretrained(tmp, safe_serialization=True)
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(3, 298, (n,), generator=g).tolist() for n in (5, 100, 41)]
        want = [hf.generate(torch.tensor([p]), max_new_tokens=20, do_sample=False, eos_token_id=None,
                            pad_token_id=0)[0, len(p):].tolist() for p in prompts]
        llm = LLM(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64,
                  max_extend_tokens=32)
        assert llm.engine.swa is not None and llm.engine.kv_layers == 1 and llm.engine.swa_kv_cache.num_layers == 3
        got = [o.token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=20, ignore_eos=True))]
        llm.engine.swa.check()
        llm.shutdown()
    assert got == want
