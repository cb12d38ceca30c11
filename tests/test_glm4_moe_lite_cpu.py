"""The GLM-4.x MoE "lite" family (multi-head latent attention, sigmoid routing with a selection
bias and shared experts, a dense first layer) on the CPU oracle path against the Hugging Face
implementation of the same checkpoint."""
import tempfile

import pytest
import torch

transformers = pytest.importorskip("transformers")


def _hf(tmp, n_group=1, topk_group=1, q_lora=24):
    from transformers import Glm4MoeLiteConfig, Glm4MoeLiteForCausalLM

    cfg = Glm4MoeLiteConfig(
        vocab_size=300, hidden_size=64, intermediate_size=128, moe_intermediate_size=32, num_hidden_layers=3,
        num_attention_heads=4, num_key_value_heads=4, n_shared_experts=1, n_routed_experts=8,
        routed_scaling_factor=1.8, kv_lora_rank=32, q_lora_rank=q_lora, qk_rope_head_dim=8, v_head_dim=32,
        qk_nope_head_dim=24, n_group=n_group, topk_group=topk_group, num_experts_per_tok=2,
        max_position_embeddings=512, eos_token_id=299, bos_token_id=None, pad_token_id=None)
    torch.manual_seed(0)
    model = Glm4MoeLiteForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for _, p in model.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn_like(p) * 0.08)
        for n, b in model.named_buffers():
            if "e_score_correction_bias" in n:
                b.copy_(torch.randn_like(b) * 0.1)
    model.save_pretrained(tmp, safe_serialization=True)
    return model


@pytest.mark.parametrize("n_group,topk_group,q_lora", [(1, 1, 24), (4, 2, None)])
def test_glm4_moe_lite_matches_transformers(n_group, topk_group, q_lora):
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    with tempfile.TemporaryDirectory() as tmp:
        hf = _hf(tmp, n_group, topk_group, q_lora)
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, 298, (n,), generator=g).tolist() for n in (5, 23, 41)]
        want = [hf.generate(torch.tensor([p]), max_new_tokens=8, do_sample=False)[0, len(p):].tolist() for p in prompts]
        llm = LLM(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64,
                  max_extend_tokens=32)
        mc = llm.engine.model_config
        assert mc.is_mla and mc.head_dim == 32 and mc.rotary_config.rotary_dim == 8 and mc.rotary_config.interleaved
        got = [o.token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))]
        llm.shutdown()
    assert got == want
