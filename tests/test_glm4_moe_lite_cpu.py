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


def test_next_token_layer_of_the_checkpoint_drafts_exactly():
    """``--spec-algorithm mtp`` on a checkpoint with ``num_nextn_predict_layers`` builds the layer stored
    after the decoder (``model.layers.<L>``: enorm, hnorm, eh_proj, latent attention, experts,
    shared_head.norm) from the target's own layer class. Its output equals a dense Hugging Face
    restatement of the same tensors, and generation equals plain decoding."""
    import json

    from safetensors.torch import load_file, save_file
    from transformers.models.glm4_moe_lite import modeling_glm4_moe_lite as m

    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    with tempfile.TemporaryDirectory() as tmp:
        hf = _hf(tmp)
        cfg = hf.config
        cfg._attn_implementation = "eager"
        torch.manual_seed(3)
        L = cfg.num_hidden_layers
        layer = m.Glm4MoeLiteDecoderLayer(cfg, L - 1).float().eval()          # an expert layer, like the stored one
        eh = torch.nn.Linear(2 * cfg.hidden_size, cfg.hidden_size, bias=False)
        en, hn, sn = (m.Glm4MoeLiteRMSNorm(cfg.hidden_size, eps=cfg.rms_norm_eps) for _ in range(3))
        with torch.no_grad():
            for mod in (layer, eh, en, hn, sn):
                for p in mod.parameters():
                    p.copy_(torch.randn_like(p) * (0.08 if p.dim() >= 2 else 0.1) + (1.0 if p.dim() == 1 else 0.0))
            for n, b in layer.named_buffers():
                if "e_score_correction_bias" in n:
                    b.copy_(torch.randn_like(b) * 0.1)
        st = load_file(f"{tmp}/model.safetensors")
        for k, v in layer.state_dict().items():
            st[f"model.layers.{L}.{k}"] = v.contiguous()
        st[f"model.layers.{L}.eh_proj.weight"] = eh.weight.detach()
        st[f"model.layers.{L}.enorm.weight"] = en.weight.detach()
        st[f"model.layers.{L}.hnorm.weight"] = hn.weight.detach()
        st[f"model.layers.{L}.shared_head.norm.weight"] = sn.weight.detach()
        st[f"model.layers.{L}.shared_head.head.weight"] = hf.lm_head.weight.detach().clone()
        st[f"model.layers.{L}.embed_tokens.weight"] = hf.model.embed_tokens.weight.detach().clone()
        save_file(st, f"{tmp}/model.safetensors")
        c = json.load(open(f"{tmp}/config.json"))
        c["num_nextn_predict_layers"] = 1
        json.dump(c, open(f"{tmp}/config.json", "w"))

        g = torch.Generator().manual_seed(2)
        ids = torch.randint(0, 298, (1, 19), generator=g)
        n = ids.shape[1] - 1
        with torch.no_grad():
            hid = hf(ids, output_hidden_states=True).hidden_states[-1][0]
            emb = hf.model.embed_tokens(ids)[0]
            x = eh(torch.cat([en(emb[1:]), hn(hid[:-1])], -1))[None]
            pos = torch.arange(n)[None]
            pe = m.Glm4MoeLiteRotaryEmbedding(cfg)(x, pos)
            mask = torch.full((n, n), float("-inf")).triu(1)[None, None]
            y = layer(x, position_embeddings=pe, attention_mask=mask, position_ids=pos)
            y = (y[0] if isinstance(y, tuple) else y)[0]
            want_logits = hf.lm_head(sn(y[-1:]))

        kw = dict(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64)
        llm = LLM(spec_algorithm="mtp", spec_num_draft=2, **kw)
        prop = llm.proposer
        assert type(prop).__name__ == "MTPProposer" and type(prop.draft).__name__ == "GlmMTPDraft"
        assert prop.loaded_tensors >= 10
        got_hidden, got_logits = prop.draft.forward_rows(-7, emb[1:], hid[:-1], torch.arange(n, dtype=torch.int32))
        prop.draft.drop(-7)
        assert torch.allclose(got_hidden, y, atol=2e-5), float((got_hidden - y).abs().max())
        assert torch.allclose(got_logits, want_logits, atol=2e-5)
        prompts = [ids[0].tolist(), torch.randint(0, 298, (9,), generator=g).tolist()]
        sp = SamplingParams(max_tokens=12, ignore_eos=True)
        got = [o.token_ids for o in llm.generate(prompts, sp)]
        assert llm.stats["spec_drafted"] > 0
        llm.shutdown()
        plain = LLM(**kw)
        want = [o.token_ids for o in plain.generate(prompts, sp)]
        plain.shutdown()
    assert got == want


@pytest.mark.parametrize("yarn", [False, True])
def test_deepseek_v3_with_narrower_value_heads_matches_transformers(yarn):
    """DeepSeek-V3 geometry: the value heads (16 here, 128 in the released models) are narrower than
    the key heads (nope + rope = 32 here, 192 there). Queries, keys and values are zero-padded to one
    width in the paged pool, which changes no dot product; the padding channels of the output are dropped
    before the output projection. With YaRN as DeepSeek configures it (``mscale`` and ``mscale_all_dim``: the
    rotary table carries the ratio of the two magnitude factors, the softmax scale the square of the second)
    and prompts past the original context length."""
    from transformers import DeepseekV3Config, DeepseekV3ForCausalLM

    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM
    from minisglang_rdna4_b200.models.config import ModelConfig

    cfg = DeepseekV3Config(
        vocab_size=300, hidden_size=64, intermediate_size=128, moe_intermediate_size=32, num_hidden_layers=3,
        num_attention_heads=4, num_key_value_heads=4, n_shared_experts=1, n_routed_experts=8, routed_scaling_factor=2.5,
        kv_lora_rank=32, q_lora_rank=24, qk_rope_head_dim=8, v_head_dim=16, qk_nope_head_dim=24, n_group=2,
        topk_group=1, num_experts_per_tok=2, first_k_dense_replace=1, max_position_embeddings=512, eos_token_id=299,
        bos_token_id=None, pad_token_id=None,
        **(dict(rope_parameters=dict(rope_type="yarn", factor=4.0, original_max_position_embeddings=64, beta_fast=32,
                                     beta_slow=1, mscale=1.0, mscale_all_dim=0.7, rope_theta=10000.0)) if yarn else {}))
    torch.manual_seed(0)
    hf = DeepseekV3ForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for _, p in hf.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn_like(p) * 0.08)
        for n, b in hf.named_buffers():
            if "e_score_correction_bias" in n:
                b.copy_(torch.randn_like(b) * 0.1)
    # the released geometry is stored 256 wide (192 key channels, 128 value channels)
    real = ModelConfig.from_hf(dict(cfg.to_dict(), qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
                                    num_attention_heads=16, hidden_size=512, kv_lora_rank=512, q_lora_rank=None))
    assert real.head_dim == 256 and real.rotary_config.rotary_dim == 64
    with tempfile.TemporaryDirectory() as tmp:
        hf.save_pretrained(tmp, safe_serialization=True)
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, 298, (n,), generator=g).tolist() for n in ((5, 150, 90) if yarn else (5, 23, 41))]
        want = [hf.generate(torch.tensor([p]), max_new_tokens=8, do_sample=False)[0, len(p):].tolist() for p in prompts]
        llm = LLM(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64,
                  max_extend_tokens=32)
        assert llm.engine.model_config.head_dim == 32
        got = [o.token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))]
        llm.shutdown()
    assert got == want


def test_deepseek_v2_softmax_routing_matches_transformers():
    """DeepSeek-V2: the same latent attention, experts scored with a softmax and no selection bias,
    plain top-k (``topk_method: greedy`` ignores the groups the config lists), weights times the
    routed scaling factor without renormalisation."""
    from transformers import DeepseekV2Config, DeepseekV2ForCausalLM

    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM
    from minisglang_rdna4_b200.ops import ref

    cfg = DeepseekV2Config(
        vocab_size=300, hidden_size=64, intermediate_size=128, moe_intermediate_size=32, num_hidden_layers=3,
        num_attention_heads=4, num_key_value_heads=4, n_shared_experts=1, n_routed_experts=8, routed_scaling_factor=1.3,
        kv_lora_rank=32, q_lora_rank=None, qk_rope_head_dim=8, v_head_dim=16, qk_nope_head_dim=24, n_group=2,
        topk_group=1, num_experts_per_tok=2, first_k_dense_replace=1, topk_method="greedy", norm_topk_prob=False,
        max_position_embeddings=512, eos_token_id=299, bos_token_id=None, pad_token_id=None)
    torch.manual_seed(0)
    hf = DeepseekV2ForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for _, p in hf.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn_like(p) * 0.08)
    with tempfile.TemporaryDirectory() as tmp:
        hf.save_pretrained(tmp, safe_serialization=True)
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(3, 298, (n,), generator=g).tolist() for n in (5, 41, 23)]
        want = [hf.generate(torch.tensor([p]), max_new_tokens=10, do_sample=False, eos_token_id=None, pad_token_id=0
                            )[0, len(p):].tolist() for p in prompts]
        llm = LLM(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64,
                  max_extend_tokens=32)
        mc = llm.engine.model_config
        assert mc.scoring_func == "softmax" and mc.n_group == 1
        got = [o.token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=10, ignore_eos=True))]
        llm.shutdown()
    assert got == want
    # group_limited_greedy: a group is as good as its best expert; only the best groups' experts are eligible
    logits = torch.tensor([[3.0, 0.0, 0.0, 0.0, 2.9, 2.8, 2.7, 2.6]])
    w, ids = ref.moe_route_grouped(logits, 2, False, "softmax", None, 1.0, n_group=2, topk_group=1)
    assert min(ids[0].tolist()) == 0 and max(ids[0].tolist()) < 4     # the first group holds the single best expert
    bias = torch.zeros(8)
    w2, ids2 = ref.moe_route_grouped(logits, 2, False, "softmax", bias, 1.0, n_group=2, topk_group=1)
    assert min(ids2[0].tolist()) >= 4               # with a selection bias: the sum of the two best decides


def test_glm4_moe_next_token_layer_drafts_exactly():
    """GLM-4.5's next-token layer (``model.layers.<L>`` with enorm / hnorm / eh_proj around an ordinary
    grouped-query attention layer with q/k/v biases, QK norm and partial rotary embedding, the expert
    block, shared_head.norm) against a Hugging Face restatement; generation equals plain decoding."""
    import json

    import transformers as T
    from safetensors.torch import load_file, save_file
    from transformers.models.glm4_moe import modeling_glm4_moe as m

    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    cfg = T.Glm4MoeConfig(
        vocab_size=300, hidden_size=64, intermediate_size=128, moe_intermediate_size=32, num_hidden_layers=3,
        num_attention_heads=4, num_key_value_heads=2, head_dim=32, n_shared_experts=1, n_routed_experts=8,
        routed_scaling_factor=1.7, n_group=2, topk_group=1, num_experts_per_tok=2, first_k_dense_replace=1,
        use_qk_norm=True, attention_bias=True, max_position_embeddings=512, eos_token_id=299, bos_token_id=None,
        pad_token_id=None, tie_word_embeddings=False)
    cfg._attn_implementation = "eager"
    torch.manual_seed(0)
    hf = T.Glm4MoeForCausalLM(cfg).float().eval()
    L = cfg.num_hidden_layers
    layer = m.Glm4MoeDecoderLayer(cfg, L - 1).float().eval()
    eh = torch.nn.Linear(2 * cfg.hidden_size, cfg.hidden_size, bias=False)
    en, hn, sn = (m.Glm4MoeRMSNorm(cfg.hidden_size, eps=cfg.rms_norm_eps) for _ in range(3))
    with torch.no_grad():
        for mod in (hf, layer, eh, en, hn, sn):
            for name, p in mod.named_parameters():
                if p.dim() >= 2:
                    p.copy_(torch.randn_like(p) * 0.1)
                elif "bias" in name:
                    p.copy_(torch.randn_like(p) * 0.1)
                else:
                    p.copy_(0.1 * torch.randn_like(p) + 1.0)
            for name, b in mod.named_buffers():
                if "e_score_correction_bias" in name:
                    b.copy_(torch.randn_like(b) * 0.1)
    with tempfile.TemporaryDirectory() as tmp:
        hf.save_pretrained(tmp, safe_serialization=True)
        st = load_file(f"{tmp}/model.safetensors")
        for k, v in layer.state_dict().items():
            st[f"model.layers.{L}.{k}"] = v.contiguous()
        st[f"model.layers.{L}.eh_proj.weight"] = eh.weight.detach()
        st[f"model.layers.{L}.enorm.weight"] = en.weight.detach()
        st[f"model.layers.{L}.hnorm.weight"] = hn.weight.detach()
        st[f"model.layers.{L}.shared_head.norm.weight"] = sn.weight.detach()
        save_file(st, f"{tmp}/model.safetensors")
        c = json.load(open(f"{tmp}/config.json"))
        c["num_nextn_predict_layers"] = 1
        json.dump(c, open(f"{tmp}/config.json", "w"))
        g = torch.Generator().manual_seed(2)
        ids = torch.randint(0, 298, (1, 19), generator=g)
        n = ids.shape[1] - 1
        with torch.no_grad():
            hid = hf(ids, output_hidden_states=True).hidden_states[-1][0]
            emb = hf.model.embed_tokens(ids)[0]
            x = eh(torch.cat([en(emb[1:]), hn(hid[:-1])], -1))[None]
            pos = torch.arange(n)[None]
            pe = m.Glm4MoeRotaryEmbedding(cfg)(x, pos)
            mask = torch.full((n, n), float("-inf")).triu(1)[None, None]
            y = layer(x, position_embeddings=pe, attention_mask=mask, position_ids=pos)
            y = (y[0] if isinstance(y, tuple) else y)[0]
            want_logits = hf.lm_head(sn(y[-1:]))
        kw = dict(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64)
        llm = LLM(spec_algorithm="mtp", spec_num_draft=2, **kw)
        prop = llm.proposer
        assert type(prop.draft).__name__ == "Glm4MoeMTPDraft" and prop.loaded_tensors >= 10
        got_hidden, got_logits = prop.draft.forward_rows(-7, emb[1:], hid[:-1], torch.arange(n, dtype=torch.int32))
        prop.draft.drop(-7)
        assert torch.allclose(got_hidden, y, atol=2e-5), float((got_hidden - y).abs().max())
        assert torch.allclose(got_logits, want_logits, atol=2e-5)
        prompts = [ids[0].tolist(), torch.randint(0, 298, (9,), generator=g).tolist()]
        sp = SamplingParams(max_tokens=12, ignore_eos=True)
        got = [o.token_ids for o in llm.generate(prompts, sp)]
        assert llm.stats["spec_drafted"] > 0
        llm.shutdown()
        plain = LLM(**kw)
        want = [o.token_ids for o in plain.generate(prompts, sp)]
        plain.shutdown()
    assert got == want


@pytest.mark.parametrize("family", ["glm_lite", "deepseek_v3"])
def test_latent_pool_with_absorbed_attention_matches_transformers(family, monkeypatch):
    """MSGL_MLA_LATENT: the pool holds kv_lora_rank + rope values per token and layer (40 here against
    256 for per-head keys and values); queries go through the key half of kv_b_proj into the latent
    space and the attended latents come back through its value half. Chunked prefill (the second
    chunk attends to latents stored by the first), batched decode and prefix reuse give the tokens of the
    Hugging Face model, which expands the latents per head."""
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.kvcache.mla_pool import MLALatentCache
    from minisglang_rdna4_b200.llm import LLM

    monkeypatch.setenv("MSGL_MLA_LATENT", "1")
    with tempfile.TemporaryDirectory() as tmp:
        if family == "glm_lite":
            hf = _hf(tmp, 4, 2, 24)
        else:
            from transformers import DeepseekV3Config, DeepseekV3ForCausalLM

            cfg = DeepseekV3Config(
                vocab_size=300, hidden_size=64, intermediate_size=128, moe_intermediate_size=32, num_hidden_layers=3,
                num_attention_heads=4, num_key_value_heads=4, n_shared_experts=1, n_routed_experts=8,
                routed_scaling_factor=2.5, kv_lora_rank=32, q_lora_rank=None, qk_rope_head_dim=8, v_head_dim=16,
                qk_nope_head_dim=24, n_group=2, topk_group=1, num_experts_per_tok=2, first_k_dense_replace=1,
                max_position_embeddings=512, eos_token_id=299, bos_token_id=None, pad_token_id=None,
                rope_parameters=dict(rope_type="yarn", factor=4.0, original_max_position_embeddings=64, beta_fast=32,
                                     beta_slow=1, mscale=1.0, mscale_all_dim=0.7, rope_theta=10000.0))
            torch.manual_seed(0)
            hf = DeepseekV3ForCausalLM(cfg).float().eval()
            with torch.no_grad():
                for _, p in hf.named_parameters():
                    if p.dim() >= 2:
                        p.copy_(torch.randn_like(p) * 0.08)
            hf.save_pretrained(tmp, safe_serialization=True)
        g = torch.Generator().manual_seed(1)
        shared = torch.randint(0, 298, (48,), generator=g).tolist()
        prompts = [torch.randint(0, 298, (n,), generator=g).tolist() for n in (5, 90, 41)]
        prompts.append(shared + [7, 8, 9])
        want = [hf.generate(torch.tensor([p]), max_new_tokens=8, do_sample=False)[0, len(p):].tolist() for p in prompts]
        llm = LLM(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64,
                  max_extend_tokens=32)
        pool = llm.engine.kv_cache
        assert isinstance(pool, MLALatentCache) and pool.width == 40 and llm.engine.graph_runner is None
        got = [o.token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))]
        # a second request over the same 48-token prefix reads the latents the first one left in the pool
        again = shared + [11, 12]
        want2 = hf.generate(torch.tensor([again]), max_new_tokens=6, do_sample=False)[0, len(again):].tolist()
        got2 = llm.generate([again], SamplingParams(max_tokens=6, ignore_eos=True))[0]
        llm.shutdown()
    assert got == want
    assert got2.token_ids == want2 and got2.cached_tokens >= 32


def test_latent_pool_refuses_what_it_cannot_serve(monkeypatch):
    from minisglang_rdna4_b200.llm import LLM

    monkeypatch.setenv("MSGL_MLA_LATENT", "1")
    with tempfile.TemporaryDirectory() as tmp:
        _hf(tmp)
        with pytest.raises(ValueError, match="does not verify drafts"):
            LLM(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64,
                spec_algorithm="ngram")
