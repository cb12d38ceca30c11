import torch

from minisglang_rdna4_b200.ops import ref
from minisglang_rdna4_b200.weights import HostExpertTier, SLRUCache


def test_slru_protects_hot_keys_from_a_scan():
    c = SLRUCache(4, protected_fraction=0.5)
    for k in (1, 2):
        assert c.touch(k) is None
        c.admit(k)
    assert c.touch(1) is not None and c.touch(2) is not None      # promoted to protected
    for k in (10, 11, 12, 13, 14):                                # a scan of one-off keys
        assert c.touch(k) is None
        c.admit(k, pinned=[k])
    assert 1 in c and 2 in c and len(c) == 4
    assert c.evictions == 3
    slots = {c.slot_of(k) for k in (1, 2, 13, 14)}
    assert len(slots) == 4                                        # no slot is shared
    assert c.stats()["hit_rate"] > 0


def test_host_tier_matches_all_resident_experts():
    torch.manual_seed(0)
    e, h, inter, k, t = 16, 32, 24, 2, 12
    w13 = torch.randn(e, 2 * inter, h) * 0.1
    w2 = torch.randn(e, h, inter) * 0.1
    tier = HostExpertTier(w13, w2, slots=6, device="cpu")
    for step in range(6):
        x = torch.randn(t, h)
        # keep each step within the slab: route to at most 6 distinct experts
        pool = torch.randperm(e)[:5]
        ids = pool[torch.randint(0, 5, (t, k))].to(torch.int32)
        w = torch.rand(t, k)
        got = tier.forward(x, w, ids)
        want = ref.moe_forward(x, w13, w2, w, ids)
        assert torch.allclose(got, want, atol=1e-5), step
    assert tier.cache.misses > 0 and tier.cache.evictions > 0 and tier.bytes_copied > 0


def test_engine_with_host_expert_tier_matches_resident_engine():
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM
    from minisglang_rdna4_b200.models.config import ModelConfig, RotaryConfig

    cfg = ModelConfig(num_layers=2, num_qo_heads=2, num_kv_heads=1, head_dim=32, hidden_size=64, vocab_size=300,
                      intermediate_size=128, rms_norm_eps=1e-6, rotary_config=RotaryConfig(32, 32, 512, 1e4),
                      model_type="qwen3_moe", architectures=("Qwen3MoeForCausalLM",), qk_norm=True, num_experts=16,
                      num_experts_per_tok=2, moe_intermediate_size=32, torch_dtype="float32",
                      max_position_embeddings=512)
    prompts = [list(range(5, 25)), list(range(40, 49))]
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    kw = dict(model_config=cfg, use_dummy_weight=True, device="cpu", page_size=16, max_running_req=4,
              num_page_override=64, seed=2)
    want = [o.token_ids for o in LLM(**kw).generate(prompts, sp)]
    # 2 layers x 16 experts x 3*64*32*4 B = 786 KiB in total; allow roughly half of it on the "device"
    tiered = LLM(expert_cache_gb=0.0004, **kw)
    got = [o.token_ids for o in tiered.generate(prompts, sp)]
    assert got == want
    tiers = [m._tier for m in tiered.engine.model.modules() if getattr(m, "_tier", None) is not None]
    assert len(tiers) == 2 and all(t.slots < 16 for t in tiers) and sum(t.cache.misses for t in tiers) > 0
    from minisglang_rdna4_b200.layers.moe import MoELayer
    MoELayer.offload_slots = 0


def test_cpu_expert_tier_matches_fp32_reference():
    """The host library's e2m1 expert MLPs (fp32-activation and int8-activation inner products)
    against the PyTorch restatement, including a skipped (negative) expert id."""
    import torch

    from minisglang_rdna4_b200.quant import mxfp4
    from minisglang_rdna4_b200.weights.cpu_experts import CpuExpertTier

    torch.manual_seed(0)
    experts, hidden, inter = 6, 256, 128
    tier = CpuExpertTier(experts, hidden, inter, group=32, threads=4)
    for e in range(experts - 1):  # the last expert is not resident on the host
        w13, sf13 = mxfp4.quantize_mxfp4(torch.randn(2 * inter, hidden) * 0.05)
        w2, sf2 = mxfp4.quantize_mxfp4(torch.randn(hidden, inter) * 0.05)
        tier.set_expert(e, w13, torch.pow(2.0, sf13.float() - 127), w2, torch.pow(2.0, sf2.float() - 127))
    x = torch.randn(9, hidden)
    ids = torch.randint(0, experts, (9, 3), dtype=torch.int32)
    ids[0, 0] = -1
    w = torch.softmax(torch.randn(9, 3), -1)
    want = tier.reference(x, ids, w)
    got = tier.forward(x, ids, w)
    assert float((got - want).abs().max()) < 1e-4 * max(1.0, float(want.abs().max()))
    got8 = tier.forward(x, ids, w, int8_activations=True)
    assert float((got8 - want).abs().max()) < 0.05 * float(want.abs().max())
    assert tier.isa in ("scalar", "avx512-fp32", "avx512-vnni-int8")
    tier.close()
