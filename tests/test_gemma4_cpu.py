"""Gemma-4 text decoders on the CPU oracle path against the Hugging Face implementation of the same
checkpoint: per-layer head geometry, keys reused as values, K/V shared by the last layers, per-layer
input embeddings, the layer scalar and the expert block beside the dense MLP."""
import tempfile

import pytest
import torch

transformers = pytest.importorskip("transformers")

_KINDS = {
    # the small models: one K/V head, per-layer input embeddings, the last layers read earlier K/V and have
    # a double-wide MLP
    "shared_kv_ple": dict(num_hidden_layers=6, num_key_value_heads=1, num_kv_shared_layers=3, use_double_wide_mlp=True,
                          hidden_size_per_layer_input=8, vocab_size_per_layer_input=300,
                          layer_types=["sliding_attention", "full_attention", "sliding_attention", "sliding_attention",
                                       "sliding_attention", "full_attention"]),
    # the dense large model: global layers with fewer, wider K/V heads whose keys are their values
    "k_eq_v": dict(num_hidden_layers=4, num_key_value_heads=2, num_global_key_value_heads=1, attention_k_eq_v=True,
                   hidden_size_per_layer_input=0,
                   layer_types=["sliding_attention", "sliding_attention", "sliding_attention", "full_attention"]),
    # the sparse model: experts beside the MLP
    "moe": dict(num_hidden_layers=3, num_key_value_heads=2, enable_moe_block=True, num_experts=8, top_k_experts=2,
                moe_intermediate_size=16, hidden_size_per_layer_input=0, final_logit_softcapping=30.0,
                layer_types=["sliding_attention", "sliding_attention", "full_attention"]),
}


def _hf(tmp, kind):
    from transformers import Gemma4ForCausalLM, Gemma4TextConfig

    cfg = Gemma4TextConfig(vocab_size=300, hidden_size=64, intermediate_size=96, num_attention_heads=4, head_dim=16,
                           global_head_dim=32, sliding_window=16, max_position_embeddings=512, eos_token_id=299,
                           bos_token_id=None, pad_token_id=0, **_KINDS[kind])
    torch.manual_seed(0)
    model = Gemma4ForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn_like(p) * 0.08)
            elif "norm" in name or "scale" in name:
                p.copy_(1.0 + torch.randn_like(p) * 0.1)
        for name, b in model.named_buffers():
            if name.endswith("layer_scalar"):
                b.copy_(torch.rand_like(b) * 0.5 + 0.75)
    model.save_pretrained(tmp, safe_serialization=True)
    return model


@pytest.mark.parametrize("kind", list(_KINDS))
def test_gemma4_matches_transformers(kind):
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    with tempfile.TemporaryDirectory() as tmp:
        hf = _hf(tmp, kind)
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(1, 298, (n,), generator=g).tolist() for n in (5, 70, 41)]
        want = [hf.generate(torch.tensor([p]), max_new_tokens=8, do_sample=False)[0, len(p):].tolist() for p in prompts]
        llm = LLM(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64,
                  max_extend_tokens=32)
        mc = llm.engine.model_config
        assert mc.mixed_kv_geometry and mc.num_kv_layers == mc.num_layers - mc.num_kv_shared_layers
        got = [o.token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))]
        llm.shutdown()
    assert got == want


def test_gemma4_with_the_sliding_window_pool(monkeypatch):
    """Two pools, each with the geometry of its layers (one narrow K/V head for the sliding layers, one wide
    head for the global ones); layers that share K/V follow their donor into its pool. A second request over
    the same prefix reuses pages of both pools."""
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    monkeypatch.setenv("MSGL_SWA_POOL", "1")
    with tempfile.TemporaryDirectory() as tmp:
        hf = _hf(tmp, "shared_kv_ple")
        g = torch.Generator().manual_seed(3)
        shared = torch.randint(1, 298, (64,), generator=g).tolist()
        prompts = [torch.randint(1, 298, (n,), generator=g).tolist() for n in (5, 70)] + [shared + [3, 4, 5]]
        again = shared + [9, 8]
        want = [hf.generate(torch.tensor([p]), max_new_tokens=8, do_sample=False)[0, len(p):].tolist()
                for p in prompts + [again]]
        llm = LLM(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64,
                  max_extend_tokens=32)
        eng = llm.engine
        assert eng.swa is not None and eng.kv_cache.head_dim == 32 and eng.swa_kv_cache.head_dim == 16
        assert eng.kv_cache.num_layers == 1 and eng.swa_kv_cache.num_layers == 2       # 3 of 6 layers keep K/V
        got = [o.token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))]
        second = llm.generate([again], SamplingParams(max_tokens=8, ignore_eos=True))[0]
        llm.shutdown()
    assert got == want[:3]
    assert second.token_ids == want[3] and second.cached_tokens >= 32


def test_gemma4_moe_tp2_matches_transformers():
    """Heads, MLP and expert width split over two ranks; the router and the per-layer pieces are replicated."""
    import multiprocessing as mp
    import os

    from test_tp_cpu import _worker

    with tempfile.TemporaryDirectory() as tmp:
        hf = _hf(tmp, "moe")
        g = torch.Generator().manual_seed(2)
        prompts = [torch.randint(1, 298, (n,), generator=g).tolist() for n in (9, 40)]
        want = [hf.generate(torch.tensor([p]), max_new_tokens=6, do_sample=False)[0, len(p):].tolist() for p in prompts]
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        port = 22100 + (os.getpid() % 1500)
        procs = [ctx.Process(target=_worker, args=(r, 2, port, tmp, prompts, q, False)) for r in range(2)]
        for p in procs:
            p.start()
        got = q.get(timeout=240)
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    assert got == want
