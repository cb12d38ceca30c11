"""End-to-end engine checks on a GPU: the kernel path against the fp32 oracle path."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _cfg(layers=2, qk_norm=True):
    from minisglang_rdna4_b200.models.config import ModelConfig, RotaryConfig

    return ModelConfig(
        num_layers=layers, num_qo_heads=8, num_kv_heads=2, head_dim=128, hidden_size=512, vocab_size=2048,
        intermediate_size=1024, rms_norm_eps=1e-6,
        rotary_config=RotaryConfig(head_dim=128, rotary_dim=128, max_position=2048, base=1e6),
        model_type="qwen3", architectures=("Qwen3ForCausalLM",), qk_norm=qk_norm, max_position_embeddings=2048,
    )


def _prompts():
    g = torch.Generator().manual_seed(3)
    shared = torch.randint(0, 2048, (48,), generator=g).tolist()
    out = []
    for i, n in enumerate((33, 70, 150, 9, 200, 64)):
        body = torch.randint(0, 2048, (n,), generator=g).tolist()
        out.append(shared + body if i % 2 == 0 else body)
    return out


@pytest.mark.parametrize("quant,kv", [(None, "bf16"), ("mxfp4", "fp8"), ("fp8", "fp8")])
def test_generate_graph_matches_eager(quant, kv):
    """CUDA-graph decode must reproduce eager decode token for token, and a chunked prefill
    (small step budget) must reproduce an unchunked one."""
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM
    from minisglang_rdna4_b200.ops import cuda as K

    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    outs = {}
    for name, kw in (("graph", dict()), ("eager", dict(cuda_graph_max_bs=-1)),
                     ("chunked", dict(cuda_graph_max_bs=-1, max_extend_tokens=96))):
        llm = LLM(model_config=_cfg(), use_dummy_weight=True, quantization=quant, kv_cache_dtype=kv,
                  device="cuda", page_size=16, max_running_req=8, num_page_override=256, seed=0, **kw)
        outs[name] = [o.token_ids for o in llm.generate(_prompts(), sp)]
        assert K.gemm_status() == 0 and K.attn_status() == 0
        llm.cache.check_integrity()
        llm.shutdown()
    assert outs["graph"] == outs["eager"]
    assert outs["chunked"] == outs["eager"]


def test_bf16_engine_tracks_fp32_oracle():
    """Same random weights on the CPU fp32 oracle path: the first generated tokens agree for
    most prompts (bf16 rounding may flip near-ties later in a sequence)."""
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    gpu = LLM(model_config=_cfg(), use_dummy_weight=True, device="cuda", page_size=16, max_running_req=8,
              num_page_override=256, seed=0, cuda_graph_max_bs=-1)
    state = {k: v.float().cpu() for k, v in gpu.engine.model.state_dict().items()}
    got = [o.token_ids for o in gpu.generate(_prompts(), sp)]
    gpu.shutdown()
    cpu = LLM(model_config=_cfg(), use_dummy_weight=True, device="cpu", page_size=16, max_running_req=8,
              num_page_override=256, seed=0)
    cpu.engine.model.load_state_dict(state, strict=False)
    want = [o.token_ids for o in cpu.generate(_prompts(), sp)]
    cpu.shutdown()
    first_ok = sum(g[0] == w[0] for g, w in zip(got, want))
    assert first_ok >= len(want) - 1, (got, want)
