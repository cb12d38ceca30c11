"""Nemotron-H (Mamba-2 + attention + non-gated MoE hybrid) against the ``transformers`` implementation
on CPU: logits of a prompt through the engine's packed / paged / recurrent-state path, then greedy
decoding, which exercises the per-request convolution and state-space states across steps."""
import tempfile

import pytest
import torch

transformers = pytest.importorskip("transformers")


def _hf_model():
    from transformers.models.nemotron_h import NemotronHConfig, NemotronHForCausalLM

    torch.manual_seed(0)
    cfg = NemotronHConfig(
        vocab_size=300, hidden_size=64, layers_block_type=["mamba", "moe", "attention", "moe", "mamba"],
        num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=128, ssm_state_size=16,
        mamba_num_heads=4, mamba_head_dim=32, n_groups=2, n_routed_experts=4, num_experts_per_tok=2,
        moe_intermediate_size=32, moe_shared_expert_intermediate_size=48, chunk_size=8, n_group=1, topk_group=1,
        routed_scaling_factor=1.5, tie_word_embeddings=False, eos_token_id=299, max_position_embeddings=256)
    m = NemotronHForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith("A_log"):
                p.copy_(torch.log(torch.empty_like(p).uniform_(1.0, 8.0)))
            elif n.endswith(("dt_bias", ".D")):
                p.copy_(torch.randn_like(p) * 0.5)
            elif n.endswith("conv1d.bias"):
                p.copy_(torch.randn_like(p) * 0.1)
            elif "norm" in n:
                p.copy_(1 + 0.1 * torch.randn_like(p))
            else:
                p.copy_(torch.randn_like(p) * 0.08)
        for n, b in m.named_buffers():
            if n.endswith("e_score_correction_bias"):
                b.copy_(torch.randn_like(b) * 0.2)
    return cfg, m


def test_nemotron_h_matches_transformers():
    from safetensors.torch import save_file

    from minisglang_rdna4_b200 import LLM, SamplingParams

    cfg, hf = _hf_model()
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 298, (n,), generator=g).tolist() for n in (19, 7, 33)]
    new = 6
    want = []
    with torch.no_grad():
        for p in prompts:
            out = hf.generate(torch.tensor([p]), max_new_tokens=new, do_sample=False, use_cache=False)
            want.append(out[0, len(p):].tolist())
    with tempfile.TemporaryDirectory() as tmp:
        cfg.save_pretrained(tmp)
        state = {k: v.contiguous() for k, v in hf.state_dict().items()}
        save_file(state, f"{tmp}/model.safetensors")
        llm = LLM(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64,
                  max_extend_tokens=16)          # prompts longer than a chunk: states carry over between chunks
        try:
            assert llm.engine.model_config.layer_types == ("mamba", "moe", "attention", "moe", "mamba")
            assert llm.engine.kv_layers == 1 and llm.engine.gdn_state is not None
            got = [o.token_ids for o in llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=new,
                                                                             ignore_eos=True))]
        finally:
            llm.shutdown()
    assert got == want


def test_mamba2_reference_ops_agree_with_the_transformers_mixer():
    """The fp32 restatements of the three mixer ops (conv, scan, gate-first norm) reproduce the
    library mixer's output for a whole sequence and for the same sequence fed in two pieces."""
    from minisglang_rdna4_b200.ops import ref

    cfg, hf = _hf_model()
    mix = hf.model.layers[0].mixer
    x = torch.randn(1, 11, cfg.hidden_size) * 0.5
    with torch.no_grad():
        want = mix.torch_forward(x)[0]
        h, p, n, gr = cfg.mamba_num_heads, cfg.mamba_head_dim, cfg.ssm_state_size, cfg.n_groups
        inter, conv_dim = h * p, h * p + 2 * gr * n
        proj = x[0] @ mix.in_proj.weight.t()
        z, xbc_in, dt = proj[:, :inter], proj[:, inter:inter + conv_dim], proj[:, inter + conv_dim:]
        conv_state = torch.zeros(2, conv_dim, cfg.conv_kernel - 1)
        ssm = torch.zeros(2, h, p, n)
        slots = torch.tensor([1], dtype=torch.int32)
        outs = []
        for lo, hi, has in ((0, 4, 0), (4, 11, 1)):
            cu = torch.tensor([0, hi - lo], dtype=torch.int32)
            hs = torch.tensor([has], dtype=torch.int32)
            xbc = ref.causal_conv1d(xbc_in[lo:hi].contiguous(), mix.conv1d.weight[:, 0, :], conv_state, cu, slots, hs,
                                    mix.conv1d.bias)
            xs, b, c = xbc.split([inter, gr * n, gr * n], dim=-1)
            y = ref.mamba2_scan(xs.reshape(-1, h, p), dt[lo:hi], b.reshape(-1, gr, n), c.reshape(-1, gr, n), mix.A_log,
                                mix.D, mix.dt_bias, ssm, cu, slots, hs, cfg.time_step_min)
            y = ref.rms_norm_gate_first(y.reshape(-1, inter), z[lo:hi], mix.norm.weight, cfg.layer_norm_epsilon,
                                        inter // gr)
            outs.append(y @ mix.out_proj.weight.t())
        got = torch.cat(outs)
    assert torch.allclose(got, want, atol=2e-4, rtol=2e-3), float((got - want).abs().max())
