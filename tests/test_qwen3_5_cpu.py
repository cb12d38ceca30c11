"""The Qwen3.5 hybrid family (gated-delta-net + gated full attention) on the CPU oracle path against
the Hugging Face implementation of the same checkpoint: prefill logits agree, greedy decoding
through the engine (chunked prefill, recurrent state per request slot) reproduces the tokens the
Hugging Face model generates."""
import tempfile

import pytest
import torch

transformers = pytest.importorskip("transformers")


def _hf_model(tmp, moe=False):
    from transformers import Qwen3_5ForCausalLM, Qwen3_5TextConfig

    cfg = Qwen3_5TextConfig(
        vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
        num_key_value_heads=2, head_dim=32, linear_conv_kernel_dim=4, linear_key_head_dim=16,
        linear_value_head_dim=16, linear_num_key_heads=2, linear_num_value_heads=4, max_position_embeddings=512,
        rms_norm_eps=1e-6, tie_word_embeddings=False, eos_token_id=299, pad_token_id=None, bos_token_id=None,
    )
    torch.manual_seed(0)
    model = Qwen3_5ForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for name, p in model.named_parameters():
            if name.endswith("norm.weight") and "linear_attn" not in name:
                p.copy_(torch.randn_like(p) * 0.1)         # (1 + w) norms away from their neutral point
            elif "A_log" in name:
                p.copy_(torch.log(torch.empty_like(p).uniform_(1.0, 8.0)))
            elif "dt_bias" in name:
                p.copy_(torch.randn_like(p) * 0.5)
            elif p.dim() >= 2:
                p.copy_(torch.randn_like(p) * 0.08)
    model.save_pretrained(tmp, safe_serialization=True)
    return model


def test_qwen3_5_hybrid_matches_transformers():
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    with tempfile.TemporaryDirectory() as tmp:
        hf = _hf_model(tmp)
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, 298, (n,), generator=g).tolist() for n in (5, 23, 41)]
        want = []
        for p in prompts:
            out = hf.generate(torch.tensor([p]), max_new_tokens=8, do_sample=False, use_cache=True)
            want.append(out[0, len(p):].tolist())
        for extend in (4096, 16):                      # one-shot prefill and chunked prefill
            llm = LLM(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4,
                      num_page_override=64, max_extend_tokens=extend)
            assert llm.engine.model_config.is_recurrent and llm.engine.gdn_state is not None
            got = [o.token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))]
            assert got == want, (extend, got, want)
            # slots are reused: a second wave starts from clean states
            again = [o.token_ids for o in llm.generate(prompts[::-1], SamplingParams(max_tokens=8, ignore_eos=True))]
            assert again == want[::-1]
            llm.shutdown()


def test_gdn_reference_ops_match_transformers_kernels():
    """The recurrent rule, the causal convolution and the gated norm of ``ops.ref`` against the
    chunked / recurrent torch implementations that ship with transformers."""
    from transformers.models.qwen3_5 import modeling_qwen3_5 as M

    from minisglang_rdna4_b200.ops import ref

    torch.manual_seed(0)
    t, hk, hv, dk, dv = 37, 2, 4, 16, 16
    q, k = torch.randn(t, hk, dk), torch.randn(t, hk, dk)
    v = torch.randn(t, hv, dv)
    a, b = torch.randn(t, hv), torch.randn(t, hv)
    a_log, dt_bias = torch.log(torch.empty(hv).uniform_(1, 8)), torch.randn(hv) * 0.3
    g, beta = ref.gdn_gates(a, b, a_log, dt_bias)
    state = torch.zeros(3, hv, dk, dv)
    cu = torch.tensor([0, 20, 37], dtype=torch.int32)
    out = ref.gdn_recurrent(q, k, v, g, beta, state, cu, torch.tensor([2, 0]), torch.tensor([0, 0]))
    for lo, hi, slot in ((0, 20, 2), (20, 37, 0)):
        qq = q[lo:hi].repeat_interleave(hv // hk, 1)[None]
        kk = k[lo:hi].repeat_interleave(hv // hk, 1)[None]
        want, last = M.torch_chunk_gated_delta_rule(qq, kk, v[lo:hi][None], g[lo:hi][None], beta[lo:hi][None],
                                                    output_final_state=True, use_qk_l2norm_in_kernel=True)
        assert torch.allclose(out[lo:hi], want[0], atol=2e-4, rtol=1e-3)
        assert torch.allclose(state[slot], last[0], atol=2e-4, rtol=1e-3)
    # continuing from a stored state equals running the whole sequence at once
    state2 = torch.zeros(1, hv, dk, dv)
    z = torch.tensor([0])
    first = ref.gdn_recurrent(q[:11], k[:11], v[:11], g[:11], beta[:11], state2, torch.tensor([0, 11]), z, z)
    rest = ref.gdn_recurrent(q[11:20], k[11:20], v[11:20], g[11:20], beta[11:20], state2, torch.tensor([0, 9]), z,
                             torch.tensor([1]))
    assert torch.allclose(torch.cat([first, rest]), out[:20], atol=1e-5)
    # convolution with a rolling state
    c, kw = 24, 4
    x = torch.randn(t, c)
    w = torch.randn(c, kw)
    conv_state = torch.zeros(2, c, kw - 1)
    y = ref.causal_conv1d(x, w, conv_state, torch.tensor([0, 37]), z, z)
    want = torch.nn.functional.silu(torch.nn.functional.conv1d(x.t()[None], w[:, None], padding=kw - 1, groups=c)
                                    [0, :, :t].t())
    assert torch.allclose(y, want, atol=1e-5)
    conv_state.zero_()
    y1 = ref.causal_conv1d(x[:10], w, conv_state, torch.tensor([0, 10]), z, z)
    y2 = ref.causal_conv1d(x[10:], w, conv_state, torch.tensor([0, 27]), z, torch.tensor([1]))
    assert torch.allclose(torch.cat([y1, y2]), want, atol=1e-5)


def test_recurrent_model_reuses_a_prefix_through_state_snapshots(monkeypatch):
    """A hybrid model can take a prefix-cache hit only at a boundary whose recurrent state was kept.
    Snapshots are taken at page-aligned chunk ends and every N tokens; a later request that shares
    the prefix starts from the deepest such boundary, and generates exactly what it generates
    without any reuse."""
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    with tempfile.TemporaryDirectory() as tmp:
        _hf_model(tmp)
        g = torch.Generator().manual_seed(5)
        shared = torch.randint(0, 298, (100,), generator=g).tolist()
        first = shared + torch.randint(0, 298, (9,), generator=g).tolist()
        second = shared + torch.randint(0, 298, (21,), generator=g).tolist()
        third = first + [7, 8, 9]                                # a follow-up turn of the first request
        sp = SamplingParams(max_tokens=6, ignore_eos=True)
        kw = dict(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64,
                  max_extend_tokens=48)
        monkeypatch.setenv("MSGL_RECURRENT_SNAPSHOT_MIB", "0")
        plain = LLM(**kw)
        assert type(plain.cache.prefix_cache).__name__ == "NaivePrefixCache"
        want = [plain.generate([p], sp)[0].token_ids for p in (first, second, third)]
        plain.shutdown()
        monkeypatch.setenv("MSGL_RECURRENT_SNAPSHOT_MIB", "64")
        monkeypatch.setenv("MSGL_RECURRENT_SNAPSHOT_TOKENS", "32")
        llm = LLM(**kw)
        assert type(llm.cache.prefix_cache).__name__ == "SnapshotRadixCache"
        outs = [llm.generate([p], sp)[0] for p in (first, second, third)]
        assert [o.token_ids for o in outs] == want
        assert outs[0].cached_tokens == 0
        # the shared 100 tokens end inside a page; the deepest kept boundary below them is 96
        assert outs[1].cached_tokens == 96, outs[1].cached_tokens
        # the follow-up turn continues from a boundary inside the first request's own output
        assert outs[2].cached_tokens >= 96
        assert llm.cache.prefix_cache.num_snapshots > 0
        assert llm.engine.gdn_state.num_snapshots == llm.cache.prefix_cache.num_snapshots
        llm.cache.check_integrity()
        llm.shutdown()
        # the same with the snapshots in host frames of one slab (room for a few only: the cache evicts)
        monkeypatch.setenv("MSGL_RECURRENT_SNAPSHOT_HOST_MIB", "1")
        host = LLM(**kw)
        arena = host.engine.gdn_state._arena
        assert arena is not None and arena.num_frames >= 4
        outs = [host.generate([p], sp)[0] for p in (first, second, third)]
        assert [o.token_ids for o in outs] == want
        assert outs[1].cached_tokens == 96
        assert arena.num_free < arena.num_frames                     # kept snapshots live in frames
        assert len(host.engine.gdn_state._frames) == host.engine.gdn_state.num_snapshots
        host.shutdown()


@pytest.mark.parametrize("family", ["qwen3_5", "nemotron_h"])
def test_speculative_decoding_rolls_the_recurrent_state_back(family, monkeypatch):
    """A verify step advances the recurrent layers over every draft row. When part of the draft is
    rejected the states from before the step are put back and advanced again over the kept rows only,
    so a speculative engine generates what plain decoding generates."""
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    monkeypatch.setenv("MSGL_RECURRENT_SNAPSHOT_MIB", "0")
    g = torch.Generator().manual_seed(9)
    base = torch.randint(0, 298, (5,), generator=g).tolist()
    prompts = [base * 5, torch.randint(0, 298, (23,), generator=g).tolist(), (base[:3] + [11]) * 6]
    sp = SamplingParams(max_tokens=24, ignore_eos=True)
    with tempfile.TemporaryDirectory() as tmp:
        if family == "qwen3_5":
            _hf_model(tmp)
        else:
            from safetensors.torch import save_file
            from test_nemotron_h_cpu import _hf_model as nemotron

            cfg, hf = nemotron()
            cfg.save_pretrained(tmp)
            save_file({k: v.contiguous() for k, v in hf.state_dict().items()}, f"{tmp}/model.safetensors")
        kw = dict(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64)
        plain = LLM(**kw)
        want = [o.token_ids for o in plain.generate(prompts, sp)]
        plain.shutdown()
        llm = LLM(spec_algorithm="ngram", spec_num_draft=3, **kw)
        got = [o.token_ids for o in llm.generate(prompts, sp)]
        stats = dict(llm.stats)
        llm.shutdown()
    assert got == want
    assert stats["spec_drafted"] > 0
    assert 0 < stats["spec_accepted"] < stats["spec_drafted"], stats    # both full and cut-short drafts occurred


def test_draft_head_proposers_run_against_a_hybrid_target(monkeypatch):
    """EAGLE3 / MTP draft heads only need the target's hidden states and the verify step's accept
    record; with the recurrent rollback they serve hybrid targets too (random head: every draft is
    rejected, i.e. every step rolls back, and the output still equals plain decoding)."""
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    monkeypatch.setenv("MSGL_RECURRENT_SNAPSHOT_MIB", "0")
    g = torch.Generator().manual_seed(9)
    prompts = [torch.randint(0, 298, (n,), generator=g).tolist() for n in (25, 9)]
    sp = SamplingParams(max_tokens=10, ignore_eos=True)
    with tempfile.TemporaryDirectory() as tmp:
        _hf_model(tmp)
        kw = dict(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64)
        plain = LLM(**kw)
        want = [o.token_ids for o in plain.generate(prompts, sp)]
        plain.shutdown()
        llm = LLM(spec_algorithm="mtp", spec_num_draft=2, **kw)
        got = [o.token_ids for o in llm.generate(prompts, sp)]
        assert llm.stats["spec_steps"] > 0
        llm.shutdown()
        with pytest.raises(ValueError, match="tree verification"):
            LLM(spec_algorithm="ngram", spec_num_draft=2, spec_tree_width=3, **kw)
    assert got == want
