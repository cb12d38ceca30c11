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

    common = dict(
        vocab_size=300, hidden_size=64, num_hidden_layers=4, num_attention_heads=4,
        num_key_value_heads=2, head_dim=32, linear_conv_kernel_dim=4, linear_key_head_dim=16,
        linear_value_head_dim=16, linear_num_key_heads=2, linear_num_value_heads=4, max_position_embeddings=512,
        rms_norm_eps=1e-6, tie_word_embeddings=False, eos_token_id=299, pad_token_id=None, bos_token_id=None,
    )
    torch.manual_seed(0)
    if moe:
        from transformers import Qwen3_5MoeForCausalLM, Qwen3_5MoeTextConfig

        cfg = Qwen3_5MoeTextConfig(moe_intermediate_size=32, shared_expert_intermediate_size=48, num_experts=8,
                                   num_experts_per_tok=2, **common)
        model = Qwen3_5MoeForCausalLM(cfg).float().eval()
    else:
        cfg = Qwen3_5TextConfig(intermediate_size=128, **common)
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


@pytest.mark.parametrize("moe", [False, True])
def test_qwen3_5_hybrid_matches_transformers(moe):
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    with tempfile.TemporaryDirectory() as tmp:
        hf = _hf_model(tmp, moe)
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


def _add_mtp_head(tmp, hf):
    """Append a random next-token head (``mtp.*``) to the checkpoint in ``tmp``; returns torch
    modules that restate it: a Hugging Face full-attention decoder layer between the fusing
    projection and the final norm."""
    import json

    from safetensors.torch import load_file, save_file

    cfg = hf.config
    cfg._attn_implementation = "eager"
    torch.manual_seed(1)
    if hasattr(cfg, "num_experts"):
        from transformers.models.qwen3_5_moe import modeling_qwen3_5_moe as m

        layer_cls, norm_cls, rotary_cls = m.Qwen3_5MoeDecoderLayer, m.Qwen3_5MoeRMSNorm, m.Qwen3_5MoeTextRotaryEmbedding
    else:
        from transformers.models.qwen3_5 import modeling_qwen3_5 as m

        layer_cls, norm_cls, rotary_cls = m.Qwen3_5DecoderLayer, m.Qwen3_5RMSNorm, m.Qwen3_5TextRotaryEmbedding
    layer = layer_cls(cfg, 3).float().eval()                           # layer 3 of the pattern is full attention
    fc = torch.nn.Linear(2 * cfg.hidden_size, cfg.hidden_size, bias=False)
    ne, nh, nf = (norm_cls(cfg.hidden_size, eps=cfg.rms_norm_eps) for _ in range(3))
    with torch.no_grad():
        for mod in (layer, fc, ne, nh, nf):
            for p in mod.parameters():
                p.copy_(torch.randn_like(p) * (0.1 if p.dim() == 1 else 0.08))
    st = load_file(f"{tmp}/model.safetensors")
    for k, v in layer.state_dict().items():
        st["mtp.layers.0." + k] = v.contiguous()
    st["mtp.fc.weight"] = fc.weight.detach()
    st["mtp.pre_fc_norm_embedding.weight"] = ne.weight.detach()
    st["mtp.pre_fc_norm_hidden.weight"] = nh.weight.detach()
    st["mtp.norm.weight"] = nf.weight.detach()
    save_file(st, f"{tmp}/model.safetensors")
    c = json.load(open(f"{tmp}/config.json"))
    c["mtp_num_hidden_layers"] = 1
    json.dump(c, open(f"{tmp}/config.json", "w"))

    def head(hidden, embeds):
        """Dense causal restatement: row i pairs hidden[i] with embeds[i] (the token after it)."""
        n = hidden.shape[0]
        with torch.no_grad():
            x = fc(torch.cat([ne(embeds), nh(hidden)], -1))[None]
            pos = torch.arange(n)[None]
            pe = rotary_cls(cfg)(x, pos)
            mask = torch.full((n, n), float("-inf")).triu(1)[None, None]
            y = layer(x, position_embeddings=pe, attention_mask=mask, position_ids=pos)
            y = y[0] if isinstance(y, tuple) else y
            out = nf(y)[0]
            return out, hf.lm_head(out)

    return head


@pytest.mark.parametrize("moe", [False, True])
def test_checkpoint_mtp_head_matches_a_dense_restatement_and_drafts_exactly(moe, monkeypatch):
    """``--spec-algorithm mtp`` on a checkpoint that carries ``mtp.*`` tensors builds the head from the
    target's own layer class and loads it through the decoder's loader. Its hidden states and logits
    equal a dense Hugging Face restatement, the draft it proposes after the prefill is that
    restatement's arg-max, and generation equals plain decoding."""
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    monkeypatch.setenv("MSGL_RECURRENT_SNAPSHOT_MIB", "0")
    with tempfile.TemporaryDirectory() as tmp:
        hf = _hf_model(tmp, moe)
        head = _add_mtp_head(tmp, hf)
        g = torch.Generator().manual_seed(2)
        ids = torch.randint(0, 298, (1, 21), generator=g)
        with torch.no_grad():
            hid = hf(ids, output_hidden_states=True).hidden_states[-1][0]      # final, normalised
            emb = hf.model.embed_tokens(ids)[0]
        want_hidden, want_logits = head(hid[:-1], emb[1:])
        kw = dict(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64)
        llm = LLM(spec_algorithm="mtp", spec_num_draft=2, **kw)
        prop = llm.proposer
        assert type(prop).__name__ == "MTPProposer" and prop.loaded_tensors >= 15
        assert prop.draft.layer._is_moe == moe
        n = ids.shape[1] - 1
        got_hidden, got_logits = prop.draft.forward_rows(-7, emb[1:], hid[:-1], torch.arange(n, dtype=torch.int32))
        prop.draft.drop(-7)
        assert torch.allclose(got_hidden, want_hidden, atol=1e-5)
        assert torch.allclose(got_logits, want_logits[-1:], atol=1e-5)

        first = {}
        inner = prop.propose

        def recording(reqs):
            out = inner(reqs)
            for r, d in zip(reqs, out):
                first.setdefault(r.prompt_len, list(d))
            return out

        prop.propose = recording
        prompts = [ids[0].tolist(), torch.randint(0, 298, (9,), generator=g).tolist()]
        sp = SamplingParams(max_tokens=12, ignore_eos=True)
        outs = llm.generate(prompts, sp)
        got = [o.token_ids for o in outs]
        assert llm.stats["spec_steps"] > 0
        llm.shutdown()
        # the first draft of the 21-token prompt: rows 0..20 pair every position's hidden state with the
        # token after it (the last one is the token the prefill sampled)
        seq = torch.tensor([prompts[0] + got[0][:1]])
        with torch.no_grad():
            hid2 = hf(seq[:, :-1], output_hidden_states=True).hidden_states[-1][0]
            emb2 = hf.model.embed_tokens(seq)[0]
        _, logits2 = head(hid2, emb2[1:])
        assert first[21][0] == int(logits2[-1].argmax())
        plain = LLM(**kw)
        want = [o.token_ids for o in plain.generate(prompts, sp)]
        plain.shutdown()
    assert got == want


def test_qwen3_next_grouped_projections_match_transformers():
    """Qwen3-Next stores the linear-attention input projections grouped per key head
    (``in_proj_qkvz``: q ‖ k ‖ v ‖ z of one key head's value heads; ``in_proj_ba``); the loader regroups
    them into the per-kind blocks of the layer. Greedy decoding equals the Hugging Face model."""
    from transformers import Qwen3NextConfig, Qwen3NextForCausalLM

    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    cfg = Qwen3NextConfig(
        vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
        num_key_value_heads=2, head_dim=32, linear_conv_kernel_dim=4, linear_key_head_dim=16, linear_value_head_dim=16,
        linear_num_key_heads=2, linear_num_value_heads=4, max_position_embeddings=512, rms_norm_eps=1e-6,
        tie_word_embeddings=False, moe_intermediate_size=32, shared_expert_intermediate_size=48, num_experts=8,
        num_experts_per_tok=2, eos_token_id=299, pad_token_id=None, bos_token_id=None, decoder_sparse_step=1,
        mlp_only_layers=[])
    torch.manual_seed(0)
    hf = Qwen3NextForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for name, p in hf.named_parameters():
            if name.endswith("norm.weight") and "linear_attn" not in name:
                p.copy_(torch.randn_like(p) * 0.1)
            elif "A_log" in name:
                p.copy_(torch.log(torch.empty_like(p).uniform_(1.0, 8.0)))
            elif "dt_bias" in name:
                p.copy_(torch.randn_like(p) * 0.5)
            elif p.dim() >= 2:
                p.copy_(torch.randn_like(p) * 0.08)
    with tempfile.TemporaryDirectory() as tmp:
        hf.save_pretrained(tmp, safe_serialization=True)
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, 298, (n,), generator=g).tolist() for n in (5, 23, 41)]
        want = [hf.generate(torch.tensor([p]), max_new_tokens=8, do_sample=False)[0, len(p):].tolist() for p in prompts]
        llm = LLM(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64,
                  max_extend_tokens=16)
        got = [o.token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))]
        llm.shutdown()
    assert got == want
