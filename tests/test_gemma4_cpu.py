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


def _diffusion_gemma(tmp):
    """A block-diffusion checkpoint in miniature: the Gemma-4 text weights under ``model.decoder.*``, loose layer
    scalars on the encoder side, the self-conditioning block, ``canvas_length`` on the top-level config and no
    ``attention_k_eq_v`` field although the global layers have no value projection."""
    import json
    import os

    from safetensors.torch import save_file
    from transformers import Gemma4ForCausalLM, Gemma4TextConfig

    cfg = Gemma4TextConfig(vocab_size=300, hidden_size=64, intermediate_size=96, num_attention_heads=4, head_dim=16,
                           global_head_dim=32, sliding_window=8, max_position_embeddings=512, eos_token_id=298,
                           bos_token_id=None, pad_token_id=0, num_hidden_layers=3, num_key_value_heads=2,
                           num_global_key_value_heads=1, attention_k_eq_v=True, enable_moe_block=True, num_experts=4,
                           top_k_experts=2, moe_intermediate_size=16, hidden_size_per_layer_input=0,
                           final_logit_softcapping=30.0,
                           layer_types=["sliding_attention", "sliding_attention", "full_attention"])
    torch.manual_seed(0)
    hf = Gemma4ForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for name, p in hf.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn_like(p) * 0.08)
            elif "norm" in name or "scale" in name:
                p.copy_(1.0 + torch.randn_like(p) * 0.1)
    g = torch.Generator().manual_seed(5)
    sc = {"gate_proj.weight": torch.randn(96, 64, generator=g) * 0.08, "up_proj.weight": torch.randn(96, 64, generator=g) * 0.08,
          "down_proj.weight": torch.randn(64, 96, generator=g) * 0.08, "pre_norm.weight": 1.0 + torch.randn(64, generator=g) * 0.1}
    tensors = {}
    for name, t in hf.state_dict().items():
        if name == "lm_head.weight":
            continue
        tensors["model.decoder." + name[len("model."):]] = t.detach().clone().contiguous()
        if name.endswith("layer_scalar"):
            tensors["model.encoder." + name[len("model."):]] = t.detach().clone()
    for name, t in sc.items():
        tensors["model.self_conditioning." + name] = t.contiguous()
    save_file(tensors, os.path.join(tmp, "model.safetensors"))
    text = {k: v for k, v in cfg.to_dict().items() if k != "attention_k_eq_v"}
    text["model_type"] = "diffusion_gemma_text"
    json.dump({"model_type": "diffusion_gemma", "architectures": ["DiffusionGemmaForBlockDiffusion"], "canvas_length": 5,
               "mask_token_id": 299, "tie_word_embeddings": True, "text_config": text},
              open(os.path.join(tmp, "config.json"), "w"))
    json.dump({"max_denoising_steps": 3, "confidence_threshold": 0.6, "mask_token_id": 299,
               "sampler_config": {"_cls_name": "MaskConfidenceSamplerConfig"}},
              open(os.path.join(tmp, "generation_config.json"), "w"))
    return hf, sc


def _dense_self_conditioned_decode(hf, sc, prompt, cfg, max_tokens, window):
    """Full-sequence forwards of the Hugging Face layers with explicit masks: committed text causal (inside
    the window on sliding layers), canvas rows see the whole canvas and the text (inside their window on
    sliding layers); the canvas embeddings go through the self-conditioning block with the previous step's
    probability-weighted embedding."""
    import torch.nn.functional as F

    from minisglang_rdna4_b200.diffusion import Canvas

    def unit_norm(x):
        return x * torch.pow(x.pow(2).mean(-1, keepdim=True) + 1e-6, -0.5)

    emb = hf.model.embed_tokens
    ids, out = list(prompt), []
    while len(out) < max_tokens:
        n = min(cfg.block, max_tokens - len(out))
        st = Canvas(cfg, n, "cpu", torch.Generator().manual_seed(0))
        signal = None
        while not st.finished:
            c, t = len(ids), len(ids) + n
            x = emb(torch.tensor([ids + st.tokens.tolist()]))[0]
            canvas = x[c:]
            if signal is not None:
                s = unit_norm(signal) * sc["pre_norm.weight"]
                mlp = F.gelu(s @ sc["gate_proj.weight"].t(), approximate="tanh") * (s @ sc["up_proj.weight"].t())
                canvas = canvas + mlp @ sc["down_proj.weight"].t()
            x = torch.cat([x[:c], unit_norm(canvas)])
            q, k = torch.arange(t)[:, None], torch.arange(t)[None, :]
            full = torch.where(k > q, float("-inf"), 0.0)
            full[c:, :] = 0.0
            sliding = torch.where((k > q) | (k <= q - window), float("-inf"), 0.0)
            sliding[c:, c:] = 0.0
            with torch.no_grad():
                h = hf.model(inputs_embeds=x[None], attention_mask={"full_attention": full[None, None],
                                                                    "sliding_attention": sliding[None, None]},
                             use_cache=False).last_hidden_state
                logits = torch.tanh(hf.lm_head(h[0, c:]) / 30.0) * 30.0
            st.advance(logits.float())
            signal = torch.softmax(logits.float(), -1) @ emb.weight * (64 ** 0.5)
        for tok in st.emit.tolist():
            out.append(tok)
            ids.append(tok)
            if len(out) >= max_tokens:
                break
    return out


def test_diffusion_gemma_with_self_conditioning_equals_a_dense_restatement():
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    with tempfile.TemporaryDirectory() as tmp:
        hf, sc = _diffusion_gemma(tmp)
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(1, 290, (n,), generator=g).tolist() for n in (7, 33, 18)]
        llm = LLM(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64,
                  max_extend_tokens=24)
        mc = llm.engine.model_config
        assert type(llm.engine.model).__name__ == "DiffusionGemmaForBlockDiffusion"
        assert mc.attention_k_eq_v and mc.canvas_length == 5 and llm.diffusion.cfg.kind == "mask_confidence"
        cfg = llm.diffusion.cfg
        budgets = (12, 10, 7)
        outs = llm.generate(prompts, [SamplingParams(max_tokens=m, ignore_eos=True) for m in budgets])
        got = [o.token_ids for o in outs]
        llm.shutdown()
    for p, m, have in zip(prompts, budgets, got):
        assert have == _dense_self_conditioned_decode(hf, sc, p, cfg, m, window=8), (len(p), m)


def _assistant_ckpt(tmp, layer_types=("sliding_attention", "full_attention")):
    """A drafter checkpoint with random weights in the published naming."""
    import json
    import os

    from safetensors.torch import save_file

    hid, inter, heads, d_s, d_g, backbone = 32, 48, 4, 16, 32, 64
    g = torch.Generator().manual_seed(9)
    rnd = lambda *shape: torch.randn(*shape, generator=g) * 0.15
    w = {"pre_projection.weight": rnd(hid, 2 * backbone), "post_projection.weight": rnd(backbone, hid),
         "model.norm.weight": 1.0 + rnd(hid), "model.embed_tokens.weight": rnd(300, hid)}
    for i, kind in enumerate(layer_types):
        d = d_s if kind == "sliding_attention" else d_g
        p = f"model.layers.{i}."
        for n in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm"):
            w[p + n + ".weight"] = 1.0 + rnd(hid)
        w[p + "self_attn.q_norm.weight"] = 1.0 + rnd(d)
        w[p + "self_attn.q_proj.weight"] = rnd(heads * d, hid)
        w[p + "self_attn.o_proj.weight"] = rnd(hid, heads * d)
        w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"] = rnd(inter, hid), rnd(inter, hid)
        w[p + "mlp.down_proj.weight"] = rnd(hid, inter)
        w[p + "layer_scalar"] = torch.rand(1, generator=g) * 0.5 + 0.75
    os.makedirs(tmp, exist_ok=True)
    save_file({k: v.contiguous() for k, v in w.items()}, os.path.join(tmp, "model.safetensors"))
    json.dump({"model_type": "gemma4_assistant", "backbone_hidden_size": backbone,
               "text_config": {"model_type": "gemma4_text", "hidden_size": hid, "intermediate_size": inter,
                               "num_attention_heads": heads, "num_key_value_heads": 1, "head_dim": d_s,
                               "global_head_dim": d_g, "num_hidden_layers": len(layer_types), "vocab_size": 300,
                               "layer_types": list(layer_types), "rms_norm_eps": 1e-6, "sliding_window": 16,
                               "hidden_size_per_layer_input": 0, "max_position_embeddings": 512,
                               "tie_word_embeddings": True}}, open(os.path.join(tmp, "config.json"), "w"))
    return w


def _restate_draft_chain(hf, w, ids, k, window=16):
    """The drafter's chain for a request whose first ``len(ids) - 1`` tokens have K/V in the target: queries
    only, over the keys and values the Hugging Face target computes in its last layers that keep K/V."""
    import torch.nn.functional as F

    from transformers.models.gemma4.modeling_gemma4 import apply_rotary_pos_emb

    rms = lambda x, wt=None: (x * torch.pow(x.pow(2).mean(-1, keepdim=True) + 1e-6, -0.5)) * (1.0 if wt is None else wt)
    tcfg = hf.config
    L = len(ids) - 1
    with torch.no_grad():
        # with a cache: without one the Hugging Face layers that share K/V compute their own
        out = hf.model(torch.tensor([ids[:L]]), output_hidden_states=True, use_cache=True)
        seed = out.last_hidden_state[0, L - 1]
        pos = torch.arange(L)[None]
        own = tcfg.num_hidden_layers - tcfg.num_kv_shared_layers
        kv = {}
        for kind in ("sliding_attention", "full_attention"):
            li = max(i for i in range(own) if tcfg.layer_types[i] == kind)
            layer = hf.model.layers[li]
            att = layer.self_attn
            h = layer.input_layernorm(out.hidden_states[li])
            cos, sin = hf.model.rotary_emb(h, pos, kind)
            kk = att.k_proj(h).view(1, L, -1, att.head_dim)
            vv = att.v_proj(h).view(1, L, -1, att.head_dim) if att.v_proj is not None else kk
            kv[kind] = (apply_rotary_pos_emb(att.k_norm(kk), cos, sin, unsqueeze_dim=2)[0], att.v_norm(vv)[0],
                        (cos[0, L - 1], sin[0, L - 1]))
        tok, drafts = ids[L], []
        kinds = [t for t in ("sliding_attention", "full_attention")]
        n_layers = sum(1 for name in w if name.endswith("self_attn.q_proj.weight"))
        for _ in range(k):
            e = hf.model.embed_tokens(torch.tensor([tok]))[0]
            x = w["pre_projection.weight"] @ torch.cat([e, seed])
            for i in range(n_layers):
                p = f"model.layers.{i}."
                d = w[p + "self_attn.q_norm.weight"].numel()
                kind = "sliding_attention" if d == 16 else "full_attention"
                keys, vals, (cos, sin) = kv[kind]
                q = (w[p + "self_attn.q_proj.weight"] @ rms(x, w[p + "input_layernorm.weight"])).view(-1, d)
                q = rms(q, w[p + "self_attn.q_norm.weight"])
                q = q * cos + torch.cat([-q[:, d // 2:], q[:, : d // 2]], -1) * sin
                lo = max(0, L - window) if kind == "sliding_attention" else 0
                kh = keys[lo:, 0]                                   # one K/V head in the target
                prob = torch.softmax(q @ kh.t(), -1)
                a = w[p + "self_attn.o_proj.weight"] @ (prob @ vals[lo:, 0]).reshape(-1)
                x = x + rms(a, w[p + "post_attention_layernorm.weight"])
                hm = rms(x, w[p + "pre_feedforward_layernorm.weight"])
                m = w[p + "mlp.down_proj.weight"] @ (F.gelu(w[p + "mlp.gate_proj.weight"] @ hm, approximate="tanh")
                                                     * (w[p + "mlp.up_proj.weight"] @ hm))
                x = (x + rms(m, w[p + "post_feedforward_layernorm.weight"])) * w[p + "layer_scalar"]
            dn = rms(x, w["model.norm.weight"])
            tok = int((w["model.embed_tokens.weight"] @ dn).argmax())
            seed = w["post_projection.weight"] @ dn
            drafts.append(tok)
    return drafts


def test_gemma4_assistant_drafter_reads_the_targets_kv():
    """Speculative decoding with the query-only drafter: tokens equal the target's own greedy decoding
    (verification decides), and the drafter's chains equal a restatement over the keys and values the Hugging
    Face target computes, whether the drafted tokens were accepted or not."""
    import os

    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM
    from minisglang_rdna4_b200.spec.gemma4_assistant import Gemma4AssistantProposer

    with tempfile.TemporaryDirectory() as tmp:
        hf = _hf(tmp, "shared_kv_ple")
        w = _assistant_ckpt(os.path.join(tmp, "assistant"))
        g = torch.Generator().manual_seed(4)
        prompts = [torch.randint(1, 298, (n,), generator=g).tolist() for n in (6, 45)]
        want = [hf.generate(torch.tensor([p]), max_new_tokens=8, do_sample=False)[0, len(p):].tolist() for p in prompts]
        llm = LLM(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64,
                  max_extend_tokens=32, spec_algorithm="mtp", spec_num_draft=3,
                  spec_draft_model_path=os.path.join(tmp, "assistant"))
        prop = llm.proposer
        assert isinstance(prop, Gemma4AssistantProposer)
        seen = []
        inner = prop.propose

        def spy(reqs):
            out = inner(reqs)
            for r, d in zip(reqs, out):
                if d:
                    L = prop._len[r.uid]
                    seen.append((r.input_ids[: L + 1].tolist(), list(d)))
            return out

        prop.propose = spy
        got = [o.token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))]
        llm.shutdown()
    assert got == want
    assert len(seen) >= 4
    for ids, drafts in seen[:6]:
        assert drafts == _restate_draft_chain(hf, w, ids, len(drafts)), len(ids)


@pytest.mark.parametrize("bidirectional", [False, True])
def test_gemma4_image_input_matches_transformers(bidirectional):
    """A multimodal Gemma-4 checkpoint in miniature (vision tower with the two-dimensional rotary embedding and
    k x k pooling, projector, text decoder with per-layer inputs): image features equal the Hugging Face
    tower's, and greedy generation over a prompt with an image equals Hugging Face's with the same patches.
    ``bidirectional``: the larger models let the tokens of one image see each other in both directions."""
    from transformers import Gemma4Config, Gemma4ForConditionalGeneration
    from transformers.models.gemma4.image_processing_gemma4 import convert_image_to_patches

    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    text = dict(vocab_size=300, hidden_size=64, intermediate_size=96, num_attention_heads=4, head_dim=16,
                global_head_dim=32, sliding_window=16, max_position_embeddings=512, eos_token_id=299, bos_token_id=None,
                pad_token_id=0, use_bidirectional_attention="vision" if bidirectional else None, **_KINDS["shared_kv_ple"])
    vision = dict(hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=2,
                  num_key_value_heads=2, head_dim=16, patch_size=4, pooling_kernel_size=2, position_embedding_size=64)
    cfg = Gemma4Config(text_config=text, vision_config=vision, audio_config=None, image_token_id=290, boi_token_id=291,
                       eoi_token_id=292, vision_soft_tokens_per_image=9)
    torch.manual_seed(0)
    hf = Gemma4ForConditionalGeneration(cfg).float().eval()
    with torch.no_grad():
        for name, p in hf.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn_like(p) * 0.08)
            elif "norm" in name or "scale" in name:
                p.copy_(1.0 + torch.randn_like(p) * 0.1)
    g = torch.Generator().manual_seed(6)
    side = 3 * 2 * 4                                            # 3 soft tokens per side x pooling 2 x patch 4
    image = torch.randint(0, 256, (3, side, side), generator=g, dtype=torch.uint8)
    patches = convert_image_to_patches(image.float() / 255.0, 4)[None]
    grid = side // 4
    pos = torch.stack(torch.meshgrid(torch.arange(grid), torch.arange(grid), indexing="xy"), -1).reshape(1, -1, 2)
    head = torch.randint(1, 280, (7,), generator=g).tolist()
    tail = torch.randint(1, 280, (12,), generator=g).tolist()
    ids = head + [291] + [290] * 9 + [292] + tail
    kinds = torch.tensor([[1 if t == 290 else 0 for t in ids]])
    with torch.no_grad():
        want_feats = hf.model.get_image_features(patches, pos).pooler_output
        want = hf.generate(torch.tensor([ids]), pixel_values=patches, image_position_ids=pos, mm_token_type_ids=kinds,
                           max_new_tokens=8, do_sample=False)[0, len(ids):].tolist()
    with tempfile.TemporaryDirectory() as tmp:
        hf.save_pretrained(tmp, safe_serialization=True)
        llm = LLM(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64,
                  max_extend_tokens=64)
        eng = llm.engine
        assert eng.vision is not None and eng.vision.cfg.tokens_per_image == 9 and eng.vision.cfg.image_size == side
        assert eng.model_config.image_bidirectional == bidirectional
        feats = eng.vision.image_embeddings((image[None].float() / 255.0 - 0.5) / 0.5)
        torch.testing.assert_close(feats, want_feats.reshape(-1, 64), rtol=2e-4, atol=2e-4)
        out = llm.generate([head + [291] + tail], SamplingParams(max_tokens=8, ignore_eos=True), images=[[image]])[0]
        llm.shutdown()
    assert out.token_ids == want


def test_published_gemma4_shapes_parse():
    """The default Hugging Face configurations (the small multimodal model's shape) and the dense large model's
    geometry go through the config parser: per-layer geometry, K/V sharing, rotary tables, vision budget."""
    from transformers import Gemma4Config, Gemma4TextConfig, Gemma4VisionConfig

    from minisglang_rdna4_b200.models.config import ModelConfig

    small = Gemma4Config(text_config=Gemma4TextConfig(num_hidden_layers=35, num_kv_shared_layers=20, num_key_value_heads=1,
                                                      hidden_size=1536, use_double_wide_mlp=True).to_dict(),
                         vision_config=Gemma4VisionConfig().to_dict(), audio_config=None)
    mc = ModelConfig.from_hf(small.to_dict())
    assert mc.architectures[0].startswith("Gemma4") and mc.num_kv_layers == 15 and mc.mixed_kv_geometry
    assert mc.attn_geometry(0) == (1, 256) and mc.attn_geometry(5) == (1, 512) and mc.layer_types[-1] == "full_attention"
    assert mc.kv_donor(14) is None and mc.kv_donor(15) == 14 and mc.kv_donor(34) == 11      # last own sliding / full layer
    assert mc.rotary_config.head_dim == 512 and mc.rotary_config.scaling["rope_type"] == "proportional"
    assert mc.rope_local_base_freq == 10000.0 and mc.hidden_size_per_layer_input == 256 and not mc.image_bidirectional
    v = mc.vision
    assert v.kind == "gemma4" and v.tokens_per_image == 256 and v.image_size == 16 * 3 * 16 and v.head_dim == 64
    dense = Gemma4TextConfig(num_hidden_layers=60, hidden_size=5376, num_attention_heads=32, num_key_value_heads=16,
                             num_global_key_value_heads=4, attention_k_eq_v=True, hidden_size_per_layer_input=0,
                             use_bidirectional_attention="vision")
    mc = ModelConfig.from_hf(dense.to_dict())
    assert mc.attn_geometry(0) == (16, 256) and mc.attn_geometry(5) == (4, 512) and mc.num_kv_layers == 60
    assert mc.image_bidirectional and mc.hidden_size_per_layer_input == 0 and mc.swa_layers[:6] == (0, 1, 2, 3, 4, 6)


def test_published_gemma4_shapes_build_on_the_meta_device():
    """The three published text shapes instantiate (no memory behind them) with the parameter counts their
    names promise."""
    from transformers import Gemma4TextConfig

    from minisglang_rdna4_b200.models import ModelConfig, create_model

    shapes = {
        "31b": (dict(num_hidden_layers=60, hidden_size=5376, intermediate_size=21504, num_attention_heads=32,
                     num_key_value_heads=16, num_global_key_value_heads=4, attention_k_eq_v=True,
                     hidden_size_per_layer_input=0), 30.7),
        "26b-a4b": (dict(num_hidden_layers=30, hidden_size=2816, intermediate_size=2112, num_attention_heads=16,
                         num_key_value_heads=8, num_global_key_value_heads=2, attention_k_eq_v=True,
                         hidden_size_per_layer_input=0, enable_moe_block=True, num_experts=128, top_k_experts=8,
                         moe_intermediate_size=704), 25.2),
        "e2b": (dict(num_hidden_layers=35, num_kv_shared_layers=20, num_key_value_heads=1, hidden_size=1536,
                     intermediate_size=6144, use_double_wide_mlp=True), 4.6),
    }
    for name, (kw, billions) in shapes.items():
        mc = ModelConfig.from_hf(Gemma4TextConfig(**kw).to_dict())
        model = create_model(mc, torch.bfloat16, "meta")
        n = sum(t.numel() for _, t, _, _ in model.named_parameters())
        assert abs(n / 1e9 - billions) < 0.1, (name, n)
