"""Laguna decoder against a dense restatement of its published forward: a query-head count per layer, YaRN over
half of the head on the global layers and a plain table on the sliding ones, the softplus gate per head, a dense
first MLP, then sigmoid-routed experts with a selection bias and an always-on shared expert."""
import json
import os
import tempfile

import torch
import torch.nn.functional as F

H, KV, D, INTER, MOE_I, SHARED_I, E, TOPK, VOCAB, WINDOW = 48, 2, 16, 64, 24, 32, 6, 2, 200, 8
KINDS = ["full_attention", "sliding_attention", "sliding_attention", "full_attention"]
HEADS = [4, 6, 6, 4]
EPS, SCALE = 1e-6, 2.5
ROPE = {"full_attention": {"rope_type": "yarn", "rope_theta": 50000.0, "factor": 4.0, "partial_rotary_factor": 0.5,
                           "original_max_position_embeddings": 32, "beta_fast": 32.0, "beta_slow": 1.0},
        "sliding_attention": {"rope_type": "default", "rope_theta": 10000.0}}


def _checkpoint(tmp):
    from safetensors.torch import save_file

    g = torch.Generator().manual_seed(0)
    rnd = lambda *s: torch.randn(*s, generator=g) * 0.15
    w = {"model.embed_tokens.weight": rnd(VOCAB, H), "model.norm.weight": 1.0 + rnd(H), "lm_head.weight": rnd(VOCAB, H)}
    for i, heads in enumerate(HEADS):
        p = f"model.layers.{i}."
        w[p + "input_layernorm.weight"], w[p + "post_attention_layernorm.weight"] = 1.0 + rnd(H), 1.0 + rnd(H)
        w[p + "self_attn.q_proj.weight"], w[p + "self_attn.g_proj.weight"] = rnd(heads * D, H), rnd(heads, H)
        w[p + "self_attn.k_proj.weight"], w[p + "self_attn.v_proj.weight"] = rnd(KV * D, H), rnd(KV * D, H)
        w[p + "self_attn.q_norm.weight"], w[p + "self_attn.k_norm.weight"] = 1.0 + rnd(D), 1.0 + rnd(D)
        w[p + "self_attn.o_proj.weight"] = rnd(H, heads * D)
        if i == 0:
            w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"] = rnd(INTER, H), rnd(INTER, H)
            w[p + "mlp.down_proj.weight"] = rnd(H, INTER)
            continue
        w[p + "mlp.gate.weight"] = rnd(E, H)
        w[p + "mlp.experts.e_score_correction_bias"] = rnd(E)
        for e in range(E):
            q = p + f"mlp.experts.{e}."
            w[q + "gate_proj.weight"], w[q + "up_proj.weight"] = rnd(MOE_I, H), rnd(MOE_I, H)
            w[q + "down_proj.weight"] = rnd(H, MOE_I)
        q = p + "mlp.shared_expert."
        w[q + "gate_proj.weight"], w[q + "up_proj.weight"], w[q + "down_proj.weight"] = rnd(SHARED_I, H), rnd(SHARED_I, H), rnd(H, SHARED_I)
    save_file({k: v.contiguous() for k, v in w.items()}, os.path.join(tmp, "model.safetensors"))
    json.dump({"model_type": "laguna", "architectures": ["LagunaForCausalLM"], "hidden_size": H,
               "num_attention_heads": 4, "num_attention_heads_per_layer": HEADS, "num_key_value_heads": KV, "head_dim": D,
               "intermediate_size": INTER, "moe_intermediate_size": MOE_I, "shared_expert_intermediate_size": SHARED_I,
               "num_experts": E, "num_experts_per_tok": TOPK, "norm_topk_prob": True, "routed_scaling_factor": SCALE,
               "first_k_dense_replace": 1, "vocab_size": VOCAB, "num_hidden_layers": len(HEADS), "layer_types": KINDS,
               "sliding_window": WINDOW, "rms_norm_eps": EPS, "rope_parameters": ROPE, "max_position_embeddings": 256,
               "tie_word_embeddings": False, "eos_token_id": VOCAB - 1, "hidden_act": "silu"},
              open(os.path.join(tmp, "config.json"), "w"))
    return w


def _dense_logits(w, ids):
    from minisglang_rdna4_b200.ops.ref import build_cos_sin_cache

    rms = lambda x, wt: (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + EPS)) * wt
    t = len(ids)
    x = w["model.embed_tokens.weight"][torch.tensor(ids)]
    q_pos, k_pos = torch.arange(t)[:, None], torch.arange(t)[None, :]
    tables = {"full_attention": (build_cos_sin_cache(D // 2, 256, 50000.0, {k: v for k, v in ROPE["full_attention"].items()
                                                                           if k != "rope_theta"}), D // 2),
              "sliding_attention": (build_cos_sin_cache(D, 256, 10000.0, None), D)}
    for i, heads in enumerate(HEADS):
        p = f"model.layers.{i}."
        h = rms(x, w[p + "input_layernorm.weight"])
        q = rms((h @ w[p + "self_attn.q_proj.weight"].t()).view(t, heads, D), w[p + "self_attn.q_norm.weight"])
        k = rms((h @ w[p + "self_attn.k_proj.weight"].t()).view(t, KV, D), w[p + "self_attn.k_norm.weight"])
        v = (h @ w[p + "self_attn.v_proj.weight"].t()).view(t, KV, D)
        table, rd = tables[KINDS[i]]
        cs = table[:t]
        cos, sin = cs[:, None, : rd // 2], cs[:, None, rd // 2:]

        def rot(z):
            a, b, rest = z[..., : rd // 2], z[..., rd // 2: rd], z[..., rd:]
            return torch.cat([a * cos - b * sin, b * cos + a * sin, rest], -1)

        q, k = rot(q), rot(k)
        k, v = k.repeat_interleave(heads // KV, 1), v.repeat_interleave(heads // KV, 1)
        s = torch.einsum("qhd,khd->hqk", q, k) / D ** 0.5
        hide = k_pos > q_pos
        if KINDS[i] == "sliding_attention":
            hide = hide | (k_pos <= q_pos - WINDOW)
        o = torch.einsum("hqk,khd->qhd", torch.softmax(s.masked_fill(hide[None], float("-inf")), -1), v)
        o = o * F.softplus(h @ w[p + "self_attn.g_proj.weight"].t())[:, :, None]
        x = x + o.reshape(t, -1) @ w[p + "self_attn.o_proj.weight"].t()
        h = rms(x, w[p + "post_attention_layernorm.weight"])
        mlp = lambda z, q_: (F.silu(z @ w[q_ + "gate_proj.weight"].t()) * (z @ w[q_ + "up_proj.weight"].t())) \
            @ w[q_ + "down_proj.weight"].t()
        if i == 0:
            x = x + mlp(h, p + "mlp.")
            continue
        score = torch.sigmoid(h @ w[p + "mlp.gate.weight"].t())
        pick = (score + w[p + "mlp.experts.e_score_correction_bias"]).topk(TOPK, -1).indices
        wt = score.gather(-1, pick)
        wt = wt / wt.sum(-1, keepdim=True) * SCALE
        routed = torch.zeros_like(h)
        for r in range(t):
            for j in range(TOPK):
                routed[r] += wt[r, j] * mlp(h[r], p + f"mlp.experts.{int(pick[r, j])}.")
        x = x + routed + mlp(h, p + "mlp.shared_expert.")
    return rms(x, w["model.norm.weight"]) @ w["lm_head.weight"].t()


def test_laguna_equals_a_dense_restatement():
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    with tempfile.TemporaryDirectory() as tmp:
        w = _checkpoint(tmp)
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, VOCAB - 1, (n,), generator=g).tolist() for n in (5, 45, 20)]
        llm = LLM(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64,
                  max_extend_tokens=16)
        mc = llm.engine.model_config
        assert mc.attn_head_counts == (4, 6, 6, 4) and mc.rotary_config.rotary_dim == 8 and mc.sliding_rotary.rotary_dim == 16
        got = [o.token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))]
        llm.shutdown()
    for p, have in zip(prompts, got):
        ids = list(p)
        for _ in range(6):
            ids.append(int(_dense_logits(w, ids)[-1].argmax()))
        assert have == ids[len(p):], len(p)


def test_laguna_tp2_ep_and_window_pool(monkeypatch):
    """Two tensor-parallel ranks (per-layer head counts, gate heads and expert width split), the experts split
    over the ranks instead, and one rank with the window pool: same tokens as the plain single-rank run."""
    import multiprocessing as mp

    from test_tp_cpu import _single, _worker

    with tempfile.TemporaryDirectory() as tmp:
        _checkpoint(tmp)
        g = torch.Generator().manual_seed(2)
        prompts = [torch.randint(0, VOCAB - 1, (n,), generator=g).tolist() for n in (9, 30)]
        want = _single(tmp, prompts)
        for k, ep in enumerate((False, True)):
            ctx = mp.get_context("spawn")
            q = ctx.Queue()
            port = 20100 + (os.getpid() % 1500) + 3 * k
            procs = [ctx.Process(target=_worker, args=(r, 2, port, tmp, prompts, q, ep)) for r in range(2)]
            for p in procs:
                p.start()
            got = q.get(timeout=240)
            for p in procs:
                p.join(timeout=60)
                assert p.exitcode == 0
            assert got == want, ep
        monkeypatch.setenv("MSGL_SWA_POOL", "1")
        assert _single(tmp, prompts) == want
