"""Muse-Glimmer text decoder against a dense restatement of its published forward: weight-less embedding and
q/k norms, (1 + w) sandwich norms with a second epsilon, sliding layers with rotary embedding and global layers
without any positional encoding, the sigmoid gate on the attention output, logits multiplied before the cap."""
import json
import os
import tempfile

import torch
import torch.nn.functional as F

H, HEADS, KV, D, INTER, VOCAB, LAYERS, WINDOW = 48, 4, 2, 16, 64, 200, 4, 8
KINDS = ["sliding_attention", "full_attention", "sliding_attention", "full_attention"]
THETA = [10000.0, 0.0, 10000.0, 0.0]
EPS, EPS_POST, QK_SCALE, MULT, CAP = 1e-5, 1e-8, 3.87, 26 ** -0.5, 30.0


def _checkpoint(tmp):
    from safetensors.torch import save_file

    g = torch.Generator().manual_seed(0)
    rnd = lambda *s: torch.randn(*s, generator=g) * 0.15
    w = {"model.language_model.embed_tokens.weight": rnd(VOCAB, H), "model.language_model.norm.weight": 1.0 + rnd(H),
         "lm_head.weight": rnd(VOCAB, H), "model.vision_tower.stub.weight": rnd(2, 2)}
    for i in range(LAYERS):
        p = f"model.language_model.layers.{i}."
        for n in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm"):
            w[p + n + ".weight"] = rnd(H)
        w[p + "self_attn.q_proj.weight"], w[p + "self_attn.gate_proj.weight"] = rnd(HEADS * D, H), rnd(HEADS * D, H)
        w[p + "self_attn.k_proj.weight"], w[p + "self_attn.v_proj.weight"] = rnd(KV * D, H), rnd(KV * D, H)
        w[p + "self_attn.o_proj.weight"] = rnd(H, HEADS * D)
        w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"] = rnd(INTER, H), rnd(INTER, H)
        w[p + "mlp.down_proj.weight"] = rnd(H, INTER)
    save_file({k: v.contiguous() for k, v in w.items()}, os.path.join(tmp, "model.safetensors"))
    text = {"model_type": "muse_glimmer_text", "hidden_size": H, "num_attention_heads": HEADS, "num_key_value_heads": KV,
            "head_dim": D, "intermediate_size": INTER, "vocab_size": VOCAB, "num_hidden_layers": LAYERS,
            "layer_types": KINDS, "layer_rope_theta": THETA, "sliding_window": WINDOW, "rms_norm_eps": EPS,
            "post_norm_eps": EPS_POST, "qk_scale_factor": QK_SCALE, "output_multiplier": MULT,
            "final_logit_softcapping": CAP, "hidden_activation": "gelu_pytorch_tanh", "max_position_embeddings": 256,
            "rope_theta": 10000.0, "tie_word_embeddings": False, "eos_token_id": VOCAB - 1}
    json.dump({"model_type": "muse_glimmer", "architectures": ["MuseGlimmerForConditionalGeneration"],
               "text_config": text, "vision_config": {"hidden_size": 8}}, open(os.path.join(tmp, "config.json"), "w"))
    return {k.replace("model.language_model.", "model."): v for k, v in w.items()}


def _dense_logits(w, ids):
    rms = lambda x, eps, wt=None: (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)) * (1.0 if wt is None else wt)
    t = len(ids)
    x = rms(w["model.embed_tokens.weight"][torch.tensor(ids)], EPS)
    q_pos, k_pos = torch.arange(t)[:, None], torch.arange(t)[None, :]
    for i in range(LAYERS):
        p = f"model.layers.{i}."
        h = rms(x, EPS, 1.0 + w[p + "input_layernorm.weight"])
        q = rms((h @ w[p + "self_attn.q_proj.weight"].t()).view(t, HEADS, D), EPS)
        k = rms((h @ w[p + "self_attn.k_proj.weight"].t()).view(t, KV, D), EPS)
        v = (h @ w[p + "self_attn.v_proj.weight"].t()).view(t, KV, D)
        if THETA[i]:
            inv = 1.0 / (THETA[i] ** (torch.arange(0, D, 2).float() / D))
            ang = torch.arange(t).float()[:, None] * inv[None]
            cos, sin = torch.cat([ang.cos(), ang.cos()], -1)[:, None], torch.cat([ang.sin(), ang.sin()], -1)[:, None]
            rot = lambda z: z * cos + torch.cat([-z[..., D // 2:], z[..., : D // 2]], -1) * sin
            q, k = rot(q), rot(k)
        k, v = k.repeat_interleave(HEADS // KV, 1), v.repeat_interleave(HEADS // KV, 1)
        s = torch.einsum("qhd,khd->hqk", q * QK_SCALE, k) / D ** 0.5
        hide = k_pos > q_pos
        if KINDS[i] == "sliding_attention":
            hide = hide | (k_pos <= q_pos - WINDOW)
        o = torch.einsum("hqk,khd->qhd", torch.softmax(s.masked_fill(hide[None], float("-inf")), -1), v).reshape(t, -1)
        o = o * torch.sigmoid(h @ w[p + "self_attn.gate_proj.weight"].t())
        x = x + rms(o @ w[p + "self_attn.o_proj.weight"].t(), EPS_POST, 1.0 + w[p + "post_attention_layernorm.weight"])
        h = rms(x, EPS, 1.0 + w[p + "pre_feedforward_layernorm.weight"])
        m = (F.gelu(h @ w[p + "mlp.gate_proj.weight"].t(), approximate="tanh") * (h @ w[p + "mlp.up_proj.weight"].t())) \
            @ w[p + "mlp.down_proj.weight"].t()
        x = x + rms(m, EPS_POST, 1.0 + w[p + "post_feedforward_layernorm.weight"])
    logits = rms(x, EPS, w["model.norm.weight"]) @ w["lm_head.weight"].t()
    return torch.tanh(logits * MULT / CAP) * CAP


def test_muse_glimmer_equals_a_dense_restatement():
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    with tempfile.TemporaryDirectory() as tmp:
        w = _checkpoint(tmp)
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, VOCAB - 1, (n,), generator=g).tolist() for n in (5, 37, 20)]
        llm = LLM(model_path=tmp, device="cpu", dtype="fp32", page_size=16, max_running_req=4, num_page_override=64,
                  max_extend_tokens=16)
        mc = llm.engine.model_config
        assert mc.swa_layers == (0, 2) and mc.layer_rope_theta[1] == 0.0 and mc.hidden_act == "gelu_pytorch_tanh"
        got = [o.token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))]
        llm.shutdown()
    for p, have in zip(prompts, got):
        ids = list(p)
        for _ in range(6):
            ids.append(int(_dense_logits(w, ids)[-1].argmax()))
        assert have == ids[len(p):], len(p)


def test_muse_glimmer_tp2_and_window_pool(monkeypatch):
    """Two tensor-parallel ranks (heads, gate channels and MLP width split), and one rank with the sliding layers
    in the window pool: same tokens as the plain single-rank run."""
    import multiprocessing as mp

    from test_tp_cpu import _single, _worker

    with tempfile.TemporaryDirectory() as tmp:
        _checkpoint(tmp)
        g = torch.Generator().manual_seed(2)
        prompts = [torch.randint(0, VOCAB - 1, (n,), generator=g).tolist() for n in (9, 30)]
        want = _single(tmp, prompts)
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        port = 21100 + (os.getpid() % 1500)
        procs = [ctx.Process(target=_worker, args=(r, 2, port, tmp, prompts, q, False)) for r in range(2)]
        for p in procs:
            p.start()
        got = q.get(timeout=240)
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
        assert got == want
        monkeypatch.setenv("MSGL_SWA_POOL", "1")
        assert _single(tmp, prompts) == want
