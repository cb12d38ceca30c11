"""Tensor parallelism with CPU ranks over gloo: sharded linears, vocabulary-parallel
embedding / LM head and the checkpoint loader must reproduce the single-rank result."""
import os
import tempfile

import pytest
import torch
import torch.multiprocessing as mp


def _cfg_dict(moe=False):
    d = dict(model_type="qwen3_moe" if moe else "qwen3", architectures=["Qwen3MoeForCausalLM" if moe else "Qwen3ForCausalLM"],
             num_hidden_layers=2, hidden_size=128, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
             intermediate_size=256, vocab_size=515, rms_norm_eps=1e-6, rope_theta=1e6, max_position_embeddings=512,
             tie_word_embeddings=False, torch_dtype="float32")
    if moe:
        d.update(num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64, norm_topk_prob=True)
    return d


def _worker(rank, world, port, ckpt, prompts, out_q, ep, extra=None):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["RANK"] = str(rank)
    os.environ["WORLD_SIZE"] = str(world)
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    try:
        llm = LLM(model_path=ckpt, device="cpu", tp_size=world, tp_rank=rank, page_size=16, max_running_req=4,
                  num_page_override=64, enable_ep=ep, dtype="fp32", **(extra or {}))
        outs = llm.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))
    except Exception as exc:                     # the parent must not wait out its timeout on a failed rank
        out_q.put(f"rank {rank}: {type(exc).__name__}: {exc}")
        raise
    if rank == 0:
        out_q.put([o.token_ids for o in outs])
    llm.shutdown()


def _single(ckpt, prompts):
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    llm = LLM(model_path=ckpt, device="cpu", page_size=16, max_running_req=4, num_page_override=64, dtype="fp32")
    return [o.token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))]


def _make_ckpt(tmp, moe):
    from minisglang_rdna4_b200.models import ModelConfig, create_model
    from minisglang_rdna4_b200.models.weight import save_dummy_checkpoint

    cfgd = _cfg_dict(moe)
    cfg = ModelConfig.from_hf(cfgd)
    model = create_model(cfg, torch.float32, "cpu")
    model.init_dummy(seed=7, std=0.05)
    save_dummy_checkpoint(model, tmp, cfgd)
    return tmp


@pytest.mark.parametrize("moe,ep", [(False, False), (True, False), (True, True)])
def test_tp2_matches_tp1_on_cpu(moe, ep):
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 515, (n,), generator=g).tolist() for n in (9, 21)]
    with tempfile.TemporaryDirectory() as tmp:
        ckpt = _make_ckpt(tmp, moe)
        want = _single(ckpt, prompts)
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        port = 29500 + (os.getpid() % 2000) + (2 if moe else 0) + (1 if ep else 0)
        procs = [ctx.Process(target=_worker, args=(r, 2, port, ckpt, prompts, q, ep)) for r in range(2)]
        for p in procs:
            p.start()
        got = q.get(timeout=240)
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    assert got == want


def _dp_worker(rank, world, port, ckpt, prompts_by_rank, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    llm = LLM(model_path=ckpt, device="cpu", dp_size=world, dp_rank=rank, page_size=16, max_running_req=4,
              num_page_override=64, enable_ep=True, dtype="fp32")
    # replica 1 is done after two tokens and has to stay in step with replica 0 until that one is done too
    outs = llm.generate(prompts_by_rank[rank], SamplingParams(max_tokens=6 if rank == 0 else 2, ignore_eos=True))
    out_q.put((rank, [o.token_ids for o in outs], llm.engine.ctx.ep.calls))
    llm.shutdown()


def test_dp2_expert_parallel_lockstep_matches_single_replica():
    """Two replicas with disjoint expert halves and different workloads (one finishes early and
    has to keep running dummy steps) reproduce what one replica with all experts generates."""
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 515, (n,), generator=g).tolist() for n in (9, 21, 14)]
    by_rank = {0: prompts[:2], 1: prompts[2:]}
    with tempfile.TemporaryDirectory() as tmp:
        ckpt = _make_ckpt(tmp, True)
        from minisglang_rdna4_b200 import SamplingParams
        from minisglang_rdna4_b200.llm import LLM

        llm = LLM(model_path=ckpt, device="cpu", page_size=16, max_running_req=4, num_page_override=64, dtype="fp32")
        want = [o.token_ids for o in llm.generate(prompts[:2], SamplingParams(max_tokens=6, ignore_eos=True))]
        want += [o.token_ids for o in llm.generate(prompts[2:], SamplingParams(max_tokens=2, ignore_eos=True))]
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        port = 29900 + os.getpid() % 1000
        procs = [ctx.Process(target=_dp_worker, args=(r, 2, port, ckpt, by_rank, q)) for r in range(2)]
        for p in procs:
            p.start()
        got = dict()
        calls = dict()
        for _ in procs:
            r, toks, n = q.get(timeout=240)
            got[r], calls[r] = toks, n
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    assert got[0] + got[1] == want
    assert calls[0] == calls[1] > 0   # both replicas issued the same number of exchanges


def _dp_timeout_worker(rank, world, port, ckpt, prompts_by_rank, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      MSGL_COMM_HEALTH_STEPS="1")
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    llm = LLM(model_path=ckpt, device="cpu", dp_size=world, dp_rank=rank, page_size=16, max_running_req=4,
              num_page_override=64, enable_ep=True, dtype="fp32")
    ep = llm.engine.ctx.ep
    ep.healthy = True
    polls = [0]

    def poll_status():           # the device status word of a fused exchange: a wait ran out on replica 1 once
        polls[0] += 1
        return 407 if rank == 1 and polls[0] == 3 and ep.healthy else 0

    ep.poll_status = poll_status
    outs = llm.generate(prompts_by_rank[rank], SamplingParams(max_tokens=8, ignore_eos=True))
    out_q.put((rank, [(o.finish_reason, o.error is not None, len(o.token_ids)) for o in outs], ep.healthy))
    llm.shutdown()


def test_exchange_timeout_on_one_replica_is_agreed_and_ends_running_requests():
    """A device-side wait that ran out on one replica reaches the others through the per-step
    agreement: all leave the fused exchange on the same step and the requests that were running
    end with an error instead of continuing on possibly incomplete sums."""
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 515, (n,), generator=g).tolist() for n in (9, 21, 14)]
    by_rank = {0: prompts[:2], 1: prompts[2:]}
    with tempfile.TemporaryDirectory() as tmp:
        ckpt = _make_ckpt(tmp, True)
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        port = 27100 + os.getpid() % 1000
        procs = [ctx.Process(target=_dp_timeout_worker, args=(r, 2, port, ckpt, by_rank, q)) for r in range(2)]
        for p in procs:
            p.start()
        got = dict()
        for _ in procs:
            r, outs, healthy = q.get(timeout=240)
            got[r] = (outs, healthy)
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    for r in (0, 1):
        outs, healthy = got[r]
        assert healthy is False
        assert all(reason == "error" and has_error and n < 8 for reason, has_error, n in outs), outs


def _health_worker(rank, world, port, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist

    from minisglang_rdna4_b200.parallel.symm import agree_status

    dist.init_process_group("gloo", rank=rank, world_size=world)
    # step 1: nobody timed out; step 2: a wait ran out on rank 1 only
    clean = agree_status(0, dist.group.WORLD, world)
    bad = agree_status(3 if rank == 1 else 0, dist.group.WORLD, world)
    out_q.put((rank, clean, bad))
    dist.barrier()
    dist.destroy_process_group()


def test_ranks_agree_on_a_collective_timeout_seen_by_one_rank():
    """The status word of the peer-memory collectives is local to a rank; the health check takes
    the MAX over the control group so that every rank leaves the fused path on the same step."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 28100 + os.getpid() % 1000
    procs = [ctx.Process(target=_health_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got == [(0, 0, 3), (1, 0, 3)]


def _hybrid_ckpt(tmp, family):
    import sys

    sys.path.insert(0, os.path.dirname(__file__))
    if family == "qwen3_5":
        from test_qwen3_5_cpu import _hf_model

        _hf_model(tmp)
    else:
        from safetensors.torch import save_file
        from test_nemotron_h_cpu import _hf_model

        cfg, hf = _hf_model()
        cfg.save_pretrained(tmp)
        save_file({k: v.contiguous() for k, v in hf.state_dict().items()}, f"{tmp}/model.safetensors")
    return tmp


@pytest.mark.parametrize("family", ["qwen3_5", "nemotron_h"])
def test_hybrid_models_tp2_matches_tp1_on_cpu(family):
    """Recurrent layers under tensor parallelism: heads (and the convolution channels, gates and state
    that belong to them) are split over the ranks, the output projection sums."""
    pytest.importorskip("transformers")
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 298, (n,), generator=g).tolist() for n in (9, 21)]
    with tempfile.TemporaryDirectory() as tmp:
        ckpt = _hybrid_ckpt(tmp, family)
        want = _single(ckpt, prompts)
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        port = 29800 + (os.getpid() % 1500) + (7 if family == "qwen3_5" else 11)
        procs = [ctx.Process(target=_worker, args=(r, 2, port, ckpt, prompts, q, False)) for r in range(2)]
        for p in procs:
            p.start()
        got = q.get(timeout=300)
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    assert got == want


def test_speculative_decoding_under_tp2_matches_plain_tp1_on_cpu():
    """Drafts are proposed from the token history, which is identical on all tensor-parallel ranks,
    and the verified arg-max ids are agreed across ranks: a speculative TP2 engine generates what a
    plain single-rank engine generates."""
    g = torch.Generator().manual_seed(6)
    base = torch.randint(0, 515, (6,), generator=g).tolist()
    prompts = [base * 4, torch.randint(0, 515, (17,), generator=g).tolist()]     # one repetitive prompt for the lookup
    with tempfile.TemporaryDirectory() as tmp:
        ckpt = _make_ckpt(tmp, False)
        want = _single(ckpt, prompts)
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        port = 28300 + (os.getpid() % 1500)
        extra = dict(spec_algorithm="ngram", spec_num_draft=3)
        procs = [ctx.Process(target=_worker, args=(r, 2, port, ckpt, prompts, q, False, extra)) for r in range(2)]
        for p in procs:
            p.start()
        got = q.get(timeout=300)
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    assert got == want


def _dp_spec_worker(rank, world, port, ckpt, prompts_by_rank, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    try:
        llm = LLM(model_path=ckpt, device="cpu", dp_size=world, dp_rank=rank, page_size=16, max_running_req=4,
                  num_page_override=64, enable_ep=True, dtype="fp32", spec_algorithm="ngram", spec_num_draft=3)
        outs = llm.generate(prompts_by_rank[rank], SamplingParams(max_tokens=10 if rank == 0 else 4, ignore_eos=True))
        out_q.put((rank, [o.token_ids for o in outs], dict(llm.stats), llm.engine.ctx.ep.calls))
        llm.shutdown()
    except Exception as exc:
        out_q.put((rank, f"{type(exc).__name__}: {exc}", {}, 0))
        raise


def test_speculative_decoding_under_dp2_expert_parallel_lockstep():
    """Replicas that share their experts agree on every step's row count before anybody launches. A
    replica that takes a speculative step proposes and plans it first (its rows are 1 + draft length
    per request), the others pad to the agreed count or run a dummy step; outputs equal a single
    replica that holds all experts and decodes plainly."""
    g = torch.Generator().manual_seed(4)
    base = torch.randint(0, 515, (5,), generator=g).tolist()
    prompts = [base * 4, torch.randint(0, 515, (21,), generator=g).tolist(), (base[:3] + [9]) * 5]
    by_rank = {0: prompts[:2], 1: prompts[2:]}
    with tempfile.TemporaryDirectory() as tmp:
        ckpt = _make_ckpt(tmp, True)
        from minisglang_rdna4_b200 import SamplingParams
        from minisglang_rdna4_b200.llm import LLM

        llm = LLM(model_path=ckpt, device="cpu", page_size=16, max_running_req=4, num_page_override=64, dtype="fp32")
        want = [o.token_ids for o in llm.generate(prompts[:2], SamplingParams(max_tokens=10, ignore_eos=True))]
        want += [o.token_ids for o in llm.generate(prompts[2:], SamplingParams(max_tokens=4, ignore_eos=True))]
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        port = 26900 + os.getpid() % 1000
        procs = [ctx.Process(target=_dp_spec_worker, args=(r, 2, port, ckpt, by_rank, q)) for r in range(2)]
        for p in procs:
            p.start()
        got, stats, calls = dict(), dict(), dict()
        for _ in procs:
            r, toks, st, n = q.get(timeout=300)
            got[r], stats[r], calls[r] = toks, st, n
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    assert got[0] + got[1] == want, (got, want)
    assert calls[0] == calls[1] > 0
    assert stats[0]["spec_steps"] > 0 and stats[0]["spec_drafted"] > 0


def test_chunked_all_reduce_of_moe_prefill_matches_tp1(monkeypatch):
    """MSGL_TP_OVERLAP: a large prefill step of a MoE layer under tensor parallelism reduces its
    output row chunk by row chunk (on the GPU: on a second stream, under the experts of the next
    chunk) and hands finished rows to the next norm. Same tokens as a single rank."""
    monkeypatch.setenv("MSGL_TP_OVERLAP", "1")
    monkeypatch.setenv("MSGL_TP_OVERLAP_MIN_ROWS", "16")
    monkeypatch.setenv("MSGL_TP_OVERLAP_CHUNKS", "3")
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 515, (n,), generator=g).tolist() for n in (9, 37)]
    with tempfile.TemporaryDirectory() as tmp:
        ckpt = _make_ckpt(tmp, True)
        want = _single(ckpt, prompts)
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        port = 25300 + (os.getpid() % 1500)
        procs = [ctx.Process(target=_worker, args=(r, 2, port, ckpt, prompts, q, False)) for r in range(2)]
        for p in procs:
            p.start()
        got = q.get(timeout=240)
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    assert got == want

    from minisglang_rdna4_b200.layers import tp_overlap
    from minisglang_rdna4_b200.parallel import info

    info.set_tp_info(0, 2)
    try:
        assert tp_overlap.applies(16) and not tp_overlap.applies(15)
        monkeypatch.setenv("MSGL_TP_OVERLAP", "0")
        assert not tp_overlap.applies(4096)
    finally:
        info.reset_parallel_info()


def test_block_diffusion_under_tp2_matches_tp1_on_cpu():
    """Block-diffusion decoding on two tensor-parallel ranks: both gather the canvas logits, hold the same
    per-request generator state and so advance their canvases identically; tokens equal a single rank's."""
    import json

    g = torch.Generator().manual_seed(8)
    prompts = [torch.randint(0, 500, (n,), generator=g).tolist() for n in (9, 21)]
    with tempfile.TemporaryDirectory() as tmp:
        ckpt = _make_ckpt(tmp, False)
        cfg = json.load(open(os.path.join(ckpt, "config.json")))
        cfg.update(canvas_length=4, mask_token_id=514)
        json.dump(cfg, open(os.path.join(ckpt, "config.json"), "w"))
        json.dump({"max_denoising_steps": 3, "confidence_threshold": 0.7, "mask_token_id": 514,
                   "sampler_config": {"_cls_name": "MaskConfidenceSamplerConfig"}},
                  open(os.path.join(ckpt, "generation_config.json"), "w"))
        want = _single(ckpt, prompts)
        assert all(len(w) == 6 for w in want)
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        port = 24300 + (os.getpid() % 1500)
        procs = [ctx.Process(target=_worker, args=(r, 2, port, ckpt, prompts, q, False)) for r in range(2)]
        for p in procs:
            p.start()
        got = q.get(timeout=240)
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    assert got == want


@pytest.mark.parametrize("mode", ["tp", "ep", "tp_latent"])
def test_deepseek_v3_tp2_matches_tp1_on_cpu(mode, monkeypatch):
    """Latent attention with zero-padded value heads and the grouped sigmoid routing under tensor parallelism
    (heads and expert width split) and with the experts split over the ranks instead. ``tp_latent``: the two
    ranks keep the compressed latents (each its own copy; its heads' slices of kv_b_proj absorb and expand)
    and give the tokens of one rank with per-head K/V."""
    ep = mode == "ep"
    T = pytest.importorskip("transformers")
    cfg = T.DeepseekV3Config(
        vocab_size=300, hidden_size=64, intermediate_size=128, moe_intermediate_size=32, num_hidden_layers=3,
        num_attention_heads=4, num_key_value_heads=4, n_shared_experts=1, n_routed_experts=8, routed_scaling_factor=2.5,
        kv_lora_rank=32, q_lora_rank=24, qk_rope_head_dim=8, v_head_dim=16, qk_nope_head_dim=24, n_group=2,
        topk_group=1, num_experts_per_tok=2, first_k_dense_replace=1, max_position_embeddings=512, eos_token_id=299,
        bos_token_id=None, pad_token_id=None)
    torch.manual_seed(0)
    hf = T.DeepseekV3ForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for _, p in hf.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn_like(p) * 0.1)
        for n, b in hf.named_buffers():
            if "e_score_correction_bias" in n:
                b.copy_(torch.randn_like(b) * 0.1)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 298, (n,), generator=g).tolist() for n in (9, 21)]
    with tempfile.TemporaryDirectory() as tmp:
        hf.save_pretrained(tmp, safe_serialization=True)
        want = _single(tmp, prompts)
        if mode == "tp_latent":
            monkeypatch.setenv("MSGL_MLA_LATENT", "1")      # the spawned ranks inherit it
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        port = 23100 + (os.getpid() % 1500) + {"tp": 0, "ep": 3, "tp_latent": 6}[mode]
        procs = [ctx.Process(target=_worker, args=(r, 2, port, tmp, prompts, q, ep)) for r in range(2)]
        for p in procs:
            p.start()
        got = q.get(timeout=240)
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    assert got == want
