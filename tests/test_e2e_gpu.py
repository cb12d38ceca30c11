"""End-to-end engine checks on a GPU: the kernel path against the fp32 oracle path."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _cfg(layers=2, qk_norm=True, **extra):
    from minisglang_rdna4_b200.models.config import ModelConfig, RotaryConfig

    return ModelConfig(
        num_layers=layers, num_qo_heads=8, num_kv_heads=2, head_dim=128, hidden_size=512, vocab_size=2048,
        intermediate_size=1024, rms_norm_eps=1e-6,
        rotary_config=RotaryConfig(head_dim=128, rotary_dim=128, max_position=2048, base=1e6),
        model_type="qwen3", architectures=("Qwen3ForCausalLM",), qk_norm=qk_norm, max_position_embeddings=2048,
        **extra,
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


def _tp_worker(rank, world, port, env, out_q):
    import os

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0", **env)
    torch.cuda.set_device(rank)
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM
    from minisglang_rdna4_b200.ops import cuda as K
    from minisglang_rdna4_b200.parallel.comm import get_comm

    llm = LLM(model_config=_cfg(layers=3), use_dummy_weight=True, quantization="mxfp4", kv_cache_dtype="fp8",
              device="cuda", tp_size=world, tp_rank=rank, page_size=16, max_running_req=8,
              num_page_override=512, seed=0)
    outs = llm.generate(_prompts(), SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    calls = dict(get_comm().calls)
    ok = K.gemm_status() == 0 and K.attn_status() == 0
    if rank == 0:
        out_q.put(([o.token_ids for o in outs], calls, ok))
    llm.shutdown()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp2_fused_paths_track_nccl_only_path():
    """Two tensor-parallel ranks: the peer-memory paths (one-shot all-reduce + norm for decode,
    GEMM -> reduce-scatter -> norm -> all-gather -> GEMM for the 800-token prefill step,
    vocabulary-parallel arg-max) against the same engine with every collective on NCCL. The
    fused kernels round once after adding the residual, NCCL rounds the sum first, so late
    tokens of a sequence may differ; the first tokens must agree."""
    import os

    import torch.multiprocessing as mp

    results = {}
    for name, env in (("fused", {}), ("nccl", {"MSGL_DISABLE_FUSED_COMM": "1"})):
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        port = 29300 + os.getpid() % 500 + (7 if name == "nccl" else 0)
        procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, env, q)) for r in range(2)]
        for p in procs:
            p.start()
        results[name] = q.get(timeout=300)
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
    (fused, calls, ok), (nccl, calls_nccl, ok2) = results["fused"], results["nccl"]
    assert ok and ok2
    assert calls.get("fused_rs_ag", 0) > 0 and calls.get("fused_ar_norm", 0) > 0 and calls.get("vocab_argmax", 0) > 0
    assert calls_nccl.get("fused_rs_ag", 0) == 0 and calls_nccl.get("fused_ar_norm", 0) == 0
    same_first = sum(a[:3] == b[:3] for a, b in zip(fused, nccl))
    assert same_first >= len(fused) - 1, (fused, nccl)


def _moe_cfg():
    from minisglang_rdna4_b200.models.config import ModelConfig, RotaryConfig

    return ModelConfig(
        num_layers=2, num_qo_heads=8, num_kv_heads=2, head_dim=128, hidden_size=512, vocab_size=2048,
        intermediate_size=1024, rms_norm_eps=1e-6,
        rotary_config=RotaryConfig(head_dim=128, rotary_dim=128, max_position=2048, base=1e6),
        model_type="qwen3_moe", architectures=("Qwen3MoeForCausalLM",), qk_norm=True, max_position_embeddings=2048,
        num_experts=16, num_experts_per_tok=4, moe_intermediate_size=256, norm_topk_prob=True,
    )


def _moe_hf_cfg():
    return dict(model_type="qwen3_moe", architectures=["Qwen3MoeForCausalLM"], num_hidden_layers=2, hidden_size=512,
                num_attention_heads=8, num_key_value_heads=2, head_dim=128, intermediate_size=1024, vocab_size=2048,
                rms_norm_eps=1e-6, rope_theta=1e6, max_position_embeddings=2048, tie_word_embeddings=False,
                torch_dtype="bfloat16", num_experts=16, num_experts_per_tok=4, moe_intermediate_size=256,
                norm_topk_prob=True)


def _dp_ep_worker(rank, world, port, ckpt, out_q):
    import os

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM
    from minisglang_rdna4_b200.ops import cuda as K

    llm = LLM(model_path=ckpt, device="cuda", dp_size=world, dp_rank=rank, enable_ep=True, page_size=16,
              max_running_req=8, num_page_override=256, seed=0)
    prompts = _prompts()[rank::world]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    ep = llm.engine.ctx.ep
    ok = K.gemm_status() == 0 and K.attn_status() == 0 and ep.check_health()
    out_q.put((rank, [o.token_ids for o in outs], ok, getattr(ep, "fused_calls", 0),
               llm.engine.graph_runner.replays if llm.engine.graph_runner is not None else -1))
    llm.shutdown()


def test_dp_ep_replicas_match_one_replica():
    """Two replicas, each holding half of the experts of one checkpoint, exchanging rows through
    the peer-memory all-to-all with captured decode graphs: their greedy output equals that of one
    engine that holds all experts."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import os
    import tempfile

    import torch.multiprocessing as mp

    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM
    from minisglang_rdna4_b200.models import ModelConfig, create_model
    from minisglang_rdna4_b200.models.weight import save_dummy_checkpoint

    with tempfile.TemporaryDirectory() as tmp:
        cfgd = _moe_hf_cfg()
        model = create_model(ModelConfig.from_hf(cfgd), torch.bfloat16, "cpu")
        model.init_dummy(seed=7, std=0.05)
        save_dummy_checkpoint(model, tmp, cfgd)
        llm = LLM(model_path=tmp, device="cuda", page_size=16, max_running_req=8, num_page_override=256, seed=0)
        want = [o.token_ids for o in llm.generate(_prompts(), SamplingParams(temperature=0.0, max_tokens=10,
                                                                             ignore_eos=True))]
        llm.shutdown()
        del llm
        torch.cuda.empty_cache()
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        port = 27100 + os.getpid() % 500
        procs = [ctx.Process(target=_dp_ep_worker, args=(r, 2, port, tmp, q)) for r in range(2)]
        for p in procs:
            p.start()
        got = {}
        for _ in procs:
            rank, toks, ok, fused, replays = q.get(timeout=420)
            assert ok and fused > 0 and replays > 0, (rank, ok, fused, replays)
            got[rank] = toks
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
    merged = [None] * len(want)
    for r in (0, 1):
        for i, t in enumerate(got[r]):
            merged[r + 2 * i] = t
    same_first = sum(a[:4] == b[:4] for a, b in zip(merged, want))
    assert same_first >= len(want) - 1, (merged, want)


@pytest.mark.parametrize("quant", [None, "mxfp4", "fp8_block", "fp8"])
def test_moe_model_graph_matches_eager(quant):
    """A small Qwen3-MoE-shaped model end to end on the GPU: fused routing, grouped expert GEMMs
    (16-bit, or W4A8 MXFP4 experts when quantised) and the gate-weighted combine, with CUDA-graph
    decode reproducing eager decode."""
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM
    from minisglang_rdna4_b200.models.config import ModelConfig, RotaryConfig
    from minisglang_rdna4_b200.ops import cuda as K

    cfg = ModelConfig(
        num_layers=2, num_qo_heads=8, num_kv_heads=2, head_dim=128, hidden_size=512, vocab_size=2048,
        intermediate_size=1024, rms_norm_eps=1e-6,
        rotary_config=RotaryConfig(head_dim=128, rotary_dim=128, max_position=2048, base=1e6),
        model_type="qwen3_moe", architectures=("Qwen3MoeForCausalLM",), qk_norm=True, max_position_embeddings=2048,
        num_experts=16, num_experts_per_tok=4, moe_intermediate_size=256, norm_topk_prob=True,
    )
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    outs = {}
    for name, kw in (("graph", dict()), ("eager", dict(cuda_graph_max_bs=-1))):
        llm = LLM(model_config=cfg, use_dummy_weight=True, quantization=quant, device="cuda", page_size=16,
                  max_running_req=8, num_page_override=256, seed=0, **kw)
        outs[name] = [o.token_ids for o in llm.generate(_prompts(), sp)]
        assert K.gemm_status() == 0 and K.attn_status() == 0
        if quant == "mxfp4":
            assert "moe_gemm_grouped_w4a8" in K.LEDGER
        llm.shutdown()
    assert outs["graph"] == outs["eager"]
    assert all(len(t) == 10 for t in outs["graph"])


def test_gemma_style_model_tracks_fp32_oracle():
    """The Gemma-family decoder on the kernel path ((1 + w) norms, GeGLU, sliding-window layers,
    custom query scale, scaled embeddings) against the CPU fp32 oracle path with the same weights."""
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM
    from minisglang_rdna4_b200.models.config import ModelConfig, RotaryConfig

    def cfg():
        return ModelConfig(
            num_layers=4, num_qo_heads=4, num_kv_heads=2, head_dim=128, hidden_size=512, vocab_size=2048,
            intermediate_size=1024, rms_norm_eps=1e-6, hidden_act="gelu_pytorch_tanh",
            rotary_config=RotaryConfig(head_dim=128, rotary_dim=128, max_position=2048, base=1e6),
            model_type="gemma3_text", architectures=("Gemma3ForCausalLM",), qk_norm=True, tie_word_embeddings=True,
            max_position_embeddings=2048, sliding_window=64, query_pre_attn_scalar=96.0, rope_local_base_freq=1e4,
            layer_types=("sliding_attention", "full_attention", "sliding_attention", "full_attention"),
        )

    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    gpu = LLM(model_config=cfg(), use_dummy_weight=True, device="cuda", page_size=16, max_running_req=8,
              num_page_override=256, seed=0)
    state = {k: v.float().cpu() for k, v in gpu.engine.model.state_dict().items()}
    got = [o.token_ids for o in gpu.generate(_prompts(), sp)]
    gpu.shutdown()
    cpu = LLM(model_config=cfg(), use_dummy_weight=True, device="cpu", page_size=16, max_running_req=8,
              num_page_override=256, seed=0)
    cpu.engine.model.load_state_dict(state, strict=False)
    want = [o.token_ids for o in cpu.generate(_prompts(), sp)]
    cpu.shutdown()
    first_ok = sum(g[0] == w[0] for g, w in zip(got, want))
    assert first_ok >= len(want) - 1, (got, want)


@pytest.mark.parametrize("quant,kv,layers", [(None, "bf16", 2), ("mxfp4", "fp8", 2), (None, "bf16", 12)])
def test_speculative_decoding_is_exact_on_the_gpu(quant, kv, layers):
    """Greedy output with a proposer (n-gram, EAGLE3 draft head) equals plain greedy decoding on
    the kernel path: verify rows go through the tree-mask attention kernel and the same GEMM code
    path as decode rows."""
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM
    from minisglang_rdna4_b200.ops import cuda as K

    def make(**kw):
        return LLM(model_config=_cfg(layers=layers), use_dummy_weight=True, quantization=quant, kv_cache_dtype=kv,
                   device="cuda", page_size=16, max_running_req=8, num_page_override=256, seed=0, **kw)

    from minisglang_rdna4_b200.spec.base import Proposer

    class NoDraft(Proposer):
        """Never proposes: every step verifies one row per request, i.e. plain greedy decoding on
        the code path a speculative engine uses (general attention kernel, unsplit K)."""

        name = "none"

        def propose(self, reqs):
            return [[] for _ in reqs]

    prompts = _prompts() + [[5, 6, 7, 8, 9, 10, 11, 12] * 8]   # a repetitive prompt for the n-gram lookup
    sp = SamplingParams(temperature=0.0, max_tokens=20, ignore_eos=True)
    plain = make(spec_algorithm="ngram", spec_num_draft=4)
    plain.proposer = NoDraft(4)
    want = [o.token_ids for o in plain.generate(prompts, sp)]
    assert plain.stats["spec_accepted"] == 0
    plain.shutdown()
    for algo, draft in (("ngram", 4), ("eagle3", 3)):
        spec = make(spec_algorithm=algo, spec_num_draft=draft)
        got = [o.token_ids for o in spec.generate(prompts, sp)]
        assert K.gemm_status() == 0 and K.attn_status() == 0
        assert spec.stats["spec_steps"] > 0 and spec.stats["spec_drafted"] > 0
        # the step ran on the device (propose / verify / accept in one captured graph per bucket)
        assert spec._spec_runner is not None and spec._spec_runner.replays > 0
        assert "spec_accept" in K.LEDGER
        spec.cache.check_integrity()
        spec.shutdown()
        assert got == want, algo
    # the host-driven step (tree verification, sampled acceptance) stays exact as well
    import os

    os.environ["MSGL_SPEC_HOST_STEP"] = "1"
    try:
        host = make(spec_algorithm="ngram", spec_num_draft=4)
        assert [o.token_ids for o in host.generate(prompts, sp)] == want
        host.shutdown()
    finally:
        os.environ.pop("MSGL_SPEC_HOST_STEP", None)


def test_tree_verification_with_the_draft_head_is_exact_and_accepts_siblings():
    """Device tree step (chain + siblings per depth, constant mask, tree acceptance, K/V move). A
    random-init draft head never guesses right, so the head's candidates are replaced by an oracle
    built from the plain run: right at depth 1, while at depth 2 the chain goes wrong and the
    right token sits among the siblings. Every step must then accept the chain token of depth 1, the
    sibling of depth 2 and the bonus token, and the output must still be
    exactly the plain greedy output (which it can only be if the sibling's K/V was moved into place)."""
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM
    from minisglang_rdna4_b200.ops import cuda as K

    def make(**kw):
        return LLM(model_config=_cfg(layers=3), use_dummy_weight=True, device="cuda", page_size=16, max_running_req=8,
                   num_page_override=256, seed=0, **kw)

    prompts = _prompts()
    sp = SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True)
    plain = make(spec_algorithm="eagle3", spec_num_draft=3)
    want = [o.token_ids for o in plain.generate(prompts, sp)]
    plain.shutdown()
    # next-token oracle keyed by (position of the previous token, previous token)
    vocab = _cfg().vocab_size
    oracle = torch.zeros((2048, vocab), dtype=torch.int32)
    for p, w in zip(prompts, want):
        seq = list(p) + list(w)
        for i in range(len(p) - 1, len(seq) - 1):
            oracle[i, seq[i]] = seq[i + 1]
    spec = make(spec_algorithm="eagle3", spec_num_draft=3, spec_tree_width=3)
    from minisglang_rdna4_b200.scheduler.spec_step import device_runner

    runner = device_runner(spec)
    assert runner is not None and runner.T == 3 and runner.R == 10
    assert int(runner.draft.m._draft_vocab) == vocab and not bool(runner.draft.m.d2t.any())
    oracle_d = oracle.cuda()
    state = {"depth": 0, "prev": None}
    eng = spec.engine

    def fake_topk(h_rows, width):
        bs = h_rows.shape[0]
        depth = state["depth"]
        root_pos = runner._v("positions", bs * runner.R).view(bs, runner.R)[:, 0].long()
        if depth == 0:
            root_idx = runner._v("token_idx", bs * runner.R).view(bs, runner.R)[:, 0].long()
            state["prev"] = eng.token_pool.view(-1)[root_idx].long()
        right = oracle_d[(root_pos + depth).clamp_max(2047), state["prev"]].long()
        state["prev"] = right
        state["depth"] = (depth + 1) % runner.K
        wrong = (right + 1) % vocab
        cand = torch.stack([right, wrong, (right + 2) % vocab], dim=1)
        if depth == 1:                       # depth 2 of the tree: the chain is wrong, sibling 0 is right
            cand = torch.stack([wrong, right, (right + 2) % vocab], dim=1)
        return cand.to(torch.int32)

    runner.draft.head_topk = fake_topk
    runner.graphs.clear()
    runner.capture()                         # capture again, now with the oracle in the graphs
    got = [o.token_ids for o in spec.generate(prompts, sp)]
    assert K.gemm_status() == 0 and K.attn_status() == 0
    assert got == want
    steps, emitted = spec.stats["spec_steps"], spec.stats["spec_emitted"]
    assert runner.replays > 0 and "spec_kv_compact" in K.LEDGER
    # chain depth 1 + sibling at depth 2 + bonus = 3 tokens per request-step, except the last steps of a request
    tree_steps = spec.stats["spec_drafted"] // runner.K
    assert tree_steps > 0 and spec.stats["spec_accepted"] >= 1.6 * tree_steps, (steps, emitted, spec.stats)
    spec.cache.check_integrity()
    spec.shutdown()


def test_host_expert_tier_matches_resident_experts_on_the_gpu():
    """MoE experts that do not fit the device budget live in pinned host memory and are copied in
    on a side stream when routed to (SLRU residency cache): the slab forward agrees with the all-resident
    grouped GEMM to 16-bit rounding (a prefill wider than the slab runs in rounds, each rounded to the
    model dtype before the fp32 sum), and an engine built on it generates the same greedy tokens for
    most requests of a random-weight model whose logits are nearly flat."""
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.layers.moe import MoELayer
    from minisglang_rdna4_b200.llm import LLM
    from minisglang_rdna4_b200.models.config import ModelConfig, RotaryConfig

    cfg = ModelConfig(
        num_layers=2, num_qo_heads=8, num_kv_heads=2, head_dim=128, hidden_size=512, vocab_size=2048,
        intermediate_size=1024, rms_norm_eps=1e-6,
        rotary_config=RotaryConfig(head_dim=128, rotary_dim=128, max_position=2048, base=1e6),
        model_type="qwen3_moe", architectures=("Qwen3MoeForCausalLM",), qk_norm=True, max_position_embeddings=2048,
        num_experts=16, num_experts_per_tok=2, moe_intermediate_size=256, norm_topk_prob=True,
    )
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    kw = dict(model_config=cfg, use_dummy_weight=True, device="cuda", page_size=16, max_running_req=8,
              num_page_override=256, seed=0, cuda_graph_max_bs=-1)
    try:
        full = LLM(**kw)
        want = [o.token_ids for o in full.generate(_prompts(), sp)]
        full.shutdown()
        # 2 layers x 16 experts x 3 * 512 * 256 * 2 B = 24 MiB; allow about a third of it on the device
        tiered = LLM(expert_cache_gb=0.008, **kw)
        got = [o.token_ids for o in tiered.generate(_prompts(), sp)]
        tiers = [m._tier for m in tiered.engine.model.modules() if getattr(m, "_tier", None) is not None]
        assert len(tiers) == 2 and all(t.slots < 16 for t in tiers) and sum(t.cache.misses for t in tiers) > 0
        tiered.shutdown()
    finally:
        MoELayer.offload_slots = 0
    assert sum(g == w for g, w in zip(got, want)) >= len(want) - 2, (got, want)

    from minisglang_rdna4_b200 import ops
    from minisglang_rdna4_b200.weights import HostExpertTier

    torch.manual_seed(0)
    e, h, inter, k = 16, 512, 256, 2
    w13 = (torch.randn(e, 2 * inter, h, device="cuda") * 0.05).bfloat16()
    w2 = (torch.randn(e, h, inter, device="cuda") * 0.05).bfloat16()
    tier = HostExpertTier(w13, w2, slots=6, device="cuda")
    for t in (4, 300):  # a decode step inside the slab; a prefill that needs three rounds
        x = torch.randn(t, h, device="cuda").bfloat16()
        ids = torch.randint(0, e if t > 6 else 3, (t, k), device="cuda", dtype=torch.int32)
        w = torch.rand(t, k, device="cuda")
        got_y = tier.forward(x, w, ids).float()
        want_y = ops.moe_forward(x, w13, w2, w, ids, 0).float()
        assert float((got_y - want_y).abs().max()) <= 0.02 * float(want_y.abs().max()) + 1e-3, t
    assert tier.cache.misses > 0 and tier.cache.evictions > 0 and tier.bytes_copied > 0


def test_qwen3_5_hybrid_model_tracks_fp32_oracle():
    """The gated-delta-net / gated-attention hybrid on the kernel path (256-wide attention heads with
    rotary on their first quarter, 128-wide delta-rule heads, recurrent state slots, CUDA-graph decode)
    against the CPU fp32 oracle path with the same weights; graph decode reproduces eager decode."""
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM
    from minisglang_rdna4_b200.models.config import ModelConfig, RotaryConfig

    def cfg():
        return ModelConfig(
            num_layers=4, num_qo_heads=4, num_kv_heads=2, head_dim=256, hidden_size=512, vocab_size=2048,
            intermediate_size=1024, rms_norm_eps=1e-6,
            rotary_config=RotaryConfig(head_dim=256, rotary_dim=64, max_position=2048, base=1e7),
            model_type="qwen3_5_text", architectures=("Qwen3_5ForCausalLM",), qk_norm=True,
            max_position_embeddings=2048, attn_output_gate=True, norm_plus_one=True,
            layer_types=("linear_attention", "linear_attention", "linear_attention", "full_attention"),
            linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=128, linear_value_head_dim=128,
            linear_conv_kernel_dim=4,
        )

    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    outs = {}
    state = None
    for name, kw in (("graph", dict()), ("eager", dict(cuda_graph_max_bs=-1)),
                     ("chunked", dict(cuda_graph_max_bs=-1, max_extend_tokens=96))):
        gpu = LLM(model_config=cfg(), use_dummy_weight=True, device="cuda", page_size=16, max_running_req=8,
                  num_page_override=256, seed=0, **kw)
        if state is None:
            state = {k: v.float().cpu() for k, v in gpu.engine.model.state_dict().items()}
        outs[name] = [o.token_ids for o in gpu.generate(_prompts(), sp)]
        gpu.shutdown()
    assert outs["graph"] == outs["eager"]
    cpu = LLM(model_config=cfg(), use_dummy_weight=True, device="cpu", page_size=16, max_running_req=8,
              num_page_override=256, seed=0)
    cpu.engine.model.load_state_dict(state, strict=False)
    want = [o.token_ids for o in cpu.generate(_prompts(), sp)]
    cpu.shutdown()
    for got in (outs["eager"], outs["chunked"]):
        first_ok = sum(g[0] == w[0] for g, w in zip(got, want))
        assert first_ok >= len(want) - 1, (got, want)


def test_nemotron_h_hybrid_model_tracks_fp32_oracle():
    """Mamba-2 / attention / non-gated MoE hybrid on the kernel path (state-space scan with a register-
    resident state row per thread, convolution with bias, gate-first grouped norm, attention without
    rotary embedding, squared-ReLU experts through the grouped GEMM) against the CPU fp32 oracle path with
    the same weights; graph decode reproduces eager decode and a chunked prefill carries the states over."""
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM
    from minisglang_rdna4_b200.models.config import ModelConfig, RotaryConfig

    def cfg():
        return ModelConfig(
            num_layers=5, num_qo_heads=8, num_kv_heads=2, head_dim=128, hidden_size=512, vocab_size=2048,
            intermediate_size=1024, rms_norm_eps=1e-5,
            rotary_config=RotaryConfig(head_dim=128, rotary_dim=0, max_position=2048, base=1e4),
            model_type="nemotron_h", architectures=("NemotronHForCausalLM",), max_position_embeddings=2048,
            layer_types=("mamba", "moe", "attention", "mlp", "mamba"),
            mamba_num_heads=16, mamba_head_dim=64, ssm_state_size=128, mamba_n_groups=4, time_step_min=0.001,
            mlp_hidden_act="relu2", num_experts=8, num_experts_per_tok=2, moe_intermediate_size=256,
            shared_expert_intermediate_size=512, scoring_func="sigmoid", routed_scaling_factor=1.5,
        )

    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    outs = {}
    state = None
    for name, kw in (("graph", dict()), ("eager", dict(cuda_graph_max_bs=-1)),
                     ("chunked", dict(cuda_graph_max_bs=-1, max_extend_tokens=96))):
        gpu = LLM(model_config=cfg(), use_dummy_weight=True, device="cuda", page_size=16, max_running_req=8,
                  num_page_override=256, seed=0, **kw)
        if state is None:
            state = {k: v.float().cpu() for k, v in gpu.engine.model.state_dict().items()}
        outs[name] = [o.token_ids for o in gpu.generate(_prompts(), sp)]
        gpu.shutdown()
    assert outs["graph"] == outs["eager"]
    cpu = LLM(model_config=cfg(), use_dummy_weight=True, device="cpu", page_size=16, max_running_req=8,
              num_page_override=256, seed=0)
    cpu.engine.model.load_state_dict(state, strict=False)
    want = [o.token_ids for o in cpu.generate(_prompts(), sp)]
    cpu.shutdown()
    for got in (outs["eager"], outs["chunked"]):
        first_ok = sum(g[0] == w[0] for g, w in zip(got, want))
        assert first_ok >= len(want) - 1, (got, want)


def test_glm4_moe_lite_model_tracks_fp32_oracle():
    """Latent-attention + sigmoid-routed MoE decoder on the kernel path (materialised 256-wide heads
    with interleaved rotary on their first 64 channels, selection bias in the routing kernel, shared
    experts, a dense first layer) against the CPU fp32 oracle path with the same weights."""
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM
    from minisglang_rdna4_b200.models.config import ModelConfig, RotaryConfig

    def cfg():
        return ModelConfig(
            num_layers=3, num_qo_heads=4, num_kv_heads=4, head_dim=256, hidden_size=512, vocab_size=2048,
            intermediate_size=1024, rms_norm_eps=1e-5,
            rotary_config=RotaryConfig(head_dim=256, rotary_dim=64, max_position=2048, base=1e6, interleaved=True),
            model_type="glm4_moe_lite", architectures=("Glm4MoeLiteForCausalLM",), max_position_embeddings=2048,
            num_experts=16, num_experts_per_tok=4, moe_intermediate_size=128, norm_topk_prob=True,
            n_shared_experts=1, routed_scaling_factor=1.8, scoring_func="sigmoid", mlp_only_layers=(0,),
            kv_lora_rank=128, q_lora_rank=96, qk_nope_head_dim=192, qk_rope_head_dim=64, v_head_dim=256,
        )

    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    outs = {}
    state = None
    for name, kw in (("graph", dict()), ("eager", dict(cuda_graph_max_bs=-1))):
        gpu = LLM(model_config=cfg(), use_dummy_weight=True, device="cuda", page_size=16, max_running_req=8,
                  num_page_override=256, seed=0, **kw)
        if state is None:
            state = {k: v.float().cpu() for k, v in gpu.engine.model.state_dict().items()}
        outs[name] = [o.token_ids for o in gpu.generate(_prompts(), sp)]
        gpu.shutdown()
    assert outs["graph"] == outs["eager"]
    cpu = LLM(model_config=cfg(), use_dummy_weight=True, device="cpu", page_size=16, max_running_req=8,
              num_page_override=256, seed=0)
    cpu.engine.model.load_state_dict(state, strict=False)
    want = [o.token_ids for o in cpu.generate(_prompts(), sp)]
    cpu.shutdown()
    first_ok = sum(g[0] == w[0] for g, w in zip(outs["eager"], want))
    assert first_ok >= len(want) - 1, (outs["eager"], want)


_CHECKED_ENGINE_CHILD = r"""
import sys
sys.path.insert(0, "tests")
import torch
from test_e2e_gpu import _cfg, _prompts
from minisglang_rdna4_b200 import SamplingParams
from minisglang_rdna4_b200.llm import LLM
from minisglang_rdna4_b200.ops import cuda as K
assert K.bounds_checks_enabled()
sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
outs = []
for kw in (dict(), dict(cuda_graph_max_bs=-1)):
    llm = LLM(model_config=_cfg(), use_dummy_weight=True, quantization="mxfp4", kv_cache_dtype="fp8", device="cuda",
              page_size=16, max_running_req=8, num_page_override=256, seed=0, **kw)
    outs.append([o.token_ids for o in llm.generate(_prompts(), sp)])
    llm.engine.check_device_bounds()       # raises on a recorded index or a touched guard zone
    assert K._GUARDED, "no workspace was guarded"
    llm.shutdown()
assert outs[0] == outs[1]
print("CHECKED-ENGINE-OK")
"""


def test_engine_runs_clean_under_the_bounds_checking_build():
    """A whole engine (graphs and eager) on the bounds-checking kernel library: nothing recorded,
    guard zones intact, same tokens."""
    import os
    import subprocess
    import sys

    from minisglang_rdna4_b200.ops import _lib

    if not os.path.exists(_lib.CHECKED_LIB_PATH):
        from minisglang_rdna4_b200 import build

        build.build_cuda(checked=True)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-c", _CHECKED_ENGINE_CHILD], capture_output=True, text=True, timeout=900,
                         env=dict(os.environ, MSGL_CHECK_BOUNDS="1"), cwd=root)
    assert out.returncode == 0 and "CHECKED-ENGINE-OK" in out.stdout, out.stdout[-2000:] + out.stderr[-4000:]


def test_speculative_decoding_on_a_hybrid_model_rolls_state_back_exactly():
    """Hybrid target on the kernel path with drafts that are right for two tokens and wrong at the
    third: every verify step keeps three of its four rows, so every step restores the recurrent
    states and re-advances them over the kept rows (convolution and delta-rule kernels in their
    multi-row form from a given state). The output equals draft-free decoding token for token."""
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM
    from minisglang_rdna4_b200.models.config import ModelConfig, RotaryConfig

    def cfg():
        return ModelConfig(
            num_layers=4, num_qo_heads=4, num_kv_heads=2, head_dim=256, hidden_size=512, vocab_size=2048,
            intermediate_size=1024, rms_norm_eps=1e-6,
            rotary_config=RotaryConfig(head_dim=256, rotary_dim=64, max_position=2048, base=1e7),
            model_type="qwen3_5_text", architectures=("Qwen3_5ForCausalLM",), qk_norm=True,
            max_position_embeddings=2048, attn_output_gate=True, norm_plus_one=True,
            layer_types=("linear_attention", "linear_attention", "linear_attention", "full_attention"),
            linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=128, linear_value_head_dim=128,
            linear_conv_kernel_dim=4,
        )

    prompts = _prompts()
    sp = SamplingParams(temperature=0.0, max_tokens=20, ignore_eos=True)
    kw = dict(model_config=cfg(), use_dummy_weight=True, device="cuda", page_size=16, max_running_req=8,
              num_page_override=256, seed=0)
    # baseline: the same engine with a proposer that never drafts (one verify row per request per step, so
    # both runs take the same kernels and differ only in what the recurrent layers have to undo)
    plain = LLM(spec_algorithm="ngram", spec_num_draft=3, **kw)
    plain.proposer.propose = lambda reqs: [[] for _ in reqs]
    want = [o.token_ids for o in plain.generate(prompts, sp)]
    assert plain.stats["spec_drafted"] == 0
    plain.shutdown()
    kw["model_config"] = cfg()
    llm = LLM(spec_algorithm="ngram", spec_num_draft=3, **kw)
    by_prompt = {tuple(p): w for p, w in zip(prompts, want)}

    def propose(reqs):
        out = []
        for r in reqs:
            truth = by_prompt[tuple(r.input_ids[: r.prompt_len].tolist())]
            g = r.num_generated                                # tokens generated so far
            d = list(truth[g:g + 3])
            if len(d) == 3:
                d[2] = (d[2] + 1) % 2048                       # the third draft token is wrong
            out.append(d)
        return out

    llm.proposer.propose = propose
    got = [o.token_ids for o in llm.generate(prompts, sp)]
    stats = dict(llm.stats)
    llm.shutdown()
    assert got == want
    assert stats["spec_accepted"] >= 2 * (stats["spec_steps"] // 2), stats
    assert stats["spec_accepted"] < stats["spec_drafted"]


def test_checkpoint_mtp_head_drafts_for_a_hybrid_target_on_the_gpu():
    """The target's own next-token head (one gated-attention decoder layer fed with the final hidden
    state) as the draft model of a hybrid engine: the speculative engine reproduces the output of the
    same engine with drafting switched off, and the head's draft steps really ran."""
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM
    from minisglang_rdna4_b200.models.config import ModelConfig, RotaryConfig

    def cfg():
        return ModelConfig(
            num_layers=4, num_qo_heads=4, num_kv_heads=2, head_dim=256, hidden_size=512, vocab_size=2048,
            intermediate_size=1024, rms_norm_eps=1e-6,
            rotary_config=RotaryConfig(head_dim=256, rotary_dim=64, max_position=2048, base=1e7),
            model_type="qwen3_5_text", architectures=("Qwen3_5ForCausalLM",), qk_norm=True,
            max_position_embeddings=2048, attn_output_gate=True, norm_plus_one=True,
            layer_types=("linear_attention", "linear_attention", "linear_attention", "full_attention"),
            linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=128, linear_value_head_dim=128,
            linear_conv_kernel_dim=4, mtp_num_hidden_layers=1,
        )

    prompts = _prompts()[:4]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    outs = {}
    for name in ("off", "mtp"):
        llm = LLM(model_config=cfg(), use_dummy_weight=True, device="cuda", page_size=16, max_running_req=8,
                  num_page_override=256, seed=0, spec_algorithm="mtp", spec_num_draft=2)
        assert type(llm.proposer).__name__ == "MTPProposer"
        if name == "off":
            llm.proposer.propose = lambda reqs: [[] for _ in reqs]
        outs[name] = [o.token_ids for o in llm.generate(prompts, sp)]
        if name == "mtp":
            assert llm.stats["spec_drafted"] > 0
        llm.shutdown()
    assert outs["mtp"] == outs["off"]


def test_sliding_window_pool_reproduces_the_one_pool_engine_on_the_gpu(monkeypatch):
    """Sliding-window layers in a pool of their own (pages recycled as they leave the window, slots and
    block table derived on the device, inside the decode graphs too): same tokens as the engine that
    keeps every layer's full-length K/V, eager and under graphs, with chunked prefill."""
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM
    from minisglang_rdna4_b200.models.config import ModelConfig, RotaryConfig

    def cfg():
        return ModelConfig(
            num_layers=4, num_qo_heads=4, num_kv_heads=2, head_dim=128, hidden_size=512, vocab_size=2048,
            intermediate_size=1024, rms_norm_eps=1e-6, hidden_act="gelu_pytorch_tanh",
            rotary_config=RotaryConfig(head_dim=128, rotary_dim=128, max_position=2048, base=1e6),
            model_type="gemma3_text", architectures=("Gemma3ForCausalLM",), qk_norm=True, tie_word_embeddings=True,
            max_position_embeddings=2048, sliding_window=64, query_pre_attn_scalar=96.0, rope_local_base_freq=1e4,
            layer_types=("sliding_attention", "full_attention", "sliding_attention", "full_attention"),
        )

    sp = SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True)
    outs = {}
    for name, env, kw in (("one pool", "0", dict()), ("swa graphs", "1", dict()),
                          ("swa eager", "1", dict(cuda_graph_max_bs=-1, max_extend_tokens=96))):
        monkeypatch.setenv("MSGL_SWA_POOL", env)
        llm = LLM(model_config=cfg(), use_dummy_weight=True, device="cuda", page_size=16, max_running_req=8,
                  num_page_override=256, seed=0, **kw)
        assert (llm.engine.swa is not None) == (env == "1")
        outs[name] = [o.token_ids for o in llm.generate(_prompts(), sp)]
        if env == "1":
            llm.engine.swa.check()
            swa = llm.engine.swa
            # what is still held are windows kept for prefix reuse (64 / 16 = 4 pages each)
            assert swa.peak_in_use > 0 and swa.in_use <= 4 * swa.num_snapshots
            if name == "swa graphs":
                assert llm.engine.graph_runner is not None and llm.engine.graph_runner.replays > 0
        llm.shutdown()
    assert outs["swa graphs"] == outs["one pool"]
    # chunked prefill takes the general attention kernel for some rows the one-shot prefill gives to the
    # tensor-core kernel: the first tokens agree, later ones may part at a near-tie
    assert sum(a[0] == b[0] for a, b in zip(outs["swa eager"], outs["one pool"])) >= len(outs["one pool"]) - 1


def test_block_diffusion_decoding_on_the_gpu_tracks_the_cpu_engine():
    """Absorbing-state block diffusion on the kernel path: prompt encode without a sampled row, canvas
    rows through the general attention kernel with a zero mask over the block (windowed-mask form),
    commit and causal re-encode. Same weights on the CPU oracle path: the first block agrees."""
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    over = {"max_denoising_steps": 4, "confidence_threshold": 0.5, "mask_token_id": 2047,
            "sampler_config": {"_cls_name": "MaskConfidenceSamplerConfig"}}

    def make(device):
        return LLM(model_config=_cfg(layers=2, canvas_length=8, mask_token_id=2047), use_dummy_weight=True,
                   device=device, page_size=16, max_running_req=8, num_page_override=256, seed=0,
                   diffusion_overrides=over)

    prompts = _prompts()[:4]
    sp = SamplingParams(temperature=0.0, max_tokens=20, ignore_eos=True)
    gpu = make("cuda")
    assert gpu.diffusion is not None
    state = {k: v.float().cpu() for k, v in gpu.engine.model.state_dict().items()}
    got = [o.token_ids for o in gpu.generate(prompts, sp)]
    again = [o.token_ids for o in gpu.generate(prompts, sp)]
    assert gpu.stats["blocks"] == 2 * 4 * 3 and all(len(x) == 20 for x in got)   # 8 + 8 + 4 tokens per request
    gpu.shutdown()
    assert got == again                                    # greedy: a second pass over the same prompts repeats itself
    cpu = make("cpu")
    cpu.engine.model.load_state_dict(state, strict=False)
    want = [o.token_ids for o in cpu.generate(prompts, sp)]
    cpu.shutdown()
    agree = sum(g[:8] == w[:8] for g, w in zip(got, want))
    assert agree >= len(want) - 1, (got, want)
