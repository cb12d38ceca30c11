import torch

from minisglang_rdna4_b200.ops import ref
from minisglang_rdna4_b200.weights import HostExpertTier, SLRUCache


def test_slru_protects_hot_keys_from_a_scan():
    c = SLRUCache(4, protected_fraction=0.5)
    for k in (1, 2):
        assert c.touch(k) is None
        c.admit(k)
    assert c.touch(1) is not None and c.touch(2) is not None      # promoted to protected
    for k in (10, 11, 12, 13, 14):                                # a scan of one-off keys
        assert c.touch(k) is None
        c.admit(k, pinned=[k])
    assert 1 in c and 2 in c and len(c) == 4
    assert c.evictions == 3
    slots = {c.slot_of(k) for k in (1, 2, 13, 14)}
    assert len(slots) == 4                                        # no slot is shared
    assert c.stats()["hit_rate"] > 0


def test_host_tier_matches_all_resident_experts():
    torch.manual_seed(0)
    e, h, inter, k, t = 16, 32, 24, 2, 12
    w13 = torch.randn(e, 2 * inter, h) * 0.1
    w2 = torch.randn(e, h, inter) * 0.1
    tier = HostExpertTier(w13, w2, slots=6, device="cpu")
    for step in range(6):
        x = torch.randn(t, h)
        # keep each step within the slab: route to at most 6 distinct experts
        pool = torch.randperm(e)[:5]
        ids = pool[torch.randint(0, 5, (t, k))].to(torch.int32)
        w = torch.rand(t, k)
        got = tier.forward(x, w, ids)
        want = ref.moe_forward(x, w13, w2, w, ids)
        assert torch.allclose(got, want, atol=1e-5), step
    assert tier.cache.misses > 0 and tier.cache.evictions > 0 and tier.bytes_copied > 0


def test_engine_with_host_expert_tier_matches_resident_engine():
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM
    from minisglang_rdna4_b200.models.config import ModelConfig, RotaryConfig

    cfg = ModelConfig(num_layers=2, num_qo_heads=2, num_kv_heads=1, head_dim=32, hidden_size=64, vocab_size=300,
                      intermediate_size=128, rms_norm_eps=1e-6, rotary_config=RotaryConfig(32, 32, 512, 1e4),
                      model_type="qwen3_moe", architectures=("Qwen3MoeForCausalLM",), qk_norm=True, num_experts=16,
                      num_experts_per_tok=2, moe_intermediate_size=32, torch_dtype="float32",
                      max_position_embeddings=512)
    prompts = [list(range(5, 25)), list(range(40, 49))]
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    kw = dict(model_config=cfg, use_dummy_weight=True, device="cpu", page_size=16, max_running_req=4,
              num_page_override=64, seed=2)
    want = [o.token_ids for o in LLM(**kw).generate(prompts, sp)]
    # 2 layers x 16 experts x 3*64*32*4 B = 786 KiB in total; allow roughly half of it on the "device"
    tiered = LLM(expert_cache_gb=0.0004, **kw)
    got = [o.token_ids for o in tiered.generate(prompts, sp)]
    assert got == want
    tiers = [m._tier for m in tiered.engine.model.modules() if getattr(m, "_tier", None) is not None]
    assert len(tiers) == 2 and all(t.slots < 16 for t in tiers) and sum(t.cache.misses for t in tiers) > 0
    from minisglang_rdna4_b200.layers.moe import MoELayer
    MoELayer.offload_slots = 0


def test_cpu_expert_tier_matches_fp32_reference():
    """The host library's e2m1 expert MLPs (fp32-activation and int8-activation inner products)
    against the PyTorch restatement, including a skipped (negative) expert id."""
    import torch

    from minisglang_rdna4_b200.quant import mxfp4
    from minisglang_rdna4_b200.weights.cpu_experts import CpuExpertTier

    torch.manual_seed(0)
    experts, hidden, inter = 6, 256, 128
    tier = CpuExpertTier(experts, hidden, inter, group=32, threads=4)
    for e in range(experts - 1):  # the last expert is not resident on the host
        w13, sf13 = mxfp4.quantize_mxfp4(torch.randn(2 * inter, hidden) * 0.05)
        w2, sf2 = mxfp4.quantize_mxfp4(torch.randn(hidden, inter) * 0.05)
        tier.set_expert(e, w13, torch.pow(2.0, sf13.float() - 127), w2, torch.pow(2.0, sf2.float() - 127))
    x = torch.randn(9, hidden)
    ids = torch.randint(0, experts, (9, 3), dtype=torch.int32)
    ids[0, 0] = -1
    w = torch.softmax(torch.randn(9, 3), -1)
    want = tier.reference(x, ids, w)
    got = tier.forward(x, ids, w)
    assert float((got - want).abs().max()) < 1e-4 * max(1.0, float(want.abs().max()))
    got8 = tier.forward(x, ids, w, int8_activations=True)
    assert float((got8 - want).abs().max()) < 0.05 * float(want.abs().max())
    assert tier.isa in ("scalar", "avx512-fp32", "avx512-vnni-int8")
    tier.close()


def test_offload_plan_resolver_and_agreement():
    import pytest

    from minisglang_rdna4_b200.weights import ExpertGeometry, PlanError, TierBudgets, resolve_plan
    from minisglang_rdna4_b200.weights.plan import check_agreement

    geo = ExpertGeometry(num_moe_layers=4, num_experts=64, experts_per_token=8, bytes_per_expert=1 << 20)
    fits = resolve_plan(geo, TierBudgets(device_bytes=4 * 64 << 20))
    assert not fits.offloaded and fits.host_bytes == 0 and fits.device_bytes == 4 * 64 << 20
    half = resolve_plan(geo, TierBudgets(device_bytes=4 * 32 << 20))
    assert half.offloaded and [p.device_slots for p in half.layers] == [32] * 4
    assert all(p.host_experts == 64 and p.disk_experts == 0 for p in half.layers)   # every expert has a host home
    tiny = resolve_plan(geo, TierBudgets(device_bytes=1 << 20))
    assert tiny.layers[0].device_slots == 16 and tiny.notes                       # raised to two steps' worth
    with pytest.raises(PlanError):
        resolve_plan(geo, TierBudgets(device_bytes=4 * 32 << 20, host_bytes=4 * 40 << 20))
    disk = resolve_plan(geo, TierBudgets(device_bytes=4 * 32 << 20, host_bytes=4 * 40 << 20, disk=True))
    assert disk.layers[0].host_experts == 40 and disk.layers[0].disk_experts == 24
    assert half.digest == resolve_plan(geo, TierBudgets(device_bytes=4 * 32 << 20)).digest != disk.digest
    check_agreement([half.digest, half.digest])
    with pytest.raises(PlanError):
        check_agreement([half.digest, disk.digest])


def test_memory_ledger_host_capacity_and_boot_timeline():
    import pytest

    from minisglang_rdna4_b200.weights import BootTimeline, MemoryLedger
    from minisglang_rdna4_b200.weights.host_capacity import check_pinned, pinned_budget

    led = MemoryLedger(capacity_bytes=10 << 30)
    led.add("weights", 4 << 30)
    led.add("kv pool", 5 << 30)
    led.add("weights", 1 << 29)
    assert led.total == (9 << 30) + (1 << 29) and led.entries()[0][0] == "kv pool"
    assert led.would_fit(1 << 28) and not led.would_fit(1 << 30)
    led.release("kv pool", 1 << 30)
    assert led.headroom() == (1 << 30) + (1 << 29) and "weights 4.50 GiB" in led.report()

    meminfo = lambda: "MemTotal: 100 kB\nMemAvailable:   10485760 kB\n"
    assert pinned_budget(0.2, meminfo, (-1, -1)) == int(10 * (1 << 30) * 0.8)
    assert pinned_budget(0.2, meminfo, (2 << 30, 2 << 30)) == 2 << 30
    check_pinned(7 << 30, read_meminfo=meminfo, memlock=(-1, -1))
    with pytest.raises(MemoryError):
        check_pinned(9 << 30, read_meminfo=meminfo, memlock=(-1, -1))

    ticks = iter([0.0, 1.0, 4.0, 4.5])
    tl = BootTimeline(clock=lambda: next(ticks))
    assert tl.mark("weights") == 1.0 and tl.mark("kv pool") == 3.0 and tl.mark("graphs") == 0.5
    out = tl.render()
    assert "4.50 s" in out and "kv pool" in out and "66.7 %" in out


def test_route_trace_and_disk_tier(tmp_path):
    from minisglang_rdna4_b200.weights import DiskExpertTier, ExpertFile, HostExpertTier, RouteTrace

    tr = RouteTrace(8)
    tr.record(0, [1, 1, 3, -1, 9])
    tr.record(0, torch.tensor([1, 2]).numpy())
    tr.record(2, [7])
    assert tr.hottest(0, 2) == [1, 2] and tr.hottest(1, 3) == [] and tr.skew(0) == 0.6
    path = str(tmp_path / "trace.json")
    tr.save(path)
    again = RouteTrace.load(path)
    assert again.hottest(0, 3) == [1, 2, 3] and again.steps == 3

    torch.manual_seed(0)
    w13 = torch.randn(8, 6, 4)
    tier = HostExpertTier(w13, torch.randn(8, 4, 3), slots=4, device="cpu")
    tier.trace, tier.layer_index = RouteTrace(8), 5
    tier.prewarm([1, 2])
    misses = tier.cache.misses
    tier.forward(torch.randn(2, 4), torch.rand(2, 2), torch.tensor([[1, 2], [2, 1]], dtype=torch.int32))
    assert tier.cache.misses == misses and tier.trace.hottest(5, 2) == [1, 2]

    f = ExpertFile(str(tmp_path / "w13.bin"), layers=2, experts=8, shape=(6, 4), dtype=torch.float32)
    f.create()
    for e in range(8):
        f.write(1, e, w13[e])
    assert f.stride == 4096 and f.offset(1, 3) == (8 + 3) * 4096
    disk = DiskExpertTier({"w13": f}, workers=2)
    out = {"w13": torch.empty(3, 6, 4)}
    disk.fetch(1, [5, 0, 7], out)
    assert torch.equal(out["w13"], w13[[5, 0, 7]]) and disk.bytes_read == 3 * 96
    disk.close()


def test_three_tier_engine_matches_resident_engine(tmp_path):
    """Device slab < pinned arena < expert set: misses of the arena are read from the flat files."""
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.layers.moe import MoELayer
    from minisglang_rdna4_b200.llm import LLM
    from minisglang_rdna4_b200.models.config import ModelConfig, RotaryConfig

    cfg = ModelConfig(num_layers=2, num_qo_heads=2, num_kv_heads=1, head_dim=32, hidden_size=64, vocab_size=300,
                      intermediate_size=128, rms_norm_eps=1e-6, rotary_config=RotaryConfig(32, 32, 512, 1e4),
                      model_type="qwen3_moe", architectures=("Qwen3MoeForCausalLM",), qk_norm=True, num_experts=16,
                      num_experts_per_tok=2, moe_intermediate_size=32, torch_dtype="float32",
                      max_position_embeddings=512)
    prompts = [list(range(5, 25)), list(range(40, 49))]
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    kw = dict(model_config=cfg, use_dummy_weight=True, device="cpu", page_size=16, max_running_req=4,
              num_page_override=64, seed=2)
    try:
        want = [o.token_ids for o in LLM(**kw).generate(prompts, sp)]
        per_layer = 3 * 64 * 32 * 4                                      # bytes of one expert
        tiered = LLM(expert_cache_gb=2 * 6 * per_layer / (1 << 30),      # 6 device slots per layer
                     expert_host_gb=2 * 10 * per_layer / (1 << 30),      # 10 pinned rows per layer
                     expert_disk_dir=str(tmp_path), **kw)
        got = [o.token_ids for o in tiered.generate(prompts, sp)]
        tiers = [m._tier for m in tiered.engine.model.modules() if getattr(m, "_tier", None) is not None]
        assert len(tiers) == 2 and all(t.slots == 6 and t.host_cache.capacity == 10 for t in tiers)
        assert sum(t.disk.bytes_read for t in tiers) > 0 and sum(t.host_cache.evictions for t in tiers) > 0
        assert tiered.engine.offload_plan.layers[0].disk_experts == 6
    finally:
        MoELayer.offload_slots, MoELayer.offload_host_experts, MoELayer.offload_disk_dir = 0, 0, ""
    assert got == want


def test_pinned_arena_places_regions_before_it_allocates():
    """Placement is integer arithmetic (aligned offsets, no region across two chunks, an oversized
    region alone in its chunk); memory appears at attach(), after which the arena is frozen."""
    import torch

    from minisglang_rdna4_b200.weights.pinned_arena import ALIGN, ChunkPlan, PinnedArena

    plan = ChunkPlan(chunk_bytes=4096)
    a = plan.reserve("a", (100,), torch.float32)          # 400 B -> 512
    b = plan.reserve("b", (3, 500), torch.uint8)          # 1500 B -> 1536
    c = plan.reserve("c", (600,), torch.float32)          # 2400 B -> does not fit behind a + b
    d = plan.reserve("d", (3000,), torch.float32)         # 12000 B > chunk: a chunk of its own
    assert (a.chunk, a.offset, b.chunk, b.offset) == (0, 0, 0, 512)
    assert (c.chunk, c.offset) == (1, 0) and (d.chunk, d.offset) == (2, 0)
    assert all(r.offset % ALIGN == 0 for r in plan.regions.values())
    assert plan.chunk_sizes == [2048, 2560, 12288]

    arena = PinnedArena(pin=False, chunk_bytes=4096)
    arena.reserve("w13", (4, 8, 16), torch.bfloat16)
    arena.reserve("w2", (4, 16, 4), torch.bfloat16)
    assert arena.num_chunks == 0
    arena.attach()
    assert arena.num_chunks == 1 and arena.frozen
    w13, w2 = arena.get("w13"), arena.get("w2")
    w13.fill_(1.0)
    w2.fill_(2.0)
    assert float(w13.float().sum()) == 4 * 8 * 16 and float(w2.float().sum()) == 2 * 4 * 16 * 4   # no overlap
    import pytest

    with pytest.raises(RuntimeError):
        arena.reserve("late", (4,), torch.float32)
    one_call = PinnedArena(pin=False)
    t = torch.arange(12, dtype=torch.float32).view(3, 4)
    assert torch.equal(one_call.put("x", t), t) and torch.equal(one_call.put("y", t * 2), t * 2)
    assert torch.equal(one_call.get("x"), t)


def test_frame_arena_recycles_frames_first_released_first():
    import torch

    from minisglang_rdna4_b200.kvcache.host_arena import FrameLayout, PinnedFrameArena

    layout = FrameLayout([("conv", (2, 6, 3), torch.bfloat16), ("ssm", (2, 4, 8, 8), torch.float32)])
    assert layout.components[1].offset == 256 and layout.frame_bytes == 256 + 2048
    assert layout.frames_in(10_000) == 4
    arena = PinnedFrameArena(layout, 3, pin=False)
    f = [arena.alloc() for _ in range(3)]
    assert f == [0, 1, 2] and arena.alloc() is None
    for i in f:
        v = arena.views(i)
        v["conv"].fill_(i + 1)
        v["ssm"].fill_(10 * (i + 1))
    assert [float(arena.views(i)["ssm"][0, 0, 0, 0]) for i in f] == [10.0, 20.0, 30.0]   # frames do not overlap
    arena.release(1)
    arena.release(1)                      # dropping twice is harmless
    arena.release(0)
    assert arena.num_free == 2
    assert arena.alloc() == 1 and arena.alloc() == 0 and arena.alloc() is None


def test_baked_checkpoint_round_trip(tmp_path, monkeypatch):
    """First boot with MSGL_BAKED_DIR parses the checkpoint and writes the rank's tensors to one flat
    file; the second boot streams that file instead (same tensors, same tokens); a changed
    checkpoint (other fingerprint) is loaded the ordinary way and re-baked; a damaged file is caught
    by the checksums."""
    import json
    import os
    import sys

    import pytest
    import torch

    sys.path.insert(0, os.path.dirname(__file__))
    from test_tp_cpu import _make_ckpt

    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM
    from minisglang_rdna4_b200.weights import bake

    ckpt = _make_ckpt(str(tmp_path / "ckpt"), moe=True)
    baked = str(tmp_path / "baked")
    monkeypatch.setenv("MSGL_BAKED_DIR", baked)
    kw = dict(model_path=ckpt, device="cpu", page_size=16, max_running_req=4, num_page_override=64, dtype="fp32")
    prompts = [[5, 6, 7, 8, 9], list(range(40, 61))]
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    first = LLM(**kw)
    assert first.engine.baked_bytes is None                         # nothing to read yet: parsed, then written
    data, index = bake.paths(baked, 0)
    assert os.path.isfile(data) and os.path.isfile(index)
    meta = json.load(open(index))
    assert all(e["offset"] % 4096 == 0 for e in meta["tensors"]) and meta["bytes"] == os.path.getsize(data)
    want_state = {k: v.clone() for k, v in first.engine.model.state_dict().items()}
    want = [o.token_ids for o in first.generate(prompts, sp)]
    first.shutdown()

    monkeypatch.setenv("MSGL_BAKED_VERIFY", "1")
    second = LLM(**kw)
    assert second.engine.baked_bytes == meta["bytes"]
    got_state = second.engine.model.state_dict()
    assert set(got_state) == set(want_state)
    assert all(torch.equal(got_state[k], want_state[k]) for k in want_state)
    assert [o.token_ids for o in second.generate(prompts, sp)] == want
    second.shutdown()

    # a flipped byte inside a tensor
    with open(data, "r+b") as fh:
        fh.seek(meta["tensors"][3]["offset"] + 5)
        b = fh.read(1)
        fh.seek(meta["tensors"][3]["offset"] + 5)
        fh.write(bytes([b[0] ^ 0xFF]))
    with pytest.raises(IOError, match="checksum"):
        LLM(**kw)

    # another checkpoint in the same place: the fingerprint differs, the old file is not used
    cfg = json.load(open(os.path.join(ckpt, "config.json")))
    cfg["rms_norm_eps"] = 2e-6
    json.dump(cfg, open(os.path.join(ckpt, "config.json"), "w"))
    third = LLM(**kw)
    assert third.engine.baked_bytes is None
    assert json.load(open(index))["fingerprint"] != meta["fingerprint"]
    third.shutdown()
