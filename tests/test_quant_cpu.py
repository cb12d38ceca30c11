"""Quantisation: codecs against hand-computed values, config parsing of every producer, and a
save → load round trip of a tiny model in every checkpoint format (the reloaded engine must
generate the same tokens as the engine that produced the checkpoint)."""
import json
import os
import tempfile

import pytest
import torch

from minisglang_rdna4_b200 import SamplingParams
from minisglang_rdna4_b200.llm import LLM
from minisglang_rdna4_b200.models.weight import save_dummy_checkpoint
from minisglang_rdna4_b200.ops import ref
from minisglang_rdna4_b200.quant import int4, mxfp4, nvfp4
from minisglang_rdna4_b200.quant.config import QuantConfig


# ------------------------------------------------------------------------------------------ codecs
def test_e2m1_rounding_and_e8m0_scales():
    x = torch.tensor([0.0, 0.24, 0.25, 0.26, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.75, -6.5])
    codes = mxfp4.quantize_e2m1(x)
    lut = torch.tensor(ref.E2M1_VALUES)
    assert lut[codes.long()].tolist() == [0.0, 0.0, 0.0, 0.5, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, -1.0, -6.0]
    s = torch.tensor([0, 126, 127, 128, 254, 255], dtype=torch.uint8)
    f = ref.e8m0_to_float(s)
    assert f[1] == 0.5 and f[2] == 1.0 and f[3] == 2.0 and torch.isnan(f[5]) and f[0] == 2.0 ** -127
    w = torch.randn(8, 64)
    packed, sf = mxfp4.quantize_mxfp4(w)
    assert packed.shape == (8, 32) and sf.shape == (8, 2)
    back = ref.dequant_mxfp4(packed, sf)
    assert (back - w).abs().max() <= w.abs().max() * 0.26
    # low nibble is the even k
    one = torch.zeros(1, 32)
    one[0, 0], one[0, 1] = 1.0, -2.0
    p, _ = mxfp4.quantize_mxfp4(one * 4)
    # amax 8 -> shared scale 2: 4.0 -> +2.0 (code 4) in the low nibble, -8.0 -> -4.0 (code 14) in the high one
    assert int(p[0, 0]) & 0xF == 4 and int(p[0, 0]) >> 4 == 14
    atoms = mxfp4.pack_sf_atoms(sf)
    assert atoms.shape == (1, 1, 32, 4, 4) and torch.equal(mxfp4.unpack_sf_atoms(atoms, 8, 2), sf)


def test_nvfp4_global_scale_conventions_and_int4_layouts():
    w = torch.randn(16, 64) * 0.1
    packed, blk, glob = nvfp4.quantize_nvfp4(w)
    back = ref.dequant_nvfp4(packed, blk, glob)
    assert (back - w).abs().max() <= w.abs().max() * 0.3
    # compressed-tensors stores the reciprocal (divide), ModelOpt the multiplier
    ct = nvfp4.normalise_global_scale(1.0 / glob[:1], 16, divides=True)
    mo = nvfp4.normalise_global_scale(glob[:1], 16, divides=False)
    assert torch.allclose(ct, mo)
    codes, scales, zeros = int4.quantize_int4(w, 32)
    want = int4.dequant_int4(codes, scales, zeros)
    c2, s2, z2 = int4.awq_to_canonical(*int4.pack_awq(codes, scales, zeros))
    assert torch.equal(c2, codes) and torch.allclose(int4.dequant_int4(c2, s2, z2), want, atol=1e-3)
    c3, s3, z3 = int4.gptq_to_canonical(*int4.pack_gptq(codes, scales, zeros), symmetric=False)
    assert torch.equal(c3, codes) and torch.equal(z3, zeros)
    for twos in (False, True):
        packed_ct, sc = int4.pack_ct(codes, scales, twos=twos)
        assert int4.detect_ct_sign_convention(packed_ct) == ("twos" if twos else "offset")
        c4, s4, z4 = int4.ct_to_canonical(packed_ct, sc, None)
        assert torch.equal(c4, codes)
    flat = torch.randint(0, 16, (64, 8), dtype=torch.uint8)     # uniform nibbles: no convention stands out
    amb, _ = int4.pack_ct(flat.view(8, 64), torch.ones(8, 2))
    with pytest.raises(ValueError):
        int4.detect_ct_sign_convention(amb, margin=0.05)


# ------------------------------------------------------------------------------------------ configs
def test_quant_config_producers():
    awq = QuantConfig.from_hf({"quant_method": "awq", "bits": 4, "group_size": 128, "zero_point": True})
    assert awq.default.name == "int4" and awq.default.fmt == "awq" and not awq.default.symmetric
    with pytest.raises(ValueError):
        QuantConfig.from_hf({"quant_method": "gptq", "bits": 4, "desc_act": True})
    ct = QuantConfig.from_hf({"quant_method": "compressed-tensors", "format": "mxfp4-pack-quantized",
                              "config_groups": {"g0": {"targets": ["Linear"], "weights": {
                                  "num_bits": 4, "type": "float", "group_size": 32}}},
                              "ignore": ["lm_head"], "kv_cache_scheme": {"num_bits": 8, "type": "float"}})
    assert ct.default.name == "mxfp4" and ct.kv_cache_fp8
    assert not ct.for_module("lm_head").quantized and ct.for_module("model.layers.0.mlp.down_proj").quantized
    blk = QuantConfig.from_hf({"quant_method": "fp8", "weight_block_size": [128, 128]})
    assert blk.default.name == "fp8_block" and blk.default.block == (128, 128)
    mo = QuantConfig.from_hf({"quantization": {"quant_algo": "NVFP4", "group_size": 16, "kv_cache_quant_algo": "FP8",
                                               "exclude_modules": ["lm_head", "model.layers.*.mlp.gate"]}})
    assert mo.default.name == "nvfp4" and not mo.default.global_scale_divides and mo.kv_cache_fp8
    assert not mo.for_module("model.layers.3.mlp.gate").quantized
    assert QuantConfig.from_hf({"quant_algo": "FP8_PER_CHANNEL_PER_TOKEN"}).default.name == "fp8_channel"
    qk = QuantConfig.from_hf({"quant_method": "quark", "global_quant_config": {"weight": {
        "dtype": "fp4", "scale_format": "e8m0", "group_size": 32}}, "export": {"pack_method": "reorder"}})
    assert qk.default.name == "mxfp4"
    mixed = QuantConfig.from_hf({"quant_method": "compressed-tensors", "config_groups": {
        "a": {"targets": ["re:.*self_attn.*"], "weights": {"num_bits": 8, "type": "float", "strategy": "channel"}},
        "b": {"targets": ["re:.*mlp.*"], "weights": {"num_bits": 4, "type": "int", "group_size": 32}}}})
    assert mixed.for_module("model.layers.0.self_attn.qkv_proj").name == "fp8_channel"
    assert mixed.for_module("model.layers.0.mlp.down_proj").name == "int4"
    assert not mixed.for_module("lm_head").quantized


# ------------------------------------------------------------------------------------------ round trips
_HF = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=128,
           num_attention_heads=2, num_key_value_heads=1, head_dim=128, intermediate_size=256, vocab_size=300,
           rms_norm_eps=1e-6, rope_theta=1e6, max_position_embeddings=512, tie_word_embeddings=True,
           torch_dtype="float32")

_QCFG = {
    "fp8": {"quant_method": "compressed-tensors", "format": "float-quantized", "ignore": ["lm_head"],
            "config_groups": {"g": {"targets": ["Linear"], "weights": {"num_bits": 8, "type": "float",
                                                                        "strategy": "channel"}}}},
    "fp8_block": {"quant_method": "fp8", "weight_block_size": [128, 128]},
    "mxfp4": {"quant_method": "compressed-tensors", "format": "mxfp4-pack-quantized", "ignore": ["lm_head"],
              "config_groups": {"g": {"targets": ["Linear"], "weights": {"num_bits": 4, "type": "float",
                                                                          "group_size": 32}}}},
    "nvfp4": {"quant_method": "compressed-tensors", "format": "nvfp4-pack-quantized", "ignore": ["lm_head"],
              "config_groups": {"g": {"targets": ["Linear"], "weights": {"num_bits": 4, "type": "float",
                                                                          "group_size": 16}}}},
    "int4": {"quant_method": "gptq", "bits": 4, "group_size": 128, "sym": True},
}


@pytest.mark.parametrize("quant", ["fp8", "fp8_block", "mxfp4", "nvfp4", "int4"])
def test_quantized_checkpoint_round_trip(quant):
    from minisglang_rdna4_b200.models.config import ModelConfig

    cfg = ModelConfig.from_hf(dict(_HF))
    kw = dict(device="cpu", page_size=16, max_running_req=4, num_page_override=64, dtype="fp32")
    prompts = [list(range(3, 30)), list(range(100, 111))]
    sp = SamplingParams(max_tokens=5, ignore_eos=True)
    src = LLM(model_config=cfg, use_dummy_weight=True, quantization=quant, seed=11, **kw)
    state = src.engine.model
    with tempfile.TemporaryDirectory() as tmp:
        # the checkpoint has to be written from the pre-repack tensors: rebuild a fresh model
        from minisglang_rdna4_b200.models import create_model
        from minisglang_rdna4_b200.engine.engine import resolve_model_config
        from minisglang_rdna4_b200.config import EngineConfig

        mc = resolve_model_config(EngineConfig(model_config=cfg, quantization=quant))
        raw = create_model(mc, torch.float32, "cpu")
        raw.init_dummy(seed=11)
        save_dummy_checkpoint(raw, tmp, dict(_HF, quantization_config=_QCFG[quant]))
        want = [o.token_ids for o in src.generate(prompts, sp)]
        dst = LLM(model_path=tmp, **kw)
        assert dst.engine.model_config.quant is not None
        got = [o.token_ids for o in dst.generate(prompts, sp)]
    assert got == want
    del state


def test_fp8_kv_calibration_run_writes_the_sidecar_an_fp8_engine_loads():
    """A calibration run (16-bit pool, recorded amax of every stored K / V row) writes per-(layer, head)
    descales; an fp8-KV engine on the same directory picks them up and its greedy output stays close
    to the 16-bit run, where identity scales would clip or underflow."""
    import tempfile

    from minisglang_rdna4_b200 import LLM, SamplingParams
    from minisglang_rdna4_b200.kvcache.calibrate import calibrate
    from minisglang_rdna4_b200.models import ModelConfig, create_model

    cfgd = dict(_HF)
    cfg = ModelConfig.from_hf(cfgd)
    model = create_model(cfg, torch.float32, "cpu")
    model.init_dummy(seed=11, std=0.05)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (40, 23, 64)]
    with tempfile.TemporaryDirectory() as tmp:
        save_dummy_checkpoint(model, tmp, cfgd)
        kw = dict(device="cpu", page_size=16, max_running_req=4, num_page_override=64, dtype="fp32")
        k, v = calibrate(tmp, prompts, max_new_tokens=4, **kw)
        assert os.path.exists(os.path.join(tmp, "kv_scales.safetensors"))
        assert k.shape == (cfg.num_layers, cfg.num_kv_heads) and v.shape == k.shape
        assert float(k.min()) > 0 and not torch.allclose(k, torch.ones_like(k))
        llm = LLM(model_path=tmp, kv_cache_dtype="fp8", **kw)
        try:
            assert torch.allclose(llm.engine.kv_cache.k_scale.cpu(), k) and torch.allclose(
                llm.engine.kv_cache.v_scale.cpu(), v)
            # every stored byte is inside the e4m3 range by construction: |row| / scale <= 448
            out = llm.generate(prompts, SamplingParams(max_tokens=4, ignore_eos=True))
            assert all(len(o.token_ids) == 4 for o in out)
        finally:
            llm.shutdown()
