import json

from minisglang_rdna4_b200.utils import hf


class _Tok:
    eos_token_id = 7
    chat_template = None


def test_stop_tokens_sampling_defaults_and_templates(tmp_path, monkeypatch):
    d = tmp_path / "model"
    d.mkdir()
    (d / "generation_config.json").write_text(json.dumps(
        {"eos_token_id": [128001, 128008, 128009], "temperature": 0.6, "top_p": 0.95, "top_k": 20, "do_sample": True}))
    path = str(d)
    hf.load_generation_config.cache_clear()
    assert hf.resolve_stop_token_ids(path, _Tok(), (128001, 5)) == [128001, 128008, 128009, 7, 5]
    assert hf.sampling_defaults(path) == {"temperature": 0.6, "top_p": 0.95, "top_k": 20}
    assert hf.resolve_stop_token_ids(str(tmp_path / "missing"), None, (3,)) == [3]

    assert hf.side_chat_template(path) is None
    (d / "chat_template.jinja").write_text("{{ jinja }}")
    assert hf.side_chat_template(path) == "{{ jinja }}"
    (d / "chat_template.json").write_text(json.dumps({"chat_template": "{{ from_json }}"}))
    assert hf.side_chat_template(path) == "{{ from_json }}"
    tok = hf.apply_chat_template_sources(_Tok(), path)
    assert tok.chat_template == "{{ from_json }}"

    monkeypatch.setenv("MSGL_CHAT_TEMPLATE", "{{ literal }}")
    monkeypatch.setenv("MSGL_CHAT_TEMPLATE_MODEL", path)
    assert hf.chat_template_override(path) == "{{ literal }}" and hf.chat_template_override("other") is None
    own = _Tok()
    own.chat_template = "{{ own }}"
    assert hf.apply_chat_template_sources(own, path).chat_template == "{{ literal }}"   # the override wins
    f = tmp_path / "t.jinja"
    f.write_text("{{ file }}")
    monkeypatch.setenv("MSGL_CHAT_TEMPLATE", str(f))
    assert hf.chat_template_override(path) == "{{ file }}"


def test_engine_model_config_unions_generation_config_stops(tmp_path):
    from minisglang_rdna4_b200.config import EngineConfig
    from minisglang_rdna4_b200.engine.engine import resolve_model_config

    d = tmp_path / "m"
    d.mkdir()
    (d / "config.json").write_text(json.dumps({
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 64, "intermediate_size": 128,
        "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "vocab_size": 1000,
        "rms_norm_eps": 1e-5, "max_position_embeddings": 512, "eos_token_id": 2, "torch_dtype": "float32"}))
    (d / "generation_config.json").write_text(json.dumps({"eos_token_id": [2, 9, 11]}))
    hf.load_generation_config.cache_clear()
    mc = resolve_model_config(EngineConfig(model_path=str(d), device="cpu"))
    assert mc.eos_token_ids == (2, 9, 11)


def test_server_applies_generation_defaults_to_unset_fields(tmp_path):
    from minisglang_rdna4_b200.server import api_server as S

    d = tmp_path / "m"
    d.mkdir()
    (d / "generation_config.json").write_text(json.dumps({"temperature": 0.7, "top_p": 0.8, "top_k": 20}))
    hf.load_generation_config.cache_clear()
    try:
        assert S.set_sampling_defaults(str(d)) == {"temperature": 0.7, "top_p": 0.8, "top_k": 20}
        req = S.OpenAICompletionRequest(model="m", messages=[{"role": "user", "content": "hi"}], top_p=0.5)
        sp = S.sampling_from_request(req, None, None)
        assert (sp.temperature, sp.top_p, sp.top_k) == (0.7, 0.5, 20)
    finally:
        S.set_sampling_defaults("")
    sp = S.sampling_from_request(S.OpenAICompletionRequest(model="m", messages=[{"role": "user", "content": "hi"}]),
                                 None, None)
    assert (sp.temperature, sp.top_p, sp.top_k) == (0.0, 1.0, -1)


def test_hub_names_resolve_through_the_local_cache_or_fail_clearly(tmp_path, monkeypatch):
    """A directory or a built-in shape passes through; a repository name is looked up in the local hub cache
    (a snapshot laid out the way the hub client stores it) and, with downloads off, fails with a message that
    says what was tried."""
    import pytest

    from minisglang_rdna4_b200.utils.hub import looks_like_repo, resolve_model_path

    assert resolve_model_path(str(tmp_path)) == str(tmp_path)
    assert resolve_model_path("qwen3-4b") == "qwen3-4b" and resolve_model_path("") == "" and resolve_model_path(None) is None
    assert looks_like_repo("acme/tiny-model") and not looks_like_repo("/abs/path") and not looks_like_repo("a/b/c")
    cache = tmp_path / "hub"
    snap = cache / "models--acme--tiny-model" / "snapshots" / "abc123"
    snap.mkdir(parents=True)
    (snap / "config.json").write_text("{}")
    refs = cache / "models--acme--tiny-model" / "refs"
    refs.mkdir()
    (refs / "main").write_text("abc123")
    monkeypatch.setenv("HF_HUB_CACHE", str(cache))
    monkeypatch.setenv("HF_HOME", str(tmp_path))
    import huggingface_hub.constants as C

    monkeypatch.setattr(C, "HF_HUB_CACHE", str(cache))
    got = resolve_model_path("acme/tiny-model")
    assert got is not None and got.endswith("abc123") and (tmp_path / "hub").as_posix() in got
    monkeypatch.setenv("MSGL_HUB_OFFLINE", "1")
    with pytest.raises(FileNotFoundError, match="downloads are off"):
        resolve_model_path("acme/other-model")
