"""Image input for Gemma-3 multimodal checkpoints: the SigLIP tower and projector against the Hugging
Face model, prompts with images through the engine (placeholder rows take the image features, chunked
prefill across an image, prefix cache that tells images apart), preprocessing, the chat API's image
parts and the tokenizer worker's placeholder expansion."""
import base64
import io
import json
import tempfile

import pytest
import torch

T = pytest.importorskip("transformers")


def _tiny(tmp):
    tc = dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=4, num_attention_heads=4,
              num_key_value_heads=2, head_dim=64, max_position_embeddings=512, rms_norm_eps=1e-6, sliding_window=16,
              query_pre_attn_scalar=48, rope_theta=1e6, rope_local_base_freq=1e4,
              layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"],
              tie_word_embeddings=True, pad_token_id=0, bos_token_id=2, eos_token_id=1)
    vc = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2, image_size=56,
              patch_size=14)
    cfg = T.Gemma3Config(text_config=tc, vision_config=vc, mm_tokens_per_image=4, image_token_index=500,
                         boi_token_index=501, eoi_token_index=502)
    torch.manual_seed(0)
    hf = T.Gemma3ForConditionalGeneration(cfg).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "vision" in n or "multi_modal" in n:
                p.copy_(torch.randn_like(p) * 0.2)
            elif "norm" in n:
                p.copy_(0.1 * torch.randn_like(p))
    hf.save_pretrained(tmp, safe_serialization=True)
    return hf


def _expand(p):
    out = []
    for t in p:
        out += ([501] + [500] * 4 + [502]) if t == 501 else [t]
    return out


def _norm(img):
    return (img.float() / 255.0 - 0.5) / 0.5


def test_vision_tower_and_projector_match_transformers():
    from minisglang_rdna4_b200.models.siglip import VisionConfig, VisionTower

    with tempfile.TemporaryDirectory() as tmp:
        hf = _tiny(tmp)
        px = torch.randn(2, 3, 56, 56)
        with torch.no_grad():
            want = hf.get_image_features(px)
            want = want.pooler_output if hasattr(want, "pooler_output") else want
        vc = VisionConfig.from_hf(json.load(open(f"{tmp}/config.json")))
        assert (vc.tokens_per_image, vc.image_token_id, vc.boi_token_id, vc.patches_per_side) == (4, 500, 501, 4)
        tower = VisionTower(vc, torch.float32, "cpu")
        assert tower.load(tmp) > 20
        got = tower.image_embeddings(px)
        assert got.shape == (8, 128)
        assert torch.allclose(got, want.reshape(-1, want.shape[-1]), atol=1e-5)


@pytest.mark.parametrize("bidirectional", [True, False])
def test_prompts_with_images_match_transformers_and_the_prefix_cache_tells_images_apart(bidirectional, monkeypatch):
    """Image placeholder rows take the projected vision features (unscaled, as the published model inserts
    them); prefill chunks of 16 tokens stop before an image or take all of it; the same prompt with another
    image must not hit the first one's cached pages, the same image again does. The tokens of one image
    attend to each other in both directions during the prefill, as the published model does when it is
    given ``token_type_ids`` (global and sliding-window layers get their own masks); with
    MSGL_IMAGE_BIDIRECTIONAL=0 attention stays causal, which is the published model without them."""
    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM

    monkeypatch.setenv("MSGL_IMAGE_BIDIRECTIONAL", "1" if bidirectional else "0")
    with tempfile.TemporaryDirectory() as tmp:
        hf = _tiny(tmp)
        g = torch.Generator().manual_seed(3)
        imgs = torch.randint(0, 256, (3, 3, 56, 56), generator=g, dtype=torch.uint8)

        def text(n):
            return torch.randint(3, 490, (n,), generator=g).tolist()

        pa = text(5) + [501] + text(20) + [501] + text(7)        # two images inside the text
        pb = text(30)                                           # none
        pc = [501] + text(30)                                   # an image first

        def reference(p, im):
            ids = torch.tensor([_expand(p)])
            kw = {} if im is None else {"pixel_values": _norm(im)}
            if im is not None and bidirectional:
                kw["token_type_ids"] = (ids == 500).long()
            with torch.no_grad():
                out = hf.generate(input_ids=ids, max_new_tokens=8, do_sample=False, eos_token_id=None, pad_token_id=0,
                                  **kw)
            return out[0, ids.shape[1]:].tolist()

        want = [reference(pa, imgs[:2]), reference(pb, None), reference(pc, imgs[2:])]
        llm = LLM(model_path=tmp, device="cpu", dtype="float32", page_size=16, max_running_req=4, num_page_override=64,
                  max_extend_tokens=16)
        assert llm.engine.vision is not None
        sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
        outs = llm.generate([pa, pb, pc], sp, images=[list(imgs[:2]), None, [imgs[2]]])
        assert [o.token_ids for o in outs] == want
        other = llm.generate([pc], sp, images=[[imgs[0]]])[0]
        assert other.token_ids == reference(pc, imgs[:1]) and other.cached_tokens == 0
        again = llm.generate([pc], sp, images=[[imgs[2]]])[0]
        assert again.token_ids == want[2] and again.cached_tokens == 32
        assert not llm.mm                                         # features are dropped with the request
        with pytest.raises(ValueError, match="image marker"):    # an image without its marker in the prompt
            llm.generate([pb], sp, images=[[imgs[0]]])
        llm.shutdown()


def _png(color):
    from PIL import Image

    buf = io.BytesIO()
    Image.new("RGB", (20, 30), color).save(buf, format="PNG")
    return buf.getvalue()


def test_preprocessor_resizes_and_expands_markers():
    from minisglang_rdna4_b200.tokenizer.vision import VisionPreprocessor

    pre = VisionPreprocessor(image_size=56, tokens_per_image=4, image_token_id=500, boi_token_id=501, eoi_token_id=502)
    red = pre.load(_png((255, 0, 0)))
    assert red.shape == (3, 56, 56) and red.dtype == torch.uint8
    assert int(red[0].min()) == 255 and int(red[1].max()) == 0
    url = "data:image/png;base64," + base64.b64encode(_png((0, 0, 255))).decode()
    assert int(pre.load(url)[2].min()) == 255
    assert pre.batch([_png((1, 2, 3)), red]).shape == (2, 3, 56, 56)
    assert pre.expand_placeholders([7, 501, 8], 1) == [7, 501, 500, 500, 500, 500, 502, 8]
    with pytest.raises(ValueError):
        pre.expand_placeholders([7, 8], 1)
    with pytest.raises(ValueError):
        pre.load("http://example.com/cat.png")


def test_chat_api_image_parts_and_worker_expansion(tmp_path):
    from minisglang_rdna4_b200.config import ServerArgs
    from minisglang_rdna4_b200.core import SamplingParams
    from minisglang_rdna4_b200.message import TokenizeMsg
    from minisglang_rdna4_b200.server.api_server import RequestRejected, extract_images
    from minisglang_rdna4_b200.tokenizer.server import TokenizerWorker

    url = "data:image/png;base64," + base64.b64encode(_png((9, 9, 9))).decode()
    msgs = [{"role": "user", "content": [{"type": "text", "text": "what is this?"},
                                         {"type": "image_url", "image_url": {"url": url}},
                                         {"type": "image", "image": url}]}]
    images = extract_images(msgs)
    assert len(images) == 2 and images[0][:4] == b"\x89PNG"
    assert msgs[0]["content"][1] == {"type": "image"} and msgs[0]["content"][2] == {"type": "image"}
    with pytest.raises(RequestRejected):
        extract_images([{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "http://x/y.png"}}]}])

    _tiny(str(tmp_path))

    class Tok:                                        # renders every image part as the begin-of-image marker
        chat_template = None

        def apply_chat_template(self, messages, **kw):
            out = []
            for m in messages:
                for part in m["content"]:
                    out.append("<boi>" if part["type"] == "image" else part["text"])
            return " ".join(out)

        def encode(self, text, add_special_tokens=False):
            return [501 if w == "<boi>" else 10 + len(w) for w in text.split()]

        def decode(self, ids, **kw):
            return ""

    worker = TokenizerWorker(ServerArgs(model_path=str(tmp_path)), tokenizer=Tok())
    replica, user = worker.on_tokenize(TokenizeMsg(1, msgs, SamplingParams(max_tokens=4), images=images))
    assert replica == 0 and user.images.shape == (2, 3, 56, 56)
    ids = user.input_ids.tolist()
    assert ids.count(500) == 8 and ids.count(501) == 2 and ids.count(502) == 2
    none, reply = worker.on_tokenize(TokenizeMsg(2, "plain text", SamplingParams(max_tokens=4), images=images))
    assert none is None and "image" in reply.error
