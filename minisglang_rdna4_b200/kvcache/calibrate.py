"""Offline calibration of the fp8 KV cache scales (tools/kv_fp8_calibrate.py in the reference).

    python -m minisglang_rdna4_b200.kvcache.calibrate --model DIR [--prompts FILE] [--tokens N]

runs the model with a 16-bit KV pool over calibration prompts (one per line of ``--prompts``, or
random token ids when none is given), records the largest |value| per (layer, kv head) of every
K and V row that reaches the pool, and writes ``kv_scales.safetensors`` (``k_scale`` / ``v_scale``
``[layers, kv_heads]`` = amax * margin / 448) next to the checkpoint. An engine started with
``--kv-cache-dtype fp8`` on that directory then uses these scales instead of 1.0.
"""
from __future__ import annotations

import argparse
import os
from typing import List, Optional

import torch


def calibrate(model_path: str, prompts: Optional[List] = None, out: Optional[str] = None, margin: float = 1.0,
              max_new_tokens: int = 16, random_tokens: int = 4096, seed: int = 0, **llm_kwargs):
    """Returns ``(k_scale, v_scale)`` and writes the side-car (``out`` or ``<model>/kv_scales.safetensors``)."""
    from ..core import SamplingParams
    from ..llm import LLM

    keep = os.environ.get("MSGL_KV_FP8_CALIBRATE")
    os.environ["MSGL_KV_FP8_CALIBRATE"] = "1"
    try:
        llm = LLM(model_path, kv_cache_dtype="auto", **llm_kwargs)
        try:
            if not prompts:
                g = torch.Generator().manual_seed(seed)
                vocab = llm.engine.model_config.vocab_size
                per = min(512, max(random_tokens, 1))
                prompts = [torch.randint(0, vocab, (per,), generator=g).tolist()
                           for _ in range(max(random_tokens // per, 1))]
            llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=max_new_tokens, ignore_eos=True))
            return llm.engine.finish_kv_calibration(out, margin)
        finally:
            llm.shutdown()
    finally:
        if keep is None:
            os.environ.pop("MSGL_KV_FP8_CALIBRATE", None)
        else:
            os.environ["MSGL_KV_FP8_CALIBRATE"] = keep


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True)
    ap.add_argument("--prompts", help="text file, one calibration prompt per line")
    ap.add_argument("--tokens", type=int, default=4096, help="random calibration tokens when no prompt file is given")
    ap.add_argument("--out", help="side-car path (default: <model>/kv_scales.safetensors)")
    ap.add_argument("--margin", type=float, default=1.0, help="head-room factor on the recorded amax")
    ap.add_argument("--max-new-tokens", type=int, default=16)
    ap.add_argument("--device", default=None)
    a = ap.parse_args(argv)
    prompts = None
    if a.prompts:
        with open(a.prompts) as f:
            prompts = [ln.rstrip("\n") for ln in f if ln.strip()]
    kw = {"device": a.device} if a.device else {}
    k, v = calibrate(a.model, prompts, a.out, a.margin, a.max_new_tokens, a.tokens, **kw)
    print(f"k_scale {tuple(k.shape)} range [{float(k.min()):.4g}, {float(k.max()):.4g}]; "
          f"v_scale range [{float(v.min()):.4g}, {float(v.max()):.4g}]")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
