"""Reference arm of the benchmark: drives the UNMODIFIED reference package (installed under
``baseline/_ref``) through its own offline API, ``minisgl.llm.LLM.generate``.

Nothing of this repository's package is imported here. The reference's kernels are gfx1201 HIP
packages that do not exist on an NVIDIA box, so the run uses the knobs the reference itself
documents for that case: ``MINISGL_TAIL_HIP=0`` (torch elementwise ops,
python/minisgl/layers/_tail_hip.py:22), its attention back-end selector (``auto`` resolves to
the flashinfer TRT-LLM kernels on sm_100, python/minisgl/engine/engine.py:2569-2580; ``fi`` is
the plain flashinfer back-end) and ``use_pynccl=False`` (``--disable-pynccl``). The reference has
no quantised execution path on NVIDIA GPUs, so the arm runs the same model shape and the same
request mix in bf16 with a bf16 KV cache and says so in its result line.

The model directory (``config.json`` plus a word-level tokenizer of the right vocabulary size)
is written to a temporary folder: there is no checkpoint and no network; weights are the
reference's own ``use_dummy_weight`` random initialisation.

Prints one JSON line on rank 0. Exit code 0 with ``{"impl": "reference", "unavailable": ...}``
when the run cannot be made.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import time
import traceback

SHAPES = {
    "qwen3-4b": dict(
        architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=36, hidden_size=2560,
        num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=9728, vocab_size=151936,
        tie_word_embeddings=True, rms_norm_eps=1e-6, rope_theta=1e6, max_position_embeddings=40960,
        hidden_act="silu", attention_bias=False, torch_dtype="bfloat16", bos_token_id=1, eos_token_id=2),
    "qwen3-8b": dict(
        architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=36, hidden_size=4096,
        num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=151936,
        tie_word_embeddings=False, rms_norm_eps=1e-6, rope_theta=1e6, max_position_embeddings=40960,
        hidden_act="silu", attention_bias=False, torch_dtype="bfloat16", bos_token_id=1, eos_token_id=2),
    "qwen3-30b-a3b": dict(
        architectures=["Qwen3MoeForCausalLM"], model_type="qwen3_moe", num_hidden_layers=48, hidden_size=2048,
        num_attention_heads=32, num_key_value_heads=4, head_dim=128, intermediate_size=6144,
        moe_intermediate_size=768, num_experts=128, num_experts_per_tok=8, norm_topk_prob=True,
        decoder_sparse_step=1, mlp_only_layers=[], vocab_size=151936, tie_word_embeddings=False,
        rms_norm_eps=1e-6, rope_theta=1e6, max_position_embeddings=40960, hidden_act="silu",
        attention_bias=False, torch_dtype="bfloat16", bos_token_id=1, eos_token_id=2),
    "llama3-70b": dict(
        architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=80, hidden_size=8192,
        num_attention_heads=64, num_key_value_heads=8, head_dim=128, intermediate_size=28672, vocab_size=128256,
        tie_word_embeddings=False, rms_norm_eps=1e-5, rope_theta=5e5, max_position_embeddings=8192,
        hidden_act="silu", attention_bias=False, mlp_bias=False, torch_dtype="bfloat16", bos_token_id=1,
        eos_token_id=2),
}


def write_model_dir(model: str, path: str) -> None:
    cfg = dict(SHAPES[model])
    with open(os.path.join(path, "config.json"), "w") as fh:
        json.dump(cfg, fh)
    with open(os.path.join(path, "generation_config.json"), "w") as fh:
        json.dump({"bos_token_id": 1, "eos_token_id": 2}, fh)
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    vocab = {f"t{i}": i for i in range(cfg["vocab_size"])}
    vocab["<unk>"] = vocab.pop("t0")
    vocab["<s>"] = vocab.pop("t1")
    vocab["</s>"] = vocab.pop("t2")
    tok = Tokenizer(models.WordLevel(vocab=vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="<unk>", bos_token="<s>", eos_token="</s>")
    fast.save_pretrained(path)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--model", default="qwen3-4b")
    ap.add_argument("--requests", type=int, default=256)
    ap.add_argument("--in-min", type=int, default=512)
    ap.add_argument("--in-max", type=int, default=2048)
    ap.add_argument("--out-len", type=int, default=256)
    ap.add_argument("--max-extend", type=int, default=8192)
    ap.add_argument("--memory-ratio", type=float, default=0.85)
    ap.add_argument("--attention-backend", default="auto")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--model-dir", default=None)
    return ap.parse_args()


def main() -> None:
    args = parse_args()
    os.environ.setdefault("MINISGL_TAIL_HIP", "0")
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    import numpy as np
    import torch

    model_dir = args.model_dir
    if model_dir is None:
        model_dir = tempfile.mkdtemp(prefix="ref_model_")
        write_model_dir(args.model, model_dir)

    from minisgl.core import SamplingParams
    from minisgl.distributed import DistributedInfo
    from minisgl.llm import LLM

    # the reference's engine asserts that CUDA is not initialised before it picks its device
    llm = LLM(
        model_dir, dtype=torch.bfloat16, tp_info=DistributedInfo(rank, world), use_dummy_weight=True,
        max_running_req=args.requests, max_extend_tokens=args.max_extend, memory_ratio=args.memory_ratio,
        attention_backend=args.attention_backend, page_size=args.page_size, use_pynccl=False,
        max_seq_len_override=4096, cuda_graph_max_bs=args.requests,
    )
    eng = llm.engine
    vocab = SHAPES[args.model]["vocab_size"]
    sp = SamplingParams(temperature=0.0, max_tokens=args.out_len, ignore_eos=True)

    # timing only: CUDA events around the reference's own forward calls
    step_events = []
    orig_forward = eng.forward_batch
    stream = getattr(eng, "stream", None) or torch.cuda.current_stream()

    def timed_forward(*a, **kw):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(stream)
        out = orig_forward(*a, **kw)
        e.record(stream)
        step_events.append((s, e))
        return out

    eng.forward_batch = timed_forward

    def make_prompts(seed: int):
        g = np.random.default_rng(seed)
        lens = g.integers(args.in_min, args.in_max + 1, size=args.requests)
        return [g.integers(0, vocab, size=int(n), dtype=np.int32).tolist() for n in lens]

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def one_pass(seed: int):
        prompts = make_prompts(seed)
        step_events.clear()
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        t0 = time.perf_counter()
        outs = llm.generate(prompts, sp)
        ev1.record(stream)
        barrier()
        host_ms = (time.perf_counter() - t0) * 1e3
        n_out = sum(len(o["token_ids"]) for o in outs)
        dev_ms = sum(s.elapsed_time(e) for s, e in step_events)
        return dict(wall_ms=max(ev0.elapsed_time(ev1), 0.0) or host_ms, host_ms=host_ms, dev_ms=dev_ms, n_out=n_out,
                    steps=len(step_events), in_tokens=sum(len(p) for p in prompts))

    for w in range(args.warmup):
        one_pass(1000 + w)
    results = [one_pass(2000 + i) for i in range(args.steps)]

    def reduce_max(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return float(t.item())

    dev_ms = reduce_max(sum(r["dev_ms"] for r in results))
    wall_ms = reduce_max(sum(r["host_ms"] for r in results))
    n_out = sum(r["n_out"] for r in results)
    if rank == 0:
        print(json.dumps({
            "impl": "reference", "metric": "output tok/s (device-timed, max over ranks)",
            "value": n_out / (dev_ms / 1e3) if dev_ms > 0 else None, "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (uniform-random token ids, the reference's own dummy weights)",
            "config": {
                "model": f"{args.model}-shaped, bf16 weights, bf16 KV (the reference has no quantised NVIDIA path)",
                "same_config": False, "global_batch": args.requests,
                "seq_len": f"in U[{args.in_min},{args.in_max}], out {args.out_len}", "parallelism": f"tp{world}",
                "attention_backend": str(getattr(llm.config, "attention_backend", args.attention_backend)),
                "page_size": int(getattr(llm.config, "page_size", args.page_size)),
                "knobs": "MINISGL_TAIL_HIP=0, use_pynccl=False",
                "engine_steps_per_pass": results[-1]["steps"], "prompt_tokens_per_pass": results[-1]["in_tokens"],
            },
            "e2e": {"value": n_out / (wall_ms / 1e3), "unit": "tok/s", "ms_per_pass": wall_ms / args.steps},
        }))
    sys.stdout.flush()


if __name__ == "__main__":
    try:
        main()
    except BaseException as exc:  # the caller decides what to do with a failed attempt
        if isinstance(exc, SystemExit) and exc.code in (0, None):
            raise
        traceback.print_exc()
        sys.stderr.flush()
        os._exit(17)
