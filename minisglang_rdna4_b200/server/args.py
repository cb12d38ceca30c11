"""Command line → ``ServerArgs``. Flag names and aliases follow the reference
(python/minisgl/server/args.py:101-458) so existing launch lines keep working; flags that
selected one of its several backends are accepted and ignored."""
from __future__ import annotations

import argparse
import json
from typing import List, Optional

from ..config import ServerArgs


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="python -m minisglang_rdna4_b200", description="B200-native LLM server")
    p.add_argument("--model-path", "--model", dest="model_path", required=True)
    p.add_argument("--served-model-name", default=None)
    p.add_argument("--dtype", default="auto", choices=["auto", "fp16", "bf16", "fp32"])
    p.add_argument("--tensor-parallel-size", "--tp-size", "--tp", dest="tp_size", type=int, default=1)
    p.add_argument("--data-parallel-size", "--dp-size", "--dp", dest="dp_size", type=int, default=1)
    p.add_argument("--enable-ep", action="store_true")
    p.add_argument("--max-running-requests", dest="max_running_req", type=int, default=256)
    p.add_argument("--max-seq-len-override", type=int, default=None)
    p.add_argument("--distributed-timeout", type=float, default=60.0)
    p.add_argument("--memory-ratio", type=float, default=0.9)
    p.add_argument("--weight-offload-gb", type=float, default=0.0)
    p.add_argument("--weight-offload-device-gb", type=float, default=0.0)
    p.add_argument("--expert-cache-gb", type=float, default=0.0)
    p.add_argument("--expert-host-gb", type=float, default=0.0,
                   help="pinned host budget of the expert tier; 0 pins every expert")
    p.add_argument("--expert-disk-dir", default="", help="directory of the disk tier's flat expert files")
    p.add_argument("--weight-offload-cpu-layers", type=int, default=0)
    p.add_argument("--weight-offload-stream-layers", type=int, default=0)
    p.add_argument("--dummy-weight", dest="use_dummy_weight", action="store_true")
    p.add_argument("--disable-pynccl", dest="use_pynccl", action="store_false")
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=1919)
    p.add_argument("--cuda-graph-max-bs", "--graph", dest="cuda_graph_max_bs", type=int, default=None)
    p.add_argument("--num-tokenizer", "--tokenizer-count", dest="num_tokenizer", type=int, default=0)
    p.add_argument("--max-prefill-length", "--max-extend-length", dest="max_extend_tokens", type=int, default=8192)
    p.add_argument("--num-pages", dest="num_page_override", type=int, default=None)
    p.add_argument("--page-size", type=int, default=16)
    p.add_argument("--attention-backend", "--attn", dest="attention_backend", default="auto")
    p.add_argument("--model-source", default="huggingface", choices=["huggingface", "modelscope"])
    p.add_argument("--cache-type", default="radix", choices=["radix", "naive"])
    p.add_argument("--gdn-radix", dest="gdn_radix", action="store_true", default=True)
    p.add_argument("--no-gdn-radix", dest="gdn_radix", action="store_false")
    p.add_argument("--moe-backend", default="auto")
    p.add_argument("--kv-cache-dtype", default="auto", choices=["auto", "bf16", "fp8"])
    p.add_argument("--quantization", default=None, choices=[None, "mxfp4", "nvfp4", "fp8", "fp8_block", "int4"])
    p.add_argument("--shell-mode", action="store_true")
    p.add_argument("--chat-template", default=None)
    p.add_argument("--chat-template-kwargs", default=None, help="JSON object merged into every template call")
    p.add_argument("--reasoning-parser", default="auto")
    p.add_argument("--spec-algorithm", default="none", choices=["none", "ngram", "mtp", "eagle3", "dflash", "tidar"])
    p.add_argument("--spec-draft-model-path", "--spec-draft-model", dest="spec_draft_model_path", default=None)
    p.add_argument("--spec-num-draft", type=int, default=4)
    p.add_argument("--spec-ngram-max", type=int, default=3)
    p.add_argument("--spec-ngram-min", type=int, default=1)
    p.add_argument("--spec-tree-width", type=int, default=1)
    p.add_argument("--disable-overlap", action="store_true")
    p.add_argument("--device", default="auto", choices=["auto", "cuda", "cpu"])
    # recursive self-aggregation (python/minisgl/rsa/config.py:157-228): N rollouts, T rounds in which
    # every rollout is rewritten from K candidates, then a vote over the final answers
    p.add_argument("--rsa-n", type=int, default=4)
    p.add_argument("--rsa-k", type=int, default=2)
    p.add_argument("--rsa-t", type=int, default=2)
    p.add_argument("--rsa-tail-tokens", type=int, default=1024)
    p.add_argument("--rsa-max-tokens", type=int, default=1024)
    p.add_argument("--rsa-agg-max-tokens", type=int, default=1024)
    p.add_argument("--rsa-temperature", type=float, default=0.7)
    p.add_argument("--rsa-top-p", type=float, default=0.95)
    p.add_argument("--rsa-selection", default="vote", choices=["vote", "first", "longest"])
    p.add_argument("--rsa-max-concurrency", type=int, default=8)
    p.add_argument("--rsa-max-retries", type=int, default=1)
    p.add_argument("--rsa-effort-ladder", action="store_true",
                   help="`reasoning_effort` medium / high / max runs the request through self-aggregation")
    # shorthands for environment switches (the engine processes inherit the environment)
    p.add_argument("--swa-pool", action="store_true",
                   help="sliding-window layers keep their K/V in a pool of their own with recycled pages (MSGL_SWA_POOL)")
    p.add_argument("--mla-latent", action="store_true",
                   help="latent-attention models keep the compressed latent per token instead of per-head K/V: far more "
                        "tokens in the pool, attention through tensor ops on eager steps (MSGL_MLA_LATENT)")
    p.add_argument("--baked-dir", default="",
                   help="directory of baked checkpoints: written on the first boot, streamed on later ones (MSGL_BAKED_DIR)")
    p.add_argument("--tp-overlap", action="store_true",
                   help="MoE prefill steps under tensor parallelism reduce row chunks on a second stream (MSGL_TP_OVERLAP)")
    p.add_argument("--print-env", action="store_true", help="list every MSGL_* variable and exit")
    return p


def parse_args(argv: Optional[List[str]] = None) -> ServerArgs:
    import sys

    if "--print-env" in (argv if argv is not None else sys.argv[1:]):   # needs no model
        from ..env import ENV

        print(ENV.describe())
        raise SystemExit(0)
    ns = build_parser().parse_args(argv)
    import os

    for flag, var, value in ((ns.swa_pool, "MSGL_SWA_POOL", "1"), (ns.baked_dir, "MSGL_BAKED_DIR", ns.baked_dir),
                             (ns.tp_overlap, "MSGL_TP_OVERLAP", "1"), (ns.mla_latent, "MSGL_MLA_LATENT", "1")):
        if flag:
            os.environ[var] = value
    from ..utils.hub import resolve_model_path

    ns.model_path = resolve_model_path(ns.model_path)
    ns.spec_draft_model_path = resolve_model_path(ns.spec_draft_model_path)
    if ns.enable_ep and ns.tp_size * ns.dp_size == 1:
        raise SystemExit("--enable-ep needs --tp-size > 1 or --dp-size > 1")
    kwargs = json.loads(ns.chat_template_kwargs) if ns.chat_template_kwargs else None
    chat_template = ns.chat_template
    if chat_template and chat_template.endswith((".jinja", ".j2", ".txt")):
        with open(chat_template) as fh:
            chat_template = fh.read()
    max_running = ns.max_running_req
    if ns.cuda_graph_max_bs is not None and ns.cuda_graph_max_bs > 0:
        # a graph cap lowers the running-request cap (python/minisgl/server/args.py:535-537)
        max_running = min(max_running, max(ns.cuda_graph_max_bs, 1))
    return ServerArgs(
        model_path=ns.model_path, dtype=ns.dtype, tp_size=ns.tp_size, dp_size=ns.dp_size, enable_ep=ns.enable_ep,
        max_running_req=max_running, max_seq_len_override=ns.max_seq_len_override,
        distributed_timeout=ns.distributed_timeout, memory_ratio=ns.memory_ratio,
        use_dummy_weight=ns.use_dummy_weight, use_pynccl=ns.use_pynccl, cuda_graph_max_bs=ns.cuda_graph_max_bs,
        num_page_override=ns.num_page_override, page_size=ns.page_size, attention_backend=ns.attention_backend,
        moe_backend=ns.moe_backend, model_source=ns.model_source, cache_type=ns.cache_type,
        kv_cache_dtype=ns.kv_cache_dtype, quantization=ns.quantization, device=ns.device,
        spec_algorithm=ns.spec_algorithm, spec_draft_model_path=ns.spec_draft_model_path,
        spec_num_draft=ns.spec_num_draft, spec_ngram_max=ns.spec_ngram_max, spec_ngram_min=ns.spec_ngram_min,
        spec_tree_width=ns.spec_tree_width, weight_offload_gb=ns.weight_offload_gb, expert_cache_gb=ns.expert_cache_gb, expert_host_gb=ns.expert_host_gb,
        expert_disk_dir=ns.expert_disk_dir,
        max_extend_tokens=ns.max_extend_tokens, disable_overlap=ns.disable_overlap, host=ns.host, port=ns.port,
        served_model_name=ns.served_model_name, num_tokenizer=ns.num_tokenizer, shell_mode=ns.shell_mode,
        chat_template=chat_template, chat_template_kwargs=kwargs, reasoning_parser=ns.reasoning_parser,
        rsa=_rsa_defaults(ns), rsa_effort_ladder=ns.rsa_effort_ladder,
    )


def _rsa_defaults(ns):
    from ..rsa import RSAParams

    return RSAParams(n=ns.rsa_n, k=ns.rsa_k, t=ns.rsa_t, tail_tokens=ns.rsa_tail_tokens, max_tokens=ns.rsa_max_tokens,
                     agg_max_tokens=ns.rsa_agg_max_tokens, temperature=ns.rsa_temperature, top_p=ns.rsa_top_p,
                     selection=ns.rsa_selection, max_concurrency=ns.rsa_max_concurrency,
                     max_retries=ns.rsa_max_retries)
