"""Serving benchmark: output tokens per second of the named workload on N GPUs of one node.

Workload (the quantised dense configuration of the baseline description): a Qwen3-4B-shaped
decoder (36 layers, hidden 2560, 32 q / 8 kv heads of 128, QK-norm, SwiGLU 9728, vocab
151936, tied embeddings), MXFP4 weights run W4A8 with per-token e4m3 activations, e4m3 KV
cache, random-init weights (seed 1), tensor parallel over the N GPUs; 256 concurrent
requests of uniform-random token ids with lengths uniform in [512, 2048], 256 greedy output
tokens each. One *step* is one full pass of that workload through the public offline API
(``LLM.generate``); every pass draws fresh prompts, so the prefix cache never skips work.

Reported: ``value`` = output tokens / device time of the forward steps (CUDA events around
every engine step, max over ranks); ``e2e`` = output tokens / time of the whole
``generate`` call, which stages every step's index arrays and prompt ids from pinned host
memory and reads the sampled ids back each step.

Launch: ``python bench.py --gpus 1`` or, for N > 1,
``python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1
--master-port P bench.py --gpus N``.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BASELINE_TOK_S = None  # the reference publishes no B200 number for this configuration


# The named benchmark configurations (the workload shapes of the baseline description). The
# default, ``dense``, is the headline; the others are selected with ``--config``. Explicit flags
# override a preset's values.
PRESETS = {
    # Qwen3-4B-shaped dense decoder, MXFP4 W4A8 + fp8 KV, tensor parallel
    "dense": dict(model="qwen3-4b", quant="mxfp4", kv="fp8", requests=256, in_min=512, in_max=2048, out_len=256,
                  parallel="tp"),
    # Qwen3-30B-A3B-shaped MoE, block-scaled fp8 W8A8, attention data-parallel + expert-parallel
    # with the all-to-all exchange: every GPU is a replica holding E / N experts
    "moe-ep": dict(model="qwen3-30b-a3b", quant="fp8_block", kv="fp8", requests=512, in_min=256, in_max=1024,
                   out_len=256, parallel="dp-ep"),
    # Llama-3-70B-shaped dense decoder, fp8 W8A8 per channel + fp8 KV, tensor parallel; all requests
    # share a 2048-token random prefix followed by a unique 256-token suffix
    "prefix70b": dict(model="llama3-70b", quant="fp8", kv="fp8", requests=512, in_min=256, in_max=256, out_len=128,
                      shared_prefix=2048, parallel="tp"),
    # Qwen3-8B-shaped bf16 target with an EAGLE3-style one-layer draft head, draft length 4, greedy
    "spec": dict(model="qwen3-8b", quant="none", kv="bf16", requests=64, in_min=1024, in_max=1024, out_len=256,
                 spec="eagle3", spec_draft=4, spec_tree_width=4, parallel="tp"),
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="dense", choices=sorted(PRESETS))
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default=None)
    ap.add_argument("--quant", default=None)
    ap.add_argument("--kv", default=None)
    ap.add_argument("--requests", type=int, default=None)
    ap.add_argument("--in-min", type=int, default=None)
    ap.add_argument("--in-max", type=int, default=None)
    ap.add_argument("--out-len", type=int, default=None)
    ap.add_argument("--shared-prefix", type=int, default=None)
    ap.add_argument("--parallel", default=None, choices=["tp", "dp-ep"])
    ap.add_argument("--spec", default=None, choices=["none", "ngram", "eagle3", "mtp"])
    ap.add_argument("--spec-draft", type=int, default=None)
    ap.add_argument("--spec-tree-width", type=int, default=None)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--max-extend", type=int, default=8192)
    ap.add_argument("--memory-ratio", type=float, default=0.85)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--layers", type=int, default=0,
                    help="profiling only: cut the model to this many layers (the result line is marked reduced)")
    ap.add_argument("--no-matched", action="store_true",
                    help="skip the extra bf16-weights / bf16-KV run of this repository that is reported beside "
                         "the quantised number for a like-for-like ratio against the bf16 reference arm")
    args = ap.parse_args()
    preset = dict(shared_prefix=0, spec="none", spec_draft=4, spec_tree_width=1)
    preset.update(PRESETS[args.config])
    for key, val in preset.items():
        if getattr(args, key, None) is None:
            setattr(args, key, val)
    return args


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self) -> None:
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        clocks, reasons, mx = [], set(), None
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    clocks.append(float(parts[1]))
                    mx = float(parts[2])
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                     parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if clocks:
            # the median over samples taken under load (the upper half of the samples)
            clocks.sort()
            out["sm_mhz"] = statistics.median(clocks)
        out["sm_max_mhz"] = mx
        out["reasons"] = sorted(reasons)
        out["samples"] = len(clocks)
        return out


def _reference_attempt(args, backend: str, small: bool, timeout: float):
    """One run of ``baseline/reference_arm.py`` (the unmodified reference through its own
    ``minisgl.llm.LLM``) in a child process that sees the reference package only."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    cmd = [sys.executable, os.path.join(ROOT, "baseline", "reference_arm.py"), "--gpus", str(args.gpus),
           "--model", args.model, "--attention-backend", backend, "--page-size", str(args.page_size),
           "--max-extend", str(args.max_extend), "--memory-ratio", str(args.memory_ratio)]
    if small:
        cmd += ["--steps", "1", "--warmup", "1", "--requests", "8", "--in-min", "64", "--in-max", "128",
                "--out-len", "8"]
    else:
        cmd += ["--steps", str(args.steps), "--warmup", str(args.warmup), "--requests", str(args.requests),
                "--in-min", str(args.in_min), "--in-max", str(args.in_max), "--out-len", str(args.out_len)]
    env = dict(os.environ, PYTHONPATH=ref_dir, MINISGL_TAIL_HIP="0")
    env.pop("MSGL_BENCH_PROFILE", None)
    try:
        proc = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=timeout, cwd=tempfile.gettempdir())
    except subprocess.TimeoutExpired:
        return None, f"attention backend {backend}: no result within {int(timeout)} s"
    line = None
    for ln in proc.stdout.splitlines():
        if ln.startswith("{") and '"impl": "reference"' in ln:
            line = ln
    if proc.returncode == 0 and line is not None:
        return json.loads(line), None
    err = [ln for ln in proc.stderr.strip().splitlines() if ln.strip()]
    sys.stderr.write(f"[reference arm, backend {backend}] rc={proc.returncode}\n" + "\n".join(err[-25:]) + "\n")
    exc = [ln for ln in err if re.match(r"^[A-Za-z_.]+(Error|Exception|Exit)\b", ln)]
    return None, f"attention backend {backend}: rc={proc.returncode}: " + ((exc or err or ["no output"])[-1])[:400]


def run_reference(args) -> None:
    """The reference arm: the unmodified reference, installed under ``baseline/_ref``, through
    its own offline API (``baseline/reference_arm.py``), with the knobs the reference documents
    for a box without its gfx1201 HIP kernel packages (``MINISGL_TAIL_HIP=0``, torch sampler
    fallback, its own attention back-end selector). The reference has no W4A8 / fp8-KV path on
    NVIDIA GPUs, so this arm is bf16 and marks ``same_config: false``. Each back-end is first
    tried on a few short requests; the first that works runs the named workload."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "minisgl")):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "the reference is not installed under baseline/_ref"}))
        return
    if world > 1:
        # every rank runs its own child with the launcher's RANK / WORLD_SIZE / LOCAL_RANK
        result, why = _reference_attempt(args, os.environ.get("MSGL_REF_BACKEND", "fi"), False, 1500)
        if rank == 0:
            print(json.dumps(result if result is not None else {"impl": "reference", "unavailable": why}))
        return
    reasons = []
    t_start = time.time()
    for backend in ("auto", "fi"):
        probe, why = _reference_attempt(args, backend, True, 420)
        if probe is None:
            reasons.append(why)
            continue
        left = max(300.0, 1650.0 - (time.time() - t_start))
        result, why = _reference_attempt(args, backend, False, left)
        if result is not None:
            print(json.dumps(result))
            return
        reasons.append(why)
    print(json.dumps({"impl": "reference", "unavailable": "the unmodified reference (MINISGL_TAIL_HIP=0, bf16) did not "
                      "complete on this box: " + " | ".join(reasons)}))


def run_matched_bf16(args):
    """This repository on the reference arm's precision (bf16 weights, bf16 KV), same workload,
    in a child process before the main engine takes the device memory."""
    cmd = [sys.executable, os.path.abspath(__file__), "--gpus", "1", "--quant", "none", "--kv", "bf16",
           "--steps", "2", "--warmup", "3", "--no-matched", "--model", args.model,
           "--requests", str(args.requests), "--in-min", str(args.in_min), "--in-max", str(args.in_max),
           "--out-len", str(args.out_len), "--page-size", str(args.page_size), "--max-extend", str(args.max_extend),
           "--memory-ratio", str(args.memory_ratio)] + (["--no-graph"] if args.no_graph else [])
    try:
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
        for ln in proc.stdout.splitlines():
            if ln.startswith("{") and '"metric"' in ln:
                d = json.loads(ln)
                return {"tok_s": d["value"], "e2e_tok_s": d["e2e"]["value"], "dtype": "bf16 weights, bf16 KV",
                        "p50_tpot_ms": d["config"]["p50_tpot_ms"], "steps": d["steps"], "warmup": d["warmup"]}
        return {"error": (proc.stderr.strip().splitlines() or ["no result line"])[-1][:300]}
    except Exception as exc:  # the headline run does not depend on this one
        return {"error": repr(exc)[:300]}


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
        return

    matched = None
    if (args.gpus == 1 and args.quant != "none" and not args.no_matched and args.config == "dense"
            and not os.environ.get("MSGL_BENCH_PROFILE")):
        matched = run_matched_bf16(args)

    import numpy as np
    import torch
    import torch.distributed as dist

    from minisglang_rdna4_b200 import SamplingParams
    from minisglang_rdna4_b200.llm import LLM
    from minisglang_rdna4_b200.ops import cuda as K

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)

    model_config = None
    if args.layers > 0:
        import dataclasses

        from minisglang_rdna4_b200.models.config import NAMED_CONFIGS

        model_config = dataclasses.replace(NAMED_CONFIGS[args.model](), num_layers=args.layers)
    dp_ep = args.parallel == "dp-ep" and world > 1
    par = dict(dp_size=world, dp_rank=rank, enable_ep=True) if dp_ep else dict(tp_size=world, tp_rank=rank)
    spec = {}
    if args.spec != "none":
        spec = dict(spec_algorithm=args.spec, spec_num_draft=args.spec_draft, spec_tree_width=args.spec_tree_width)
    local_requests = -(-args.requests // world) if dp_ep else args.requests
    llm = LLM(
        model_path=args.model, model_config=model_config, use_dummy_weight=True,
        quantization=None if args.quant == "none" else args.quant,
        kv_cache_dtype=args.kv, page_size=args.page_size,
        max_running_req=local_requests, max_extend_tokens=args.max_extend, memory_ratio=args.memory_ratio,
        seed=1, cuda_graph_max_bs=(-1 if args.no_graph else None),
        max_seq_len_override=max(4096, args.shared_prefix + args.in_max + args.out_len + 16), **par, **spec,
    )
    eng = llm.engine
    vocab = eng.model_config.vocab_size
    sp = SamplingParams(temperature=0.0, max_tokens=args.out_len, ignore_eos=True)

    # per-step device timing: events around every engine forward
    step_events = []
    orig_forward = eng.forward_batch

    # MSGL_BENCH_PROFILE="first:count" brackets engine steps [first, first+count) of the LAST
    # timed pass with cudaProfilerStart/Stop (for `ncu --profile-from-start off`)
    prof = os.environ.get("MSGL_BENCH_PROFILE")
    prof_first, prof_count = (int(x) for x in prof.split(":")) if prof else (-1, 0)
    prof_state = {"armed": False}

    def timed_forward(batch, plan, sargs, return_logits=False):
        idx = len(step_events)
        if prof_state["armed"] and idx == prof_first:
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
        if prof_state["armed"] and idx == prof_first + prof_count:
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        stream = eng.stream
        s.record(stream)
        out = orig_forward(batch, plan, sargs, return_logits)
        e.record(stream)
        step_events.append((s, e, batch.phase, plan.num_tokens))
        return out

    eng.forward_batch = timed_forward
    runner = getattr(llm, "_spec_runner", None)
    if runner:
        # the speculative step runs on the device without passing through forward_batch: time it too
        orig_run = runner.run

        def timed_run(rows, staged):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(eng.stream)
            with torch.cuda.stream(eng.stream):
                out = orig_run(rows, staged)
            e.record(eng.stream)
            step_events.append((s, e, "decode", len(rows) * runner.W))
            return out

        runner.run = timed_run

    def make_prompts(seed: int):
        g = np.random.default_rng(seed)
        lens = g.integers(args.in_min, args.in_max + 1, size=args.requests)
        prefix = g.integers(0, vocab, size=args.shared_prefix, dtype=np.int32)
        prompts = [np.concatenate([prefix, g.integers(0, vocab, size=int(n), dtype=np.int32)]) for n in lens]
        # data-parallel replicas serve disjoint slices of the request set
        return prompts[rank::world] if dp_ep else prompts

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def one_pass(seed: int):
        prompts = make_prompts(seed)  # identical on every rank
        step_events.clear()
        t_first = {}
        t_last = {}
        orig_send = llm.send_result

        def send(replies):
            now = time.perf_counter()
            for r in replies:
                t_first.setdefault(r.uid, now)
                t_last[r.uid] = now
            orig_send(replies)

        llm.send_result = send
        h2d0, d2h0, l0 = eng.h2d_bytes, eng.d2h_bytes, K.LAUNCHES
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(eng.stream)
        t0 = time.perf_counter()
        outs = llm.generate(prompts, sp)
        ev1.record(eng.stream)
        barrier()
        llm.send_result = orig_send
        wall_ms = ev0.elapsed_time(ev1)
        dev_ms = sum(s.elapsed_time(e) for s, e, _, _ in step_events)
        prefill_ms = sum(s.elapsed_time(e) for s, e, ph, _ in step_events if ph == "prefill")
        n_out = sum(len(o.token_ids) for o in outs)
        assert n_out == len(prompts) * args.out_len, (n_out, len(prompts) * args.out_len)
        ttft = sorted((t_first[u] - t0) * 1e3 for u in t_first)
        tpot = sorted((t_last[u] - t_first[u]) * 1e3 / max(args.out_len - 1, 1) for u in t_first)
        n_steps = len(step_events)
        return dict(wall_ms=wall_ms, dev_ms=dev_ms, prefill_ms=prefill_ms, n_out=n_out, steps=n_steps,
                    h2d=(eng.h2d_bytes - h2d0) / max(n_steps, 1), d2h=(eng.d2h_bytes - d2h0) / max(n_steps, 1),
                    launches=K.LAUNCHES - l0, ttft_p50=ttft[len(ttft) // 2], tpot_p50=tpot[len(tpot) // 2],
                    in_tokens=sum(len(p) for p in prompts))

    for w in range(args.warmup):
        one_pass(1000 + w)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    results = []
    for i in range(args.steps):
        prof_state["armed"] = prof_first >= 0 and i == args.steps - 1
        results.append(one_pass(2000 + i))
    if prof_state["armed"]:
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    clocks = sampler.stop() if rank == 0 else {}

    def reduce_max(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    dev_ms = reduce_max(sum(r["dev_ms"] for r in results))
    wall_ms = reduce_max(sum(r["wall_ms"] for r in results))
    n_out = sum(r["n_out"] for r in results)
    if dp_ep:  # every replica produced its own share of the output tokens
        t = torch.tensor([float(n_out)], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        n_out = int(t.item())
    value = n_out / (dev_ms / 1e3)
    e2e = n_out / (wall_ms / 1e3)
    last = results[-1]
    if rank == 0:
        line = {
            "metric": "output tok/s (device-timed, max over ranks)",
            "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": (value / BASELINE_TOK_S) if BASELINE_TOK_S else None,
            "dtype": (f"w4a8-mxfp4+{args.kv}-kv" if args.quant == "mxfp4" else
                      ("bf16" if args.quant == "none" else f"{args.quant}+{args.kv}-kv")),
            "data": "synthetic (uniform-random token ids, random-init weights seed 1)",
            "impl": "ours",
            "config": {
                "model": f"{args.model}-shaped {'MoE' if eng.model_config.is_moe else 'dense'}, {args.quant}"
                         f"{' W4A8' if args.quant == 'mxfp4' else ''}, {args.kv} KV",
                "global_batch": args.requests, "seq_len": f"in U[{args.in_min},{args.in_max}], out {args.out_len}",
                "parallelism": (f"dp{world}+ep{world} (all-to-all over peer memory)" if dp_ep else f"tp{world}"),
                "preset": args.config, "shared_prefix": args.shared_prefix,
                "spec": ({"algorithm": args.spec, "draft": args.spec_draft, "tree_width_requested": args.spec_tree_width,
                          "tree_width_verified": (getattr(llm._spec_runner, "T", 1)
                                                  if getattr(llm, "_spec_runner", None) is not None
                                                  else args.spec_tree_width),
                          "verify_rows_per_request": (getattr(llm._spec_runner, "R", None)
                                                      if getattr(llm, "_spec_runner", None) is not None else None),
                          "verify_steps": llm.stats.get("spec_steps", 0),
                          "verify_step_ms_p50": (sorted(s.elapsed_time(e) for s, e, ph, _ in step_events
                                                        if ph == "decode") or [None])[len([1 for x in step_events if x[2] == "decode"]) // 2],
                          "accepted_tokens_per_request_step": (llm.stats.get("spec_accepted", 0)
                                                               / max(llm.stats.get("spec_drafted", 0), 1) * args.spec_draft),
                          "accepted_per_step": (llm.stats.get("spec_emitted", 0) / max(llm.stats.get("spec_steps", 0), 1))}
                         if args.spec != "none" else None),
                "step": "one full pass of the workload (prefill + decode)",
                "l2": "inputs larger than L2 (weights + KV pool >> 126 MB)",
                "p50_ttft_ms": last["ttft_p50"], "p50_tpot_ms": last["tpot_p50"],
                "prefill_ms_per_pass": last["prefill_ms"], "engine_steps_per_pass": last["steps"],
                "prompt_tokens_per_pass": last["in_tokens"], "cuda_graphs": not args.no_graph,
                "matched_bf16": matched,
                **({"reduced_layers": args.layers, "valid": False} if args.layers > 0 else {}),
            },
            "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": last["h2d"],
                    "d2h_bytes_per_step": last["d2h"], "ms_per_pass": wall_ms / args.steps},
            "gpu_launches": sum(r["launches"] for r in results),
            "clocks": clocks,
        }
        print(json.dumps(line))
    sys.stdout.flush()
    llm.shutdown()
    if world == 1:
        return  # normal interpreter exit
    # Multi-rank: every rank has passed the shutdown barrier. Run the exit handlers now, then leave
    # without the interpreter's module teardown: destroying NCCL communicators that captured graphs
    # still reference has been seen to block one rank forever, which would stall the launcher.
    sys.stderr.flush()
    import atexit
    try:
        atexit._run_exitfuncs()
    finally:
        os._exit(0)


if __name__ == "__main__":
    main()
