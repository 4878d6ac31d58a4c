#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Llama 3.2 1B sizes with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl ours|reference]
                    [--sizes 1b|3b|8b] [--prompt-len P] [--gen-len G] [--context C] [--all-configs]

A "step" is one decode step of `--batch` requests, each with a 2,048-token prompt already in the
cache. `value` is decoded tokens per second timed on the device: the steps are planned ahead, and
the timed loop only uploads each step's metadata and replays the step's CUDA graph (no scheduler,
no reads; CUDA events around exactly K steps; the median of several such regions, since one region
of K steps may last only milliseconds). `e2e` is the same through the Python entry point
(`LLM.add_request` / `LLM.step`), host tokens in and out. The same line carries the 2,048-token
prefill, the decode step's HBM roofline, decode at batch 1 and 64, and a record of the run (GPU,
driver, CUDA, commit). Prints ONE JSON line. One GPU only.

The defaults are the benchmark's configuration (Llama 3.2 1B sizes, batch 8, 2,048-token prompts,
256 generated); --sizes / --prompt-len / --gen-len / --context run the same measurements at other
layer sizes and context lengths. --all-configs adds, as further `points` of the same line, each
with its own roofline fraction: a serving run of 64 mixed requests at Llama 3.2 3B sizes, decode at
batch 64 with 8,192-token contexts at Llama 3.1 8B sizes, and one 32,768-token prompt prefilled
through the scheduler in portions of 2,048 at 8B sizes.

Other modes (measurement aids; each prints lines of its own, not the benchmark's line):
    --serve N          N requests of mixed lengths handed to LLM.generate at once
    --kernel NAME ...  one kernel on synthetic operands larger than L2, for profilers
    --timeline         per-kernel start / ready times of one decode step (needs VOB_TIMELINE=1)
"""
from __future__ import annotations

import argparse
import hashlib
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode tok/s at batch 1/8/64; prefill tok/s at 2,048 tokens (Llama 3.2 1B)"
PROMPT_LEN = 2048
GEN_LEN = 256
MIN_TIMED_SECONDS = 0.25       # a timed region of K steps is repeated until so much time has been measured ...
MAX_TIMED_STEPS = 320          # ... or so many steps have run (contexts grow by one token per step)
# Layer sizes of the three Llama models the reference's plan names (config.json values).
SIZES = {
    "1b": dict(name="llama-3.2-1b-sizes", layers=16, hidden=2048, heads=32, head_dim=64, inter=8192, rope_factor=32.0, tied=True),
    "3b": dict(name="llama-3.2-3b-sizes", layers=28, hidden=3072, heads=24, head_dim=128, inter=8192, rope_factor=32.0, tied=True),
    "8b": dict(name="llama-3.1-8b-sizes", layers=32, hidden=4096, heads=32, head_dim=128, inter=14336, rope_factor=8.0, tied=False),
}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    try:
        with open(p) as f:
            d = json.load(f)
        if "hbm_gbs" in d:
            peaks["hbm_gbs"] = float(d["hbm_gbs"])
        if "bf16_tflops" in d:
            peaks["bf16_tflops"] = float(d["bf16_tflops"])
        peaks["source"] = "measured"
    except (OSError, ValueError):
        pass
    return peaks


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed regions run."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        threading.Thread(target=self._read, daemon=True).start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
        sm = sorted(int(s[0]) for s in self.samples if s[0].isdigit())
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples)}


def run_record():
    """GPU, driver, CUDA, torch and the commit of the code that ran (the reference records these with
    every measurement, CLAUDE.md:96). A copy of the repository without its .git folder has no commit
    to name: it is identified by a hash over its source files instead."""
    import torch
    rec = {"gpu": torch.cuda.get_device_name(0), "cuda": torch.version.cuda, "torch": torch.__version__}
    try:
        out = subprocess.run(["nvidia-smi", "-i", "0", "--query-gpu=driver_version", "--format=csv,noheader"],
                             capture_output=True, text=True, timeout=20)
        rec["driver"] = out.stdout.strip().splitlines()[0] if out.returncode == 0 and out.stdout.strip() else None
    except (OSError, subprocess.SubprocessError):
        rec["driver"] = None
    try:
        out = subprocess.run(["git", "-C", ROOT, "rev-parse", "HEAD"], capture_output=True, text=True, timeout=20)
        rec["commit"] = out.stdout.strip() if out.returncode == 0 else None
    except (OSError, subprocess.SubprocessError):
        rec["commit"] = None
    h = hashlib.sha256()
    pkg = os.path.join(ROOT, "vllm_oxide_b200")
    for base, dirs, files in sorted(os.walk(pkg)):
        dirs[:] = sorted(d for d in dirs if d not in ("_build", "__pycache__"))
        for f in sorted(files):
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                h.update(os.path.relpath(os.path.join(base, f), pkg).encode())
                with open(os.path.join(base, f), "rb") as fh:
                    h.update(fh.read())
    with open(os.path.abspath(__file__), "rb") as fh:
        h.update(fh.read())
    rec["source_sha256"] = h.hexdigest()[:16]
    return rec


def reference_arm():
    # The reference is a Rust workspace (Cargo.toml, crates/engine) with no Python packaging and
    # no GPU code; neither pip nor cargo can build it on this machine.
    print(json.dumps({"impl": "reference", "unavailable":
                      "the reference is a CPU-only Rust workspace (no setup.py/pyproject, no cargo/rustc here); "
                      "pip install of its source tree fails and it has no GPU path to run"}))
    return 0


# ------------------------------------------------------------------------------------------------ engines
def make_config(sz, layers):
    from vllm_oxide_b200.config import LlamaConfig, RopeScaling
    return LlamaConfig(hidden_size=sz["hidden"], intermediate_size=sz["inter"], num_hidden_layers=layers,
                       num_attention_heads=sz["heads"], num_key_value_heads=8, head_dim=sz["head_dim"], vocab_size=128256,
                       max_position_embeddings=131072, rms_norm_eps=1e-5, rope_theta=500000.0,
                       rope_scaling=RopeScaling(sz["rope_factor"], 1.0, 4.0, 8192), tie_word_embeddings=sz["tied"],
                       bos_token_id=128000, eos_token_ids=(128001,))


ENGINE_OVERRIDES = {}          # EngineConfig fields set from the command line (experiments)


def make_engine(sz, layers, max_seqs, tokens_per_request, context, graphs=True):
    """(config, LLM) with random weights made on the device and a pool for `max_seqs` requests of
    `tokens_per_request` tokens."""
    import torch
    from vllm_oxide_b200 import models
    from vllm_oxide_b200.config import EngineConfig
    from vllm_oxide_b200.engine import LLM, ModelRunner
    from vllm_oxide_b200.weights import random_tensors
    cfg = make_config(sz, layers)
    pages_per_req = -(-(tokens_per_request + 16) // 16)
    fields = dict(max_batch_tokens=2048, max_seqs=max_seqs, max_model_len=context, block_size=16,
                  num_pages=max_seqs * pages_per_req + 8, dtype="bfloat16", cuda_graphs=graphs)
    fields.update(ENGINE_OVERRIDES)         # --engine FIELD=VALUE replaces what the benchmark would set
    engine = EngineConfig(**fields)
    tensors = random_tensors(models.llama_manifest(cfg), seed=0, std=0.02, dtype=torch.bfloat16, device="cuda:0")
    runner = ModelRunner(cfg, tensors, engine)
    del tensors
    return cfg, LLM(runner)


def model_flops(cfg, layers):
    """(flops per token of the products of all layers, attention flops per (query, key) pair of all layers)."""
    lin = layers * (cfg.hidden_size * (cfg.q_dim + 2 * cfg.kv_dim) + cfg.q_dim * cfg.hidden_size
                    + 3 * cfg.hidden_size * cfg.intermediate_size)
    return 2.0 * lin, layers * 4.0 * cfg.q_dim


def never_stop(n):
    from vllm_oxide_b200.sampling import SamplingParams
    return SamplingParams(max_new_tokens=n, temperature=0.0, stop_token_ids=())


def prefill_all(llm, ids, prompt_len):
    """Step until every request has its first token (none may finish on the way)."""
    for _ in range(2 * (len(ids) * prompt_len // 2048 + len(ids)) + 32):
        if all(llm._generated.get(r, 0) >= 1 for r in ids):
            return
        llm.step()
    raise RuntimeError("bench: the prompts did not finish prefilling")


def median(xs):
    xs = sorted(xs)
    return xs[len(xs) // 2]


def decode_device(llm, prompts, B, steps, warmup, prompt_len, gen_len):
    """B requests with their prompts in the cache. The decode steps to come are planned first
    (metadata built, placeholders booked); the timed loop then only uploads a step's metadata and
    replays its graph, the step's input tokens being the previous step's picks on the device.
    Returns (median ms per step over the regions of exactly `steps` steps, mean context length,
    kernel launches per region, regions timed)."""
    import torch
    from vllm_oxide_b200 import kernels
    r, sched = llm.runner, llm.scheduler
    ids = [llm.add_request(prompts[i], never_stop(gen_len)) for i in range(B)]
    prefill_all(llm, ids, prompt_len)
    for _ in range(warmup):
        llm.step()
    llm.drain()
    max_regions = max(1, MAX_TIMED_STEPS // steps)
    planned = []
    for _ in range(max_regions * steps):
        plan = sched.schedule()
        if not plan.decode_only or plan.preempted or plan.admitted:
            raise RuntimeError("bench: the scheduler planned something else than a decode step")
        planned.append((plan, r.decode_arrays(sched, plan)))
        sched.advance(plan)
    ctx0 = sum(r.manager.length(i) for i in ids) - len(planned) * B        # before the first planned step
    ev = lambda: torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    times, launches, measured = [], 0, 0.0
    for region in range(max_regions):
        n0 = kernels.launch_count()
        e0, e1 = ev(), ev()
        e0.record()
        for i, (plan, arrays) in enumerate(planned[region * steps:(region + 1) * steps]):
            # alternating result and metadata buffers, as the engine's loop does when it runs ahead
            r.decode_step_graph(None, plan, feed_from_device=True, read=False, parity=i & 1, arrays=arrays)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / steps)
        launches = kernels.launch_count() - n0
        measured += times[-1] * steps / 1e3
        if measured >= MIN_TIMED_SECONDS:
            break
    mean_ctx = ctx0 / B + (len(times) * steps + 1) / 2.0
    r.check_kernels()
    for i in ids:
        llm.abort(i)
    return median(times), mean_ctx * B, launches, len(times)


def decode_e2e(llm, prompts, B, steps, warmup, prompt_len, gen_len):
    """The same through `LLM.step()`: host tokens in (metadata upload), picked tokens out (D2H read).
    Wall clock around regions of exactly `steps` steps; the median region."""
    import torch
    ids = [llm.add_request(prompts[i], never_stop(gen_len)) for i in range(B)]
    prefill_all(llm, ids, prompt_len)
    for _ in range(warmup):
        llm.step()
    rates, measured = [], 0.0
    for _ in range(max(1, MAX_TIMED_STEPS // steps)):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            llm.step()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        rates.append(B * steps / dt)
        measured += dt
        if measured >= MIN_TIMED_SECONDS:
            break
    for i in ids:
        llm.abort(i)
    return median(rates)


def timed_prefill(llm, tokens, n):
    """One step of the first `n` tokens (at most 2,048) of a prompt, events around the step; median of 5 after 3."""
    import torch
    runner, rt = llm.runner, llm.runner.rt

    def once(rid):
        runner.admit(rid)
        runner.manager.reserve(rid, n)
        arrays = runner.build_arrays([rt.StepEntry(rid, tokens[:n], [n - 1])])
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.step(arrays)
        e1.record()
        torch.cuda.synchronize()
        runner.manager.release(rid)
        return e0.elapsed_time(e1)
    for i in range(3):
        once(900000 + i)
    return median([once(900100 + i) for i in range(5)])


def prefill_through_scheduler(llm, tokens):
    """Seconds from handing a prompt to the engine to its first token, the prompt cut into portions
    by the scheduler (the reference's prefill time, crates/engine/examples/generate.rs:5-6,43-52)."""
    import torch
    rid = llm.add_request(tokens, never_stop(2))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    steps = 0
    while llm._generated.get(rid, 0) < 1:
        llm.step()
        steps += 1
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    llm.abort(rid)
    return dt, steps


def serve_measure(llm, cfg, layers, n_requests, len_min, len_max, gen_len, peaks):
    """Many requests of different lengths at once through the public entry point: the scheduler
    cuts prompts into portions under the token budget and mixes them with the decoding of the
    requests that are through. Wall-clock time of generate(), host token ids in and out. The
    roofline of such a run is the sum over its steps of the larger of (the step's flops / the
    tensor peak) and (the bytes the step must read / the HBM peak)."""
    import torch
    g = torch.Generator().manual_seed(7)
    lens = torch.randint(len_min, len_max + 1, (n_requests,), generator=g).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    params = never_stop(gen_len)
    for _ in range(2):                  # warm-up: the same run twice (library handles; a step's shape class is
        llm.generate(prompts, params)   # recorded as a CUDA graph when it comes the second time)
    torch.cuda.synchronize()
    runner = llm.runner
    lin_flops, attn_flops = model_flops(cfg, layers)
    head_flops = 2.0 * cfg.vocab_size * cfg.hidden_size
    ideal = [0.0]
    upload = runner.upload

    def logging_upload(arrays, *args, **kwargs):
        flops = lin_flops * arrays.rows + head_flops * arrays.logit_count
        keys = 0
        for rid, n in zip(arrays.ids, arrays.new_counts):
            ctx = runner.manager.length(rid)
            flops += attn_flops * n * (ctx + (n + 1) / 2.0)
            keys += ctx + n
        nbytes = runner.step_read_bytes(keys)
        ideal[0] += max(flops / (peaks["bf16_tflops"] * 1e12), nbytes / (peaks["hbm_gbs"] * 1e9))
        return upload(arrays, *args, **kwargs)
    runner.upload = logging_upload
    steps0, pre0 = runner.steps_run, llm.stats.get("preemptions", 0)
    t0 = time.perf_counter()
    outs = llm.generate(prompts, params)
    torch.cuda.synchronize()
    secs = time.perf_counter() - t0
    runner.upload = upload
    generated = sum(len(o.token_ids) for o in outs)
    return {"value": generated / secs, "unit": "generated tok/s", "total_tok_s": (sum(lens) + generated) / secs, "seconds": secs,
            "requests": n_requests, "prompt_tokens": sum(lens), "generated": generated, "engine_steps": runner.steps_run - steps0,
            "preemptions": llm.stats.get("preemptions", 0) - pre0,
            "roofline": {"bound": "per step: tensor or hbm", "ideal_seconds": ideal[0], "frac": ideal[0] / secs, "of": peaks["source"]}}


def free_engine(llm):
    import gc
    import torch
    llm.runner._graphs.clear()
    llm.runner._step_graphs.clear()
    del llm
    gc.collect()
    torch.cuda.empty_cache()


def all_config_points(peaks, steps, warmup):
    """The other rows of the reference's plan, each measured with all layers of its model."""
    import torch
    points = {}
    # Llama 3.2 3B sizes: 64 mixed requests, prompts uniform in [128, 4096], 256 new tokens each
    sz = SIZES["3b"]
    cfg, llm = make_engine(sz, sz["layers"], 64, 4096 + 256, 8192)
    points["serve64_3b"] = serve_measure(llm, cfg, sz["layers"], 64, 128, 4096, 256, peaks)
    free_engine(llm)
    # Llama 3.1 8B sizes: decode at batch 64 with 8,192-token contexts from the paged cache
    sz = SIZES["8b"]
    k = min(steps, 32)
    gen = 64 * 8192 // 2048 + warmup + MAX_TIMED_STEPS + 32
    cfg, llm = make_engine(sz, sz["layers"], 64, 8192 + gen, 16384)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (8192,), generator=g).tolist() for _ in range(64)]
    ms, ctx_sum, _, regions = decode_device(llm, prompts, 64, k, warmup, 8192, gen)
    nbytes = llm.runner.step_read_bytes(ctx_sum)
    gbs = nbytes / (ms / 1e3) / 1e9
    points["decode_b64_ctx8192_8b"] = {"value": 64 / (ms / 1e3), "unit": "tok/s", "ms_per_step": ms, "steps": k, "regions": regions,
                                       "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                                    "frac": gbs / peaks["hbm_gbs"], "of": peaks["source"]}}
    free_engine(llm)
    # Llama 3.1 8B sizes: one 32,768-token prompt through the scheduler (16 portions of 2,048 over a growing cache)
    cfg, llm = make_engine(sz, sz["layers"], 2, 32768 + 64, 40960)
    tokens = torch.randint(0, cfg.vocab_size, (32768,), generator=g).tolist()
    prefill_through_scheduler(llm, tokens)                       # twice untimed: the portions' shape classes are recorded
    prefill_through_scheduler(llm, tokens)
    secs, nsteps = min(prefill_through_scheduler(llm, tokens) for _ in range(2))
    lin_flops, attn_flops = model_flops(cfg, sz["layers"])
    flops = lin_flops * 32768 + attn_flops * 32768 * (32768 + 1) / 2.0 + 2.0 * cfg.vocab_size * cfg.hidden_size
    points["prefill_32768_8b"] = {"value": 32768 / secs, "unit": "tok/s", "seconds": secs, "engine_steps": nsteps, "tflop": flops / 1e12,
                                  "roofline": {"bound": "tensor", "achieved": flops / secs / 1e12, "peak": peaks["bf16_tflops"],
                                               "unit": "TFLOP/s", "frac": flops / secs / (peaks["bf16_tflops"] * 1e12),
                                               "of": peaks["source"]}}
    free_engine(llm)
    return points


# ------------------------------------------------------------------------------------------------ measurement aids
def kernel_case(argv):
    """Single kernels on synthetic operands, for profilers:
        python bench.py --kernel gemm --rows 8 --out 16384 --in 2048 [--copies 6] [--iters 3]
        python bench.py --kernel gemm_pair --rows 2048 --out 16384 --in 2048      (the two-SM product)
        python bench.py --kernel gemm_pair_swiglu --rows 2048 --out 16384 --in 2048
        python bench.py --kernel attn_decode --batch 8 --context 2200
        python bench.py --kernel attn_prefill --tokens 2048 [--impl-attn sm100|mma]
    Each launch works on operands of its own (several copies, together larger than L2), so that DRAM
    counters mean something; device time per launch is printed from CUDA events."""
    import torch
    from vllm_oxide_b200 import kernels
    from vllm_oxide_b200.tuning import TUNING
    ap = argparse.ArgumentParser(prog="bench.py --kernel")
    ap.add_argument("--kernel", required=True, choices=["gemm", "gemm_pair", "gemm_pair_swiglu", "gemm_library", "gemm_fused",
                                                         "attn_decode", "attn_prefill"])
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--out", type=int, default=16384)
    ap.add_argument("--in", dest="inner", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2200)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--page", type=int, default=16)
    ap.add_argument("--copies", type=int, default=6)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--graph", action="store_true", help="time the launches back to back, replayed from one CUDA graph")
    ap.add_argument("--merge", default="auto", choices=["auto", "cluster", "global"],
                    help="attn_decode: how the blocks of a request merge (auto: the engine's choice)")
    ap.add_argument("--impl-attn", default="sm100", choices=["sm100", "mma"], help="attn_prefill: the tcgen05 or the mma.sync kernel")
    ap.add_argument("--epilogue", default="store", choices=["store", "swiglu", "resid"], help="gemm_fused: the epilogue")
    ap.add_argument("--splits", type=int, default=None, help="attn_decode: blocks per request and kv head; gemm_fused: blocks that share K (default: the engine's choice)")
    a = ap.parse_args(argv)
    dev = "cuda:0"
    bf = torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s: torch.randn(*s, generator=g, device=dev).to(bf)
    if a.kernel.startswith("gemm"):
        x = rnd(a.rows, a.inner)
        ws = [rnd(a.out, a.inner) for _ in range(a.copies)]
        if a.kernel == "gemm_pair_swiglu":          # --out counts the rows of [Wg; Wu]
            out = torch.empty(a.rows, a.out // 2, dtype=bf, device=dev)
            launches = [lambda w=w: kernels.gemm_pair_swiglu(x, w, out) for w in ws]
        elif a.kernel == "gemm_fused":
            fused = kernels.gemm_fused
            if a.epilogue == "swiglu":
                out = torch.empty(a.rows, a.out // 2, dtype=bf, device=dev)
                launches = [lambda w=w: fused(x, w, out, kernels.EPI_SWIGLU, a.out // 2, splits=a.splits) for w in ws]
            elif a.epilogue == "resid":
                out = torch.empty(a.rows, a.out, dtype=bf, device=dev)
                resid = torch.zeros(a.rows, a.out, dtype=torch.float32, device=dev)
                nw = torch.ones(a.out, dtype=torch.float32, device=dev)
                ssq = torch.zeros(-(-a.out // 128), 64, dtype=torch.float32, device=dev)
                ssq = torch.zeros(-(-a.out // 128), 64, dtype=torch.float32, device=dev)
                launches = [lambda w=w: fused(x, w, None, kernels.EPI_RESID, a.out, resid=(resid, nw, out, ssq), splits=a.splits) for w in ws]
            else:
                out = torch.empty(a.rows, a.out, dtype=bf, device=dev)
                launches = [lambda w=w: fused(x, w, out, kernels.EPI_STORE, a.out, splits=a.splits) for w in ws]
        else:
            out = torch.empty(a.rows, a.out, dtype=bf, device=dev)
            if a.kernel == "gemm_library":           # the library product the engine uses for many rows, for comparison
                launches = [lambda w=w: torch.mm(x, w.t(), out=out) for w in ws]
            else:
                fn = kernels.gemm_sm100 if a.kernel == "gemm" else kernels.gemm_sm100_pair
                launches = [lambda w=w: fn(x, w, out) for w in ws]
        nbytes = a.out * a.inner * 2 + a.rows * a.inner * 2 + out.numel() * 2
        flops = 2.0 * a.rows * a.out * a.inner
    else:
        H, KV, hd, page = a.heads, a.kv_heads, a.head_dim, a.page
        if a.kernel == "attn_decode":
            S, ctx, new = a.batch, a.context, 1
        else:
            S, ctx, new = 1, 0, a.tokens
        L = ctx + new
        pages_per = -(-L // page)
        caches = [(rnd(S * pages_per, KV, page, hd), rnd(S * pages_per, KV, page, hd)) for _ in range(a.copies)]
        bt = torch.arange(S * pages_per, dtype=torch.int32, device=dev).view(S, pages_per).contiguous()
        q = rnd(S * new, H * hd)
        out = torch.empty_like(q)
        scale = 1.0 / math.sqrt(hd)
        if a.kernel == "attn_decode":
            pos = torch.full((S,), L - 1, dtype=torch.int32, device=dev)
            # auto: the engine's choice (parts/attention.py decode_split_rule): a cluster of up to 8 blocks per
            # request and kv head, or, for few requests with long contexts, up to 64 that merge through global memory
            from vllm_oxide_b200.parts.attention import decode_split_rule
            sms = torch.cuda.get_device_properties(dev).multi_processor_count
            if a.merge == "auto":
                splits, wide = decode_split_rule(S, KV, sms, ctx > TUNING.long_context_keys)
            else:
                wide = a.merge == "global" and 3 * sms // (S * KV) >= 4
                splits = max(1, min(64, 3 * sms // (S * KV))) if wide else max(1, min(8, -(-2 * sms // (S * KV))))
            if a.splits:
                splits = a.splits
            partials = torch.empty(kernels.attn_decode_partial_floats(S, KV, hd, splits), device=dev) if wide else None
            arrived = torch.zeros(S * KV, dtype=torch.int32, device=dev) if wide else None
            launches = [lambda kc=kc, vc=vc: kernels.attn_decode_mma(q, out, kc, vc, bt, pos, H, KV, hd, scale, 0, splits,
                                                                     partials, arrived)
                        for kc, vc in caches]
            nbytes = 2 * S * L * KV * hd * 2
            flops = 4.0 * S * H * hd * L
        else:
            starts = torch.tensor([0, new], dtype=torch.int32, device=dev)
            ctxs = torch.zeros(1, dtype=torch.int32, device=dev)
            if a.impl_attn == "sm100":
                launches = [lambda kc=kc, vc=vc: kernels.attn_prefill_sm100(q, out, kc, vc, bt, starts, ctxs, 1, new, H, KV, hd, scale)
                            for kc, vc in caches]
            else:
                launches = [lambda kc=kc, vc=vc: kernels.attn_prefill_mma(q, out, kc, vc, bt, starts, ctxs, 1, new, H, KV, hd, scale, 0)
                            for kc, vc in caches]
            nbytes = 2 * L * KV * hd * 2 + 2 * new * H * hd * 2
            flops = 4.0 * H * hd * new * (new + 1) / 2
    for f in launches:
        f()
    torch.cuda.synchronize()
    kernels.gemm_sm100_check()
    if a.graph:
        kernels.set_pdl(True)
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for _ in range(2):
                for f in launches:
                    f()
        gr.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(max(a.iters, 3)):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            gr.replay()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) * 1e3 / (2 * len(launches)))
        us = median(times)
        print(f"{a.kernel}: {us:.1f} us per launch (events around a CUDA graph of {2 * len(launches)} launches back to back); "
              f"{nbytes / us / 1e3:.0f} GB/s of the bytes it must read; {flops / us / 1e6:.1f} TFLOP/s")
        return 0
    times = []
    for _ in range(a.iters):
        for f in launches:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            f()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) * 1e3)
    us = median(times)
    print(f"{a.kernel}: {us:.1f} us per launch (events, single launches); {nbytes / us / 1e3:.0f} GB/s of the bytes it must read; "
          f"{flops / us / 1e6:.1f} TFLOP/s")
    return 0


KERNEL_TAGS = {1: "embed", 2: "add_rmsnorm", 4: "rope_kv_write", 5: "swiglu", 6: "paged_attention", 7: "attn_prefill_mma",
               8: "attn_decode_mma", 9: "pick_partial", 10: "pick_final", 11: "gemm_f32", 12: "gemm_sm100", 13: "gemm_sm100_persistent",
               14: "attn_prefill_sm100", 15: "gemm_sm100_pair"}


def timeline_of_a_decode_step(llm, prompts, B, prompt_len, gen_len):
    """With kernel libraries built with VOB_TIMELINE=1 in the environment (a different build: block 0
    of every kernel notes the global timer when it starts and when its wait for the kernel in front
    returns): the kernels of one decode step in order, with the time from each kernel's ready point
    to the next one's. Without that build nothing is recorded."""
    import collections
    import ctypes
    import torch
    from vllm_oxide_b200.csrc.build import _loaded
    ids = [llm.add_request(prompts[i], never_stop(gen_len)) for i in range(B)]
    prefill_all(llm, ids, prompt_len)
    for _ in range(6):
        llm.step()
    llm.drain()
    buf = torch.zeros(1 + 3 * 4096, dtype=torch.int64, device="cuda:0")

    def set_buffer(t):
        for name, lib in list(_loaded.items()):
            f = getattr(lib, f"vob_set_timeline_{name}", None)
            if f is not None:
                f.argtypes, f.restype = [ctypes.c_void_p], ctypes.c_int
                f(ctypes.c_void_p(t.data_ptr() if t is not None else 0))
    set_buffer(buf)
    torch.cuda.synchronize()
    llm.step()
    llm.drain()
    torch.cuda.synchronize()
    set_buffer(None)
    h = buf.cpu().tolist()
    n = min(h[0], 4096)
    rows = sorted(((KERNEL_TAGS.get(h[1 + 3 * e], str(h[1 + 3 * e])), h[2 + 3 * e], h[3 + 3 * e]) for e in range(n)), key=lambda x: x[2])
    if not rows:
        print("timeline: nothing recorded (build the kernel libraries with VOB_TIMELINE=1 in the environment)")
        return 1
    t0 = rows[0][1]
    print(f"{len(rows)} kernels; step span {(rows[-1][2] - t0) / 1000:.1f} us (batch {B})")
    agg = collections.OrderedDict()
    for i, (name, st, rd) in enumerate(rows):
        dur = (rows[i + 1][2] - rd) if i + 1 < len(rows) else 0
        c, d, lead = agg.get(name, (0, 0, 0))
        agg[name] = (c + 1, d + dur, lead + rd - st)
    for name, (c, d, lead) in agg.items():
        print(f"{name:22s} n={c:3d} time to next ready {d / 1000:8.1f} us (avg {d / c / 1000:6.2f})   avg waited at its wait {lead / c / 1000:6.2f} us")
    layers = llm.runner.config.num_hidden_layers
    per = max(1, (len(rows) - 4) // layers)
    mid = layers // 2
    print(f"layer {mid} in detail:")
    for i in range(1 + mid * per, min(len(rows) - 1, 1 + (mid + 1) * per + 1)):
        name, st, rd = rows[i]
        print(f"  {name:18s} start {(st - t0) / 1000:8.2f}  ready {(rd - t0) / 1000:8.2f}  (waited {(rd - st) / 1000:5.2f})"
              f"  -> next ready in {(rows[i + 1][2] - rd) / 1000:5.2f} us")
    for i in ids:
        llm.abort(i)
    return 0


# ------------------------------------------------------------------------------------------------ main
def main():
    if "--kernel" in sys.argv[1:]:
        return kernel_case(sys.argv[1:])
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--sizes", default="1b", choices=sorted(SIZES), help="layer sizes (Llama 3.2 1B / 3.2 3B / 3.1 8B)")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN)
    ap.add_argument("--gen-len", type=int, default=GEN_LEN)
    ap.add_argument("--context", type=int, default=8192, help="max_model_len of the engine")
    ap.add_argument("--all-configs", action="store_true",
                    help="add to `points`: the 3B serving run, 8B decode at batch 64 with 8,192-token contexts, "
                         "one 32,768-token prefill at 8B sizes (some minutes more, all layers, 90 GB on the device)")
    ap.add_argument("--serve", type=int, default=0, metavar="N",
                    help="instead of the step measurements: N requests with prompts of seeded uniform lengths in "
                         "[--serve-min, --serve-max], --gen-len tokens each, all handed to LLM.generate at once "
                         "(chunked prefill mixed with decoding); prints one line with total tokens a second")
    ap.add_argument("--serve-min", type=int, default=128)
    ap.add_argument("--serve-max", type=int, default=4096)
    ap.add_argument("--timeline", action="store_true", help="per-kernel times of one decode step (VOB_TIMELINE=1 build)")
    ap.add_argument("--tuning", action="append", default=[], metavar="FIELD=VALUE",
                    help="set a field of vllm_oxide_b200.tuning.TUNING (experiments)")
    ap.add_argument("--fold-rows", type=int, default=None, metavar="R",
                    help="an experiment: steps of up to R rows (at most 64) take the fused few-row kernels instead of the "
                         "engine's own switch-over point")
    ap.add_argument("--engine", action="append", default=[], metavar="FIELD=VALUE",
                    help="an experiment: set an EngineConfig field (booleans as 0 / 1), e.g. --engine pick_in_head=0")
    a = ap.parse_args()
    for kv in a.engine:
        k, _, v = kv.partition("=")
        ENGINE_OVERRIDES[k] = bool(int(v)) if v in ("0", "1") else int(v)
    if a.impl == "reference":
        return reference_arm()
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    a.warmup = max(a.warmup, 3)
    a.steps = max(a.steps, 1)
    prompt_len, gen_len = a.prompt_len, a.gen_len
    max_b = max(a.batch, 1 if (a.no_points or a.serve or a.timeline) else 64)
    if a.serve:
        prompt_len, max_b = a.serve_max, a.serve
    else:
        # requests that finish their prompt early decode while the others still prefill, and the warm-up and
        # the timed regions come on top: no request may run out of tokens before the measurement ends
        gen_len = max(gen_len, max_b * prompt_len // 2048 + a.warmup + max(a.steps, MAX_TIMED_STEPS) + 32)
    if prompt_len + gen_len + 16 > a.context:
        print(f"bench.py: --context {a.context} is too short for prompts of {prompt_len} plus {gen_len} generated tokens")
        return 2

    import torch
    for kv in a.tuning:
        from vllm_oxide_b200.tuning import TUNING
        k, _, v = kv.partition("=")
        if not hasattr(TUNING, k):
            print(f"bench.py: TUNING has no field {k!r}")
            return 2
        setattr(TUNING, k, int(v))
    if a.fold_rows is not None:
        from vllm_oxide_b200.tuning import TUNING
        TUNING.few_rows = a.fold_rows
    sz = SIZES[a.sizes]
    full_layers = sz["layers"]
    layers = a.layers or full_layers
    peaks = load_peaks()
    cfg, llm = make_engine(sz, layers, max_b, prompt_len + gen_len, a.context, graphs=not a.no_graphs)
    runner = llm.runner
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (prompt_len,), generator=g).tolist() for _ in range(max_b)]
    if a.serve:
        sampler = ClockSampler()
        sampler.start()
        res = serve_measure(llm, cfg, layers, a.serve, a.serve_min, a.serve_max, gen_len, peaks)
        res.update({"metric": f"serving run through LLM.generate ({sz['name']}): generated tok/s", "n_gpus": 1, "dtype": "bf16",
                    "data": "synthetic: random weights N(0,0.02), seeded uniform token ids and prompt lengths",
                    "config": {"model": sz["name"], "layers": layers, "layers_full": full_layers, "requests": a.serve,
                               "prompt_len_min": a.serve_min, "prompt_len_max": a.serve_max, "generated_per_request": gen_len,
                               "max_batch_tokens": 2048, "page_size": 16},
                    "clocks": sampler.stop(), "run": run_record(), "impl": "ours"})
        print(json.dumps(res))
        return 0
    if a.timeline:
        return timeline_of_a_decode_step(llm, prompts, a.batch, prompt_len, gen_len)

    sampler = ClockSampler()
    sampler.start()
    # ---------------------------------------------------------------- prefill of 2,048 tokens, one step
    PREFILL = min(2048, prompt_len)
    pre_ms = timed_prefill(llm, prompts[0], PREFILL)
    lin_flops, attn_flops = model_flops(cfg, layers)
    pre_flops = lin_flops * PREFILL + attn_flops * PREFILL * (PREFILL + 1) / 2 + 2.0 * cfg.vocab_size * cfg.hidden_size
    prefill = {"value": PREFILL / (pre_ms / 1e3), "tokens": PREFILL, "ms": pre_ms,
               "frac": pre_flops / (pre_ms / 1e3) / (peaks["bf16_tflops"] * 1e12)}
    # ---------------------------------------------------------------- decode, device-timed and end to end
    ms_step, ctx_sum, launches, regions = decode_device(llm, prompts, a.batch, a.steps, a.warmup, prompt_len, gen_len)
    value = a.batch / (ms_step / 1e3)
    read_bytes = runner.step_read_bytes(ctx_sum)
    achieved = read_bytes / (ms_step / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "of": peaks["source"]}
    e2e_val = decode_e2e(llm, prompts, a.batch, a.steps, a.warmup, prompt_len, gen_len)
    e2e = {"value": e2e_val, "unit": "tok/s", "h2d_bytes_per_step": runner.last_upload_bytes, "d2h_bytes_per_step": 4 * a.batch}
    points = {}
    if not a.no_points:
        for B in (1, 64):
            ms_b, ctx_b, _, _ = decode_device(llm, prompts, B, min(a.steps, 64), a.warmup, prompt_len, gen_len)
            points[f"decode_b{B}"] = B / (ms_b / 1e3)
            gbs = runner.step_read_bytes(ctx_b) / (ms_b / 1e3) / 1e9
            points[f"decode_b{B}_hbm_frac"] = gbs / peaks["hbm_gbs"]
    weights_gb = runner.spec.weight_bytes / 1e9
    graphs_on = bool(runner.graphs_enabled)
    if a.all_configs:
        free_engine(llm)
        del runner
        points.update(all_config_points(peaks, a.steps, a.warmup))
    clocks = sampler.stop()

    out = {
        "metric": METRIC if a.sizes == "1b" else METRIC.replace("Llama 3.2 1B", sz["name"]), "value": value, "unit": "tok/s",
        "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), seeded uniform token ids",
        "config": {"model": sz["name"], "layers": layers, "layers_full": full_layers, "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "global_batch": a.batch,
                   "seq_len": a.context, "prompt_len": prompt_len, "generated": gen_len, "page_size": 16,
                   "parallelism": "single-gpu", "l2": f"inputs larger than L2 (weights {weights_gb:.1f} GB per step)",
                   "cuda_graphs": graphs_on, "timed_regions": regions},
        "e2e": e2e, "gpu_launches": launches, "prefill": prefill, "roofline": roofline, "points": points,
        "clocks": clocks, "run": run_record(), "impl": "ours",
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
