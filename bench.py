#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Llama 3.2 1B sizes with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl ours|reference]
                    [--sizes 1b|3b|8b] [--prompt-len P] [--gen-len G] [--context C]

A "step" is one decode step of `--batch` requests, each with a 2,048-token prompt already in the
cache. `value` is decoded tokens per second timed on the device (CUDA events around K steps, each
step uploading its own metadata and replaying the step's kernels); `e2e` is the same number
through the Python entry point (`LLM.add_request` / `LLM.step`), host tokens in and out. The same
line carries the 2,048-token prefill, the decode step's HBM roofline, and decode at batch 1 and 64.
Prints ONE JSON line. One GPU only. The defaults are the benchmark's configuration (Llama 3.2 1B
sizes, batch 8, 2,048-token prompts, 256 generated); --sizes / --prompt-len / --gen-len / --context
run the same measurements at the other layer sizes and context lengths.
"""
from __future__ import annotations

import argparse
import json
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


def reference_arm():
    # The reference is a Rust workspace (Cargo.toml, crates/engine) with no Python packaging and
    # no GPU code; neither pip nor cargo can build it on this machine.
    print(json.dumps({"impl": "reference", "unavailable":
                      "the reference is a CPU-only Rust workspace (no setup.py/pyproject, no cargo/rustc here); "
                      "pip install of its source tree fails and it has no GPU path to run"}))
    return 0


def serve_run(a, llm, cfg, sz, layers, full_layers, gen_len, params):
    """Many requests of different lengths at once through the public entry point: the scheduler
    cuts prompts into portions under the token budget and mixes them with the decoding of the
    requests that are through. Wall-clock time of generate(), host token ids in and out."""
    import time
    import torch
    g = torch.Generator().manual_seed(7)
    lens = torch.randint(a.serve_min, a.serve_max + 1, (a.serve,), generator=g).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    for _ in range(2):                  # warm-up: the same run twice (library handles; a step's shape class is
        llm.generate(prompts, params)   # recorded as a CUDA graph when it comes the second time)
    torch.cuda.synchronize()
    sampler = ClockSampler()
    sampler.start()
    steps0 = llm.runner.steps_run
    t0 = time.perf_counter()
    outs = llm.generate(prompts, params)
    torch.cuda.synchronize()
    secs = time.perf_counter() - t0
    clocks = sampler.stop()
    generated = sum(len(o.token_ids) for o in outs)
    print(json.dumps({
        "metric": f"serving run through LLM.generate ({sz['name']}): generated tok/s", "value": generated / secs, "unit": "tok/s",
        "total_tok_s": (sum(lens) + generated) / secs, "seconds": secs, "engine_steps": llm.runner.steps_run - steps0,
        "preemptions": llm.stats.get("preemptions", 0), "n_gpus": 1, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), seeded uniform token ids and prompt lengths",
        "config": {"model": sz["name"], "layers": layers, "layers_full": full_layers, "requests": a.serve,
                   "prompt_len_min": a.serve_min, "prompt_len_max": a.serve_max, "prompt_tokens": sum(lens),
                   "generated_per_request": gen_len, "max_batch_tokens": 2048, "page_size": 16},
        "clocks": clocks, "impl": "ours"}))
    return 0


def main():
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
    ap.add_argument("--serve", type=int, default=0, metavar="N",
                    help="instead of the step measurements: N requests with prompts of seeded uniform lengths in "
                         "[--serve-min, --serve-max], --gen-len tokens each, all handed to LLM.generate at once "
                         "(chunked prefill mixed with decoding); prints one line with total tokens a second")
    ap.add_argument("--serve-min", type=int, default=128)
    ap.add_argument("--serve-max", type=int, default=4096)
    a = ap.parse_args()
    prompt_len, gen_len = a.prompt_len, a.gen_len
    # requests that finish their prompt early decode while the others still prefill, and the timed
    # steps come on top: no request may run out of tokens before the measurement ends
    max_b_guard = max(a.batch, 1 if a.no_points else 64)
    if not a.serve:
        gen_len = max(gen_len, max_b_guard * prompt_len // 2048 + max(a.warmup, 3) + a.steps + 16)
    if a.impl == "reference":
        return reference_arm()
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    a.warmup = max(a.warmup, 3)
    if a.serve:
        prompt_len = a.serve_max
    if prompt_len + gen_len + 16 > a.context:
        print(f"bench.py: --context {a.context} is too short for prompts of {prompt_len} plus {gen_len} generated tokens")
        return 2

    import torch
    from vllm_oxide_b200 import models  # noqa: F401
    from vllm_oxide_b200.config import EngineConfig, LlamaConfig, RopeScaling
    from vllm_oxide_b200.engine import LLM, ModelRunner
    from vllm_oxide_b200.sampling import SamplingParams
    from vllm_oxide_b200.weights import random_tensors
    from vllm_oxide_b200 import kernels

    sz = SIZES[a.sizes]
    full_layers = sz["layers"]
    layers = a.layers or full_layers
    cfg = LlamaConfig(hidden_size=sz["hidden"], intermediate_size=sz["inter"], num_hidden_layers=layers,
                      num_attention_heads=sz["heads"], num_key_value_heads=8, head_dim=sz["head_dim"], vocab_size=128256,
                      max_position_embeddings=131072, rms_norm_eps=1e-5, rope_theta=500000.0,
                      rope_scaling=RopeScaling(sz["rope_factor"], 1.0, 4.0, 8192), tie_word_embeddings=sz["tied"],
                      bos_token_id=128000, eos_token_ids=(128001,))
    context_len = a.context
    max_b = 64 if not a.no_points else max(a.batch, 1)
    max_b = max(max_b, a.batch)
    if a.serve:
        max_b = a.serve
    pages_per_req = -(-(prompt_len + gen_len + 16) // 16)
    engine = EngineConfig(max_batch_tokens=2048, max_seqs=max_b, max_model_len=context_len, block_size=16,
                          num_pages=max_b * pages_per_req + 8, dtype="bfloat16", cuda_graphs=not a.no_graphs)
    dev = "cuda:0"
    tensors = random_tensors(models.llama_manifest(cfg), seed=0, std=0.02, dtype=torch.bfloat16, device=dev)
    runner = ModelRunner(cfg, tensors, engine)
    del tensors
    llm = LLM(runner)
    peaks = load_peaks()
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (prompt_len,), generator=g).tolist() for _ in range(max_b)]
    never_stop = SamplingParams(max_new_tokens=gen_len, temperature=0.0, stop_token_ids=())
    if a.serve:
        return serve_run(a, llm, cfg, sz, layers, full_layers, gen_len, never_stop)
    PREFILL = min(2048, prompt_len)          # the timed prefill is one step of this many tokens

    def ev():
        return torch.cuda.Event(enable_timing=True)

    # ---------------------------------------------------------------- prefill of 2,048 tokens
    rt = runner.rt
    def prefill_once(rid):
        runner.admit(rid)
        runner.manager.reserve(rid, PREFILL)
        arrays = runner.build_arrays([rt.StepEntry(rid, prompts[0][:PREFILL], [PREFILL - 1])])
        e0, e1 = ev(), ev()
        e0.record()
        runner.step(arrays)
        e1.record()
        torch.cuda.synchronize()
        runner.manager.release(rid)
        return e0.elapsed_time(e1)
    for i in range(3):
        prefill_once(900000 + i)
    sampler = ClockSampler()
    sampler.start()
    pre_ms = sorted(prefill_once(900100 + i) for i in range(5))[2]
    lin_params = layers * (cfg.hidden_size * (cfg.q_dim + 2 * cfg.kv_dim) + cfg.q_dim * cfg.hidden_size
                           + 3 * cfg.hidden_size * cfg.intermediate_size)
    pre_flops = 2.0 * lin_params * PREFILL + layers * 2.0 * 2.0 * cfg.q_dim * PREFILL * (PREFILL + 1) / 2 \
        + 2.0 * cfg.vocab_size * cfg.hidden_size
    prefill = {"value": PREFILL / (pre_ms / 1e3), "tokens": PREFILL, "ms": pre_ms,
               "frac": pre_flops / (pre_ms / 1e3) / (peaks["bf16_tflops"] * 1e12)}

    def prefill_all(ids):
        """Step until every request has its first token (none may finish on the way: GEN_LEN is
        far above the number of steps that takes)."""
        for _ in range(2 * (len(ids) * prompt_len // 2048 + len(ids)) + 32):
            if all(llm._generated.get(r, 0) >= 1 for r in ids):
                return
            llm.step()
        raise RuntimeError("bench: the prompts did not finish prefilling")

    # ---------------------------------------------------------------- decode, device-timed
    def decode_device(B, steps, warmup):
        """B requests with their prompts in the cache; time `steps` decode steps on the device."""
        ids = []
        for i in range(B):
            ids.append(llm.add_request(prompts[i], never_stop))
        prefill_all(ids)                                          # chunked prefill through the scheduler
        for _ in range(warmup):
            llm.step()
        torch.cuda.synchronize()
        launches0 = kernels.launch_count()
        ctx0 = sum(runner.manager.length(r) for r in ids)
        e0, e1 = ev(), ev()
        e0.record()
        for _ in range(steps):
            llm.step_async()
        e1.record()
        torch.cuda.synchronize()
        llm.drain_async()
        ctx1 = sum(runner.manager.length(r) for r in ids)
        ms = e0.elapsed_time(e1) / steps
        launches = kernels.launch_count() - launches0
        for r in ids:
            llm.abort(r)
        return ms, (ctx0 + ctx1) / 2.0, launches

    ms_step, mean_ctx, launches = decode_device(a.batch, a.steps, a.warmup)
    value = a.batch / (ms_step / 1e3)
    read_bytes = runner.spec.weight_bytes + mean_ctx * runner.pools.bytes_per_token()
    achieved = read_bytes / (ms_step / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "of": peaks["source"]}

    # ---------------------------------------------------------------- decode, end to end
    def decode_e2e(B, steps, warmup):
        ids = [llm.add_request(prompts[i], never_stop) for i in range(B)]
        prefill_all(ids)
        for _ in range(warmup):
            llm.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            llm.step()                      # host tokens in (metadata upload), picked tokens out (D2H read)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        for r in ids:
            llm.abort(r)
        return B * steps / dt
    e2e_steps = max(1, min(a.steps, gen_len - a.warmup - 2))
    e2e_val = decode_e2e(a.batch, e2e_steps, a.warmup)
    e2e = {"value": e2e_val, "unit": "tok/s", "h2d_bytes_per_step": runner.last_upload_bytes,
           "d2h_bytes_per_step": 4 * a.batch}

    points = {}
    if not a.no_points:
        for B in (1, 64):
            ms_b, _, _ = decode_device(B, min(a.steps, 64), a.warmup)
            points[f"decode_b{B}"] = B / (ms_b / 1e3)
    clocks = sampler.stop()

    out = {
        "metric": METRIC if a.sizes == "1b" else METRIC.replace("Llama 3.2 1B", sz["name"]), "value": value, "unit": "tok/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), seeded uniform token ids",
        "config": {"model": sz["name"], "layers": layers, "layers_full": full_layers, "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "global_batch": a.batch,
                   "seq_len": context_len, "prompt_len": prompt_len, "generated": gen_len, "page_size": 16,
                   "parallelism": "single-gpu", "l2": "inputs larger than L2 (weights 2.5 GB per step)",
                   "cuda_graphs": bool(runner.graphs_enabled)},
        "e2e": e2e, "gpu_launches": launches, "prefill": prefill, "roofline": roofline, "points": points,
        "clocks": clocks, "impl": "ours",
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
