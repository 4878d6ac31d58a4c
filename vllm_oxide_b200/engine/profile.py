"""Per-op device time of one decode step (the CLI's --profile; the reference's per-op totals,
crates/engine/examples/generate.rs:56-67)."""
from __future__ import annotations

from .. import kernels
from ..parts.base import LONG_CONTEXT_KEYS


def profile_decode_step(runner, prompt, steps: int = 4):
    """Prefill `prompt` for a scratch request, then time `steps` single-token steps op by op."""
    rt = runner.rt
    rid = (1 << 40) + runner.steps_run
    if runner.admit(rid) < 0:
        return []
    try:
        toks = list(prompt)
        runner.manager.reserve(rid, len(toks))
        arrays = runner.build_arrays([rt.StepEntry(rid, toks, [len(toks) - 1])])
        nxt = runner.step(arrays).tokens()[0]
        runner.manager.commit(rid, len(toks))
        with kernels.OpProfile() as prof:
            for _ in range(steps):
                if not runner.manager.reserve(rid, 1):
                    break
                arrays = runner.build_arrays([rt.StepEntry(rid, [max(nxt, 0)], [0])])
                nxt = runner.step(arrays).tokens()[0]
                runner.manager.commit(rid, 1)
        return prof.totals()
    finally:
        runner.manager.release(rid)


# ------------------------------------------------------------------------------------------------
# Single kernels on synthetic operands, for profilers:
#   python -m vllm_oxide_b200.engine.profile gemm --rows 8 --out 16384 --in 2048 [--copies 6] [--iters 3]
#   python -m vllm_oxide_b200.engine.profile gemm_pair --rows 2048 --out 16384 --in 2048      (the two-SM product)
#   python -m vllm_oxide_b200.engine.profile gemm_pair_swiglu --rows 2048 --out 16384 --in 2048
#   python -m vllm_oxide_b200.engine.profile attn_decode --batch 8 --context 2200
#   python -m vllm_oxide_b200.engine.profile attn_prefill --tokens 2048 [--impl sm100|mma]
# Each launch works on operands of its own (several copies, together larger than L2), so that DRAM
# counters mean something; device time per launch is printed from CUDA events.
# ------------------------------------------------------------------------------------------------
def _kernel_cases(argv):
    import argparse
    import math
    import torch
    ap = argparse.ArgumentParser(prog="vllm_oxide_b200.engine.profile")
    ap.add_argument("kernel", choices=["gemm", "gemm_pair", "gemm_pair_swiglu", "gemm_library", "attn_decode", "attn_prefill"])
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
    ap.add_argument("--impl", default="sm100", choices=["sm100", "mma"], help="attn_prefill: the tcgen05 or the mma.sync kernel")
    a = ap.parse_args(argv)
    dev = "cuda:0"
    bf = torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s: torch.randn(*s, generator=g, device=dev).to(bf)
    if a.kernel in ("gemm", "gemm_pair", "gemm_pair_swiglu", "gemm_library"):
        x = rnd(a.rows, a.inner)
        ws = [rnd(a.out, a.inner) for _ in range(a.copies)]
        if a.kernel == "gemm_pair_swiglu":          # --out counts the rows of [Wg; Wu]
            out = torch.empty(a.rows, a.out // 2, dtype=bf, device=dev)
            launches = [lambda w=w: kernels.gemm_pair_swiglu(x, w, out) for w in ws]
        else:
            out = torch.empty(a.rows, a.out, dtype=bf, device=dev)
            if a.kernel == "gemm_library":           # the library product the engine uses above 32 rows, for comparison
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
            # the engine's choice (parts/attention.py decode_splits): a cluster of up to 8 blocks per
            # request and kv head, or, for one few requests with long contexts, up to 64 that merge through global memory
            sms = torch.cuda.get_device_properties(dev).multi_processor_count
            wide = 3 * sms // (S * KV) >= 4 and (ctx > LONG_CONTEXT_KEYS if a.merge == "auto" else a.merge == "global")
            splits = max(1, min(64, 3 * sms // (S * KV))) if wide else max(1, min(8, -(-2 * sms // (S * KV))))
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
            if a.impl == "sm100":
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
    if a.graph:
        kernels.set_pdl(True)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(2):
                for f in launches:
                    f()
        g.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(max(a.iters, 3)):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) * 1e3 / (2 * len(launches)))
        us = sorted(times)[len(times) // 2]
        print(f"{a.kernel}: {us:.1f} us per launch (events around a CUDA graph of {2 * len(launches)} launches back to back); "
              f"{nbytes / us / 1e3:.0f} GB/s of the bytes it must read; {flops / us / 1e6:.1f} TFLOP/s")
        return
    times = []
    for _ in range(a.iters):
        for f in launches:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            f()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) * 1e3)
    us = sorted(times)[len(times) // 2]
    print(f"{a.kernel}: {us:.1f} us per launch (events, single launches); {nbytes / us / 1e3:.0f} GB/s of the bytes it must read; "
          f"{flops / us / 1e6:.1f} TFLOP/s")


if __name__ == "__main__":
    import sys
    _kernel_cases(sys.argv[1:])
