"""Per-op device time of one decode step (the CLI's --profile; the reference's per-op totals,
crates/engine/examples/generate.rs:56-67)."""
from __future__ import annotations

from .. import kernels


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
