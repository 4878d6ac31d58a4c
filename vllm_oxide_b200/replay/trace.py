"""Trace replay: feed given token ids through the model step by step and write logits.

The role of the reference's oracle tooling (tools/reference/dump_logits.py:37-92 records logits
at chosen steps; crates/engine/tests/hf_match.rs:99-168 replays and compares). This program
samples nothing and has no forward pass, cache or loader of its own: it drives the engine's
`ModelRunner.step`, cache manager and kernels, the ones generation uses.

Input: one JSON object per line on standard input,
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
All entries of a step run as one batch. For a step that wants logits, `<out>/<step>.f32` holds
them as little-endian float32 [wanted, vocab], in the order of the entries and of `want`.
After every step a line `done <step>` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


class TraceSession:
    """Replays trace steps on a `ModelRunner`: admits a request at its first entry, reserves
    pages for the tokens an entry brings, runs the batch, commits, and gives back what ended."""

    def __init__(self, runner):
        from ..csrc.build import runtime_module
        self.runner = runner
        self.rt = runtime_module()
        self.ids = {}          # request name -> integer id
        self.next_id = 0

    def run_step(self, msg: dict):
        """Run one step; returns float32 [wanted, vocab] on the host, or None if nothing is wanted."""
        runner, step = self.runner, msg.get("step")
        entries = []
        for e in msg.get("entries", []):
            name = e["id"]
            tokens = [int(t) for t in e["tokens"]]
            if not tokens:
                continue
            if name not in self.ids:
                self.ids[name] = self.next_id
                self.next_id += 1
                if runner.admit(self.ids[name]) < 0:
                    raise RuntimeError(f"step {step}: no state slot left for request {name!r}")
            rid = self.ids[name]
            if not runner.manager.reserve(rid, len(tokens)):
                raise RuntimeError(f"step {step}: the cache pool cannot take {len(tokens)} more tokens "
                                   f"of request {name!r}")
            entries.append(self.rt.StepEntry(rid, tokens, [int(w) for w in e.get("want", [])]))
        out = None
        if entries:
            arrays = runner.build_arrays(entries)
            R = arrays.logit_count
            out = torch.empty((R, runner.spec.vocab_size), dtype=torch.float32) if R else None
            runner.step(arrays, logits_out=out)
            torch.cuda.synchronize()
            runner.check_kernels()
            for rid, n in zip(arrays.ids, arrays.new_counts):
                runner.manager.commit(rid, n)
        for name in msg.get("end", []):
            if name in self.ids:
                runner.manager.release(self.ids.pop(name))
        return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder the logits files are written to")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time; the cache pool is made for this many")
    ap.add_argument("--page-size", type=int, default=16)
    args = ap.parse_args(argv)

    from ..config import EngineConfig
    from ..engine import ModelRunner

    os.makedirs(args.out, exist_ok=True)
    page = args.page_size
    num_pages = max(1, -(-args.max_tokens // page))
    cap = num_pages * page
    engine = EngineConfig(max_batch_tokens=cap, max_seqs=8, max_model_len=cap, block_size=page,
                          num_pages=num_pages, dtype=args.dtype, cuda_graphs=False)
    print(f"[trace_run] loading {args.model} ({args.dtype}); kernels are compiled at the first call",
          file=sys.stderr, flush=True)
    session = TraceSession(ModelRunner.from_dir(args.model, engine))
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        msg = json.loads(line)
        try:
            out = session.run_step(msg)
        except RuntimeError as e:
            raise SystemExit(f"trace_run: {e}")
        if out is not None:
            path = os.path.join(args.out, f"{msg['step']}.f32")
            out.numpy().astype("<f4", copy=False).tofile(path + ".tmp")
            os.replace(path + ".tmp", path)
        print(f"done {msg['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
