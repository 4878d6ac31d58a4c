"""Command line, in the reference's manner.

    python -m vllm_oxide_b200 generate [model_dir] "prompt" [max_new] [--profile]

is the reference's `generate` example with its positional arguments, defaults and log fields
(crates/engine/examples/generate.rs:3,17-27,42-69: model folder default models/Llama-3.2-1B, prompt
default "The capital of France is", max_new default 64, stop at the model's eos, prefill tok/s =
prompt tokens / prefill time, decode tok/s = tokens after the first / decode time). Options
beyond the reference's: --prompt-ids / --prompt-len (token ids instead of text, for model folders
without a tokenizer), --random-weights SEED (the folder needs only config.json; weights are drawn
from the seed), --temperature, --seed, --dtype, and the engine limits by their `EngineConfig` names.

    python -m vllm_oxide_b200 load_weights [model_dir]         (crates/engine/examples/load_weights.rs:11-28)
    python -m vllm_oxide_b200 random_weights model_dir --config config.json --seed N [--std S]
    python -m vllm_oxide_b200 replay ...                       (same as bin/trace_run)
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def _engine_args(ap):
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--max-batch-tokens", type=int, default=2048)
    ap.add_argument("--max-seqs", type=int, default=32)
    ap.add_argument("--max-model-len", type=int, default=8192)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--kv-pool-bytes", type=int, default=2 << 30)
    ap.add_argument("--num-pages", type=int, default=None)
    ap.add_argument("--prefill-chunk", type=int, default=None)
    ap.add_argument("--no-cuda-graphs", action="store_true")


def _engine_kwargs(a):
    return dict(max_batch_tokens=a.max_batch_tokens, max_seqs=a.max_seqs, max_model_len=a.max_model_len,
                block_size=a.block_size, kv_pool_bytes=a.kv_pool_bytes, num_pages=a.num_pages,
                prefill_chunk=a.prefill_chunk, cuda_graphs=not a.no_cuda_graphs)


def cmd_generate(argv):
    ap = argparse.ArgumentParser(prog="vllm_oxide_b200 generate")
    ap.add_argument("model_dir", nargs="?", default="models/Llama-3.2-1B")
    ap.add_argument("prompt", nargs="?", default="The capital of France is")
    ap.add_argument("max_new", nargs="?", type=int, default=64)
    ap.add_argument("--profile", action="store_true", help="per-kernel device time of one decode step")
    ap.add_argument("--prompt-ids", default=None, help="comma-separated token ids instead of text")
    ap.add_argument("--prompt-len", type=int, default=None, help="a seeded random prompt of this many tokens")
    ap.add_argument("--max-new", dest="max_new_opt", type=int, default=None, help="same as the positional max_new")
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                    help="read only config.json and draw the weights from this seed")
    ap.add_argument("--random-weights-std", type=float, default=0.02, metavar="S", help="their standard deviation")
    _engine_args(ap)
    a = ap.parse_args(argv)
    if a.max_new_opt is not None:
        a.max_new = a.max_new_opt
    import torch
    from .engine import LLM
    from .sampling import SamplingParams
    t = time.perf_counter()
    llm = LLM(a.model_dir, dtype=a.dtype, random_weights_seed=a.random_weights, random_weights_std=a.random_weights_std,
              **_engine_kwargs(a))
    print(f"loaded secs={time.perf_counter() - t:.3f}", file=sys.stderr)
    if a.prompt_ids is not None:
        ids = [int(x) for x in a.prompt_ids.split(",") if x.strip()]
    elif a.prompt_len is not None:
        g = torch.Generator().manual_seed(a.seed)
        ids = torch.randint(0, llm.runner.spec.vocab_size, (a.prompt_len,), generator=g).tolist()
    else:
        ids = llm.encode(a.prompt)
    from .engine import Generator
    gen = Generator(llm)
    if a.temperature > 0:
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = llm.generate([ids], SamplingParams(max_new_tokens=a.max_new, temperature=a.temperature, seed=a.seed))[0]
        torch.cuda.synchronize()
        tokens, prefill_s, decode_s = out.token_ids, float("nan"), time.perf_counter() - t0
    else:
        eos = llm.runner.spec.eos_token_ids
        res = gen.greedy(ids, a.max_new, eos[0] if eos else None)
        tokens, prefill_s, decode_s = res.tokens, res.prefill_time, res.decode_time
    decoded = max(len(tokens) - 1, 0)
    print(json.dumps({
        "prompt_tokens": len(ids), "generated": len(tokens), "prefill_ms": prefill_s * 1e3,
        "prefill_tok_s": len(ids) / prefill_s if prefill_s == prefill_s else None,
        "decode_tok_s": decoded / decode_s if decode_s > 0 else None,
        "ms_per_decode_token": decode_s * 1e3 / max(decoded, 1),
        "workspace_high_water_mb": llm.runner.workspace.high_water / 1e6}), file=sys.stderr)
    if a.profile:
        from .engine.profile import profile_decode_step
        for name, calls, ms in profile_decode_step(llm.runner, ids[:16] or [0]):
            print(f"profile op={name} calls={calls} total_ms={ms:.4f}", file=sys.stderr)
    text = llm.decode(tokens)
    print(text if text is not None else " ".join(str(t) for t in tokens))
    return 0


def cmd_load_weights(argv):
    ap = argparse.ArgumentParser(prog="vllm_oxide_b200 load_weights")
    ap.add_argument("model_dir", nargs="?", default="models/Llama-3.2-1B")
    a = ap.parse_args(argv)
    from . import models  # noqa: F401
    from .config import architecture_for, read_config_json
    from .weights import load_safetensors_weights
    t = time.perf_counter()
    d = read_config_json(a.model_dir)
    arch = architecture_for(d)
    cfg = arch.config_cls.from_dict(d)
    w = load_safetensors_weights(a.model_dir, arch.manifest(cfg))
    n = w.param_count()
    print(f"params={n} expected={cfg.param_count()} gb={n * 2 / 1e9:.3f} secs={time.perf_counter() - t:.3f}")
    return 0 if n == cfg.param_count() else 1


def cmd_random_weights(argv):
    ap = argparse.ArgumentParser(prog="vllm_oxide_b200 random_weights")
    ap.add_argument("model_dir")
    ap.add_argument("--config", required=True, help="a config.json to take the sizes from")
    ap.add_argument("--seed", type=int, required=True)
    ap.add_argument("--std", type=float, default=0.02)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    a = ap.parse_args(argv)
    from . import models  # noqa: F401
    from .config import architecture_for, parse_dtype
    from .weights import write_random_model
    with open(a.config) as f:
        d = json.load(f)
    cfg = architecture_for(d, a.config).config_cls.from_dict(d, a.config)
    write_random_model(a.model_dir, cfg, a.seed, a.std, parse_dtype(a.dtype))
    print(f"wrote {a.model_dir}/config.json and model.safetensors ({cfg.param_count()} parameters, seed {a.seed})")
    return 0


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    cmds = {"generate": cmd_generate, "load_weights": cmd_load_weights, "random_weights": cmd_random_weights}
    if argv and argv[0] == "replay":
        from .replay.trace import main as replay_main
        return replay_main(argv[1:])
    if not argv or argv[0] not in cmds:
        print(__doc__, file=sys.stderr)
        return 2
    from .errors import EngineError
    try:
        return cmds[argv[0]](argv[1:])
    except EngineError as e:                      # a user's mistake or a limit: one line, no traceback
        print(f"{argv[0]}: {type(e).__name__}: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
