"""The Python entry point: load a model folder, generate.

`Generator.greedy(prompt, max_new, stop, capture)` is the reference's library call with its names
and meanings (crates/engine/src/generate.rs:33-54): token ids in, `GenerateOutput{tokens, captured,
prefill_time, decode_time}` out, the stop token kept, an empty prompt or max_new = 0 refused.
`LLM.generate` is the batched form over the scheduler: many prompts, continuous batching,
chunked prefill, preemption when pages run out. Both run every token through
`ModelRunner.step`. The loop is the one the reference plans for its engine thread
(CLAUDE.md:68): schedule, prepare inputs, forward, sample, emit.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Union

import torch

from ..config import EngineConfig
from ..errors import CapacityError, EngineError, NaNError, ShapeError
from ..sampling import SamplingParams
from .runner import ModelRunner
from .tokenizer import TextTokenizer


@dataclass
class RequestOutput:
    request_id: int
    prompt_token_ids: List[int]
    token_ids: List[int]
    finish_reason: str                      # "stop", "length", "capacity", "abort"
    text: Optional[str] = None
    logits: Dict[int, torch.Tensor] = field(default_factory=dict)   # generated position -> float32 [vocab]
    preemptions: int = 0


@dataclass
class GenerateOutput:
    """crates/engine/src/generate.rs:22-30."""
    tokens: List[int]
    captured: List[tuple]                   # (generated index, float32 [vocab])
    prefill_time: float
    decode_time: float


class LLM:
    def __init__(self, model: Union[str, ModelRunner], dtype="bfloat16", random_weights_seed: Optional[int] = None,
                 random_weights_std: float = 0.02, **engine_kwargs):
        """`model`: a folder with config.json and safetensors weights (and, for text prompts, a
        tokenizer.json), or a `ModelRunner`. `random_weights_seed`: read only config.json and draw
        the weights from this seed (N(0, `random_weights_std`), norm weights 1). Everything else is
        an `EngineConfig` field."""
        if isinstance(model, ModelRunner):
            self.runner = model
        else:
            self.runner = ModelRunner.from_dir(model, EngineConfig(dtype=dtype, **engine_kwargs),
                                               random_weights_seed=random_weights_seed, random_weights_std=random_weights_std)
        r = self.runner
        e = r.engine
        self.scheduler = r.rt.Scheduler(r.manager, e.max_batch_tokens, e.max_seqs, r.max_model_len,
                                        e.prefill_chunk or 0)
        self.scheduler.set_admission_watermark(int(getattr(e, "admission_watermark_pages", 0)))
        self._next_id = 0
        self._params: Dict[int, SamplingParams] = {}
        self._prompts: Dict[int, List[int]] = {}
        self._captured: Dict[int, Dict[int, torch.Tensor]] = {}
        self._generated: Dict[int, int] = {}
        self._preempt: Dict[int, int] = {}
        self._tokenizer = None
        # called as on_token(request id, token) for every generated token as soon as the host has read
        # it, in generation order per request (a token computed past a stop token is never reported)
        self.on_token = None
        self._logit_buf = None
        self._inflight = None            # a decode step launched but not read yet: (plan, ids, parity, event)
        self._late: List[RequestOutput] = []
        self._capturing = 0              # live requests that want logits (they are never run ahead of)
        self.run_ahead = bool(e.run_ahead) and bool(e.cuda_graphs)
        self.stats = {"steps": 0, "preemptions": 0, "decode_steps": 0, "graph_steps": 0, "ahead_steps": 0}
        if isinstance(model, (str, os.PathLike)):
            self._tokenizer = TextTokenizer.load(str(model))

    # ------------------------------------------------------------------ requests
    def encode(self, text: str) -> List[int]:
        """Token ids of `text` with the special tokens the tokenizer's post-processor defines
        (a leading BOS for Llama 3: crates/engine/src/tokenizer.rs:25-30)."""
        if self._tokenizer is None:
            raise ShapeError("generate", "text prompts need a tokenizer.json in the model folder; pass token ids")
        return self._tokenizer.encode(text)

    def decode(self, ids: Sequence[int]) -> Optional[str]:
        """Text of `ids`, special tokens (BOS, EOS) skipped (crates/engine/src/tokenizer.rs:33-38);
        None without a tokenizer."""
        if self._tokenizer is None:
            return None
        return self._tokenizer.decode(ids)

    def add_request(self, prompt: Union[str, Sequence[int]], params: SamplingParams) -> int:
        ids = self.encode(prompt) if isinstance(prompt, str) else [int(t) for t in prompt]
        vocab = self.runner.spec.vocab_size
        for t in ids:
            if not 0 <= t < vocab:
                raise ShapeError("generate", f"token {t} is outside the vocabulary of {vocab}")
        stops = list(self.runner.spec.eos_token_ids) if params.stop_token_ids is None else [int(s) for s in params.stop_token_ids]
        rid = self._next_id
        self._next_id += 1
        rt = self.runner.rt
        try:
            self.scheduler.add_request(rid, ids, rt.SamplingParams(int(params.max_new_tokens), float(params.temperature),
                                                                   int(params.seed), stops))
        except rt.RuntimeFault as e:
            msg = str(e)
            if msg.startswith("capacity"):
                need = len(ids) + params.max_new_tokens - 1
                raise CapacityError("sequence length", need, self.runner.max_model_len) from e
            raise ShapeError("generate", msg) from e
        self._params[rid] = params
        self._prompts[rid] = ids
        self._captured[rid] = {}
        self._generated[rid] = 0
        if params.capture_logits:
            self._capturing += 1
        return rid

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished() or self._inflight is not None or bool(self._late)

    # ------------------------------------------------------------------ one engine step
    def step(self) -> List[RequestOutput]:
        """One engine step: schedule -> arrays -> forward -> pick -> update. Returns the requests
        that finished.

        While every running request decodes and none can end by length with its next token, the
        engine runs one step ahead of its own reads: this call launches step n + 1, whose input
        tokens are step n's picks taken on the device, and only then waits for step n's tokens
        (`EngineConfig.run_ahead`). The GPU never waits for the host between such steps; a request
        that picks a stop token is seen one step late and what it was given since is dropped.
        Tokens do not depend on whether steps are run ahead."""
        outs, self._late = self._late, []
        fl = self._inflight
        if fl is None:
            if self._may_run_ahead():
                self._launch_ahead(feed=False, parity=0)
                return outs
            return outs + self._step_now()
        nxt = None
        if self._may_run_ahead() and list(self.scheduler.running()) == fl[1]:
            nxt = self._launch_ahead(feed=True, parity=1 - fl[2])
        else:
            self._inflight = None
        ended = self._resolve(fl, 1 if nxt else 0)
        if ended and nxt:
            # the rows of the step in flight no longer match the running set: read it now
            self._inflight = None
            ended += self._resolve(nxt, 0)
        return outs + ended

    def _may_run_ahead(self) -> bool:
        return self.run_ahead and self._capturing == 0 and self.scheduler.steady_decode()

    def _launch_ahead(self, feed: bool, parity: int):
        r, sched = self.runner, self.scheduler
        plan = sched.schedule()
        if not plan.decode_only or plan.preempted or plan.admitted:
            raise EngineError("run-ahead: the scheduler planned something else than a steady decode step")
        ids = plan.sampling_ids()
        event = r.decode_step_graph(sched, plan, feed_from_device=feed, read=False, parity=parity)
        sched.advance(plan)
        for rid in ids:
            self._generated[rid] += 1
        self.stats["steps"] += 1
        self.stats["decode_steps"] += 1
        self.stats["graph_steps"] += 1
        self.stats["ahead_steps"] += 1
        if self.stats["steps"] % 64 == 0:
            r.check_kernels()
        self._inflight = (plan, ids, parity, event)
        return self._inflight

    def _resolve(self, flight, ahead: int) -> List[RequestOutput]:
        plan, ids, parity, event = flight
        sampled = self.runner.read_decode(event, len(ids), parity)
        if min(sampled, default=0) < 0:
            raise NaNError("pick_tokens")            # crates/engine/src/backend/cpu/mod.rs:377-379
        if self.on_token is not None:
            for rid, tok in zip(ids, sampled):
                if rid in self._params:              # not one that ended on a stop token a step earlier
                    self.on_token(rid, tok)
        return self._outputs(self.scheduler.resolve(plan, sampled, ahead))

    def _finish_inflight(self) -> None:
        """Read the step in flight, if any; requests it ends are handed out by the next `step`."""
        fl, self._inflight = self._inflight, None
        if fl is not None:
            self._late += self._resolve(fl, 0)

    def _step_now(self) -> List[RequestOutput]:
        r, sched = self.runner, self.scheduler
        plan = sched.schedule()
        self.stats["preemptions"] += len(plan.preempted)
        for rid in plan.preempted:
            self._preempt[rid] = self._preempt.get(rid, 0) + 1
        for rid in plan.admitted:
            r.pools.reset_slot(r.manager.state_slot(rid))
        done = []
        if plan.num_entries:
            decode_only = plan.decode_only
            sampling = plan.sampling_ids()
            want_logits = any(self._params[i].capture_logits for i in sampling)
            if decode_only and r.graphs_enabled and not want_logits:
                sampled = r.decode_step_graph(sched, plan)
                self.stats["graph_steps"] += 1
            else:
                arrays = sched.arrays(plan, r.rows_cap, r.seqs_cap, r.logits_cap, r.max_pages, r.spec.vocab_size)
                buf = None
                if want_logits:
                    if self._logit_buf is None:
                        self._logit_buf = torch.empty((r.seqs_cap, r.spec.vocab_size), dtype=torch.float32, device=r.device)
                    buf = self._logit_buf
                sampled = r.step(arrays, logits_out=buf).tokens()
                if want_logits:
                    for row, rid in enumerate(sampling):
                        g = self._generated[rid]
                        if g in self._params[rid].capture_logits:
                            self._captured[rid][g] = buf[row].cpu()
            if min(sampled, default=0) < 0:
                raise NaNError("pick_tokens")        # crates/engine/src/backend/cpu/mod.rs:377-379
            self.stats["steps"] += 1
            self.stats["decode_steps"] += int(decode_only)
            if self.stats["steps"] % 64 == 0:
                r.check_kernels()                    # one word from the device: a kernel's bounded wait that expired
            gen = self._generated
            for rid in sampling:
                gen[rid] += 1
            if self.on_token is not None:
                for rid, tok in zip(sampling, sampled):
                    self.on_token(rid, tok)
            done = sched.update(plan, sampled)
        else:
            done = sched.take_done()
            if not done and not plan.preempted and sched.has_unfinished():
                raise CapacityError("scheduler made no progress: pages", 1, 0)
        return self._outputs(done)

    def _outputs(self, done) -> List[RequestOutput]:
        outs = []
        for f in done:
            rid = f.id
            if self._params[rid].capture_logits:
                self._capturing -= 1
            outs.append(RequestOutput(rid, self._prompts.pop(rid), list(f.output), f.reason,
                                      self.decode(f.output), self._captured.pop(rid), self._preempt.pop(rid, 0)))
            self._params.pop(rid)
            self._generated.pop(rid)
        return outs

    def drain(self) -> None:
        """Wait for the step that was launched ahead, if any, and book its tokens; requests it ends
        are handed out by the next `step`. Afterwards nothing of this engine is in flight."""
        self._finish_inflight()

    def abort(self, request_id: int) -> None:
        self._finish_inflight()
        if request_id not in self._params:
            return
        if self.scheduler.abort(request_id):
            self.scheduler.take_done()
        self._forget(request_id)

    def _forget(self, rid: int) -> None:
        if rid in self._params and self._params[rid].capture_logits:
            self._capturing -= 1
        for d in (self._params, self._prompts, self._captured, self._generated, self._preempt):
            d.pop(rid, None)

    # ------------------------------------------------------------------ whole jobs
    def generate(self, prompts, sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 on_token=None) -> List[RequestOutput]:
        """Run every prompt to its end; outputs come back in the order of `prompts`. `on_token(index
        of the prompt, token)` is called for every generated token as soon as the host has read it."""
        if isinstance(prompts, str) or (prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        if sampling_params is None:
            sampling_params = SamplingParams()
        plist = [sampling_params] * len(prompts) if isinstance(sampling_params, SamplingParams) else list(sampling_params)
        if len(plist) != len(prompts):
            raise ShapeError("generate", f"{len(prompts)} prompts but {len(plist)} sampling parameter sets")
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, plist)]
        results: Dict[int, RequestOutput] = {}
        mine, before = {rid: i for i, rid in enumerate(ids)}, self.on_token
        if on_token is not None:
            self.on_token = lambda rid, tok: on_token(mine[rid], tok) if rid in mine else None
        try:
            while self.has_unfinished():
                for out in self.step():
                    results[out.request_id] = out
        finally:
            self.on_token = before
        self.runner.check_kernels()
        return [results[i] for i in ids]


class Generator:
    """The reference's single-sequence driver (crates/engine/src/generate.rs:16-54) over this
    engine: one request, greedy, timed. The same engine and pool serve call after call."""

    def __init__(self, model: Union[str, ModelRunner, LLM], **kwargs):
        self.llm = model if isinstance(model, LLM) else LLM(model, **kwargs)

    def model(self) -> ModelRunner:
        return self.llm.runner

    def greedy(self, prompt: Sequence[int], max_new: int, stop: Optional[int] = None,
               capture: Sequence[int] = ()) -> GenerateOutput:
        if len(prompt) == 0 or max_new == 0:
            raise ShapeError("generate", "empty prompt or max_new = 0")       # generate.rs:55-60
        sp = SamplingParams(max_new_tokens=max_new, temperature=0.0, stop_token_ids=() if stop is None else (stop,),
                            capture_logits=tuple(capture))
        llm = self.llm
        rid = llm.add_request(prompt, sp)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = None
        prefill_time = None
        while out is None:
            for o in llm.step():
                if o.request_id == rid:
                    out = o
            if prefill_time is None and (out is not None or llm._generated.get(rid, 0) >= 1):
                torch.cuda.synchronize()
                prefill_time = time.perf_counter() - t0       # up to and including the first token
        torch.cuda.synchronize()
        total = time.perf_counter() - t0
        return GenerateOutput(list(out.token_ids), sorted(out.logits.items()), prefill_time, total - prefill_time)
