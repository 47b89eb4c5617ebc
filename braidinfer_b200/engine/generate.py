"""The generation loop: batches of unequal prompts, stop tokens, sequences that end
earlier, and as many batches one after another as there are requests.

For one sequence it does what the reference's loop does
(crates/braidinfer-runtime/src/generate.rs:314-439): the prompt in one step, the next
token from the last logits, then one token a step; a stop token ends the sequence
before it is emitted (:405-407) and is not returned (:435); at most `max_new_tokens`
tokens come back.  Batching is this library's own: the sequences of a batch start
together, a finished sequence leaves the batch at once and its slot and pages go back
to the cache, and the next batch starts when the last sequence of this one has ended.

The loop talks to an engine (`open`, `close`, `step`) and a sampler (`choose`) only
through those calls, so its decisions are tested on the CPU with stand-ins.

`BRAIDINFER_LOGIT_TRACE=<file>` (the reference's name and meaning, generate.rs:380-396) appends a line
`step=<k> tok=<token> logit_hash=<16 hex digits> seq=<request>` for every token chosen: k counts the
request's tokens from 0, the hash is over the float32 logits the token was chosen from
(`Engine.logit_hash`).  Two runs that should agree are compared by these files, and the first line that
differs names the step to look at.  Tracing runs the loop unpipelined.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Union

import torch

from ..sampling.params import SamplingParams
from ..sampling.rng import entropy_seed

from ..cache import PAGE_SIZE as PAGE     # a sequence's tokens are counted in units of the cache's page


@dataclass
class Completion:
    tokens: List[int]
    finish_reason: str            # "stop" or "length"
    prompt_tokens: int


@dataclass
class GenerationStats:
    prompt_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_tokens: int = 0
    decode_seconds: float = 0.0
    batches: int = 0
    steps: int = 0

    def pptg_line(self) -> str:
        """The reference's timing line (generate.rs:427-433)."""
        pp = self.prompt_tokens / self.prefill_seconds if self.prefill_seconds > 0 else 0.0
        tg = self.decode_tokens / self.decode_seconds if self.decode_seconds > 0 else 0.0
        return (f"PPTG pp={pp:.1f} tok/s ({self.prompt_tokens} prompt tok / {self.prefill_seconds:.3f}s) "
                f"tg={tg:.1f} tok/s ({self.decode_tokens} tok / {self.decode_seconds:.3f}s)")


def plan_batches(prompt_lens: Sequence[int], max_new_tokens: Sequence[int], capacity_tokens: int,
                 max_batch: int) -> List[List[int]]:
    """Cut requests, in order, into batches that fit: at most `max_batch` sequences, and
    the sum over the batch of (prompt + new tokens, rounded up to a page) within the
    cache's capacity.  A request that cannot fit alone is an error."""
    if max_batch < 1:
        raise ValueError("max_batch must be at least 1")
    batches: List[List[int]] = []
    cur: List[int] = []
    used = 0
    for i, (p, m) in enumerate(zip(prompt_lens, max_new_tokens)):
        need = -(-(p + m) // PAGE) * PAGE
        if need > capacity_tokens:
            raise ValueError(f"request {i} needs room for {p + m} tokens ({need} with page rounding); "
                             f"the cache holds {capacity_tokens}")
        if cur and (len(cur) >= max_batch or used + need > capacity_tokens):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


class GenerationLoop:
    def __init__(self, engine, sampler, max_batch: int = 64, pipeline: bool = True,
                 logit_trace: Optional[str] = None) -> None:
        self._logit_trace_arg = logit_trace       # None: ask the environment at every call of generate
        self.logit_trace: Optional[str] = logit_trace
        self.engine = engine
        self.sampler = sampler
        self.max_batch = max_batch
        self.pipeline = pipeline
        self.stats = GenerationStats()

    def generate(self, prompts: Sequence[Sequence[int]],
                 params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 max_new_tokens: Union[int, Sequence[int]] = 64,
                 stop_tokens: Sequence[int] = ()) -> List[Completion]:
        n = len(prompts)
        self.logit_trace = (self._logit_trace_arg if self._logit_trace_arg is not None
                            else (os.environ.get("BRAIDINFER_LOGIT_TRACE") or None))
        if params is None:
            params = SamplingParams.greedy()
        plist = [params] * n if isinstance(params, SamplingParams) else list(params)
        mlist = [int(max_new_tokens)] * n if isinstance(max_new_tokens, int) else [int(m) for m in max_new_tokens]
        if len(plist) != n or len(mlist) != n:
            raise ValueError("params and max_new_tokens must be single values or one per prompt")
        for i, p in enumerate(prompts):
            if len(p) == 0:
                raise ValueError(f"prompt {i} is empty; a sequence needs at least one token")
        seeds = [p.seed if p.seed is not None else entropy_seed() for p in plist]
        stop = frozenset(int(t) for t in stop_tokens)
        results: List[Optional[Completion]] = [None] * n
        todo = []
        for i in range(n):
            if mlist[i] <= 0:
                results[i] = Completion([], "length", len(prompts[i]))
            else:
                todo.append(i)
        capacity = getattr(self.engine, "max_tokens")
        batches = plan_batches([len(prompts[i]) for i in todo], [mlist[i] for i in todo], capacity,
                               min(self.max_batch, getattr(self.engine, "max_slots", self.max_batch)))
        pipelined = (self.pipeline and not self.logit_trace and hasattr(self.sampler, "choose_async")
                     and all(p.repetition_penalty == 1.0 for p in plist))
        for b in batches:
            run = self._run_batch_pipelined if pipelined else self._run_batch
            run([todo[j] for j in b], prompts, plist, seeds, mlist, stop, results)
        return results   # type: ignore[return-value]

    def _run_batch_pipelined(self, ids, prompts, plist, seeds, mlist, stop, results) -> None:
        """The same decisions as `_run_batch`, with the host off the critical path: the
        tokens a step chose stay on the device and feed the next step at once, while their
        copy to the host (for stop tokens and the results) overlaps that step.  A sequence
        that turns out to have stopped has then run one step too many; its result is
        dropped and its slot freed.  Sequences known to end by length are not continued."""
        eng, smp = self.engine, self.sampler
        self.stats.batches += 1
        slots = {i: eng.open() for i in ids}
        generated = {i: [] for i in ids}
        try:
            live = list(ids)
            t0 = time.perf_counter()
            logits = eng.step([(slots[i], list(prompts[i])) for i in live], want="last")
            pending = smp.choose_async(logits, [plist[i] for i in live], [seeds[i] for i in live], live,
                                       [0] * len(live))
            first = True
            while live:
                cont = [i for i in live if len(generated[i]) + 1 < mlist[i]]       # may go on after this token
                nxt_logits = None
                if cont:
                    rows = [live.index(i) for i in cont]
                    nxt_logits = eng.step([(slots[i], [0]) for i in cont], want="last",
                                          device_tokens=(pending.device, rows))
                toks = pending.read()
                now = time.perf_counter()
                self.stats.steps += 1
                if first:
                    self.stats.prefill_seconds += now - t0
                    self.stats.prompt_tokens += sum(len(prompts[i]) for i in live)
                    first = False
                else:
                    self.stats.decode_seconds += now - t0
                    self.stats.decode_tokens += len(live)
                t0 = now
                survivors = []
                for i, tok in zip(live, toks):
                    if tok in stop:
                        results[i] = Completion(generated[i], "stop", len(prompts[i]))
                    else:
                        generated[i].append(tok)
                        if len(generated[i]) >= mlist[i]:
                            results[i] = Completion(generated[i], "length", len(prompts[i]))
                    if results[i] is not None:
                        eng.close(slots.pop(i))
                    else:
                        survivors.append(i)
                if survivors:
                    if survivors != cont:              # some stopped: keep the rows of those that go on
                        keep = torch.tensor([cont.index(i) for i in survivors], device=nxt_logits.device)
                        nxt_logits = nxt_logits.index_select(0, keep)
                    pending = smp.choose_async(nxt_logits, [plist[i] for i in survivors],
                                               [seeds[i] for i in survivors], survivors,
                                               [len(generated[i]) for i in survivors])
                live = survivors
            check = getattr(eng, "check", None)
            if check is not None:
                check()
        finally:
            for s in slots.values():
                eng.close(s)

    def _trace_logits(self, ids, steps, toks, logits) -> None:
        hashes = self.engine.logit_hash(logits)
        with open(self.logit_trace, "a") as f:
            for i, k, tok, h in zip(ids, steps, toks, hashes):
                f.write(f"step={k} tok={int(tok)} logit_hash={h:016x} seq={i}\n")

    def _run_batch(self, ids, prompts, plist, seeds, mlist, stop, results) -> None:
        eng = self.engine
        self.stats.batches += 1
        slots = {i: eng.open() for i in ids}
        generated = {i: [] for i in ids}
        try:
            live = list(ids)
            t0 = time.perf_counter()
            logits = eng.step([(slots[i], list(prompts[i])) for i in live], want="last")
            first = True
            while live:
                now_live = list(live)
                toks = self.sampler.choose(logits, [plist[i] for i in live], [seeds[i] for i in live],
                                           live, [len(generated[i]) for i in live],
                                           lambda: [list(prompts[i]) + generated[i] for i in now_live])
                if self.logit_trace:
                    self._trace_logits(live, [len(generated[i]) for i in live], toks, logits)
                now = time.perf_counter()
                self.stats.steps += 1
                if first:
                    self.stats.prefill_seconds += now - t0
                    self.stats.prompt_tokens += sum(len(prompts[i]) for i in live)
                    first = False
                else:
                    self.stats.decode_seconds += now - t0
                    self.stats.decode_tokens += len(live)
                t0 = now
                nxt, entries = [], []
                for i, tok in zip(live, toks):
                    if tok in stop:
                        results[i] = Completion(generated[i], "stop", len(prompts[i]))
                    else:
                        generated[i].append(tok)
                        if len(generated[i]) >= mlist[i]:
                            results[i] = Completion(generated[i], "length", len(prompts[i]))
                    if results[i] is not None:
                        eng.close(slots.pop(i))          # the slot and its pages go back at once
                    else:
                        nxt.append(i)
                        entries.append((slots[i], [tok]))
                live = nxt
                if live:
                    logits = eng.step(entries, want="last")
            check = getattr(eng, "check", None)
            if check is not None:
                check()                                    # sticky device error flags, once per batch
        finally:
            for s in slots.values():                       # only on an error: nothing stays held
                eng.close(s)
