"""Continuous batching above the step function.

Policy, after the reference's scheduler (sched/Scheduler.cajeta:414-605):

* states WAITING -> RUNNING -> DONE and RUNNING <-> PREEMPTED; finish reasons
  NONE / BUDGET / EOS / STOP / CANCEL (sched/Request.cajeta:11-23);
* admission at the start and at the end of every iteration: preempted requests first
  (oldest preemption first), then waiters in submission order; a request needs a free
  slot and pages for its whole uncached suffix plus one page of decode headroom per
  cache group (in a windowed group: for no more than the window plus one step's tokens,
  since such a group gives pages back as the request goes on), counted against the free
  pages that running requests have not yet claimed for their own prompts; admission stops at the first request that does not
  fit, nothing is skipped (sched/Scheduler.cajeta:1068-1151);
* every iteration is ONE mixed step under a token budget: the single decode tokens of
  all running requests first, then prompt portions in admission order until the budget
  is used; ``chunk`` > 0 also caps a portion (the reference gives each running request
  one item of at most ``chunk`` tokens per iteration and runs them as separate model
  calls, sched/Scheduler.cajeta:472-560);
* when the pages for an item are not there, the YOUNGEST running request (latest
  admission) is preempted: its pages are given back, it forgets what it had cached
  and is later re-admitted ahead of new work and recomputed from its tokens (prompt
  plus generated) through the same chunked path; if the youngest is the request
  itself, it yields; if nothing can be preempted the request can never fit and the
  scheduler raises (sched/Scheduler.cajeta:495-509,1263-1315);
* a request finishes on a stop token (by default the engine's end-of-generation set)
  -> EOS, or when it has generated ``max_new_tokens`` -> BUDGET; its slot and pages are
  free for a request admitted in the same iteration (sched/Scheduler.cajeta:732-757,575).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

from ..sampling.params import SamplingParams
from ..sampling.sampler import Xorshift64
from .step import OutOfPages, StepEntry


class RequestState(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    PREEMPTED = "preempted"
    DONE = "done"


class FinishReason(enum.Enum):
    NONE = "none"
    BUDGET = "budget"
    EOS = "eos"
    STOP = "stop"
    CANCEL = "cancel"


class SchedulerError(RuntimeError):
    pass


@dataclass
class Request:
    id: int
    prompt: List[int]
    params: SamplingParams
    stop_tokens: Tuple[int, ...]
    generated: List[int] = field(default_factory=list)
    state: RequestState = RequestState.WAITING
    finish_reason: FinishReason = FinishReason.NONE
    slot: Optional[int] = None
    cached_len: int = 0
    admit_stamp: int = -1
    preempt_stamp: int = -1
    rng: Optional[Xorshift64] = None

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.generated

    @property
    def total_len(self) -> int:
        return len(self.prompt) + len(self.generated)

    @property
    def is_done(self) -> bool:
        return self.state == RequestState.DONE

    def generated_count(self) -> int:
        return len(self.generated)


@dataclass
class Counters:
    admitted: int = 0
    preempted: int = 0
    resumed: int = 0
    steps: int = 0
    recomputed_tokens: int = 0
    prefill_rows: int = 0
    decode_rows: int = 0


class Scheduler:
    def __init__(self, runner, sampler, max_batch_tokens: int = 2048, chunk: int = 0,
                 eog_token_ids: Sequence[int] = (), lookahead: bool = True):
        """``runner`` offers admit / release / step and a ``cache`` with pages_needed,
        free_pages and length; ``sampler.sample(logits, params, rngs, histories)`` returns
        one token per row."""
        if max_batch_tokens < 1:
            raise SchedulerError(f"max_batch_tokens must be >= 1, found {max_batch_tokens}")
        self.runner = runner
        self.sampler = sampler
        self.max_batch_tokens = max_batch_tokens
        self.chunk = chunk
        self.eog_token_ids = tuple(eog_token_ids)
        self.lookahead = lookahead
        self.requests: Dict[int, Request] = {}
        self.waiting: List[Request] = []
        self.preempted: List[Request] = []
        self.running: List[Request] = []
        self.counters = Counters()
        self.sink: Optional[Callable[[int, int], None]] = None
        self._next_id = 0
        self._stamp = 0

    # -- submission ------------------------------------------------------------------
    def submit(self, prompt: Sequence[int], params: SamplingParams) -> int:
        if len(prompt) == 0:
            raise SchedulerError("a request needs at least one prompt token")
        stops = params.stop_token_ids if params.stop_token_ids is not None else self.eog_token_ids
        r = Request(id=self._next_id, prompt=[int(t) for t in prompt], params=params, stop_tokens=tuple(stops),
                    rng=Xorshift64(params.seed))
        self._next_id += 1
        self.requests[r.id] = r
        self.waiting.append(r)
        return r.id

    def request(self, request_id: int) -> Request:
        return self.requests[request_id]

    def cancel(self, request_id: int) -> bool:
        """Between steps; False when the request is done or unknown (sched/Scheduler.cajeta:293-313)."""
        r = self.requests.get(request_id)
        if r is None or r.state == RequestState.DONE:
            return False
        if r.state == RequestState.RUNNING:
            self.runner.release(r.slot)
            self.running.remove(r)
        elif r.state == RequestState.WAITING:
            self.waiting.remove(r)
        else:
            self.preempted.remove(r)
        self._finish(r, FinishReason.CANCEL, release=False)
        return True

    @property
    def has_work(self) -> bool:
        return bool(self.waiting or self.preempted or self.running)

    # -- admission -------------------------------------------------------------------
    def _claimed(self) -> List[int]:
        """Pages per group that running requests still need for their known tokens."""
        cache = self.runner.cache
        total = [0] * len(cache.free_pages())
        for r in self.running:
            need = cache.pages_to_hold(r.slot, r.total_len - r.cached_len, self._step_tokens())
            total = [a + b for a, b in zip(total, need)]
        return total

    def _step_tokens(self) -> int:
        """The most tokens one request brings in one step (what a windowed cache group is sized by)."""
        return min(self.max_batch_tokens, self.chunk) if self.chunk > 0 else self.max_batch_tokens

    def _admit_phase(self) -> None:
        cache = self.runner.cache
        while True:
            queue = self.preempted if self.preempted else self.waiting
            if not queue:
                return
            r = queue[0]
            slot = self.runner.admit()
            if slot is None:
                return
            need = cache.pages_to_hold(slot, r.total_len, self._step_tokens())
            free = cache.free_pages()
            claimed = self._claimed()
            fits = all(n + 1 + c <= f for n, c, f in zip(need, claimed, free))
            if not fits:
                self.runner.release(slot)
                if not self.running:
                    # nothing runs, so every page is free: the request can never fit
                    queue.pop(0)
                    self._finish(r, FinishReason.CANCEL, release=False)
                    raise SchedulerError(
                        f"request {r.id} holds {r.total_len} tokens and can never fit the cache pool "
                        f"({cache.free_pages()} free pages per group with nothing else running)")
                return
            queue.pop(0)
            r.slot = slot
            r.cached_len = 0
            r.admit_stamp = self._stamp
            self._stamp += 1
            if r.state == RequestState.PREEMPTED:
                self.counters.resumed += 1
            self.counters.admitted += 1
            r.state = RequestState.RUNNING
            self.running.append(r)

    # -- one iteration ---------------------------------------------------------------
    def plan_step(self) -> List[Tuple[Request, int]]:
        """(request, number of its next tokens) for this iteration: decode tokens first,
        then prompt portions in admission order under the token budget; preempts the
        youngest running request while the plan's pages are not there."""
        cache = self.runner.cache
        order = sorted(self.running, key=lambda r: r.admit_stamp)
        decodes = [r for r in order if r.total_len - r.cached_len == 1]
        prompts = [r for r in order if r.total_len - r.cached_len > 1]
        plan: List[Tuple[Request, int]] = []
        budget = self.max_batch_tokens
        for r in decodes:
            if budget < 1:
                break
            plan.append((r, 1))
            budget -= 1
        for r in prompts:
            if budget < 1:
                break
            n = min(r.total_len - r.cached_len, budget)
            if self.chunk > 0:
                n = min(n, self.chunk)
            plan.append((r, n))
            budget -= n
        # pages: walk the plan in order; when the pages run out preempt the youngest
        while True:
            free = cache.free_pages()
            used = [0] * len(free)
            short_at = None
            for i, (r, n) in enumerate(plan):
                need = cache.pages_needed(r.slot, n)
                used = [a + b for a, b in zip(used, need)]
                if any(u > f for u, f in zip(used, free)):
                    short_at = i
                    break
            if short_at is None:
                return plan
            victim = max(self.running, key=lambda r: r.admit_stamp)
            blocked = plan[short_at][0]
            if victim is blocked and len(self.running) == 1:
                raise SchedulerError(
                    f"request {blocked.id} needs more pages than the pool holds even alone "
                    f"({cache.pages_needed(blocked.slot, plan[short_at][1])} new, {free} free)")
            self._preempt(victim)
            plan = [(r, n) for r, n in plan if r is not victim]

    def _preempt(self, r: Request) -> None:
        self.runner.release(r.slot)
        self.running.remove(r)
        self.counters.preempted += 1
        self.counters.recomputed_tokens += r.cached_len
        r.slot = None
        r.cached_len = 0
        r.state = RequestState.PREEMPTED
        r.preempt_stamp = self._stamp
        self._stamp += 1
        self.preempted.append(r)
        self.preempted.sort(key=lambda q: q.preempt_stamp)

    def step_once(self) -> int:
        """One iteration; returns the number of tokens it ran."""
        self._admit_phase()
        if not self.running:
            if self.has_work:
                raise SchedulerError("requests are waiting but none can be admitted")
            return 0
        plan = self.plan_step()
        if not plan:
            return 0
        entries, finishing = [], []
        for r, n in plan:
            toks = r.tokens[r.cached_len: r.cached_len + n]
            completes = r.cached_len + n == r.total_len
            entries.append(StepEntry(slot=r.slot, tokens=toks, want=[n - 1] if completes else []))
            if completes:
                finishing.append(r)
            if n == 1 and completes and r.generated:
                self.counters.decode_rows += 1
            else:
                self.counters.prefill_rows += n
        logits = self.runner.step(entries)
        for r, n in plan:
            r.cached_len += n
        self.counters.steps += 1
        if finishing:
            tokens = self.sampler.sample(logits, [r.params for r in finishing], [r.rng for r in finishing],
                                         [r.generated for r in finishing])
            for r, tok in zip(finishing, tokens):
                self._consume(r, int(tok))
        self._admit_phase()
        return sum(n for _, n in plan)

    def _consume(self, r: Request, token: int) -> None:
        r.generated.append(token)
        if self.sink is not None:
            self.sink(r.id, token)
        if token in r.stop_tokens:
            self._finish(r, FinishReason.EOS)
        elif len(r.generated) >= r.params.max_new_tokens:
            self._finish(r, FinishReason.BUDGET)

    def _finish(self, r: Request, reason: FinishReason, release: bool = True) -> None:
        if release and r.slot is not None:
            self.runner.release(r.slot)
            self.running.remove(r)
        r.slot = None
        r.state = RequestState.DONE
        r.finish_reason = reason

    def run_all(self, max_steps: int = 0) -> int:
        """Iterate until nothing is left (or ``max_steps`` iterations, 0 = no limit)."""
        steps = 0
        while self.has_work and (max_steps <= 0 or steps < max_steps):
            if self._can_run_ahead():
                steps += self._run_ahead(max_steps - steps if max_steps > 0 else 0)
            else:
                self.step_once()
                steps += 1
        return steps

    # -- decoding one step ahead of the host -------------------------------------------------
    # While every running request is decoding and nothing waits, the host has nothing to decide
    # between two steps except whether a request has ended.  The next step is then launched
    # BEFORE the host has seen the tokens of the one in flight: the sampler leaves them on the
    # device and the next step reads them there, so the device never waits for the host's
    # bookkeeping.  A request that turns out to have ended (a stop token) has ridden along for
    # one step too many; its row of that step is dropped.  Ends that can be foreseen (the
    # budget) are: a request is only taken along while it has two tokens of budget left.
    # Not used while a sink wants every token before the next step, nor with a repetition
    # penalty (the sampler would need the token the host has not seen).
    def _can_run_ahead(self) -> bool:
        if not self.lookahead or self.sink is not None or self.waiting or self.preempted or not self.running:
            return False
        if not hasattr(self.runner, "step_chained") or not hasattr(self.sampler, "sample_device"):
            return False
        if len(self.running) > self.max_batch_tokens:
            return False
        for r in self.running:
            if r.total_len - r.cached_len != 1 or r.params.repeat_penalty != 1.0:
                return False
            if len(r.generated) + 2 > r.params.max_new_tokens:
                return False
        return True

    def _run_ahead(self, max_steps: int = 0) -> int:
        """Steps while the condition above holds; returns how many it ran (at least one)."""
        import torch
        reqs = sorted(self.running, key=lambda r: r.admit_stamp)
        slots = [r.slot for r in reqs]
        params, rngs = [r.params for r in reqs], [r.rng for r in reqs]
        n = len(reqs)
        try:
            logits = self.runner.step([StepEntry(slot=r.slot, tokens=[r.tokens[-1]], want=[0]) for r in reqs])
        except OutOfPages:
            self.step_once()               # the ordinary iteration decides whom to preempt
            return 1
        steps = 1
        for r in reqs:
            r.cached_len += 1
        self.counters.steps += 1
        self.counters.decode_rows += n
        dev = self.sampler.sample_device(logits, params, rngs, [r.generated for r in reqs])
        bufs = [torch.empty((n,), dtype=torch.int32, pin_memory=True) for _ in range(2)]
        events = [torch.cuda.Event(), torch.cuda.Event()]
        cur = 0
        bufs[cur].copy_(dev, non_blocking=True)
        events[cur].record()
        while True:
            # the step after the one in flight, launched before its tokens are known here
            ahead = None
            surely = all(len(r.generated) + 2 <= r.params.max_new_tokens for r in reqs)
            if surely and (max_steps <= 0 or steps < max_steps):
                try:
                    ahead = self.runner.step_chained(slots, dev)
                except OutOfPages:
                    ahead = None
            if ahead is not None:
                dev = self.sampler.sample_device(ahead, params, rngs, [r.generated for r in reqs])
                bufs[cur ^ 1].copy_(dev, non_blocking=True)
                events[cur ^ 1].record()
            # now the tokens of the step in flight
            events[cur].synchronize()
            tokens = bufs[cur].tolist()
            for r, tok in zip(reqs, tokens):
                self._consume(r, int(tok))
            ended = [r.state == RequestState.DONE for r in reqs]
            if ahead is None:
                return steps
            steps += 1
            self.counters.steps += 1
            self.counters.decode_rows += n - sum(ended)
            for r, e in zip(reqs, ended):
                if not e:
                    r.cached_len += 1
            cur ^= 1
            if any(ended):
                # the step ahead carried rows of requests that had ended: drop those rows, take the rest
                events[cur].synchronize()
                for r, e, tok in zip(reqs, ended, bufs[cur].tolist()):
                    if not e:
                        self._consume(r, int(tok))
                return steps
