"""The scheduler: admission, portions under a token budget, decoding, finishing.

Host-side decisions only; it talks to the cache manager for pages and slots and
hands the step function a list of (request, next tokens).  Compared with the
reference's loop (fastgen/generate.py:427-613, 898-932):

* the reference prefills admitted prompts whole, in calls separate from
  decoding; here every step may mix prompt portions with the single tokens of
  decoding requests, under one token budget (``max_prefill``);
* admission takes the pages of the whole prompt plus one token up front (the
  reference asks for the prompt plus 128 tokens, generate.py:535-536,562), in
  arrival order, preempted requests first (generate.py:543-544); it stops at
  the first request that does not fit;
* when a decoding request needs a page and none is free, the most recently
  admitted request is preempted: its pages and slot are given back and it
  waits at the head of the queue, to be recomputed from its prompt and the
  tokens it already produced (generate.py:497-507, 772).  A request that is
  alone is capped at what the empty cache holds, so it never runs out;
* a request that could never fit an empty cache is finished at once with an
  error instead of waiting forever (the reference would spin on it).
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Any, Deque, List, Optional, Sequence

from ..cache import CacheManager, OutOfPages


@dataclass(eq=False)
class Request:
    """A request in flight (compared and hashed by identity)."""

    thread_id: Any
    prompt: List[int]
    key: int  # what the sampler's draws are keyed by (admission-independent)
    temperature: float = 0.0
    max_gen: Optional[int] = None
    maxlen: int = 0
    generated: List[int] = field(default_factory=list)
    logprobs: List[float] = field(default_factory=list)
    fed: int = 0  # tokens of prompt+generated whose keys/values are cached
    error: Optional[str] = None
    preemptions: int = 0

    def all_tokens(self) -> List[int]:
        return self.prompt + self.generated

    def tokens_between(self, a: int, b: int) -> List[int]:
        """Tokens ``a .. b-1`` of prompt + generated, without joining the two lists."""
        n = len(self.prompt)
        if b <= n:
            return self.prompt[a:b]
        if a >= n:
            return self.generated[a - n : b - n]
        return self.prompt[a:] + self.generated[: b - n]

    def __len__(self) -> int:
        return len(self.prompt) + len(self.generated)


@dataclass
class PlanEntry:
    request: Request
    tokens: List[int]
    samples: bool  # the last of these tokens is the request's last: sample after it


class Scheduler:
    def __init__(
        self,
        cache: CacheManager,
        max_batch: int,
        token_budget: int,
        stop_tokens: Sequence[int] = (),
        max_gen: Optional[int] = None,
        min_prefill: int = 0,
        min_prefill_batch: int = 1,
    ) -> None:
        if token_budget < 1:
            raise ValueError("the token budget of a step must be at least 1")
        self.cache = cache
        self.max_batch = min(max_batch, cache.max_requests)
        self.token_budget = token_budget
        self.stop_tokens = set(stop_tokens)
        self.default_max_gen = max_gen
        self.capacity = min(
            [cache.max_length] + [g.pool.n_pages * g.page_size for g in cache.groups]
        )
        # the reference's rule for batching prompts (generate.py:600-608): while requests are
        # decoding and more input may come, fewer than ``min_prefill_batch`` newly admitted
        # requests with fewer than ``min_prefill`` tokens together wait for company
        self.min_prefill = min_prefill
        self.min_prefill_batch = min_prefill_batch
        self.input_ended = False  # set by the caller once no more requests will be added
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []  # in admission order
        self.finished: List[Request] = []
        self._next_key = 0
        self.n_preemptions = 0

    # -- input -----------------------------------------------------------------
    def add(self, thread_id, prompt: Sequence[int], temperature: float = 0.0,
            max_gen: Optional[int] = None) -> Request:
        max_gen = max_gen or self.default_max_gen
        req = Request(thread_id, list(prompt), self._next_key, temperature, max_gen)
        self._next_key += 1
        if not req.prompt:
            req.error = "empty prompt"
        elif len(req.prompt) + 1 > self.capacity:
            req.error = (
                f"a prompt of {len(req.prompt)} tokens can never fit: the cache holds "
                f"{self.capacity} tokens per request"
            )
        if req.error:
            self.finished.append(req)
            return req
        limit = self.capacity
        if max_gen is not None:
            limit = min(limit, len(req.prompt) + max_gen)
        req.maxlen = limit
        self.waiting.append(req)
        return req

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # -- decisions ---------------------------------------------------------------
    def _admit(self) -> None:
        n_before = len(self.running)
        self._admit_all()
        new = self.running[n_before:]
        if (new and n_before > 0 and not self.input_ended and len(new) < self.min_prefill_batch
                and sum(len(r) for r in new) < self.min_prefill):
            # wait some more before prefilling: give slots and pages back, keep the order
            for req in reversed(new):
                self.cache.release(id(req))
                self.waiting.appendleft(req)
            del self.running[n_before:]

    def _admit_all(self) -> None:
        while self.waiting and len(self.running) < self.max_batch:
            req = self.waiting[0]
            if self.cache.free_slots() == 0:
                break
            handle = self.cache.admit(id(req))
            try:
                self.cache.reserve(handle, len(req) + 1 if len(req) < req.maxlen else len(req))
            except OutOfPages:
                self.cache.release(id(req))
                break
            self.waiting.popleft()
            req.fed = 0
            self.running.append(req)

    def _preempt(self, req: Request) -> None:
        self.cache.release(id(req))
        self.running.remove(req)
        req.fed = 0
        req.preemptions += 1
        self.n_preemptions += 1
        self.waiting.appendleft(req)

    def plan(self) -> List[PlanEntry]:
        """Decide the next step.  Decoding requests first (one token each), then
        prompt portions in admission order, all within the token budget."""
        self._admit()
        entries: List[PlanEntry] = []
        budget = self.token_budget
        order = sorted(self.running, key=lambda r: (len(r) - r.fed != 1,))  # stable: decoders first
        preempted = set()
        for req in order:
            if req in preempted:
                continue  # preempted while planning
            if budget == 0:
                break
            remaining = len(req) - req.fed
            n = min(remaining, budget)
            handle = self.cache.get(id(req))
            while True:
                try:
                    self.cache.reserve(handle, req.fed + n)
                    break
                except OutOfPages:
                    victim = self.running[-1]
                    planned = [e for e in entries if e.request is victim]
                    for e in planned:
                        entries.remove(e)
                        budget += len(e.tokens)
                    self._preempt(victim)
                    preempted.add(victim)
                    if victim is req:
                        n = 0
                        break
            if n == 0:
                continue
            toks = req.tokens_between(req.fed, req.fed + n)
            entries.append(PlanEntry(req, toks, samples=(req.fed + n == len(req))))
            budget -= n
        return entries

    def plan_decode_run(self, max_steps: int) -> int:
        """How many decode steps may run back to back without the host looking at the
        tokens in between (the reference's ``sync_freq``, generate.py:692-699): more than
        one only when every running request is decoding, nothing waits for admission,
        nobody reaches its length limit inside the run and the pages for the whole run
        can be reserved now.  Returns 1 when the ordinary one-step path should be taken."""
        if max_steps <= 1 or not self.running or self.waiting:
            return 1
        n = max_steps
        for req in self.running:
            if len(req) - req.fed != 1:
                return 1
            n = min(n, req.maxlen - len(req))
            if req.max_gen is not None:
                n = min(n, req.max_gen - len(req.generated))
        if n <= 1:
            return 1
        free = self.cache.free_pages()
        total = [0] * len(free)
        handles = []
        for req in self.running:
            handle = self.cache.get(id(req))
            handles.append(handle)
            for gi, need in enumerate(self.cache.pages_needed(handle, req.fed + n)):
                total[gi] += need
        if any(t > f for t, f in zip(total, free)):
            return 1  # not enough pages for the whole run: the one-step path decides (and preempts)
        for req, handle in zip(self.running, handles):
            self.cache.reserve(handle, req.fed + n)
        return n

    def commit_decode_run(self, requests: Sequence[Request], sampled: Sequence[Sequence[int]],
                          logprobs: Optional[Sequence[Sequence[float]]] = None) -> List[Request]:
        """Record a run of ``len(sampled)`` decode steps: ``sampled[k][i]`` is the token
        request ``i`` drew at step ``k``.  A request's tokens are cut after its first stop
        token (what it decoded after that is dropped, generate.py:647-662)."""
        n = len(sampled)
        done: List[Request] = []
        for i, req in enumerate(requests):
            handle = self.cache.get(id(req))
            self.cache.advance(handle, req.fed + n)
            req.fed += n
            ended = False
            for k in range(n):
                tok = int(sampled[k][i])
                req.generated.append(tok)
                if logprobs is not None:
                    req.logprobs.append(float(logprobs[k][i]))
                if tok in self.stop_tokens or len(req) >= req.maxlen or (
                        req.max_gen is not None and len(req.generated) >= req.max_gen):
                    ended = True
                    break
            if ended:
                self.cache.release(id(req))
                self.running.remove(req)
                done.append(req)
        return done

    def commit(self, entries: Sequence[PlanEntry], sampled: Sequence[int],
               logprobs: Optional[Sequence[float]] = None) -> List[Request]:
        """Record a step's outcome.  ``sampled`` holds one token per entry that
        samples, in order.  Returns the requests that finished."""
        done: List[Request] = []
        it = iter(range(len(sampled)))
        for e in entries:
            req = e.request
            handle = self.cache.get(id(req))
            self.cache.advance(handle, req.fed + len(e.tokens))
            req.fed += len(e.tokens)
            if not e.samples:
                continue
            i = next(it)
            tok = int(sampled[i])
            req.generated.append(tok)
            if logprobs is not None:
                req.logprobs.append(float(logprobs[i]))
            ended = tok in self.stop_tokens or len(req) >= req.maxlen
            if req.max_gen is not None and len(req.generated) >= req.max_gen:
                ended = True
            if ended:
                self.cache.release(id(req))
                self.running.remove(req)
                done.append(req)
        return done

    def fail(self, requests: Sequence[Request], message: str) -> List[Request]:
        """End running requests with an error (a kernel of their step recorded a fault, so
        what the step computed for them cannot be trusted): pages and slots are given back."""
        done: List[Request] = []
        for req in requests:
            if req not in self.running:
                continue
            self.cache.release(id(req))
            self.running.remove(req)
            req.error = message
            done.append(req)
        return done

    def take_finished(self) -> List[Request]:
        out, self.finished = self.finished, []
        return out
