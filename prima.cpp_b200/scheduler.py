"""Batch scheduler over the engine's sequence slots and ragged batch step (``pb200_batch_step``).

Static batching: the waiting requests that fit (free slots, token budget) start together as one prompt batch and are then decoded
together, one token per step; a request that finishes leaves the batch and gives its slot back, nobody joins a running batch.
``step()`` is the primitive both ``generate()`` and a replayed trace use: it maps request ids to sequence slots, runs one batch step
and releases the slots of finished requests.
"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class Request:
    rid: object
    prompt: list
    max_new_tokens: int
    eos: int | None = None
    out: list = field(default_factory=list)
    done: bool = False


class BatchScheduler:
    def __init__(self, model, max_batch: int | None = None, max_tokens: int | None = None):
        self.model = model
        self.max_batch = min(max_batch or model.n_seq, model.n_seq)
        self.max_tokens = max_tokens          # most tokens the live requests may hold (None: no budget)
        self.slots: dict = {}                 # request id -> sequence slot
        self.waiting: list[Request] = []
        self._next_id = 0

    # ---- the primitive ----
    def step(self, entries, end=(), greedy: bool = False):
        """entries: [(request id, tokens, want)].  A request id seen for the first time gets a fresh slot.  Requests listed in ``end``
        give their slot back after the step.  Returns (logits rows, greedy tokens or None) like ``Model.batch_step``."""
        batch = []
        for rid, tokens, want in entries:
            if rid not in self.slots:
                self.slots[rid] = self.model.seq_alloc()
            batch.append((self.slots[rid], tokens, want))
        try:
            out = self.model.batch_step(batch, greedy=greedy) if batch else (None, None)
        finally:
            for rid in end:
                slot = self.slots.pop(rid, None)
                if slot is not None:
                    self.model.seq_free(slot)
        return out

    def live_tokens(self) -> int:
        return sum(self.model.seq_length(s) for s in self.slots.values())

    # ---- generation ----
    def submit(self, prompt, max_new_tokens: int, eos: int | None = None, rid=None) -> Request:
        if rid is None:
            rid = ("req", self._next_id)
            self._next_id += 1
        r = Request(rid, list(prompt), int(max_new_tokens), eos)
        self.waiting.append(r)
        return r

    def _admit(self) -> list[Request]:
        batch, budget = [], self.max_tokens
        while self.waiting and len(batch) < self.max_batch:
            r = self.waiting[0]
            need = len(r.prompt) + r.max_new_tokens
            if budget is not None and need > budget and batch:
                break
            if budget is not None:
                budget -= need
            batch.append(self.waiting.pop(0))
        return batch

    def run(self) -> None:
        """Runs every submitted request to completion (greedy sampling on the device)."""
        while self.waiting:
            batch = self._admit()
            live = [r for r in batch if r.max_new_tokens > 0 and r.prompt]
            for r in batch:
                if r not in live:
                    r.done = True
            if not live:
                continue
            feed = {r.rid: r.prompt for r in live}
            while live:
                ending = []
                for r in live:          # a request ends with this step if the token the step yields is its last one
                    if len(r.out) + 1 >= r.max_new_tokens:
                        ending.append(r.rid)
                _, toks = self.step([(r.rid, feed[r.rid], []) for r in live], end=[], greedy=True)
                nxt = []
                for r, t in zip(live, toks):
                    r.out.append(int(t))
                    if r.rid in ending or (r.eos is not None and t == r.eos):
                        r.done = True
                        slot = self.slots.pop(r.rid, None)
                        if slot is not None:
                            self.model.seq_free(slot)
                    else:
                        feed[r.rid] = [int(t)]
                        nxt.append(r)
                live = nxt

    def generate(self, prompts, max_new_tokens: int, eos: int | None = None) -> list[list]:
        reqs = [self.submit(p, max_new_tokens, eos) for p in prompts]
        self.run()
        return [r.out for r in reqs]
