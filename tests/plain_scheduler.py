"""A plain restatement of the scheduling policy, for tests: which tokens of which request every step runs.

It shares no code with the engine's scheduler (the native `Sched` of stride_b200/csrc/runtime.cpp); it keeps its own
count of pages. The policy is arhaamatiq/stride's (src/scheduler.cpp:72-304):

* intake (src/scheduler.cpp:82-89): an empty prompt, or one that leaves no room in the context, ends at once; the
  number of new tokens is cut to the room left;
* admission (src/scheduler.cpp:95-118): in arrival order, while fewer than max_seqs run and a slot is free; beside
  running requests only if the free pages cover the request's tokens plus one page of growth for each running request
  plus one;
* the batch (src/scheduler.cpp:120-190): every running request with exactly one unprocessed token, one row each, in
  running order; then portions of at most prefill_chunk tokens of the others, in running order; all under max_rows;
* pages short (src/scheduler.cpp:160-178): the youngest running request gives its pages back, returns to the front of
  the queue and starts again from its first token (prompt and generated tokens alike); one request alone that does
  not fit is an error;
* after the step: a chosen token ends its request if it is a stop token or the limit is reached.
"""
from __future__ import annotations


class PlainScheduler:
    def __init__(self, *, pages: int, page_size: int, max_slots: int, max_context: int, max_seqs: int, max_rows: int,
                 prefill_chunk: int):
        self.free_pages, self.page, self.free_slots = pages, page_size, max_slots
        self.max_context, self.max_seqs, self.max_rows, self.chunk = max_context, max_seqs, max_rows, prefill_chunk
        self.waiting, self.running, self.arrivals = [], [], 0
        self.preemptions = 0

    def submit(self, name, prompt, max_new, stops=()):
        arrival, self.arrivals = self.arrivals, self.arrivals + 1
        room = self.max_context - len(prompt)
        if not prompt or room <= 0:
            return "empty_prompt" if not prompt else "context_length"
        self.waiting.append(dict(name=name, tokens=list(prompt), done=0, held=0, new=0, limit=min(max_new, room), stops=set(stops),
                                 arrival=arrival))
        return None

    def _pages(self, tokens: int) -> int:
        return -(-tokens // self.page)

    def plan(self):
        """[(name, first position, tokens, wants a new token)] of the next step, or None when nothing runs."""
        while self.waiting and len(self.running) < self.max_seqs and self.free_slots:
            r = self.waiting[0]
            if self.running and self.free_pages < self._pages(len(r["tokens"])) + len(self.running) + 1:
                break
            self.free_slots -= 1
            r["done"] = r["held"] = 0
            self.running.append(self.waiting.pop(0))
        while True:
            if not self.running:
                return None
            budget, batch = self.max_rows, []
            for r in self.running:
                if len(r["tokens"]) - r["done"] == 1 and budget > 0:
                    batch.append((r, 1))
                    budget -= 1
            for r in self.running:
                left = len(r["tokens"]) - r["done"]
                if left > 1 and budget > 0:
                    n = min(left, self.chunk, budget)
                    batch.append((r, n))
                    budget -= n
            need = sum(max(0, self._pages(r["done"] + n) - r["held"]) for r, n in batch)
            if need <= self.free_pages:
                break
            if len(self.running) <= 1:
                raise RuntimeError("the cache pool is too small for one sequence")
            victim = max(self.running, key=lambda r: r["arrival"])
            self.free_pages += victim["held"]
            self.free_slots += 1
            victim["held"] = 0
            self.preemptions += 1
            self.running.remove(victim)
            self.waiting.insert(0, victim)
        out = []
        for r, n in batch:
            grow = max(0, self._pages(r["done"] + n) - r["held"])
            self.free_pages -= grow
            r["held"] += grow
            out.append((r["name"], r["done"], r["tokens"][r["done"]:r["done"] + n], r["done"] + n == len(r["tokens"])))
            r["done"] += n
        return out

    def chosen(self, name, token):
        """The token chosen for a request whose last known token ran. Returns "stop", "length" or None."""
        r = next(x for x in self.running if x["name"] == name)
        r["tokens"].append(token)
        r["new"] += 1
        reason = "stop" if token in r["stops"] else "length" if r["new"] >= r["limit"] else None
        if reason:
            self.free_pages += r["held"]
            self.free_slots += 1
            self.running.remove(r)
        return reason
