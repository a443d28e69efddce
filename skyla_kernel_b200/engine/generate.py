"""The generation loop above the step function.

The reference's loop lives outside its repository; what shows of it is: the
prompt in one go, then a step per token until a stop token, ``-n`` tokens, or a
full context (docs/roadmap.md:122-123,230; skyla-engine/src/engine.rs:100).  Here
many requests are served: they are cut into batches that fit the cache, a
batch's prompts (of unequal length) run in one step, then every live sequence
gets one token per step; a sequence that ends leaves the batch and its slot goes
back at once; when the batch is empty the next one starts and reuses the slots.

The loop only decides; it computes nothing.  What it drives is a *backend* with
``alloc_slot()``, ``free_slot(slot)``, ``step(items) -> logits``,
``sample(logits, req_ids, steps) -> list[int]`` and ``pages_free()`` /
``page_size``; tests drive it with a fake one on the CPU.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from .batch import StepItem


@dataclass
class Request:
    prompt: Sequence[int]
    max_new_tokens: int
    stop_ids: Sequence[int] = ()


@dataclass
class Finished:
    tokens: List[int] = field(default_factory=list)
    reason: str = ""  # "stop", "length"


def pages_for(n_tokens: int, page_size: int) -> int:
    return -(-n_tokens // page_size)


def plan_batches(requests: Sequence[Request], n_pages: int, page_size: int, max_batch: int,
                 max_slots: int) -> List[List[int]]:
    """Cut the requests, in order, into batches whose worst-case pages fit the cache."""
    batches: List[List[int]] = []
    cur: List[int] = []
    used = 0
    for i, r in enumerate(requests):
        if len(r.prompt) == 0:
            raise ValueError(f"request {i} has an empty prompt")
        need = pages_for(len(r.prompt) + max(r.max_new_tokens, 0), page_size)
        if need > n_pages:
            raise ValueError(f"request {i} needs {need * page_size} cache positions, the cache "
                             f"holds {n_pages * page_size}")
        if cur and (used + need > n_pages or len(cur) >= min(max_batch, max_slots)):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


def generate(backend, requests: Sequence[Request], max_batch: int = 64, emit_stop: bool = False,
             on_step: Optional[Callable[[int, int], None]] = None) -> List[Finished]:
    """Serve all requests; results in request order."""
    results = [Finished() for _ in requests]
    batches = plan_batches(requests, backend.n_pages, backend.page_size, max_batch, backend.max_slots)
    for batch in batches:
        live = []  # (request index, slot)
        try:
            for i in batch:
                live.append((i, backend.alloc_slot()))
            produced = {i: 0 for i in batch}
            # prompts of unequal length in one step, logits at each prompt's last place
            todo = [(i, s) for i, s in live if requests[i].max_new_tokens > 0]
            for i, s in live:
                if requests[i].max_new_tokens <= 0:
                    results[i].reason = "length"
                    backend.free_slot(s)
            live = todo
            items = [StepItem(s, list(requests[i].prompt), [len(requests[i].prompt) - 1]) for i, s in live]
            step_no = 0
            while live:
                logits = backend.step(items)
                tokens = backend.sample(logits, [i for i, _ in live], [produced[i] for i, _ in live])
                if on_step is not None:
                    on_step(step_no, len(live))
                step_no += 1
                nxt, items = [], []
                for (i, s), tok in zip(live, tokens):
                    r = requests[i]
                    produced[i] += 1
                    stop = tok in r.stop_ids
                    if not stop or emit_stop:
                        results[i].tokens.append(int(tok))
                    if stop:
                        results[i].reason = "stop"
                    elif produced[i] >= r.max_new_tokens:
                        results[i].reason = "length"
                    if results[i].reason:
                        backend.free_slot(s)  # the slot goes back as soon as the sequence ends
                    else:
                        nxt.append((i, s))
                        items.append(StepItem(s, [int(tok)], [0]))
                live = nxt
        except BaseException:
            for _, s in live:
                try:
                    backend.free_slot(s)
                except Exception:
                    pass
            raise
    return results
