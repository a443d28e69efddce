"""The generation loop above the step function.

The reference's loop lives outside its repository; what shows of it is: the
prompt in one go, then a step per token until a stop token, ``-n`` tokens, or a
full context (docs/roadmap.md:122-123,230; skyla-engine/src/engine.rs:100).  Here
many requests are served: they are cut into batches that fit the cache, a
batch's prompts (of unequal length) run in one step, then every live sequence
gets one token per step; a sequence that ends leaves the batch and its slot goes
back at once; when the batch is empty the next one starts and reuses the slots.

The loop only decides; it computes nothing.  What it drives is a *backend* with
``alloc_slot()``, ``free_slot(slot)``, ``n_pages``, ``page_size``, ``max_slots`` and either

* ``step(items) -> logits`` and ``sample(logits, req_ids, steps) -> list[int]``: the loop
  waits for every step's tokens before it decides the next step; or
* ``step_async(items, req_ids, steps) -> handle`` with ``handle.tokens() -> list[int]``: the
  loop starts step k+1 before it has seen the tokens of step k, feeding them on the device
  (``StepItem.device_token = (handle, row)``), so that the host's work hides behind the
  device's.  Which sequences end by length is known beforehand; one that ends on a stop
  token is found out a step late, runs that one step for nothing, and its extra token is
  dropped.  The results are the same as in the first manner.

Tests drive both manners with fake backends on the CPU.
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
    """Serve all requests; results in request order.  ``on_step(step, rows)`` is called when the
    tokens of a step have reached the host."""
    results = [Finished() for _ in requests]
    batches = plan_batches(requests, backend.n_pages, backend.page_size, max_batch, backend.max_slots)
    run = _run_batch_pipelined if hasattr(backend, "step_async") else _run_batch
    for batch in batches:
        run(backend, requests, batch, results, emit_stop, on_step)
    return results


def _start_batch(backend, requests, batch, results):
    """Slots for the batch; requests that want no tokens end at once.  Returns [(request, slot)]."""
    live = []
    try:
        for i in batch:
            live.append((i, backend.alloc_slot()))
    except BaseException:
        _free_all(backend, live)
        raise
    todo = []
    for i, s in live:
        if requests[i].max_new_tokens <= 0:
            results[i].reason = "length"
            backend.free_slot(s)
        else:
            todo.append((i, s))
    return todo


def _free_all(backend, live):
    for _, s in live:
        try:
            backend.free_slot(s)
        except Exception:
            pass


def _take(requests, results, i, tok, produced, emit_stop) -> bool:
    """Book one generated token of request ``i``; True if the request goes on."""
    r = requests[i]
    produced[i] += 1
    stop = tok in r.stop_ids
    if not stop or emit_stop:
        results[i].tokens.append(int(tok))
    if stop:
        results[i].reason = "stop"
    elif produced[i] >= r.max_new_tokens:
        results[i].reason = "length"
    return not results[i].reason


def _run_batch(backend, requests, batch, results, emit_stop, on_step):
    live = _start_batch(backend, requests, batch, results)
    try:
        produced = {i: 0 for i, _ in live}
        # prompts of unequal length in one step, logits at each prompt's last place
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
                if _take(requests, results, i, tok, produced, emit_stop):
                    nxt.append((i, s))
                    items.append(StepItem(s, [int(tok)], [0]))
                else:
                    backend.free_slot(s)  # the slot goes back as soon as the sequence ends
            live = nxt
    except BaseException:
        _free_all(backend, live)
        raise


def _run_batch_pipelined(backend, requests, batch, results, emit_stop, on_step):
    live = _start_batch(backend, requests, batch, results)
    held = dict((i, s) for i, s in live)  # request -> slot, until the slot is given back
    try:
        produced = {i: 0 for i, _ in live}   # tokens booked on the host
        launched = {i: 0 for i, _ in live}   # tokens whose step has been started
        items = [StepItem(s, list(requests[i].prompt), [len(requests[i].prompt) - 1]) for i, s in live]
        handle = backend.step_async(items, [i for i, _ in live], [0 for _ in live])
        for i, _ in live:
            launched[i] = 1
        in_flight = (live, handle)
        step_no = 0
        while in_flight is not None:
            rows, handle = in_flight
            # start the next step before looking at this one's tokens: every sequence that still
            # lacks tokens by count goes on, fed from the device
            nxt = [(i, s) for i, s in rows if not results[i].reason and launched[i] < requests[i].max_new_tokens]
            next_flight = None
            if nxt:
                row_of = {i: r for r, (i, _) in enumerate(rows)}
                items = [StepItem(s, [0], [0], device_token=(handle, row_of[i])) for i, s in nxt]
                h2 = backend.step_async(items, [i for i, _ in nxt], [launched[i] for i, _ in nxt])
                for i, _ in nxt:
                    launched[i] += 1
                next_flight = (nxt, h2)
            tokens = handle.tokens()  # waits for this step only; the next one is already queued
            if on_step is not None:
                on_step(step_no, len(rows))
            step_no += 1
            for (i, s), tok in zip(rows, tokens):
                if results[i].reason:
                    continue  # ended on a stop token a step ago: this token was computed for nothing
                if not _take(requests, results, i, tok, produced, emit_stop):
                    backend.free_slot(held.pop(i))
            in_flight = next_flight
    except BaseException:
        _free_all(backend, list(held.items()))
        raise
