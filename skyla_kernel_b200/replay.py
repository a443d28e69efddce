"""Trace replay: given token ids go through the engine step by step, logits come out.

The ancestors in the reference are ``skyla ref --expect`` (a token list teacher-forced
through the CPU model, docs/roadmap.md:208-213) and ``skyla run --check`` (engine and
oracle in lockstep, README.md:206-208).  Nothing is sampled; the model, step function,
cache and kernels are the ones generation uses.
"""
from __future__ import annotations

import json
import os
import sys
from typing import IO


def replay(model: str, dtype: str, out: str, max_tokens: int, device: str = "cuda:0",
           lines: IO[str] = None, done: IO[str] = None) -> int:
    """Read steps (one JSON object a line) from ``lines``; write ``<out>/<step>.f32`` for the
    steps that want logits; print ``done <step>`` after each."""
    lines = lines if lines is not None else sys.stdin
    done = done if done is not None else sys.stdout
    print("[skyla] loading the library ...", file=sys.stderr, flush=True)
    import torch

    from .engine import Engine, StepItem
    os.makedirs(out, exist_ok=True)
    engine = Engine.from_folder(model, dtype=dtype, max_tokens=max_tokens, device=device)
    print("[skyla] model ready", file=sys.stderr, flush=True)
    slots = {}
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        items = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if rid not in slots:
                slots[rid] = engine.alloc_slot()
            items.append(StepItem(slots[rid], e["tokens"], e.get("want", [])))
        logits = engine.step(items, borrow=True)
        if logits.shape[0]:
            arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
            tmp = os.path.join(out, f".{step}.f32.tmp")
            arr.tofile(tmp)
            os.replace(tmp, os.path.join(out, f"{step}.f32"))
        torch.cuda.synchronize()  # a fault shows at the step that caused it
        engine.check_errors()
        for rid in rec.get("end", []):
            if rid in slots:
                engine.free_slot(slots.pop(rid))
        print(f"done {step}", file=done, flush=True)
    return 0
