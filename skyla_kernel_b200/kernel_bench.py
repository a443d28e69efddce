"""Times one kernel on its own (CUDA events, a CUDA graph of back-to-back launches over
different weights so that nothing is served from L2), the way the reference times a single
dispatch (skyla-vk/src/submit.rs:31-76).  Also the target of profiler captures:

    skyla kernel-bench linear --tokens 8 --n-out 4096 --n-in 12288 --mode accumulate
    skyla kernel-bench attention-decode --batch 8 --context 2048
    skyla kernel-bench attention-prefill --tokens 2048
    skyla kernel-bench step --tokens 2048 --batch 1 --layers 4      (a prompt step of the 8B layer sizes)
    skyla kernel-bench step --tokens 1 --batch 8 --context 2048 --layers 4   (a decode step)
"""
from __future__ import annotations

import json
import math

import torch

from .kernels import ops

DEV = "cuda:0"


def _time(fn, copies: int, reps: int) -> float:
    """Microseconds per call of ``fn(i)``, i = 0..copies-1, replayed as one graph."""
    for i in range(copies):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(copies):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        g.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / reps / copies


def linear(tokens: int, n_out: int, n_in: int, mode: str, copies: int = 0, reps: int = 5) -> dict:
    """The tensor-core product as the linear part would launch it for this many tokens."""
    from .parts.base import Runtime
    from .parts.feedforward import fuse_gate_up
    from .parts.linear import ACCUMULATE, GATED, STORE, Linear
    rt = Runtime(torch.device(DEV), "bfloat16")
    gated = mode == "gated"
    rows = n_out * (2 if gated else 1)
    copies = copies or max(2, min(24, int(400e6 // (rows * n_in * 2)) + 1))  # > L2 in total
    lins = []
    for i in range(copies):
        w = torch.empty(rows, n_in, dtype=torch.bfloat16, device=DEV)
        ops.fill_normal(w, 0.0, 0.02, i)
        lins.append(Linear(w, rt, gated=gated))
    x = torch.randn(tokens, n_in, device=DEV).to(torch.bfloat16)
    if mode == "accumulate":
        y = torch.zeros(tokens, n_out, device=DEV)
        fn = lambda i: lins[i].forward(x, y, ACCUMULATE)
    elif gated:
        y = torch.empty(tokens, n_out, dtype=torch.bfloat16, device=DEV)
        fn = lambda i: lins[i].forward(x, y, GATED)
    elif mode == "ahead":  # the prompt kernel's accumulate with the next norm's input prepared on the way
        y = torch.zeros(tokens, n_out, device=DEV)
        nw = torch.ones(n_out, device=DEV)
        xw = torch.empty(tokens, n_out, dtype=torch.bfloat16, device=DEV)
        shares = torch.empty(ops.prompt_ahead_parts(n_out), tokens, device=DEV)
        fn = lambda i: ops.gemm_prompt(x, lins[i].weight_map(), n_out, y, ops.TC_ACCUM_F32, norm_ahead=(nw, xw, shares))
    elif mode == "heads":  # the prompt kernel's q/k/v product: heads of 128 normed, rotated, written to q and the cache
        hd = 128
        nkv = max(1, n_out // hd // 6)
        nq = n_out // hd - 2 * nkv
        y = torch.empty(tokens, nq * hd, dtype=torch.bfloat16, device=DEV)
        pages = -(-tokens // 64)
        pools = [torch.zeros(pages, nkv, 64, hd, dtype=torch.bfloat16, device=DEV) for _ in range(2)]
        ang = torch.arange(tokens, device=DEV, dtype=torch.float32)[:, None] * torch.rand(hd // 2, device=DEV)[None, :]
        i32 = lambda t: t.to(torch.int32).to(DEV).contiguous()
        prep = dict(nq=nq, nkv=nkv, hd=hd, q_norm=torch.ones(hd, device=DEV), k_norm=torch.ones(hd, device=DEV), eps=1e-6,
                    cos=torch.cos(ang), sin=torch.sin(ang), tok_pos=i32(torch.arange(tokens)),
                    tok_slot=i32(torch.zeros(tokens)), k_pool=pools[0], v_pool=pools[1],
                    page_table=i32(torch.arange(pages)[None, :]), page_size=64)
        fn = lambda i: lins[i].forward_heads(x, y, prep)
    elif mode == "store-f32":
        y = torch.empty(tokens, n_out, device=DEV)
        fn = lambda i: lins[i].forward(x, y, STORE)
    else:
        y = torch.empty(tokens, n_out, dtype=torch.bfloat16, device=DEV)
        fn = lambda i: lins[i].forward(x, y, STORE)
    us = _time(fn, copies, reps)
    flops = 2.0 * tokens * rows * n_in
    return {"kernel": "linear", "tokens": tokens, "n_out": n_out, "n_in": n_in, "mode": mode, "us": us,
            "weight_GBps": rows * n_in * 2 / us / 1e3, "TFLOPs": flops / us / 1e6,
            "rows_kernel": lins[0].streams(tokens), "plan": lins[0].rows_plans[ops.token_tile(min(tokens, ops.ROWS_MAX_TOKENS))]}


def _paged(batch: int, context: int, nkv: int, hd: int):
    pages = -(-context // 64)
    width = 8
    while width < pages:
        width *= 2
    pool = batch * width
    k = torch.randn(pool, nkv, 64, hd, device=DEV).to(torch.bfloat16)
    v = torch.randn(pool, nkv, 64, hd, device=DEV).to(torch.bfloat16)
    table = torch.randperm(pool, device=DEV).to(torch.int32).view(batch, width).contiguous()
    return k, v, table, width


def attention_decode(batch: int, context: int, nq: int = 32, nkv: int = 8, hd: int = 128, reps: int = 5) -> dict:
    """Split-context decode attention plus its merge, cut as the attention part would cut it."""
    from .config import PartSpec
    from .parts.attention import GQAttention
    from .parts.base import Runtime
    k, v, table, width = _paged(batch, context, nkv, hd)
    q = torch.randn(batch, nq * hd, device=DEV).to(torch.bfloat16)
    out = torch.empty_like(q)
    pos = torch.full((batch,), context - 1, dtype=torch.int32, device=DEV)
    part = GQAttention(PartSpec("gqa_attention", {"hidden_size": nq * hd, "num_heads": nq, "num_kv_heads": nkv,
                                                  "head_dim": hd}), Runtime(torch.device(DEV), "bfloat16"))
    n_blocks = part.step_plans[0].blocks(batch, width)
    plan = torch.from_numpy(ops.decode_plan([context - 1] * batch, nkv, 0, 64, n_blocks)).to(DEV)
    scratch = torch.empty(ops.attention_decode_scratch(batch, nq, nkv, hd, n_blocks), device=DEV)
    us = _time(lambda i: ops.attention_decode(q, out, scratch, nq, nkv, hd, k, v, table, 64, pos, 1 / math.sqrt(hd), 0,
                                              n_blocks, plan), 8, reps)
    kv_bytes = 2 * batch * context * nkv * hd * 2
    return {"kernel": "attention-decode", "batch": batch, "context": context, "us": us, "blocks": n_blocks,
            "kv_GBps": kv_bytes / us / 1e3}


def attention_prefill(tokens: int, nq: int = 32, nkv: int = 8, hd: int = 128, reps: int = 5) -> dict:
    k, v, table, width = _paged(1, tokens, nkv, hd)
    q = torch.randn(tokens, nq * hd, device=DEV).to(torch.bfloat16)
    out = torch.empty_like(q)
    i32 = lambda t: t.to(torch.int32).to(DEV)
    pos = i32(torch.arange(tokens))
    n_tiles = -(-tokens // 64)
    tile_seq, tile_tok0 = i32(torch.zeros(n_tiles)), i32(torch.arange(n_tiles) * 64)
    tile_rows = i32(torch.tensor([min(64, tokens - 64 * i) for i in range(n_tiles)]))
    us = _time(lambda i: ops.attention_prefill(q, out, nq, nkv, hd, k, v, table, 64, pos, tile_seq, tile_tok0, tile_rows,
                                               1 / math.sqrt(hd), 0), 4, reps)
    flops = 4.0 * nq * hd * tokens * (tokens + 1) / 2
    return {"kernel": "attention-prefill", "tokens": tokens, "us": us, "TFLOPs": flops / us / 1e6}


def step(tokens: int, batch: int, context: int, layers: int, reps: int = 3) -> dict:
    """Whole steps of a model with the Qwen3-8B layer sizes and ``layers`` layers, random weights drawn on
    the device: ``batch`` prompts of ``tokens`` tokens in one step (``tokens`` > 1), or one token for each
    of ``batch`` sequences that hold ``context`` positions (``tokens`` == 1).  With an event after each
    stage on the last repetition (for a decode step that repetition is launched kernel by kernel, not as
    its graph, so its stage times are those of the host).  The launches of the last repetition are what a
    profiler's launch list should look at."""
    from .engine import StepItem
    from .measure import random_engine
    length = tokens if tokens > 1 else context
    eng, cfg = random_engine("8b", layers, max_tokens=batch * (length + 128), max_slots=batch, device=DEV)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (length,), generator=g).tolist() for _ in range(batch)]
    times = []
    if tokens > 1:
        for r in range(reps + 2):  # one untimed, `reps` timed, one with stage events
            slots = [eng.alloc_slot() for _ in range(batch)]
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            eng.step([StepItem(s, p, [length - 1]) for s, p in zip(slots, prompts)], profile=(r == reps + 1))
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
            for s in slots:
                eng.free_slot(s)
    else:
        slots = [eng.alloc_slot() for _ in range(batch)]
        per = max(1, 16384 // length)
        for i in range(0, batch, per):
            eng.step([StepItem(s, p, [length - 1]) for s, p in zip(slots[i:i + per], prompts[i:i + per])])
        for r in range(reps + 4):  # three untimed (the first records the graph), `reps` timed, one with stage events
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            eng.step([StepItem(s, [5], [0]) for s in slots], profile=(r == reps + 3))
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
    stages = {}
    for label, ns in eng.last_step_profile():
        stages[label] = stages.get(label, 0.0) + ns / 1e3
    timed = sorted(times[-1 - reps:-1])
    return {"kernel": "step", "tokens": tokens, "batch": batch, "context": length, "layers": layers,
            "ms": timed[len(timed) // 2], "ms_with_stage_events": times[-1],
            "stage_us": {k: round(v, 1) for k, v in stages.items()}}


def main(a) -> int:
    if a.kernel == "step":
        r = step(a.tokens, a.batch, a.context, a.layers, reps=a.reps)
    elif a.kernel == "linear":
        r = linear(a.tokens, a.n_out, a.n_in, a.mode, reps=a.reps)
    elif a.kernel == "attention-decode":
        r = attention_decode(a.batch, a.context, reps=a.reps)
    else:
        r = attention_prefill(a.tokens, reps=a.reps)
    print(json.dumps(r))
    return 0
