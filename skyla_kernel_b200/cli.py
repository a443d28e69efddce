"""The ``skyla`` command line, with the reference's command names and option meanings where
it has them (``run --check --profile --warmup -n``, ``bench-bw --reps``: README.md:145,207,247,
docs/roadmap.md:186,230-231) plus what a library without a tokenizer needs: token ids in and out,
a random-weights writer and the replay program.

    skyla run MODEL --prompt-ids 1,2,3 -n 16 [--temperature T --top-k K --top-p P --seed S]
                    [--dtype bfloat16|float32] [--check] [--profile] [--warmup]
    skyla bench MODEL [--batch 8] [--prompt-len 512] [-n 64]
    skyla bench-bw [--mib 512] [--reps 9]
    skyla random --config CONFIG.json --out DIR [--seed S] [--dtype bfloat16|float32]
    skyla kernel-bench linear|attention-decode|attention-prefill|step [sizes]
    skyla replay --model DIR --dtype D --out DIR --max-tokens N   (same as bin/trace_run)
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from typing import List


def _ids(text: str) -> List[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def cmd_run(a) -> int:
    import torch

    from . import load
    from .engine import StepItem
    prompts = [_ids(p) for p in a.prompt_ids]
    pages = sum(-(-(len(p) + a.n) // 64) for p in prompts)
    model = load(a.model, dtype=a.dtype, max_tokens=max(a.max_tokens or 0, 64 * pages))
    kw = dict(max_new_tokens=a.n, temperature=a.temperature, top_k=a.top_k, top_p=a.top_p, seed=a.seed,
              stop_ids=a.stop_id if a.stop_id is not None else None)
    if a.warmup:  # as the reference: the prompt once first (README.md:247)
        model.generate(prompts, **dict(kw, max_new_tokens=1))
    marks = []
    t0 = time.perf_counter()
    out = model.generate(prompts, on_step=lambda s, live: marks.append((time.perf_counter(), live)), **kw)
    dt = time.perf_counter() - t0
    for p, o in zip(prompts, out):
        print(" ".join(map(str, o)))
    n_new = sum(len(o) for o in out)
    if len(marks) > 1:
        decode_tokens = sum(live for _, live in marks[1:])
        print(f"# prompt {sum(map(len, prompts))} tokens in {marks[0][0] - t0:.3f} s; "
              f"{decode_tokens} tokens decoded at {decode_tokens / max(marks[-1][0] - marks[0][0], 1e-9):.1f} tok/s",
              file=sys.stderr)
    else:
        print(f"# {n_new} tokens in {dt:.3f} s", file=sys.stderr)
    if a.profile:
        eng = model.engine
        s = eng.alloc_slot()
        eng.step([StepItem(s, prompts[0], [len(prompts[0]) - 1])])
        eng.step([StepItem(s, [prompts[0][-1]], [0])], profile=True)
        eng.free_slot(s)
        prof = eng.last_step_profile()
        total = sum(ns for _, ns in prof) or 1.0
        print(f"# one decode step at position {len(prompts[0])}: {total / 1e6:.3f} ms", file=sys.stderr)
        for label, ns in prof:
            print(f"#   {label:30s} {ns / 1e3:9.1f} us {100 * ns / total:5.1f} %", file=sys.stderr)
    if a.check:
        return _check(a, prompts, out)
    return 0


NEAR_TIE = 0.02  # probability: "top-2 margin under 2 points" (docs/roadmap.md:89-92 of the reference)


def near_tie(logits) -> bool:
    """Whether the two most likely tokens of a row of logits are within 2 points of probability,
    the reference's rule for a top-1 disagreement that rounding alone explains."""
    import torch
    p = torch.softmax(logits.double(), dim=-1)
    top = torch.topk(p, 2).values
    return bool(top[0] - top[1] < NEAR_TIE)


def judge(logits, oracle):
    """One step of the lockstep: (top of ``logits``, top of ``oracle``, largest difference, verdict);
    the verdict is "" when the tops agree, "near tie" when they differ at a near tie of the oracle,
    else "DISAGREE"."""
    ta, tb = int(logits.argmax()), int(oracle.argmax())
    diff = float((logits - oracle).abs().max())
    return ta, tb, diff, "" if ta == tb else ("near tie" if near_tie(oracle) else "DISAGREE")


def _check(a, prompts, out) -> int:
    """Lockstep against the true 32-bit path: top token of each and the largest logit
    difference at every step (the reference's ``run --check``, README.md:206-208).
    Returns 1 (the command's exit code) if the top tokens disagree anywhere but at a near
    tie of the 32-bit path, else 0."""
    import torch

    from . import load
    from .engine import StepItem
    worst_all, mismatches, real = 0.0, 0, 0
    engines = [load(a.model, dtype=d, max_tokens=64 * (-(-(max(map(len, prompts)) + a.n) // 64))).engine
               for d in (a.dtype, "float32")]
    for p, o in zip(prompts, out):
        slots = [e.alloc_slot() for e in engines]
        feed = list(p)
        for step, tok in enumerate(o + [None]):
            want = [len(feed) - 1]
            la, lb = (e.step([StepItem(s, feed, want)]) for e, s in zip(engines, slots))
            ta, tb, diff, verdict = judge(la[0], lb[0])
            worst_all = max(worst_all, diff)
            mismatches += verdict != ""
            real += verdict == "DISAGREE"
            print(f"# check step {step}: {a.dtype} top {ta}, float32 top {tb}, largest logit difference {diff:.4f}"
                  + (f" ({verdict})" if verdict else ""), file=sys.stderr)
            if tok is None:
                break
            feed = [tok]
        for e, s in zip(engines, slots):
            e.free_slot(s)
    print(f"# check: {mismatches} top-1 disagreements ({real} outside near ties), worst logit difference {worst_all:.4f}",
          file=sys.stderr)
    return 1 if real else 0


def cmd_bench(a) -> int:
    import torch

    from . import load
    from .engine import StepItem
    max_tokens = a.batch * 64 * (-(-(a.prompt_len + a.n + 8) // 64))
    model = load(a.model, dtype=a.dtype, max_tokens=max_tokens)
    eng = model.engine
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, eng.vocab_size, (a.prompt_len,), generator=g).tolist() for _ in range(a.batch)]
    slots = [eng.alloc_slot() for _ in prompts]
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    ev[0].record()
    eng.step([StepItem(s, p, [a.prompt_len - 1]) for s, p in zip(slots, prompts)], borrow=True)
    ev[1].record()
    for i in range(a.n + 4):
        if i == 4:
            ev[1].record()
        eng.step([StepItem(s, [1], [0]) for s in slots], borrow=True)
    ev[2].record()
    torch.cuda.synchronize()
    ms = ev[1].elapsed_time(ev[2]) / a.n
    step_bytes = eng.weight_bytes() + a.batch * (a.prompt_len + a.n // 2) * eng.cache.bytes_per_token()
    print(json.dumps({"device": eng.device_name(), "batch": a.batch, "prompt_len": a.prompt_len,
                      "decode_ms_per_step": ms, "decode_tok_s": a.batch * 1e3 / ms,
                      "decode_GBps": step_bytes / ms / 1e6, "weight_bytes": eng.weight_bytes()}))
    return 0


def cmd_bench_bw(a) -> int:
    """Streaming-read roofline, as the reference's ``bench-bw`` (docs/roadmap.md:184-195)."""
    import torch

    from .kernels import ops
    n = a.mib * (1 << 20) // 4
    buf = torch.ones(n, dtype=torch.int32, device="cuda:0")
    sink = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    best = (0.0, 0)
    for blocks in (148, 296, 592, 1184, 2368):
        times = []
        for _ in range(a.reps + 1):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            ops.bandwidth_read(buf, blocks, sink)
            e.record()
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e))
        gbs = n * 4 / (min(times[1:]) * 1e-3) / 1e9
        print(f"{blocks:5d} blocks: {gbs:8.1f} GB/s")
        best = max(best, (gbs, blocks))
    print(json.dumps({"read_GBps": best[0], "blocks": best[1], "mib": a.mib, "reps": a.reps}))
    return 0


def cmd_random(a) -> int:
    from .config import config_from_dict
    from .weights import write_model_folder
    with open(a.config) as f:
        cfg = config_from_dict(json.load(f))
    write_model_folder(a.out, cfg, a.seed, a.dtype, a.linear_std, a.norm_std)
    print(a.out)
    return 0


def cmd_replay(a) -> int:
    from .replay import replay
    return replay(a.model, a.dtype, a.out, a.max_tokens)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="skyla", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name in ("run", "generate"):
        p = sub.add_parser(name, help="generate token ids from prompt token ids")
        p.add_argument("model")
        p.add_argument("--prompt-ids", action="append", required=True, help="token ids, comma or space separated; repeatable")
        p.add_argument("-n", type=int, default=16, help="tokens to generate per prompt")
        p.add_argument("--temperature", type=float, default=0.0)
        p.add_argument("--top-k", type=int, default=0)
        p.add_argument("--top-p", type=float, default=1.0)
        p.add_argument("--seed", type=int, default=0)
        p.add_argument("--stop-id", type=int, action="append")
        p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
        p.add_argument("--max-tokens", type=int, default=0)
        p.add_argument("--check", action="store_true", help="lockstep against the 32-bit path")
        p.add_argument("--profile", action="store_true", help="per-stage times of one decode step")
        p.add_argument("--warmup", action="store_true", help="run the prompt once first")
        p.set_defaults(fn=cmd_run)
    p = sub.add_parser("bench", help="decode throughput of a model folder")
    p.add_argument("model")
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--prompt-len", type=int, default=512)
    p.add_argument("-n", type=int, default=64)
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.set_defaults(fn=cmd_bench)
    p = sub.add_parser("bench-bw", help="streaming-read bandwidth of the device")
    p.add_argument("--mib", type=int, default=512)
    p.add_argument("--reps", type=int, default=9)
    p.set_defaults(fn=cmd_bench_bw)
    p = sub.add_parser("random", help="write a model folder with seeded random weights")
    p.add_argument("--config", required=True)
    p.add_argument("--out", required=True)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--linear-std", type=float, default=0.02)
    p.add_argument("--norm-std", type=float, default=0.02)
    p.set_defaults(fn=cmd_random)
    p = sub.add_parser("kernel-bench", help="time one kernel on its own (also the target of profiler captures)")
    p.add_argument("kernel", choices=["linear", "attention-decode", "attention-prefill", "step"])
    p.add_argument("--layers", type=int, default=4, help="step: layers of the 8B-shaped model")
    p.add_argument("--tokens", type=int, default=8)
    p.add_argument("--n-out", type=int, default=4096)
    p.add_argument("--n-in", type=int, default=4096)
    p.add_argument("--mode", choices=["store", "store-f32", "accumulate", "gated", "ahead", "heads"], default="store",
                   help="linear: the epilogue (ahead, heads: of the prompt kernel, 129 tokens or more)")
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=2048)
    p.add_argument("--reps", type=int, default=5)
    p.set_defaults(fn=lambda a: __import__("skyla_kernel_b200.kernel_bench", fromlist=["main"]).main(a))
    p = sub.add_parser("replay", help="replay a token trace from standard input (bin/trace_run)")
    p.add_argument("--model", required=True)
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--out", required=True)
    p.add_argument("--max-tokens", type=int, required=True)
    p.set_defaults(fn=cmd_replay)
    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
