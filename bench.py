"""Decode and prefill throughput of the Qwen3-8B-shaped model with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--shape 8b|4b|32b]
    python bench.py --shape 4b --workload unequal16     (16 unequal prompts, 256 sampled tokens, checked)

One "step" is one decode step of the batch.  Prints ONE JSON line: decoded tokens
per second on the device (`value`), the same through the Python entry point with
host tokens in and out (`e2e`), a 2,048-token prefill, the decode step's HBM
roofline fraction, and in `points` decode at batch 1 and 64 from 2,048-token prompts and
at batch 1, 8 and 64 at the far end of the 4,096-token context, each with its own
fraction of the roofline (`frac_*`).  Every timed loop follows at least 40 untimed
steps (more if --warmup asks for more): right after long prompts the GPU is still coming
back from its power cap.  The library runs on one GPU only; for --gpus N > 1 it says so
and exits with 2.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from skyla_kernel_b200.measure import SHAPES  # layer sizes of the Qwen3-8B (default), -4B and -32B shapes

PROMPT_LEN = 2048
CONTEXT = 4096
FALLBACK_HBM_GBS = 6650.0       # an earlier measurement on this pool, used when no peaks file exists
FALLBACK_BF16_TFLOPS = 1590.0


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured", d.get("bf16_tflops_sustained")
        except (OSError, ValueError, KeyError):
            pass
    return FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback", None


class ClockSampler:
    """SM clock and throttle reasons during the timed region (reads only): NVML from a thread every
    few milliseconds, so that short regions are seen too; nvidia-smi in the background where the
    NVML binding is missing."""
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0, period_s=0.004):
        self.index, self.period = index, period_s
        self.proc = self.thread = None
        self.samples, self.max_mhz, self.reasons = [], None, set()
        self.mem_samples, self.power_samples = [], []
        self._stop = threading.Event()

    def _nvml_loop(self, nvml, handle):
        masks = {"hw_slowdown": nvml.nvmlClocksThrottleReasonHwSlowdown,
                 "hw_thermal_slowdown": nvml.nvmlClocksThrottleReasonHwThermalSlowdown,
                 "sw_thermal_slowdown": nvml.nvmlClocksThrottleReasonSwThermalSlowdown,
                 "sw_power_cap": nvml.nvmlClocksThrottleReasonSwPowerCap}
        while not self._stop.is_set():
            try:
                self.samples.append(float(nvml.nvmlDeviceGetClockInfo(handle, nvml.NVML_CLOCK_SM)))
                self.mem_samples.append(float(nvml.nvmlDeviceGetClockInfo(handle, nvml.NVML_CLOCK_MEM)))
                self.power_samples.append(nvml.nvmlDeviceGetPowerUsage(handle) / 1000.0)
                bits = nvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                self.reasons.update(n for n, m in masks.items() if bits & m)
            except Exception:
                pass
            self._stop.wait(self.period)

    def start(self):
        try:
            import pynvml as nvml
            nvml.nvmlInit()
            handle = nvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(nvml.nvmlDeviceGetMaxClockInfo(handle, nvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._nvml_loop, args=(nvml, handle), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.thread is not None:
            self._stop.set()
            self.thread.join(timeout=2)
            sm = self.samples
            out = {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.max_mhz,
                   "reasons": sorted(self.reasons), "samples": len(sm), "how": "nvml"}
            if self.mem_samples:
                out["mem_mhz"] = statistics.median(self.mem_samples)
            if self.power_samples:
                out["power_w"] = round(statistics.median(self.power_samples), 1)
            return out
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no clock reading available"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(self.NAMES, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "how": "nvidia-smi"}


def build_model(layers: int, max_tokens: int, max_slots: int, seed: int = 0, shape: str = "8b"):
    """The model of ``shape``'s layer sizes with seeded random weights drawn on the device."""
    import skyla_kernel_b200 as skyla
    from skyla_kernel_b200.measure import random_engine
    engine, cfg = random_engine(shape, layers, max_tokens=max_tokens, max_slots=max_slots, seed=seed)
    return skyla.Model(engine), cfg


def random_prompts(n, length, vocab, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (length,), generator=g).tolist() for _ in range(n)]


def prefill_flops(cfg, T, n_logit_rows=1):
    H, nq, nkv, hd, I, V, L = (cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                               cfg.intermediate_size, cfg.vocab_size, cfg.num_hidden_layers)
    per_tok = 2 * L * (H * (nq + 2 * nkv) * hd + nq * hd * H + 3 * H * I)
    attn = L * 4 * nq * hd * (T * (T + 1) // 2)  # causal: QK^T and PV over the visible half
    return per_tok * T + attn + 2 * n_logit_rows * H * V


def device_decode(model, batch, prompt_len, steps, warmup, vocab, sampler):
    """Prefill `batch` prompts, then time `steps` decode steps on the device with CUDA events."""
    import torch
    from skyla_kernel_b200.engine import StepItem
    from skyla_kernel_b200.kernels import ops
    eng = model.engine
    warmup = max(warmup, MIN_WARMUP)
    prompts = random_prompts(batch, prompt_len, vocab, 11 + batch)
    slots = [eng.alloc_slot() for _ in range(batch)]
    toks = []
    chunk = max(1, 16384 // prompt_len)  # prompts per prefill step
    for i in range(0, batch, chunk):
        items = [StepItem(slots[j], prompts[j], [prompt_len - 1]) for j in range(i, min(batch, i + chunk))]
        logits = eng.step(items)
        toks += torch.argmax(logits, dim=-1).tolist()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    kv_bytes = 0
    launches0 = 0
    for s in range(warmup + steps):
        if s == warmup:
            torch.cuda.synchronize()
            launches0 = ops.LAUNCHES
            sampler.start()
            start.record()
        if s >= warmup:
            kv_bytes += sum(eng.cache.length(sl) + 1 for sl in slots) * eng.cache.bytes_per_token()
        logits = eng.step([StepItem(sl, [t], [0]) for sl, t in zip(slots, toks)], borrow=True)
        toks = torch.argmax(logits, dim=-1).tolist() if s < warmup else toks  # timed steps feed fixed tokens
    end.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = start.elapsed_time(end)
    launches = ops.LAUNCHES - launches0
    ctx_end = eng.cache.length(slots[0])
    for sl in slots:
        eng.free_slot(sl)
    step_bytes = eng.weight_bytes() + kv_bytes / steps
    return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "kv_bytes_per_step": kv_bytes / steps,
            "launches": launches, "clocks": clocks, "context_end": ctx_end,
            "GBps": step_bytes / (ms / steps / 1e3) / 1e9}


class _NoSampler:
    def start(self): pass
    def stop(self): return None


#: After a long prompt step the GPU runs at about half its clock for the next 80 to 100 ms (it has just been
#: capped at its power limit and takes that long to come back: decode steps of the 8B shape take up to 5.2 ms
#: there instead of 3.6, and at 4,094 positions 3.66 instead of 3.36 at batch 1).  Every decode number here
#: is meant as steady decoding, so every timed loop, on the device and end to end, first runs at least this
#: many untimed steps, however few --warmup asks for; `config.warmup_steps_run` says how many were run.
MIN_WARMUP = 40
E2E_MIN_WARMUP = MIN_WARMUP


def e2e_decode(model, batch, prompt_len, steps, warmup, vocab):
    """The same through model.generate: host token ids in, host token ids out every step."""
    import torch
    warmup = max(warmup, E2E_MIN_WARMUP)
    prompts = random_prompts(batch, prompt_len, vocab, 23 + batch)
    marks = {}

    from skyla_kernel_b200.engine.batch import BatchBuilder

    def on_step(step, live):
        # step 0 is the prefill; the tokens of step s have reached the host when this runs
        if step == warmup:
            marks["t0"], marks["b0"] = time.perf_counter(), BatchBuilder.h2d_bytes
        if step == warmup + steps:
            marks["t1"], marks["b1"] = time.perf_counter(), BatchBuilder.h2d_bytes

    model.generate(prompts, max_new_tokens=warmup + steps + 1, stop_ids=[], max_batch=batch, on_step=on_step)
    dt = marks["t1"] - marks["t0"]
    # what the step's builder copied: tokens, positions, rows, slots, page lists, the attention's plan
    h2d = (marks["b1"] - marks["b0"]) // steps
    return {"value": batch * steps / dt, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * (batch + 1),
            "ms_per_step": dt / steps * 1e3, "warmup_steps": warmup}


def prefill_once(model, cfg, length, reps=5, warmup=3):
    import torch
    from skyla_kernel_b200.engine import StepItem
    eng = model.engine
    prompt = random_prompts(1, length, cfg.vocab_size, 5)[0]
    times = []
    for r in range(warmup + reps):
        s = eng.alloc_slot()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        eng.step([StepItem(s, prompt, [length - 1])])
        b.record()
        torch.cuda.synchronize()
        eng.free_slot(s)
        if r >= warmup:
            times.append(a.elapsed_time(b))
    return statistics.median(times)


def unequal16(args, hbm_gbs) -> dict:
    """The 4B benchmark configuration: 16 sequences that start together with prompts uniform in
    [64, 1536], 256 decode steps at temperature 0.7 through the Python entry point; then the
    bfloat16 path's logits at each sequence's last position against the 32-bit path on the same
    tokens (the reference's lockstep check at model size, README.md:206-208, docs/roadmap.md:264-265)."""
    import torch
    import skyla_kernel_b200 as skyla
    from skyla_kernel_b200.engine import Engine, StepItem
    from skyla_kernel_b200.measure import random_config, random_tensors_on_device
    n_seq, n_new, tail = 16, 256, 8
    cfg = random_config(args.shape, args.layers)
    g = torch.Generator().manual_seed(16)
    lens = torch.randint(64, 1537, (n_seq,), generator=g).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    max_tokens = sum(-(-(n + n_new) // 64) * 64 for n in lens)
    tensors = random_tensors_on_device(cfg, seed=0)
    model = skyla.Model(Engine(cfg, dict(tensors), "bfloat16", max_tokens=max_tokens, max_slots=n_seq))
    kw = dict(max_new_tokens=n_new, temperature=0.7, seed=7, stop_ids=[], max_batch=n_seq)
    model.generate(prompts, **kw)  # the workload once untimed: kernels are loaded and the decode graphs recorded
    marks = []
    t0 = time.perf_counter()
    out = model.generate(prompts, on_step=lambda s, live: marks.append(time.perf_counter()), **kw)
    decode_s = marks[-1] - marks[0]
    # the check: all but the last `tail` tokens as a prompt, then `tail` single tokens (the decode kernels, as
    # graphs), in bfloat16; the whole sequence at once in 32-bit; logits after the last token of both
    seqs = [p + o for p, o in zip(prompts, out)]
    eng = model.engine
    slots = [eng.alloc_slot() for _ in seqs]
    eng.step([StepItem(s, q[:-tail], []) for s, q in zip(slots, seqs)])
    for t in range(tail, 0, -1):
        low = eng.step([StepItem(s, [q[-t]], [0]) for s, q in zip(slots, seqs)])
    eng.check_errors()
    for s in slots:
        eng.free_slot(s)
    ref_eng = Engine(cfg, tensors, "float32", max_tokens=max_tokens, max_slots=n_seq)
    del tensors
    rows = []
    for q in seqs:  # one at a time: the 32-bit path's activations of a step are wide
        s = ref_eng.alloc_slot()
        rows.append(ref_eng.step([StepItem(s, q, [len(q) - 1])]))
        ref_eng.free_slot(s)
    ref = torch.cat(rows)
    diff = (low - ref).abs()
    scale = float(ref.abs().max())
    return {"tok_s": n_seq * (len(marks) - 1) / decode_s, "ms_per_step": decode_s / (len(marks) - 1) * 1e3,
            "prompt_lens": [min(lens), max(lens)], "prompt_tokens": sum(lens), "prefill_s": marks[0] - t0,
            "logit_diff_abs": float(diff.max()), "logit_diff_rel": float(diff.max()) / scale,
            "logit_diff_mean_rel": float(diff.mean()) / scale, "largest_logit": scale,
            "top1_agree": int((low.argmax(-1) == ref.argmax(-1)).sum()), "of": n_seq, "layers": cfg.num_hidden_layers}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--shape", choices=sorted(SHAPES), default="8b", help="layer sizes: Qwen3-8B (the default), -4B or -32B")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the shape has (0: all)")
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64 and at the long context")
    ap.add_argument("--workload", choices=["decode", "unequal16"], default="decode",
                    help="unequal16: 16 unequal prompts, 256 sampled tokens, bfloat16 logits checked against 32-bit")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust workspace with Vulkan/Metal backends: no pip-installable package, "
                          "no cargo/rustc and no graphics stack on this box"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    shape = SHAPES[args.shape]
    args.layers = args.layers or shape["num_hidden_layers"]

    import torch
    hbm_gbs, bf16_tflops, peak_kind, bf16_sustained = peaks()
    if args.workload == "unequal16":
        r = unequal16(args, hbm_gbs)
        print(json.dumps({"metric": "decode tokens/s through the entry point, Qwen3-%s shape bf16, 16 unequal prompts, "
                                    "256 tokens at temperature 0.7" % args.shape.upper(), "value": r["tok_s"],
                          "unit": "tokens/s", "n_gpus": 1, "dtype": "bf16", "workload": r}))
        return 0
    batches = [args.batch] + ([] if args.no_points else [b for b in (1, 64) if b != args.batch])
    max_tokens = max(batches) * (-(-CONTEXT // 64) * 64)
    t_build = time.time()
    model, cfg = build_model(args.layers, max_tokens=max_tokens, max_slots=max(batches), shape=args.shape)
    print(f"[bench] model built in {time.time() - t_build:.1f} s: {args.layers} layers, "
          f"{model.engine.weight_bytes() / 1e9:.2f} GB of weights per step", file=sys.stderr, flush=True)
    V = cfg.vocab_size

    # prefill of 2,048 tokens
    pre_ms = prefill_once(model, cfg, PROMPT_LEN)
    pre_flops = prefill_flops(cfg, PROMPT_LEN)
    prefill = {"value": PROMPT_LEN / (pre_ms / 1e3), "tokens": PROMPT_LEN, "ms": pre_ms,
               "frac": pre_flops / (pre_ms / 1e3) / (bf16_tflops * 1e12)}
    if bf16_sustained:  # the step is 28 ms of products at the power limit: beside the burst peak, the sustained one
        prefill["frac_of_sustained"] = pre_flops / (pre_ms / 1e3) / (float(bf16_sustained) * 1e12)
    print(f"[bench] prefill {PROMPT_LEN} tokens: {pre_ms:.1f} ms", file=sys.stderr, flush=True)

    sampler = ClockSampler()
    main_run = device_decode(model, args.batch, PROMPT_LEN, args.steps, args.warmup, V, sampler)
    print(f"[bench] decode batch {args.batch}: {main_run['ms_per_step']:.3f} ms/step", file=sys.stderr, flush=True)
    e2e = e2e_decode(model, args.batch, PROMPT_LEN, args.steps, args.warmup, V)
    points = {}
    for b in batches[1:]:
        r = device_decode(model, b, PROMPT_LEN, args.steps, args.warmup, V, _NoSampler())
        points[f"decode_b{b}"] = r["tok_s"]
        points[f"frac_b{b}"] = r["GBps"] / hbm_gbs
        print(f"[bench] decode batch {b}: {r['ms_per_step']:.3f} ms/step", file=sys.stderr, flush=True)
    points[f"decode_b{args.batch}"] = main_run["tok_s"]
    points[f"frac_b{args.batch}"] = main_run["GBps"] / hbm_gbs
    if not args.no_points:
        # the far end of the context: the timed steps end just under CONTEXT positions
        long_prompt = max(64, CONTEXT - max(args.warmup, MIN_WARMUP) - args.steps - 2)
        for b in sorted(set(batches)):
            r = device_decode(model, b, long_prompt, args.steps, args.warmup, V, _NoSampler())
            points[f"decode_b{b}_ctx{CONTEXT}"] = r["tok_s"]
            points[f"frac_b{b}_ctx{CONTEXT}"] = r["GBps"] / hbm_gbs
            print(f"[bench] decode batch {b} at context {r['context_end']}: {r['ms_per_step']:.3f} ms/step",
                  file=sys.stderr, flush=True)

    achieved = main_run["GBps"]
    line = {
        "metric": "decode tokens/s, Qwen3-%s shape bf16, batch %d, 2048-token prompts" % (args.shape.upper(), args.batch),
        "value": main_run["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": main_run["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights N(0,0.02), norms 1+N(0,0.02), uniform token ids",
        "config": {
            "model": "Qwen3-%s shape" % args.shape.upper(), "global_batch": args.batch, "seq_len": CONTEXT, "parallelism": "single GPU",
            "layers": args.layers, "layers_of_config": shape["num_hidden_layers"],
            "hidden_size": cfg.hidden_size, "num_attention_heads": cfg.num_attention_heads,
            "num_key_value_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "intermediate_size": cfg.intermediate_size, "vocab_size": cfg.vocab_size,
            "prompt_len": PROMPT_LEN, "context_at_end_of_timing": main_run["context_end"],
            "kv_cache": "bf16 paged, 64 positions per page", "l2": "inputs larger than L2 (weights read every step)",
            "peaks": peak_kind, "warmup_steps_run": max(args.warmup, MIN_WARMUP),
        },
        "e2e": e2e, "gpu_launches": main_run["launches"], "clocks": main_run["clocks"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s", "frac": achieved / hbm_gbs},
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
