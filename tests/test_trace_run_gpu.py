"""bin/trace_run replays the same requests whole, with the last 32 tokens one by one,
in batches of unequal lengths and in mixed chunks, in both precisions, against the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from helpers import TINY, assert_close, make_folder, random_tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _replay(folder, dtype, steps, out, max_tokens):
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                           "--out", out, "--max-tokens", str(max_tokens)],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split("\n")[:-1] == [f"done {s['step']}" for s in steps]
    return proc


def _read(out, step, vocab):
    return torch.from_numpy(np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4").reshape(-1, vocab).copy())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_replay_every_way(tmp_path, name, dtype):
    folder = make_folder(tmp_path, name)
    cfg, w = plain.read_folder(folder)
    V = cfg["vocab_size"]
    lens = [45, 100, 64, 33, 129]
    reqs = {f"r{i}": random_tokens(n, V, 70 + i) for i, n in enumerate(lens)}
    refs = {k: plain.forward(cfg, w, v) for k, v in reqs.items()}
    steps, expect = [], {}   # expect[step] = list of (request, first place, count)
    n = 0
    # 1) each request alone and whole
    for k, toks in reqs.items():
        steps.append({"step": n, "entries": [{"id": k + "w", "tokens": toks, "want": list(range(len(toks)))}], "end": [k + "w"]})
        expect[n] = [(k, 0, len(toks))]; n += 1
    # 2) whole minus 32, then the last 32 one by one
    for k, toks in reqs.items():
        head = len(toks) - 32
        steps.append({"step": n, "entries": [{"id": k + "d", "tokens": toks[:head], "want": list(range(head))}], "end": []})
        expect[n] = [(k, 0, head)]; n += 1
        for t in range(head, len(toks)):
            steps.append({"step": n, "entries": [{"id": k + "d", "tokens": [toks[t]], "want": [0]}],
                          "end": [k + "d"] if t == len(toks) - 1 else []})
            expect[n] = [(k, t, 1)]; n += 1
    # 3) batches of unequal lengths; shorter requests end earlier; a second batch reuses what the first gave back
    first_batch_step = n
    for batch in (["r0", "r1", "r2"], ["r3", "r4", "r0"]):
        if batch[0] == "r3":
            second_batch_step = n
        cut = {k: max(1, len(reqs[k]) - 20 - 7 * i) for i, k in enumerate(batch)}
        steps.append({"step": n, "entries": [{"id": k + "b", "tokens": reqs[k][:cut[k]], "want": [cut[k] - 1]} for k in batch], "end": []})
        expect[n] = [(k, cut[k] - 1, 1) for k in batch]; n += 1
        t = 0
        while True:
            live = [k for k in batch if cut[k] + t < len(reqs[k])]
            if not live:
                break
            ending = [k + "b" for k in live if cut[k] + t == len(reqs[k]) - 1]
            steps.append({"step": n, "entries": [{"id": k + "b", "tokens": [reqs[k][cut[k] + t]], "want": [0]} for k in live], "end": ending})
            expect[n] = [(k, cut[k] + t, 1) for k in live]; n += 1
            t += 1
    # 4) mixed chunks: 50 / 30 / 1 on a filled cache, a chunk of 15 for two requests at once, the rest one by one
    #    (the program passes any cut on to the step function; the reference cuts its prompts at 128,
    #    skyla-engine/src/engine.rs:144-152)
    chunk_step = n
    chunked = ["r1", "r2", "r4"]   # 2 + 1 + 3 pages: they are live together
    cut = {}
    for k in chunked:
        toks = reqs[k]
        o = 0
        for c in (50, 30, 1):
            c = min(c, len(toks) - 1 - o)
            if c <= 0:
                break
            steps.append({"step": n, "entries": [{"id": k + "c", "tokens": toks[o:o + c], "want": list(range(c))}], "end": []})
            expect[n] = [(k, o, c)]; n += 1
            o += c
        cut[k] = o
    pair = ["r1", "r4"]
    steps.append({"step": n, "entries": [{"id": k + "c", "tokens": reqs[k][cut[k]:cut[k] + 15], "want": list(range(15))} for k in pair], "end": []})
    expect[n] = [(k, cut[k], 15) for k in pair]; n += 1
    for k in pair:
        cut[k] += 15
    t = 0
    while True:
        live = [k for k in chunked if cut[k] + t < len(reqs[k])]
        if not live:
            break
        ending = [k + "c" for k in live if cut[k] + t == len(reqs[k]) - 1]
        steps.append({"step": n, "entries": [{"id": k + "c", "tokens": [reqs[k][cut[k] + t]], "want": [0]} for k in live], "end": ending})
        expect[n] = [(k, cut[k] + t, 1) for k in live]; n += 1
        t += 1
    # one step that wants nothing writes no file
    steps.append({"step": n, "entries": [{"id": "q", "tokens": [1, 2, 3], "want": []}], "end": ["q"]})
    out = str(tmp_path / f"out_{dtype}")
    _replay(folder, dtype, steps, out, max_tokens=64 * 7)  # the second batch only fits because the first gave its pages back
    assert not os.path.exists(os.path.join(out, f"{n}.f32"))
    # rows of one request in one way of replaying are compared as one block
    blocks = {}
    for s, parts in sorted(expect.items()):
        got = _read(out, s, V)
        o = 0
        for k, first, count in parts:
            mode = (0 if s < len(reqs) else 1 if s < first_batch_step else 2 if s < second_batch_step
                    else 3 if s < chunk_step else 4)
            blocks.setdefault((mode, k), []).append((first, got[o:o + count]))
            o += count
        assert o == got.shape[0]
    assert len(blocks) == 5 + 5 + 6 + 3
    whole = {k: torch.cat([g for _, g in blocks[(0, k)]]) for k in reqs}
    for (mode, k), rows in blocks.items():
        places = [f + i for f, g in rows for i in range(g.shape[0])]
        assert places == list(range(places[0], places[0] + len(places)))
        got = torch.cat([g for _, g in rows])
        assert_close(got, refs[k][places[0]:places[-1] + 1], dtype, f"{name} {dtype} way {mode} request {k}")
        if dtype == "float32":  # the 32-bit path sums every element in one order, however the tokens are cut
            assert torch.equal(got, whole[k][places[0]:places[-1] + 1]), \
                f"{name} float32 way {mode} request {k}: not the bits of the whole run"
