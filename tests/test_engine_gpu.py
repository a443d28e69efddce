"""The engine against the plain implementation, in every way of cutting the work."""
import pytest
import torch

import plain_qwen3 as plain
from helpers import TINY, assert_close, make_folder, random_tokens

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
NAMES = ["A", "B", "C", "D"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    d = tmp_path_factory.mktemp("models")
    return {n: make_folder(d, n) for n in NAMES}


def _engine(folder, dtype, max_tokens=2048):
    from skyla_kernel_b200.engine import Engine
    return Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens)


_MODELS = {}


def _check(folder, tokens, got, dtype, what):
    """Compare with the plain 32-bit implementation."""
    if folder not in _MODELS:
        _MODELS[folder] = plain.read_folder(folder)
    cfg, w = _MODELS[folder]
    assert_close(got, plain.forward(cfg, w, tokens), dtype, what)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_sequence_alone(folders, name, dtype):
    from skyla_kernel_b200.engine import StepItem
    eng = _engine(folders[name], dtype)
    V = TINY[name][0]["vocab_size"]
    for n, seed in ((1, 3), (5, 4), (70, 5), (150, 6), (300, 7)):
        toks = random_tokens(n, V, seed)
        s = eng.alloc_slot()
        got = eng.step([StepItem(s, toks, list(range(n)))])
        eng.free_slot(s)
        _check(folders[name], toks, got, dtype, f"{name} {dtype} whole n={n}")
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_last_32_one_by_one(folders, name, dtype):
    from skyla_kernel_b200.engine import StepItem
    eng = _engine(folders[name], dtype)
    V = TINY[name][0]["vocab_size"]
    n = 100
    toks = random_tokens(n, V, 11)
    s = eng.alloc_slot()
    head = n - 32
    rows = [eng.step([StepItem(s, toks[:head], list(range(head)))])]
    for t in range(head, n):
        rows.append(eng.step([StepItem(s, [toks[t]], [0])]))
    got = torch.cat(rows)
    _check(folders[name], toks, got, dtype, f"{name} {dtype} last 32 one by one")
    eng.free_slot(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_with_slot_reuse(folders, name, dtype):
    """Batches of unequal prompts, then one token each; shorter requests end earlier;
    one batch after another in a cache that only fits one, so slots and pages are reused."""
    from skyla_kernel_b200.engine import StepItem
    V = TINY[name][0]["vocab_size"]
    eng = _engine(folders[name], dtype, max_tokens=4 * 128)
    for round_ in range(3):
        lens = [(1, 9), (7, 3), (32, 20), (50, 12)] if round_ != 1 else [(64, 5), (63, 2), (65, 70)]
        seqs = [random_tokens(p + d, V, 100 * round_ + i) for i, (p, d) in enumerate(lens)]
        slots = [eng.alloc_slot() for _ in seqs]
        got = [[] for _ in seqs]
        out = eng.step([StepItem(slots[i], seqs[i][:p], list(range(p))) for i, (p, d) in enumerate(lens)])
        o = 0
        for i, (p, d) in enumerate(lens):
            got[i].append(out[o:o + p]); o += p
        live = list(range(len(seqs)))
        t = 0
        while live:
            live = [i for i in live if t < lens[i][1]]
            if not live:
                break
            out = eng.step([StepItem(slots[i], [seqs[i][lens[i][0] + t]], [0]) for i in live])
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
            for i in list(live):
                if t + 1 >= lens[i][1]:
                    eng.free_slot(slots[i]); slots[i] = None
            t += 1
        for i in range(len(seqs)):
            _check(folders[name], seqs[i], torch.cat(got[i]), dtype, f"{name} {dtype} round {round_} request {i}")
        eng.cache.check()
        assert eng.cache.slots.n_held == 0 and all(g.pages.n_held == 0 for g in eng.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "D"])
def test_a_batch_of_twenty_decodes(folders, name, dtype):
    """Twenty unequal prompts in one step, then six tokens each: the batch sizes between the few
    tokens of the other tests and a prompt's many have kernels of their own."""
    from skyla_kernel_b200.engine import StepItem
    V = TINY[name][0]["vocab_size"]
    eng = _engine(folders[name], dtype, max_tokens=20 * 128)
    lens = [3 + (7 * i) % 38 for i in range(20)]
    seqs = [random_tokens(p + 6, V, 300 + i) for i, p in enumerate(lens)]
    slots = [eng.alloc_slot() for _ in seqs]
    out = eng.step([StepItem(slots[i], seqs[i][:p], list(range(p))) for i, p in enumerate(lens)])
    got, o = [], 0
    for p in lens:
        got.append([out[o:o + p]]); o += p
    for t in range(6):
        out = eng.step([StepItem(slots[i], [seqs[i][p + t]], [0]) for i, p in enumerate(lens)])
        for i in range(len(seqs)):
            got[i].append(out[i:i + 1])
    for i in range(len(seqs)):
        _check(folders[name], seqs[i], torch.cat(got[i]), dtype, f"{name} {dtype} batch of twenty, request {i}")
    for sl in slots:
        eng.free_slot(sl)
    eng.cache.check()


def test_the_wide_configuration_reaches_the_blackwell_kernels(folders):
    """Configuration D is there for the kernels that small sizes never reach: a prompt of 150 tokens
    must go through the token-major product (with its tiles cut along K) and the tcgen05 attention."""
    from skyla_kernel_b200.engine import StepItem
    from skyla_kernel_b200.kernels import ops
    base = TINY["D"][0]
    eng = _engine(folders["D"], "bfloat16")
    before = dict(ops.LAUNCHES_BY_MODULE)
    s = eng.alloc_slot()
    eng.step([StepItem(s, random_tokens(150, base["vocab_size"], 1), [149])])
    eng.free_slot(s)
    made = {m: n - before.get(m, 0) for m, n in ops.LAUNCHES_BY_MODULE.items()}
    L = base["num_hidden_layers"]
    assert made.get("gemm_prompt", 0) == 4 * L, made   # q/k/v, o, gate+up, down
    assert made.get("attention_tc", 0) == L, made
    assert made.get("attn_prep", 0) == 0, made          # the heads are finished in the q/k/v product
    if torch.cuda.get_device_properties(0).multi_processor_count >= 64:
        assert ops.prompt_cut_blocks(150, base["hidden_size"], base["hidden_size"], False, "cuda:0") > 0
