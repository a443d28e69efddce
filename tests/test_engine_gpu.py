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


def test_a_hundred_sequences_decode_on_the_widest_token_tile(folders):
    """65 to 128 tokens a step go to the weight-streaming product with its widest token tile (K cut into
    a cluster, the next norm's input prepared on the way) and to a q/k/v preparation of their own: 100
    sequences of the wide configuration decode together."""
    from skyla_kernel_b200.engine import StepItem
    from skyla_kernel_b200.kernels import ops
    name, dtype = "D", "bfloat16"
    V = TINY[name][0]["vocab_size"]
    eng = _engine(folders[name], dtype, max_tokens=100 * 128)
    mixer = eng.model.blocks[0].mixer
    assert mixer.qkv.streams(100) and mixer.qkv.rows_plans[128][1] > 1
    assert not mixer.out.streams(100)      # 512 inputs are too few to cut: this one stays on the tile kernel
    lens = [2 + (11 * i) % 60 for i in range(100)]
    seqs = [random_tokens(p + 3, V, 900 + i) for i, p in enumerate(lens)]
    slots = [eng.alloc_slot() for _ in seqs]
    got = [[] for _ in seqs]
    out = eng.step([StepItem(slots[j], seqs[j][:lens[j]], [lens[j] - 1]) for j in range(100)])
    for j in range(100):
        got[j].append(out[j:j + 1])
    before = ops.LAUNCHES
    for t in range(3):
        out = eng.step([StepItem(slots[j], [seqs[j][lens[j] + t]], [0]) for j in range(100)])
        for j in range(100):
            got[j].append(out[j:j + 1])
    assert ops.LAUNCHES > before
    cfg, w = plain.read_folder(folders[name])
    for j in range(0, 100, 9):
        ref = plain.forward(cfg, w, seqs[j])[lens[j] - 1:]
        assert_close(torch.cat(got[j]), ref, dtype, f"request {j} of 100")
    for sl in slots:
        eng.free_slot(sl)
    eng.cache.check()
    eng.check_errors()


def test_more_sequences_than_attention_blocks(folders):
    """With more (sequence, key/value head) pairs than the decode attention has blocks, the step's pages are cut
    into even runs and a block reads the end of one pair and the beginning of the next: 120 sequences of
    unequal lengths (three key/value heads each) decode together, some of them across a page's end."""
    from skyla_kernel_b200.engine import StepItem
    from skyla_kernel_b200.kernels import ops
    name, dtype = "C", "bfloat16"
    V = TINY[name][0]["vocab_size"]
    eng = _engine(folders[name], dtype, max_tokens=120 * 192)
    lens = [2 + (37 * i) % 150 for i in range(120)]
    lens[5], lens[77] = 63, 127                       # their second new token opens a page
    seqs = [random_tokens(p + 3, V, 700 + i) for i, p in enumerate(lens)]
    slots = [eng.alloc_slot() for _ in seqs]
    got = [[] for _ in seqs]
    for i in range(0, 120, 30):                       # the prompts, thirty a step
        out = eng.step([StepItem(slots[j], seqs[j][:lens[j]], [lens[j] - 1]) for j in range(i, i + 30)])
        for k, j in enumerate(range(i, i + 30)):
            got[j].append(out[k:k + 1])
    for t in range(3):
        out = eng.step([StepItem(slots[j], [seqs[j][lens[j] + t]], [0]) for j in range(120)])
        for j in range(120):
            got[j].append(out[j:j + 1])
    # what the attention part asked for: fewer blocks than pairs, so even runs
    plan = eng.model.step_plans()[0]
    n_blocks = plan.blocks(120, 8)
    assert n_blocks < 120 * plan.nkv
    rows = ops.decode_plan([p + 2 for p in lens], plan.nkv, plan.window, 64, n_blocks)[: 8 * n_blocks].reshape(-1, 8)
    assert rows[:, 3].max() <= -(-sum(-(-(p + 3) // 64) for p in lens) * plan.nkv // n_blocks)
    cfg, w = plain.read_folder(folders[name])
    for j in range(0, 120, 7):
        ref = plain.forward(cfg, w, seqs[j])[lens[j] - 1:]
        assert_close(torch.cat(got[j]), ref, dtype, f"request {j} of 120")
    for sl in slots:
        eng.free_slot(sl)
    eng.cache.check()
    eng.check_errors()


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


def _feed(eng, slot, toks, cuts):
    """Feed ``toks`` to ``slot`` in steps of the sizes ``cuts`` (their sum is the length); all logits."""
    from skyla_kernel_b200.engine import StepItem
    rows, o = [], 0
    for c in cuts:
        rows.append(eng.step([StepItem(slot, toks[o:o + c], list(range(c)))]))
        o += c
    assert o == len(toks)
    return torch.cat(rows)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "D"])
def test_mixed_chunks_of_one_request(folders, name, dtype):
    """A request cut into chunks of many tokens that land on a filled cache (the reference cuts its
    prompts at 128, skyla-engine/src/engine.rs:144-152): 50, 30, 1, 140 (from 129 tokens on the
    token-major product finishes the heads and the tcgen05 attention starts inside a sequence), a few
    single tokens, a chunk that starts inside a page, single tokens again."""
    from skyla_kernel_b200.kernels import ops
    V = TINY[name][0]["vocab_size"]
    eng = _engine(folders[name], dtype)
    cuts = [50, 30, 1, 140, 1, 1, 1, 37, 1, 1]
    toks = random_tokens(sum(cuts), V, 41)
    s = eng.alloc_slot()
    before = dict(ops.LAUNCHES_BY_MODULE)
    got = _feed(eng, s, toks, cuts)
    eng.free_slot(s)
    _check(folders[name], toks, got, dtype, f"{name} {dtype} mixed chunks {cuts}")
    if name == "D" and dtype == "bfloat16":
        made = {m: n - before.get(m, 0) for m, n in ops.LAUNCHES_BY_MODULE.items()}
        L = TINY[name][0]["num_hidden_layers"]
        assert made.get("gemm_prompt", 0) >= 4 * L and made.get("attention_tc", 0) >= L, made
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "D"])
def test_steps_that_mix_chunks_and_single_tokens(folders, name, dtype):
    """Steps in which one sequence brings a chunk on a filled cache while its neighbours bring one
    token each: few tokens in all (the weight-streaming products), 17 to 64, and 129 and more."""
    from skyla_kernel_b200.engine import StepItem
    V = TINY[name][0]["vocab_size"]
    eng = _engine(folders[name], dtype, max_tokens=4 * 320)
    # per step, the tokens each of the four sequences brings
    plan = [(60, 7, 33, 90), (40, 1, 1, 1), (1, 130, 1, 1), (1, 1, 1, 1), (1, 1, 17, 20), (3, 1, 2, 1),
            (1, 1, 1, 1), (1, 64, 1, 65), (1, 1, 1, 1)]
    total = [sum(p[i] for p in plan) for i in range(4)]
    seqs = [random_tokens(total[i], V, 500 + i) for i in range(4)]
    slots = [eng.alloc_slot() for _ in seqs]
    got = [[] for _ in seqs]
    at = [0] * 4
    for p in plan:
        out = eng.step([StepItem(slots[i], seqs[i][at[i]:at[i] + p[i]], list(range(p[i]))) for i in range(4)])
        o = 0
        for i in range(4):
            got[i].append(out[o:o + p[i]]); o += p[i]; at[i] += p[i]
        assert o == out.shape[0]
    for i in range(4):
        _check(folders[name], seqs[i], torch.cat(got[i]), dtype, f"{name} {dtype} mixed steps, request {i}")
        eng.free_slot(slots[i])
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "D"])
@pytest.mark.parametrize("prompt", [500, 1010])
def test_decoding_across_a_page_list_bucket(folders, name, dtype, prompt):
    """Decode steps replay graphs recorded per (batch, width of the page lists); at 512 and 1,024
    positions a sequence moves to a wider list, a new graph, other context splits and longer rotary
    tables.  A long request decodes across that edge beside a short neighbour; every row is compared."""
    from skyla_kernel_b200.engine import StepItem
    V = TINY[name][0]["vocab_size"]
    eng = _engine(folders[name], dtype, max_tokens=1280)
    n_dec = 40
    long_, short = random_tokens(prompt + n_dec, V, 61), random_tokens(9 + n_dec, V, 62)
    a, b = eng.alloc_slot(), eng.alloc_slot()
    out = eng.step([StepItem(a, long_[:prompt], [prompt - 2, prompt - 1]), StepItem(b, short[:9], list(range(9)))])
    got_a, got_b = [out[:2]], [out[2:]]
    keys = set()
    for t in range(n_dec):
        out = eng.step([StepItem(a, [long_[prompt + t]], [0]), StepItem(b, [short[9 + t]], [0])])
        got_a.append(out[:1]); got_b.append(out[1:])
        if eng.graphs is not None:
            keys.add(eng.graphs.last_key)
    if eng.graphs is not None:
        assert len(keys) == 2, f"the decode crossed no bucket: {keys}"
    if folders[name] not in _MODELS:
        _MODELS[folders[name]] = plain.read_folder(folders[name])
    cfg, w = _MODELS[folders[name]]
    ref = plain.forward(cfg, w, long_)
    assert_close(torch.cat(got_a), ref[prompt - 2:], dtype, f"{name} {dtype} long request across position {prompt}")
    _check(folders[name], short, torch.cat(got_b), dtype, f"{name} {dtype} the short neighbour")
    eng.free_slot(a); eng.free_slot(b)
    eng.cache.check()


@pytest.mark.parametrize("name", NAMES)
def test_float32_logits_are_the_same_bits_in_every_cut(folders, name):
    """In the 32-bit path every output element is summed in one order that the batch does not change:
    whole, in chunks, token by token, and beside other requests give equal bits, not close ones."""
    from skyla_kernel_b200.engine import StepItem
    V = TINY[name][0]["vocab_size"]
    eng = _engine(folders[name], "float32", max_tokens=2048)
    n = 150
    toks = random_tokens(n, V, 77)
    others = [random_tokens(m, V, 78 + i) for i, m in enumerate((140, 20, 66))]
    s = eng.alloc_slot()
    whole = _feed(eng, s, toks, [n]); eng.free_slot(s)
    s = eng.alloc_slot()
    chunks = _feed(eng, s, toks, [50, 30, 1, 37, 32]); eng.free_slot(s)
    s = eng.alloc_slot()
    single = _feed(eng, s, toks, [n - 32] + [1] * 32); eng.free_slot(s)
    # beside others: the prompt in a batch of unequal prompts, then tokens beside a chunk and single tokens
    slots = [eng.alloc_slot() for _ in range(4)]
    out = eng.step([StepItem(slots[1], others[0][:100], [99]), StepItem(slots[0], toks[:90], list(range(90))),
                    StepItem(slots[2], others[1][:5], [4]), StepItem(slots[3], others[2][:66], [65])])
    rows = [out[1:91]]
    for t in range(90, n):
        j = t - 90
        items = [StepItem(slots[0], [toks[t]], [0])]
        if j < 15:
            items.insert(0, StepItem(slots[2], [others[1][5 + j]], [0]))
        if j == 3:
            items.append(StepItem(slots[1], others[0][100:140], [39]))
        out = eng.step(items)
        rows.append(out[1:2] if j < 15 else out[0:1])
    batched = torch.cat(rows)
    for sl in slots:
        eng.free_slot(sl)
    for what, got in (("chunks", chunks), ("token by token", single), ("beside other requests", batched)):
        assert torch.equal(whole, got), (f"{name} float32 {what}: differs from the whole run in "
                                         f"{int((whole != got).any(-1).sum())} rows, first row "
                                         f"{int((whole != got).any(-1).nonzero()[0])}, "
                                         f"largest difference {float((whole - got).abs().max()):.3e}")
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_layer_taps(folders, name, dtype):
    """The residual stream after every layer, read through ``Engine.step(taps=...)`` (the reference's
    ``Engine::residuals``, skyla-engine/src/taps.rs:7-46), against the plain implementation's: the
    tool for finding the layer in which a difference starts."""
    from skyla_kernel_b200.engine import StepItem
    base = TINY[name][0]
    V, L, H = base["vocab_size"], base["num_hidden_layers"], base["hidden_size"]
    eng = _engine(folders[name], dtype)
    toks = random_tokens(70, V, 91)
    s = eng.alloc_slot()
    # a prompt, then two single tokens (with taps a decode step runs eagerly, not as a graph)
    got = {i: [] for i in range(L)}
    for lo, hi in ((0, 68), (68, 69), (69, 70)):
        taps = {i: torch.empty(hi - lo, H, dtype=torch.float32, device="cuda:0") for i in range(L)}
        eng.step([StepItem(s, toks[lo:hi], [hi - lo - 1])], taps=taps)
        for i in range(L):
            got[i].append(taps[i].cpu())
    eng.free_slot(s)
    cfg, w = plain.read_folder(folders[name])
    ref = []
    plain.forward(cfg, w, toks, taps=ref)
    assert len(ref) == L
    for i in range(L):
        assert_close(torch.cat(got[i]), ref[i], dtype, f"{name} {dtype} residual stream after layer {i}")


@pytest.mark.parametrize("name", NAMES)
def test_bfloat16_on_models_with_flat_attention_within_tighter_limits(tmp_path_factory, name):
    """The sharp models of the other tests make rounding noise large, and the limits with it.  The same
    comparisons on models with unit q/k norm weights have a sixth of the noise and limits to match: whole,
    the last 32 one by one, and an unequal batch whose requests then decode together."""
    from skyla_kernel_b200.engine import StepItem
    folder = make_folder(tmp_path_factory.mktemp("flat"), name, sharp=1.0)
    eng = _engine(folder, "bfloat16")
    V = TINY[name][0]["vocab_size"]
    for n, seed in ((5, 4), (150, 6), (333, 9)):
        toks = random_tokens(n, V, seed)
        s = eng.alloc_slot()
        head = max(1, n - 32)
        rows = [eng.step([StepItem(s, toks[:head], list(range(head)))])]
        for t in range(head, n):
            rows.append(eng.step([StepItem(s, [toks[t]], [0])]))
        eng.free_slot(s)
        _check(folder, toks, torch.cat(rows), "bfloat16 flat", f"{name} flat, n={n}, last 32 one by one")
    lens = (70, 9, 200, 33)
    seqs = [random_tokens(n + 20, V, 40 + i) for i, n in enumerate(lens)]
    slots = [eng.alloc_slot() for _ in lens]
    got = [[] for _ in lens]
    first = eng.step([StepItem(s, q[:n], list(range(n))) for s, q, n in zip(slots, seqs, lens)])
    o = 0
    for i, n in enumerate(lens):
        got[i].append(first[o:o + n])
        o += n
    for t in range(20):
        step = eng.step([StepItem(s, [q[n + t]], [0]) for s, q, n in zip(slots, seqs, lens)])
        for i in range(len(lens)):
            got[i].append(step[i:i + 1])
    for i, q in enumerate(seqs):
        _check(folder, q, torch.cat(got[i]), "bfloat16 flat", f"{name} flat, request {i} of an unequal batch")
    eng.check_errors()
