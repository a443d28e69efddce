"""What an engine's kernels keep between launches belongs to that engine, and what they report
reaches the host: two engines side by side, the error word, tokens that no table holds."""
import pytest
import torch

import plain_qwen3 as plain
from helpers import TINY, assert_close, make_folder, random_tokens

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    d = tmp_path_factory.mktemp("state")
    return {n: make_folder(d, n) for n in "BD"}


@pytest.mark.parametrize("name", ["B", "D"])
def test_two_engines_on_two_streams_step_side_by_side(folders, name):
    """Two engines of the same model, each on a stream of its own, fed different requests without a
    wait between them: counters, scratch and flags are per engine, so each gives what it gives alone.
    (Configuration D goes through the kernels that count arrivals and cut tiles along K.)"""
    from skyla_kernel_b200.engine import Engine, StepItem
    V = TINY[name][0]["vocab_size"]
    engines = [Engine.from_folder(folders[name], dtype="bfloat16", max_tokens=1024) for _ in range(2)]
    assert engines[0].rt.kernel_state is not engines[1].rt.kernel_state
    streams = [torch.cuda.Stream(device=DEV) for _ in range(2)]
    prompts = [[random_tokens(n, V, 900 + 10 * e + i) for i, n in enumerate((150, 40, 300))] for e in range(2)]
    n_dec = 12
    tails = [[random_tokens(n_dec, V, 950 + 10 * e + i) for i in range(3)] for e in range(2)]

    def run(order, sync):
        outs = [[] for _ in engines]
        slots = [[eng.alloc_slot() for _ in range(3)] for eng in engines]
        for t in range(-1, n_dec):
            for e in order:
                with torch.cuda.stream(streams[e]):
                    if t < 0:
                        items = [StepItem(s, p, [len(p) - 1]) for s, p in zip(slots[e], prompts[e])]
                    else:
                        items = [StepItem(s, [tl[t]], [0]) for s, tl in zip(slots[e], tails[e])]
                    outs[e].append(engines[e].step(items))
                if sync:
                    torch.cuda.synchronize()
        torch.cuda.synchronize()
        for e, eng in enumerate(engines):
            eng.check_errors()
            for s in slots[e]:
                eng.free_slot(s)
        return [torch.cat(o) for o in outs]

    alone = run([0, 1], sync=True)        # one step at a time, the device idle in between
    together = run([0, 1], sync=False)    # both engines' kernels in flight at once
    again = run([1, 0], sync=False)
    for e in range(2):
        assert torch.equal(alone[e], together[e]) and torch.equal(alone[e], again[e]), f"engine {e} was disturbed"
    cfg, w = plain.read_folder(folders[name])
    for i in range(3):  # and what they give is right: the last row of each request
        seq = prompts[0][i] + tails[0][i]
        ref = plain.forward(cfg, w, seq)[len(prompts[0][i]) - 1:]
        got = torch.stack([alone[0][i]] + [alone[0][3 * (t + 1) + i] for t in range(n_dec)])
        assert_close(got, ref, "bfloat16", f"{name} engine 0 request {i}")


def test_error_word_raises_and_clears_what_a_kernel_left(folders):
    """No wait is made to run out on purpose; the word a kernel would leave is written by hand, with
    the litter such a kernel leaves (raised flags, counters that did not come back to zero)."""
    from skyla_kernel_b200.engine import Engine, StepItem
    from skyla_kernel_b200.kernels.ops import KernelError
    eng = Engine.from_folder(folders["D"], dtype="bfloat16", max_tokens=512)
    V = TINY["D"][0]["vocab_size"]
    st = eng.rt.kernel_state
    s = eng.alloc_slot()
    toks = random_tokens(140, V, 5)
    first = eng.step([StepItem(s, toks, [139])])
    eng.check_errors()                       # nothing happened: no error
    eng.free_slot(s)
    st.error_flag.fill_(13)
    st.merge_counters()[:7].fill_(2)
    st.prompt_shares()[1].fill_(1)
    with pytest.raises(KernelError, match="bounded wait ran out .code 13."):
        eng.check_errors()
    assert int(st.error_flag) == 0 and int(st.merge_counters().abs().sum()) == 0
    assert int(st.prompt_shares()[1].abs().sum()) == 0
    eng.check_errors()                       # cleared: the next check passes
    s = eng.alloc_slot()
    again = eng.step([StepItem(s, toks, [139])])
    eng.check_errors()
    assert torch.equal(first, again)         # and the engine works as before
    # the generation loop reads the word with every step's tokens
    import skyla_kernel_b200 as skyla
    model = skyla.Model(eng)
    eng.free_slot(s)
    st.error_flag.fill_(2)
    with pytest.raises(KernelError, match="code 2"):
        model.generate([toks[:9]], max_new_tokens=4, stop_ids=[])
    assert eng.cache.slots.n_held == 0       # the loop gave its slots back on the way out
    assert model.generate([toks[:9]], max_new_tokens=4, stop_ids=[])[0] == model.generate([toks[:9]], max_new_tokens=4, stop_ids=[])[0]


def test_a_row_of_nan_logits_gives_a_valid_token_and_is_reported():
    """Every logit NaN: nothing compares, so no candidate is ever taken.  The sampler then gives token 0
    (inside every vocabulary) and raises the error word, greedy and with a temperature."""
    from skyla_kernel_b200.kernels import ops
    st = ops.KernelState(DEV)
    logits = torch.randn(3, 777, device=DEV)
    logits[1] = float("nan")
    ids = torch.zeros(3, dtype=torch.int32, device=DEV)
    for temperature in (0.0, 0.8):
        out = torch.full((3,), -1, dtype=torch.int32, device=DEV)
        ops.sample(logits, out, temperature, 0, 1.0, 7, ids, ids, state=st)
        got = out.tolist()
        assert got[1] == 0 and all(0 <= t < 777 for t in got)
        assert got[0] == int(logits[0].argmax()) or temperature > 0
        with pytest.raises(ops.KernelError, match="no token in a row of logits"):
            st.check()
        st.check()
    # a row with some NaN among numbers is not an error: the numbers compete
    logits[1] = torch.randn(777, device=DEV)
    logits[1, ::2] = float("nan")
    out = torch.full((3,), -1, dtype=torch.int32, device=DEV)
    ops.sample(logits, out, state=st)
    assert out[1].item() % 2 == 1
    st.check()


def test_a_token_outside_the_table_reads_nothing():
    from skyla_kernel_b200.kernels import ops
    st = ops.KernelState(DEV)
    table = torch.randn(50, 24, device=DEV).to(torch.bfloat16)
    tokens = torch.tensor([3, 0x7fffffff, 49, -1, 50], dtype=torch.int32, device=DEV)
    out = torch.full((5, 24), float("nan"), device=DEV)
    ops.embed_gather(tokens, table, out, state=st)
    assert torch.equal(out[0], table[3].float()) and torch.equal(out[2], table[49].float())
    assert (out[[1, 3, 4]] == 0).all()
    with pytest.raises(ops.KernelError, match="outside the embedding table"):
        st.check()
    ops.embed_gather(tokens[:1], table, out[:1], state=st)
    st.check()
