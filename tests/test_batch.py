"""The step's packed arrays, built on the host (no GPU): tokens, positions, wanted rows, token tiles
of the heights the mixers asked for, page lists of a fixed width, and the plans that parts asked for."""
import numpy as np
import torch

from skyla_kernel_b200.cache import KVNeed, SequenceCache
from skyla_kernel_b200.engine.batch import BatchBuilder, StepItem
from skyla_kernel_b200.parts.base import Runtime


def test_packed_arrays_of_an_unequal_batch():
    rt = Runtime(torch.device("cpu"), "float32", n_sms=1)
    cache = SequenceCache([KVNeed(2, 16), KVNeed(1, 32, 100)], [None, None], 64 * 12, 4, torch.float32, None)
    a, b, c = cache.alloc_slot(), cache.alloc_slot(), cache.alloc_slot()
    cache.reserve([(b, 70)]); cache.advance([(b, 70)])           # b already holds 70 positions
    items = [StepItem(a, list(range(100, 230)), [0, 129]), StepItem(b, [7], [0]), StepItem(c, [1, 2, 3], [])]
    cache.reserve([(a, 130), (b, 1), (c, 3)])
    ctx = BatchBuilder(rt, cache, tile_heights=(64, 16)).build(items)
    assert (ctx.n_tokens, ctx.n_seqs, ctx.n_want, ctx.max_new, ctx.max_context, ctx.max_position) == (134, 3, 3, 130, 130, 129)
    assert not ctx.is_decode
    assert ctx.tokens.tolist() == list(range(100, 230)) + [7, 1, 2, 3]
    assert ctx.tok_pos.tolist() == list(range(130)) + [70, 0, 1, 2]
    assert ctx.tok_seq.tolist() == [0] * 130 + [1] + [2] * 3
    assert ctx.seq_slot.tolist() == [a, b, c] and ctx.seq_start.tolist() == [0, 70, 0] and ctx.seq_n.tolist() == [130, 1, 3]
    assert ctx.cu.tolist() == [0, 130, 131, 134] and ctx.want.tolist() == [0, 129, 130]
    seq, tok0, rows = (t.tolist() for t in ctx.tiles[64])
    # in ascending order of the last position a tile sees (the kernels start from the list's end): sequence c's
    # three tokens, a's first 64, b's token at position 70, a's next 64, a's last two
    assert (seq, tok0, rows) == ([2, 0, 1, 0, 0], [131, 0, 130, 64, 128], [3, 64, 1, 64, 2])
    seq, tok0, rows = (t.tolist() for t in ctx.tiles[16])
    assert seq == [2] + [0] * 4 + [1] + [0] * 5 and tok0[1:5] == [0, 16, 32, 48] and rows == [3] + [16] * 4 + [1] + [16] * 4 + [2]
    assert all(p.shape == (3, 3) for p in ctx.pages)
    for g in range(2):
        for row, slot in enumerate((a, b, c)):
            held = cache.pages_of(g, slot)
            assert ctx.pages[g][row, :len(held)].tolist() == held
    # a fixed width keeps the layout of a decode step the same from step to step (recorded graphs rely on it)
    cache.advance([(a, 130), (b, 1), (c, 3)])
    cache.reserve([(a, 1), (b, 1), (c, 1)])
    d = BatchBuilder(rt, cache, tile_heights=(64,)).build([StepItem(s, [9], [0]) for s in (a, b, c)], pages_width=8)
    assert d.is_decode and d.pages[0].shape == (3, 8) and d.tok_pos.tolist() == [130, 71, 3]
    assert [t.tolist() for t in d.tiles[64]] == [[2, 1, 0], [2, 1, 0], [1, 1, 1]]   # c holds the fewest positions
    # no mixer asked for tiles: none are made
    assert BatchBuilder(rt, cache).build([StepItem(a, [9], [0])]).tiles == {}


def _walk(plan, positions, nkv, window, n_blocks, page_size=64):
    """Follow a decode plan the way the kernel does: {(sequence, head): [(block, first page, pages)]}."""
    first = [max(0, p - window + 1) if window else 0 for p in positions]
    n_pages = [p // page_size + 1 - f // page_size for p, f in zip(positions, first)]
    rows, table = plan[: 8 * n_blocks].reshape(n_blocks, 8), plan[8 * n_blocks:].reshape(-1, 2)
    pieces = {}
    for j, (b, kvh, page0, left, pos, j_first, n_parts, _) in enumerate(rows.tolist()):
        if left:  # what the row says of the item it starts in is what the table says
            assert pos == positions[b] and [j_first, n_parts] == table[b * nkv + kvh].tolist()
        while left > 0:
            n = min(left, n_pages[b] - page0)
            assert n > 0
            pieces.setdefault((b, kvh), []).append((j, page0, n))
            left -= n
            page0 = 0
            kvh += 1
            if kvh == nkv:
                kvh, b = 0, b + 1
    return pieces, n_pages, rows, table


def test_decode_plan_deals_every_page_once_and_evenly():
    from skyla_kernel_b200.kernels import ops
    rng = np.random.default_rng(3)
    for nkv, window, n_seqs, n_blocks in ((8, 0, 64, 296), (2, 0, 5, 7), (1, 130, 9, 40), (3, 0, 1, 50), (4, 70, 16, 3),
                                          (8, 0, 16, 296), (2, 0, 3, 1), (8, 0, 8, 296)):
        positions = rng.integers(0, 3000, n_seqs).tolist()
        for even_only in (False, True):
            plan = ops.decode_plan(positions, nkv, window, 64, n_blocks, even_only=even_only)
            assert plan.shape == (ops.decode_plan_ints(n_seqs, nkv, n_blocks),) and plan.dtype == np.int32
            pieces, n_pages, rows, table = _walk(plan, positions, nkv, window, n_blocks)
            total = nkv * sum(n_pages)
            assert rows[:, 3].sum() == total
            assert sorted(pieces) == [(b, h) for b in range(n_seqs) for h in range(nkv)]
            for (b, h), got in pieces.items():
                # an item's pieces follow one another, page after page, in consecutive blocks, as the table says
                assert [p[1] for p in got] == [0] + list(np.cumsum([p[2] for p in got])[:-1])
                assert sum(p[2] for p in got) == n_pages[b]
                assert [p[0] for p in got] == list(range(got[0][0], got[0][0] + len(got)))
                assert table[b * nkv + h].tolist() == [got[0][0], len(got)]
            # slot = block + item is a piece's own
            slots = [j + b * nkv + h for (b, h), got in pieces.items() for j, _, _ in got]
            assert len(set(slots)) == len(slots) and max(slots) < n_blocks + n_seqs * nkv
            if even_only:  # nobody reads more than an even share
                assert rows[:, 3].max() <= -(-total // n_blocks)
            else:          # never slower than even runs, by the planner's own measure
                even = _walk(ops.decode_plan(positions, nkv, window, 64, n_blocks, even_only=True), positions, nkv,
                             window, n_blocks)[0]
                def cost(pc):
                    per_block = {}
                    for got in pc.values():
                        for j, _, n in got:
                            per_block[j] = per_block.get(j, 0) + n + 3
                    return max(per_block.values())
                assert cost(pieces) <= cost(even)
    # eight equal sequences and room for all: every item in equal pieces, no block starts a second item
    plan = ops.decode_plan([2100] * 8, 8, 0, 64, 296)
    pieces, _, rows, _ = _walk(plan, [2100] * 8, 8, 0, 296)
    assert all(len(got) == 4 and [n for _, _, n in got] == [8, 8, 8, 9] for got in pieces.values())
    assert (rows[:, 3] > 0).sum() == 256
    # sixty-four: more items than blocks, so the pages are cut evenly and a block reads into the next item
    plan = ops.decode_plan([2100] * 64, 8, 0, 64, 296)
    pieces, _, rows, _ = _walk(plan, [2100] * 64, 8, 0, 296)
    assert rows[:, 3].max() == -(-64 * 8 * 33 // 296) and max(len(got) for got in pieces.values()) == 2


def test_a_parts_plan_travels_with_the_step():
    from skyla_kernel_b200.parts.attention import DecodePages
    rt = Runtime(torch.device("cpu"), "float32", n_sms=4)
    cache = SequenceCache([KVNeed(2, 16)], [None], 64 * 12, 4, torch.float32, None)
    a, b = cache.alloc_slot(), cache.alloc_slot()
    cache.reserve([(a, 200), (b, 70)]); cache.advance([(a, 200), (b, 70)])
    plan = DecodePages(nkv=2, window=0, n_sms=4)
    builder = BatchBuilder(rt, cache, plans=(plan,))
    cache.reserve([(a, 1), (b, 1)])
    ctx = builder.build([StepItem(a, [5], [0]), StepItem(b, [6], [0])], pages_width=8)
    got = ctx.plans[plan.key]
    n_blocks = plan.blocks(2, 8)
    from skyla_kernel_b200.kernels import ops
    assert 1 <= n_blocks <= 8 and got.numel() == ops.decode_plan_ints(2, 2, n_blocks) and got.data_ptr() % 16 == 0
    assert np.array_equal(got.numpy(), ops.decode_plan([200, 70], 2, 0, 64, n_blocks))
    assert ctx.pages[0].shape == (2, 8) and ctx.tok_pos.tolist() == [200, 70]   # the arrays beside it are whole
    # a step that is no decode step has no such plan
    cache.advance([(a, 1), (b, 1)])
    cache.reserve([(a, 3)])
    assert builder.build([StepItem(a, [1, 2, 3], [])]).plans == {}


def test_any_part_can_ask_for_a_plan():
    """The mechanism knows nothing of attention: a plan of a test's own, for every kind of step."""
    from skyla_kernel_b200.parts.base import StepPlan

    class EndsOfSequences(StepPlan):
        key = ("toy", "ends")

        def size(self, n_seqs, pages_width, decode):
            return n_seqs + 1

        def fill(self, out, starts, ns, page_size):
            out[:-1] = starts + ns
            out[-1] = page_size

    rt = Runtime(torch.device("cpu"), "float32", n_sms=2)
    cache = SequenceCache([KVNeed(1, 16)], [None], 64 * 8, 4, torch.float32, None)
    a, b = cache.alloc_slot(), cache.alloc_slot()
    cache.reserve([(a, 70), (b, 3)])
    builder = BatchBuilder(rt, cache, tile_heights=(16,), plans=(EndsOfSequences(), EndsOfSequences()))
    ctx = builder.build([StepItem(a, list(range(70)), [69]), StepItem(b, [1, 2, 3], [])])
    assert ctx.plans[("toy", "ends")].tolist() == [70, 3, 64] and ctx.plans[("toy", "ends")].data_ptr() % 16 == 0
    assert ctx.tok_pos.tolist() == list(range(70)) + [0, 1, 2] and ctx.want.tolist() == [69]
    cache.advance([(a, 70), (b, 3)])
    cache.reserve([(a, 1), (b, 1)])
    ctx = builder.build([StepItem(a, [5], [0]), StepItem(b, [6], [0])], pages_width=8)
    assert ctx.plans[("toy", "ends")].tolist() == [71, 4, 64]
