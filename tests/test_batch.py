"""The step's packed arrays, built on the host (no GPU): tokens, positions, wanted rows, token tiles
of the heights the mixers asked for, page lists of a fixed width."""
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
    assert (seq, tok0, rows) == ([0, 0, 0, 1, 2], [0, 64, 128, 130, 131], [64, 64, 2, 1, 3])
    seq, tok0, rows = (t.tolist() for t in ctx.tiles[16])
    assert seq == [0] * 9 + [1, 2] and tok0[:9] == list(range(0, 130, 16)) and rows[8:] == [2, 1, 3]
    assert int(ctx.pages_needed) == 3 and all(p.shape == (3, 3) for p in ctx.pages)
    for g in range(2):
        for row, slot in enumerate((a, b, c)):
            held = cache.pages_of(g, slot)
            assert ctx.pages[g][row, :len(held)].tolist() == held
    # a fixed width keeps the layout of a decode step the same from step to step (recorded graphs rely on it)
    cache.advance([(a, 130), (b, 1), (c, 3)])
    cache.reserve([(a, 1), (b, 1), (c, 1)])
    d = BatchBuilder(rt, cache, tile_heights=(64,)).build([StepItem(s, [9], [0]) for s in (a, b, c)], pages_width=8)
    assert d.is_decode and d.pages[0].shape == (3, 8) and d.tok_pos.tolist() == [130, 71, 3]
    assert [t.tolist() for t in d.tiles[64]] == [[0, 1, 2], [0, 1, 2], [1, 1, 1]]
    # no mixer asked for tiles: none are made
    assert BatchBuilder(rt, cache).build([StepItem(a, [9], [0])]).tiles == {}
