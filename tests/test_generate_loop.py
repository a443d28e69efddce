"""The generation loop's decisions, driven with a fake engine on the CPU."""
import pytest

from skyla_kernel_b200.engine.generate import Request, generate, plan_batches


class FakeBackend:
    """Counts what the loop does.  The "model": next token = (sum of the sequence) % 50."""

    def __init__(self, n_pages=8, page_size=64, max_slots=4):
        self.n_pages, self.page_size, self.max_slots = n_pages, page_size, max_slots
        self.free = list(range(max_slots))
        self.seqs = {}
        self.steps = []
        self.peak_pages = 0

    def alloc_slot(self):
        s = self.free.pop(0)
        self.seqs[s] = []
        return s

    def free_slot(self, s):
        assert s in self.seqs, "slot freed twice"
        del self.seqs[s]
        self.free.append(s)
        self.free.sort()

    def step(self, items):
        assert len({it.slot for it in items}) == len(items)
        kinds = {len(self.seqs[it.slot]) == 0 for it in items}
        assert len(kinds) == 1, "a step mixes starting and continuing sequences"
        if False in kinds:
            assert all(len(it.tokens) == 1 for it in items)
        for it in items:
            self.seqs[it.slot].extend(it.tokens)
            assert list(it.want) == [len(it.tokens) - 1]
        self.steps.append([it.slot for it in items])
        pages = sum(-(-len(v) // self.page_size) for v in self.seqs.values())
        assert pages <= self.n_pages
        self.peak_pages = max(self.peak_pages, pages)
        return [sum(self.seqs[it.slot]) % 50 for it in items]

    def sample(self, logits, req_ids, steps):
        self.last_keys = (list(req_ids), list(steps))
        return list(logits)


def _expect(prompt, n, stops=(), emit_stop=False):
    seq, out = list(prompt), []
    for _ in range(n):
        t = sum(seq) % 50
        if t in stops:
            if emit_stop:
                out.append(t)
            return out, "stop"
        out.append(t)
        seq.append(t)
    return out, "length"


def test_unequal_prompts_shorter_requests_end_earlier():
    b = FakeBackend()
    reqs = [Request([1, 2, 3], 5), Request([4], 2), Request([5, 6], 9), Request([7] * 10, 1)]
    done = generate(b, reqs)
    for r, d in zip(reqs, done):
        assert (d.tokens, d.reason) == _expect(r.prompt, r.max_new_tokens)
    assert [len(s) for s in b.steps] == [4, 3, 2, 2, 2, 1, 1, 1, 1]  # rows shrink as requests end
    assert not b.seqs and b.free == [0, 1, 2, 3]


def test_stop_tokens_and_emit_option():
    reqs = [Request([3, 4], 20, stop_ids=(28,)), Request([1], 4, stop_ids=(2,))]
    for emit in (False, True):
        done = generate(FakeBackend(), reqs, emit_stop=emit)
        for r, d in zip(reqs, done):
            assert (d.tokens, d.reason) == _expect(r.prompt, r.max_new_tokens, r.stop_ids, emit)
    assert done[0].reason == "stop" and done[1].reason == "stop"


def test_batches_follow_one_another_and_reuse_slots():
    b = FakeBackend(n_pages=4, max_slots=2)
    reqs = [Request([i + 1] * (10 + i), 3) for i in range(5)]
    done = generate(b, reqs, max_batch=8)
    for r, d in zip(reqs, done):
        assert (d.tokens, d.reason) == _expect(r.prompt, 3)
    firsts = [s for s in b.steps if len(s) == 2 or s == [0]]
    assert b.steps[0] == [0, 1] and b.steps[3] == [0, 1] and b.steps[6] == [0]  # slots come back
    assert b.free == [0, 1]


def test_plan_respects_pages_batch_and_slots():
    reqs = [Request([0] * 100, 28), Request([0] * 10, 10), Request([0] * 64, 1), Request([0] * 1, 200)]
    assert plan_batches(reqs, n_pages=4, page_size=64, max_batch=8, max_slots=8) == [[0, 1], [2], [3]]
    assert plan_batches(reqs, n_pages=64, page_size=64, max_batch=3, max_slots=8) == [[0, 1, 2], [3]]
    assert plan_batches(reqs, n_pages=64, page_size=64, max_batch=8, max_slots=1) == [[0], [1], [2], [3]]
    with pytest.raises(ValueError, match="cache"):
        plan_batches(reqs, n_pages=3, page_size=64, max_batch=8, max_slots=8)
    with pytest.raises(ValueError, match="empty prompt"):
        plan_batches([Request([], 3)], 4, 64, 8, 8)


def test_sampler_keys_are_request_and_step():
    b = FakeBackend()
    generate(b, [Request([1], 3), Request([2], 1), Request([3], 3)])
    assert b.last_keys == ([0, 2], [2, 2])  # request indices and how many tokens each has so far


def test_zero_new_tokens_and_failure_frees_slots():
    b = FakeBackend()
    done = generate(b, [Request([1, 2], 0), Request([3], 2)])
    assert done[0].tokens == [] and done[0].reason == "length" and len(done[1].tokens) == 2
    assert b.free == [0, 1, 2, 3]

    class Failing(FakeBackend):
        def step(self, items):
            if len(self.steps) == 2:
                raise RuntimeError("boom")
            return super().step(items)

    f = Failing()
    with pytest.raises(RuntimeError, match="boom"):
        generate(f, [Request([1], 9), Request([2], 9)])
    assert f.free == [0, 1, 2, 3] and not f.seqs
