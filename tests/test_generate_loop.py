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


class AsyncFake(FakeBackend):
    """The same model with the pipelined interface; counts steps that ran for nothing."""

    class Handle:
        def __init__(self, toks):
            self.device_tokens = toks  # a list stands in for device memory
            self.asked = False

        def tokens(self):
            self.asked = True
            return list(self.device_tokens)

    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        self.handles = []
        self.keys = []

    def step_async(self, items, req_ids, steps):
        fed = [it for it in items if it.device_token is not None]
        if fed:
            assert len(fed) == len(items)
            for it in items:
                h, row = it.device_token
                assert not h.asked or True  # the tokens may or may not have been read on the host yet
                it.tokens = [h.device_tokens[row]]
        out = self.step(items)
        self.keys.append((list(req_ids), list(steps)))
        h = AsyncFake.Handle(out)
        self.handles.append(h)
        return h


def _same_results(reqs, emit=False, **kw):
    a = generate(FakeBackend(**kw), reqs, emit_stop=emit)
    b_backend = AsyncFake(**kw)
    b = generate(b_backend, reqs, emit_stop=emit)
    assert [(x.tokens, x.reason) for x in a] == [(x.tokens, x.reason) for x in b]
    assert not b_backend.seqs and b_backend.free == sorted(b_backend.free) and len(b_backend.free) == b_backend.max_slots
    return a, b_backend


def test_pipelined_loop_gives_the_same_results():
    reqs = [Request([1, 2, 3], 5), Request([4], 2), Request([5, 6], 9), Request([7] * 10, 1)]
    done, b = _same_results(reqs)
    for r, d in zip(reqs, done):
        assert (d.tokens, d.reason) == _expect(r.prompt, r.max_new_tokens)
    # ends by count are known beforehand: no step runs for nothing
    assert [len(s) for s in b.steps] == [4, 3, 2, 2, 2, 1, 1, 1, 1]
    # the sampler's keys are (request, tokens generated before this one)
    assert b.keys[0] == ([0, 1, 2, 3], [0, 0, 0, 0]) and b.keys[1] == ([0, 1, 2], [1, 1, 1])


def test_pipelined_loop_finds_stop_tokens_a_step_late_and_drops_the_extra_token():
    reqs = [Request([3, 4], 20, stop_ids=(28,)), Request([1], 6, stop_ids=(2,)), Request([9], 4)]
    for emit in (False, True):
        done, b = _same_results(reqs, emit)
        assert done[0].reason == "stop" and done[1].reason == "stop" and done[2].reason == "length"
    # request 1 stops at its 2nd token; the step after that still carried it (3 rows), the next did not
    assert [len(s) for s in b.steps][:4] == [3, 3, 3, 2]


def test_pipelined_loop_batches_zero_tokens_and_failures():
    reqs = [Request([i + 1] * (10 + i), 3) for i in range(5)] + [Request([1, 2], 0)]
    _same_results(reqs, n_pages=4, max_slots=2)

    class Failing(AsyncFake):
        def step_async(self, items, req_ids, steps):
            if len(self.steps) == 2:
                raise RuntimeError("boom")
            return super().step_async(items, req_ids, steps)

    f = Failing()
    with pytest.raises(RuntimeError, match="boom"):
        generate(f, [Request([1], 9), Request([2], 9)])
    assert f.free == [0, 1, 2, 3] and not f.seqs


def test_lockstep_check_tells_a_near_tie_from_a_disagreement():
    """``skyla run --check`` fails on a top-1 disagreement unless the oracle's two most likely tokens are
    within two points of probability (the reference's rule, docs/roadmap.md:89-92 and 206-212: "France"
    0.1799 against "Italy" 0.1680 counted as a near tie)."""
    import math

    import torch

    from skyla_kernel_b200.cli import judge, near_tie
    base = torch.full((50,), -4.0)
    prob = torch.full((50,), (1.0 - 0.1799 - 0.1680) / 48)
    prob[3], prob[7] = 0.1799, 0.1680
    tie = torch.log(prob)
    assert near_tie(tie)
    moved = tie.clone(); moved[7] += 0.2
    assert judge(moved, tie)[3] == "near tie" and judge(moved, tie)[:2] == (7, 3)
    clear = base.clone(); clear[3], clear[7] = 2.0, 1.0
    assert not near_tie(clear)
    wrong = clear.clone(); wrong[7] = 2.5
    assert judge(wrong, clear)[3] == "DISAGREE"
    assert judge(clear + 0.01, clear)[3] == "" and abs(judge(clear + 0.01, clear)[2] - 0.01) < 1e-6
