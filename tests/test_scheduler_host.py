"""The scheduler's decisions, with a stand-in for the model (no GPU)."""
import pytest

from cajeta_llm_b200.cache.pages import CacheBooks, GroupSpec
from cajeta_llm_b200.engine.scheduler import FinishReason, RequestState, Scheduler, SchedulerError
from cajeta_llm_b200.engine.step import OutOfPages
from cajeta_llm_b200.sampling.params import SamplingParams


class FakeCache:
    def __init__(self, books):
        self.books = books

    def pages_needed(self, slot, n):
        return self.books.pages_needed(slot, n)

    def pages_to_hold(self, slot, n, step_tokens=0):
        return self.books.pages_to_hold(slot, n, step_tokens)

    def free_pages(self):
        return self.books.free_pages()

    def length(self, slot):
        return int(self.books.length[slot])


class FakeRunner:
    """Keeps the books like the real runner and 'computes' a next token from the
    request's whole history, so that any loss of cached tokens would show."""

    def __init__(self, pages, page_tokens=4, max_seqs=4, ctx=256, groups=None):
        groups = groups or [GroupSpec(1, 8, 0)]
        counts = pages if isinstance(pages, (list, tuple)) else [pages] * len(groups)
        self.books = CacheBooks(groups, list(counts), page_tokens, max_seqs, ctx)
        self.cache = FakeCache(self.books)
        self.history = {}
        self.log = []

    def admit(self):
        s = self.books.admit()
        if s is not None:
            self.history[s] = []
        return s

    def release(self, slot):
        self.books.release(slot)
        del self.history[slot]

    def step(self, entries):
        self.log.append([(e.slot, len(e.tokens), list(e.want)) for e in entries])
        needs = [self.books.pages_needed(e.slot, len(e.tokens)) for e in entries]
        if not self.books.fits(needs):
            raise OutOfPages("no pages")
        out = []
        for e in entries:
            assert self.books.reserve(e.slot, len(e.tokens))
            self.books.commit(e.slot, len(e.tokens))
            self.history[e.slot].extend(e.tokens)
            for w in e.want:
                assert w == len(e.tokens) - 1
                h = self.history[e.slot]
                out.append((sum((i + 1) * t for i, t in enumerate(h)) * 31 + len(h)) % 1000)
        self.books.check()
        return out


class FakeSampler:
    def sample(self, logits, params, rngs, histories):
        return list(logits)


def solo(prompt, n):
    r = FakeRunner(pages=64)
    s = Scheduler(r, FakeSampler(), max_batch_tokens=512)
    i = s.submit(prompt, SamplingParams(max_new_tokens=n))
    s.run_all()
    return s.request(i).generated


def test_chunking_does_not_change_the_tokens():
    prompt = list(range(3, 30))
    want = solo(prompt, 6)
    for chunk, budget in ((1, 512), (4, 512), (64, 512), (0, 5), (0, 2)):
        r = FakeRunner(pages=64)
        s = Scheduler(r, FakeSampler(), max_batch_tokens=budget, chunk=chunk)
        i = s.submit(prompt, SamplingParams(max_new_tokens=6))
        s.run_all()
        assert s.request(i).generated == want
        assert s.request(i).finish_reason == FinishReason.BUDGET
        cap = min(chunk or budget, budget)
        assert all(n <= cap for step in r.log for _, n, _ in step)
        assert all(sum(n for _, n, _ in step) <= budget for step in r.log)


def test_decode_tokens_come_first_and_prompt_portions_fill_the_budget():
    r = FakeRunner(pages=64)
    s = Scheduler(r, FakeSampler(), max_batch_tokens=8)
    a = s.submit([1, 2, 3], SamplingParams(max_new_tokens=20))
    s.step_once()                                    # a: whole prompt
    b = s.submit(list(range(40)), SamplingParams(max_new_tokens=2))
    s.step_once()
    slot_a, slot_b = s.request(a).slot, s.request(b).slot
    assert r.log[-1] == [(slot_a, 1, [0]), (slot_b, 7, [])]          # one decode token beside a portion of 7
    for _ in range(4):
        s.step_once()
        assert r.log[-1][0] == (slot_a, 1, [0]) and r.log[-1][1][1] == 7     # a emits every iteration
    s.run_all()
    assert s.request(a).generated == solo([1, 2, 3], 20)
    assert s.request(b).generated == solo(list(range(40)), 2)


def test_admission_waits_for_pages_and_follows_completion_in_the_same_step():
    r = FakeRunner(pages=8, page_tokens=4)                           # 32 tokens of cache
    s = Scheduler(r, FakeSampler(), max_batch_tokens=64)
    a = s.submit(list(range(18)), SamplingParams(max_new_tokens=2))  # 5 pages + headroom
    b = s.submit(list(range(50, 62)), SamplingParams(max_new_tokens=3))      # 3 pages + headroom: does not fit beside a
    s.step_once()
    assert s.request(a).state == RequestState.RUNNING and s.request(b).state == RequestState.WAITING
    s.step_once()                                                    # a finishes; b admitted at the end of this iteration
    assert s.request(a).is_done and s.request(b).state == RequestState.RUNNING
    s.run_all()
    assert s.request(b).generated == solo(list(range(50, 62)), 3)
    assert s.counters.preempted == 0
    assert r.books.free_pages() == [8]


def test_no_free_slot_means_waiting():
    r = FakeRunner(pages=64, max_seqs=2)
    s = Scheduler(r, FakeSampler(), max_batch_tokens=64)
    ids = [s.submit([5 + i, 6, 7], SamplingParams(max_new_tokens=3)) for i in range(3)]
    s.step_once()
    assert [s.request(i).state for i in ids] == [RequestState.RUNNING, RequestState.RUNNING, RequestState.WAITING]
    s.run_all()
    assert all(s.request(i).generated == solo([5 + k, 6, 7], 3) for k, i in enumerate(ids))


def test_when_pages_run_out_the_youngest_is_preempted_and_recomputed():
    r = FakeRunner(pages=6, page_tokens=4)                           # 24 tokens of cache
    s = Scheduler(r, FakeSampler(), max_batch_tokens=64)
    a = s.submit(list(range(7)), SamplingParams(max_new_tokens=12))
    b = s.submit(list(range(20, 27)), SamplingParams(max_new_tokens=12))
    s.run_all()
    assert s.counters.preempted >= 1 and s.counters.resumed == s.counters.preempted
    assert s.counters.recomputed_tokens > 0
    assert s.request(a).generated == solo(list(range(7)), 12)         # the older one was never disturbed
    assert s.request(b).generated == solo(list(range(20, 27)), 12)    # the preempted one resumes identically
    assert r.books.free_pages() == [6]
    r.books.check()


def test_a_request_that_can_never_fit_is_refused_loudly():
    r = FakeRunner(pages=2, page_tokens=4)
    s = Scheduler(r, FakeSampler(), max_batch_tokens=64)
    s.submit(list(range(9)), SamplingParams(max_new_tokens=1))
    with pytest.raises(SchedulerError, match="can never fit"):
        s.run_all()
    r2 = FakeRunner(pages=3, page_tokens=4)
    s2 = Scheduler(r2, FakeSampler(), max_batch_tokens=64)
    s2.submit(list(range(6)), SamplingParams(max_new_tokens=30))       # fits at first, outgrows the pool alone
    with pytest.raises(SchedulerError, match="even alone"):
        s2.run_all()


def test_stop_tokens_budget_cancel_and_sink():
    want = solo([9, 8, 7], 8)
    r = FakeRunner(pages=64)
    s = Scheduler(r, FakeSampler(), max_batch_tokens=64, eog_token_ids=(want[3],))
    seen = []
    s.sink = lambda rid, tok: seen.append((rid, tok))
    a = s.submit([9, 8, 7], SamplingParams(max_new_tokens=8))                          # engine's end set
    b = s.submit([9, 8, 7], SamplingParams(max_new_tokens=8, stop_token_ids=(want[1],)))  # its own stop set
    c = s.submit([9, 8, 7], SamplingParams(max_new_tokens=8, stop_token_ids=()))
    s.step_once()
    assert s.cancel(c) and not s.cancel(c) and not s.cancel(99)
    s.run_all()
    assert s.request(a).generated == want[:4] and s.request(a).finish_reason == FinishReason.EOS
    assert s.request(b).generated == want[:2] and s.request(b).finish_reason == FinishReason.EOS
    assert s.request(c).finish_reason == FinishReason.CANCEL and s.request(c).generated == want[:1]
    assert [t for rid, t in seen if rid == a] == want[:4]
    assert r.books.free_pages() == [64 ]


def test_a_windowed_group_is_sized_by_its_window_not_by_the_request():
    """Two cache groups: one keeps every key, one a window of 10 tokens.  With steps of at most 6
    tokens a request never holds more than ceil((10 + 6) / 4) + 1 = 5 pages of the windowed
    group, so a pool of 2 x 5 + 1 pages serves two requests of 100 tokens, which would need 25
    pages each in a group that kept everything; admission counts accordingly."""
    groups = [GroupSpec(1, 8, 0), GroupSpec(1, 8, 10)]
    r = FakeRunner(pages=[64, 11], page_tokens=4, max_seqs=2, ctx=128, groups=groups)
    s = Scheduler(r, FakeSampler(), max_batch_tokens=6)
    prompts = [list(range(5, 95)), list(range(200, 270))]
    ids = [s.submit(p, SamplingParams(max_new_tokens=10)) for p in prompts]
    most = 0
    while s.has_work:
        s.step_once()
        for q in s.running:
            g = r.books.groups[1]
            most = max(most, int(g.next_page[q.slot]) - int(g.first_live[q.slot]))
        assert len(s.running) == 2 or not s.waiting              # both run side by side from the start
    assert 3 <= most <= 5 and s.counters.preempted == 0      # seen after each step, when the pages behind the window are back
    want = []
    for p in prompts:
        solo_runner = FakeRunner(pages=64, groups=groups)
        one = Scheduler(solo_runner, FakeSampler(), max_batch_tokens=512)
        i = one.submit(p, SamplingParams(max_new_tokens=10))
        one.run_all()
        want.append(one.request(i).generated)
    assert [s.request(i).generated for i in ids] == want
    assert r.books.free_pages() == [64, 11]
    r.books.check()
    # in one step of a whole request the windowed group would need as much as the other one
    slot = r.books.admit()
    assert r.books.pages_to_hold(slot, 90) == [23, 23] and r.books.pages_to_hold(slot, 90, 6) == [23, 5]
