"""The cache manager (no page lost, held twice or freed twice, under random orders of
requests), windowed groups giving pages back, and the scheduler's decisions on a scripted
step function (no GPU, no model)."""
import random

import pytest
import torch

from vapi_b200.cache import CacheManager, OutOfPages, OutOfSlots, PagePool, SlotPool
from vapi_b200.engine.scheduler import AdmitError, Scheduler, SchedulerConfig
from vapi_b200.engine.step import StepEntry, StepError, validate_step
from vapi_b200.parts.base import PagedSpec, StateSpec
from vapi_b200.sampling.params import FinishReason, SamplingParams


def make_cache(num_pages=8, page=16, max_requests=4, window=0, watermark=0.0, extra=()):
    sites = [(0, StateSpec("shortconv", (2, 8))), (1, PagedSpec.kv(2, 16, window)), (2, StateSpec("shortconv", (2, 8))),
             (3, PagedSpec.kv(2, 16, window))] + list(extra)
    return CacheManager(sites, page_size=page, num_pages=num_pages, max_requests=max_requests,
                        dtype=torch.float32, device="cpu", watermark=watermark)


def test_pool_refuses_double_free_and_exhaustion():
    p = PagePool(3)
    a, b, c = p.allocate(), p.allocate(), p.allocate()
    with pytest.raises(OutOfPages):
        p.allocate()
    p.free(b)
    with pytest.raises(ValueError, match="freed twice"):
        p.free(b)
    assert p.allocate() == b            # a freed page is handed out again first
    p.check_invariants()
    s = SlotPool(1)
    x = s.acquire()
    with pytest.raises(OutOfSlots):
        s.acquire()
    s.release(x)
    with pytest.raises(ValueError, match="released twice"):
        s.release(x)


def test_groups_and_tensors():
    c = make_cache(extra=[(4, PagedSpec.kv(1, 32, 0))])
    assert len(c.paged) == 2 and len(c.state) == 1
    # pages are flat: [sites, pages, page_size * elements per token]; the buffers are views into them
    assert c.paged[0].tensor.shape == (2, 8, 16 * 2 * 2 * 16) and c.paged[1].tensor.shape == (1, 8, 16 * 2 * 32)
    assert c.state[0].tensor.shape == (5, 2, 2, 8)          # 4 slots + the scratch slot
    assert c.site_tensor(3).shape == (8, 16 * 64) and c.site_tensor(2).shape == (5, 2, 8)
    assert c.site_tensor(3).data_ptr() == c.paged[0].tensor[1].data_ptr()
    assert c.bytes_per_token() == (2 * 2 * 2 * 16 + 1 * 2 * 32) * 4
    bufs = c.site_buffers(3)
    assert sorted(bufs) == ["k", "v"] and bufs["k"].shape == (8, 2, 16, 16)
    assert bufs["v"].data_ptr() - bufs["k"].data_ptr() == 2 * 16 * 16 * 4      # values follow the keys inside a page
    c.site_tensor(3).zero_()
    bufs["v"][5, 1, 3, 7] = 2.0
    from vapi_b200.parts.base import CacheView
    kv = CacheView("paged", c.site_tensor(3), None, True, bufs, c.site_spec(3)).stacked()
    assert kv.shape == (8, 2, 2, 16, 16) and float(kv[5, 1, 1, 3, 7]) == 2.0 and float(kv.sum()) == 2.0


def test_buffers_of_unlike_shapes_share_a_page():
    """A spec whose buffers differ (a wide row and a narrow one per token): the page holds them one
    after the other, and each is reachable as its own view."""
    from vapi_b200.parts.base import CacheView, PagedBuffer
    spec = PagedSpec((PagedBuffer("latent", 1, 24), PagedBuffer("rope_key", 2, 8)), 0)
    assert spec.elems_per_token() == 40 and not spec.uniform()
    c = CacheManager([(0, spec), (1, PagedSpec.rows(24))], page_size=16, num_pages=4, max_requests=2, dtype=torch.float32,
                     device="cpu")
    assert len(c.paged) == 2 and c.paged[0].tensor.shape == (1, 4, 16 * 40)
    bufs = c.site_buffers(0)
    assert bufs["latent"].shape == (4, 1, 16, 24) and bufs["rope_key"].shape == (4, 2, 16, 8)
    c.site_tensor(0).zero_()
    bufs["latent"][2, 0, 15, 23] = 1.0
    bufs["rope_key"][2, 1, 0, 0] = 3.0
    flat = c.site_tensor(0)
    assert float(flat[2, 16 * 24 - 1]) == 1.0 and float(flat[2, 16 * 24 + 16 * 8]) == 3.0 and float(flat.sum()) == 4.0
    with pytest.raises(ValueError, match="equal shape"):
        CacheView("paged", flat, None, True, bufs, spec).stacked()
    # one row per token: the pages read as one long table of rows, indexed by page * page_size + offset
    rows = c.site_buffers(1)["row"]
    assert rows.shape == (4, 1, 16, 24) and rows.reshape(64, 24).data_ptr() == rows.data_ptr()


def test_reserve_is_all_or_nothing_and_close_gives_everything_back():
    c = make_cache(num_pages=4)
    a = c.open("a")
    assert c.reserve(a, 33)                       # 3 pages
    b = c.open("b")
    assert not c.reserve(b, 17)                   # would need 2, only 1 left: nothing taken
    assert c.paged[0].pool.num_free == 1 and b.tables == [[]]
    assert c.reserve(b, 16)
    c.check_invariants()
    c.close(a)
    assert c.paged[0].pool.num_free == 3 and c.slots.num_free == 3
    with pytest.raises(ValueError, match="closed twice"):
        c.close(a)
    c.close(b)
    c.check_invariants()
    assert c.paged[0].pool.num_free == 4 and c.slots.num_free == 4


def test_window_group_gives_pages_back_as_the_window_passes():
    c = make_cache(num_pages=4, page=16, window=20)
    a = c.open("a")
    for total in range(1, 200):
        assert c.reserve(a, total), f"a window of 20 never needs more than 3 pages of 16 (at {total})"
        c.commit(a, total)
        c.check_invariants()
        held = [p for p in a.tables[0] if p >= 0]
        assert len(held) <= 3
        # every position a later query can still see lies in a held page
        for pos in range(max(0, total - 20 + 1), total):
            assert a.tables[0][pos // 16] >= 0
    c.close(a)
    assert c.paged[0].pool.num_free == 4


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_of_requests_keep_the_books(seed):
    rng = random.Random(seed)
    c = make_cache(num_pages=10, page=16, max_requests=3, window=rng.choice([0, 0, 24]))
    live = {}
    for step in range(400):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            try:
                live[step] = c.open(step)
            except OutOfSlots:
                assert c.slots.num_free == 0
        elif op < 0.75 and live:
            k = rng.choice(list(live))
            rc = live[k]
            total = rc.num_tokens + rng.choice([1, 1, 2, 7, 16, 40])
            before = [list(t) for t in rc.tables]
            if c.reserve(rc, total):
                c.commit(rc, total)
            else:
                assert [list(t) for t in rc.tables] == before
        elif live:
            k = rng.choice(list(live))
            c.close(live.pop(k))
        c.check_invariants()
    for rc in live.values():
        c.close(rc)
    c.check_invariants()
    assert all(g.pool.num_free == g.pool.num_pages for g in c.paged) and c.slots.num_free == 3


def test_validate_step_catches_bad_batches():
    c = make_cache()
    a = c.open("a")
    with pytest.raises(StepError, match="at least one entry"):
        validate_step([], c, 100, 64)
    with pytest.raises(StepError, match="do not cover"):
        validate_step([StepEntry(a, [1, 2, 3], [0])], c, 100, 64)
    c.reserve(a, 3)
    validate_step([StepEntry(a, [1, 2, 3], [0, 2])], c, 100, 64)
    with pytest.raises(StepError, match="outside the vocabulary"):
        validate_step([StepEntry(a, [1, 100, 3])], c, 100, 64)
    with pytest.raises(StepError, match="wanted place"):
        validate_step([StepEntry(a, [1, 2, 3], [3])], c, 100, 64)
    with pytest.raises(StepError, match="appears twice"):
        validate_step([StepEntry(a, [1]), StepEntry(a, [2])], c, 100, 64)
    with pytest.raises(StepError, match="brings no tokens"):
        validate_step([StepEntry(a, [])], c, 100, 64)
    with pytest.raises(StepError, match="would pass position"):
        validate_step([StepEntry(a, [1, 2, 3])], c, 100, 2)
    c.close(a)
    with pytest.raises(StepError, match="has ended"):
        validate_step([StepEntry(a, [1])], c, 100, 64)


# ---------------------------------------------------------------------------------------
# scheduler on a scripted step function


class Script:
    """Plays the part of the model: request r's k-th generated token is script[r][k]."""

    def __init__(self, sched, script):
        self.sched, self.script, self.plans, self.portions = sched, script, [], []

    def run(self, max_steps=1000):
        for _ in range(max_steps):
            if self.sched.is_idle():
                return
            plan = self.sched.schedule()
            self.plans.append(plan)
            self.portions += [(sid, e.start, len(e.tokens)) for sid, e in zip(plan.batch_seqs, plan.entries)]
            # invariants of every plan: positions continue, pages cover, rows match
            validate_step(plan.entries, self.sched.cache, 10 ** 6, 10 ** 6) if plan.entries else None
            sampled = []
            for sid in plan.sampled_seqs:
                seq = self.sched.seqs[sid]
                sampled.append(self.script[seq.request_id][seq.num_generated])
            # the step function would commit the cache; do what it does
            for e in plan.entries:
                self.sched.cache.commit(e.cache, e.start + len(e.tokens))
            self.sched.commit(plan, sampled)
            self.sched.cache.check_invariants()
        raise AssertionError("the scheduler did not finish")


def sched(num_pages=8, page=16, max_requests=4, eos=(99,), **kw):
    cache = make_cache(num_pages=num_pages, page=page, max_requests=max_requests, watermark=kw.pop("watermark", 0.0))
    return Scheduler(SchedulerConfig(**kw), cache, eos)


def test_admission_errors():
    s = sched(max_context=32)
    with pytest.raises(AdmitError, match="empty"):
        s.admit("a", [], SamplingParams())
    with pytest.raises(AdmitError, match="context limit"):
        s.admit("a", list(range(32)), SamplingParams())
    with pytest.raises(ValueError, match="max_tokens"):
        s.admit("a", [1], SamplingParams(max_tokens=0))
    s2 = sched(num_pages=2, max_context=4096)
    with pytest.raises(AdmitError, match="whole cache"):
        s2.admit("a", list(range(40)), SamplingParams())


def test_prompt_is_cut_into_portions_and_only_the_last_asks_for_logits():
    s = sched(prefill_chunk_tokens=7, max_context=256)
    s.admit("a", list(range(18)), SamplingParams(max_tokens=2, temperature=0.0))
    sc = Script(s, {"a": [5, 6]})
    sc.run()
    sizes = [[len(e.tokens) for e in p.entries] for p in sc.plans]
    assert sizes == [[7], [7], [4], [1]]
    assert [len(p.sampled_seqs) for p in sc.plans] == [0, 0, 1, 1]
    (seq,) = s.drain_finished()
    assert seq.generated == [5, 6] and seq.finish_reason == FinishReason.LENGTH


def test_decodes_go_first_and_share_the_budget_with_portions():
    s = sched(num_pages=16, max_batched_tokens=10, prefill_chunk_tokens=8, max_context=256)
    s.admit("a", [1, 2, 3], SamplingParams(max_tokens=4, temperature=0.0))
    sc = Script(s, {"a": [5, 6, 7, 8], "b": [9, 9, 9, 9]})
    p0 = s.schedule()
    for e in p0.entries:
        s.cache.commit(e.cache, e.start + len(e.tokens))
    s.commit(p0, [5])
    s.admit("b", list(range(20)), SamplingParams(max_tokens=4, temperature=0.0))
    p1 = s.schedule()
    # a's decode token first, then b's portion limited by chunk (8) and by what is left of the budget (9)
    assert [len(e.tokens) for e in p1.entries] == [1, 8]
    assert p1.entries[0].tokens == [5] and p1.sampled_seqs == [0]


def test_eos_stops_only_after_a_generated_token_and_stop_ids_work():
    s = sched(max_context=256)
    s.admit("a", [99, 99], SamplingParams(max_tokens=8, temperature=0.0))        # EOS in the prompt is not a stop
    s.admit("b", [1], SamplingParams(max_tokens=8, temperature=0.0, stop_token_ids=(42,)))
    s.admit("c", [1], SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True))
    Script(s, {"a": [4, 99, 1], "b": [3, 42, 1], "c": [99] * 8}).run()
    done = {q.request_id: q for q in s.drain_finished()}
    assert done["a"].generated == [4, 99] and done["a"].finish_reason == FinishReason.STOP
    assert done["b"].generated == [3, 42] and done["b"].finish_reason == FinishReason.STOP
    assert done["c"].generated == [99] * 8 and done["c"].finish_reason == FinishReason.LENGTH


def test_context_limit_ends_a_request():
    s = sched(max_context=6)
    s.admit("a", [1, 2, 3], SamplingParams(max_tokens=100, temperature=0.0))
    Script(s, {"a": list(range(10, 30))}).run()
    (seq,) = s.drain_finished()
    assert seq.total_len == 6 and seq.finish_reason == FinishReason.LENGTH


def test_running_out_of_pages_preempts_by_recompute_and_everyone_finishes():
    """Six requests over eight pages of sixteen tokens: the pool is oversubscribed, requests
    are preempted and recomputed, every one ends with exactly its scripted tokens and nothing
    leaks (the shape of the reference's crates/vapi-engine/tests/scheduler.rs:487-522)."""
    s = sched(num_pages=8, page=16, max_requests=4, max_context=200, prefill_chunk_tokens=16)
    script = {}
    for i in range(6):
        s.admit(i, list(range(1, 20 + i)), SamplingParams(max_tokens=30, temperature=0.0))
        script[i] = [1000 + 10 * i + k for k in range(30)]
    sc = Script(s, script)
    sc.run(5000)
    done = {q.request_id: q for q in s.drain_finished()}
    assert sorted(done) == list(range(6))
    assert all(done[i].generated == script[i] for i in range(6))
    assert sum(q.preemptions for q in done.values()) > 0, "this pool must force preemptions"
    assert sum(len(p.preempted) for p in sc.plans) == sum(q.preemptions for q in done.values())
    assert all(g.pool.num_free == g.pool.num_pages for g in s.cache.paged) and s.cache.slots.num_free == 4
    # a preempted request starts again from position 0 with prompt + generated text as its known text
    starts = [sid for sid, start, _ in sc.portions if start == 0]
    assert len(starts) == 6 + sum(q.preemptions for q in done.values())
    # and its portions continue without a gap each time
    pos = {}
    for sid, start, q in sc.portions:
        assert start == 0 or pos[sid] == start
        pos[sid] = start + q


def test_a_big_request_is_not_starved_by_small_ones_behind_it():
    s = sched(num_pages=8, page=16, max_requests=4, max_context=200)
    s.admit("small0", list(range(40)), SamplingParams(max_tokens=1, temperature=0.0))     # 3 pages
    s.admit("big", list(range(100)), SamplingParams(max_tokens=1, temperature=0.0))       # 7 pages: must wait
    s.admit("small1", list(range(10)), SamplingParams(max_tokens=1, temperature=0.0))     # would fit, but is behind
    p = s.schedule()
    assert [s.seqs[i].request_id for i in p.started] == ["small0"]
    assert list(s.waiting) == [1, 2]


def test_watermark_is_kept_at_admission():
    s = sched(num_pages=10, page=16, max_requests=4, max_context=400, watermark=0.2)   # 2 pages held back
    s.admit("a", list(range(100)), SamplingParams(max_tokens=1))      # 7 pages: 10 - 7 >= 2, fits
    s.admit("b", list(range(20)), SamplingParams(max_tokens=1))       # 2 pages: 3 - 2 < 2, waits
    p = s.schedule()
    assert [s.seqs[i].request_id for i in p.started] == ["a"]


def test_a_page_set_aside_for_padding_is_not_counted_as_room():
    """A page that was taken out of circulation (for the padding rows of fixed-shape decode steps)
    never comes back: a prompt that needs every page of the pool is refused at admission, and one
    that was admitted before the page was set aside ends with ``length`` instead of waiting for
    room that cannot appear."""
    s = sched(num_pages=4, page=16, max_requests=4, max_context=400)
    s.admit("early", list(range(60)), SamplingParams(max_tokens=1, temperature=0.0))    # 61 positions: all 4 pages
    assert s.cache.set_aside_pages() is not None
    with pytest.raises(AdmitError, match="whole cache"):
        s.admit("late", list(range(60)), SamplingParams(max_tokens=1, temperature=0.0))
    s.admit("fits", list(range(40)), SamplingParams(max_tokens=1, temperature=0.0))     # 3 pages
    Script(s, {"early": [1], "fits": [2]}).run()
    done = {q.request_id: q for q in s.drain_finished()}
    assert done["early"].finish_reason == FinishReason.LENGTH and done["early"].generated == []
    assert done["fits"].generated == [2]
    s.cache.check_invariants()


def test_cancel_and_fail_all_free_everything():
    s = sched(max_context=256)
    a = s.admit("a", list(range(30)), SamplingParams(max_tokens=5))
    b = s.admit("b", list(range(30)), SamplingParams(max_tokens=5))
    s.schedule()
    s.cancel(a)
    assert s.seqs[a].finish_reason == FinishReason.CANCELLED
    s.fail_all()
    done = {q.request_id: q.finish_reason for q in s.drain_finished()}
    assert done == {"a": FinishReason.CANCELLED, "b": FinishReason.ERROR}
    assert all(g.pool.num_free == g.pool.num_pages for g in s.cache.paged) and s.cache.slots.num_free == 4
    assert s.is_idle()


# ---------------------------------------------------------------------------------------
# planning one step ahead of the sampled tokens


class ScriptAhead(Script):
    """The engine's way of running one step ahead, on the scripted model: a step is planned and
    advanced before the tokens of the step before it are given to the scheduler."""

    def run(self, max_steps=1000):
        inflight = None
        self.ahead = 0
        for _ in range(max_steps):
            if self.sched.is_idle() and inflight is None:
                return
            if inflight is not None and not self.sched.can_run_ahead():
                self.sched.resolve(*inflight)
                inflight = None
            plan = self.sched.schedule()
            self.plans.append(plan)
            assert not plan.preempted or inflight is None, "a preemption while a token is unknown"
            if plan.is_empty():
                if inflight is not None:
                    self.sched.resolve(*inflight)
                    inflight = None
                continue
            # what the scripted model will sample for this step: decided by how many tokens the
            # request has, unknown ones included
            sampled = []
            for sid in plan.sampled_seqs:
                seq = self.sched.seqs[sid]
                sampled.append(self.script[seq.request_id][seq.num_generated])
            for e in plan.entries:
                self.sched.cache.commit(e.cache, e.start + len(e.tokens))
            self.sched.advance(plan)
            if inflight is not None:
                self.ahead += 1
                self.sched.resolve(*inflight)
            inflight = (plan, sampled)
            self.sched.cache.check_invariants()
        raise AssertionError("the scheduler did not finish")


@pytest.mark.parametrize("pages", [64, 9])
def test_planning_one_step_ahead_ends_every_request_the_same_way(pages):
    script, results = {}, {}
    for i in range(6):
        script[i] = [1000 + 10 * i + k for k in range(30)]
    script[1][4] = 99            # EOS in the middle
    script[3][9] = 42            # a stop id in the middle
    script[4][0] = 99            # EOS as the very first generated token
    for cls in (Script, ScriptAhead):
        s = sched(num_pages=pages, page=16, max_requests=4, max_context=200, prefill_chunk_tokens=16)
        for i in range(6):
            s.admit(i, list(range(1, 20 + i)), SamplingParams(max_tokens=12 + 3 * i, temperature=0.0,
                                                              stop_token_ids=(42,) if i == 3 else ()))
        sc = cls(s, script)
        sc.run(5000)
        results[cls] = {q.request_id: (q.generated, q.finish_reason, q.total_len) for q in s.drain_finished()}
        assert all(g.pool.num_free == g.pool.num_pages for g in s.cache.paged) and s.cache.slots.num_free == 4
        if cls is ScriptAhead:
            assert sc.ahead > 10
    assert results[Script] == results[ScriptAhead]
    r = results[Script]
    assert r[1][0] == script[1][:5] and r[1][1] == FinishReason.STOP
    assert r[3][0] == script[3][:10] and r[3][1] == FinishReason.STOP
    assert r[4][0] == [99] and r[0][1] == FinishReason.LENGTH and len(r[0][0]) == 12


def test_an_unknown_token_is_marked_for_the_device_to_fetch():
    s = sched(num_pages=16, max_context=256)
    s.admit("a", [1, 2, 3], SamplingParams(max_tokens=5, temperature=0.0))
    s.admit("b", [4, 5], SamplingParams(max_tokens=5, temperature=0.0))
    p0 = s.schedule()
    assert not p0.has_unknown and p0.sampled_seqs == [0, 1]
    for e in p0.entries:
        s.cache.commit(e.cache, e.start + len(e.tokens))
    s.advance(p0)
    p1 = s.schedule()                      # both decode a token nobody knows yet
    assert p1.has_unknown and p1.pure_decode
    assert s._list(13, 2) == [0, 1]        # token sources: rows of the step before
    for e in p1.entries:
        s.cache.commit(e.cache, e.start + 1)
    s.advance(p1)
    assert s.resolve(p0, [7, 99]) == [True, True]          # b ends on EOS ...
    assert s.resolve(p1, [8, 9]) == [True, False]          # ... so what the step ahead made for it is dropped
    done = {q.request_id: q.generated for q in s.drain_finished()}
    assert done == {"b": [99]} and s.seqs[0].generated == [7, 8]
