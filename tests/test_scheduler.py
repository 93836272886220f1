"""The scheduler's decisions, with a stand-in for the engine that keeps the real cache bookkeeping (no GPU)."""
import numpy as np
import pytest

from purhie_b200.cache import CacheManager, CacheNeed
from purhie_b200.engine.scheduler import (STOP_CANCELLED, STOP_CONTEXT_FULL, STOP_EOG, STOP_MAX_TOKENS, Request,
                                          Scheduler)
from purhie_b200.sampling import SamplerParams


class FakeEngine:
    """Runs no model: logits of a row put all weight on (sum of the request's tokens so far) % vocab, so the
    generated tokens are a pure function of the request's history and any change of order or cut shows."""

    vocab = 50

    def __init__(self, num_pages, page_size=4, max_requests=4, window=None, max_position=1 << 20):
        self.cache = CacheManager([CacheNeed.pages(1, 8, window)], page_size, num_pages, max_requests)
        self.max_position = max_position
        self.history = {}
        self.batches = []

    def step(self, entries):
        rows = []
        for e in entries:
            self.cache.reserve(e.request_id, len(e.tokens))
        for e in entries:
            if self.cache.length(e.request_id) == 0:
                self.history[e.request_id] = []          # new, or preempted and starting over
            h = self.history[e.request_id]
            assert len(h) == self.cache.length(e.request_id)
            for i, t in enumerate(e.tokens):
                h.append(t)
                if i in e.want:
                    row = np.zeros(self.vocab, dtype=np.float32)
                    row[(sum(h) * 7 + len(h)) % self.vocab] = 5.0
                    rows.append(row)
            self.cache.advance(e.request_id, len(e.tokens))
        self.batches.append([(e.request_id, len(e.tokens), list(e.want)) for e in entries])
        self.cache.check()
        return np.stack(rows) if rows else None

    def sample(self, logits, samplers):
        return [s.sample(row) for s, row in zip(samplers, logits)]

    def forget(self, rid):
        self.history.pop(rid, None)


def expected_output(prompt, n, vocab=50):
    h = list(prompt)
    out = []
    for _ in range(n):
        t = (sum(h) * 7 + len(h)) % vocab
        out.append(t); h.append(t)
    return out


def run_all(sched, eng):
    guard = 0
    while sched.has_work():
        before = set(sched.finished)
        sched.step()
        for r in list(sched.waiting):
            eng.forget(r.request_id)                 # a preempted request starts over
        guard += 1
        assert guard < 10000
    return sched.finished


def test_prompts_are_cut_under_the_token_budget_and_decodes_come_first():
    eng = FakeEngine(num_pages=64)
    s = Scheduler(eng, max_batch_tokens=16, prefill_chunk=10)
    s.add(Request("a", list(range(1, 24)), max_new_tokens=3))
    s.add(Request("b", list(range(5, 12)), max_new_tokens=3))
    run_all(s, eng)
    b = eng.batches
    assert b[0] == [("a", 10, []), ("b", 6, [])]                       # chunk cap 10, budget 16
    assert b[1] == [("a", 10, []), ("b", 1, [0])]                     # oldest first; b's last prompt token is sampled
    assert b[2] == [("b", 1, [0]), ("a", 3, [2])]                     # decode row first, then the prompt's end
    assert s.finished["a"].output == expected_output(range(1, 24), 3)
    assert s.finished["b"].output == expected_output(range(5, 12), 3)
    assert s.finished["a"].stop_reason == STOP_MAX_TOKENS
    assert eng.cache.free_pages() == [64] and eng.cache.slots.num_free == 4


def test_admission_waits_for_a_slot_and_is_first_come_first_served():
    eng = FakeEngine(num_pages=64, max_requests=2)
    s = Scheduler(eng, max_batch_tokens=64, prefill_chunk=64)
    for i in range(4):
        s.add(Request(i, [i + 1, i + 2, i + 3], max_new_tokens=2 + i))
    s.step()
    assert [r.request_id for r in s.running] == [0, 1] and [r.request_id for r in s.waiting] == [2, 3]
    run_all(s, eng)
    order = [rid for batch in eng.batches for rid, n, w in batch if n == 3]
    assert order == [0, 1, 2, 3]
    for i in range(4):
        assert s.finished[i].output == expected_output([i + 1, i + 2, i + 3], 2 + i)


def test_pages_run_out_preempts_the_newest_and_the_result_does_not_change():
    prompts = {"a": list(range(1, 14)), "b": list(range(3, 12)), "c": list(range(2, 9))}
    big = FakeEngine(num_pages=64)
    s0 = Scheduler(big, max_batch_tokens=64, prefill_chunk=64)
    for k, p in prompts.items():
        s0.add(Request(k, p, max_new_tokens=12))
    run_all(s0, big)
    small = FakeEngine(num_pages=11)                                  # 44 tokens; the three need 65 at the end
    s1 = Scheduler(small, max_batch_tokens=64, prefill_chunk=64)
    for k, p in prompts.items():
        s1.add(Request(k, p, max_new_tokens=12))
    run_all(s1, small)
    assert s1.preemptions > 0
    assert s1.finished["c"].preemptions >= 1 and s1.finished["a"].preemptions == 0      # newest first, oldest never
    for k in prompts:
        assert s1.finished[k].output == s0.finished[k].output == expected_output(prompts[k], 12)
        assert s1.finished[k].stop_reason == STOP_MAX_TOKENS
    assert small.cache.free_pages() == [11]


def test_a_request_too_large_for_the_empty_pool_ends_with_context_full():
    eng = FakeEngine(num_pages=4)                                      # 16 tokens
    s = Scheduler(eng, max_batch_tokens=64)
    s.add(Request("big", list(range(1, 30)), max_new_tokens=4))
    s.add(Request("ok", [1, 2, 3], max_new_tokens=2))
    run_all(s, eng)
    assert s.finished["big"].stop_reason == STOP_CONTEXT_FULL and s.finished["big"].output == []
    assert s.finished["ok"].output == expected_output([1, 2, 3], 2)


def test_a_lone_request_that_outgrows_the_pool_ends_with_context_full():
    eng = FakeEngine(num_pages=3)                                      # 12 tokens
    s = Scheduler(eng, max_batch_tokens=64)
    s.add(Request("x", [1, 2, 3, 4, 5], max_new_tokens=50))
    run_all(s, eng)
    r = s.finished["x"]
    assert r.stop_reason == STOP_CONTEXT_FULL and r.output == expected_output([1, 2, 3, 4, 5], len(r.output))
    assert 6 <= len(r.output) <= 8 and eng.cache.free_pages() == [3]


def test_context_limit_eos_callback_and_cancel():
    eng = FakeEngine(num_pages=64)
    s = Scheduler(eng, n_ctx=10)
    s.add(Request("ctx", [1, 2, 3, 4], max_new_tokens=50))
    run_all(s, eng)
    assert s.finished["ctx"].stop_reason == STOP_CONTEXT_FULL and len(s.finished["ctx"].tokens()) == 10
    first = expected_output([4, 4], 3)
    s = Scheduler(eng)
    s.add(Request("eos", [4, 4], max_new_tokens=50, eos_ids=[first[2]]))
    s.add(Request("noeos", [4, 4], max_new_tokens=4, eos_ids=[first[2]], ignore_eos=True))
    seen = []
    s.add(Request("cb", [9], max_new_tokens=50, on_token=lambda r, t: seen.append(t) or len(seen) == 3))
    s.add(Request("gone", [7, 7, 7], max_new_tokens=50))
    s.step()
    assert s.cancel("gone") and not s.cancel("gone")
    run_all(s, eng)
    assert s.finished["eos"].stop_reason == STOP_EOG and s.finished["eos"].output == first[:2]     # EOS is not emitted
    assert s.finished["noeos"].output == expected_output([4, 4], 4)
    assert s.finished["cb"].stop_reason == "callback" and len(s.finished["cb"].output) == 3
    assert s.finished["gone"].stop_reason == STOP_CANCELLED
    assert eng.cache.free_pages() == [64] and eng.cache.slots.num_free == 4


def test_decisions_depend_on_arrival_order_only():
    def run():
        eng = FakeEngine(num_pages=9)
        s = Scheduler(eng, max_batch_tokens=12, prefill_chunk=5)
        for i in range(5):
            s.add(Request(i, list(range(1, 4 + 3 * i)), SamplerParams.pure_temperature(0.9, seed=i), max_new_tokens=6))
        run_all(s, eng)
        return eng.batches, {k: v.output for k, v in s.finished.items()}
    assert run() == run()


def test_window_group_lets_a_long_request_live_in_few_pages():
    eng = FakeEngine(num_pages=4, window=6)                           # 16 tokens of pages, window 6
    s = Scheduler(eng, max_batch_tokens=8, prefill_chunk=8)
    s.add(Request("w", [1, 2, 3], max_new_tokens=40))
    run_all(s, eng)
    assert s.finished["w"].stop_reason == STOP_MAX_TOKENS and len(s.finished["w"].output) == 40


class AheadEngine(FakeEngine):
    """A FakeEngine that also takes a step's token ids "from the device" (what the step before sampled, not yet
    handed to the host) and samples without being waited for, as the scheduler's decode_ahead uses them."""

    class Pending:
        def __init__(self, toks):
            self.ids = toks

        def result(self):
            return list(self.ids)

    def decodes_as_graph(self, entries):
        return all(len(e.tokens) == 1 for e in entries)

    def step(self, entries, device_tokens=None):
        if device_tokens is not None:
            entries = [type(e)(e.request_id, [int(t)], e.want) for e, t in zip(entries, device_tokens)]
        return super().step(entries)

    def sample_async(self, logits, samplers):
        return self.Pending(self.sample(logits, samplers))


def run_to_the_end(sched, eng):
    guard = 0
    while sched.has_work():
        if not sched.decode_ahead():
            sched.step()
        for r in list(sched.waiting):
            eng.forget(r.request_id)
        guard += 1
        assert guard < 10000
    return sched.finished


def test_decoding_ahead_of_the_host_changes_no_output_and_ends():
    """Budgets that end at different steps, an end-of-generation id on the way, pages that run out in the middle of a
    run ahead: the same outputs and stop reasons as step by step, and the loop ends."""
    prompts = {"a": list(range(1, 14)), "b": list(range(3, 12)), "c": list(range(2, 9)), "d": [4, 4]}
    budgets = {"a": 12, "b": 5, "c": 9, "d": 30}
    eos = [expected_output(prompts["d"], 30)[11]]
    for pages in (64, 13):
        outs = []
        for ahead in (False, True):
            eng = AheadEngine(num_pages=pages)
            s = Scheduler(eng, max_batch_tokens=64, prefill_chunk=64)
            s.run_ahead = ahead
            for k, p in prompts.items():
                s.add(Request(k, p, max_new_tokens=budgets[k], eos_ids=eos if k == "d" else ()))
            run_to_the_end(s, eng)
            outs.append({k: (s.finished[k].output, s.finished[k].stop_reason) for k in prompts})
            assert eng.cache.free_pages() == [pages] and eng.cache.slots.num_free == 4
        assert outs[0] == outs[1]
        assert outs[0]["d"][1] == STOP_EOG and outs[0]["b"][1] == STOP_MAX_TOKENS


def test_a_cut_portion_ends_the_step_on_a_multiple_of_the_row_tile():
    """With align_rows a portion that is a cut anyway is shortened so that the step's rows are a multiple of it;
    the end of a prompt, a step below one tile and a cut that would lose more than half stay as they are, and the
    outputs do not change."""
    def run(align):
        eng = FakeEngine(num_pages=4096, page_size=16, max_requests=40)
        s = Scheduler(eng, max_batch_tokens=2048, prefill_chunk=512, align_rows=align)
        for i in range(32):
            s.add(Request(("d", i), [i + 1, i + 2], max_new_tokens=12))
        s.step()                                                     # the 32 short prompts: 64 rows, all ends
        s.add(Request("long", [(7 * i) % 50 for i in range(1300)], max_new_tokens=2))
        run_all(s, eng)
        return s, eng
    s0, e0 = run(None)
    s1, e1 = run(256)
    sizes = lambda eng: [sum(n for _, n, _ in b) for b in eng.batches]
    assert sizes(e0)[1:4] == [32 + 512, 32 + 512, 32 + 276]
    assert sizes(e1)[1:4] == [512, 512, 32 + 340]                    # 480 + 32 twice, then the prompt's end as it is
    for rid in s0.finished:
        assert s0.finished[rid].output == s1.finished[rid].output
    # below one tile nothing is cut; a cut that would take more than half is not made
    eng = FakeEngine(num_pages=4096, page_size=16, max_requests=4)
    s = Scheduler(eng, max_batch_tokens=2048, prefill_chunk=100, align_rows=256)
    s.add(Request("p", [1] * 1000, max_new_tokens=1))
    s.step(); s.step(); s.step()
    assert [sum(n for _, n, _ in b) for b in eng.batches] == [100, 100, 100]
