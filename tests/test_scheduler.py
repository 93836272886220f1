"""The scheduler's decisions, with a stand-in for the engine that keeps the real cache bookkeeping (no GPU).

The scheduler under test is the host library's own (engine/scheduler.cpp), driven through
``purhie_b200.engine.probe``; request ids are integers and the batches the stand-in ran come back as
[[id, tokens, want places]]."""
import pytest

from purhie_b200.engine.probe import SchedulerProbe, expected_output
from purhie_b200.sampling import SamplerParams

A, B, C, D = 1, 2, 3, 4


def batches(state):
    return [[tuple(x[:2]) + (x[2],) for x in b] for b in state["batches"]]


def test_prompts_are_cut_under_the_token_budget_and_decodes_come_first():
    s = SchedulerProbe(num_pages=64, max_batch_tokens=16, prefill_chunk=10)
    s.add(A, list(range(1, 24)), max_new_tokens=3)
    s.add(B, list(range(5, 12)), max_new_tokens=3)
    st = s.run()
    b = batches(st)
    assert b[0] == [(A, 10, []), (B, 6, [])]                       # chunk cap 10, budget 16
    assert b[1] == [(A, 10, []), (B, 1, [0])]                     # oldest first; b's last prompt token is sampled
    assert b[2] == [(B, 1, [0]), (A, 3, [2])]                     # decode row first, then the prompt's end
    assert st["finished"][A]["output"] == expected_output(range(1, 24), 3)
    assert st["finished"][B]["output"] == expected_output(range(5, 12), 3)
    assert st["finished"][A]["stop_reason"] == "max_tokens"
    assert st["cache"]["free_pages"] == [64] and st["cache"]["free_slots"] == 4


def test_admission_waits_for_a_slot_and_is_first_come_first_served():
    s = SchedulerProbe(num_pages=64, max_requests=2, max_batch_tokens=64, prefill_chunk=64)
    for i in range(4):
        s.add(i, [i + 1, i + 2, i + 3], max_new_tokens=2 + i)
    s.step()
    st = s.state()
    assert st["running"] == [0, 1] and st["waiting"] == [2, 3]
    st = s.run()
    order = [rid for batch in batches(st) for rid, n, w in batch if n == 3]
    assert order == [0, 1, 2, 3]
    for i in range(4):
        assert st["finished"][i]["output"] == expected_output([i + 1, i + 2, i + 3], 2 + i)


def test_pages_run_out_preempts_the_newest_and_the_result_does_not_change():
    prompts = {A: list(range(1, 14)), B: list(range(3, 12)), C: list(range(2, 9))}
    big = SchedulerProbe(num_pages=64, max_batch_tokens=64, prefill_chunk=64)
    small = SchedulerProbe(num_pages=11, max_batch_tokens=64, prefill_chunk=64)      # 44 tokens; the three need 65 at the end
    for s in (big, small):
        for k, p in prompts.items():
            s.add(k, p, max_new_tokens=12)
    s0, s1 = big.run(), small.run()
    assert s1["preemptions"] > 0 and s0["preemptions"] == 0
    assert s1["finished"][C]["preemptions"] >= 1 and s1["finished"][A]["preemptions"] == 0      # newest first, oldest never
    for k in prompts:
        assert s1["finished"][k]["output"] == s0["finished"][k]["output"] == expected_output(prompts[k], 12)
        assert s1["finished"][k]["stop_reason"] == "max_tokens"
    assert s1["cache"]["free_pages"] == [11]


def test_a_request_too_large_for_the_empty_pool_ends_with_context_full():
    s = SchedulerProbe(num_pages=4, max_batch_tokens=64)                           # 16 tokens
    s.add(A, list(range(1, 30)), max_new_tokens=4)
    s.add(B, [1, 2, 3], max_new_tokens=2)
    st = s.run()
    assert st["finished"][A]["stop_reason"] == "context_full" and st["finished"][A]["output"] == []
    assert st["finished"][B]["output"] == expected_output([1, 2, 3], 2)


def test_a_lone_request_that_outgrows_the_pool_ends_with_context_full():
    s = SchedulerProbe(num_pages=3, max_batch_tokens=64)                           # 12 tokens
    s.add(A, [1, 2, 3, 4, 5], max_new_tokens=50)
    r = s.run()["finished"][A]
    assert r["stop_reason"] == "context_full" and r["output"] == expected_output([1, 2, 3, 4, 5], len(r["output"]))
    assert 6 <= len(r["output"]) <= 8 and s.state()["cache"]["free_pages"] == [3]


def test_context_limit_eos_callback_and_cancel():
    s = SchedulerProbe(num_pages=64, n_ctx=10)
    s.add(A, [1, 2, 3, 4], max_new_tokens=50)
    r = s.run()["finished"][A]
    assert r["stop_reason"] == "context_full" and r["n_tokens"] == 10
    first = expected_output([4, 4], 3)
    s = SchedulerProbe(num_pages=64)
    s.add(A, [4, 4], max_new_tokens=50, eos_ids=[first[2]])
    s.add(B, [4, 4], max_new_tokens=4, eos_ids=[first[2]], ignore_eos=True)
    s.add(C, [9], max_new_tokens=50, stop_after=3)
    s.add(D, [7, 7, 7], max_new_tokens=50)
    s.step()
    assert s.cancel(D) and not s.cancel(D)
    st = s.run()
    assert st["finished"][A]["stop_reason"] == "eog" and st["finished"][A]["output"] == first[:2]     # EOS is not emitted
    assert st["finished"][B]["output"] == expected_output([4, 4], 4)
    assert st["finished"][C]["stop_reason"] == "callback" and len(st["finished"][C]["output"]) == 3
    assert st["finished"][D]["stop_reason"] == "cancelled"
    assert st["cache"]["free_pages"] == [64] and st["cache"]["free_slots"] == 4


def test_decisions_depend_on_arrival_order_only():
    def run():
        s = SchedulerProbe(num_pages=9, max_batch_tokens=12, prefill_chunk=5)
        for i in range(5):
            s.add(i, list(range(1, 4 + 3 * i)), SamplerParams.pure_temperature(0.9, seed=i), max_new_tokens=6)
        st = s.run()
        return st["batches"], {k: v["output"] for k, v in st["finished"].items()}
    assert run() == run()


def test_window_group_lets_a_long_request_live_in_few_pages():
    s = SchedulerProbe(num_pages=4, window=6, max_batch_tokens=8, prefill_chunk=8)     # 16 tokens of pages, window 6
    s.add(A, [1, 2, 3], max_new_tokens=40)
    r = s.run()["finished"][A]
    assert r["stop_reason"] == "max_tokens" and len(r["output"]) == 40


def test_decoding_ahead_of_the_host_changes_no_output_and_ends():
    """Budgets that end at different steps, an end-of-generation id on the way, pages that run out in the middle of a
    run ahead: the same outputs and stop reasons as step by step, and the loop ends."""
    prompts = {A: list(range(1, 14)), B: list(range(3, 12)), C: list(range(2, 9)), D: [4, 4]}
    budgets = {A: 12, B: 5, C: 9, D: 30}
    eos = [expected_output(prompts[D], 30)[11]]
    for pages in (64, 13):
        outs = []
        for ahead in (False, True):
            s = SchedulerProbe(num_pages=pages, ahead=True, max_batch_tokens=64, prefill_chunk=64, run_ahead=ahead)
            for k, p in prompts.items():
                s.add(k, p, max_new_tokens=budgets[k], eos_ids=eos if k == D else ())
            st = s.run(ahead=True)
            outs.append({k: (st["finished"][k]["output"], st["finished"][k]["stop_reason"]) for k in prompts})
            assert st["cache"]["free_pages"] == [pages] and st["cache"]["free_slots"] == 4
            if ahead and pages == 64:
                assert st["steps"] > len(st["batches"]) - 1 > 0
        assert outs[0] == outs[1]
        assert outs[0][D][1] == "eog" and outs[0][B][1] == "max_tokens"


def test_a_cut_portion_ends_the_step_on_a_multiple_of_the_row_tile():
    """With align_rows a portion that is a cut anyway is shortened so that the step's rows are a multiple of it;
    the end of a prompt, a step below one tile and a cut that would lose more than half stay as they are, and the
    outputs do not change."""
    def run(align):
        s = SchedulerProbe(num_pages=4096, page_size=16, max_requests=40, max_batch_tokens=2048, prefill_chunk=512,
                           align_rows=align)
        for i in range(32):
            s.add(i, [i + 1, i + 2], max_new_tokens=12)
        s.step()                                                     # the 32 short prompts: 64 rows, all ends
        s.add(100, [(7 * i) % 50 for i in range(1300)], max_new_tokens=2)
        return s.run()
    s0, s1 = run(0), run(256)
    sizes = lambda st: [sum(n for _, n, _ in b) for b in batches(st)]
    assert sizes(s0)[1:4] == [32 + 512, 32 + 512, 32 + 276]
    assert sizes(s1)[1:4] == [512, 512, 32 + 340]                    # 480 + 32 twice, then the prompt's end as it is
    for rid in s0["finished"]:
        assert s0["finished"][rid]["output"] == s1["finished"][rid]["output"]
    # below one tile nothing is cut; a cut that would take more than half is not made
    s = SchedulerProbe(num_pages=4096, page_size=16, max_requests=4, max_batch_tokens=2048, prefill_chunk=100, align_rows=256)
    s.add(A, [1] * 1000, max_new_tokens=1)
    s.step(); s.step(); s.step()
    assert [sum(n for _, n, _ in b) for b in batches(s.state())] == [100, 100, 100]
