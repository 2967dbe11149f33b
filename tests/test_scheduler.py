"""The scheduler's decisions on the CPU, against a cache manager without tensors and a fake step
(in the manner of the fakes of tests/test_single_model_path.py:12-46 in SnowLLM)."""
import pytest

from snowllm_b200.cache import CacheManager
from snowllm_b200.engine.request import Request, SamplingParams
from snowllm_b200.engine.scheduler import Scheduler
from snowllm_b200.errors import CapacityError, SnowLLMError
from snowllm_b200.parts.spec import PagedKVSpec, SlotStateSpec

SPECS = {0: PagedKVSpec(2, 16), 1: SlotStateSpec(((2, 8),))}


def make(num_pages=16, max_seqs=4, budget=32, max_len=256, page=16, preempt=True):
    cm = CacheManager(SPECS, page, num_pages, max_seqs)
    return cm, Scheduler(cm, max_seqs, budget, max_len, preempt)


def req(n, new=8):
    return Request(prompt=list(range(1, n + 1)), params=SamplingParams(temperature=0, max_new_tokens=new))


def fake_step(sched, plan, token=7):
    """What the engine does after the model ran: record progress, append a token where logits came."""
    for s in plan:
        assert s.request.cache.num_tokens == s.start
        sched.cache.commit(s.request.cache, s.start + s.count)
        s.request.num_computed += s.count
        if s.wants_logits:
            s.request.out.append(token)
            if len(s.request.out) >= s.request.params.max_new_tokens:
                s.request.done, s.request.finish_reason = True, "length"


def run(sched, limit=1000):
    log = []
    for _ in range(limit):
        sched.retire_finished()
        plan = sched.schedule()
        if not plan:
            break
        log.append([(s.request, s.start, s.count, s.wants_logits) for s in plan])
        fake_step(sched, plan)
    sched.retire_finished()
    return log


def test_prompt_is_cut_into_portions_under_the_budget():
    cm, s = make(budget=32)
    r = req(70, new=2)
    s.add(r)
    log = run(s)
    assert [(st, n, w) for _, st, n, w in (step[0] for step in log)] == \
        [(0, 32, False), (32, 32, False), (64, 6, True), (70, 1, True)]
    assert r.done and r.out == [7, 7] and r.cache is None
    assert cm.free_pages()[("paged", None)] == 16 and cm.slots.free_count == 4


def test_decodes_go_first_and_prompts_fill_the_rest():
    cm, s = make(budget=10, num_pages=32)
    a, b = req(4, new=50), req(25, new=3)
    s.add(a)
    fake_step(s, s.schedule())             # a is prefilled whole, now decoding
    s.add(b)
    plan = s.schedule()
    assert [(x.request, x.start, x.count) for x in plan] == [(a, 4, 1), (b, 0, 9)]
    fake_step(s, plan)
    plan = s.schedule()
    assert [(x.request, x.start, x.count, x.wants_logits) for x in plan] == [(a, 5, 1, True), (b, 9, 9, False)]
    fake_step(s, plan)
    plan = s.schedule()
    assert [(x.request, x.start, x.count, x.wants_logits) for x in plan] == [(a, 6, 1, True), (b, 18, 7, True)]


def test_admission_respects_slots_and_pages():
    cm, s = make(num_pages=4, max_seqs=2, budget=100)
    a, b, c = req(30), req(30), req(10)
    for r in (a, b, c):
        s.add(r)
    plan = s.schedule()
    assert [x.request for x in plan] == [a, b]          # c: no slot left
    assert list(s.waiting) == [c] and cm.free_pages()[("paged", None)] == 0


def test_request_longer_than_max_model_len_is_refused():
    _, s = make(max_len=64)
    with pytest.raises(SnowLLMError, match="max_model_len"):
        s.add(req(60, new=8))
    with pytest.raises(SnowLLMError):
        s.add(Request(prompt=[], params=SamplingParams()))


def test_pages_run_out_the_last_admitted_is_preempted_and_replayed():
    # two requests of 30 tokens in 4 pages of 16: both fit; at token 33 one needs a third page
    cm, s = make(num_pages=4, max_seqs=2, budget=100)
    a, b = req(30, new=8), req(30, new=8)
    s.add(a)
    s.add(b)
    log = run(s)
    assert s.preemptions >= 1 and b.preemptions >= 1 and a.preemptions == 0
    assert a.done and b.done and len(a.out) == 8 and len(b.out) == 8
    # b was prefilled again over its prompt and what it had generated
    replays = [(st, n) for step in log for r, st, n, _ in step if r is b and st == 0]
    assert len(replays) == 1 + b.preemptions and replays[1][1] > 30
    assert cm.free_pages()[("paged", None)] == 4 and cm.slots.free_count == 2


def test_request_that_the_pool_cannot_hold_alone_is_refused_when_added():
    """Prompt plus every token it may generate must fit the pool with nothing else in it; the refusal
    touches nothing else."""
    cm, s = make(num_pages=2, max_seqs=2, budget=100, max_len=100)
    ok = req(20, new=12)                              # 32 tokens: the two pages exactly
    s.add(ok)
    with pytest.raises(CapacityError, match="even alone.*4 pages"):
        s.add(req(31, new=20))
    with pytest.raises(CapacityError, match="even alone"):
        s.add(req(40, new=1))
    assert list(s.waiting) == [ok]
    run(s)
    assert ok.done and ok.finish_reason == "length" and len(ok.out) == 12
    assert cm.free_pages()[("paged", None)] == 2 and cm.slots.free_count == 2


def test_lone_request_without_a_page_ends_in_error_and_the_queue_goes_on():
    """What add() cannot foresee (here: the pool shrank under a running request) ends that request with
    finish_reason "error"; it gives everything back and the next request runs."""
    cm, s = make(num_pages=3, max_seqs=1, budget=100, max_len=100)
    a, b = req(31, new=10), req(10, new=2)
    s.add(a)
    s.add(b)
    fake_step(s, s.schedule())                        # a's prompt: two pages, one token out
    held = cm.groups[("paged", None)].alloc(1)        # someone else takes the last page
    plan = s.schedule()                               # position 31 fits a's second page
    fake_step(s, plan)
    plan = s.schedule()                               # position 32 needs a third page: none, and a runs alone
    assert a.done and a.finish_reason == "error" and "cannot hold one request" in a.error
    assert a.cache is None and s.failed == 1
    assert [x.request for x in plan] == [b]           # admitted in the same round, into a's slot
    cm.groups[("paged", None)].release(held)
    fake_step(s, plan)
    run(s)
    assert b.done and b.finish_reason == "length"
    assert cm.free_pages()[("paged", None)] == 3 and cm.slots.free_count == 1


def test_preemption_off_ends_the_request_that_found_no_page():
    cm, s = make(num_pages=4, max_seqs=2, budget=100, preempt=False)
    a, b = req(30, new=8), req(30, new=8)
    s.add(a)
    s.add(b)
    run(s)
    failed = [r for r in (a, b) if r.finish_reason == "error"]
    assert len(failed) == 1 and "preemption is off" in failed[0].error
    other = b if failed[0] is a else a
    assert other.finish_reason == "length" and len(other.out) == 8
    assert cm.free_pages()[("paged", None)] == 4 and cm.slots.free_count == 2


def test_decode_pass_takes_turns_when_the_budget_is_below_the_number_of_decoders():
    cm, s = make(num_pages=32, max_seqs=4, budget=16, max_len=64)
    reqs = [req(4, new=6) for _ in range(4)]
    for r in reqs:
        s.add(r)
    fake_step(s, s.schedule())                        # all four prompts in one step
    assert all(len(r.out) == 1 for r in reqs)
    s.max_num_batched_tokens = 3                      # fewer tokens per step than decoding requests
    served = []
    for _ in range(4):
        plan = s.schedule()
        assert len(plan) == 3 and all(x.count == 1 for x in plan)
        served.append([reqs.index(x.request) for x in plan])
        fake_step(s, plan)
    assert served == [[0, 1, 2], [3, 0, 1], [2, 3, 0], [1, 2, 3]]
    assert all(len(r.out) == 4 for r in reqs)         # everyone advanced alike
    run(s)
    assert all(r.finish_reason == "length" for r in reqs)


def test_abort_gives_everything_back():
    cm, s = make()
    a, b = req(20), req(20)
    s.add(a)
    s.add(b)
    fake_step(s, s.schedule())
    s.abort(a)
    assert a.finish_reason == "abort" and a.cache is None and s.running == [b]
    assert cm.slots.free_count == 3


def test_finished_requests_pages_serve_the_next_request_in_the_next_step():
    cm, s = make(num_pages=2, max_seqs=1, budget=100)
    a, b = req(20, new=1), req(20, new=1)
    s.add(a)
    s.add(b)
    fake_step(s, s.schedule())
    pages_a = None
    assert a.done
    s.retire_finished()
    plan = s.schedule()
    assert plan[0].request is b and sorted(b.cache.tables[("paged", None)]) == [0, 1]


def test_tokens_in_flight_count_as_generated_and_appear_as_references():
    """Overlapped steps: a sampled token that the host has not read yet (``in_flight``: its place among the
    device's pending tokens) is scheduled like a known token, appears in the segment as -(place + 1), and a
    request whose token in flight is its last is not scheduled again."""
    cm, s = make(budget=32)
    a, b = req(5, new=3), req(6, new=1)
    s.add(a)
    s.add(b)
    plan = s.schedule()                               # both prompts whole, logits wanted
    assert [(x.start, x.count, x.wants_logits) for x in plan] == [(0, 5, True), (0, 6, True)]
    for i, x in enumerate(plan):                      # the step ran; its tokens stay on the device
        cm.commit(x.request.cache, x.count)
        x.request.num_computed += x.count
        x.request.in_flight = i
    assert a.generated == 1 and a.pending == 1 and not a.at_length
    assert b.generated == 1 and b.at_length           # its only new token is the one in flight
    plan = s.schedule()
    assert [x.request for x in plan] == [a]           # b waits for its token to land, it is not run again
    assert plan[0].tokens == [-1] and plan[0].start == 5 and plan[0].wants_logits
    # the tokens land: b is done, a goes on with a known token and a new one in flight
    a.in_flight, b.in_flight = -1, -1
    a.out.append(11)
    b.out.append(12)
    b.done, b.finish_reason = True, "length"
    cm.commit(a.cache, 6)
    a.num_computed += 1
    a.in_flight = 0
    s.retire_finished()
    assert b.cache is None and s.running == [a]
    plan = s.schedule()
    assert plan[0].tokens == [-1] and plan[0].start == 6 and a.tokens[-2:] == [11, -1]


def test_a_segments_tokens_are_cut_without_joining_the_lists():
    """Request.tokens_at(start, count) is tokens[start:start + count] for every cut, with and without a
    token still on the device (a decode step of a long request must not copy its whole history)."""
    import random
    rng = random.Random(0)
    for _ in range(2000):
        r = Request(prompt=list(range(100, 100 + rng.randint(1, 9))), params=SamplingParams())
        r.out = list(range(500, 500 + rng.randint(0, 6)))
        r.in_flight = rng.choice([-1, 0, 3])
        full = r.tokens
        start = rng.randint(0, len(full))
        count = rng.randint(0, len(full) - start + 2)
        assert r.tokens_at(start, count) == full[start:start + count]
