"""The Engine's host side on the CPU, against a fake step function, a fake sampler and a fake status
watch (in the manner of the fakes of tests/test_single_model_path.py:12-46 in SnowLLM): a step that
fails ends its requests with finish_reason "error", gives their pages and slots back and leaves the
engine serving; a kernel's status word is surfaced; the budget of captured steps."""
import pytest
import torch

from snowllm_b200.cache import CacheManager
from snowllm_b200.config.engine import EngineConfig
from snowllm_b200.engine.engine import Engine
from snowllm_b200.engine.graphs import GraphCache
from snowllm_b200.engine.request import SamplingParams
from snowllm_b200.errors import KernelError, SnowLLMError
from snowllm_b200.parts.spec import PagedKVSpec, SlotStateSpec

SPECS = {0: PagedKVSpec(2, 16), 1: SlotStateSpec(((2, 8),))}
VOCAB = 50


class FakeModel:
    vocab_size = VOCAB
    dtype = torch.float32


class FakeRunner:
    """Stands in for the step function: commits what it is given, returns one row of "logits" per wanted
    place whose argmax is (last token + 1) % VOCAB; raises when told to."""

    def __init__(self, cache):
        self.cache = cache
        self.pending_tokens = torch.zeros(256, dtype=torch.int32)
        self.fail_on: set = set()          # step numbers that raise
        self.fail_after_commit = False
        self.calls = 0

    def step(self, entries):
        self.calls += 1
        if self.calls in self.fail_on and not self.fail_after_commit:
            raise RuntimeError(f"injected failure in step {self.calls}")
        rows = []
        for e in entries:
            for w in e.want:
                row = torch.zeros(VOCAB)
                row[(int(e.tokens[w]) + 1) % VOCAB] = 1.0
                rows.append(row)
            self.cache.commit(e.cache, e.cache.num_tokens + len(e.tokens))
        if self.calls in self.fail_on:
            raise RuntimeError(f"injected failure in step {self.calls}")
        return torch.stack(rows) if rows else torch.zeros(0, VOCAB)


class FakeSampler:
    stop_token_ids = frozenset()

    @staticmethod
    def needs_history(rows):
        return False

    def sample(self, logits, rows):
        return logits.argmax(-1).tolist()

    def append(self, r, token):
        r.out.append(int(token))
        if len(r.out) >= r.params.max_new_tokens:
            r.done, r.finish_reason = True, "length"


class FakeStatus:
    def __init__(self):
        self.word = 0
        self.peeks = 0

    def peek(self):
        self.peeks += 1

    def check(self):
        if self.word:
            word, self.word = self.word, 0
            raise KernelError(f"a bounded wait ran out inside a kernel (code {word})")


def make(num_pages=16, max_seqs=3, budget=8, status=None):
    cache = CacheManager(SPECS, 16, num_pages, max_seqs)
    runner = FakeRunner(cache)
    eng = Engine(FakeModel(), runner=runner, sampler=FakeSampler(), status=status, device="cpu",
                 max_num_seqs=max_seqs, max_model_len=num_pages * 16, prefill_chunk=budget, overlap_steps=False)
    return eng, runner, cache


def everything_is_back(cache, num_pages, max_seqs):
    return cache.free_pages()[("paged", None)] == num_pages and cache.slots.free_count == max_seqs


def expected(prompt, n):
    out, last = [], prompt[-1]
    for _ in range(n):
        last = (last + 1) % VOCAB
        out.append(last)
    return out


def test_fake_engine_generates():
    eng, runner, cache = make()
    reqs = [eng.add([1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11], SamplingParams(temperature=0, max_new_tokens=4)),
            eng.add([20, 21], SamplingParams(temperature=0, max_new_tokens=6))]
    eng.run()
    assert [r.out for r in reqs] == [expected(r.prompt, r.params.max_new_tokens) for r in reqs]
    assert all(r.finish_reason == "length" for r in reqs)
    assert everything_is_back(cache, 16, 3)


@pytest.mark.parametrize("after_commit", [False, True])
def test_failed_step_ends_its_requests_and_the_engine_goes_on(after_commit):
    eng, runner, cache = make(max_seqs=2)
    runner.fail_on, runner.fail_after_commit = {3}, after_commit
    a = eng.add(list(range(1, 6)), SamplingParams(temperature=0, max_new_tokens=8))
    b = eng.add(list(range(10, 13)), SamplingParams(temperature=0, max_new_tokens=8))
    c = eng.add(list(range(30, 34)), SamplingParams(temperature=0, max_new_tokens=3))      # waits: two slots only
    kinds = []
    while eng.scheduler.has_work():
        kinds.append(eng.step())
        assert len(kinds) < 100
    eng.scheduler.retire_finished()
    assert kinds.count("error") == 1 and kinds.index("error") == 2
    assert a.finish_reason == "error" and b.finish_reason == "error"
    assert "injected failure in step 3" in a.error and a.cache is None and b.cache is None
    assert len(a.out) == 2 and a.out == expected(a.prompt, 2)       # what it had generated stays readable
    assert c.finish_reason == "length" and c.out == expected(c.prompt, 3)
    assert eng.step_errors == 1 and "injected failure" in eng.last_error
    assert eng.stats().failed_requests == 2
    assert everything_is_back(cache, 16, 2)
    d = eng.add([40, 41], SamplingParams(temperature=0, max_new_tokens=2))                 # and it still serves
    eng.run()
    assert d.out == expected(d.prompt, 2) and everything_is_back(cache, 16, 2)


def test_host_side_refusal_inside_a_step_ends_the_requests_of_that_step():
    """An exception raised before anything ran on the device (a check of the step's inputs) is handled like
    any other failure: the step's requests end in error, later requests run."""
    eng, runner, cache = make(max_seqs=2, budget=4)
    a = eng.add(list(range(1, 4)), SamplingParams(temperature=0, max_new_tokens=5))
    eng.step()                                                       # a's prompt
    eng.step()                                                       # a decodes
    b = eng.add([0] * 3, SamplingParams(temperature=0, max_new_tokens=2))
    real = runner.step

    def picky(entries):
        if any(list(e.tokens) == [0, 0, 0] for e in entries):
            # the step holds a's token and b's prompt; the host-side check on b's portion raises
            raise SnowLLMError("portion refused")
        return real(entries)
    runner.step = picky
    assert eng.step() == "error"
    assert b.finish_reason == "error" and a.finish_reason == "error"   # both were in the step
    assert everything_is_back(cache, 16, 2)
    runner.step = real
    c = eng.add([5, 6], SamplingParams(temperature=0, max_new_tokens=2))
    eng.run()
    assert c.out == expected(c.prompt, 2)


def test_status_word_of_a_kernel_is_surfaced_as_a_failed_step():
    status = FakeStatus()
    eng, runner, cache = make(max_seqs=2, status=status)
    a = eng.add(list(range(1, 6)), SamplingParams(temperature=0, max_new_tokens=4))
    w = eng.add(list(range(7, 9)), SamplingParams(temperature=0, max_new_tokens=2))
    assert eng.step() == "prefill" and status.peeks == 1
    status.word = 2                                                   # a wait ran out inside the next step
    assert eng.step() == "error"
    assert a.finish_reason == "error" and "bounded wait" in a.error and "code 2" in eng.last_error
    assert w.finish_reason == "error"                                 # a device fault ends everything that ran
    assert everything_is_back(cache, 16, 2)
    ok = eng.add([3, 4], SamplingParams(temperature=0, max_new_tokens=3))
    eng.run()
    assert ok.out == expected(ok.prompt, 3) and ok.finish_reason == "length"


def test_engine_settings_are_validated_and_named_as_in_the_reference():
    c = EngineConfig.from_kwargs(max_num_seqs=2, prefill_chunk=64, stop_token_ids=[3, 4], max_model_len=128)
    assert c.max_num_batched_tokens == 64 and c.stop_token_ids == (3, 4)
    with pytest.raises(SnowLLMError, match="max_num_seqs=0"):
        EngineConfig(max_num_seqs=0)
    with pytest.raises(SnowLLMError, match="max_num_seqs=300.*gpu_memory_utilization=1.5"):
        EngineConfig(max_num_seqs=300, gpu_memory_utilization=1.5)
    with pytest.raises(SnowLLMError, match="no setting 'chunk'"):
        EngineConfig.from_kwargs(chunk=3)
    eng, _, _ = make()
    assert eng.config.max_num_batched_tokens == 8 and eng.prefill_chunk == 8
    with pytest.raises(SnowLLMError, match="not both"):
        Engine(FakeModel(), EngineConfig(), runner=FakeRunner(CacheManager(SPECS, 16, 4, 2)), max_num_seqs=2)


# --- captured steps under a budget ---------------------------------------------------------

class FakeMemory:
    def __init__(self, in_use=0):
        self.in_use = in_use
        self.released = 0

    def __call__(self):
        return self.in_use

    def release(self):
        self.released += 1


def capture(mem, cost, log, key, fail=False):
    def run():
        if fail:
            raise MemoryError("out of memory while capturing")
        mem.in_use += cost
        log.append(key)
        return f"graph{key}"
    return run


def test_graph_cache_keeps_the_most_recently_used_captures():
    mem, log = FakeMemory(), []
    g = GraphCache(max_graphs=3, ceiling_bytes=None, in_use=mem, release=mem.release)
    for key in (1, 2, 3):
        assert g.get(key, capture(mem, 10, log, key)) == f"graph{key}"
    assert g.get(1, capture(mem, 10, log, 1)) == "graph1" and log == [1, 2, 3]     # a hit captures nothing
    assert g.get(4, capture(mem, 10, log, 4)) == "graph4"                         # 2 is the least recently used
    assert list(g.entries) == [3, 1, 4] and g.evictions == 1
    assert g.get(2, capture(mem, 10, log, 2)) == "graph2" and list(g.entries) == [1, 4, 2]
    assert g.snapshot()["captures"] == 5 and not g.full


def test_graph_cache_stops_at_the_memory_ceiling_and_steps_run_launch_by_launch():
    mem, log = FakeMemory(in_use=100), []
    g = GraphCache(max_graphs=100, ceiling_bytes=150, in_use=mem, release=mem.release)
    assert g.get("a", capture(mem, 20, log, "a")) == "grapha"         # the first costs nothing known yet
    assert g.largest == 20
    assert g.get("b", capture(mem, 15, log, "b")) == "graphb"         # 120 + 20 <= 150
    assert g.get("c", capture(mem, 20, log, "c")) is None             # 135 + 20 > 150: no capture
    assert g.full and g.refused == 1 and log == ["a", "b"]
    assert g.get("a", capture(mem, 20, log, "a")) == "grapha"         # what exists keeps serving
    assert g.get("d", capture(mem, 1, log, "d")) is None and g.refused == 2


def test_graph_cache_survives_out_of_memory_inside_a_capture():
    mem, log = FakeMemory(), []
    g = GraphCache(max_graphs=8, ceiling_bytes=None, in_use=mem, release=mem.release)
    assert g.get(1, capture(mem, 10, log, 1)) == "graph1"
    assert g.get(2, capture(mem, 10, log, 2, fail=True)) is None
    assert g.full and mem.released == 1 and list(g.entries) == [1]
    assert g.get(1, None) == "graph1"
    assert g.get(3, capture(mem, 10, log, 3)) is None                 # nothing more is captured
    zero = GraphCache(max_graphs=0, ceiling_bytes=None, in_use=mem)
    assert zero.get(1, capture(mem, 10, log, 1)) is None
