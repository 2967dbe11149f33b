"""Decode steps as captured CUDA graphs in bfloat16, at the head sizes the tensor-core decode kernels take
(64 and 128): what the measurements time.  A captured step is built for a rounded-up number of key chunks and
a rounded-up block-table width and is replayed over changing lengths; its logits must be those of the same
step run launch by launch, over hundreds of steps that cross chunk edges (256 keys) and the edges at which a
new capture is made (powers of two)."""
import pytest
import torch

from helpers import check_against_plain, decode_tail_trace, max_live_tokens, random_prompt, run_in_process
from tiny_configs import ALL

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["tiny_e", "tiny_f"])
def test_captured_decode_steps_give_the_logits_of_launch_by_launch_steps(model_dirs, name):
    import snowllm_b200
    from snowllm_b200.cache import CacheManager
    from snowllm_b200.engine import ModelRunner, StepEntry
    model = snowllm_b200.load(model_dirs(name, "bfloat16"), "bfloat16")
    V = ALL[name]["vocab_size"]
    prompts = [random_prompt(V, n, 70 + i) for i, n in enumerate((200, 250, 500))]
    steps = 340                                        # lengths 200..540, 250..590, 500..840
    feed = [random_prompt(V, steps, 80 + i) for i in range(3)]
    runs = []
    for graphs in (False, True):
        cache = CacheManager(model.cache_specs(), 16, 3 * 56, 3, model.dtype, "cuda")
        runner = ModelRunner(model, cache, "cuda", use_graphs=graphs)
        rcs = [cache.admit() for _ in prompts]
        for rc, p in zip(rcs, prompts):
            assert cache.ensure(rc, len(p))
        runner.step([StepEntry(rc, p, []) for rc, p in zip(rcs, prompts)])
        outs = []
        for i in range(steps):
            for rc in rcs:
                assert cache.ensure(rc, rc.num_tokens + 1)
            outs.append(runner.step([StepEntry(rc, [feed[b][i]], [0]) for b, rc in enumerate(rcs)]).clone())
        runs.append((torch.stack(outs), runner))
    (eager, eager_runner), (graph, graph_runner) = runs
    assert eager_runner.graph_replays == 0 and graph_runner.graph_replays == steps
    assert len(graph_runner.graphs) >= 2, "the lengths were meant to cross an edge at which a new capture is made"
    worst = float(((graph - eager).norm(dim=-1) / eager.norm(dim=-1)).max())
    assert worst < 1e-5, f"captured steps differ from launch-by-launch steps (rel {worst:.3g})"
    from snowllm_b200.ops import kernels
    assert kernels.attention_decode_status() == 0


@pytest.mark.parametrize("name,page_size", [("tiny_e", 16), ("tiny_f", 16), ("tiny_e", 64)])
def test_decode_tail_through_captured_steps_matches_the_plain_implementation(model_dirs, name, page_size):
    """The decode-tail cut (most of a request in one step, its last tokens one by one) with the one-token
    steps replayed from captures, against the plain implementation; the routers' picks come from the same
    trace run launch by launch (a tapped step is never a captured one)."""
    d = model_dirs(name, "bfloat16")
    V = ALL[name]["vocab_size"]
    reqs = {k: random_prompt(V, n, 90 + i) for i, (k, n) in enumerate({"a": 310, "b": 530, "c": 77}.items())}
    steps = decode_tail_trace(reqs, tail=70)
    stats = {}
    captured, _ = run_in_process(d, "bfloat16", steps, max_live_tokens(steps), use_graphs=True, taps=False, stats=stats,
                                 page_size=page_size)
    assert stats["graph_replays"] == 3 * 70
    plainly, routes = run_in_process(d, "bfloat16", steps, max_live_tokens(steps), page_size=page_size)
    for a, b in zip(captured, plainly):
        assert float(((a - b).norm(dim=-1) / b.norm(dim=-1)).max()) < 1e-5
    check_against_plain(d, "bfloat16", reqs, steps, captured, routes)
