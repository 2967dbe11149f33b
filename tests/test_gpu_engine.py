"""Generation through the Python entry point and the command line: greedy tokens against the plain
implementation, chunked prefill, batching, preemption and replay, sampling, and the smoke entry."""
import json
import pathlib
import subprocess
import sys

import pytest
import torch

import plain_lfm2 as plain
from helpers import random_prompt
from tiny_configs import ALL

pytestmark = pytest.mark.gpu
ROOT = pathlib.Path(__file__).resolve().parent.parent


def engine_for(model_dir, dtype="float32", **kw):
    import snowllm_b200
    from snowllm_b200.engine import Engine
    model = snowllm_b200.load(model_dir, dtype)
    kw.setdefault("max_model_len", 512)
    if "num_kv_blocks" in kw:
        kw.setdefault("page_size", 16)          # the tests that count pages count pages of 16 tokens
    return Engine(model, **kw)


def assert_greedy_follows_plain(model_dir, prompt, out, slack):
    """Each generated token is the plain implementation's argmax given the same prefix, or within
    ``slack`` of it (a near-tie that rounding may turn)."""
    cfg, tensors = plain.read_model_dir(model_dir)
    logits = plain.logits(cfg, tensors, prompt + out)
    for i, tok in enumerate(out):
        row = logits[len(prompt) - 1 + i]
        assert float(row.max() - row[tok]) <= slack, (i, tok, int(row.argmax()), float(row.max() - row[tok]))


def test_greedy_generation_tiny_a_float32(model_dirs):
    """16-token prompts, 8 generated tokens, equal to whole-sequence greedy decoding."""
    from snowllm_b200.engine import SamplingParams
    d = model_dirs("tiny_a", "float32")
    cfg, tensors = plain.read_model_dir(d)
    eng = engine_for(d, max_num_seqs=2)
    prompts = [random_prompt(256, 16, s) for s in range(3)]
    outs = eng.generate(prompts, SamplingParams(temperature=0, max_new_tokens=8))
    for p, o in zip(prompts, outs):
        assert len(o) == 8
        assert_greedy_follows_plain(d, p, o, slack=1e-4)
    assert outs[0] == plain.greedy(cfg, tensors, prompts[0], 8)
    st = eng.stats()
    assert st.running == 0 and st.waiting == 0 and st.free_slots == 2
    assert st.accounting["prefill_tokens"] == 48 and st.accounting["decode_tokens"] == 21


@pytest.mark.parametrize("name,dtype,slack", [("tiny_b", "float32", 1e-4), ("tiny_dense", "bfloat16", 0.2)])
def test_mixed_batch(model_dirs, name, dtype, slack):
    """Three prompts of 5, 23 and 40 tokens together, 12 generated tokens each.  In bfloat16 the
    model without a router is used: a router pick that rounding turns changes the continuation, which
    the replay tests handle by forcing the plain implementation onto the engine's picks."""
    from snowllm_b200.engine import SamplingParams
    d = model_dirs(name, dtype)
    eng = engine_for(d, dtype, max_num_seqs=4, prefill_chunk=16)
    prompts = [random_prompt(ALL[name]["vocab_size"], n, 7 + n) for n in (5, 23, 40)]
    reqs = [eng.add(p, SamplingParams(temperature=0, max_new_tokens=12)) for p in prompts]
    kinds = []
    while eng.scheduler.has_work():
        kinds.append(eng.step())
    assert "mixed" in kinds                      # prompt portions ran beside decoded tokens
    for p, r in zip(prompts, reqs):
        assert r.done and r.finish_reason == "length" and len(r.out) == 12
        assert_greedy_follows_plain(d, p, r.out, slack)


def test_chunked_prefill_and_batching_do_not_change_greedy_tokens(model_dirs):
    from snowllm_b200.engine import SamplingParams
    d = model_dirs("tiny_b", "float32")
    params = SamplingParams(temperature=0, max_new_tokens=24)
    prompts = [random_prompt(384, n, 50 + n) for n in (37, 90, 12)]
    eng = engine_for(d, max_num_seqs=1, prefill_chunk=64)
    alone = [eng.generate([p], params)[0] for p in prompts]
    eng.prefill_chunk = 3
    assert [eng.generate([p], params)[0] for p in prompts] == alone
    together = engine_for(d, max_num_seqs=3, prefill_chunk=7).generate(prompts, params)
    assert together == alone


def test_pages_run_out_preemption_replays_to_the_same_tokens(model_dirs):
    """Two requests of 90 tokens and 40 new tokens in a pool of 13 pages of 16: one is preempted,
    prefilled again over what it had generated, and ends with the tokens of an undisturbed run
    (SnowLLM: tests/test_lfm2_scheduling.py:24-48)."""
    from snowllm_b200.engine import SamplingParams
    d = model_dirs("tiny_a", "float32")
    params = SamplingParams(temperature=0, max_new_tokens=40)
    prompts = [random_prompt(256, 90, s) for s in (1, 2)]
    calm = engine_for(d, max_num_seqs=2, max_model_len=256).generate(prompts, params)
    tight = engine_for(d, max_num_seqs=2, max_model_len=256, num_kv_blocks=13)
    got = tight.generate(prompts, params)
    assert tight.stats().preemptions > 0
    assert got == calm
    assert tight.stats().free_kv_blocks == 13 and tight.stats().free_slots == 2


def test_stop_tokens_and_limits(model_dirs):
    from snowllm_b200.engine import SamplingParams
    from snowllm_b200.errors import SnowLLMError
    d = model_dirs("tiny_a", "float32")
    eng = engine_for(d, max_num_seqs=2, max_model_len=64)
    p = random_prompt(256, 10, 3)
    free = eng.generate([p], SamplingParams(temperature=0, max_new_tokens=12))[0]
    r = eng.add(p, SamplingParams(temperature=0, max_new_tokens=12, stop_token_ids=(free[4],)))
    eng.run()
    first = free.index(free[4])
    assert r.finish_reason == "stop" and r.out == free[:first + 1]
    with pytest.raises(SnowLLMError, match="max_model_len"):
        eng.add(random_prompt(256, 60, 1), SamplingParams(max_new_tokens=8))
    with pytest.raises(SnowLLMError, match="token id"):
        eng.add([1, 2, 999], SamplingParams())
    full = eng.add(random_prompt(256, 56, 2), SamplingParams(temperature=0, max_new_tokens=8))
    eng.run()                                     # up to exactly max_model_len
    assert len(full.out) == 8


def test_overlapped_steps_give_the_tokens_of_steps_read_back_one_by_one(model_dirs):
    """Tokens that stay on the device for a step (overlap_steps) change nothing: the same requests with
    stop tokens, with mixed lengths, with a seeded draw, and through a preemption."""
    from snowllm_b200.engine import SamplingParams
    d = model_dirs("tiny_a", "float32")
    prompts = [random_prompt(256, n, 30 + n) for n in (5, 23, 40, 17)]
    free = engine_for(d, max_num_seqs=4, overlap_steps=False).generate(
        prompts, SamplingParams(temperature=0, max_new_tokens=20))
    stops = (free[0][6], free[2][11])

    def run(overlap, **kw):
        eng = engine_for(d, max_num_seqs=4, prefill_chunk=16, seed=5, overlap_steps=overlap, **kw)
        pages = eng.stats().free_kv_blocks
        reqs = [eng.add(p, SamplingParams(temperature=0, max_new_tokens=20, stop_token_ids=stops)) for p in prompts[:3]]
        reqs.append(eng.add(prompts[3], SamplingParams(temperature=0.9, top_k=20, max_new_tokens=9)))
        eng.run()
        assert all(r.done and r.in_flight < 0 for r in reqs)
        assert eng.stats().running == 0 and eng.stats().free_slots == 4 and eng.stats().free_kv_blocks == pages
        return [(r.out, r.finish_reason) for r in reqs], eng
    one_by_one, _ = run(False)
    overlapped, eng = run(True)
    assert overlapped == one_by_one
    assert one_by_one[0][1] == "stop" and one_by_one[0][0] == free[0][:free[0].index(stops[0]) + 1]
    # few pages: a request is preempted while tokens are in flight
    params = SamplingParams(temperature=0, max_new_tokens=40)
    long = [random_prompt(256, 90, s) for s in (1, 2)]
    calm = engine_for(d, max_num_seqs=2, max_model_len=256, overlap_steps=False).generate(long, params)
    tight = engine_for(d, max_num_seqs=2, max_model_len=256, num_kv_blocks=13, overlap_steps=True)
    assert tight.generate(long, params) == calm and tight.stats().preemptions > 0


def test_graph_steps_follow_launch_by_launch_steps_across_key_chunks(model_dirs):
    """Decoding from 500 to 830 tokens crosses several 256-key chunks inside one captured graph's range
    (the chunk count is rounded up to a power of two): the captured steps must look at every chunk."""
    from snowllm_b200.engine import SamplingParams
    d = model_dirs("tiny_e", "float32")
    prompts = [random_prompt(ALL["tiny_e"]["vocab_size"], n, n) for n in (500, 300)]
    params = SamplingParams(temperature=0, max_new_tokens=330)
    eager = engine_for(d, max_num_seqs=2, max_model_len=2048, enforce_eager=True).generate(prompts, params)
    eng = engine_for(d, max_num_seqs=2, max_model_len=2048)
    assert eng.generate(prompts, params) == eager
    assert eng.runner.graph_replays > 300


def test_sampling_is_seeded_and_penalties_bite(model_dirs):
    from snowllm_b200.engine import SamplingParams
    d = model_dirs("tiny_a", "float32", flavour="baseline")
    p = random_prompt(256, 12, 9)
    hot = SamplingParams(temperature=1.0, top_k=40, top_p=0.95, max_new_tokens=24)
    a = engine_for(d, seed=11).generate([p], hot)[0]
    b = engine_for(d, seed=11).generate([p], hot)[0]
    c = engine_for(d, seed=12).generate([p], hot)[0]
    assert a == b and a != c and all(0 <= t < 256 for t in a)
    # with these weights greedy decoding repeats itself; a ban on repeated 2-grams must not
    eng = engine_for(d)
    plain_out = eng.generate([p], SamplingParams(temperature=0, max_new_tokens=40))[0]
    banned = eng.generate([p], SamplingParams(temperature=0, max_new_tokens=40, no_repeat_ngram_size=2))[0]
    seq = p + banned
    grams = [tuple(seq[i:i + 2]) for i in range(len(seq) - 1)]
    new = grams[len(p) - 1:]
    assert len(set(new)) == len(new) and not set(new) & set(grams[:len(p) - 1])
    # penalties through the engine: every token it picks is the best one of the plain logits with the penalties
    # applied by hand (snowllm/engine/sampler.py:187-219: seen tokens' logits divided by the repetition penalty
    # when positive, multiplied when negative; minus frequency x count and presence for generated tokens)
    rep, freq, pres = 1.5, 0.02, 0.01
    pen = eng.generate([p], SamplingParams(temperature=0, max_new_tokens=24, repetition_penalty=rep,
                                            frequency_penalty=freq, presence_penalty=pres))[0]
    assert pen != plain_out[:24], "the penalties changed nothing"
    cfg, tensors = plain.read_model_dir(d)
    from collections import Counter
    for i, tok in enumerate(pen):
        row = plain.logits(cfg, tensors, p + pen[:i])[-1].clone()
        counts = Counter(pen[:i])
        for t in set(p) | set(pen[:i]):
            row[t] = row[t] / rep if row[t] > 0 else row[t] * rep
            row[t] -= freq * counts.get(t, 0) + (pres if counts.get(t, 0) else 0.0)
        assert float(row.max() - row[tok]) <= 1e-4, f"token {i}: {tok} is not the best penalised token"


def test_command_line_generates(model_dirs):
    d = model_dirs("tiny_a", "float32")
    p = random_prompt(256, 9, 21)
    proc = subprocess.run([sys.executable, "-m", "snowllm_b200", str(d), "--dtype", "float32", "--prompt-ids",
                           ",".join(map(str, p)), "--default-max-tokens", "6", "--max-model-len", "128",
                           "--max-num-seqs", "2", "--temperature", "0"],
                          capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = json.loads(proc.stdout.strip().splitlines()[-1])
    cfg, tensors = plain.read_model_dir(d)
    assert line["tokens"] == plain.greedy(cfg, tensors, p, 6) and line["finish_reason"] == "length"


def test_random_weights_command_and_missing_extension_is_loud(tmp_path):
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(ALL["tiny_dense"]))
    proc = subprocess.run([sys.executable, "-m", "snowllm_b200", "random-weights", str(cfg), str(tmp_path / "m"),
                           "--seed", "4", "--dtype", "float32"], capture_output=True, text=True, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr
    c, tensors = plain.read_model_dir(tmp_path / "m")
    assert plain.logits(c, tensors, [1, 2, 3]).shape == (3, 200)
    from snowllm_b200.errors import KernelError
    from snowllm_b200.ops import kernels
    with pytest.raises(KernelError, match="CUDA tensor"):
        kernels.swiglu(torch.zeros(2, 4))        # no CPU path


def test_smoke_entry():
    sys.path.insert(0, str(ROOT))
    import __graft_entry__
    __graft_entry__.smoke()


@pytest.mark.parametrize("overlap,max_graphs", [(True, 3), (False, 64)])
def test_many_requests_under_pressure_match_calm_runs(model_dirs, overlap, max_graphs):
    """Thirty requests of random lengths and reply limits, some with stop tokens, one aborted on the way, arriving
    a few at a time while others run, four at a time in a pool so small that requests are preempted and
    replayed, portions of 24 tokens, captured decode steps (with room for three captures only, so that
    captures are dropped and made again): every request ends with the tokens it gets when it runs alone in a
    roomy engine, and every page and slot comes back."""
    import random

    from snowllm_b200.engine import SamplingParams
    d = model_dirs("tiny_a", "float32")
    rng = random.Random(7)
    jobs = []
    for i in range(30):
        prompt = random_prompt(256, rng.randint(3, 90), 200 + i)
        jobs.append((prompt, rng.randint(4, 40)))
    roomy = engine_for(d, max_num_seqs=1, max_model_len=256)
    alone = []
    for prompt, n in jobs:
        alone.append(roomy.generate([prompt], SamplingParams(temperature=0, max_new_tokens=n))[0])
    # stop tokens for every fourth request: a token its calm run produced in the middle
    params = []
    for i, ((prompt, n), out) in enumerate(zip(jobs, alone)):
        stop = (out[len(out) // 2],) if i % 4 == 0 else ()
        params.append(SamplingParams(temperature=0, max_new_tokens=n, stop_token_ids=stop))
    tight = engine_for(d, max_num_seqs=4, max_model_len=160, num_kv_blocks=11, prefill_chunk=24, overlap_steps=overlap,
                       max_graphs=max_graphs)
    arrivals = list(zip(jobs, params))
    reqs = [tight.add(prompt, p) for (prompt, _), p in arrivals[:12]]
    steps = 0
    while tight.scheduler.has_work() or len(reqs) < len(arrivals):
        if steps % 9 == 0:                               # the others arrive while the first ones run
            for (prompt, _), p in arrivals[len(reqs):len(reqs) + 2]:
                reqs.append(tight.add(prompt, p))
        tight.step()
        steps += 1
        if steps == 25:
            tight.abort(reqs[11])
        assert steps < 5000
    tight.run()
    assert tight.stats().preemptions > 0, "the pool was meant to be too small for four requests at a time"
    if max_graphs == 3:
        assert tight.stats().graphs["evictions"] > 0, "three captures were meant to be too few"
    for i, (r, out, p) in enumerate(zip(reqs, alone, params)):
        if i == 11:
            assert r.finish_reason in ("abort", "length", "stop")
            assert r.out == out[:len(r.out)]
            continue
        want = out[:out.index(p.stop_token_ids[0]) + 1] if p.stop_token_ids else out
        assert r.out == want, f"request {i}: {r.out} against {want} (preempted {r.preemptions} times)"
        assert r.finish_reason == ("stop" if p.stop_token_ids else "length")
    st = tight.stats()
    assert st.free_kv_blocks == 11 and st.free_slots == 4 and st.running == 0 and st.waiting == 0
    assert st.step_errors == 0 and st.failed_requests == 0


def test_named_spans_show_up_on_a_profilers_timeline(model_dirs, tmp_path):
    """With tracing on, the engine's step and every part's work carry a name in a torch.profiler session; the
    command line's --enable-profiler writes a Chrome trace."""
    from torch.profiler import ProfilerActivity, profile

    from snowllm_b200 import trace
    from snowllm_b200.engine import SamplingParams
    d = model_dirs("tiny_a", "float32")
    eng = engine_for(d, max_num_seqs=2, enforce_eager=True)
    assert trace.span("x") is trace.span("y")              # off: one shared do-nothing context
    with profile(activities=[ProfilerActivity.CPU]) as prof:   # a running session switches the spans on
        eng.generate([random_prompt(256, 9, 1)], SamplingParams(temperature=0, max_new_tokens=3))
    names = {e.name for e in prof.events()}
    for want in ("engine.step", "embedding", "mixer:ShortConv", "mixer:Attention", "ffn:SigmoidMoE", "ffn:SwiGLU",
                 "norm:RMSNorm", "head", "run[2]:layer2"):
        assert want in names, f"no span named {want!r} (have {sorted(n for n in names if ':' in n)[:8]} ...)"
    out = tmp_path / "prof"
    proc = subprocess.run([sys.executable, "-m", "snowllm_b200", str(d), "--dtype", "float32", "--prompt-ids", "1,2,3",
                           "--default-max-tokens", "2", "--max-model-len", "64", "--enable-profiler", "--profile-dir",
                           str(out)], capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert (out / "trace.json").stat().st_size > 1000
