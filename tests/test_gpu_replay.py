"""The engine against the plain implementation under every way of cutting the work, in float32 and
in bfloat16: each request alone and whole; most of it in one step and the last 32 tokens one by
one; portions of changing size; and mixed, up to four live requests with so few pages that they are
used again.  In-process through the replay driver (with the routers' picks tapped), and once per
dtype through the ``bin/trace_run`` program itself."""
import json
import pathlib
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_lfm2 as plain
from helpers import (check_against_plain, check_parts, decode_tail_trace, gather_logits, max_live_tokens, mixed_trace,
                     portions_trace, random_prompt, rel_rows, run_in_process, whole_trace)
from tiny_configs import ALL

pytestmark = pytest.mark.gpu
ROOT = pathlib.Path(__file__).resolve().parent.parent

LENGTHS = {"a": 70, "b": 133, "c": 45, "d": 97, "e": 150, "f": 64}
CUTS = {"whole": whole_trace, "decode_tail": decode_tail_trace, "portions": portions_trace, "mixed": mixed_trace}


def requests_for(cfg, seed=0):
    return {k: random_prompt(cfg["vocab_size"], n, seed + i) for i, (k, n) in enumerate(LENGTHS.items())}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c", "tiny_dense", "tiny_e", "tiny_f"])
@pytest.mark.parametrize("cut", list(CUTS))
def test_cuts_match_the_plain_implementation(model_dirs, name, dtype, cut):
    d = model_dirs(name, dtype)
    reqs = requests_for(ALL[name])
    steps = CUTS[cut](reqs)
    stats = {}
    outputs, routes = run_in_process(d, dtype, steps, max_live_tokens(steps), stats=stats)
    check_parts(d, dtype, stats["parts"], routes)
    check_against_plain(d, dtype, reqs, steps, outputs, routes)


def test_cuts_agree_with_one_another_in_float32(model_dirs):
    """Whole, decoded, portioned and mixed runs of the same requests: float32 logits differ by the
    rounding of the attention's key chunking at most."""
    d = model_dirs("tiny_b", "float32")
    reqs = requests_for(ALL["tiny_b"])
    ref = None
    for cut in ("whole", "decode_tail", "portions", "mixed"):
        steps = CUTS[cut](reqs)
        outputs, _ = run_in_process(d, "float32", steps, max_live_tokens(steps))
        got = gather_logits(steps, outputs)
        if ref is None:
            ref = got
            continue
        for k in reqs:
            assert float(rel_rows(got[k], ref[k]).max()) < 1e-5, (cut, k)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page_size", [16, 64])
def test_mixed_with_reused_pages_poisoned(model_dirs, dtype, page_size):
    """Pages and state slots that are free are filled with NaN before every step, so whatever a
    request gets was poisoned since its last owner: nothing stale may be read (SnowLLM poisons
    scratch and state the same way, tests/test_lfm2.py:31-71)."""
    d = model_dirs("tiny_a", dtype)
    reqs = requests_for(ALL["tiny_a"], seed=10)
    steps = mixed_trace(reqs, seed=3)
    stats = {}
    outputs, routes = run_in_process(d, dtype, steps, max_live_tokens(steps), page_size=page_size, poison=True,
                                     stats=stats)
    assert stats["reused"], "the trace was meant to use pages again"
    got = gather_logits(steps, outputs)
    assert all(v.isfinite().all() for v in got.values()), "a stale (NaN) page or slot was read"
    check_against_plain(d, dtype, reqs, steps, outputs, routes)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(model_dirs, dtype):
    """A short prompt, then 300 tokens one by one (across many page edges); and sequences of one,
    two and three tokens, whole and token by token."""
    name = "tiny_e" if dtype == "bfloat16" else "tiny_b"      # bfloat16: the model with head size 64
    d = model_dirs(name, dtype)
    cfg = ALL[name]
    long = random_prompt(cfg["vocab_size"], 340, 5)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": long[:40], "want": list(range(40))}], "end": []}]
    steps += [{"step": i - 39, "entries": [{"id": "x", "tokens": [long[i]], "want": [0]}],
               "end": ["x"] if i == 339 else []} for i in range(40, 340)]
    outputs, routes = run_in_process(d, dtype, steps, 384)
    check_against_plain(d, dtype, {"x": long}, steps, outputs, routes)
    for n in (1, 2, 3):
        toks = random_prompt(cfg["vocab_size"], n, 20 + n)
        for cut in (whole_trace, lambda r: decode_tail_trace(r, tail=8)):
            steps = cut({"s": toks})
            outputs, routes = run_in_process(d, dtype, steps, 64)
            check_against_plain(d, dtype, {"s": toks}, steps, outputs, routes)


def run_program(model_dir, dtype, steps, out):
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype",
                           dtype, "--out", str(out), "--max-tokens", str(max_live_tokens(steps))],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == [w for s in steps for w in ("done", str(s["step"]))]
    outputs = []
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        f = out / f"{s['step']}.f32"
        if not wanted:
            assert not f.exists()
            outputs.append(None)
            continue
        data = np.fromfile(f, dtype="<f4")
        outputs.append(torch.from_numpy(data.reshape(wanted, -1)))
    return outputs


@pytest.mark.parametrize("name,dtype", [("tiny_b", "float32"), ("tiny_dense", "bfloat16"), ("tiny_b", "bfloat16")])
def test_trace_run_program(model_dirs, tmp_path, name, dtype):
    """The program itself, as a user runs it: steps on stdin, ``done`` lines, .f32 files, exit 0.
    Its logits are those of the in-process replay bit for bit (it drives the same engine), and they
    match the plain implementation (with a router, in bfloat16, through the in-process run's picks)."""
    d = model_dirs(name, dtype)
    cfg = ALL[name]
    reqs = {k: random_prompt(cfg["vocab_size"], n, 40 + i) for i, (k, n) in
            enumerate({"a": 70, "b": 133, "c": 45, "d": 97, "e": 66}.items())}
    steps = mixed_trace(reqs, seed=1)
    outputs = run_program(d, dtype, steps, tmp_path / "out")
    assert outputs[0].shape[1] == cfg["vocab_size"]
    inproc, routes = run_in_process(d, dtype, steps, max_live_tokens(steps))
    for a, b in zip(outputs, inproc):
        assert (a is None and b is None) or torch.equal(a, b)
    check_against_plain(d, dtype, reqs, steps, outputs, routes)
    # entries may want nothing, and a step may want nothing at all
    quiet = [dict(s, entries=[dict(e, want=[] if i % 2 else e["want"]) for e in s["entries"]])
             for i, s in enumerate(steps)]
    outputs2 = run_program(d, dtype, quiet, tmp_path / "out2")
    for i, (a, b) in enumerate(zip(outputs, outputs2)):
        assert (b is None) if i % 2 else torch.equal(a, b)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_conv_only", "tiny_attn_only"])
def test_models_without_pages_or_without_state(model_dirs, name, dtype):
    """Only convolutions (no paged cache group at all, 5 taps) and only attention (one head of 24, widths 104
    and 20 that the vector paths do not take): the mixed trace against the plain implementation."""
    d = model_dirs(name, dtype)
    reqs = requests_for(ALL[name], seed=30)
    steps = mixed_trace(reqs, seed=5)
    outputs, routes = run_in_process(d, dtype, steps, max_live_tokens(steps))
    check_against_plain(d, dtype, reqs, steps, outputs, routes)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_cut_with_the_one_launch_router_front_end(model_dirs, dtype, monkeypatch):
    """The switch that lets a routed feed-forward take the norm before it, the router and the sort into one
    launch (off by default) gives the same logits as the three launches, on the mixed trace."""
    from snowllm_b200.ops import kernels
    d = model_dirs("tiny_b", dtype)
    reqs = requests_for(ALL["tiny_b"], seed=50)
    steps = mixed_trace(reqs, seed=7)
    apart, _ = run_in_process(d, dtype, steps, max_live_tokens(steps))
    monkeypatch.setattr(kernels, "FUSE_ROUTER", True)
    launches = kernels.launch_count()
    together, routes = run_in_process(d, dtype, steps, max_live_tokens(steps))
    monkeypatch.setattr(kernels, "FUSE_ROUTER", False)
    for a, b in zip(apart, together):
        assert (a is None and b is None) or torch.equal(a, b)
    check_against_plain(d, dtype, reqs, steps, together, routes)
