"""Decode and prefill throughput of the engine at the layer sizes of the LFM2.5 models, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--config 8b-a1b|dense-1.2b|dense-2.6b]
                    [--batch B] [--context C] [--dtype bfloat16|float32] [--impl ours|reference]

Prints ONE JSON line.  Without flags: LFM2.5-8B-A1B sizes, 8 requests at context 8,192.

``value``: decoded tokens per second of K decode steps (a step = one token for each of ``batch`` requests
at the given context), timed on the device with CUDA events after W warm-up steps.  ``e2e``: the same
through the Python entry point (Engine.add / Engine.step): host token ids in, sampled tokens out, every
step.  ``prefill``: one fresh 2,048-token prompt in one step.  ``roofline``: the bytes a decode step has to
read (every weight it uses once, counted from the experts the routers really picked, and the cache of the
live requests) over its time, against the measured copy bandwidth.  ``points``: decode at batch 1 and 64.
``kernels``: where the decode step's time goes, kernel by kernel: launches and microseconds per step from
the CUDA profiling interface (torch.profiler, outside the timed region; launch by launch, so that each
kernel's time is its own), and for the kernels that say what they move (`kernels.ledger`) the achieved
GB/s and TFLOP/s over the measured peaks.  ``prefill.kernels``: the same for the 2,048-token step.

The dense configurations add their own workloads (sizes from the same table as the tests' configs):
``dense-1.2b``: ``value`` is decode at 64 requests of context 32,768; ``e2e`` runs 64 concurrent requests
with prompts of 128 to 2,048 tokens through the Engine (prompt tokens and generated tokens per second of
the whole run).  ``dense-2.6b``: ``value`` is the prefill rate of one 32,768-token prompt in portions of
2,048 (``roofline`` then is TFLOP/s over the measured cuBLAS rate, attention included); ``mixed`` times a
2,048-token portion and 8 decoding requests in ONE step against the two steps run apart.

Weights are seeded random values drawn on the device; prompts are seeded uniform token ids.  For the
device-timed numbers the cache is filled with random keys, values and conv histories instead of being
prefilled (a decode step's cost does not depend on what the cache holds); the end-to-end numbers prefill
their prompts through the engine.  A decode step reads several GB, far more than the 126 MB L2, so no
separate L2 flush is needed between timed steps.
"""
from __future__ import annotations

import argparse
import collections
import json
import os
import pathlib
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))


def _lfm2(layers: int, attention: tuple, **more) -> dict:
    cfg = {"vocab_size": 65536, "hidden_size": 2048, "num_hidden_layers": layers,
           "layer_types": ["full_attention" if i in attention else "conv" for i in range(layers)],
           "num_attention_heads": 32, "num_key_value_heads": 8, "conv_L_cache": 3, "conv_bias": False,
           "rope_theta": 1000000.0, "norm_eps": 1e-5, "tie_word_embeddings": True,
           "max_position_embeddings": 128000}
    cfg.update(more)
    return cfg


# LFM2.5-8B-A1B sizes: 24 layers, attention at 2, 6, 10, 14, 18, 21, the rest short convolutions.
CONFIG_8B_A1B = _lfm2(24, (2, 6, 10, 14, 18, 21), architectures=["Lfm2MoeForCausalLM"], model_type="lfm2_moe",
                      num_dense_layers=2, intermediate_size=7168, num_experts=32, num_experts_per_tok=4,
                      moe_intermediate_size=1792, norm_topk_prob=True, use_expert_bias=True,
                      routed_scaling_factor=1.0)
# LFM2.5-1.2B dense sizes: 16 layers, attention at 2, 5, 8, 10, 12, 14; feed-forward width 8,192.
CONFIG_DENSE_1_2B = _lfm2(16, (2, 5, 8, 10, 12, 14), architectures=["Lfm2ForCausalLM"], model_type="lfm2",
                          intermediate_size=8192)
# LFM2-2.6B dense sizes: 30 layers, 22 short convolutions and 8 attention layers (spread evenly here: a
# step's cost does not depend on where they sit); feed-forward width 10,752.
CONFIG_DENSE_2_6B = _lfm2(30, (2, 6, 10, 14, 18, 22, 25, 28), architectures=["Lfm2ForCausalLM"], model_type="lfm2",
                          intermediate_size=10752)
CONFIGS = {
    "8b-a1b": dict(label="LFM2.5-8B-A1B sizes", json=CONFIG_8B_A1B, batch=8, context=8192),
    "dense-1.2b": dict(label="LFM2.5-1.2B dense sizes", json=CONFIG_DENSE_1_2B, batch=64, context=32768),
    "dense-2.6b": dict(label="LFM2-2.6B dense sizes", json=CONFIG_DENSE_2_6B, batch=1, context=32768),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
PREFILL_TOKENS = 2048


def peaks() -> tuple[dict, str]:
    """Roofline denominators: the copy bandwidth, and the cuBLAS bf16 rate as a burst (a kernel alone) and
    sustained (a kernel inside a long step)."""
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            d = json.loads(f.read_text())
            burst = float(d["bf16_tflops"])
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": burst,
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", burst))}, "measured"
        except (ValueError, KeyError, TypeError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


def device_id() -> str:
    """What ``nvidia-smi -i`` takes for the device this process computes on: its UUID (the process's device 0
    is rarely the machine's GPU 0 on a shared host)."""
    try:
        import torch
        return "GPU-" + str(torch.cuda.get_device_properties(torch.cuda.current_device()).uuid)
    except Exception:  # noqa: BLE001 - an older torch without the field
        first = os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0].strip()
        return first or "0"


class ClockSampler:
    """nvidia-smi in the background while the timed region runs (reads settings, changes none)."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: str = "0"):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        self.device = device

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", self.device, f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        self.proc.wait()
        self.file.flush()
        rows = [r.split(",") for r in pathlib.Path(self.file.name).read_text().splitlines() if r.count(",") >= 5]
        os.unlink(self.file.name)
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"], "gpu": self.device}
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = sorted({n for r in rows for n, v in zip(names, r[2:6]) if v.strip().lower().startswith("active")})
        sm = [float(r[0]) for r in rows if r[0].strip().replace(".", "").isdigit()]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": float(rows[0][1]),
                "reasons": reasons, "samples": len(rows), "gpu": self.device}


def cache_bytes(cache, live) -> int:
    """Bytes of cache the live requests hold: keys and values up to their length, and their slots."""
    total = sum(rc.num_tokens for rc in live) * cache.bytes_per_token()
    for t in cache.state_tensors():
        total += len(live) * t[0].numel() * t.element_size()
    return total


def prefill_flops(cfg, tokens: int, start: int = 0) -> float:
    """Multiply-adds times two of ``tokens`` prompt tokens that follow ``start`` cached ones: every product,
    causal attention over all keys so far, the head for one row."""
    H, nh, nkv = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = cfg.get("head_dim", H // nh)
    dense_layers = cfg.get("num_dense_layers", cfg["num_hidden_layers"])
    pairs = sum(range(start + 1, start + tokens + 1))          # (query, key) pairs under the causal mask
    T = tokens
    fl = 0.0
    for i, kind in enumerate(cfg["layer_types"]):
        if kind == "conv":
            fl += 2 * T * H * (3 * H + H)
        else:
            fl += 2 * T * H * ((nh + 2 * nkv) * hd) + 2 * T * (nh * hd) * H
            fl += 2 * 2 * nh * hd * pairs
        if i < dense_layers:
            fl += 2 * T * 3 * H * cfg["intermediate_size"]
        else:
            fl += 2 * T * H * cfg["num_experts"]
            fl += 2 * T * cfg["num_experts_per_tok"] * 3 * H * cfg["moe_intermediate_size"]
    return fl + 2 * H * cfg["vocab_size"]


def fill_cache_random(cache, rc, tokens: int, gen) -> None:
    """Make ``rc`` hold ``tokens`` positions of random keys, values and conv history."""
    import torch
    assert cache.ensure(rc, tokens), "the bench pool is too small"
    cache.commit(rc, tokens)
    for pool in cache.paged_tensors():
        pages = torch.tensor([p for t in rc.tables.values() for p in t if p >= 0], device=pool.device)
        for lo in range(0, len(pages), 512):                   # in pieces: the float staging stays small
            part = pages[lo:lo + 512]
            shape = (len(part),) + tuple(pool.shape[1:])
            pool[part] = torch.randn(shape, device=pool.device, dtype=torch.float32, generator=gen).to(pool.dtype)
    for t in cache.state_tensors():
        t[rc.slot] = (0.1 * torch.randn(t[rc.slot].shape, device=t.device, dtype=torch.float32,
                                        generator=gen)).to(t.dtype)


# --- where a step's time goes ---------------------------------------------------------------

def _kernel_events(prof):
    import torch
    out = []
    for e in prof.events():
        if e.device_type != torch.autograd.DeviceType.CUDA:
            continue
        name = e.name
        if name.startswith(("Memcpy", "Memset")) or "memcpy" in name.lower() or "memset" in name.lower():
            continue
        out.append(e)
    out.sort(key=lambda e: e.time_range.start)
    return out


def _short(name: str) -> str:
    name = name.split("(")[0].replace("void ", "").replace("snk::", "").replace("(anonymous namespace)::", "")
    name = name.replace("__nv_bfloat16", "bf16")
    return name if len(name) <= 64 else name[:61] + "..."


def kernel_report(step, eager_step, steps: int, pk: dict, top: int = 10) -> list:
    """[{name, launches, us, share, gbs, tflops, frac}] per step, largest first.

    Times: ``steps`` calls of ``step`` under the CUDA profiling interface, launch by launch and without
    programmatic dependent launch: a kernel that is launched early spends its wait for the kernel before it
    inside its own measured time, which would blow up the small kernels' shares.  (The step as a whole is
    timed elsewhere, with graphs and dependent launches; the kernels' sum here is a little above it.)
    Work: one call of ``eager_step`` (the same step launch by launch) with the kernels' ledger on; its
    launches and the profiler's kernels of that call are laid side by side in launch order, which gives
    every kernel name the bytes and flops of its launches.  ``frac`` is the larger of GB/s over the copy
    bandwidth and TFLOP/s over the sustained cuBLAS rate."""
    import torch
    from torch.profiler import ProfilerActivity, profile

    from snowllm_b200.ops import kernels
    kernels.ledger = []
    try:
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            eager_step()
            torch.cuda.synchronize()
    finally:
        ledger, kernels.ledger = kernels.ledger, None
    events = _kernel_events(prof)
    work: dict = collections.defaultdict(lambda: [0, 0.0, 0.0, True])      # name -> launches, bytes, flops, all known
    if len(events) == sum(n for _, n, _, _ in ledger):
        i = 0
        for _, n, nbytes, flops in ledger:
            for j in range(n):
                w = work[_short(events[i].name)]
                w[0] += 1
                if j == 0:
                    if nbytes is None:
                        w[3] = False
                    else:
                        w[1] += nbytes
                        w[2] += flops
                i += 1
    kernels.set_pdl(False)
    try:
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(steps):
                step()
            torch.cuda.synchronize()
    finally:
        kernels.set_pdl(os.environ.get("SNOWLLM_B200_PDL", "1") != "0")
    agg: dict = collections.defaultdict(lambda: [0, 0.0])
    for e in _kernel_events(prof):
        a = agg[_short(e.name)]
        a[0] += 1
        a[1] += e.device_time if hasattr(e, "device_time") else e.cuda_time
    total = sum(v[1] for v in agg.values()) or 1.0
    rows = []
    for name, (count, us) in sorted(agg.items(), key=lambda kv: -kv[1][1])[:top]:
        row = {"name": name, "launches": round(count / steps, 1), "us": round(us / steps, 1),
               "share": round(us / total, 4)}
        w = work.get(name)
        if w and w[3] and w[0] == round(count / steps) and us > 0:
            gbs = w[1] / (us / steps) * 1e-3
            tfl = w[2] / (us / steps) * 1e-6
            row.update(gbs=round(gbs, 1), tflops=round(tfl, 1),
                       frac=round(max(gbs / pk["hbm_gbs"], tfl / pk["bf16_tflops_sustained"]), 3))
        rows.append(row)
    return rows


# --- the measurements -------------------------------------------------------------------

def decode_run(model, batch: int, context: int, steps: int, warmup: int, page_size: int, seed: int = 0,
               count_experts: bool = False, graphs: bool = True, report=None):
    """Device-timed decode: returns (ms per step, launches in the timed region, bytes read per step, experts
    touched, kernel report or None).  ``report``: the peaks, to ask for the per-kernel report."""
    import torch

    from snowllm_b200.cache import CacheManager
    from snowllm_b200.engine import ModelRunner, StepEntry
    from snowllm_b200.ops import kernels
    total = context + steps + warmup + 16
    pages = batch * (-(-total // page_size))
    cache = CacheManager(model.cache_specs(), page_size, pages, batch, model.dtype, "cuda")
    runner = ModelRunner(model, cache, "cuda", use_graphs=graphs)
    gen = torch.Generator(device="cuda").manual_seed(seed)
    live = [cache.admit() for _ in range(batch)]
    for rc in live:
        fill_cache_random(cache, rc, context, gen)
    V = model.vocab_size
    ids = torch.randint(0, V, (steps + warmup + 16, batch), generator=torch.Generator().manual_seed(seed)).tolist()
    turn = [0]

    def one():
        i = turn[0]
        turn[0] += 1
        for rc in live:
            assert cache.ensure(rc, rc.num_tokens + 1)
        logits = runner.step([StepEntry(rc, [ids[i][b]], [0]) for b, rc in enumerate(live)])
        return kernels.argmax(logits)

    for i in range(warmup):
        one()
    touched = None
    if count_experts:
        runner.taps = []
        one()
        picks = [t for name, t in runner.taps if name == "moe_route"]
        moe_entries = [i for i, e in enumerate(model.run) if hasattr(model.blocks[e.layer].ffn, "route")]
        touched = {i: int(p.unique().numel()) for i, p in zip(moe_entries, picks)}
        runner.taps = None
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = kernels.launch_count()
    start.record()
    for i in range(steps):
        one()
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    nbytes = model.weight_bytes_per_step(touched) + cache_bytes(cache, live)
    # a replayed graph launches what its capture launched: count one step's launches and scale
    launches = kernels.launch_count() - launches0
    replayed = runner.graph_replays > 0

    def eager():
        runner.use_graphs = False
        try:
            return one()
        finally:
            runner.use_graphs = graphs
    if replayed:
        l0 = kernels.launch_count()
        eager()
        launches = (kernels.launch_count() - l0) * steps
    rows = kernel_report(eager, eager, 3, report) if report else None
    for rc in live:
        cache.free(rc)
    del cache, runner
    torch.cuda.empty_cache()
    return ms, launches, nbytes, touched, rows


def prefill_run(model, tokens: int, page_size: int, chunk: int | None = None, repeats: int = 3, report=None):
    """One fresh prompt of ``tokens`` in portions of ``chunk`` (None: whole), logits of its last row only:
    (median ms of the whole prompt, kernel report of its last portion or None)."""
    import torch

    from snowllm_b200.cache import CacheManager
    from snowllm_b200.engine import ModelRunner, StepEntry
    chunk = chunk or tokens
    cache = CacheManager(model.cache_specs(), page_size, -(-tokens // page_size) + 1, 1, model.dtype, "cuda")
    runner = ModelRunner(model, cache, "cuda")
    ids = torch.randint(0, model.vocab_size, (tokens,), generator=torch.Generator().manual_seed(1)).tolist()
    cuts = [(lo, min(lo + chunk, tokens)) for lo in range(0, tokens, chunk)]
    times = []
    rc = None

    def whole():
        nonlocal rc
        rc = cache.admit()
        assert cache.ensure(rc, tokens)
        for lo, hi in cuts:
            runner.step([StepEntry(rc, ids[lo:hi], [hi - lo - 1] if hi == tokens else [])])

    for i in range(repeats + 1):
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        whole()
        end.record()
        torch.cuda.synchronize()
        if i:
            times.append(start.elapsed_time(end))
        cache.free(rc)
    rows = None
    if report:
        lo, hi = cuts[-1]

        def last():                        # the last portion again, over the cache that the portions before left
            rc.num_tokens = lo
            runner.step([StepEntry(rc, ids[lo:hi], [hi - lo - 1])])
        whole()
        rows = kernel_report(last, last, 2, report)
        cache.free(rc)
    del cache, runner
    torch.cuda.empty_cache()
    return statistics.median(times), rows


def mixed_run(model, page_size: int, portion: int = 2048, prompt_at: int = 16384, decoders: int = 8,
              context: int = 8192, repeats: int = 5):
    """A prompt portion and decoding requests in ONE step against the two steps run apart: median ms of
    (portion alone, decode alone, both in one step).  Launch by launch (a step with a portion is never a
    captured one)."""
    import torch

    from snowllm_b200.cache import CacheManager
    from snowllm_b200.engine import ModelRunner, StepEntry
    pages = -(-(prompt_at + portion) // page_size) + decoders * (-(-(context + 4) // page_size)) + 4
    cache = CacheManager(model.cache_specs(), page_size, pages, decoders + 1, model.dtype, "cuda")
    runner = ModelRunner(model, cache, "cuda")
    gen = torch.Generator(device="cuda").manual_seed(3)
    prompt = cache.admit()
    fill_cache_random(cache, prompt, prompt_at, gen)
    assert cache.ensure(prompt, prompt_at + portion)
    live = [cache.admit() for _ in range(decoders)]
    for rc in live:
        fill_cache_random(cache, rc, context, gen)
        assert cache.ensure(rc, context + 1)
    ids = torch.randint(0, model.vocab_size, (portion + decoders,), generator=torch.Generator().manual_seed(4)).tolist()

    def entries(with_portion: bool, with_decode: bool):
        prompt.num_tokens = prompt_at                  # every repeat runs the same positions again
        for rc in live:
            rc.num_tokens = context
        es = [StepEntry(prompt, ids[:portion], [])] if with_portion else []
        if with_decode:
            es += [StepEntry(rc, [ids[portion + b]], [0]) for b, rc in enumerate(live)]
        return es

    out = []
    for a, b in ((True, False), (False, True), (True, True)):
        times = []
        for i in range(repeats + 2):
            es = entries(a, b)
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            runner.step(es)
            end.record()
            torch.cuda.synchronize()
            if i >= 2:
                times.append(start.elapsed_time(end))
        out.append(statistics.median(times))
    for rc in live + [prompt]:
        cache.free(rc)
    del cache, runner
    torch.cuda.empty_cache()
    return tuple(out)


def e2e_run(model, batch: int, context: int, steps: int, warmup: int, page_size: int):
    """Through the Python entry point: prompts as host token ids, sampled tokens read back."""
    import torch

    from snowllm_b200.engine import Engine, SamplingParams
    gen = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, model.vocab_size, (context,), generator=gen).tolist() for _ in range(batch)]
    # requests reach their first token one after another (the prompts are prefilled in portions, in
    # turn); none may finish before the timed steps are over, or the batch would shrink under them
    stagger = batch * -(-context // PREFILL_TOKENS)
    new = steps + warmup + stagger + 8
    engine = Engine(model, max_num_seqs=batch, max_model_len=batch * (context + new + page_size),
                    prefill_chunk=PREFILL_TOKENS, page_size=page_size)
    # one request of the same length first, untimed (the reference's own runs keep four requests after one
    # warm-up): the first use of every launch shape sets up tensor maps, kernel attributes and the allocator
    engine.add(prompts[0], SamplingParams(temperature=0, max_new_tokens=2))
    engine.run()
    torch.cuda.synchronize()
    reqs = [engine.add(p, SamplingParams(temperature=0, max_new_tokens=new)) for p in prompts]
    t0 = time.perf_counter()
    while any(not r.out for r in reqs):
        engine.step()
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    h2d0 = engine.runner.staging.bytes_uploaded
    t0 = time.perf_counter()
    for _ in range(steps):
        kind = engine.step()
        assert kind == "decode", kind
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    h2d = (engine.runner.staging.bytes_uploaded - h2d0) / steps
    for r in reqs:
        engine.abort(r)
    del engine
    torch.cuda.empty_cache()
    return batch * steps / dt, h2d, batch * 4, batch * context / prefill_s


def serve_run(model, requests: int, shortest: int, longest: int, new_tokens: int, page_size: int):
    """``requests`` concurrent requests with prompts of ``shortest``..``longest`` tokens through Engine.add /
    Engine.run, all added at once: (prompt tokens per second and generated tokens per second over the whole
    run's wall time, h2d bytes per step, d2h bytes per step, steps by kind)."""
    import torch

    from snowllm_b200.engine import Engine, SamplingParams
    gen = torch.Generator().manual_seed(5)
    lengths = torch.randint(shortest, longest + 1, (requests,), generator=gen).tolist()
    prompts = [torch.randint(0, model.vocab_size, (n,), generator=gen).tolist() for n in lengths]
    engine = Engine(model, max_num_seqs=requests, max_model_len=requests * (longest + new_tokens + page_size),
                    prefill_chunk=4 * PREFILL_TOKENS, page_size=page_size)
    # once untimed with short replies (first use compiles nothing, but captures graphs and warms the allocator)
    for p in prompts[:4]:
        engine.add(p, SamplingParams(temperature=0, max_new_tokens=4))
    engine.run()
    torch.cuda.synchronize()
    h2d0 = engine.runner.staging.bytes_uploaded
    reqs = [engine.add(p, SamplingParams(temperature=0, max_new_tokens=new_tokens)) for p in prompts]
    kinds: dict = collections.Counter()
    t0 = time.perf_counter()
    while engine.scheduler.has_work():
        kinds[engine.step()] += 1
    engine.run()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    steps = max(1, sum(kinds.values()))
    generated = sum(len(r.out) for r in reqs)
    assert all(r.finish_reason == "length" for r in reqs), [r.finish_reason for r in reqs]
    h2d = (engine.runner.staging.bytes_uploaded - h2d0) / steps
    del engine
    torch.cuda.empty_cache()
    return sum(lengths) / dt, generated / dt, h2d, generated * 4 / steps, dict(kinds)


def reference_arm() -> dict:
    """The unmodified reference from baseline/_ref through its own API, or why it cannot run here."""
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "snowllm").is_dir():
        return {"impl": "reference", "unavailable": "baseline/_ref holds no SnowLLM install (its dependency "
                "snowllm-kernels, a closed HIP library for AMD RDNA3, is not in the wheelhouse)"}
    sys.path.insert(0, str(ref))
    try:
        import snowllm.engine  # noqa: F401  (loads the kernel library at import)
    except BaseException as e:  # noqa: BLE001 - whatever stops the import is the answer
        why = str(e).strip().splitlines()[0] if str(e).strip() else type(e).__name__
        return {"impl": "reference", "unavailable": f"SnowLLM cannot be imported: {why[:200]}"}
    finally:
        sys.path.remove(str(ref))
    return {"impl": "reference", "unavailable": "SnowLLM imported, but it has no CUDA path: its kernels are a HIP "
            "library for AMD RDNA3 and its LFM loader accepts GGUF or real checkpoints only"}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--config", default="8b-a1b", choices=tuple(CONFIGS))
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--context", type=int, default=None)
    ap.add_argument("--layers", type=int, default=None, help="run the first N layers only (memory or time)")
    ap.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
    ap.add_argument("--page-size", type=int, default=None)
    ap.add_argument("--enforce-eager", action="store_true", help="no CUDA graphs for the decode steps")
    ap.add_argument("--skip", default="", help="comma list of: e2e, prefill, points, kernels, mixed")
    a = ap.parse_args()
    if a.impl == "reference":
        print(json.dumps(reference_arm()))
        return 0
    if a.gpus != 1:
        print("bench.py measures one GPU: this engine does not use more than one (got --gpus %d)" % a.gpus)
        return 2
    warmup = max(a.warmup, 3)
    import torch

    from snowllm_b200.config.engine import DEFAULT_PAGE_SIZE
    from snowllm_b200.loader import load_random
    page = a.page_size or DEFAULT_PAGE_SIZE
    chosen = CONFIGS[a.config]
    cfg = dict(chosen["json"])
    full_layers = cfg["num_hidden_layers"]
    layers = a.layers or full_layers
    if layers < full_layers:
        cfg["num_hidden_layers"] = layers
        cfg["layer_types"] = cfg["layer_types"][:layers]
        if "num_dense_layers" in cfg:
            cfg["num_dense_layers"] = min(cfg["num_dense_layers"], layers)
    batch = a.batch or chosen["batch"]
    context = a.context or chosen["context"]
    skip = set(filter(None, a.skip.split(",")))
    pk, pk_source = peaks()
    report = None if "kernels" in skip else pk
    model = load_random(cfg, seed=0, dtype=a.dtype, device="cuda")
    torch.cuda.synchronize()
    graphs = not a.enforce_eager
    moe = "num_experts" in cfg
    dtype_name = "bf16" if a.dtype == "bfloat16" else "fp32"
    tensor_peak, tensor_of = pk["bf16_tflops"], pk_source
    if a.dtype == "float32":
        # the true 32-bit path multiplies on the CUDA cores: 148 SMs x 128 lanes x 2 flops x 1.965 GHz
        tensor_peak, tensor_of = 148 * 128 * 2 * 1.965e9 / 1e12, "nominal fp32 FFMA rate"

    sampler = ClockSampler(device_id())
    sampler.start()
    ms, launches, nbytes, touched, rows = decode_run(model, batch, context, a.steps, warmup, page,
                                                     count_experts=moe, graphs=graphs, report=report)
    clocks = sampler.stop()
    value = batch / (ms / 1e3)
    achieved = nbytes / (ms / 1e3) / 1e9

    out = {
        "metric": "decode tok/s (%s, batch %d, context %d)" % (chosen["label"], batch, context),
        "value": round(value, 2), "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": dtype_name,
        "data": "synthetic: seeded random weights and uniform random token ids; cache filled with random values",
        "impl": "ours",
        "config": {"model": chosen["label"], "layers": full_layers, "layers_run": layers,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["hidden_size"] // cfg["num_attention_heads"], "conv_L": cfg["conv_L_cache"],
                   "dense_layers": cfg.get("num_dense_layers", layers), "dense_inter": cfg["intermediate_size"],
                   "experts": cfg.get("num_experts", 0), "top_k": cfg.get("num_experts_per_tok", 0),
                   "moe_inter": cfg.get("moe_intermediate_size", 0), "vocab": cfg["vocab_size"],
                   "global_batch": batch, "seq_len": context, "page_size": page, "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (%.1f GB read per step)" % (nbytes / 1e9),
                   "cuda_graphs": graphs},
        "clocks": clocks,
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk_source,
                     "bytes_per_step": nbytes,
                     "experts_touched_mean": round(statistics.mean(touched.values()), 2) if touched else None},
    }
    if rows:
        out["kernels"] = rows
    if "prefill" not in skip:
        pms, prows = prefill_run(model, PREFILL_TOKENS, page, report=report)
        fl = prefill_flops(cfg, PREFILL_TOKENS)
        out["prefill"] = {"value": round(PREFILL_TOKENS / (pms / 1e3), 1), "tokens": PREFILL_TOKENS,
                          "ms": round(pms, 3), "frac": round(fl / (pms / 1e3) / 1e12 / tensor_peak, 4),
                          "tflops": round(fl / (pms / 1e3) / 1e12, 2), "of": tensor_of}
        if prows:
            out["prefill"]["kernels"] = prows[:8]
    if "points" not in skip:
        points = {}
        for b in (1, 64):
            if b == batch:
                continue
            n = max(8, a.steps // 4)
            pms, _, pb, _, _ = decode_run(model, b, context, n, 3, page, count_experts=moe, graphs=graphs)
            points[f"decode_b{b}"] = round(b / (pms / 1e3), 2)
            points[f"decode_b{b}_ms"] = round(pms, 4)
            points[f"decode_b{b}_hbm_frac"] = round(pb / (pms / 1e3) / 1e9 / pk["hbm_gbs"], 4)
        points["decode_b%d" % batch] = round(value, 2)
        out["points"] = points

    if a.config == "dense-2.6b":
        # the long prompt in portions is this configuration's headline; the decode step stays in `points`
        long_ms, _ = prefill_run(model, context, page, chunk=PREFILL_TOKENS, repeats=2)
        fl = sum(prefill_flops(cfg, min(PREFILL_TOKENS, context - lo), lo) for lo in range(0, context, PREFILL_TOKENS))
        tfl = fl / (long_ms / 1e3) / 1e12
        out.setdefault("points", {}).update({"decode_b%d" % batch: round(value, 2),
                                             "decode_b%d_ms" % batch: round(ms, 4),
                                             "decode_b%d_hbm_frac" % batch: out["roofline"]["frac"]})
        out.update(metric="prefill tok/s (%s, one prompt of %d tokens in portions of %d)"
                   % (chosen["label"], context, PREFILL_TOKENS),
                   value=round(context / (long_ms / 1e3), 1), ms_per_step=round(long_ms / -(-context // PREFILL_TOKENS), 3),
                   steps=-(-context // PREFILL_TOKENS))
        out["roofline"] = {"bound": "tensor", "achieved": round(tfl, 1), "peak": pk["bf16_tflops_sustained"],
                           "unit": "TFLOP/s", "frac": round(tfl / pk["bf16_tflops_sustained"], 4), "of": pk_source,
                           "flops": fl, "ms": round(long_ms, 2)}
        if "mixed" not in skip:
            p_ms, d_ms, m_ms = mixed_run(model, page)
            out["mixed"] = {"portion_tokens": PREFILL_TOKENS, "portion_at": 16384, "decoders": 8,
                            "decode_context": 8192, "portion_ms": round(p_ms, 3), "decode_ms": round(d_ms, 3),
                            "mixed_ms": round(m_ms, 3), "apart_ms": round(p_ms + d_ms, 3),
                            "gain": round((p_ms + d_ms) / m_ms, 4)}
    if "e2e" not in skip:
        if a.config == "dense-1.2b":
            tin, tout, h2d, d2h, kinds = serve_run(model, 64, 128, 2048, 128, page)
            out["e2e"] = {"value": round(tout, 2), "unit": "generated tokens/s over the run", "prompt_tok_s": round(tin, 1),
                          "requests": 64, "prompt_tokens": "uniform 128..2048", "new_tokens": 128,
                          "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "steps": kinds}
        else:
            e_batch, e_ctx = (batch, context) if a.config == "8b-a1b" else (1, context)
            e, h2d, d2h, prefill_tok_s = e2e_run(model, e_batch, e_ctx, min(a.steps, 32), warmup, page)
            out["e2e"] = {"value": round(e, 2), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
                          "d2h_bytes_per_step": int(d2h), "prefill_tok_s": round(prefill_tok_s, 1),
                          "batch": e_batch, "context": e_ctx}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
