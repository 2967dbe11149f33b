"""Decode and prefill throughput of the engine on LFM2.5-8B-A1B sizes with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 8192] [--impl ours|reference]

Prints ONE JSON line.  ``value``: decoded tokens per second of K decode steps (a step = one token
for each of ``batch`` requests at the given context), timed on the device with CUDA events after W
warm-up steps.  ``e2e``: the same through the Python entry point (Engine.add / Engine.step): host
token ids in, sampled tokens out, every step.  ``prefill``: one fresh 2,048-token prompt in one
step.  ``roofline``: the bytes a decode step has to read (every weight it uses once, counted from
the experts the routers really picked, and the cache of the live requests) over its time, against
the measured copy bandwidth.  ``points``: decode at batch 1 and 64.

Weights are seeded random values drawn on the device; prompts are seeded uniform token ids.  For
the device-timed numbers the cache is filled with random keys, values and conv histories instead
of being prefilled (a decode step's cost does not depend on what the cache holds); the end-to-end
number prefills its prompts through the engine.  A decode step reads several GB, far more than
the 126 MB L2, so no separate L2 flush is needed between timed steps.
"""
from __future__ import annotations

import argparse
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

# LFM2.5-8B-A1B sizes: 24 layers, attention at 2, 6, 10, 14, 18, 21, the rest short convolutions.
ATTENTION_LAYERS = (2, 6, 10, 14, 18, 21)
CONFIG_8B_A1B = {
    "architectures": ["Lfm2MoeForCausalLM"], "model_type": "lfm2_moe",
    "vocab_size": 65536, "hidden_size": 2048, "num_hidden_layers": 24,
    "layer_types": ["full_attention" if i in ATTENTION_LAYERS else "conv" for i in range(24)],
    "num_attention_heads": 32, "num_key_value_heads": 8, "conv_L_cache": 3, "conv_bias": False,
    "num_dense_layers": 2, "intermediate_size": 7168,
    "num_experts": 32, "num_experts_per_tok": 4, "moe_intermediate_size": 1792,
    "norm_topk_prob": True, "use_expert_bias": True, "routed_scaling_factor": 1.0,
    "rope_theta": 1000000.0, "norm_eps": 1e-5, "tie_word_embeddings": True,
    "max_position_embeddings": 128000,
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
PREFILL_TOKENS = 2048


def peaks() -> tuple[dict, str]:
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            d = json.loads(f.read_text())
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"])}, "measured"
        except (ValueError, KeyError, TypeError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi in the background while the timed region runs (reads settings, changes none)."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
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
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = sorted({n for r in rows for n, v in zip(names, r[2:6]) if v.strip().lower().startswith("active")})
        sm = [float(r[0]) for r in rows if r[0].strip().replace(".", "").isdigit()]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": float(rows[0][1]),
                "reasons": reasons, "samples": len(rows)}


def weight_bytes(model, experts_touched: dict | None) -> int:
    """Bytes of weights one decode step reads: every tensor once, of the routed experts only those
    that were picked (``experts_touched``: {block index -> count}; None: all)."""
    total = 0
    for i, b in enumerate(model.blocks):
        for part in b.parts():
            for name, t in vars(part).items():
                if not hasattr(t, "element_size") or not hasattr(t, "numel"):
                    continue
                if name == "wq":            # a view of wqkv
                    continue
                n = t.numel() * t.element_size()
                if name in ("w13", "w2") and t.dim() == 3:
                    used = t.shape[0] if experts_touched is None else experts_touched.get(i, t.shape[0])
                    n = n // t.shape[0] * used
                total += n
    head = model.head.weight
    total += head.numel() * head.element_size()                 # tied: the embedding table, read as the head
    total += model.final_norm.weight.numel() * model.final_norm.weight.element_size()
    return total


def cache_bytes(cache, live) -> int:
    """Bytes of cache the live requests hold: keys and values up to their length, and their slots."""
    total = 0
    for idx, pool in cache.pools.items():
        per_token = 2 * pool.shape[2] * pool.shape[4] * pool.element_size()
        total += sum(rc.num_tokens for rc in live) * per_token
    for tensors in cache.states.values():
        for t in tensors:
            total += len(live) * t[0].numel() * t.element_size()
    return total


def prefill_flops(cfg, T: int) -> float:
    """Multiply-adds times two of one fresh T-token prompt: every product, causal attention, the
    head for one row."""
    H, nh, nkv = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = H // nh
    fl = 0.0
    for i, kind in enumerate(cfg["layer_types"]):
        if kind == "conv":
            fl += 2 * T * H * (3 * H + H)
        else:
            fl += 2 * T * H * ((nh + 2 * nkv) * hd) + 2 * T * (nh * hd) * H
            fl += 2 * 2 * nh * hd * T * (T + 1) / 2
        if i < cfg["num_dense_layers"]:
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
    for pool in cache.pools.values():
        pages = torch.tensor([p for t in rc.tables.values() for p in t if p >= 0], device=pool.device)
        shape = (len(pages),) + tuple(pool.shape[1:])
        pool[pages] = torch.randn(shape, device=pool.device, dtype=torch.float32, generator=gen).to(pool.dtype)
    for tensors in cache.states.values():
        for t in tensors:
            t[rc.slot] = (0.1 * torch.randn(t[rc.slot].shape, device=t.device, dtype=torch.float32,
                                            generator=gen)).to(t.dtype)


def decode_run(model, batch: int, context: int, steps: int, warmup: int, page_size: int, seed: int = 0,
               count_experts: bool = False, graphs: bool = True):
    """Device-timed decode: returns (ms per step, launches in the timed region, bytes read per step)."""
    import torch

    from snowllm_b200.cache import CacheManager
    from snowllm_b200.engine import ModelRunner, StepEntry
    from snowllm_b200.ops import kernels
    total = context + steps + warmup + 3
    pages = batch * (-(-total // page_size))
    cache = CacheManager(model.cache_specs(), page_size, pages, batch, model.dtype, "cuda")
    runner = ModelRunner(model, cache, "cuda", use_graphs=graphs)
    gen = torch.Generator(device="cuda").manual_seed(seed)
    live = [cache.admit() for _ in range(batch)]
    for rc in live:
        fill_cache_random(cache, rc, context, gen)
    V = model.vocab_size
    ids = torch.randint(0, V, (steps + warmup + 2, batch), generator=torch.Generator().manual_seed(seed)).tolist()

    def one(i):
        for rc in live:
            assert cache.ensure(rc, rc.num_tokens + 1)
        logits = runner.step([StepEntry(rc, [ids[i][b]], [0]) for b, rc in enumerate(live)])
        return kernels.argmax(logits)

    for i in range(warmup):
        one(i)
    touched = None
    if count_experts:
        runner.taps = []
        one(warmup)
        picks = [t for name, t in runner.taps if name == "moe_route"]
        moe_blocks = [i for i, b in enumerate(model.blocks) if hasattr(b.ffn, "route")]
        touched = {i: int(p.unique().numel()) for i, p in zip(moe_blocks, picks)}
        runner.taps = None
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = kernels.launch_count()
    start.record()
    for i in range(steps):
        one(warmup + 1 + i if count_experts else warmup + i)
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    nbytes = weight_bytes(model, touched) + cache_bytes(cache, live)
    # a replayed graph launches what its capture launched: count one step's launches and scale
    launches = kernels.launch_count() - launches0
    if runner.graph_replays:
        runner.use_graphs = False
        l0 = kernels.launch_count()
        one(steps + warmup + 1)
        launches = (kernels.launch_count() - l0) * steps
    for rc in live:
        cache.free(rc)
    del cache, runner
    torch.cuda.empty_cache()
    return ms, launches, nbytes, touched


def prefill_run(model, tokens: int, page_size: int, repeats: int = 3):
    import torch

    from snowllm_b200.cache import CacheManager
    from snowllm_b200.engine import ModelRunner, StepEntry
    cache = CacheManager(model.cache_specs(), page_size, -(-tokens // page_size) + 1, 1, model.dtype, "cuda")
    runner = ModelRunner(model, cache, "cuda")
    ids = torch.randint(0, model.vocab_size, (tokens,), generator=torch.Generator().manual_seed(1)).tolist()
    times = []
    for i in range(repeats + 1):
        rc = cache.admit()
        assert cache.ensure(rc, tokens)
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.step([StepEntry(rc, ids, [tokens - 1])])
        end.record()
        torch.cuda.synchronize()
        if i:
            times.append(start.elapsed_time(end))
        cache.free(rc)
    del cache, runner
    torch.cuda.empty_cache()
    return statistics.median(times)


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
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=24, help="run the first N layers only (memory or time)")
    ap.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
    ap.add_argument("--page-size", type=int, default=None)
    ap.add_argument("--enforce-eager", action="store_true", help="no CUDA graphs for the decode steps")
    ap.add_argument("--skip", default="", help="comma list of: e2e, prefill, points")
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
    from snowllm_b200.ops import kernels
    page = a.page_size or DEFAULT_PAGE_SIZE
    cfg = dict(CONFIG_8B_A1B)
    if a.layers < 24:
        cfg["num_hidden_layers"] = a.layers
        cfg["layer_types"] = cfg["layer_types"][:a.layers]
        cfg["num_dense_layers"] = min(2, a.layers)
    skip = set(filter(None, a.skip.split(",")))
    pk, pk_source = peaks()
    model = load_random(cfg, seed=0, dtype=a.dtype, device="cuda")
    torch.cuda.synchronize()

    sampler = ClockSampler()
    sampler.start()
    ms, launches, nbytes, touched = decode_run(model, a.batch, a.context, a.steps, warmup, page, count_experts=True,
                                                graphs=not a.enforce_eager)
    clocks = sampler.stop()
    value = a.batch / (ms / 1e3)
    achieved = nbytes / (ms / 1e3) / 1e9

    out = {
        "metric": "decode tok/s (LFM2.5-8B-A1B sizes, batch %d, context %d)" % (a.batch, a.context),
        "value": round(value, 2), "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if a.dtype == "bfloat16" else "fp32",
        "data": "synthetic: seeded random weights and uniform random token ids; cache filled with random values",
        "impl": "ours",
        "config": {"model": "LFM2.5-8B-A1B sizes", "layers": 24, "layers_run": a.layers, "hidden": 2048,
                   "heads": 32, "kv_heads": 8, "head_dim": 64, "conv_L": 3, "dense_layers": 2,
                   "dense_inter": 7168, "experts": 32, "top_k": 4, "moe_inter": 1792, "vocab": 65536,
                   "global_batch": a.batch, "seq_len": a.context, "page_size": page, "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (%.1f GB read per step)" % (nbytes / 1e9),
                   "cuda_graphs": not a.enforce_eager},
        "clocks": clocks,
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk_source,
                     "bytes_per_step": nbytes,
                     "experts_touched_mean": round(statistics.mean(touched.values()), 2) if touched else None},
    }
    if "prefill" not in skip:
        pms = prefill_run(model, PREFILL_TOKENS, page)
        fl = prefill_flops(cfg, PREFILL_TOKENS)
        out["prefill"] = {"value": round(PREFILL_TOKENS / (pms / 1e3), 1), "tokens": PREFILL_TOKENS,
                          "ms": round(pms, 3), "frac": round(fl / (pms / 1e3) / 1e12 / pk["bf16_tflops"], 4),
                          "tflops": round(fl / (pms / 1e3) / 1e12, 2), "of": pk_source}
    if "points" not in skip:
        points = {}
        for b in (1, 64):
            n = max(8, a.steps // 4)
            pms, _, pb, _ = decode_run(model, b, a.context, n, 3, page, graphs=not a.enforce_eager)
            points[f"decode_b{b}"] = round(b / (pms / 1e3), 2)
            points[f"decode_b{b}_ms"] = round(pms, 4)
        points["decode_b%d" % a.batch] = round(value, 2)
        out["points"] = points
    if "e2e" not in skip:
        e, h2d, d2h, prefill_tok_s = e2e_run(model, a.batch, a.context, min(a.steps, 32), warmup, page)
        out["e2e"] = {"value": round(e, 2), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
                      "d2h_bytes_per_step": int(d2h), "prefill_tok_s": round(prefill_tok_s, 1)}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
