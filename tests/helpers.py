"""Shared pieces of the tests: model folders with random weights, traces and comparisons."""
from __future__ import annotations

import random

import torch

import plain_lfm2 as plain
from tiny_configs import ALL

# Relative L2 error allowed between the engine's logits and the plain implementation's.
# float32: both sides sum in float32 in different orders: a few 1e-6 per product, about 1e-5 after a
# handful of layers; the bound holds for every single position.
# bfloat16: the engine is compared with the plain implementation's rounding variant
# (``plain.stores_rounded_to``), which rounds to bfloat16 exactly where the engine stores bfloat16.  Part by
# part the two agree almost bit for bit (``check_parts``).  Over a whole model they drift apart all the same:
# float sums in another order move a value by 1e-7, a value that sits on a rounding boundary then falls to
# the other side (one bfloat16 step), and attention hands a key's or value's flipped element on to every
# later position of the request.  That drift is a fraction of the rounding noise itself, and the noise is
# known: it is what the rounding variant differs from the float variant on the same request.  So the bounds
# are stated in units of it: the engine must lie closer to the rounding variant than the rounding variant
# lies to the float result (over a request; twice that for a single position), and inside the caps that the
# comparison with the float result alone used to have (SnowLLM's own acceptance bound for its bf16 kernels,
# rel-L2 < 0.025 for 3 layers, tests/test_lfm2_reference.py:66-161, scaled in quadrature with the layers;
# 0.1 for a single position).  A wrong page, slot, key, row or expert gives errors of order 1.
TOL = {"float32": 2e-5, "bfloat16": 0.1}
NOISE_SHARE_REQUEST, NOISE_SHARE_POSITION = 1.0, 2.0


def tol_request(dtype: str, num_layers: int) -> float:
    return 2e-5 if dtype == "float32" else 0.025 * (max(num_layers, 3) / 3) ** 0.5


# Bounds against an oracle WITHOUT a rounding variant (the toy architectures' written-out computations): the caps.
TOL_UNROUNDED = TOL
tol_request_unrounded = tol_request


def rel_all(got, want) -> float:
    """Relative L2 error over all rows together."""
    got, want = got.double(), want.double()
    return float((got - want).norm() / want.norm().clamp_min(1e-30))


def make_model_dir(folder, name, dtype="float32", flavour="scaled", seed=1):
    """Write config.json + model.safetensors for tiny config ``name``.  flavour "scaled": matrices
    with std 1/sqrt(fan_in) and norm weights 1 + N(0, 0.1), so that every layer matters;
    "baseline": N(0, 0.02) matrices, norm weights 1."""
    from snowllm_b200.loader import build_model, parse_dtype
    from snowllm_b200.weights import random_tensors, write_model_folder
    cfg = ALL[name]
    model = build_model(cfg, dtype)
    kw = dict(fan_in_scaled=True, norm_jitter=0.1) if flavour == "scaled" else {}
    tensors = random_tensors(model, seed, parse_dtype(dtype), **kw)
    write_model_folder(folder, model.config.to_json_dict(), tensors)
    return folder


def rel_rows(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Relative L2 error of each row."""
    got, want = got.double(), want.double()
    return (got - want).norm(dim=-1) / want.norm(dim=-1).clamp_min(1e-30)


def random_prompt(vocab: int, n: int, seed: int) -> list:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


# Router picks are compared on the router's OWN input (tapped beside the picks): the plain router runs on
# that very tensor, so the two differ only by the order of a float sum over the hidden size (products of
# bfloat16 numbers are exact in float).  A pick may differ only where the plain selection margin (gap
# between the k-th and the (k+1)-th score) is below that, and only a few picks in a hundred may.
ROUTE_MARGIN = {"float32": 1e-5, "bfloat16": 5e-4}
ROUTE_FORGIVEN = 0.02

def poison_free(rp):
    """Fill every free page and every free state slot with NaN."""
    free = [p for pool in rp.cache.groups.values() for p in pool._free]
    for pool in rp.cache.paged_tensors():
        pool[free] = float("nan")
    free_slots = list(rp.cache.slots._free) + [rp.cache.slots.dummy]
    for t in rp.cache.state_tensors():
        t[free_slots] = float("nan")


def run_in_process(model, dtype, steps, max_tokens, page_size=16, poison=False, stats=None, max_requests=4,
                   use_graphs=False, taps=True):
    """Replay ``steps`` on ``model`` (a model folder, or a model with its weights bound); returns (outputs
    per step, {request -> {layer -> (picks [T, k], the router's input [T, H])}}).  ``poison``: whatever is
    free is NaN before every step.  ``use_graphs``: decode steps as captured graphs (then without taps: a
    step that is tapped runs launch by launch)."""
    from snowllm_b200.engine.replay import Replay
    rp = Replay(model, dtype, max_tokens, max_requests=max_requests, page_size=page_size, use_graphs=use_graphs)
    moe_layers = [i for i, b in enumerate(rp.model.blocks) if hasattr(b.ffn, "route")]
    outputs, routes, route_inputs, parts = [], {}, {}, {}
    used: set = set()
    for s in steps:
        if poison:
            poison_free(rp)
        rp.runner.taps = [] if taps else None
        outputs.append(rp.step(s["entries"], s["end"]))
        if stats is not None:
            held = {p for rc in rp.live.values() for t in rc.tables.values() for p in t if p >= 0}
            stats["reused"] = stats.get("reused", False) or bool(held & used)
            used |= held
        if not taps:
            continue
        picks = [t.cpu() for name, t in rp.runner.taps if name == "moe_route"]
        inputs = [t.float().cpu() for name, t in rp.runner.taps if name == "moe_route_input"]
        assert len(picks) == len(moe_layers) == len(inputs)
        by_name = {name: [(t.dense() if hasattr(t, "dense") else t).float().cpu()
                          for n, t in rp.runner.taps if n == name] for name in PART_TAPS} if stats is not None else {}
        row = 0
        for e in s["entries"]:
            n = len(e["tokens"])
            for layer, ids, x in zip(moe_layers, picks, inputs):
                routes.setdefault(e["id"], {}).setdefault(layer, []).append(ids[row:row + n])
                route_inputs.setdefault(e["id"], {}).setdefault(layer, []).append(x[row:row + n])
            for name, per_layer in by_name.items():
                for layer, t in enumerate(per_layer):
                    parts.setdefault(e["id"], {}).setdefault(layer, {}).setdefault(name, []).append(t[row:row + n])
            row += n
    assert all(p.free_count == p.total for p in rp.cache.groups.values()), "pages were lost"
    assert rp.cache.slots.free_count == rp.cache.max_seqs
    if stats is not None:
        stats["graph_replays"] = rp.runner.graph_replays
        stats["parts"] = {k: {layer: {name: torch.cat(v) for name, v in d.items()} for layer, d in layers.items()}
                          for k, layers in parts.items()}
    routes = {k: {layer: (torch.cat(v), torch.cat(route_inputs[k][layer])) for layer, v in d.items()}
              for k, d in routes.items()}
    return outputs, routes


PART_TAPS = ("mixer_in", "mixer_out", "ffn_in", "ffn_out")
# A part's output against the plain part run on the engine's OWN input to that part (both tapped, in position
# order over all the steps of a request).  float32: the float bound.  bfloat16: the distance is measured in
# units of the part's own rounding noise (what the plain part's rounding variant differs from its float
# result on that input); a rounding too many or too few inside a part moves its output by about
# noise / sqrt(stores in the part), 0.5 to 0.7 of the noise for the two to four stores a part has.
# Measured on the tiny and the full-size models: 0.00 in the median (the same bits), up to 0.13 for feed-forwards
# and short convolutions, up to 0.30 for attention (a flipped element of a key or value reaches every later row).
PART_NOISE_SHARE = {"attention": 0.45, "other": 0.25}


def check_parts(model, dtype, parts, routes) -> None:
    """Every mixer and every feed-forward of every layer alone, on what the engine itself fed it.  The plain
    part sees the whole sequence at once, the engine saw it in the steps' cuts, through its cache."""
    cfg, tensors = model if isinstance(model, tuple) else plain.read_model_dir(model)
    dev = tensors["model.embed_tokens.weight"].device
    log = __import__("os").environ.get("SNK_TEST_NOISE_LOG")
    for k, layers in parts.items():
        for layer, t in sorted(layers.items()):
            forced = routes.get(k, {}).get(layer)
            forced = forced[0].to(dev) if forced is not None else None
            for what, run in (("mixer", lambda u: plain.layer_mixer(cfg, tensors, layer, u)),
                              ("ffn", lambda u: plain.layer_ffn(cfg, tensors, layer, u, forced))):
                u, got = t[what + "_in"].to(dev), t[what + "_out"].to(dev)
                with torch.no_grad():
                    exact = run(u)
                    with plain.stores_rounded_to(dtype):
                        want = run(u)
                err = rel_all(got, want)
                noise = rel_all(want, exact)
                paged = what == "mixer" and cfg["layer_types"][layer] != "conv"
                bound = 2e-5 if dtype == "float32" else PART_NOISE_SHARE["attention" if paged else "other"] * noise
                if log:
                    with open(log, "a") as f:
                        f.write(f"part {cfg['hidden_size']} L{layer} {cfg['layer_types'][layer][:4]} {what} T{len(u)} "
                                f"err {err:.3e} noise {noise:.3e} ratio {err / max(noise, 1e-30):.3f} "
                                f"rowmax {float(rel_rows(got, want).max()):.3e}\n")
                assert err <= bound, (f"request {k} layer {layer} {what}: rel-L2 {err:.3g} against the plain part on "
                                      f"the same input (bound {bound:.3g}, rounding noise of the part {noise:.3g})")


def check_picks(cfg, tensors, dtype, routes) -> None:
    """The engine's picks against the plain router run on the engine's own router input."""
    differing = total = 0
    for k, layers in routes.items():
        for layer, (ids, x) in layers.items():
            p = f"model.layers.{layer}.feed_forward."
            bias = tensors[p + "expert_bias"] if cfg.get("use_expert_bias") else None
            mg = []
            gate = tensors[p + "gate.weight"]
            ids, x = ids.to(gate.device), x.to(gate.device)
            want, _ = plain.route(x, gate, bias, cfg["num_experts_per_tok"],
                                  cfg.get("norm_topk_prob", False), cfg.get("routed_scaling_factor", 1.0),
                                  margins=mg)
            differs = (ids.long().sort(-1).values != want.sort(-1).values).any(-1)
            clear = mg[0] >= ROUTE_MARGIN[dtype]
            assert not (differs & clear).any(), \
                (f"request {k} layer {layer}: picks differ at positions "
                 f"{torch.nonzero(differs & clear).flatten().tolist()[:10]} where the margin is clear "
                 f"(smallest such margin {float(mg[0][differs & clear].min()):.3g})")
            differing += int(differs.sum())
            total += len(differs)
    assert differing <= ROUTE_FORGIVEN * max(total, 1), f"{differing} of {total} picks differ from the plain router's"


def check_against_plain(model, dtype, reqs, steps, outputs, routes):
    """Logits of every position against the plain implementation (for bfloat16: its rounding variant), with
    the plain experts forced onto the engine's picks, which are checked on their own (``check_picks``): a
    pick that a near-tie turned would otherwise show up as a wrong logit.  ``model``: a model folder, or
    (config, tensors as float) for the plain implementation."""
    cfg, tensors = model if isinstance(model, tuple) else plain.read_model_dir(model)
    got = gather_logits(steps, outputs)
    check_picks(cfg, tensors, dtype, routes)
    worst = 0.0
    for k, toks in reqs.items():
        dev = tensors["model.embed_tokens.weight"].device
        forced = {layer: ids.to(dev) for layer, (ids, _) in routes[k].items()} if routes.get(k) else None
        with plain.stores_rounded_to(dtype):
            want = plain.logits(cfg, tensors, toks, forced_routes=forced)
        err = rel_rows(got[k].to(dev), want).cpu()
        whole = rel_all(got[k].to(dev), want)
        per_position, per_request = TOL[dtype], tol_request(dtype, cfg["num_hidden_layers"])
        if dtype != "float32":
            noise = rel_all(want, plain.logits(cfg, tensors, toks, forced_routes=forced))
            per_position = min(per_position, NOISE_SHARE_POSITION * noise)
            per_request = min(per_request, NOISE_SHARE_REQUEST * noise)
            if __import__("os").environ.get("SNK_TEST_NOISE_LOG"):
                with open(__import__("os").environ["SNK_TEST_NOISE_LOG"], "a") as f:
                    f.write(f"logits {cfg['hidden_size']} L{cfg['num_hidden_layers']} T{len(toks)} all {whole:.5f} "
                            f"noise {noise:.5f} pos_max {float(err.max()):.5f}\n")
        worst = max(worst, float(err.max()))
        bad = torch.nonzero(err > per_position).flatten().tolist()
        assert not bad, (f"request {k}: first wrong position {bad[0]} of {len(toks)} (rel {float(err[bad[0]]):.3g}, "
                         f"bound {per_position:.3g}); all: {bad[:20]}")
        assert whole < per_request, f"request {k}: rel-L2 over all positions {whole:.3g} (bound {per_request:.3g})"
    return worst



# --- traces: lists of steps in the replay tool's format ------------------------------------

def whole_trace(reqs: dict) -> list:
    """Each request alone and whole, all logits wanted."""
    return [{"step": i, "entries": [{"id": k, "tokens": v, "want": list(range(len(v)))}], "end": [k]}
            for i, (k, v) in enumerate(reqs.items())]


def decode_tail_trace(reqs: dict, tail: int = 32) -> list:
    """Most of each request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for k, v in reqs.items():
        head = max(1, len(v) - tail)
        steps.append({"step": len(steps), "entries": [{"id": k, "tokens": v[:head], "want": list(range(head))}],
                      "end": [k] if head == len(v) else []})
        for i in range(head, len(v)):
            steps.append({"step": len(steps), "entries": [{"id": k, "tokens": v[i:i + 1], "want": [0]}],
                          "end": [k] if i == len(v) - 1 else []})
    return steps


def portions_trace(reqs: dict, sizes=(5, 2, 17, 3, 2, 33, 1, 9, 64, 2)) -> list:
    """Portions of changing size, down to two tokens (and single ones)."""
    steps = []
    for k, v in reqs.items():
        i, j = 0, 0
        while i < len(v):
            n = min(sizes[j % len(sizes)], len(v) - i)
            steps.append({"step": len(steps), "entries": [{"id": k, "tokens": v[i:i + n], "want": list(range(n))}],
                          "end": [k] if i + n == len(v) else []})
            i, j = i + n, j + 1
    return steps


def mixed_trace(reqs: dict, seed: int = 0, max_live: int = 4, decode_from: float = 0.6,
                portions=(2, 3, 5, 8, 13, 21, 34)) -> list:
    """Up to ``max_live`` requests at a time: portions of some (sizes drawn from ``portions``) beside single
    tokens of others (from the fraction ``decode_from`` of a request on); requests are sometimes left out of
    a step; a finished request's place is taken by the next."""
    rng = random.Random(seed)
    waiting = list(reqs.items())
    live: dict = {}
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live:
            k, v = waiting.pop(0)
            live[k] = [v, 0]
        entries, end = [], []
        for k, (v, done) in list(live.items()):
            if len(live) > 1 and rng.random() < 0.2:
                continue                                    # left out of this step
            left = len(v) - done
            if done >= decode_from * len(v):
                n = 1
            else:
                n = min(left, rng.choice(portions))
            entries.append({"id": k, "tokens": v[done:done + n], "want": list(range(n))})
            live[k][1] = done + n
            if done + n == len(v):
                end.append(k)
                del live[k]
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


def max_live_tokens(steps, round_to: int = 64) -> int:
    """The --max-tokens a trace needs: the most tokens live requests hold at any time, each
    request's count rounded up."""
    held: dict = {}
    most = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        most = max(most, sum(-(-n // round_to) * round_to for n in held.values()))
        for k in s["end"]:
            held.pop(k, None)
    return most


def gather_logits(steps, outputs) -> dict:
    """{request id -> [T, V] logits in position order} from per-step outputs (None where nothing
    was wanted); every position must have been wanted exactly once."""
    rows: dict = {}
    pos: dict = {}
    for s, out in zip(steps, outputs):
        r = 0
        for e in s["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                rows.setdefault(e["id"], {})[base + w] = out[r]
                r += 1
            pos[e["id"]] = base + len(e["tokens"])
    return {k: torch.stack([v[i] for i in range(len(v))]) for k, v in rows.items()}


# --- guard bands: a buffer the caller sized, with a pattern before and after it ---------------------

class Guarded:
    """A contiguous CUDA tensor of ``shape`` that lies in the middle of a larger allocation whose ends hold a
    fixed pattern.  ``intact()`` tells whether a kernel wrote before the start or past the end (the pattern
    is checked byte for byte).  The bands are 1 KiB each, so the tensor keeps a 256-byte alignment
    (in the manner of SnowLLM's tests/test_sampling_argmax.py:13-44, which over-allocates its output)."""
    BAND = 1024
    PATTERN = 0xA5

    def __init__(self, shape, dtype, fill=None, like=None):
        import math
        n = math.prod(shape) * torch.empty((), dtype=dtype).element_size()
        self.raw = torch.full((n + 2 * self.BAND,), self.PATTERN, dtype=torch.uint8, device="cuda")
        self.tensor = self.raw[self.BAND:self.BAND + n].view(dtype).view(shape)
        if like is not None:
            self.tensor.copy_(like)
        elif fill is not None:
            self.tensor.fill_(fill)
        assert self.tensor.is_contiguous() and self.tensor.data_ptr() % 256 == 0

    def intact(self) -> bool:
        n = self.raw.numel() - 2 * self.BAND
        return bool((self.raw[:self.BAND] == self.PATTERN).all() and (self.raw[self.BAND + n:] == self.PATTERN).all())


class Guards:
    """Hands out guarded tensors and checks all of them at once."""

    def __init__(self):
        self.made: list = []

    def __call__(self, shape, dtype, fill=None, like=None) -> torch.Tensor:
        g = Guarded(tuple(shape), dtype, fill, like)
        self.made.append(g)
        return g.tensor

    def check(self, what: str = "") -> None:
        torch.cuda.synchronize()
        for i, g in enumerate(self.made):
            assert g.intact(), f"{what}: buffer {i} of shape {tuple(g.tensor.shape)} was written outside its bounds"
