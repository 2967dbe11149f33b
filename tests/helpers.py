"""Shared pieces of the tests: model folders with random weights, traces and comparisons."""
from __future__ import annotations

import random

import torch

import plain_lfm2 as plain
from tiny_configs import ALL

# Relative L2 error allowed between the engine and the plain implementation.
# float32: both sides sum in float32 in different orders: a few 1e-6 per product, about 1e-5 after a
# handful of layers; the bound holds for every single position.
# bfloat16: the bound over a whole request starts from SnowLLM's own acceptance bound for its bf16
# kernels against a float reference: rel-L2 < 0.025 for a 3-layer model
# (tests/test_lfm2_reference.py:66-161).  Rounding errors of successive layers are independent and
# add in quadrature, so a model of L layers gets 0.025 * sqrt(L / 3).  A single position is one
# sample of that error, and the largest of some hundred samples lies a few times above their root
# mean square, so single positions get 0.1: enough to name the first wrong position of a real
# fault (a wrong page, slot or key gives errors of order 1), which the float32 runs of the same
# kernels pin down to 2e-5.
TOL = {"float32": 2e-5, "bfloat16": 0.1}


def tol_request(dtype: str, num_layers: int) -> float:
    return 2e-5 if dtype == "float32" else 0.025 * (max(num_layers, 3) / 3) ** 0.5


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


def mixed_trace(reqs: dict, seed: int = 0, max_live: int = 4, decode_from: float = 0.6) -> list:
    """Up to ``max_live`` requests at a time: portions of some beside single tokens of others;
    requests are sometimes left out of a step; a finished request's place is taken by the next."""
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
                n = min(left, rng.choice((2, 3, 5, 8, 13, 21, 34)))
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
