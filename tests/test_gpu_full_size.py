"""The layer sizes of LFM2.5-8B-A1B (hidden 2048, 32/8 heads of 64, 32 experts of 1792, dense 7168, vocabulary
65,536) in a model cut to four layers (conv, attention, conv with experts, attention with experts), with
random weights: float32 and bfloat16 logits against the plain implementation (run on the GPU in float32 without
TF32).  The tiny models never reach the code paths these sizes take: 512-thread norms, the 1024-thread router
and the router as a tensor-core product, tcgen05 tiles over several rounds, grouped products with thousands
of sorted pairs, the few-rows grouped product with several rows per expert, full K loops.

Cuts: one request whole, in portions and token by token; four requests mixed (portions of 16 to 512 rows
beside decoded rows, three live at a time in a pool so small that pages are used again, free pages and slots
poisoned); one step of 2,048 rows; 64 requests whose prompts run in one step and which then decode as one
step of 64 rows."""
import pytest
import torch

from helpers import (check_against_plain, check_parts, gather_logits, max_live_tokens, mixed_trace, random_prompt, rel_rows,
                     run_in_process)

pytestmark = pytest.mark.gpu

CONFIG = {
    "architectures": ["Lfm2MoeForCausalLM"], "model_type": "lfm2_moe",
    "vocab_size": 65536, "hidden_size": 2048, "num_hidden_layers": 4,
    "layer_types": ["conv", "full_attention", "conv", "full_attention"],
    "num_attention_heads": 32, "num_key_value_heads": 8, "conv_L_cache": 3, "conv_bias": False,
    "num_dense_layers": 2, "intermediate_size": 7168,
    "num_experts": 32, "num_experts_per_tok": 4, "moe_intermediate_size": 1792,
    "norm_topk_prob": True, "use_expert_bias": True, "routed_scaling_factor": 1.0,
    "rope_theta": 1000000.0, "norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 128000,
}
V = CONFIG["vocab_size"]


@pytest.fixture(scope="module")
def setup():
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    from snowllm_b200.loader import build_model
    from snowllm_b200.weights import random_tensors
    model = build_model(CONFIG, "bfloat16")
    tensors = random_tensors(model, 7, torch.bfloat16, device="cuda", fan_in_scaled=True, norm_jitter=0.1)
    plain_tensors = {k: v.float() for k, v in tensors.items()}
    yield tensors, plain_tensors
    del tensors, plain_tensors
    torch.cuda.empty_cache()


def engine_model(tensors, dtype):
    from snowllm_b200.loader import build_model
    from snowllm_b200.weights import load_tensors
    model = build_model(CONFIG, dtype)
    load_tensors(model, tensors, "cuda")
    return model


def statuses_are_clear():
    from snowllm_b200.ops import kernels
    assert kernels.gemm_tc_status() == 0 and kernels.gemm_tc2_status()[0] == 0
    assert kernels.attention_tc_status() == 0 and kernels.attention_decode_status() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_request_whole_in_portions_and_token_by_token(setup, dtype):
    tensors, plain_tensors = setup
    model = engine_model(tensors, dtype)
    toks = random_prompt(V, 150, 3)
    first = None
    for cuts in ([150], [70, 2, 33, 1, 1, 1, 42], [140] + [1] * 10):
        steps, i = [], 0
        for n in cuts:
            steps.append({"step": len(steps), "entries": [{"id": "x", "tokens": toks[i:i + n], "want": list(range(n))}],
                          "end": ["x"] if i + n == len(toks) else []})
            i += n
        outputs, routes = run_in_process(model, dtype, steps, 192, max_requests=2)
        check_against_plain((CONFIG, plain_tensors), dtype, {"x": toks}, steps, outputs, routes)
        got = gather_logits(steps, outputs)["x"]
        if dtype == "float32":
            if first is None:
                first = got
            else:
                assert float(rel_rows(got, first).max()) < 1e-5
    statuses_are_clear()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_four_requests_mixed_with_reused_poisoned_pages(setup, dtype):
    """Portions of 16 to 512 rows of some requests beside decoded rows of others, three live at a time: the
    fourth request takes the pages and the slot that the first to finish gave back, NaN in between."""
    tensors, plain_tensors = setup
    model = engine_model(tensors, dtype)
    reqs = {k: random_prompt(V, n, 11 + i) for i, (k, n) in enumerate({"a": 300, "b": 700, "c": 90, "d": 1200}.items())}
    steps = mixed_trace(reqs, seed=2, max_live=3, decode_from=0.85, portions=(16, 40, 100, 128, 200, 512))
    assert any(len(s["entries"]) > 1 and any(len(e["tokens"]) >= 16 for e in s["entries"])
               and any(len(e["tokens"]) == 1 for e in s["entries"]) for s in steps), "no portion beside a decoded row"
    stats = {}
    outputs, routes = run_in_process(model, dtype, steps, max_live_tokens(steps), poison=True, stats=stats,
                                     max_requests=3)
    assert stats["reused"], "the trace was meant to use pages again"
    got = gather_logits(steps, outputs)
    assert all(v.isfinite().all() for v in got.values()), "a stale (NaN) page or slot was read"
    check_parts((CONFIG, plain_tensors), dtype, stats["parts"], routes)
    check_against_plain((CONFIG, plain_tensors), dtype, reqs, steps, outputs, routes)
    statuses_are_clear()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_step_of_2048_rows(setup, dtype):
    """The size the prefill measurement runs: products over several rounds of tiles, 8,192 sorted (token,
    expert) pairs through the grouped products, the router as a product."""
    tensors, plain_tensors = setup
    model = engine_model(tensors, dtype)
    toks = random_prompt(V, 2048, 5)
    steps = [{"step": 0, "entries": [{"id": "p", "tokens": toks, "want": list(range(2048))}], "end": ["p"]}]
    stats = {}
    outputs, routes = run_in_process(model, dtype, steps, 2048, max_requests=1, stats=stats, page_size=64)
    check_parts((CONFIG, plain_tensors), dtype, stats["parts"], routes)
    check_against_plain((CONFIG, plain_tensors), dtype, {"p": toks}, steps, outputs, routes)
    statuses_are_clear()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_64_prompts_in_one_step_then_decode_steps_of_64_rows(setup, dtype):
    """64 requests: all prompts (20 to 83 tokens) in ONE step, then two steps that hold one decoded token of
    each: 64 rows, 8 rows per expert on average through the grouped few-rows product."""
    tensors, plain_tensors = setup
    model = engine_model(tensors, dtype)
    reqs = {f"r{i}": random_prompt(V, 22 + i, 100 + i) for i in range(64)}
    steps = [{"step": 0, "entries": [{"id": k, "tokens": v[:-2], "want": [len(v) - 3]} for k, v in reqs.items()],
              "end": []},
             {"step": 1, "entries": [{"id": k, "tokens": [v[-2]], "want": [0]} for k, v in reqs.items()], "end": []},
             {"step": 2, "entries": [{"id": k, "tokens": [v[-1]], "want": [0]} for k, v in reqs.items()],
              "end": list(reqs)}]
    outputs, routes = run_in_process(model, dtype, steps, max_live_tokens(steps), max_requests=64, page_size=64)
    assert outputs[1].shape == (64, V)
    check_tails((CONFIG, plain_tensors), dtype, reqs, outputs, routes)
    statuses_are_clear()


def check_tails(model, dtype, reqs, outputs, routes):
    """The last three positions of every request (the rows the three steps asked for) against the plain
    implementation, which runs each request whole with the engine's picks."""
    import plain_lfm2 as plain
    from helpers import NOISE_SHARE_POSITION, TOL, check_picks, rel_all
    cfg, tensors = model
    check_picks(cfg, tensors, dtype, routes)
    dev = tensors["model.embed_tokens.weight"].device
    for row, (k, toks) in enumerate(reqs.items()):
        forced = {layer: ids.to(dev) for layer, (ids, _) in routes[k].items()}
        with plain.stores_rounded_to(dtype):
            want = plain.logits(cfg, tensors, toks, forced_routes=forced)[-3:]
        bound = TOL[dtype]
        if dtype != "float32":            # in units of the rounding noise, as helpers.check_against_plain has it
            bound = min(bound, NOISE_SHARE_POSITION * rel_all(want, plain.logits(cfg, tensors, toks, forced_routes=forced)[-3:]))
        got = torch.stack([outputs[s][row] for s in range(3)]).to(dev)
        err = rel_rows(got, want)
        assert float(err.max()) < bound, f"request {k}: rel {err.tolist()} at its last three positions (bound {bound:.3g})"
