"""The layer sizes of LFM2.5-8B-A1B (hidden 2048, 32/8 heads of 64, 32 experts of 1792, dense 7168, vocabulary
65,536) in a model cut to four layers (conv, attention, conv with experts, attention with experts), with
random weights: float32 and bfloat16 logits against the plain implementation (run on the GPU in float32 without
TF32), whole, in portions and token by token.  The tiny models never reach the code paths these sizes take
(512-thread norms, 1024-thread router, tcgen05 tiles, full K loops)."""
import pytest
import torch

import plain_lfm2 as plain
from helpers import TOL, random_prompt, rel_all, rel_rows, tol_request

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


def engine_logits(tensors, dtype, toks, cuts):
    """Logits of every position of ``toks``, the prompt cut into steps of the sizes ``cuts``; the routers'
    picks per routed layer, in position order."""
    from snowllm_b200.cache import CacheManager
    from snowllm_b200.engine import ModelRunner, StepEntry
    from snowllm_b200.loader import build_model
    from snowllm_b200.weights import load_tensors
    model = build_model(CONFIG, dtype)
    load_tensors(model, tensors, "cuda")
    cache = CacheManager(model.cache_specs(), 16, 64, 2, model.dtype, "cuda")
    runner = ModelRunner(model, cache)
    rc = cache.admit()
    outs, picks, i = [], {2: [], 3: []}, 0
    for n in cuts:
        n = min(n, len(toks) - i)
        if n <= 0:
            break
        assert cache.ensure(rc, i + n)
        runner.taps = []
        outs.append(runner.step([StepEntry(rc, toks[i:i + n], list(range(n)))]).float().clone())
        for layer, (_, ids) in zip((2, 3), [t for t in runner.taps if t[0] == "moe_route"]):
            picks[layer].append(ids.clone())
        i += n
    assert i == len(toks)
    del runner, cache, model
    return torch.cat(outs), {k: torch.cat(v) for k, v in picks.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_size_layers_match_the_plain_implementation(setup, dtype):
    tensors, plain_tensors = setup
    toks = random_prompt(65536, 150, 3)
    first = None
    for cuts in ([150], [70, 2, 33, 1, 1, 1, 42], [140] + [1] * 10):
        got, picks = engine_logits(tensors, dtype, toks, cuts)
        forced = {k: v.cpu() for k, v in picks.items()}
        margins = {}
        want = plain.logits(CONFIG, plain_tensors, toks, forced_routes={k: v.cuda() for k, v in forced.items()},
                            margins=margins)
        err = rel_rows(got, want)
        bad = torch.nonzero(err > TOL[dtype]).flatten().tolist()
        assert not bad, f"cuts {cuts[:3]}...: first wrong position {bad[0]} (rel {float(err[bad[0]]):.3g})"
        assert rel_all(got, want) < tol_request(dtype, 4)
        if dtype == "float32":
            if first is None:
                first = got
            else:
                assert float(rel_rows(got, first).max()) < 1e-5
    from snowllm_b200.ops import kernels
    assert kernels.gemm_tc_status() == 0
