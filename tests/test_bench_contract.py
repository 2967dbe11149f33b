"""bench.py's contract where it needs no GPU: more than one GPU is refused with a line and exit code 2, the
reference arm answers with one JSON line, the configurations name every size BASELINE.json gives them, and the
flop count of a prompt agrees with a count made here from the shapes."""
import json
import pathlib
import subprocess
import sys

ROOT = pathlib.Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def run(*args):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, cwd=ROOT)


def test_more_than_one_gpu_is_refused_with_a_line_and_exit_code_2():
    p = run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert p.returncode == 2
    assert len(p.stdout.strip().splitlines()) == 1 and "one GPU" in p.stdout


def test_reference_arm_prints_one_json_line_and_exits_0():
    p = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert p.returncode == 0, p.stderr
    lines = p.stdout.strip().splitlines()
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and isinstance(d["unavailable"], str) and "\n" not in d["unavailable"]


def test_configurations_hold_the_sizes_of_the_baseline():
    import bench
    c = bench.CONFIGS["8b-a1b"]["json"]
    assert (c["hidden_size"], c["num_hidden_layers"], c["num_attention_heads"], c["num_key_value_heads"]) == (2048, 24, 32, 8)
    assert (c["num_experts"], c["num_experts_per_tok"], c["moe_intermediate_size"], c["intermediate_size"]) == (32, 4, 1792, 7168)
    assert c["num_dense_layers"] == 2 and c["vocab_size"] == 65536 and c["conv_L_cache"] == 3
    assert [i for i, k in enumerate(c["layer_types"]) if k == "full_attention"] == [2, 6, 10, 14, 18, 21]
    d = bench.CONFIGS["dense-1.2b"]["json"]
    assert (d["num_hidden_layers"], d["intermediate_size"]) == (16, 8192) and "num_experts" not in d
    assert [i for i, k in enumerate(d["layer_types"]) if k == "full_attention"] == [2, 5, 8, 10, 12, 14]
    e = bench.CONFIGS["dense-2.6b"]["json"]
    assert (e["num_hidden_layers"], e["intermediate_size"]) == (30, 10752)
    assert sum(k == "full_attention" for k in e["layer_types"]) == 8
    assert (bench.CONFIGS["8b-a1b"]["batch"], bench.CONFIGS["8b-a1b"]["context"]) == (8, 8192)
    assert (bench.CONFIGS["dense-1.2b"]["batch"], bench.CONFIGS["dense-1.2b"]["context"]) == (64, 32768)


def test_prompt_flops_agree_with_a_count_from_the_shapes():
    import bench
    c = bench.CONFIGS["8b-a1b"]["json"]
    T, H, V = 2048, 2048, 65536
    conv = 2 * T * H * 3 * H + 2 * T * H * H                        # in_proj, out_proj
    attn = 2 * T * H * 3072 + 2 * T * H * H                        # fused qkv (32 + 2 * 8 heads of 64), o_proj
    attn += 4 * 32 * 64 * (T * (T + 1) // 2)                       # Q K^T and P V over the causal pairs
    dense = 2 * T * 3 * H * 7168
    moe = 2 * T * H * 32 + 2 * T * 4 * 3 * H * 1792                # router, four experts of three products
    want = 18 * conv + 6 * attn + 2 * dense + 22 * moe + 2 * H * V  # and the head for one row
    assert bench.prefill_flops(c, T) == want
    # a later portion pays for the keys before it
    later = bench.prefill_flops(c, T, start=4096) - bench.prefill_flops(c, T)
    assert later == 6 * 4 * 32 * 64 * T * 4096


def test_roofline_denominators_come_from_the_measured_file_when_it_is_there():
    import bench
    pk, source = bench.peaks()
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        assert source == "measured" and pk["hbm_gbs"] == float(d["hbm_gbs"]) and pk["bf16_tflops"] == float(d["bf16_tflops"])
    else:
        assert source == "fallback" and pk == bench.FALLBACK_PEAKS


import pytest


@pytest.mark.gpu
def test_bench_line_has_the_contracts_keys():
    """A short run on four of the layers: one JSON line with every key of the contract, a flat `config` of at most
    20 keys that names both layer counts, launches counted, host bytes counted."""
    p = run("--layers", "4", "--steps", "3", "--warmup", "3")
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [ln for ln in p.stdout.strip().splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches", "prefill", "roofline", "points"):
        assert key in d, key
    assert d["n_gpus"] == 1 and d["steps"] == 3 and d["warmup"] == 3 and d["higher_is_better"] is True
    assert d["dtype"] == "bf16" and d["vs_baseline"] is None and d["value"] > 0 and d["ms_per_step"] > 0
    cfg = d["config"]
    assert len(cfg) <= 20 and all(not isinstance(v, (dict, list)) for v in cfg.values())
    assert cfg["layers"] == 24 and cfg["layers_run"] == 4 and cfg["global_batch"] == 8 and cfg["seq_len"] == 8192
    assert d["gpu_launches"] > 0
    assert {"value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step"} <= set(d["e2e"]) and d["e2e"]["h2d_bytes_per_step"] > 0
    assert {"value", "tokens", "ms", "frac"} <= set(d["prefill"]) and d["prefill"]["tokens"] == 2048
    assert {"bound", "achieved", "peak", "unit", "frac"} <= set(d["roofline"]) and d["roofline"]["bound"] == "hbm"
    assert abs(d["roofline"]["frac"] - d["roofline"]["achieved"] / d["roofline"]["peak"]) < 1e-3
    assert {"decode_b1", "decode_b64"} <= set(d["points"])
    assert {"sm_mhz", "sm_max_mhz", "reasons"} <= set(d["clocks"])
