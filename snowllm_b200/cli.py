"""Command line in the manner of snowllm/cli.py:366-495: the same option names with the same
meanings where SnowLLM has them.  SnowLLM's command line serves over HTTP; servers are out of scope
here, so ``PATH`` generates for the prompts given on the command line and prints one JSON line per
request.

    python -m snowllm_b200 PATH --prompt-ids 1,2,3 --temperature 0 --default-max-tokens 16
    python -m snowllm_b200 random-weights CONFIG.json OUT_DIR --seed 0 --dtype bfloat16
"""
from __future__ import annotations

import argparse
import json
import pathlib
import re
import sys

from .config.engine import (DEFAULT_CONTEXT_TARGET, DEFAULT_GPU_UTIL, DEFAULT_MAX_NUM_SEQS,
                            DEFAULT_PAGE_SIZE, DEFAULT_PREFILL_CHUNK)

COMMANDS = ("random-weights",)


def _size(x: str) -> int:
    """4096, 32k, 1M (snowllm/cli.py:27-31)."""
    m = re.fullmatch(r"\s*([0-9]*\.?[0-9]+)\s*([kKmM]?)\s*", x)
    if not m:
        raise argparse.ArgumentTypeError(f"{x!r} is not a size (try 4096, 32k, 1M)")
    return int(float(m.group(1)) * {"": 1, "k": 1024, "K": 1024, "m": 2 ** 20, "M": 2 ** 20}[m.group(2)])


def _fraction(x: str) -> float:
    v = float(x)
    if not 0.0 < v <= 1.0:
        raise argparse.ArgumentTypeError(f"{x!r} is not a fraction in (0, 1]")
    return v


def _ids(x: str) -> list:
    try:
        return [int(t) for t in re.split(r"[,\s]+", x.strip()) if t]
    except ValueError:
        raise argparse.ArgumentTypeError(f"{x!r} is not a list of token ids") from None


def parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(
        prog="snowllm_b200",
        usage="snowllm_b200 PATH [options]\n       snowllm_b200 random-weights CONFIG OUT [options]",
        description="Generate with an LFM2.5 model folder (config.json + safetensors) on one B200.")
    g = p.add_argument_group("generation")
    g.add_argument("model", metavar="PATH", help="Checkpoint directory.")
    g.add_argument("--prompt-ids", action="append", type=_ids, default=[], metavar="IDS",
                   help="Prompt as token ids, e.g. 1,2,3; repeatable.")
    g.add_argument("--prompt-file", type=pathlib.Path, metavar="FILE",
                   help="One JSON list of token ids per line.")
    g.add_argument("--prompt", action="append", default=[], metavar="TEXT",
                   help="Prompt as text (needs a tokenizer in the checkpoint directory); repeatable.")
    g.add_argument("--default-max-tokens", type=int, default=32, metavar="N", help="Reply limit.")
    g.add_argument("--temperature", type=float, default=0.0, help="0 decodes greedily.")
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--presence-penalty", type=float, default=0.0)
    g.add_argument("--frequency-penalty", type=float, default=0.0)
    g.add_argument("--repetition-penalty", type=float, default=1.0)
    g.add_argument("--no-repeat-ngram-size", type=int, default=0)
    g.add_argument("--stop-token-ids", type=_ids, default=[], metavar="IDS")
    g.add_argument("--seed", type=int, default=None, help="Random seed for sampling.")
    g.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16",
                   help="Compute precision; float32 runs every product in true 32-bit.")

    g = p.add_argument_group("capacity")
    g.add_argument("--max-num-seqs", type=int, default=DEFAULT_MAX_NUM_SEQS, metavar="N",
                   help="Maximum concurrent requests (up to 256).")
    g.add_argument("--max-model-len", "--max-ctx-len", type=_size, default=DEFAULT_CONTEXT_TARGET, metavar="N",
                   help="Shared KV token capacity; each request is capped at it.")
    g.add_argument("--max-gpu-mem", "--gpu-memory-utilization", dest="max_gpu_mem_util", type=_fraction,
                   default=DEFAULT_GPU_UTIL, metavar="FRACTION", help="GPU memory ceiling as a fraction.")
    g.add_argument("--num-kv-blocks", type=_size, default=None, metavar="N",
                   help="Set the KV cache block count manually.")
    g.add_argument("--kv-block-size", type=int, default=DEFAULT_PAGE_SIZE, metavar="TOKENS")

    g = p.add_argument_group("throughput")
    g.add_argument("--max-num-batched-tokens", default=DEFAULT_PREFILL_CHUNK, metavar="N", type=_size,
                   help="Token budget of one step: prefill chunk size, e.g. 8k.")
    g.add_argument("--kv-cache-dtype", choices=("bf16", "auto"), default="auto",
                   help="KV cache precision; the cache always has the compute precision.")

    g = p.add_argument_group("diagnostics")
    g.add_argument("--enforce-eager", action="store_true", help="Disable GPU graph execution.")
    g.add_argument("--stats-exact", action="store_true", help="Synchronize each step for GPU timing.")
    g.add_argument("--enable-profiler", action="store_true",
                   help="Run under torch.profiler with named spans and write a Chrome trace.")
    g.add_argument("--profiler-dir", "--profile-dir", dest="profile_dir", default="~/.cache/snowllm_b200/profiler",
                   metavar="DIR", help="Where --enable-profiler writes trace.json.")
    return p


def random_weights_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="snowllm_b200 random-weights",
                                description="Write a model folder with seeded random weights.")
    p.add_argument("config", type=pathlib.Path, help="config.json of the architecture")
    p.add_argument("out", type=pathlib.Path, help="folder to write config.json and model.safetensors to")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    p.add_argument("--std", type=float, default=0.02)
    p.add_argument("--conv-std", type=float, default=0.1)
    p.add_argument("--bias-std", type=float, default=0.01)
    return p


def _random_weights(argv) -> int:
    a = random_weights_parser().parse_args(argv)
    from .loader import build_model, parse_dtype
    from .weights import random_tensors, write_model_folder
    model = build_model(json.loads(a.config.read_text()), a.dtype)
    tensors = random_tensors(model, a.seed, parse_dtype(a.dtype), std=a.std, conv_std=a.conv_std,
                             bias_std=a.bias_std)
    write_model_folder(a.out, model.config.to_json_dict(), tensors)
    print(f"wrote {len(tensors)} tensors to {a.out}")
    return 0


def _tokenizer(path):
    try:
        from tokenizers import Tokenizer
    except ImportError:
        return None
    f = pathlib.Path(path) / "tokenizer.json"
    return Tokenizer.from_file(str(f)) if f.exists() else None


def build(a):
    """(engine, tokenizer or None) from parsed arguments (the role of snowllm/cli.py:87-358)."""
    from .config.engine import EngineConfig
    from .engine.engine import Engine
    from .loader import load
    model = load(a.model, a.dtype)
    limit = min(a.max_model_len, model.spec.max_position)
    config = EngineConfig(page_size=a.kv_block_size, num_kv_blocks=a.num_kv_blocks, max_num_seqs=a.max_num_seqs,
                          max_model_len=limit, max_num_batched_tokens=a.max_num_batched_tokens,
                          gpu_memory_utilization=a.max_gpu_mem_util, enforce_eager=a.enforce_eager,
                          seed=a.seed, stop_token_ids=tuple(a.stop_token_ids), exact_stats=a.stats_exact)
    return Engine(model, config), _tokenizer(a.model)


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "random-weights":
        return _random_weights(argv[1:])
    a = parser().parse_args(argv)
    from .engine.request import SamplingParams
    from .errors import SnowLLMError
    prompts = list(a.prompt_ids)
    if a.prompt_file:
        prompts += [json.loads(line) for line in a.prompt_file.read_text().splitlines() if line.strip()]
    try:
        engine, tok = build(a)
        for text in a.prompt:
            if tok is None:
                raise SnowLLMError("--prompt needs tokenizer.json in the model folder; give --prompt-ids")
            prompts.append(tok.encode(text).ids)
        if not prompts:
            raise SnowLLMError("no prompt given (--prompt-ids, --prompt-file or --prompt)")
        params = SamplingParams(
            temperature=a.temperature, top_p=a.top_p, top_k=a.top_k, max_new_tokens=a.default_max_tokens,
            stop_token_ids=tuple(a.stop_token_ids), presence_penalty=a.presence_penalty,
            frequency_penalty=a.frequency_penalty, repetition_penalty=a.repetition_penalty,
            no_repeat_ngram_size=a.no_repeat_ngram_size)
        requests = [engine.add(p, params) for p in prompts]
        if a.enable_profiler:
            from .trace import profile_to
            with profile_to(a.profile_dir):
                engine.run()
        else:
            engine.run()
    except SnowLLMError as e:
        print(f"snowllm_b200: {e}", file=sys.stderr)
        return 1
    for r in requests:
        line = {"prompt_tokens": len(r.prompt), "tokens": r.out, "finish_reason": r.finish_reason}
        if r.error:
            line["error"] = r.error
        if tok is not None:
            line["text"] = tok.decode(r.out)
        print(json.dumps(line))
    print(json.dumps({"stats": engine.stats().accounting}), file=sys.stderr)
    return 0
