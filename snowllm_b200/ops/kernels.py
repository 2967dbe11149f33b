"""Python side of the sm_100a kernels: checks of dtype, shape and contiguity, then one launch.

Every function launches on torch's current CUDA stream and returns without synchronising.
There is no other implementation behind these names: a tensor that is not on a CUDA device,
or a library that cannot be built, is an error (the role of snowllm/ops/_common.py:82-112).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from ..csrc import build
from ..errors import KernelError

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

P, I, F, LL = c_void_p, c_int, c_float, c_longlong
_SIGNATURES = {
    "elementwise": {
        "snk_embedding": [P, P, I, P, P, I, I, I, I, P],
        "snk_add_rmsnorm": [P, P, P, I, P, P, I, I, F, I, P, P, P, I, P],
        "snk_residual_add": [P, P, LL, P],
        "snk_swiglu": [P, P, I, I, I, I, P],
    },
    "rope_cache": {
        "snk_qk_norm_rope_cache": [P, P, P, I, I, F, P, I, P, P, P, I, I, P, P, I, I, I, I, I, I, P],
    },
    "short_conv": {
        "snk_short_conv": [P, P, I, P, P, P, P, P, P, I, I, I, I, I, P],
    },
    "attention": {
        "snk_paged_attention_scratch_bytes": [I, I, I, I],
        "snk_paged_attention": [P, P, P, I, I, P, P, P, P, I, I, I, I, I, I, I, F, I, P],
        "snk_paged_attention_rows": [P, P, P, I, I, P, P, P, P, I, I, I, I, I, I, I, F, I, P, P],
        "snk_attention_merge": [P, P, P, I, I, I, I, I, I, I, P, P],
    },
    "attention_mma": {
        "snk_attention_prefill": [P, P, P, I, I, P, I, P, I, I, I, I, F, P],
        "snk_attention_decode_mma": [P, P, P, I, I, P, P, P, P, P, I, I, I, I, I, I, F, P],
        "snk_attention_prefill_tma": [P, P, LL, P, I, I, P, I, P, I, I, I, I, F, P],
        "snk_attention_decode_tma": [P, P, LL, P, I, I, P, P, P, P, P, I, I, I, I, I, I, F, P],
        "snk_attention_decode_status": [],
        "snk_attention_decode_status_peek": [P, P],
    },
    "attention_tc": {
        "snk_attention_prefill_tc": [P, LL, P, LL, P, I, I, P, I, P, I, I, I, I, F, P],
        "snk_attention_tc_status": [],
        "snk_attention_tc_status_peek": [P, P],
    },
    "gemm": {
        "snk_gemm_simt": [P, P, P, I, I, I, P, I, P, I, I, I, I, P],
    },
    "gemm_skinny": {
        "snk_gemm_skinny": [P, P, P, I, I, I, P, I, P, I, I, I, I, P],
    },
    "gemm_tc": {
        "snk_gemm_tc": [P, P, P, I, I, I, P, I, I, I, I, P, P],
        "snk_gemm_tc_scratch_bytes": [I, I, I, I],
        "snk_gemm_tc_status": [],
        "snk_gemm_tc_status_peek": [P, P],
        "snk_gemm_tc_test_lose_loads": [I],
        "snk_gemm_tc_parts": [P, P, P, I, I, I, P, P],
        "snk_gather_rows_bf16": [P, P, P, I, I, I, P],
    },
    "gemm_tc2": {
        "snk_gemm_tc2": [P, P, P, I, I, I, P, I, I, I, P],
        "snk_gemm_tc2_status": [P],
        "snk_gemm_tc2_status_peek": [P, P],
        "snk_gemm_tc2_test_lose_loads": [I],
    },
    "moe": {
        "snk_moe_route": [P, P, I, P, P, P, I, I, I, I, I, F, I, P],
        "snk_moe_topk": [P, P, P, P, I, I, I, I, F, I, I, P],
        "snk_moe_route_sort": [P, P, I, P, P, P, P, P, P, P, I, I, I, I, I, F, I, P],
        "snk_moe_sort": [P, P, P, P, I, I, P],
        "snk_norm_route_sort": [P, P, P, I, P, I, F, P, P, P, I, P, I, P, P, P, P, P, P, I, I, I, I, F, I, P, P],
        "snk_moe_combine": [P, P, P, P, I, I, I, P],
    },
    "sampling": {
        "snk_argmax": [P, P, I, I, P],
        "snk_apply_penalties": [P, P, P, P, P, P, P, I, I, P],
        "snk_sample": [P, P, P, P, P, P, I, I, P],
    },
}
_RESTYPES = {"snk_paged_attention_scratch_bytes": LL, "snk_gemm_tc_scratch_bytes": LL}
_functions: dict[str, object] = {}
_library_of = {fn: lib for lib, fns in _SIGNATURES.items() for fn in fns}

_ERRORS = {20001: "unknown dtype code", 20002: "a size this kernel does not take",
           20003: "a pointer or pitch that is not aligned as the kernel needs"}


def register_signatures(library: str, signatures: dict, restypes: dict | None = None) -> None:
    """Let another source file of csrc/ be called through ``fn``."""
    _SIGNATURES.setdefault(library, {}).update(signatures)
    for name in signatures:
        _library_of[name] = library
    _RESTYPES.update(restypes or {})


def fn(name: str):
    f = _functions.get(name)
    if f is None:
        lib = build.load(_library_of[name])
        f = getattr(lib, name)
        f.argtypes = _SIGNATURES[_library_of[name]][name]
        f.restype = _RESTYPES.get(name, c_int)
        _functions[name] = f
    return f


def libraries_for(names) -> None:
    """Build (in parallel) the libraries that hold the named groups, before first use."""
    build.build(tuple(dict.fromkeys(names)))


def set_pdl(on: bool) -> None:
    """Switch programmatic dependent launch on or off for every library loaded so far (launches made from
    now on; a captured graph keeps what it was captured with)."""
    for name in list(_SIGNATURES):
        if build.is_loaded(name):
            f = build.load(name).snk_pdl_set
            f.argtypes, f.restype = [c_int], None
            f(int(bool(on)))


_launches = 0

# When a list: every wrapper appends (its name, kernels it launched, bytes it has to move, flops it has to do)
# for each call, in launch order: the ledger that a measurement lays beside a profiler's kernel times.  The
# bytes are the algorithmic ones (each operand and result once); None where a wrapper does not say.  Some
# figures need a look at device data (which experts own rows, how long each row's sequence is): with the
# ledger on, a wrapper may synchronise.  Off (None), it costs nothing.
ledger: list | None = None


def launch_count() -> int:
    """Kernels launched through this module so far (each wrapper reports how many it starts)."""
    return _launches


def _nbytes(*tensors) -> int:
    return sum(t.numel() * t.element_size() for t in tensors if t is not None)


def check(status: int, what: str, launches: int = 1, work=None) -> None:
    """``work``: a function giving (bytes, flops) of the call; evaluated only when the ledger is on."""
    global _launches
    if status == 0:
        _launches += launches
        if ledger is not None and launches:
            nbytes, flops = work() if work is not None else (None, None)
            ledger.append((what, launches, nbytes, flops))
        return
    if status in _ERRORS:
        raise KernelError(f"{what}: {_ERRORS[status]}")
    raise KernelError(f"{what}: CUDA error {status} ({_cuda_error_name(status)})")


def _cuda_error_name(code: int) -> str:
    try:
        rt = ctypes.CDLL("libcudart.so")
        rt.cudaGetErrorString.restype = ctypes.c_char_p
        return rt.cudaGetErrorString(code).decode()
    except OSError:
        return "?"


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def _chk(t: torch.Tensor, what: str, dtype=None, shape=None) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{what}: needs a CUDA tensor (this engine has no CPU path)")
    if dtype is not None and t.dtype not in (dtype if isinstance(dtype, tuple) else (dtype,)):
        raise KernelError(f"{what}: dtype {t.dtype}, want {dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{what}: must be contiguous")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise KernelError(f"{what}: shape {tuple(t.shape)}, want {tuple(shape)}")


def code_of(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"compute dtype {dtype} is not supported (float32 or bfloat16)") from None


def _small(t: torch.Tensor, what: str, compute: torch.dtype) -> int:
    """A small weight may be float32 or the compute dtype; returns its is-float flag."""
    _chk(t, what, (torch.float32, compute))
    return int(t.dtype == torch.float32)


# --- elementwise -----------------------------------------------------------------------

def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor | None = None,
              pending: torch.Tensor | None = None) -> torch.Tensor:
    """Float rows of ``table`` (compute dtype) at int32 ``ids``: the start of the residual stream.
    An id -(i + 1) reads its token from ``pending[i]`` (int32, on the device)."""
    M = ids.numel()
    V, H = table.shape
    _chk(ids, "embedding ids", torch.int32)
    if pending is not None:
        _chk(pending, "pending tokens", torch.int32)
    _chk(table, "embedding table", (torch.float32, torch.bfloat16))
    if out is None:
        out = torch.empty(M, H, dtype=torch.float32, device=table.device)
    _chk(out, "embedding output", torch.float32, (M, H))
    check(fn("snk_embedding")(_ptr(ids), _ptr(pending), pending.numel() if pending is not None else 0,
                              _ptr(table), _ptr(out), M, H, V, code_of(table.dtype), _stream()), "embedding",
          work=lambda: (M * H * table.element_size() + _nbytes(out, ids), 0))
    return out


class ExpertSum:
    """A residual delta that is still in pieces: the routed experts' outputs ``y`` [pairs, H] (float), where
    each (token, pick) pair's row lies (``pair_pos`` int32 [M*k]) and the picks' weights (``weights`` float
    [M, k]).  The norm that follows adds sum_j w[m, j] * y[pair_pos[m*k + j]] into the residual itself;
    ``dense()`` forms the sum for anyone else."""

    def __init__(self, y, pair_pos, weights):
        self.y, self.pair_pos, self.weights = y, pair_pos, weights
        self.shape = (weights.shape[0], y.shape[1])

    def dense(self) -> torch.Tensor:
        return moe_combine(self.y, self.pair_pos, self.weights)


def add_rmsnorm(residual: torch.Tensor, delta, gamma: torch.Tensor, eps: float,
                dtype: torch.dtype, rows: torch.Tensor | None = None,
                out: torch.Tensor | None = None) -> torch.Tensor:
    """``residual += delta`` (if given), then RMSNorm of the sum into the compute dtype.  With
    ``rows`` only those rows are normalised and the residual is left as it is.  ``delta`` is a float
    tensor [M, H] or an ``ExpertSum``."""
    M, H = residual.shape
    _chk(residual, "residual", torch.float32)
    moe = None
    if isinstance(delta, ExpertSum):
        if H % 4 == 0:
            moe, delta = delta, None
            _chk(moe.y, "expert outputs", torch.float32)
            _chk(moe.pair_pos, "pair positions", torch.int32, (M * moe.weights.shape[1],))
            _chk(moe.weights, "top-k weights", torch.float32)
        else:
            delta = delta.dense()
    if delta is not None:
        _chk(delta, "residual delta", torch.float32, (M, H))
    g32 = _small(gamma, "norm weight", dtype)
    _chk(gamma, "norm weight", shape=(H,))
    R = M if rows is None else rows.numel()
    if rows is not None:
        _chk(rows, "norm rows", torch.int32)
    if out is None:
        out = torch.empty(R, H, dtype=dtype, device=residual.device)
    _chk(out, "norm output", dtype, (R, H))
    check(fn("snk_add_rmsnorm")(_ptr(residual), _ptr(delta), _ptr(gamma), g32, _ptr(out), _ptr(rows),
                                R, H, float(eps), code_of(dtype), _ptr(moe.y if moe else None),
                                _ptr(moe.pair_pos if moe else None), _ptr(moe.weights if moe else None),
                                moe.weights.shape[1] if moe else 0, _stream()), "add_rmsnorm",
          work=lambda: (R * H * 4 + _nbytes(out, gamma) + (_nbytes(delta) + M * H * 4 if delta is not None else 0)
                        + ((moe.weights.shape[1] + 1) * M * H * 4 if moe else 0), 0))
    return out


def residual_add(residual: torch.Tensor, delta: torch.Tensor) -> None:
    _chk(residual, "residual", torch.float32)
    _chk(delta, "residual delta", torch.float32, residual.shape)
    check(fn("snk_residual_add")(_ptr(residual), _ptr(delta), residual.numel(), _stream()), "residual_add")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor | None = None, interleaved: bool = False) -> torch.Tensor:
    """[M, 2I] -> [M, I]: silu(gate) * up.  Columns are (gate | up), or with ``interleaved`` blocks of 8
    gate columns followed by the 8 up columns of the same features."""
    M, two_i = gate_up.shape
    _chk(gate_up, "swiglu input", (torch.float32, torch.bfloat16))
    if two_i % 2:
        raise KernelError("swiglu input needs an even width")
    inter = two_i // 2
    if out is None:
        out = torch.empty(M, inter, dtype=gate_up.dtype, device=gate_up.device)
    _chk(out, "swiglu output", gate_up.dtype, (M, inter))
    check(fn("snk_swiglu")(_ptr(gate_up), _ptr(out), M, inter, int(interleaved), code_of(gate_up.dtype), _stream()),
          "swiglu", work=lambda: (_nbytes(gate_up, out), 0))
    return out


# --- attention -------------------------------------------------------------------------

def qk_norm_rope_cache(qkv, q_gamma, k_gamma, eps, inv_freq, rot_dim, positions, row_seg, block_table,
                       page_size, pool, num_heads, num_kv_heads, head_dim, write_kv=True, q_out=None):
    """Per-head RMSNorm of q and k (if weights are given), rotary encoding (if ``inv_freq``), k and v
    written to the paged pool at each row's position; returns q as [M, heads, head_dim]."""
    M = qkv.shape[0]
    dtype = qkv.dtype
    width = (num_heads + (2 * num_kv_heads if write_kv else 0)) * head_dim
    _chk(qkv, "qkv", (torch.float32, torch.bfloat16), (M, width))
    has_norm = q_gamma is not None
    g32 = 0
    if has_norm:
        g32 = _small(q_gamma, "q norm weight", dtype)
        if _small(k_gamma, "k norm weight", dtype) != g32:
            raise KernelError("q and k norm weights must share a dtype")
        _chk(q_gamma, "q norm weight", shape=(head_dim,))
        _chk(k_gamma, "k norm weight", shape=(head_dim,))
    if inv_freq is not None:
        _chk(inv_freq, "inv_freq", torch.float32, (rot_dim // 2,))
    _chk(positions, "positions", torch.int32, (M,))
    _chk(row_seg, "row_seg", torch.int32, (M,))
    _chk(block_table, "block table", torch.int32)
    _chk(pool, "kv pool", dtype)
    if pool.dim() != 5 or tuple(pool.shape[1:]) != (2, num_kv_heads, page_size, head_dim):
        raise KernelError(f"kv pool shape {tuple(pool.shape)}, want [pages, 2, {num_kv_heads}, "
                          f"{page_size}, {head_dim}]")
    if q_out is None:
        q_out = torch.empty(M, num_heads, head_dim, dtype=dtype, device=qkv.device)
    _chk(q_out, "q output", dtype, (M, num_heads, head_dim))
    check(fn("snk_qk_norm_rope_cache")(
        _ptr(qkv), _ptr(q_gamma), _ptr(k_gamma), g32, int(has_norm), float(eps), _ptr(inv_freq),
        int(rot_dim if inv_freq is not None else 0), _ptr(positions), _ptr(row_seg), _ptr(block_table),
        block_table.shape[1], page_size, _ptr(pool), _ptr(q_out), M, num_heads, num_kv_heads, head_dim,
        int(write_kv), code_of(dtype), _stream()), "qk_norm_rope_cache",
        work=lambda: (2 * _nbytes(qkv), 0))
    return q_out


ATTENTION_TILE = 32


def _rows_attention_work(q, pool, positions, rows, window):
    """(bytes, flops) of attention for single rows: each row reads its keys and values of every kv head
    once (a look at the positions: only called with the ledger on)."""
    pos = positions.cpu().long()
    if rows is not None:
        pos = pos[rows.cpu().long()]
    keys = pos + 1
    if window:
        keys = keys.clamp(max=int(window))
    total = int(keys.sum())
    nh, hd = q.shape[1], q.shape[2]
    return (total * 2 * pool.shape[2] * hd * pool.element_size() + 2 * len(pos) * nh * hd * q.element_size(),
            4 * nh * hd * total)


def _tiles_attention_work(q, pool, tiles, window):
    """(bytes, flops) of attention for prompt tiles: the rows of a tile share their keys and values."""
    t = tiles.cpu().long()
    nh, hd = q.shape[1], q.shape[2]
    nbytes = flops = 0
    for _, _, n, p0 in t.tolist():
        last = p0 + n                                   # keys the tile's last row sees
        first = max(0, p0 - int(window) + 1) if window else 0
        pairs = sum(min(p + 1, int(window)) if window else p + 1 for p in range(p0, p0 + n))
        nbytes += (last - first) * 2 * pool.shape[2] * hd * pool.element_size() + 2 * n * nh * hd * q.element_size()
        flops += 4 * nh * hd * pairs
    return nbytes, flops


def attention_scratch_bytes(M: int, num_heads: int, head_dim: int, num_chunks: int) -> int:
    return int(fn("snk_paged_attention_scratch_bytes")(M, num_heads, head_dim, num_chunks))


def paged_attention(q, pool, block_table, page_size, positions, row_seg, scale, window=None,
                    chunk=None, num_chunks=1, scratch=None, out=None, rows=None):
    """Causal attention of each row of q [M, heads, head_dim] over its request's cached keys up to
    its own position.  ``chunk`` keys per block along the sequence (a multiple of 32) and
    ``num_chunks`` = the most chunks any row spans; more than one needs ``scratch`` bytes.
    ``rows`` (int32): serve only these rows of the batch; the others of ``out`` are left alone."""
    M, nh, hd = q.shape
    dtype = q.dtype
    _chk(q, "q", (torch.float32, torch.bfloat16))
    _chk(pool, "kv pool", dtype)
    nkv = pool.shape[2]
    _chk(positions, "positions", torch.int32, (M,))
    _chk(row_seg, "row_seg", torch.int32, (M,))
    _chk(block_table, "block table", torch.int32)
    if chunk is None:
        chunk = 1 << 30
        chunk -= chunk % ATTENTION_TILE
    if out is None:
        out = torch.empty(M, nh * hd, dtype=dtype, device=q.device)
    _chk(out, "attention output", dtype, (M, nh * hd))
    served = M
    if rows is not None:
        _chk(rows, "attention rows", torch.int32)
        served = rows.numel()
    if num_chunks > 1:
        need = attention_scratch_bytes(served, nh, hd, num_chunks)
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.uint8, device=q.device)
        _chk(scratch, "attention scratch", torch.uint8)
        if scratch.numel() < need:
            raise KernelError(f"attention scratch holds {scratch.numel()} bytes, needs {need}")
    check(fn("snk_paged_attention_rows")(
        _ptr(q), _ptr(pool), _ptr(block_table), block_table.shape[1], page_size, _ptr(positions),
        _ptr(row_seg), _ptr(out), _ptr(scratch), served, nh, nkv, hd, int(window or 0), int(chunk),
        int(num_chunks), float(scale), code_of(dtype), _ptr(rows), _stream()), "paged_attention",
        launches=2 if num_chunks > 1 else 1, work=lambda: _rows_attention_work(q, pool, positions, rows, window))
    return out


PREFILL_TILE_ROWS = 64
PREFILL_HEAD_DIMS = (64, 128)


def attention_prefill_ok(q) -> bool:
    """Whether the tensor-core prompt kernel takes this q [M, heads, head_dim]."""
    return q.dtype == torch.bfloat16 and q.shape[2] in PREFILL_HEAD_DIMS


def prefill_tma_page_ok(page_size: int) -> bool:
    """Page sizes whose pages a TMA box brings into a 64-key tile whole (csrc/attention_mma.cu)."""
    return page_size in (8, 16, 32, 64)


PREFILL_TMA = os.environ.get("SNOWLLM_B200_PREFILL_TMA", "1") != "0"


def attention_prefill(q, pool, block_table, page_size, tiles, scale, out, window=None, tma=None):
    """Tensor-core causal attention for prompt portions: ``tiles`` int32 [n, 4] = (segment, first row,
    rows <= 64, position of the first row); writes those rows of ``out`` [M, heads*head_dim].
    ``tma``: bring keys and values in by TMA (default: wherever the page size allows); both ways give the
    same bits."""
    M, nh, hd = q.shape
    _chk(q, "q", torch.bfloat16)
    _chk(pool, "kv pool", torch.bfloat16)
    _chk(tiles, "attention tiles", torch.int32)
    _chk(block_table, "block table", torch.int32)
    _chk(out, "attention output", torch.bfloat16, (M, nh * hd))
    if tiles.dim() != 2 or tiles.shape[1] != 4:
        raise KernelError("attention tiles must be [n, 4]")
    if tma is None:
        tma = PREFILL_TMA and prefill_tma_page_ok(page_size)
    if tma:
        check(fn("snk_attention_prefill_tma")(
            _ptr(q), _ptr(pool), pool.shape[0], _ptr(block_table), block_table.shape[1], page_size, _ptr(tiles),
            tiles.shape[0], _ptr(out), nh, pool.shape[2], hd, int(window or 0), float(scale), _stream()),
            "attention_prefill_tma", work=lambda: _tiles_attention_work(q, pool, tiles, window))
    else:
        check(fn("snk_attention_prefill")(
            _ptr(q), _ptr(pool), _ptr(block_table), block_table.shape[1], page_size, _ptr(tiles), tiles.shape[0],
            _ptr(out), nh, pool.shape[2], hd, int(window or 0), float(scale), _stream()), "attention_prefill",
            work=lambda: _tiles_attention_work(q, pool, tiles, window))
    return out


PREFILL_TC_TILE_ROWS = 128
PREFILL_TC = os.environ.get("SNOWLLM_B200_PREFILL_TC", "1") != "0"


def attention_prefill_tc_ok(q, page_size: int) -> bool:
    """Whether the tcgen05 prompt kernel (csrc/attention_tc.cu) takes this q [M, heads, head_dim] and page size."""
    return (PREFILL_TC and q.dtype == torch.bfloat16 and q.shape[2] == 64
            and page_size in (8, 16, 32, 64, 128))


def attention_prefill_tc(q, pool, block_table, page_size, tiles, scale, out, window=None):
    """Causal attention for prompt portions on the tcgen05 tensor cores: ``tiles`` int32 [n, 4] = (segment,
    first row, rows <= 128, position of the first row); writes those rows of ``out`` [M, heads*64]."""
    M, nh, hd = q.shape
    _chk(q, "q", torch.bfloat16)
    _chk(pool, "kv pool", torch.bfloat16)
    _chk(tiles, "attention tiles", torch.int32)
    _chk(block_table, "block table", torch.int32)
    _chk(out, "attention output", torch.bfloat16, (M, nh * hd))
    if tiles.dim() != 2 or tiles.shape[1] != 4:
        raise KernelError("attention tiles must be [n, 4]")
    check(fn("snk_attention_prefill_tc")(
        _ptr(q), M, _ptr(pool), pool.shape[0], _ptr(block_table), block_table.shape[1], page_size, _ptr(tiles),
        tiles.shape[0], _ptr(out), nh, pool.shape[2], hd, int(window or 0), float(scale), _stream()),
        "attention_prefill_tc", work=lambda: _tiles_attention_work(q, pool, tiles, window))
    return out


def attention_tc_status() -> int:
    """0, or the code of a wait that ran out inside the tcgen05 prompt kernel since the last call (clears it;
    synchronises the device)."""
    return int(fn("snk_attention_tc_status")())


DECODE_MMA_CHUNK = 256
DECODE_MMA_MAX_GROUP = 16


def attention_decode_mma_ok(q, num_kv_heads: int) -> bool:
    """Whether the tensor-core kernel for decoded rows takes this q [M, heads, head_dim]."""
    return (q.dtype == torch.bfloat16 and q.shape[2] in PREFILL_HEAD_DIMS
            and q.shape[1] // num_kv_heads <= DECODE_MMA_MAX_GROUP)


def decode_tma_page_ok(page_size: int) -> bool:
    """Page sizes whose pages a TMA box brings in whole (csrc/attention_mma.cu)."""
    return 8 <= page_size <= DECODE_MMA_CHUNK and page_size % 8 == 0 and DECODE_MMA_CHUNK % page_size == 0


DECODE_TMA = os.environ.get("SNOWLLM_B200_DECODE_TMA", "1") != "0"


def attention_decode_status() -> int:
    """0, or 1 when a block of the TMA decode kernel gave up waiting for its keys (clears it)."""
    return int(fn("snk_attention_decode_status")())


def attention_decode_mma(q, pool, block_table, page_size, positions, row_seg, scale, num_chunks, out,
                         window=None, scratch=None, rows=None, tma=None):
    """Tensor-core attention for rows with long runs of keys (decoded tokens): keys in chunks of 256, the
    q heads of a kv head as the rows of the MMA; chunks merged in order when there is more than one.
    ``tma``: bring keys and values in by TMA (default: wherever the page size allows); both ways give the
    same bits."""
    M, nh, hd = q.shape
    _chk(q, "q", torch.bfloat16)
    _chk(pool, "kv pool", torch.bfloat16)
    _chk(positions, "positions", torch.int32, (M,))
    _chk(row_seg, "row_seg", torch.int32, (M,))
    _chk(block_table, "block table", torch.int32)
    _chk(out, "attention output", torch.bfloat16, (M, nh * hd))
    served = M
    if rows is not None:
        _chk(rows, "attention rows", torch.int32)
        served = rows.numel()
    if num_chunks > 1:
        need = attention_scratch_bytes(served, nh, hd, num_chunks)
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.uint8, device=q.device)
        _chk(scratch, "attention scratch", torch.uint8)
        if scratch.numel() < need:
            raise KernelError(f"attention scratch holds {scratch.numel()} bytes, needs {need}")
    if tma is None:
        tma = DECODE_TMA and decode_tma_page_ok(page_size)
    if tma:
        check(fn("snk_attention_decode_tma")(
            _ptr(q), _ptr(pool), pool.shape[0], _ptr(block_table), block_table.shape[1], page_size, _ptr(positions),
            _ptr(row_seg), _ptr(rows), _ptr(out), _ptr(scratch), served, nh, pool.shape[2], hd, int(window or 0),
            int(num_chunks), float(scale), _stream()), "attention_decode_tma",
            work=lambda: _rows_attention_work(q, pool, positions, rows, window))
    else:
        check(fn("snk_attention_decode_mma")(
            _ptr(q), _ptr(pool), _ptr(block_table), block_table.shape[1], page_size, _ptr(positions), _ptr(row_seg),
            _ptr(rows), _ptr(out), _ptr(scratch), served, nh, pool.shape[2], hd, int(window or 0), int(num_chunks),
            float(scale), _stream()), "attention_decode_mma",
            work=lambda: _rows_attention_work(q, pool, positions, rows, window))
    if num_chunks > 1:
        check(fn("snk_attention_merge")(_ptr(scratch), _ptr(positions), _ptr(out), served, nh, hd, int(window or 0),
                                        DECODE_MMA_CHUNK, int(num_chunks), BF16, _ptr(rows), _stream()),
              "attention_merge", work=lambda: (served * nh * (hd + 2) * 4 * int(num_chunks) + served * nh * hd * 2, 0))
    return out


class StatusWatch:
    """The error words of the kernels whose waits are bounded (TMA and tcgen05 kernels: a wait that runs out
    makes the block give up, and its rows of the output are then not to be trusted), read where the host
    synchronises with the stream anyway.

    ``peek()`` queues, on the current stream, a copy of every loaded library's status word into pinned host
    memory; it neither waits nor clears.  After the host has synchronised with the stream (an event, a
    read-back), ``check()`` raises KernelError if a word is set, and clears it on the device.  The words are
    sticky, so an error is never lost between a peek and a later check."""
    WORDS = (("gemm_tc", "snk_gemm_tc_status_peek", 1, lambda: gemm_tc_status()),
             ("gemm_tc2", "snk_gemm_tc2_status_peek", 1, lambda: gemm_tc2_status()[0]),
             ("attention_tc", "snk_attention_tc_status_peek", 1, lambda: attention_tc_status()),
             ("attention_mma", "snk_attention_decode_status_peek", 2, lambda: attention_decode_status()))

    def __init__(self):
        self.host = torch.zeros(sum(w[2] for w in self.WORDS), dtype=torch.int32).pin_memory()
        self._base = self.host.data_ptr()

    def peek(self) -> None:
        at = 0
        for library, peek, words, _ in self.WORDS:
            if build.is_loaded(library):
                check(fn(peek)(c_void_p(self._base + 4 * at), _stream()), peek, launches=0)
            at += words

    def check(self) -> None:
        """Call after the host has synchronised with a stream position behind a ``peek``."""
        if not bool(self.host.any()):
            return
        at, found = 0, []
        for library, _, words, clear in self.WORDS:
            codes = self.host[at:at + words].tolist()
            if any(codes):
                found.append(f"{library} (code {codes if words > 1 else codes[0]})")
                clear()
            at += words
        self.host.zero_()
        raise KernelError("a bounded wait ran out inside a kernel of " + ", ".join(found) +
                          ": the step's results are not to be trusted")


# --- short convolution -----------------------------------------------------------------

def short_conv(bcx, weight, state, cu_seqlens, seg_start, seg_slot, row_seg, out=None):
    """Gated causal depthwise convolution over [M, 3H] rows (B | C | x) of a flat batch of segments;
    ``state`` [slots, L-1, H] holds each request's history and is brought up to date."""
    M, three_h = bcx.shape
    dtype = bcx.dtype
    H = three_h // 3
    _chk(bcx, "conv input", (torch.float32, torch.bfloat16), (M, 3 * H))
    w32 = _small(weight, "conv weight", dtype)
    L = weight.shape[1]
    _chk(weight, "conv weight", shape=(H, L))
    _chk(state, "conv state", dtype)
    if state.dim() != 3 or tuple(state.shape[1:]) != (max(L - 1, 0), H):
        raise KernelError(f"conv state shape {tuple(state.shape)}, want [slots, {L - 1}, {H}]")
    B = seg_start.numel()
    _chk(cu_seqlens, "cu_seqlens", torch.int32, (B + 1,))
    _chk(seg_start, "seg_start", torch.int32, (B,))
    _chk(seg_slot, "seg_slot", torch.int32, (B,))
    _chk(row_seg, "row_seg", torch.int32, (M,))
    if out is None:
        out = torch.empty(M, H, dtype=dtype, device=bcx.device)
    _chk(out, "conv output", dtype, (M, H))
    check(fn("snk_short_conv")(_ptr(bcx), _ptr(weight), w32, _ptr(state), _ptr(cu_seqlens), _ptr(seg_start),
                               _ptr(seg_slot), _ptr(row_seg), _ptr(out), M, B, H, L, code_of(dtype),
                               _stream()), "short_conv", launches=2 if L > 1 and M != B else 1,
          work=lambda: (_nbytes(bcx, out, weight) + 2 * B * max(L - 1, 0) * H * state.element_size(), 2 * M * H * (L + 2)))
    return out


# --- matrix products -------------------------------------------------------------------

def _gemm_work(rows, a, w, out, offsets):
    """(bytes, flops) of a product: a's rows and the result once, of a grouped W only the groups that own
    rows (a look at the offsets: only called with the ledger on)."""
    K = a.shape[1]
    N = w.shape[-2]
    wbytes = _nbytes(w)
    if offsets is not None:
        o = offsets.cpu()
        wbytes = wbytes // w.shape[0] * int((o[1:] > o[:-1]).sum())
    return rows * K * a.element_size() + wbytes + _nbytes(out), 2 * rows * N * K


def gemm_simt(a, w, out_dtype=None, out=None, a_rows=None, a_div=1, offsets=None, rows_out=None,
              max_rows_per_group=None):
    """a [M, K] times w [N, K]^T (or, grouped, w [G, N, K] over rows sorted by group) with float
    accumulation in k order on the CUDA cores."""
    dtype = a.dtype
    _chk(a, "gemm a", (torch.float32, torch.bfloat16))
    _chk(w, "gemm w", dtype)
    K = a.shape[1]
    grouped = offsets is not None
    if grouped:
        G, N, Kw = w.shape
        _chk(offsets, "group offsets", torch.int32, (G + 1,))
    else:
        G = 1
        N, Kw = w.shape
    if Kw != K:
        raise KernelError(f"gemm: a has K={K}, w has K={Kw}")
    M = rows_out if rows_out is not None else a.shape[0]
    if a_rows is not None:
        _chk(a_rows, "gemm row gather", torch.int32)
    out_dtype = out_dtype or dtype
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    _chk(out, "gemm out", out_dtype, (M, N))
    if out_dtype not in (dtype, torch.float32):
        raise KernelError("gemm output is the compute dtype or float32")
    check(fn("snk_gemm_simt")(_ptr(a), _ptr(w), _ptr(out), M, N, K, _ptr(a_rows), int(a_div), _ptr(offsets),
                              G, int(max_rows_per_group if grouped else M),
                              int(out_dtype == torch.float32), code_of(dtype), _stream()), "gemm_simt",
          work=lambda: _gemm_work(M, a, w, out, offsets))
    return out


def gemm_skinny_ok(a, w) -> bool:
    """Whether the few-rows bfloat16 kernel takes these operands."""
    return (a.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and a.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0)


def gemm_skinny(a, w, out_dtype=None, out=None, a_rows=None, a_div=1, offsets=None, rows_out=None,
                rows_hint=None, swiglu=False):
    """bfloat16 a [M, K] times w [N, K]^T (or grouped w [G, N, K]) for few rows: W streams from memory
    once into tensor-core fragments.  ``rows_hint``: rows expected per group (sets the pass size)."""
    _chk(a, "gemm a", torch.bfloat16)
    _chk(w, "gemm w", torch.bfloat16)
    K = a.shape[1]
    grouped = offsets is not None
    if grouped:
        G, N, Kw = w.shape
        _chk(offsets, "group offsets", torch.int32, (G + 1,))
    else:
        G = 1
        N, Kw = w.shape
    if Kw != K:
        raise KernelError(f"gemm: a has K={K}, w has K={Kw}")
    M = rows_out if rows_out is not None else a.shape[0]
    if a_rows is not None:
        _chk(a_rows, "gemm row gather", torch.int32)
    out_dtype = out_dtype or torch.bfloat16
    cols = N // 2 if swiglu else N          # swiglu: w rows are gate/up interleaved by 8, out = silu(gate) * up
    if out is None:
        out = torch.empty(M, cols, dtype=out_dtype, device=a.device)
    _chk(out, "gemm out", out_dtype, (M, cols))
    if out_dtype not in (torch.bfloat16, torch.float32) or (swiglu and out_dtype != torch.bfloat16):
        raise KernelError("gemm output is bfloat16 or float32 (bfloat16 with swiglu)")
    check(fn("snk_gemm_skinny")(_ptr(a), _ptr(w), _ptr(out), M, N, K, _ptr(a_rows), int(a_div), _ptr(offsets),
                                G, int(rows_hint if rows_hint is not None else M),
                                int(out_dtype == torch.float32), int(swiglu), _stream()), "gemm_skinny",
          work=lambda: _gemm_work(M, a, w, out, offsets))
    return out


TC_TILE = 128


def gemm_tc_ok(a, w) -> bool:
    """Whether the tcgen05 kernel takes these operands (bfloat16, K a multiple of 8, 16-byte aligned)."""
    return (a.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and a.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0)


def gemm_tc(a, w, out_dtype=None, out=None, offsets=None, swiglu=False):
    """bfloat16 a [M, K] times w [N, K]^T on the tcgen05 tensor cores, float accumulation in tensor
    memory.  Grouped: w [G, N, K], rows of ``a`` sorted by group, ``offsets`` int32 [G+1]."""
    _chk(a, "gemm a", torch.bfloat16)
    _chk(w, "gemm w", torch.bfloat16)
    M, K = a.shape
    grouped = offsets is not None
    if grouped:
        G, N, Kw = w.shape
        _chk(offsets, "group offsets", torch.int32, (G + 1,))
    else:
        G = 1
        N, Kw = w.shape
    if Kw != K:
        raise KernelError(f"gemm: a has K={K}, w has K={Kw}")
    out_dtype = out_dtype or torch.bfloat16
    cols = N // 2 if swiglu else N          # swiglu: w rows are gate/up interleaved by 8, out = silu(gate) * up
    if out is None:
        out = torch.empty(M, cols, dtype=out_dtype, device=a.device)
    _chk(out, "gemm out", out_dtype, (M, cols))
    if out_dtype not in (torch.bfloat16, torch.float32) or (swiglu and out_dtype != torch.bfloat16):
        raise KernelError("gemm output is bfloat16 or float32 (bfloat16 with swiglu)")
    row_tiles = -(-M // TC_TILE) + (G if grouped else 0)
    # few tiles: the product is split along K, and the parts' float planes need a place
    need = int(fn("snk_gemm_tc_scratch_bytes")(M, N, K, int(grouped)))
    scratch = torch.empty(need, dtype=torch.uint8, device=a.device) if need else None
    check(fn("snk_gemm_tc")(_ptr(a), _ptr(w), _ptr(out), M, N, K, _ptr(offsets), G, row_tiles,
                            int(out_dtype == torch.float32), int(swiglu), _ptr(scratch), _stream()), "gemm_tc",
          launches=2 if need else 1, work=lambda: _gemm_work(M, a, w, out, offsets))
    return out


def gemm_tc2(a, w, out_dtype=None, out=None, offsets=None, swiglu=False):
    """As ``gemm_tc``, on pairs of SMs (cta_group::2): 256 x 256 tiles of C, each block of a pair loading
    its 128 rows of ``a`` and half of the tile's rows of ``w``.  Grouped (``offsets``): the operands change
    places, each block loads 128 rows of the group's ``w`` and half of up to 256 of its rows of ``a``, and
    a group's last tile is as wide as its rows need (a multiple of 16); at most 256 groups."""
    _chk(a, "gemm a", torch.bfloat16)
    _chk(w, "gemm w", torch.bfloat16)
    M, K = a.shape
    grouped = offsets is not None
    if grouped:
        G, N, Kw = w.shape
        _chk(offsets, "group offsets", torch.int32, (G + 1,))
    else:
        G = 1
        N, Kw = w.shape
    if Kw != K:
        raise KernelError(f"gemm: a has K={K}, w has K={Kw}")
    out_dtype = out_dtype or torch.bfloat16
    cols = N // 2 if swiglu else N
    if out is None:
        out = torch.empty(M, cols, dtype=out_dtype, device=a.device)
    _chk(out, "gemm out", out_dtype, (M, cols))
    if out_dtype not in (torch.bfloat16, torch.float32) or (swiglu and out_dtype != torch.bfloat16):
        raise KernelError("gemm output is bfloat16 or float32 (bfloat16 with swiglu)")
    check(fn("snk_gemm_tc2")(_ptr(a), _ptr(w), _ptr(out), M, N, K, _ptr(offsets), G,
                             int(out_dtype == torch.float32), int(swiglu), _stream()), "gemm_tc2",
          work=lambda: _gemm_work(M, a, w, out, offsets))
    return out


def gemm_tc2_status():
    """(0 or the code of a wait that ran out inside the pair kernel since the last call, the tensor-memory
    addresses the two blocks of the first pair were given); synchronises the device."""
    addr = (ctypes.c_uint * 2)()
    return int(fn("snk_gemm_tc2_status")(addr)), (int(addr[0]), int(addr[1]))


def gemm_tc_is_split(M: int, N: int, K: int) -> bool:
    """Whether a plain tcgen05 product of these sizes is split along K (few tiles): its sums then have
    another order than the unsplit product's, so the same row may differ by rounding between the two."""
    return int(fn("snk_gemm_tc_scratch_bytes")(M, N, K, 0)) > 0


def gemm_tc_status() -> int:
    """0, or the code of a wait that ran out inside a tcgen05 kernel since the last call
    (synchronises the device; 1: operands never arrived, 2: a stage never came back, 3: the
    accumulator never became ready)."""
    return int(fn("snk_gemm_tc_status")())


def lose_loads(on: bool) -> None:
    """Test hook of the two tcgen05 product libraries: while on, their producers issue no loads, so the
    bounded waits inside the kernels run out and a launch returns with an error status (see
    ``gemm_tc_status``, ``gemm_tc2_status``, ``StatusWatch``) instead of a product."""
    check(fn("snk_gemm_tc_test_lose_loads")(int(on)), "gemm_tc test hook", 0)
    check(fn("snk_gemm_tc2_test_lose_loads")(int(on)), "gemm_tc2 test hook", 0)


def gather_rows(x, rows, div=1, out=None):
    """out[r] = x[rows[r] // div] for bfloat16 rows (the sorted copy the grouped tcgen05 product reads)."""
    _chk(x, "gather input", torch.bfloat16)
    _chk(rows, "gather rows", torch.int32)
    R, K = rows.numel(), x.shape[1]
    if out is None:
        out = torch.empty(R, K, dtype=x.dtype, device=x.device)
    _chk(out, "gather output", x.dtype, (R, K))
    check(fn("snk_gather_rows_bf16")(_ptr(x), _ptr(out), _ptr(rows), int(div), R, K, _stream()), "gather_rows",
          work=lambda: (2 * _nbytes(out), 0))
    return out


# --- routed experts --------------------------------------------------------------------

ROUTE_GEMM_MIN_ROWS = 64


def moe_route(x, router_w, bias, top_k, norm_topk_prob, scaling):
    """(ids int32 [M, k], weights float [M, k]) of the sigmoid router, computed in float."""
    M, H = x.shape
    dtype = x.dtype
    _chk(x, "router input", (torch.float32, torch.bfloat16))
    w32 = _small(router_w, "router weight", dtype)
    E = router_w.shape[0]
    _chk(router_w, "router weight", shape=(E, H))
    if bias is not None:
        _chk(bias, "expert bias", torch.float32, (E,))
    ids = torch.empty(M, top_k, dtype=torch.int32, device=x.device)
    wts = torch.empty(M, top_k, dtype=torch.float32, device=x.device)
    if (M > ROUTE_GEMM_MIN_ROWS and router_w.dtype == torch.bfloat16 and gemm_tc_ok(x, router_w)
            and gemm_tc_is_split(M, E, H)):
        # many rows, few experts: a tcgen05 product split along K (float accumulation, float output)
        # whose partial sums the selection adds itself, in the order the product's own sum has
        nbytes = int(fn("snk_gemm_tc_scratch_bytes")(M, E, H, 0))
        parts = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
        planes = ctypes.c_int(0)
        check(fn("snk_gemm_tc_parts")(_ptr(x), _ptr(router_w), _ptr(parts), M, E, H, ctypes.byref(planes),
                                      _stream()), "gemm_tc_parts",
              work=lambda: (_nbytes(x, router_w) + M * E * 4 * max(planes.value, 1), 2 * M * E * H))
        check(fn("snk_moe_topk")(_ptr(parts), _ptr(bias), _ptr(ids), _ptr(wts), M, E, top_k,
                                 int(bool(norm_topk_prob)), float(scaling), 0, planes.value, _stream()), "moe_topk")
        return ids, wts
    if M > ROUTE_GEMM_MIN_ROWS and router_w.dtype == torch.bfloat16 and gemm_skinny_ok(router_w, x):
        # many rows: the logits are a tensor-core product with float accumulation and float output.  The few
        # router rows take the place of the tokens in the few-rows kernel, which then streams x once and
        # leaves the logits transposed, [E, M].
        logits = gemm_skinny(router_w, x, out_dtype=torch.float32, rows_hint=min(E, 64))
        check(fn("snk_moe_topk")(_ptr(logits), _ptr(bias), _ptr(ids), _ptr(wts), M, E, top_k,
                                 int(bool(norm_topk_prob)), float(scaling), 1, 1, _stream()), "moe_topk")
        return ids, wts
    check(fn("snk_moe_route")(_ptr(x), _ptr(router_w), w32, _ptr(bias), _ptr(ids), _ptr(wts), M, H, E,
                              top_k, int(bool(norm_topk_prob)), float(scaling), code_of(dtype), _stream()),
          "moe_route", work=lambda: (_nbytes(x, router_w, ids, wts), 2 * M * E * H))
    return ids, wts


ROUTE_FUSED_MAX_ROWS = 32      # up to here: logits spread over the GPU, selection and sort in one block


def moe_route_sort(x, router_w, bias, top_k, norm_topk_prob, scaling):
    """Routing and the sort by expert together: (ids, weights, offsets, pair_pos, sorted_pair) as
    `moe_route` and `moe_sort` give them.  The few rows of a decode step take two launches made for
    them; a row's logits are the same numbers on every path but the tensor-core one."""
    M, H = x.shape
    E = router_w.shape[0]
    if M > ROUTE_FUSED_MAX_ROWS or 8 * E * min(M, 32) + 8 * M * top_k > 48 * 1024:
        ids, wts = moe_route(x, router_w, bias, top_k, norm_topk_prob, scaling)
        return (ids, wts) + moe_sort(ids, E)
    dtype = x.dtype
    _chk(x, "router input", (torch.float32, torch.bfloat16))
    w32 = _small(router_w, "router weight", dtype)
    _chk(router_w, "router weight", shape=(E, H))
    if bias is not None:
        _chk(bias, "expert bias", torch.float32, (E,))
    dev = x.device
    ints = torch.empty(M * top_k * 3 + E + 1, dtype=torch.int32, device=dev)
    floats = torch.empty(M * E + M * top_k, dtype=torch.float32, device=dev)
    pairs = M * top_k
    ids, pair_pos, sorted_pair = ints[:pairs].view(M, top_k), ints[pairs:2 * pairs], ints[2 * pairs:3 * pairs]
    offsets = ints[3 * pairs:]
    logits, wts = floats[:M * E], floats[M * E:].view(M, top_k)
    check(fn("snk_moe_route_sort")(_ptr(x), _ptr(router_w), w32, _ptr(bias), _ptr(logits), _ptr(ids), _ptr(wts),
                                   _ptr(offsets), _ptr(pair_pos), _ptr(sorted_pair), M, H, E, top_k,
                                   int(bool(norm_topk_prob)), float(scaling), code_of(dtype), _stream()),
          "moe_route_sort", launches=2, work=lambda: (_nbytes(x, router_w, ints, floats), 2 * M * E * H))
    return ids, wts, offsets, pair_pos, sorted_pair


NORM_ROUTE_MAX_ROWS = 32
# Off by default: measured in the decode step of the 8B-A1B sizes it gains nothing (batch 1: 1.488 ms against
# 1.471 ms with the three launches it replaces; batch 8: 3.012 against 2.966 ms).  Inside a captured step the
# three launches hide one another's start, and one block per row walks norm, 32 dot products, selection and
# sort one after the other (12.4 us against 3.3 + 4.2 + 5.4 us).
FUSE_ROUTER = os.environ.get("SNOWLLM_B200_FUSE_ROUTER", "0") != "0"


def norm_route_sort_ok(residual, delta, gamma, router_w, top_k) -> bool:
    """Whether the one-launch front of a routed feed-forward (csrc/moe.cu: norm_route_sort_kernel) takes these
    operands (the switch ``FUSE_ROUTER`` is the caller's business)."""
    M, H = residual.shape
    E = router_w.shape[0]
    plain = delta is None or isinstance(delta, ExpertSum) or (torch.is_tensor(delta) and delta.data_ptr() % 16 == 0)
    return (M <= NORM_ROUTE_MAX_ROWS and H % 4 == 0 and H <= 32768 and top_k <= 32 and plain
            and residual.data_ptr() % 16 == 0 and (max(H, 2 * E + 4) + 40 + 2 * E) * 4 <= 200 * 1024)


def norm_route_sort(residual, delta, gamma, eps, dtype, router_w, bias, top_k, norm_topk_prob, scaling, ticket):
    """``residual += delta`` (a float tensor, an ``ExpertSum`` or None), RMSNorm into ``dtype``, the sigmoid
    router on the normalised rows, and the sort of the (token, pick) pairs by expert, in one launch for the
    few rows of a decode step: (x, ids, weights, offsets, pair_pos, sorted_pair), the same values as
    ``add_rmsnorm`` followed by ``moe_route_sort`` give.  ``ticket``: one int32 on the device, zero before
    the first call; the kernel leaves it zero."""
    M, H = residual.shape
    E = router_w.shape[0]
    _chk(residual, "residual", torch.float32)
    moe = None
    if isinstance(delta, ExpertSum):
        moe, delta = delta, None
        _chk(moe.y, "expert outputs", torch.float32)
        _chk(moe.pair_pos, "pair positions", torch.int32, (M * moe.weights.shape[1],))
        _chk(moe.weights, "top-k weights", torch.float32)
    if delta is not None:
        _chk(delta, "residual delta", torch.float32, (M, H))
    g32 = _small(gamma, "norm weight", dtype)
    _chk(gamma, "norm weight", shape=(H,))
    w32 = _small(router_w, "router weight", dtype)
    _chk(router_w, "router weight", shape=(E, H))
    if bias is not None:
        _chk(bias, "expert bias", torch.float32, (E,))
    _chk(ticket, "ticket", torch.int32, (1,))
    dev = residual.device
    x = torch.empty(M, H, dtype=dtype, device=dev)
    pairs = M * top_k
    ints = torch.empty(pairs * 3 + E + 1, dtype=torch.int32, device=dev)
    wts = torch.empty(M, top_k, dtype=torch.float32, device=dev)
    ids, pair_pos, sorted_pair = ints[:pairs].view(M, top_k), ints[pairs:2 * pairs], ints[2 * pairs:3 * pairs]
    offsets = ints[3 * pairs:]
    check(fn("snk_norm_route_sort")(
        _ptr(residual), _ptr(delta), _ptr(gamma), g32, _ptr(x), H, float(eps), _ptr(moe.y if moe else None),
        _ptr(moe.pair_pos if moe else None), _ptr(moe.weights if moe else None), moe.weights.shape[1] if moe else 0,
        _ptr(router_w), w32, _ptr(bias), _ptr(ids), _ptr(wts), _ptr(offsets), _ptr(pair_pos), _ptr(sorted_pair),
        M, E, top_k, int(bool(norm_topk_prob)), float(scaling), code_of(dtype), _ptr(ticket), _stream()),
        "norm_route_sort",
        work=lambda: (2 * M * H * 4 + _nbytes(x, router_w, ints, wts) + (_nbytes(delta) if delta is not None else 0)
                      + (moe.weights.shape[1] * M * H * 4 if moe else 0), 2 * M * E * H))
    return x, ids, wts, offsets, pair_pos, sorted_pair


def moe_sort(topk_ids, num_experts):
    """(offsets int32 [E+1], pair_pos int32 [M*k], sorted_pair int32 [M*k]) of the pairs sorted by
    expert."""
    _chk(topk_ids, "top-k ids", torch.int32)
    pairs = topk_ids.numel()
    dev = topk_ids.device
    offsets = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
    pair_pos = torch.empty(pairs, dtype=torch.int32, device=dev)
    sorted_pair = torch.empty(pairs, dtype=torch.int32, device=dev)
    check(fn("snk_moe_sort")(_ptr(topk_ids), _ptr(offsets), _ptr(pair_pos), _ptr(sorted_pair), pairs,
                             num_experts, _stream()), "moe_sort")
    return offsets, pair_pos, sorted_pair


def moe_combine(y, pair_pos, topk_w, out=None):
    """out[m] = sum_j w[m, j] * y[pair_pos[m*k + j]] in float, j in order."""
    M, k = topk_w.shape
    H = y.shape[1]
    _chk(y, "expert outputs", torch.float32, (M * k, H))
    _chk(pair_pos, "pair positions", torch.int32, (M * k,))
    _chk(topk_w, "top-k weights", torch.float32)
    if out is None:
        out = torch.empty(M, H, dtype=torch.float32, device=y.device)
    _chk(out, "moe output", torch.float32, (M, H))
    check(fn("snk_moe_combine")(_ptr(y), _ptr(pair_pos), _ptr(topk_w), _ptr(out), M, H, k, _stream()),
          "moe_combine")
    return out


# --- sampling --------------------------------------------------------------------------

def argmax(logits, out=None):
    B, V = logits.shape
    _chk(logits, "logits", torch.float32)
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
    _chk(out, "argmax output", torch.int32, (B,))
    check(fn("snk_argmax")(_ptr(logits), _ptr(out), B, V, _stream()), "argmax", work=lambda: (_nbytes(logits), 0))
    return out


def apply_penalties(logits, row_offsets, ids, counts, presence, frequency, repetition):
    B, V = logits.shape
    _chk(logits, "logits", torch.float32)
    _chk(row_offsets, "penalty offsets", torch.int32, (B + 1,))
    _chk(ids, "penalty ids", torch.int32)
    _chk(counts, "penalty counts", torch.int32, ids.shape)
    for t, what in ((presence, "presence"), (frequency, "frequency"), (repetition, "repetition")):
        _chk(t, what + " penalty", torch.float32, (B,))
    check(fn("snk_apply_penalties")(_ptr(logits), _ptr(row_offsets), _ptr(ids), _ptr(counts), _ptr(presence),
                                    _ptr(frequency), _ptr(repetition), B, V, _stream()), "apply_penalties")


def sample(logits, temperature, top_k, top_p, uniform, out=None):
    B, V = logits.shape
    _chk(logits, "logits", torch.float32)
    _chk(temperature, "temperature", torch.float32, (B,))
    _chk(top_k, "top_k", torch.int32, (B,))
    _chk(top_p, "top_p", torch.float32, (B,))
    _chk(uniform, "uniform", torch.float32, (B,))
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
    _chk(out, "sample output", torch.int32, (B,))
    check(fn("snk_sample")(_ptr(logits), _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(uniform),
                           _ptr(out), B, V, _stream()), "sample", work=lambda: (_nbytes(logits), 0))
    return out
