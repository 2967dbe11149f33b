"""The attention entry point that allocates nothing (csrc/attention_static.h), called the way its
users call it: through the exported C symbol of the built library, with raw device pointers.

Those users are programs that must not allocate device memory while they run: a plugin whose host owns
the GPU's memory, a loop with a latency bound, a process at its memory limit, a C caller without a
tensor library.  The test checks that the entry point gives the regular entry point's result on two
calls in a row (the second call finds the first call's leftovers in the shared scratch array), that it
refuses a call that would not fit, and that no device memory is allocated while it runs.  The file name
makes pytest collect it last."""
import ctypes
import gc

import pytest
import torch

pytestmark = pytest.mark.gpu

ERR_STATIC_SCRATCH = 20010
STATIC_BYTES = 8 << 20


def library():
    from snowllm_b200.csrc import build
    lib = ctypes.CDLL(str(build.build(("attention",))[0]))
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.snk_paged_attention_static.argtypes = [P, P, P, I, I, P, P, P, I, I, I, I, I, I, I, F, I, P]
    lib.snk_paged_attention_static.restype = I
    lib.snk_paged_attention_static_need.argtypes = [I, I, I, I]
    lib.snk_paged_attention_static_need.restype = ctypes.c_longlong
    return lib


def make_case(dtype, seed):
    """Two decoding rows and a short prompt portion over scattered pages, long enough to need chunks."""
    torch.manual_seed(seed)
    nh, nkv, hd, P, chunk = 8, 2, 64, 16, 256
    lens = [1500, 700, 40]
    rows = [[1499], [699], list(range(30, 40))]
    pages = sum(-(-n // P) for n in lens)
    perm = torch.randperm(pages).tolist()
    pool = torch.randn(pages, 2, nkv, P, hd, device="cuda").to(dtype)
    tables = []
    for n in lens:
        need = -(-n // P)
        tables.append(perm[:need])
        perm = perm[need:]
    width = max(len(t) for t in tables)
    bt = torch.tensor([t + [0] * (width - len(t)) for t in tables], dtype=torch.int32, device="cuda")
    positions = torch.tensor(sum(rows, []), dtype=torch.int32, device="cuda")
    row_seg = torch.tensor(sum(([b] * len(r) for b, r in enumerate(rows)), []), dtype=torch.int32, device="cuda")
    q = torch.randn(len(positions), nh, hd, device="cuda").to(dtype)
    n_chunks = max(p // chunk for p in sum(rows, [])) + 1
    return dict(q=q, pool=pool, bt=bt, positions=positions, row_seg=row_seg, P=P, chunk=chunk, n_chunks=n_chunks,
                nh=nh, nkv=nkv, hd=hd)


def call_static(lib, c, out, dtype):
    return lib.snk_paged_attention_static(
        c["q"].data_ptr(), c["pool"].data_ptr(), c["bt"].data_ptr(), c["bt"].shape[1], c["P"],
        c["positions"].data_ptr(), c["row_seg"].data_ptr(), out.data_ptr(), c["q"].shape[0], c["nh"], c["nkv"],
        c["hd"], 0, c["chunk"], c["n_chunks"], c["hd"] ** -0.5, 0 if dtype == torch.float32 else 1,
        torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_entry_matches_the_regular_one_twice_in_a_row(dtype):
    from snowllm_b200.ops import kernels
    lib = library()
    first = True
    for seed in (1, 2):                               # the second call reuses the array the first one filled
        c = make_case(dtype, seed)
        want = kernels.paged_attention(c["q"], c["pool"], c["bt"], c["P"], c["positions"], c["row_seg"],
                                       c["hd"] ** -0.5, chunk=c["chunk"], num_chunks=c["n_chunks"])
        out = torch.full_like(want, float("nan"))
        need = lib.snk_paged_attention_static_need(c["q"].shape[0], c["nh"], c["hd"], c["n_chunks"])
        assert 0 < need <= STATIC_BYTES
        if first:                                     # set-up call: looks up the array's address on this device
            assert call_static(lib, c, out, dtype) == 0
            first = False
        # Nothing may be taken from the device during the call.  Tensors that earlier tests left behind can be
        # collected at any moment (and give memory back), so they are collected now, and the check is one-sided.
        gc.collect()
        torch.cuda.synchronize()
        allocated, free = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        assert call_static(lib, c, out, dtype) == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() <= allocated and torch.cuda.mem_get_info()[0] >= free, \
            "the call took device memory"
        assert out.isfinite().all()
        assert torch.equal(out, want)                     # the same kernels run on the same inputs: the same bits


def test_static_entry_refuses_what_does_not_fit():
    lib = library()
    c = make_case(torch.float32, 3)
    out = torch.zeros(c["q"].shape[0], c["nh"] * c["hd"], device="cuda")
    too_many = 100000                                 # chunks: the partial results would need far more than 8 MiB
    assert lib.snk_paged_attention_static_need(c["q"].shape[0], c["nh"], c["hd"], too_many) > STATIC_BYTES
    c["n_chunks"] = too_many
    assert call_static(lib, c, out, torch.float32) == ERR_STATIC_SCRATCH
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0              # nothing ran
