"""A bounded wait inside a kernel that runs out: the launch returns, the status word says so, the host
surfaces it as KernelError, and the device goes on working.  The failure is made without a fault: a test
hook makes the TMA producers of the tcgen05 products issue no loads, so the waits for operands run out
(about 1.5 s a launch)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def operands(rows, n, k):
    gen = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(rows, k, device="cuda", generator=gen).to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda", generator=gen) * k ** -0.5).to(torch.bfloat16)
    return x, w


def agrees(out, x, w):
    ref = x.float() @ w.float().T
    return bool(((out.float() - ref).abs() <= 2e-2 * ref.abs().max()).all())


@pytest.mark.parametrize("product", ["gemm_tc", "gemm_tc2"])
def test_wait_that_runs_out_is_reported_and_the_device_stays_usable(product):
    from snowllm_b200.errors import KernelError
    from snowllm_b200.ops import kernels
    run = getattr(kernels, product)
    status = (lambda: kernels.gemm_tc_status()) if product == "gemm_tc" else (lambda: kernels.gemm_tc2_status()[0])
    x, w = operands(512, 512, 256)
    assert agrees(run(x, w), x, w) and status() == 0
    watch = kernels.StatusWatch()
    kernels.lose_loads(True)
    try:
        run(x, w)                                    # returns after the waits have run out: no product
        watch.peek()
        torch.cuda.synchronize()
    finally:
        kernels.lose_loads(False)
    with pytest.raises(KernelError, match=f"bounded wait ran out.*{product} "):
        watch.check()                                # names the library; clears the word on the device
    assert status() == 0
    watch.peek()
    torch.cuda.synchronize()
    watch.check()                                    # nothing is left over
    assert agrees(run(x, w), x, w) and status() == 0  # the same context still computes


def test_grouped_product_gives_up_cleanly_too():
    from snowllm_b200.ops import kernels
    x, _ = operands(96, 8, 128)
    gen = torch.Generator(device="cuda").manual_seed(6)
    w = (torch.randn(3, 64, 128, device="cuda", generator=gen) * 128 ** -0.5).to(torch.bfloat16)
    offsets = torch.tensor([0, 40, 40, 96], dtype=torch.int32, device="cuda")
    kernels.lose_loads(True)
    try:
        kernels.gemm_tc2(x, w, offsets=offsets)
        torch.cuda.synchronize()
    finally:
        kernels.lose_loads(False)
    assert kernels.gemm_tc2_status()[0] != 0 and kernels.gemm_tc2_status()[0] == 0       # set once, cleared by the read
    out = kernels.gemm_tc2(x, w, offsets=offsets).float()
    for g, (a, b) in enumerate([(0, 40), (40, 40), (40, 96)]):
        if b > a:                                    # the middle group owns no rows
            ref = x[a:b].float() @ w[g].float().T
            assert (out[a:b] - ref).abs().max() <= 2e-2 * float(ref.abs().max())
