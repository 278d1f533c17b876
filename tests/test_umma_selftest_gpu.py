"""Self test of the tcgen05 / TMEM / TMA building blocks through the C ABI: one tile product
per operand layout, compared with an fp32 matmul of the same bf16 inputs."""
import pytest
import torch

from flash_lazy_attention_b200 import _lib

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("variant", [0, 1, 2])
def test_tile_product(variant):
    lib = _lib.load()
    g = torch.Generator().manual_seed(variant)
    a = torch.randn(128, 128, generator=g).bfloat16().cuda()
    b = torch.randn(128, 128, generator=g).bfloat16().cuda()
    c = torch.full((128, 128), float("nan"), device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    rc = lib.fla_selftest_umma(a.data_ptr(), b.data_ptr(), c.data_ptr(), variant, status.data_ptr(),
                               torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "fla_selftest_umma")
    torch.cuda.synchronize()
    assert status[0].item() == 0, f"bounded wait ran out: {status.tolist()}"
    ref = a.float() @ (b.float() if variant == 1 else b.float().t())
    err = (c - ref).abs().max().item()
    assert err < 1e-3, err


def test_expired_wait_is_reported_and_the_context_stays_usable():
    """Variant 3 waits (a few thousand polls) on a barrier nothing arrives on.  The kernel must return
    normally with the status words set, fla_check_status must turn them into FLA_ERR_DEVICE, and the
    next launch on the same context must work (tensor memory was freed)."""
    lib = _lib.load()
    a = torch.zeros(128, 128, dtype=torch.bfloat16, device="cuda")
    c = torch.full((128, 128), float("nan"), device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.fla_selftest_umma(a.data_ptr(), a.data_ptr(), c.data_ptr(), 3, status.data_ptr(), stream),
               "fla_selftest_umma")
    rc = lib.fla_check_status(status.data_ptr(), stream)
    assert rc == 4, rc                                    # FLA_ERR_DEVICE
    assert b"bounded wait" in lib.fla_last_error()
    assert status[0].item() == 1 and status[1].item() == 1   # the first wait of the kernel (tag 1)
    assert (c == 0).all()
    test_tile_product(0)                                  # the context and the tensor memory are intact
