"""The torch.library custom ops on the GPU: torch.library.opcheck (schema, fake implementation against the real
outputs, autograd registration, AOT dispatch) and compiled forward + backward against the eager operators."""
import pytest
import torch

import flash_lazy_attention_b200 as fla
from flash_lazy_attention_b200 import check_status, set_flags, set_path

from gpu_util import maxdiff, randn

pytestmark = pytest.mark.gpu

CHECKS = ("test_schema", "test_faketensor", "test_autograd_registration", "test_aot_dispatch_dynamic")


@pytest.fixture(autouse=True)
def _reset():
    set_path(None)
    set_flags(0)
    torch._dynamo.reset()
    yield
    check_status()


@pytest.mark.parametrize("dtype,D", [(torch.bfloat16, 128), (torch.float32, 32)])
def test_opcheck_entmax_attention(dtype, D):
    q, k, v = (randn((1, 2, 200, D), dtype, s).requires_grad_(True) for s in (1, 2, 3))
    varlen = torch.tensor([150], device="cuda")
    for args in ((q, k, v, 1.5, 10, True, None, True), (q, k, v, 2.0, 10, False, varlen, False)):
        torch.library.opcheck(torch.ops.flash_lazy.entmax_attn_fwd.default, args, test_utils=CHECKS)


def test_opcheck_lazy_attention_and_rows():
    q, k, v = (randn((1, 2, 200, 64), torch.bfloat16, s).requires_grad_(True) for s in (1, 2, 3))
    bias = (torch.randn(2, 32, device="cuda") * 0.02).requires_grad_(True)
    tau = torch.full((2,), -1.0, device="cuda", requires_grad=True)
    torch.library.opcheck(torch.ops.flash_lazy.lazy_attn_fwd.default, (q, k, v, bias, tau, 32, None), test_utils=CHECKS)
    x = torch.randn(16, 300, device="cuda", requires_grad=True)
    torch.library.opcheck(torch.ops.flash_lazy.entmax_rows_fwd.default, (x, 1.5, 10, True), test_utils=CHECKS)


def _grads(fn, leaves, do):
    leaves = [t.detach().clone().requires_grad_(True) for t in leaves]
    out = fn(*leaves)
    out.backward(do)
    return [out.detach()] + [t.grad for t in leaves]


@pytest.mark.parametrize("dtype,D,Hkv", [(torch.bfloat16, 128, 4), (torch.bfloat16, 64, 2), (torch.float32, 32, 4)])
def test_compiled_entmax_attention_equals_eager(dtype, D, Hkv):
    B, H, L = 2, 4, 300
    q, do = randn((B, H, L, D), dtype, 1), randn((B, H, L, D), dtype, 4)
    k, v = randn((B, Hkv, L, D), dtype, 2), randn((B, Hkv, L, D), dtype, 3)
    varlen = torch.tensor([300, 211], device="cuda")

    def f(a, b, c):
        return fla.adasplash(a * 1.0, b, c, alpha=1.5, is_causal=True, varlen=varlen)

    eager = _grads(f, (q, k, v), do)
    compiled = _grads(torch.compile(f, backend="aot_eager", fullgraph=True), (q, k, v), do)
    for name, a, b in zip(("out", "dq", "dk", "dv"), eager, compiled):
        assert torch.equal(a, b), (name, maxdiff(a, b))


def test_compiled_lazy_attention_and_rows_equal_eager():
    B, H, L, D, W = 2, 4, 300, 128, 64
    q, k, v, do = (randn((B, H, L, D), torch.bfloat16, s) for s in (1, 2, 3, 4))
    bias = torch.randn(H, W, device="cuda") * 0.02
    tau = torch.full((H,), -1.0, device="cuda")

    def f(a, b, c, d, e):
        return fla.lazy_attention_triton(a, b, c, d, e, window_size=W)

    eager = _grads(f, (q, k, v, bias, tau), do)
    compiled = _grads(torch.compile(f, backend="aot_eager", fullgraph=True), (q, k, v, bias, tau), do)
    for name, a, b in zip(("out", "dq", "dk", "dv", "dbias", "dtau"), eager, compiled):
        assert torch.equal(a, b), (name, maxdiff(a, b))

    x, dy = torch.randn(64, 1000, device="cuda"), torch.randn(64, 1000, device="cuda")
    g = lambda t: fla.triton_entmax(t, alpha=1.5)     # noqa: E731
    eager = _grads(g, (x,), dy)
    compiled = _grads(torch.compile(g, backend="aot_eager", fullgraph=True), (x,), dy)
    for a, b in zip(eager, compiled):
        assert torch.equal(a, b)
