"""Stand-alone entmax through the operator API against the CPU oracle; mirrors the structure
of the reference's tests/test_triton_entmax.py (oracle: converged bisection, float64)."""
import pytest
import torch

from adasplash.triton_entmax import triton_entmax
from oracle import entmax_bwd_ref, entmax_ref

pytestmark = pytest.mark.gpu
ALPHAS = [1.1, 1.333, 1.5, 1.666, 2.0]


@pytest.mark.parametrize("shape", [(2,), (2, 4), (2, 4, 8), (2, 4, 8, 16), (3, 300), (2, 1500), (2, 5000), (1, 20000)])
@pytest.mark.parametrize("alpha", ALPHAS)
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.bfloat16])
@pytest.mark.parametrize("fast_math", [False, True])
def test_forward_correctness(shape, alpha, dtype, fast_math):
    torch.manual_seed(42)
    atol = 1e-4 if dtype == torch.float32 else 1e-2     # reference tolerances (:16)
    x = torch.randn(*shape, dtype=dtype)
    ref = entmax_ref(x.float(), alpha)
    out = triton_entmax(x.cuda(), alpha=alpha, fast_math=fast_math)
    assert out.dtype == dtype and out.shape == x.shape
    assert torch.allclose(out.cpu().double(), ref, atol=atol), (out.cpu().double() - ref).abs().max()


@pytest.mark.parametrize("shape", [(37, 40), (37, 48), (21, 64), (13, 128), (29, 200), (9, 256), (11, 512), (5, 1024)])
@pytest.mark.parametrize("alpha", [1.333, 1.5, 2.0])
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.bfloat16])
def test_short_rows_sharing_a_warp(shape, alpha, dtype):
    """Rows of up to 512 values share a warp (4, 8 or 16 lanes each); the row counts here leave the last
    warp partly filled, and rows with very different scales sit side by side in one warp."""
    g = torch.Generator().manual_seed(shape[0] * 1000 + shape[1])
    x = torch.randn(*shape, generator=g) * torch.logspace(-1, 1, shape[0]).unsqueeze(1)
    x = x.to(dtype)
    atol = 1e-4 if dtype == torch.float32 else 1e-2
    ref = entmax_ref(x.float(), alpha)
    xg = x.cuda().requires_grad_(True)
    out = triton_entmax(xg, alpha=alpha)
    assert torch.allclose(out.detach().cpu().double(), ref, atol=atol), (out.detach().cpu().double() - ref).abs().max()
    assert torch.allclose(out.detach().float().sum(-1).cpu(), torch.ones(shape[0]),
                          atol=2e-2 if dtype != torch.float32 else 1e-4)
    # backward of the same shapes (rows share a warp there too), from the output the kernel itself produced
    dy = torch.randn(*shape, generator=g).to(dtype)
    out.backward(dy.cuda())
    gref = entmax_bwd_ref(out.detach().cpu().double(), dy.double(), alpha)
    gtol = 1e-4 if dtype == torch.float32 else 2e-2
    assert torch.allclose(xg.grad.cpu().double(), gref, atol=gtol, rtol=gtol), (xg.grad.cpu().double() - gref).abs().max()


@pytest.mark.parametrize("shape", [(2,), (2, 4), (2, 4, 8)])
@pytest.mark.parametrize("alpha", ALPHAS)
def test_backward_gradcheck(shape, alpha):
    torch.manual_seed(42)
    x = torch.randn(*shape, device="cuda", dtype=torch.float32, requires_grad=True)
    assert torch.autograd.gradcheck(lambda t: triton_entmax(t, alpha, 10, True), x, atol=1e-2, eps=1e-4,
                                    nondet_tol=1e-5)


@pytest.mark.parametrize("alpha", ALPHAS)
@pytest.mark.parametrize("cols", [33, 700, 3000])
def test_backward_matches_oracle(alpha, cols):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(5, cols, generator=g)
    dy = torch.randn(5, cols, generator=g)
    xg = x.cuda().requires_grad_(True)
    y = triton_entmax(xg, alpha)
    y.backward(dy.cuda())
    ref = entmax_bwd_ref(entmax_ref(x, alpha), dy.double(), alpha)
    assert torch.allclose(xg.grad.cpu().double(), ref, atol=1e-4), (xg.grad.cpu().double() - ref).abs().max()


@pytest.mark.parametrize("cols", [12000, 20000, 50000, 100000])
@pytest.mark.parametrize("alpha", [1.5, 2.0, 1.333])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_long_rows_owned_by_a_cluster(cols, alpha, dtype):
    """Rows beyond one block's register tile are spread over 2, 4 or 8 blocks of a cluster that exchange
    their partial sums through distributed shared memory; forward and backward against the oracle."""
    g = torch.Generator().manual_seed(cols)
    x = (torch.randn(3, cols, generator=g) * torch.tensor([[0.3], [1.0], [4.0]])).to(dtype)
    dy = torch.randn(3, cols, generator=g).to(dtype)
    xg = x.cuda().requires_grad_(True)
    y = triton_entmax(xg, alpha)
    y.backward(dy.cuda())
    torch.cuda.synchronize()
    p_ref = entmax_ref(x.float(), alpha)
    tol = 1e-4 if dtype == torch.float32 else 1e-2
    assert torch.allclose(y.detach().cpu().double(), p_ref, atol=tol), (y.detach().cpu().double() - p_ref).abs().max()
    ref = entmax_bwd_ref(p_ref, dy.double(), alpha)
    assert torch.allclose(xg.grad.cpu().double(), ref, atol=tol, rtol=tol), (xg.grad.cpu().double() - ref).abs().max()


@pytest.mark.parametrize("alpha", ALPHAS)
def test_numerical_stability(alpha):
    for shape in [(2,), (2, 5), (2, 4, 8)]:
        x = (torch.randn(*shape, device="cuda") * 100).requires_grad_(True)
        y = triton_entmax(x, alpha=alpha)
        assert torch.isfinite(y).all() and (y >= 0).all()
        assert torch.allclose(y.sum(-1), torch.ones(y.shape[:-1], device="cuda"), atol=1e-2)
        y.sum().backward()
        assert torch.isfinite(x.grad).all()


@pytest.mark.parametrize("alpha", [1.333, 1.5, 1.666, 2.0])
def test_edge_cases(alpha):
    for x in (torch.zeros(64, device="cuda"), torch.full((64,), 1e3, device="cuda")):
        y = triton_entmax(x, alpha=alpha)
        assert torch.allclose(y, torch.full_like(y, 1 / 64), atol=1e-2)
    x = torch.zeros(64, device="cuda")
    x[0] = 100
    y = triton_entmax(x, alpha=alpha)
    assert torch.allclose(y, torch.eye(64, device="cuda")[0], atol=1e-2)


@pytest.mark.parametrize("dim", [0, 1, 2])
def test_different_dimensions(dim):
    torch.manual_seed(0)
    x = torch.randn(32, 32, 32)
    ref = entmax_ref(x, 1.5, dim=dim)
    perm = {0: (1, 2, 0), 1: (0, 2, 1), 2: (0, 1, 2)}[dim]
    inv = {0: (2, 0, 1), 1: (0, 2, 1), 2: (0, 1, 2)}[dim]
    out = triton_entmax(x.cuda().permute(perm).contiguous(), alpha=1.5).permute(inv)
    assert torch.allclose(out.cpu().double(), ref, rtol=1e-4, atol=1e-5)


def test_run_to_run_determinism_and_autograd():
    x = torch.randn(4, 8, device="cuda", requires_grad=True)
    for fm in (False, True):
        assert torch.equal(triton_entmax(x, fast_math=fm), triton_entmax(x, fast_math=fm))
    y = triton_entmax(x, alpha=1.5)
    y.sum().backward()
    assert x.grad is not None and torch.isfinite(x.grad).all() and x.grad.abs().max() < 1e3


@pytest.mark.parametrize("dtype,cols", [(torch.bfloat16, 16384), (torch.float32, 16384), (torch.bfloat16, 65536)])
def test_thousands_of_long_rows_owned_by_clusters(dtype, cols):
    """Far more clusters than the GPU can hold at once: blocks of one cluster start at different times, and a
    block may write into a sibling's shared memory only after the sibling has started."""
    rows = 2048 if cols == 16384 else 512
    g = torch.Generator().manual_seed(3)
    x = torch.randn(rows, cols, generator=g).to(dtype)
    dy = torch.randn(rows, cols, generator=g).to(dtype)
    xg = x.cuda().requires_grad_(True)
    y = triton_entmax(xg, alpha=1.5)
    y.backward(dy.cuda())
    ref = entmax_ref(x.float(), 1.5, work_dtype=torch.float32)
    tol = 1e-4 if dtype == torch.float32 else 1e-2
    assert float((y.detach().cpu().float() - ref).abs().max()) <= tol
    # (backward from the output the kernel itself produced, as in the other cases of this file)
    dref = entmax_bwd_ref(y.detach().cpu().double(), dy.double(), 1.5)
    gtol = 1e-4 if dtype == torch.float32 else 2e-2
    assert torch.allclose(xg.grad.cpu().double(), dref, atol=gtol, rtol=gtol)
