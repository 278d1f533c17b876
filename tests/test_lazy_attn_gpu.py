"""Lazy Attention through the operator API: against fixtures produced by the reference's own
kernels, against the dense oracle, and the behaviours the reference's tests pin."""
import numpy as np
import pytest
import torch

from adasplash.lazy_attention_triton import lazy_attention_triton
from flash_lazy_attention_b200 import check_status, last_call_info, set_path
from oracle import lazy_attention_grads_analytic

from gpu_util import close, maxdiff, randn, round_to

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _auto_path():
    set_path(None)
    yield
    set_path(None)
    check_status()      # no tensor-core kernel may have reported an expired wait


def _run(q, k, v, bias, tau, do, W, varlen, train=True):
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
    leaves += [t.clone().requires_grad_(train) for t in (bias, tau)]
    out = lazy_attention_triton(*leaves, window_size=W, varlen=varlen)
    out.backward(do)
    return [out.detach()] + [l.grad for l in leaves]


@pytest.mark.parametrize("name", ["plain", "varlen", "wide_window_pos_tau", "extra_bias_cols"])
def test_matches_reference_kernels(lazy_golden, name):
    c = lazy_golden[name]
    cu = {k_: torch.from_numpy(np.asarray(val)).cuda() for k_, val in c.items()}
    vl = cu["varlen"] if c["varlen"].size else None
    train = bool(int(c["trained_params"]))
    res = _run(cu["q"], cu["k"], cu["v"], cu["bias"], cu["tau"], cu["do"], int(c["window"]), vl, train)
    names = ["out", "dq", "dk", "dv"] + (["dbias", "dtau"] if train else [])
    for nm, mine in zip(["out", "dq", "dk", "dv", "dbias", "dtau"], res):
        if nm in names:
            # fp32 on both sides; the reference's own tests use atol = rtol = 1e-2
            assert torch.allclose(mine.cpu(), torch.from_numpy(c[nm]), atol=5e-4, rtol=1e-3), (name, nm, maxdiff(mine, torch.from_numpy(c[nm])))
    if not train:
        assert res[4] is None and res[5] is None


@pytest.mark.parametrize("path", ["simt", "auto"])
@pytest.mark.parametrize("dtype,D,tol", [(torch.float32, 64, 1e-3), (torch.bfloat16, 64, 2e-2), (torch.bfloat16, 128, 2e-2),
                                         (torch.float16, 128, 2e-2), (torch.float32, 16, 1e-3)])
@pytest.mark.parametrize("L,W,varlen", [(128, 32, None), (300, 64, [300, 131]), (512, 512, None), (257, 1000, [200, 257])])
def test_against_dense_oracle(path, dtype, D, tol, L, W, varlen):
    set_path(path)
    B, H = 2, 3
    q, k, v, do = (randn((B, H, L, D), dtype, s) for s in (1, 2, 3, 4))
    bias = randn((H, W), torch.float32, 5, scale=0.3)
    tau = torch.tensor([-1.0, 0.3, -4.0], device="cuda")
    vl = None if varlen is None else torch.tensor(varlen, dtype=torch.int32, device="cuda")
    res = _run(q, k, v, bias, tau, do, W, vl)
    ref = lazy_attention_grads_analytic(q.cpu(), k.cpu(), v.cpu(), bias.cpu(), tau.cpu(), do.cpu(), W,
                                        None if vl is None else vl.cpu(), round_to=round_to(dtype))
    for nm, mine, r in zip(["out", "dq", "dk", "dv", "dbias", "dtau"], res, ref):
        # dbias / dtau are sums over the whole batch: tolerance relative to their size
        scale = 1.0 if nm in ("out", "dq", "dk", "dv") else max(1.0, float(r.abs().max()))
        assert close(mine, r, dtype, atol32=tol, scale=scale), (nm, maxdiff(mine, r), last_call_info())


def test_window_defaults_to_bias_columns_and_frozen_params():
    q, k, v = (randn((1, 2, 96, 32), torch.float32, s) for s in (1, 2, 3))
    bias = randn((2, 24), torch.float32, 4, scale=0.5)
    tau = torch.full((2,), -1.0, device="cuda")
    a = lazy_attention_triton(q, k, v, bias, tau)
    b = lazy_attention_triton(q, k, v, bias, tau, window_size=24)
    assert torch.equal(a, b)
    qg = q.clone().requires_grad_(True)
    lazy_attention_triton(qg, k, v, bias, tau).sum().backward()      # frozen bias/tau: fast path
    assert qg.grad is not None and torch.isfinite(qg.grad).all()


def test_varlen_padding_rows_and_gradients_are_zero():
    B, H, L, D, W = 2, 4, 64, 32, 16
    q, k, v = (torch.randn(B, H, L, D, device="cuda", requires_grad=True) for _ in range(3))
    bias = torch.randn(H, W, device="cuda", requires_grad=True)
    tau = torch.full((H,), -1.0, device="cuda", requires_grad=True)
    varlen = torch.tensor([32, 48], device="cuda", dtype=torch.int32)
    out = lazy_attention_triton(q, k, v, bias, tau, window_size=W, varlen=varlen)
    out.sum().backward()
    for b, n in enumerate((32, 48)):
        assert (out[b, :, n:] == 0).all()
        for t in (q, k, v):
            assert (t.grad[b, :, n:] == 0).all()
    assert torch.isfinite(bias.grad).all() and torch.isfinite(tau.grad).all()
    assert bias.grad.dtype == torch.float32 and tau.grad.shape == tau.shape


def test_very_negative_tau_gives_zero_output():
    q, k, v = (randn((1, 1, 10, 16), torch.float32, s) for s in (1, 2, 3))
    out = lazy_attention_triton(q, k, v, torch.zeros(1, 4, device="cuda"), torch.full((1,), -100.0, device="cuda"))
    assert (out == 0).all()


def test_bf16_params_cast_like_the_example_layers():
    B, H, L, D, W = 1, 2, 200, 64, 64
    q, k, v, do = (randn((B, H, L, D), torch.bfloat16, s) for s in (1, 2, 3, 4))
    bias = (randn((H, W), torch.float32, 5, scale=0.02)).requires_grad_(True)
    tau = torch.full((H,), -1.0, device="cuda", requires_grad=True)
    out = lazy_attention_triton(q, k, v, bias.to(q.dtype), tau.to(q.dtype), window_size=W)
    out.backward(do)
    assert bias.grad.dtype == torch.float32 and bias.grad.shape == bias.shape and tau.grad.shape == tau.shape


@pytest.mark.parametrize("path,dtype", [("simt", torch.float32), ("auto", torch.bfloat16)])
def test_parameter_gradients_repeat_bit_for_bit(path, dtype):
    """dbias and dtau are sums over the whole batch formed by many thread blocks; they are accumulated in fixed
    point, so the order of arrival cannot change them (the reference reduces per-block buffers in a fixed order,
    lazy_attention_triton.py:645-649)."""
    set_path(path)
    B, H, L, D, W = 3, 4, 1500, 64, 700
    q, k, v, do = (randn((B, H, L, D), dtype, s) for s in (1, 2, 3, 4))
    bias = randn((H, W), torch.float32, 5, scale=0.3)
    tau = torch.tensor([-1.0, 0.3, -4.0, -0.5], device="cuda")
    vl = torch.tensor([1500, 1111, 640], dtype=torch.int32, device="cuda")
    first = _run(q, k, v, bias, tau, do, W, vl)
    assert float(first[4].abs().max()) > 0 and float(first[5].abs().max()) > 0
    for _ in range(3):
        again = _run(q, k, v, bias, tau, do, W, vl)
        for nm, a, b in zip(["out", "dq", "dk", "dv", "dbias", "dtau"], first, again):
            assert torch.equal(a, b), (nm, maxdiff(a, b))
