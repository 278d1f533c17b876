"""Lazy Attention against the reference's own Triton module running natively on the same GPU (a copy made by
oracle/make_ref.py into the untracked oracle/_ref/; skipped where that copy is absent).  fp32 inputs pin both this
library and the dense oracle to the reference's kernels on the device; bf16 inputs check the 16-bit agreement and
record where the reference's bf16 dK departs from its own fp32 result."""
import importlib.util
import os

import pytest
import torch

from adasplash.lazy_attention_triton import lazy_attention_triton
from flash_lazy_attention_b200 import check_status, set_path
from oracle import lazy_attention_grads_analytic

from gpu_util import maxdiff, randn

pytestmark = pytest.mark.gpu
REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "lazy_attention_triton.py")


@pytest.fixture(scope="module")
def ref_mod():
    if not os.path.exists(REF):
        pytest.skip("oracle/_ref/lazy_attention_triton.py is absent (python oracle/make_ref.py <reference checkout>)")
    spec = importlib.util.spec_from_file_location("reference_lazy_attention_triton", REF)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _run(fn, q, k, v, bias, tau, do, W, varlen):
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v, bias, tau)]
    out = fn(*leaves, window_size=W, varlen=varlen)
    out.backward(do)
    return [out.detach().float()] + [t.grad.float() for t in leaves]


@pytest.mark.parametrize("varlen", [None, [700, 333]])
def test_fp32_matches_the_reference_kernels_on_the_device(ref_mod, varlen):
    set_path(None)
    B, H, L, D, W = 2, 2, 700, 64, 128
    q, k, v, do = (randn((B, H, L, D), torch.float32, s) for s in (1, 2, 3, 4))
    bias, tau = randn((H, W), torch.float32, 5, scale=0.3), torch.tensor([-1.0, 0.4], device="cuda")
    vl = None if varlen is None else torch.tensor(varlen, dtype=torch.int32, device="cuda")
    ours = _run(lazy_attention_triton, q, k, v, bias, tau, do, W, vl)
    ref = _run(ref_mod.lazy_attention_triton, q, k, v, bias, tau, do, W, vl)
    orc = lazy_attention_grads_analytic(q.cpu(), k.cpu(), v.cpu(), bias.cpu(), tau.cpu(), do.cpu(), W,
                                        None if vl is None else vl.cpu())
    names = ["out", "dq", "dk", "dv", "dbias", "dtau"]
    valid = None if varlen is None else varlen
    for nm, a, r, o in zip(names, ours, ref, orc):
        if valid is not None and nm in ("out", "dq", "dk", "dv"):   # the reference leaves padded output rows unwritten
            a, r, o = (torch.cat([t[b, :, :valid[b]].reshape(-1) for b in range(B)]) for t in (a, r, o.cuda().float()))
        scale = max(1.0, float(r.abs().max())) if nm in ("dbias", "dtau") else 1.0
        # the reference's kernels run their products in TF32 on this GPU: 2e-2 (the oracle and this library: fp32)
        assert maxdiff(a, r) <= 2e-2 * scale, (nm, "ours vs reference", maxdiff(a, r))
        assert maxdiff(o, r) <= 2e-2 * scale, (nm, "oracle vs reference", maxdiff(o, r))
        assert maxdiff(a, o) <= 2e-3 * scale, (nm, "ours vs oracle", maxdiff(a, o))
    check_status()


def test_bf16_agreement_and_the_reference_dk(ref_mod):
    set_path(None)
    B, H, L, D, W = 1, 2, 1024, 64, 128      # (the reference's fp32 kernels do not fit shared memory at D = 128)
    q, k, v, do = (randn((B, H, L, D), torch.bfloat16, s) for s in (1, 2, 3, 4))
    bias, tau = randn((H, W), torch.float32, 5, scale=0.02), torch.full((H,), -1.0, device="cuda")
    ours = _run(lazy_attention_triton, q, k, v, bias, tau, do, W, None)
    ref = _run(ref_mod.lazy_attention_triton, q, k, v, bias, tau, do, W, None)
    ref32 = _run(ref_mod.lazy_attention_triton, q.float(), k.float(), v.float(), bias, tau, do.float(), W, None)
    for nm, a, r in zip(["out", "dq", "dk", "dv", "dbias", "dtau"], ours, ref):
        if nm == "dk":
            continue
        scale = max(1.0, float(r.abs().max())) if nm in ("dbias", "dtau") else 1.0
        assert maxdiff(a, r) <= 3e-2 * scale, (nm, maxdiff(a, r))
    # dk: this library stays with the reference's own fp32 result; how far the reference's bf16 kernel is from it is
    # printed, not asserted (run with -s)
    d_ours, d_ref = maxdiff(ours[2], ref32[2]), maxdiff(ref[2], ref32[2])
    print(f"dk against the reference in fp32: this library {d_ours:.3e}, the reference's bf16 run {d_ref:.3e}")
    assert d_ours <= 5e-2
    check_status()
