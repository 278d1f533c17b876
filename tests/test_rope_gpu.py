"""Rotary embedding of q and k in one launch (fla_rope_qk) against the dense fp32 formulation the layers used
before (layers.rotary: rotate-half, angle = position / base^(j / (D/2))), forward, inverse and gradient."""
import ctypes as C

import pytest
import torch

import flash_lazy_attention_b200 as fla
from flash_lazy_attention_b200 import _lib
from flash_lazy_attention_b200.layers import rotary
from flash_lazy_attention_b200.ops import _t4, rope_qk_apply

from gpu_util import maxdiff, randn

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 2e-5, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}   # half an ulp of values up to ~4


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,L,H,Hk,D,offset", [(2, 300, 4, 4, 128, 0), (1, 1000, 8, 2, 64, 17), (3, 77, 2, 1, 32, 0), (2, 50, 3, 3, 8, 3), (1, 33, 2, 2, 20, 0),
                                                 (1, 4096, 4, 4, 128, 30000)])
def test_rope_matches_the_dense_formulation(dtype, B, L, H, Hk, D, offset):
    q = randn((B, L, H, D), dtype, 1)              # b l h d, as the projections of a layer produce it
    k = randn((B, L, Hk, D), dtype, 2)
    qr, kr = fla.rope_qk(q.transpose(1, 2), k.transpose(1, 2), 10000.0, offset)
    assert qr.shape == (B, H, L, D) and qr.stride() == q.transpose(1, 2).stride()     # no layout change, no copy
    ref_q, ref_k = rotary(q, 10000.0, offset), rotary(k, 10000.0, offset)
    # positions beyond ~1e4 make the fp32 angle itself uncertain by ~1e-3: same fp32 sequence here, so still tight
    assert maxdiff(qr.transpose(1, 2), ref_q) <= TOL[dtype], maxdiff(qr.transpose(1, 2), ref_q)
    assert maxdiff(kr.transpose(1, 2), ref_k) <= TOL[dtype]
    # contiguous [B,H,L,D] input gives the same numbers
    qc, kc = fla.rope_qk(q.transpose(1, 2).contiguous(), k.transpose(1, 2).contiguous(), 10000.0, offset)
    assert torch.equal(qc, qr) and torch.equal(kc, kr)
    # rotating back restores the input up to rounding
    q0, k0 = rope_qk_apply(qr, kr, 10000.0, offset, inverse=True)
    assert maxdiff(q0, q.transpose(1, 2)) <= 2 * TOL[dtype]


def test_rope_gradient_is_the_inverse_rotation():
    B, L, H, D = 2, 257, 4, 64
    q, k = (randn((B, H, L, D), torch.float32, s).requires_grad_(True) for s in (1, 2))
    gq, gk = randn((B, H, L, D), torch.float32, 3), randn((B, H, L, D), torch.float32, 4)
    qr, kr = fla.rope_qk(q, k, 500.0, 5)
    (qr * gq).sum().backward(retain_graph=True)
    (kr * gk).sum().backward()
    q2, k2 = (t.detach().clone().requires_grad_(True) for t in (q, k))
    r_q = rotary(q2.transpose(1, 2), 500.0, 5).transpose(1, 2)
    r_k = rotary(k2.transpose(1, 2), 500.0, 5).transpose(1, 2)
    ((r_q * gq).sum() + (r_k * gk).sum()).backward()
    assert maxdiff(q.grad, q2.grad) <= 2e-5 and maxdiff(k.grad, k2.grad) <= 2e-5
    torch.library.opcheck(torch.ops.flash_lazy.rope_qk.default, (q, k, 500.0, 5, False),
                          test_utils=("test_schema", "test_faketensor", "test_autograd_registration",
                                      "test_aot_dispatch_dynamic"))


def test_rope_in_place_and_argument_checks_through_the_c_abi():
    lib = _lib.load()
    q = randn((1, 2, 64, 128), torch.bfloat16, 1)
    expect, _ = rope_qk_apply(q, q, 10000.0, 0)
    work = q.clone()
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.fla_rope_qk(_t4(work), _t4(work), 2, None, None, 0, 1, 64, 128, 2, C.c_float(10000.0), 0, 0, stream)
    assert rc == 0 and torch.equal(work, expect)
    bad = randn((1, 2, 64, 25), torch.bfloat16, 1)          # odd head dimension
    rc = lib.fla_rope_qk(_t4(bad), _t4(bad), 2, None, None, 0, 1, 64, 25, 2, C.c_float(10000.0), 0, 0, stream)
    assert rc == 1 and b"even head dimension" in lib.fla_last_error()     # FLA_ERR_INVALID
    odd = randn((1, 2, 65, 128), torch.bfloat16, 1)[:, :, 1:, :]          # misaligned-free but offset view: still exact
    a, _ = rope_qk_apply(odd, odd, 10000.0, 0)
    b, _ = rope_qk_apply(odd.contiguous(), odd.contiguous(), 10000.0, 0)
    assert torch.equal(a, b)
    rc = lib.fla_rope_qk(_t4(q), _t4(q), 2, _t4(q), None, 2, 1, 64, 128, 2, C.c_float(10000.0), 0, 0, stream)
    assert rc == 1                                                    # FLA_ERR_INVALID: k_out missing
