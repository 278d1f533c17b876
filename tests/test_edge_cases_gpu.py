"""Edges of the domain: the longest sequence the tensor-core family takes (65536 tokens: 512 key tiles, the limit
of its tile list), a sequence just beyond it (handled by the CUDA-core family), and a batch element with no valid
token at all."""
import math

import pytest
import torch

import adasplash as pkg
from adasplash.lazy_attention_triton import lazy_attention_triton
from flash_lazy_attention_b200 import check_status, last_call_info, set_path
from oracle import entmax_attention_rows_ref, lazy_attention_rows_ref

from gpu_util import RTOL16, randn

pytestmark = pytest.mark.gpu
DT = torch.bfloat16


@pytest.fixture(autouse=True)
def _auto_path():
    set_path(None)
    yield
    set_path(None)
    check_status()


def _gen(seed, *shape):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g)


def _bar(tag, mine, ref):
    mine, ref = mine.detach().double().cpu(), ref.detach().double().cpu()
    diff = (mine - ref).abs()
    assert bool((diff <= 2e-2 + RTOL16[DT] * ref.abs()).all()), (tag, float(diff.max()))


def _rows(L):
    """The first 128 rows, 128 in the middle, and the last 128 (the only viewers of the last key tile)."""
    return torch.cat([torch.arange(128), torch.arange(L // 2 - 64, L // 2 + 64), torch.arange(L - 128, L)])


def test_entmax_at_the_longest_tensor_core_length():
    L, D = 65536, 128
    q, k, v, do = (_gen(40 + i, 1, 1, L, D).to(DT) for i in range(4))
    leaves = [t.cuda().requires_grad_(True) for t in (q, k, v)]
    out = pkg.adasplash(*leaves, alpha=1.5, niter=10, is_causal=True)
    out.backward(do.cuda())
    assert last_call_info()["path"] == "tcgen05"
    got = [t.detach().cpu()[0, 0] for t in (out, leaves[0].grad, leaves[1].grad, leaves[2].grad)]
    rows = _rows(L)
    r = entmax_attention_rows_ref(q[0, 0], k[0, 0], v[0, 0], do[0, 0], rows, 1.5, True, None, round_to=DT)
    _bar("out", got[0][rows], r["out"])
    _bar("dq", got[1][rows], r["dq"])
    last, tail = slice(L - 128, L), rows >= L - 128
    _bar("dk last tile", got[2][last], r["ds"][tail][:, last].t() @ q[0, 0][last].float() / math.sqrt(D))
    _bar("dv last tile", got[3][last], r["p"][tail][:, last].t() @ do[0, 0][last].float())


def test_lazy_at_the_longest_tensor_core_length():
    L, D, W = 65536, 128, 512
    q, k, v, do = (_gen(50 + i, 1, 1, L, D).to(DT) for i in range(4))
    bias, tau = _gen(54, 1, W) * 0.02, torch.full((1,), -1.0)
    leaves = [t.cuda().requires_grad_(True) for t in (q, k, v)]
    out = lazy_attention_triton(*leaves, bias.cuda(), tau.cuda(), window_size=W)
    out.backward(do.cuda())
    assert last_call_info()["path"] == "tcgen05"
    got = [t.detach().cpu()[0, 0] for t in (out, leaves[0].grad, leaves[1].grad, leaves[2].grad)]
    rows = _rows(L)
    r = lazy_attention_rows_ref(q[0, 0], k[0, 0], v[0, 0], do[0, 0], bias[0], tau[0], rows, W, None, round_to=DT)
    _bar("lazy out", got[0][rows], r["out"])
    _bar("lazy dq", got[1][rows], r["dq"])
    last, tail = slice(L - 128, L), rows >= L - 128
    _bar("lazy dk last tile", got[2][last], r["ds_r"][tail][:, last].t() @ q[0, 0][last].float() / math.sqrt(D))
    _bar("lazy dv last tile", got[3][last], r["a"][tail][:, last].t() @ do[0, 0][last].float())


def test_beyond_the_tensor_core_length_the_cuda_core_family_takes_over():
    """65600 tokens: one tile more than the tensor-core tile list holds.  The library must not refuse: the SIMT
    family runs the same call (forward checked on three row blocks)."""
    L, D = 65600, 64
    q, k, v = (_gen(60 + i, 1, 1, L, D).to(DT) for i in range(3))
    out = pkg.adasplash_no_block_mask(q.cuda(), k.cuda(), v.cuda(), alpha=1.5, niter=10, is_causal=True)
    assert last_call_info()["path"] == "simt"
    rows = _rows(L)
    r = entmax_attention_rows_ref(q[0, 0], k[0, 0], v[0, 0], torch.zeros(L, D).to(DT), rows, 1.5, True, None, round_to=DT)
    _bar("out", out.cpu()[0, 0][rows], r["out"])


@pytest.mark.parametrize("path", ["auto", "simt"])
def test_a_batch_element_without_any_valid_token(path):
    """varlen = 0 for one sequence: its outputs and all its gradients are zero, the others are untouched."""
    set_path(path)
    B, H, L, D = 3, 2, 300, 64
    q, k, v, do = (randn((B, H, L, D), DT, s) for s in (1, 2, 3, 4))
    varlen = torch.tensor([300, 0, 77], device="cuda")
    res = {}
    for name, lens in (("with", varlen), ("without", torch.tensor([300, 300, 77], device="cuda"))):
        leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
        out = pkg.adasplash(*leaves, alpha=1.5, is_causal=True, varlen=lens)
        out.backward(do)
        res[name] = [out.detach()] + [t.grad for t in leaves]
    for a, b in zip(res["with"], res["without"]):
        assert torch.isfinite(a).all() and (a[1] == 0).all()
        assert torch.equal(a[0], b[0]) and torch.equal(a[2], b[2])
    bias, tau = randn((H, 32), torch.float32, 5, scale=0.1).requires_grad_(True), torch.full((H,), -1.0, device="cuda",
                                                                                             requires_grad=True)
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
    out = lazy_attention_triton(*leaves, bias, tau, window_size=32, varlen=varlen)
    out.backward(do)
    for t in [out] + [x.grad for x in leaves]:
        assert torch.isfinite(t).all() and (t[1] == 0).all()
    assert torch.isfinite(bias.grad).all() and torch.isfinite(tau.grad).all()
