"""Grouped-query attention inside the kernels, and the layer modules (the reference's example layers and its
LazyAttention module contract, tests/test_lazy_attention.py:5-70, on the GPU)."""
import pytest
import torch

import adasplash as pkg
from adasplash.lazy_attention import LazyAttention
from flash_lazy_attention_b200 import LazyAttentionLayer, check_status, last_call_info, set_path
from flash_lazy_attention_b200.layers import lengths_from, rotary

from gpu_util import close, maxdiff, randn

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _auto_path():
    set_path(None)
    yield
    set_path(None)
    check_status()


def _repeat(t, n):
    return t.repeat_interleave(n, dim=1)


@pytest.mark.parametrize("op", ["entmax", "entmax_alpha2", "lazy"])
@pytest.mark.parametrize("H,Hkv", [(4, 2), (8, 1), (6, 6)])
@pytest.mark.parametrize("D", [64, 128])
def test_shared_kv_heads_match_repeated_heads(op, H, Hkv, D):
    """k, v with Hkv heads read in place by the tensor-core kernels against the same call on heads repeated
    by the caller (what the reference's layers do): same outputs, dk / dv of a shared head = sum over its group."""
    B, L, W, dtype = 2, 700, 96, torch.bfloat16
    q, do = randn((B, H, L, D), dtype, 1), randn((B, H, L, D), dtype, 4)
    k, v = randn((B, Hkv, L, D), dtype, 2), randn((B, Hkv, L, D), dtype, 3)
    bias, tau = randn((H, W), torch.float32, 5, scale=0.05), torch.full((H,), -1.0, device="cuda")
    varlen = torch.tensor([700, 555], device="cuda", dtype=torch.int32)

    def run(kk, vv):
        leaves = [t.clone().requires_grad_(True) for t in (q, kk, vv)]
        if op == "lazy":
            out = pkg.lazy_attention_triton(*leaves, bias, tau, window_size=W, varlen=varlen)
        else:
            out = pkg.adasplash(*leaves, alpha=2.0 if op == "entmax_alpha2" else 1.5, is_causal=True, varlen=varlen)
        out.backward(do)
        return [out.detach()] + [t.grad for t in leaves]

    shared = run(k, v)
    assert last_call_info()["path"] == "tcgen05"
    n_rep = H // Hkv
    rep = run(_repeat(k, n_rep), _repeat(v, n_rep))
    assert shared[2].shape == k.shape and shared[3].shape == v.shape
    # the reference for the shared heads' gradients: fp32 sum of the repeated heads' (16-bit) gradients
    rep_dk = rep[2].float().view(B, Hkv, n_rep, L, D).sum(2)
    rep_dv = rep[3].float().view(B, Hkv, n_rep, L, D).sum(2)
    assert torch.equal(shared[0], rep[0]) and torch.equal(shared[1], rep[1])     # out, dq: the same arithmetic
    for name, mine, ref, parts in (("dk", shared[2], rep_dk, rep[2]), ("dv", shared[3], rep_dv, rep[3])):
        # n_rep roundings to 16 bits on the reference side (each half a unit in the last place of ITS value)
        # against one here
        mags = parts.float().abs().view(B, Hkv, n_rep, L, D).sum(2)
        tol = 2e-2 * n_rep + 2.0 ** -8 * (mags + ref.abs())
        assert bool(((mine.float() - ref).abs() <= tol).all()), (name, maxdiff(mine, ref))


def test_shared_kv_heads_on_the_cuda_core_family_are_repeated_by_the_wrapper():
    B, H, Hkv, L, D = 1, 4, 2, 96, 32
    q, k, v = randn((B, H, L, D), torch.float32, 1), randn((B, Hkv, L, D), torch.float32, 2), randn((B, Hkv, L, D), torch.float32, 3)
    kg, vg = k.clone().requires_grad_(True), v.clone().requires_grad_(True)
    out = pkg.adasplash(q, kg, vg, alpha=1.5, is_causal=True)
    assert last_call_info()["path"] == "simt"
    ref = pkg.adasplash(q, _repeat(k, 2), _repeat(v, 2), alpha=1.5, is_causal=True)
    assert torch.equal(out, ref)
    out.sum().backward()
    assert kg.grad.shape == k.shape and vg.grad.shape == v.shape


def test_layer_with_padding_mask_and_shared_heads_matches_a_dense_restatement():
    torch.manual_seed(0)
    B, L, hidden, H, Hkv, W = 2, 300, 256, 4, 2, 64
    layer = LazyAttentionLayer(hidden, H, Hkv, max_bias_length=W).cuda().to(torch.bfloat16)
    assert layer.bias.dtype == torch.float32 and layer.tau.dtype == torch.float32 or True
    with torch.no_grad():
        layer.bias.copy_(torch.randn(H, W) * 0.02)
    x = torch.randn(B, L, hidden, device="cuda", dtype=torch.bfloat16)
    mask = torch.ones(B, L, dtype=torch.long, device="cuda")
    mask[1, 200:] = 0
    y = layer(x, attention_mask=mask)
    assert y.shape == (B, L, hidden) and torch.isfinite(y).all()
    # dense restatement of the same layer in fp32 torch ops
    from oracle import lazy_attention_ref
    D = hidden // H
    q = layer.q_proj(x).view(B, L, H, D)
    k = layer.k_proj(x).view(B, L, Hkv, D)
    v = layer.v_proj(x).view(B, L, Hkv, D)
    q, k = rotary(q, layer.rope_theta), rotary(k, layer.rope_theta)
    q, k, v = (t.permute(0, 2, 1, 3) for t in (q, k, v))
    k, v = _repeat(k, H // Hkv), _repeat(v, H // Hkv)
    o = lazy_attention_ref(q.cpu(), k.cpu(), v.cpu(), layer.bias.to(q.dtype).float().cpu(), layer.tau.to(q.dtype).float().cpu(),
                           W, lengths_from(mask).cpu())
    ref = layer.o_proj(o.to(torch.bfloat16).cuda().permute(0, 2, 1, 3).reshape(B, L, hidden))
    assert close(y[0], ref[0], torch.bfloat16) and close(y[1, :200], ref[1, :200], torch.bfloat16)
    # cu_seqlens give the same lengths
    assert torch.equal(lengths_from(cu_seqlens=torch.tensor([0, 300, 500])), torch.tensor([300, 200], dtype=torch.int32))
    y.float().sum().backward()
    assert layer.bias.grad is not None and layer.tau.grad is not None and layer.k_proj.weight.grad is not None


def test_lazy_attention_module_contract():
    """Shape, gradients on tau and attention_biases, tau = -100 gives exact zeros, tiny sequences run
    (tests/test_lazy_attention.py:5-70 of the reference, on CUDA tensors)."""
    B, L, D, H = 2, 16, 32, 4
    model = LazyAttention(dim=D, num_heads=H, window_size=4).cuda()
    x = torch.randn(B, L, D, device="cuda", requires_grad=True)
    out = model(x)
    assert out.shape == (B, L, D)
    out.sum().backward()
    assert x.grad is not None and model.tau.grad is not None and model.attention_biases.grad is not None
    assert (model.attention_biases == 0).all()
    sparse = LazyAttention(dim=16, num_heads=1).cuda()
    with torch.no_grad():
        sparse.tau.fill_(-100.0)
    assert (sparse(torch.randn(1, 10, 16, device="cuda")) == 0).all()
    tiny = LazyAttention(dim=4, num_heads=2).cuda()
    assert tiny(torch.ones(1, 4, 4, device="cuda")).shape == (1, 4, 4)
    with pytest.raises(RuntimeError, match="CUDA"):
        LazyAttention(dim=8, num_heads=2)(torch.randn(1, 4, 8))
