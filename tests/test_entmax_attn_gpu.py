"""alpha-entmax attention through the operator API against the CPU oracle; mirrors the
structure of the reference's tests/test_adasplash.py and test_adasplash_no_block_mask.py."""
import pytest
import torch

import adasplash as pkg
from flash_lazy_attention_b200 import (check_status, entmax_attention_forward, last_call_info, set_path,
                                       unpack_block_mask)
from oracle import block_mask_ref, entmax_attention_bwd_ref, entmax_attention_probs_ref, entmax_attention_ref

from gpu_util import TOL, close, maxdiff, randn, round_to

pytestmark = pytest.mark.gpu
VARIANTS = {"block_mask": pkg.adasplash, "no_block_mask": pkg.adasplash_no_block_mask}


@pytest.fixture(autouse=True)
def _auto_path():
    set_path(None)
    yield
    set_path(None)
    check_status()      # no tensor-core kernel may have reported an expired wait


@pytest.mark.parametrize("variant", ["block_mask", "no_block_mask"])
@pytest.mark.parametrize("B,H", [(1, 1), (2, 2)])
@pytest.mark.parametrize("L", [128, 256])
@pytest.mark.parametrize("D", [32, 64])
@pytest.mark.parametrize("alpha", [1.333, 1.5, 2.0])
@pytest.mark.parametrize("is_causal", [False, True])
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.bfloat16])
def test_forward_correctness(variant, B, H, L, D, alpha, is_causal, dtype):
    q, k, v = (randn((B, H, L, D), dtype, s) for s in (1, 2, 3))
    varlen = torch.randint(L // 2, L, (B,), generator=torch.Generator().manual_seed(42))
    ref = entmax_attention_ref(q.cpu(), k.cpu(), v.cpu(), alpha, varlen=varlen, is_causal=is_causal)
    out = VARIANTS[variant](q, k, v, alpha=alpha, varlen=varlen.cuda(), is_causal=is_causal)
    assert out.dtype == dtype
    assert maxdiff(out, ref) <= TOL[dtype], (maxdiff(out, ref), last_call_info())


@pytest.mark.parametrize("path", ["simt", "auto"])
@pytest.mark.parametrize("L", [256, 512])
@pytest.mark.parametrize("alpha", [1.5, 2.0, 1.333])
@pytest.mark.parametrize("dtype,D", [(torch.float32, 64), (torch.bfloat16, 64), (torch.bfloat16, 128), (torch.float16, 128)])
@pytest.mark.parametrize("is_causal", [False, True])
def test_backward_gradients(path, L, alpha, dtype, D, is_causal):
    set_path(path)
    q, k, v, do = (randn((2, 2, L, D), dtype, s) for s in (1, 2, 3, 4))
    ro, rq, rk, rv = entmax_attention_bwd_ref(q.cpu(), k.cpu(), v.cpu(), do.cpu(), alpha, is_causal=is_causal,
                                              cast=False, round_to=round_to(dtype))
    qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
    out = pkg.adasplash(qg, kg, vg, alpha=alpha, is_causal=is_causal)
    out.backward(do)
    assert close(out, ro, dtype), maxdiff(out, ro)
    for name, mine, ref in (("dq", qg.grad, rq), ("dk", kg.grad, rk), ("dv", vg.grad, rv)):
        # reference: atol 1e-2 on fp32 gradients (tests/test_adasplash.py:120-122)
        assert close(mine, ref, dtype, atol32=1e-2), (name, maxdiff(mine, ref), last_call_info())


def test_default_is_non_causal():
    q, k, v = (randn((1, 2, 128, 64), torch.float32, s) for s in (1, 2, 3))
    ref = entmax_attention_ref(q.cpu(), k.cpu(), v.cpu(), 1.5, is_causal=False)
    assert maxdiff(pkg.adasplash(q, k, v), ref) <= 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_varlen_backward_padding_is_zero_and_ignored(dtype):
    B, H, L, D = 2, 2, 320, 64
    q, k, v, do = (randn((B, H, L, D), dtype, s) for s in (1, 2, 3, 4))
    varlen = torch.tensor([200, 77])
    ro, rq, rk, rv = entmax_attention_bwd_ref(q.cpu(), k.cpu(), v.cpu(), do.cpu(), 1.5, varlen=varlen, is_causal=True,
                                              cast=False, round_to=round_to(dtype))
    qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
    out = pkg.adasplash(qg, kg, vg, alpha=1.5, is_causal=True, varlen=varlen.cuda())
    out.backward(do)
    for b in range(B):
        n = int(varlen[b])
        for t in (out, qg.grad, kg.grad, vg.grad):
            assert (t[b, :, n:] == 0).all()
    for mine, ref in ((out, ro), (qg.grad, rq), (kg.grad, rk), (vg.grad, rv)):
        assert close(mine, ref, dtype, atol32=1e-2), maxdiff(mine, ref)


@pytest.mark.parametrize("L", [512, 1024])
def test_numerical_stability(L):
    q, k, v = (randn((2, 2, L, 64), torch.float16, s, scale=100.0) for s in (1, 2, 3))
    out = pkg.adasplash(q, k, v, alpha=1.5)
    assert torch.isfinite(out).all() and out.abs().max() < 1e3


@pytest.mark.parametrize("L", [64, 128])
def test_simple_case(L):
    q = torch.zeros(1, 1, L, 64, device="cuda")
    out = pkg.adasplash(q, torch.zeros_like(q), torch.ones_like(q), alpha=1.5)
    assert torch.allclose(out, torch.ones_like(out), atol=1e-4)


def test_variable_length_handling():
    q, k, v = (torch.randn(2, 1, 256, 64, device="cuda") for _ in range(3))
    varlen = torch.tensor([128, 64], device="cuda")
    out = pkg.adasplash(q, k, v, varlen=varlen)
    assert (out[0, :, 128:] == 0).all() and (out[1, :, 64:] == 0).all()


@pytest.mark.parametrize("L", [512, 1024])
def test_large_sequences(L):
    q, k, v = (torch.randn(1, 1, L, 64, dtype=torch.float16, device="cuda") for _ in range(3))
    out = pkg.adasplash(q, k, v, alpha=1.5)
    assert out.shape == (1, 1, L, 64) and torch.isfinite(out).all()


@pytest.mark.parametrize("shape", [(1, 2, 4, 16), (1, 1, 1, 64), (2, 1, 77, 48), (1, 1, 130, 128), (1, 2, 200, 100)])
def test_ragged_and_tiny_shapes(shape):
    q, k, v = (randn(shape, torch.float32, s) for s in (1, 2, 3))
    for causal in (False, True):
        ref = entmax_attention_ref(q.cpu(), k.cpu(), v.cpu(), 1.5, is_causal=causal)
        assert maxdiff(pkg.adasplash(q, k, v, is_causal=causal), ref) <= 1e-4


def test_strided_views_match_contiguous():
    B, H, L, D = 2, 3, 160, 64
    base = [randn((B, L, H, D), torch.bfloat16, s) for s in (1, 2, 3)]
    views = [t.permute(0, 2, 1, 3) for t in base]            # b l h d -> b h l d, as the example layers do
    out_v = pkg.adasplash(*views, alpha=1.5, is_causal=True)
    out_c = pkg.adasplash(*[t.contiguous() for t in views], alpha=1.5, is_causal=True)
    assert torch.equal(out_v, out_c)


@pytest.mark.parametrize("alpha", [1.5, 2.0])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_mask_and_thresholds(alpha, causal, dtype):
    B, H, L, D = 1, 2, 520, 64
    g = torch.Generator().manual_seed(7)
    # clustered tokens so that a good share of the blocks is empty
    centres = torch.nn.functional.normalize(torch.randn(4, D, generator=g), dim=-1) * 12
    ids = (torch.arange(L) // 130) % 4
    q = (centres[ids] + 0.3 * torch.randn(L, D, generator=g)).expand(B, H, L, D).to(dtype).cuda().contiguous()
    k = (centres[ids] + 0.3 * torch.randn(L, D, generator=g)).expand(B, H, L, D).to(dtype).cuda().contiguous()
    v = randn((B, H, L, D), dtype, 3)
    varlen = torch.tensor([470])
    out, tau, _, _, mask = entmax_attention_forward(q, k, v, alpha, 10, causal, varlen.cuda(), use_block_mask=True)
    p_ref, tau_ref = entmax_attention_probs_ref(q.cpu(), k.cpu(), alpha, varlen=varlen, is_causal=causal)
    n = int(varlen[0])
    assert maxdiff(tau[:, :, :n], tau_ref[:, :, :n]) <= (1e-4 if dtype == torch.float32 else 2e-2)
    mine = unpack_block_mask(mask, L).cpu()
    ref = block_mask_ref(p_ref, varlen)
    # identical except for ties at the threshold: blocks whose largest probability is tiny may differ
    band = 1e-6 if dtype == torch.float32 else 1e-3
    firm = block_mask_ref(torch.where(p_ref > band, p_ref, torch.zeros_like(p_ref)), varlen)
    assert (mine | ~firm).all(), "a block with a clearly non-zero probability is missing from the mask"
    assert (~mine | ref).all(), "the mask marks a block the oracle has empty"
    assert 0.05 < ref.float().mean() < 0.9


def _clustered(B, H, L, D, dtype, seed, spread=0.3, scale=12.0, seg=130, n_clusters=4):
    """Tokens in contiguous segments around a few well separated centres: most (query block,
    key block) pairs hold no probability, so the block mask is sparse."""
    g = torch.Generator().manual_seed(seed)
    centres = torch.nn.functional.normalize(torch.randn(n_clusters, D, generator=g), dim=-1) * scale
    ids = (torch.arange(L) // seg) % n_clusters
    mk = lambda: (centres[ids] + spread * torch.randn(B, H, L, D, generator=g)).to(dtype).cuda().contiguous()
    return mk(), mk()


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("alpha", [1.5, 2.0])
def test_block_skipping_backward_matches_oracle_and_unmasked_variant(causal, alpha):
    B, H, L, D, dtype = 1, 2, 1100, 128, torch.bfloat16
    q, k = _clustered(B, H, L, D, dtype, 11)
    v, do = randn((B, H, L, D), dtype, 3), randn((B, H, L, D), dtype, 4)
    ref = entmax_attention_bwd_ref(q.cpu(), k.cpu(), v.cpu(), do.cpu(), alpha, is_causal=causal, cast=False,
                                   round_to=round_to(dtype))
    results = {}
    for name, fn in VARIANTS.items():
        leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
        out = fn(*leaves, alpha=alpha, is_causal=causal)
        out.backward(do)
        results[name] = [out] + [t.grad for t in leaves]
        for nm, mine, r in zip(("out", "dq", "dk", "dv"), results[name], ref):
            assert close(mine, r, dtype), (name, nm, maxdiff(mine, r))
    # skipping empty blocks must not change anything beyond the ties at the threshold (and the last place of
    # a 16-bit value where sums are formed over different tile sets)
    for a, b in zip(results["block_mask"], results["no_block_mask"]):
        assert close(a, b, dtype), maxdiff(a, b)
    _, _, _, _, mask = entmax_attention_forward(q, k, v, alpha, 10, causal, None, use_block_mask=True)
    density = unpack_block_mask(mask, L).float().mean().item()
    assert density < 0.6, density        # the input really is block sparse


@pytest.mark.gpu
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("dist", ["gauss", "heavy"])
def test_thresholds_of_long_rows_are_tight(causal, dist):
    """Rows with hundreds of entries above max-1 take the tail-model first step (alpha = 1.5) and stop
    after a short regular step; the thresholds must still agree with the converged oracle far inside
    the 16-bit tolerance, with and without that first step."""
    B, H, L, D, dtype = 1, 2, 2048, 128, torch.bfloat16
    g = torch.Generator().manual_seed(21)
    q = torch.randn(B, H, L, D, generator=g)
    k = torch.randn(B, H, L, D, generator=g)
    if dist == "heavy":   # a few dominant keys per row
        k = k * (1.0 + 3.0 * (torch.rand(B, H, L, 1, generator=g) > 0.98).float())
    q, k = q.to(dtype).cuda(), k.to(dtype).cuda()
    v = randn((B, H, L, D), dtype, 3)
    _, tau_ref = entmax_attention_probs_ref(q.cpu(), k.cpu(), 1.5, varlen=None, is_causal=causal)
    results = []
    from flash_lazy_attention_b200 import _lib, set_flags
    for flags in (0, _lib.FLAG_PLAIN_FIRST_STEP, _lib.FLAG_CANDIDATE_LIST):   # tail-model step / plain Halley / candidates
        set_flags(flags)
        try:
            out, tau, _, _, _ = entmax_attention_forward(q, k, v, 1.5, 10, causal, None, use_block_mask=True)
        finally:
            set_flags(0)
        assert last_call_info()["path"] == "tcgen05"
        assert maxdiff(tau, tau_ref) <= 5e-4, (flags, maxdiff(tau, tau_ref))
        results.append((out.float(), tau))
    assert maxdiff(results[0][1], results[1][1]) <= 2e-4
    assert maxdiff(results[0][0], results[1][0]) <= 2e-2


@pytest.mark.gpu
@pytest.mark.parametrize("niter", [0, 1, 2, 3])
@pytest.mark.parametrize("causal", [False, True])
def test_small_iteration_caps_finish_and_stay_finite(niter, causal):
    """niter caps the threshold passes; with a low cap the rows are not normalised exactly, but every
    wait of the kernels must still be met (status word clean), outputs finite, and from three passes
    on the probabilities of a row sum to 1 within a percent."""
    B, H, L, D, dtype = 1, 2, 700, 128, torch.bfloat16
    q, k, v, do = (randn((B, H, L, D), dtype, s) for s in (1, 2, 3, 4))
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
    out = pkg.adasplash(*leaves, alpha=1.5, niter=niter, is_causal=causal)
    out.backward(do)
    check_status(q.device)
    assert last_call_info()["path"] == "tcgen05"
    for t in [out] + [x.grad for x in leaves]:
        assert torch.isfinite(t).all()
    if niter >= 3:
        ones = torch.ones_like(v)
        rowsum = pkg.adasplash(q, k, ones, alpha=1.5, niter=niter, is_causal=causal).float()
        assert maxdiff(rowsum, torch.ones_like(rowsum)) <= 2e-2


@pytest.mark.gpu
@pytest.mark.parametrize("causal", [False, True])
def test_many_tiles_with_sparse_tile_bitmaps_match_the_oracle(causal):
    """35 key tiles (two bitmap words) and eight clusters: the tensor-core kernels visit a different,
    shrinking subset of tiles in every pass and the backward kernels only the blocks of the mask."""
    B, H, L, D, dtype = 1, 2, 4400, 128, torch.bfloat16
    q, k = _clustered(B, H, L, D, dtype, 5, seg=256, n_clusters=8)
    v, do = randn((B, H, L, D), dtype, 3), randn((B, H, L, D), dtype, 4)
    ref = entmax_attention_bwd_ref(q.cpu(), k.cpu(), v.cpu(), do.cpu(), 1.5, is_causal=causal, cast=False,
                                   round_to=round_to(dtype))
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
    out = pkg.adasplash(*leaves, alpha=1.5, is_causal=causal)
    out.backward(do)
    check_status(q.device)
    assert last_call_info()["path"] == "tcgen05"
    for name, mine, r in zip(("out", "dq", "dk", "dv"), [out] + [t.grad for t in leaves], ref):
        assert close(mine, r, dtype), (name, maxdiff(mine, r))
    _, _, _, _, mask = entmax_attention_forward(q, k, v, 1.5, 10, causal, None, use_block_mask=True)
    assert unpack_block_mask(mask, L).float().mean() < 0.5
