"""The two ways the tensor-core forward finds the row thresholds (candidates kept by the first pass /
passes over recomputed score tiles) against each other and the oracle, padding that holds NaN, and the
status check of the C ABI."""
import pytest
import torch

import adasplash as pkg
from flash_lazy_attention_b200 import (_lib, check_status, entmax_attention_forward, last_call_info, read_status,
                                       set_flags, set_path)
from oracle import entmax_attention_bwd_ref, entmax_attention_probs_ref, lazy_attention_grads_analytic

from gpu_util import close, maxdiff, randn, round_to

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _reset():
    set_path(None)
    set_flags(0)
    yield
    set_flags(0)
    set_path(None)
    check_status()


@pytest.mark.parametrize("alpha", [1.5, 2.0, 1.333])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("L,D", [(700, 128), (2048, 64), (2500, 128)])
def test_candidate_lists_and_score_passes_agree(alpha, causal, L, D):
    """Same inputs through both threshold solvers: thresholds within 2e-4 of the converged oracle
    for the lists (5e-4 for the passes, whose stop rule is looser), outputs within the 16-bit bar."""
    B, H, dtype = 1, 2, torch.bfloat16
    q, k, v = (randn((B, H, L, D), dtype, s) for s in (1, 2, 3))
    _, tau_ref = entmax_attention_probs_ref(q.cpu(), k.cpu(), alpha, varlen=None, is_causal=causal)
    res = {}
    for name, flags in (("lists", _lib.FLAG_CANDIDATE_LIST), ("passes", _lib.FLAG_NO_CANDIDATE_LIST)):
        set_flags(flags)
        read_status(q.device, reset=True)
        out, tau, _, _, mask = entmax_attention_forward(q, k, v, alpha, 10, causal, None, use_block_mask=True)
        st = read_status(q.device)
        assert last_call_info()["path"] == "tcgen05" and st["error"] == 0
        res[name] = (out.float(), tau, mask, st)
    tiles = B * H * ((L + 127) // 128)
    pairs = B * H * (((L + 127) // 128 + 1) // 2)    # the pass-only forward holds two query tiles per thread block
    assert res["passes"][3]["pass_ctas"] == pairs and res["passes"][3]["list_ctas"] == 0
    assert res["lists"][3]["list_ctas"] + res["lists"][3]["pass_ctas"] == tiles
    if alpha >= 1.5:      # small supports: the candidates fit the slots and the spill pool
        assert res["lists"][3]["list_ctas"] == tiles, res["lists"][3]
        # no score product beyond row max + S + P.V
        assert res["lists"][3]["tile_mmas"] < res["passes"][3]["tile_mmas"]
    assert maxdiff(res["lists"][1], tau_ref) <= 2e-4, maxdiff(res["lists"][1], tau_ref)
    assert maxdiff(res["passes"][1], tau_ref) <= 5e-4, maxdiff(res["passes"][1], tau_ref)
    assert maxdiff(res["lists"][0], res["passes"][0]) <= 2e-2


@pytest.mark.parametrize("alpha", [1.5, 1.333])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("L,D,lens", [(700, 128, None), (1409, 64, [1409, 130]), (128, 128, None), (2048, 128, [1000, 2048])])
def test_two_query_tiles_per_block_equal_one(alpha, causal, L, D, lens):
    """The pass-only forward with two query tiles per thread block (sharing every K tile it fetches) against the
    one-tile form: the same arithmetic per entry, the row sums added up in a different order (two threads per row
    taking every key tile, instead of four taking alternate ones) -- thresholds within 2e-5, outputs within one
    16-bit unit, block masks equal up to entries sitting on a threshold.  Odd tile counts, a second tile that is
    all padding, a single tile."""
    B, H, dtype = (1 if lens is None else len(lens)), 2, torch.bfloat16
    q, k, v = (randn((B, H, L, D), dtype, s) for s in (1, 2, 3))
    varlen = None if lens is None else torch.tensor(lens, device="cuda")
    res = []
    for flags in (_lib.FLAG_NO_CANDIDATE_LIST, _lib.FLAG_NO_CANDIDATE_LIST | _lib.FLAG_ONE_TILE_CTAS):
        set_flags(flags)
        out, tau, _, _, mask = entmax_attention_forward(q, k, v, alpha, 10, causal, varlen, use_block_mask=True)
        assert last_call_info()["path"] == "tcgen05"
        res.append((out, tau, mask))
    (o2, t2, m2), (o1, t1, m1) = res
    assert maxdiff(t2, t1) <= 2e-5, maxdiff(t2, t1)
    assert maxdiff(o2, o1) <= 2.0 ** -7 * max(1.0, float(o1.float().abs().max())), maxdiff(o2, o1)
    differing = int(((m2 ^ m1) != 0).sum())
    assert differing <= max(1, m1.numel() // 500), differing
    if lens is not None:
        for b_, n in enumerate(lens):
            assert (o2[b_, :, n:] == 0).all() and (t2[b_, :, n:] == 0).all()


def test_list_overflow_falls_back_to_score_passes():
    """Tiny scores put every key in the support: no thread can hold its candidates, the CTAs fall back
    to passes over score tiles, and the result is still the oracle's."""
    B, H, L, D, dtype = 1, 2, 4096, 128, torch.bfloat16
    q, k, v = (randn((B, H, L, D), dtype, s, scale=sc) for s, sc in ((1, 0.05), (2, 0.05), (3, 1.0)))
    read_status(q.device, reset=True)
    set_flags(_lib.FLAG_CANDIDATE_LIST)
    out, tau, _, _, _ = entmax_attention_forward(q, k, v, 1.5, 10, True, None, use_block_mask=False)
    st = read_status(q.device)
    assert st["error"] == 0 and st["pass_ctas"] > 0, st
    _, tau_ref = entmax_attention_probs_ref(q.cpu(), k.cpu(), 1.5, varlen=None, is_causal=True)
    assert maxdiff(tau, tau_ref) <= 5e-4


@pytest.mark.parametrize("flags", [0, 1, 4])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("alpha", [1.5, 2.0])
def test_backward_after_either_solver(flags, causal, alpha):
    B, H, L, D, dtype = 1, 2, 1300, 128, torch.bfloat16
    set_flags(flags)
    q, k, v, do = (randn((B, H, L, D), dtype, s) for s in (1, 2, 3, 4))
    varlen = torch.tensor([1111])
    ref = entmax_attention_bwd_ref(q.cpu(), k.cpu(), v.cpu(), do.cpu(), alpha, varlen=varlen, is_causal=causal,
                                   cast=False, round_to=round_to(dtype))
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
    out = pkg.adasplash(*leaves, alpha=alpha, is_causal=causal, varlen=varlen.cuda())
    out.backward(do)
    for name, mine, r in zip(("out", "dq", "dk", "dv"), [out] + [t.grad for t in leaves], ref):
        assert close(mine, r, dtype), (name, maxdiff(mine, r))


@pytest.mark.parametrize("path", ["auto", "simt"])
@pytest.mark.parametrize("causal", [False, True])
def test_entmax_padding_may_hold_nan(path, causal):
    """Rows at or beyond varlen are padding: NaN there (q, k, v and the incoming gradient) must not
    reach any valid row (the reference masks every load, lazy_attention_triton.py:41,56,171)."""
    set_path(path)
    B, H, L, D, dtype = 2, 2, 600, 128, torch.bfloat16
    lens = [333, 520]            # neither a multiple of 128 nor of 16
    q, k, v, do = (randn((B, H, L, D), dtype, s) for s in (1, 2, 3, 4))
    varlen = torch.tensor(lens)
    ref = entmax_attention_bwd_ref(q.cpu(), k.cpu(), v.cpu(), do.cpu(), 1.5, varlen=varlen, is_causal=causal,
                                   cast=False, round_to=round_to(dtype))
    for t in (q, k, v, do):
        for b, n in enumerate(lens):
            t[b, :, n:] = float("nan")
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
    out = pkg.adasplash(*leaves, alpha=1.5, is_causal=causal, varlen=varlen.cuda())
    out.backward(do)
    for name, mine, r in zip(("out", "dq", "dk", "dv"), [out] + [t.grad for t in leaves], ref):
        assert torch.isfinite(mine).all(), name
        for b, n in enumerate(lens):
            assert (mine[b, :, n:] == 0).all(), name
        assert close(mine, r, dtype), (name, maxdiff(mine, r))


@pytest.mark.parametrize("path", ["auto", "simt"])
def test_lazy_padding_may_hold_nan(path):
    set_path(path)
    B, H, L, D, W, dtype = 2, 2, 500, 128, 64, torch.bfloat16
    lens = [203, 410]
    q, k, v, do = (randn((B, H, L, D), dtype, s) for s in (1, 2, 3, 4))
    g = torch.Generator().manual_seed(5)
    bias, tau = torch.randn(H, W, generator=g) * 0.02, torch.full((H,), -1.0)
    varlen = torch.tensor(lens)
    ref = lazy_attention_grads_analytic(q.cpu(), k.cpu(), v.cpu(), bias, tau, do.cpu(), W, varlen,
                                        round_to=round_to(dtype))
    for t in (q, k, v, do):
        for b, n in enumerate(lens):
            t[b, :, n:] = float("nan")
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v, bias.cuda(), tau.cuda())]
    out = pkg.lazy_attention_triton(*leaves, window_size=W, varlen=varlen.cuda().int())
    out.backward(do)
    for name, mine, r in zip(("out", "dq", "dk", "dv", "dbias", "dtau"), [out] + [t.grad for t in leaves], ref):
        assert torch.isfinite(mine).all(), name
        scale = 1.0 if name in ("out", "dq", "dk", "dv") else max(1.0, float(r.abs().max()))
        assert close(mine, r, dtype, scale=scale), (name, maxdiff(mine, r))


def test_check_status_is_clean_after_normal_work():
    q, k, v = (randn((1, 1, 256, 128), torch.bfloat16, s) for s in (1, 2, 3))
    pkg.adasplash(q, k, v, alpha=1.5, is_causal=True)
    check_status(q.device)       # fla_check_status: FLA_OK


@pytest.mark.parametrize("alpha,flags", [(2.0, 0), (1.5, 4), (1.5, 0)])
def test_runs_repeat_bit_for_bit(alpha, flags):
    """The candidate path's bookkeeping depends on how the warps interleave; the thresholds it ends with do not
    (closed-form finish from integer sums over the support), so outputs and gradients repeat exactly."""
    B, H, L, D, dtype = 2, 4, 4096, 128, torch.bfloat16
    set_flags(flags)
    q, k, v, do = (randn((B, H, L, D), dtype, s) for s in (1, 2, 3, 4))
    runs = []
    for _ in range(3):
        leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
        out = pkg.adasplash(*leaves, alpha=alpha, is_causal=True)
        out.backward(do)
        runs.append([out.detach()] + [t.grad for t in leaves])
    for other in runs[1:]:
        for name, a, b in zip(("out", "dq", "dk", "dv"), runs[0], other):
            assert torch.equal(a, b), (name, maxdiff(a, b))
