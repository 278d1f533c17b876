"""Dense CPU restatement of alpha-entmax and alpha-entmax attention.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).  PARITY UNPINNED beyond
the analytic known answers: the reference's own implementation of this path is
not part of its checkout and the arithmetic oracle of its tests is the
third-party ``entmax`` package (``entmax_bisect``; unpinned,
``requirements-dev.txt:5``), unavailable offline.  What follows restates the
published definition:

    entmax_alpha(x)_j = [ (alpha-1) x_j - tau ]_+ ^ (1/(alpha-1)),
    tau the unique root of  f(tau) = sum_j [ (alpha-1) x_j - tau ]_+^(1/(alpha-1)) - 1,

solved by bracketed bisection on [max - 1, max - n^-(alpha-1)] (in (alpha-1)x
units) run to convergence in float64.

The attention wrapper follows ``tests/test_adasplash.py:22-60`` of the
reference: scores / sqrt(D), key-padding mask from ``varlen`` (``:10-13``),
lower-triangular causal mask (``:16-19``), entmax over the float scores
(``:53``), probabilities rounded to the input dtype before ``P @ V`` (``:53-54``),
padded query rows filled with zero (``:57-58``).
"""
from __future__ import annotations

import math
import time

import torch

BLOCK_M = 128  # query rows per block-mask bit
BLOCK_N = 64   # key columns per block-mask bit


def _tau_bisect(X: torch.Tensor, alpha: float, n_iter: int) -> torch.Tensor:
    """Threshold of every row of ``X`` (already multiplied by alpha-1; masked
    entries are -inf).  Plain bisection, ``n_iter`` halvings, returns the
    midpoint of the last bracket.  Rows without any finite entry return +inf."""
    e = 1.0 / (alpha - 1.0)
    finite = torch.isfinite(X)
    n = finite.sum(-1, keepdim=True).clamp(min=1).to(X.dtype)
    mx = torch.where(finite, X, torch.full_like(X, -torch.inf)).amax(-1, keepdim=True)
    dead = ~torch.isfinite(mx)
    mx = torch.where(dead, torch.zeros_like(mx), mx)
    lo = mx - 1.0
    hi = mx - n.pow(-(alpha - 1.0))
    for _ in range(n_iter):
        mid = 0.5 * (lo + hi)
        f = (X - mid).clamp(min=0).pow(e).sum(-1, keepdim=True) - 1.0
        ge = f >= 0
        lo = torch.where(ge, mid, lo)
        hi = torch.where(ge, hi, mid)
    tau = 0.5 * (lo + hi)
    return torch.where(dead, torch.full_like(tau, torch.inf), tau)


def entmax_ref(x: torch.Tensor, alpha: float = 1.5, dim: int = -1,
               n_iter: int | None = None, work_dtype=torch.float64) -> torch.Tensor:
    """alpha-entmax of ``x`` along ``dim``; entries equal to -inf are masked.

    ``n_iter=None`` is the converged solution (64 halvings in float64); an
    integer gives that many halvings followed by renormalisation, the recipe
    the CPU baseline is timed with.  Result in ``work_dtype``."""
    xs = x.to(work_dtype).movedim(dim, -1)
    X = xs * (alpha - 1.0)
    tau = _tau_bisect(X, alpha, 64 if n_iter is None else n_iter)
    p = (X - tau).clamp(min=0).pow(1.0 / (alpha - 1.0))
    p = torch.where(torch.isfinite(X), p, torch.zeros_like(p))
    if n_iter is not None:
        p = p / p.sum(-1, keepdim=True).clamp(min=1e-30)
    return p.movedim(-1, dim)


def entmax_bwd_ref(p: torch.Tensor, dy: torch.Tensor, alpha: float, dim: int = -1) -> torch.Tensor:
    """Vector-Jacobian product of alpha-entmax at output ``p``:
    ``dx = U * (dy - sum(U dy)/sum(U))`` with ``U = p^(2-alpha)`` on the support."""
    p_ = p.movedim(dim, -1)
    dy_ = dy.to(p.dtype).movedim(dim, -1)
    supp = p_ > 0
    u = torch.where(supp, p_.clamp(min=1e-300 if p.dtype == torch.float64 else 1e-38).pow(2.0 - alpha),
                    torch.zeros_like(p_))
    q = (u * dy_).sum(-1, keepdim=True) / u.sum(-1, keepdim=True).clamp(min=1e-30)
    return (u * (dy_ - q)).movedim(-1, dim)


def _valid_mask(B, L, varlen, is_causal, device="cpu"):
    """[B,1,L,L] boolean: key j usable by query i."""
    valid = torch.ones(B, 1, L, L, dtype=torch.bool, device=device)
    if varlen is not None:
        key_ok = torch.arange(L, device=device)[None, :] < varlen.to(device)[:, None]
        valid = valid & key_ok[:, None, None, :]
    if is_causal:
        valid = valid & torch.tril(torch.ones(L, L, dtype=torch.bool, device=device))[None, None]
    return valid


def entmax_attention_probs_ref(q, k, alpha=1.5, varlen=None, is_causal=False,
                               n_iter=None, work_dtype=torch.float64):
    """Dense probabilities P [B,H,L,L] (in ``work_dtype``) and the row thresholds
    tau [B,H,L] in (alpha-1)*score units.  Rows at or beyond ``varlen`` are
    computed like any other row here; callers zero them."""
    B, H, L, D = q.shape
    s = torch.matmul(q.to(work_dtype), k.to(work_dtype).transpose(-1, -2)) / math.sqrt(D)
    valid = _valid_mask(B, L, varlen, is_causal)
    s = s.masked_fill(~valid, -torch.inf)
    X = s * (alpha - 1.0)
    tau = _tau_bisect(X, alpha, 64 if n_iter is None else n_iter)
    p = (X - tau).clamp(min=0).pow(1.0 / (alpha - 1.0))
    p = torch.where(valid.expand_as(p), p, torch.zeros_like(p))
    if n_iter is not None:
        p = p / p.sum(-1, keepdim=True).clamp(min=1e-30)
    return p, tau.squeeze(-1)


def _row_live(B, L, varlen):
    if varlen is None:
        return torch.ones(B, 1, L, 1, dtype=torch.bool)
    return (torch.arange(L)[None, :] < varlen[:, None])[:, None, :, None]


def entmax_attention_ref(q, k, v, alpha=1.5, varlen=None, is_causal=False,
                         n_iter=None, work_dtype=torch.float64):
    """Output of alpha-entmax attention in the dtype of ``q``
    (``tests/test_adasplash.py:22-60``)."""
    B, H, L, D = q.shape
    p, _ = entmax_attention_probs_ref(q, k, alpha, varlen, is_causal, n_iter, work_dtype)
    p = p.to(q.dtype).to(work_dtype)          # probabilities are rounded to the input dtype first
    out = torch.matmul(p, v.to(work_dtype))
    out = out.masked_fill(~_row_live(B, L, varlen), 0.0)
    return out.to(q.dtype)


def entmax_attention_bwd_ref(q, k, v, do, alpha=1.5, varlen=None, is_causal=False,
                             n_iter=None, work_dtype=torch.float64, cast=True, round_to=None):
    """(out, dq, dk, dv) through the analytic entmax Jacobian
    ``diag(U) - U U^T / sum(U)``, ``U = P^(2-alpha)`` on the support; this is the
    gradient autograd produces through ``entmax_bisect`` in the reference's
    backward test (``tests/test_adasplash.py:94-122``).  Everything is kept in
    ``work_dtype``; results are cast to the dtype of ``q`` unless ``cast`` is False.

    ``round_to`` (a 16-bit dtype) rounds P and dS to that type before the second products,
    the way a 16-bit tensor-core kernel (and the reference's oracle, for P) evaluates them."""
    B, H, L, D = q.shape
    qf, kf, vf, dof = (t.to(work_dtype) for t in (q, k, v, do))
    p, _ = entmax_attention_probs_ref(q, k, alpha, varlen, is_causal, n_iter, work_dtype)
    live = _row_live(B, L, varlen).to(work_dtype)
    p = p * live
    dof = dof * live
    def rnd(t):
        return t if round_to is None else t.to(round_to).to(work_dtype)

    out = torch.matmul(p.to(q.dtype).to(work_dtype), vf)
    dv = torch.matmul(rnd(p).transpose(-1, -2), dof)
    dp = torch.matmul(dof, vf.transpose(-1, -2))
    ds = entmax_bwd_ref(p, dp, alpha)
    ds = rnd(torch.where(p > 0, ds, torch.zeros_like(ds)))
    dq = torch.matmul(ds, kf) / math.sqrt(D)
    dk = torch.matmul(ds.transpose(-1, -2), qf) / math.sqrt(D)
    return tuple(t.to(q.dtype) if cast else t for t in (out, dq, dk, dv))


def block_mask_ref(p: torch.Tensor, varlen=None, block_m: int = BLOCK_M, block_n: int = BLOCK_N):
    """[B,H,Tr,Tc] boolean: block (I,J) holds at least one non-zero probability
    of a live row.  One bit per (query block, key block), the side product the
    block-masked variant keeps (``README.md:47-48`` of the reference)."""
    B, H, L, _ = p.shape
    tr = (L + block_m - 1) // block_m
    tc = (L + block_n - 1) // block_n
    nz = (p > 0) & _row_live(B, L, varlen)
    pad = torch.zeros(B, H, tr * block_m, tc * block_n, dtype=torch.bool)
    pad[:, :, :L, :L] = nz
    return pad.view(B, H, tr, block_m, tc, block_n).any(dim=5).any(dim=3)


def entmax_exact_sort(x: torch.Tensor, alpha: float) -> torch.Tensor:
    """Closed-form entmax for alpha = 2 (sparsemax) and alpha = 1.5 by sorting,
    float64, last dim.  Independent of the bisection above; used to check it."""
    xs = x.to(torch.float64)
    n = xs.shape[-1]
    srt, _ = torch.sort(xs, dim=-1, descending=True)
    ks = torch.arange(1, n + 1, dtype=torch.float64)
    if alpha == 2.0:
        cs = srt.cumsum(-1)
        tau_k = (cs - 1.0) / ks
        supp = (srt > tau_k).sum(-1, keepdim=True)
        tau = tau_k.gather(-1, supp - 1)
        return (xs - tau).clamp(min=0)
    if alpha == 1.5:
        z = srt / 2.0
        mean = z.cumsum(-1) / ks
        mean_sq = (z * z).cumsum(-1) / ks
        ss = ks * (mean_sq - mean * mean)
        delta = ((1.0 - ss) / ks).clamp(min=0)
        tau_k = mean - delta.sqrt()
        supp = (tau_k <= z).sum(-1, keepdim=True)
        tau = tau_k.gather(-1, supp - 1)
        return (xs / 2.0 - tau).clamp(min=0) ** 2
    raise ValueError("closed form only for alpha in {1.5, 2.0}")


def bisect10_entmax(scores: torch.Tensor, alpha: float, n_iter: int = 10) -> torch.Tensor:
    """The timed CPU-baseline recipe: ``n_iter`` bisection halvings followed by
    renormalisation, in the dtype of ``scores`` (fp32 for the baseline)."""
    return entmax_ref(scores, alpha, n_iter=n_iter, work_dtype=scores.dtype)


def cpu_reference_fwd_bwd(q, k, v, do, alpha=1.5, is_causal=True, n_iter=10):
    """One forward + backward (w.r.t. q, k, v) of the dense pure-PyTorch path:
    scores = QK^T/sqrt(D) -> entmax by ``n_iter`` bisection steps -> PV, then the
    Jacobian backward.  All in the dtype of ``q`` on the host cores.  Returns
    (out, dq, dk, dv, seconds)."""
    B, H, L, D = q.shape
    t0 = time.perf_counter()
    s = torch.matmul(q, k.transpose(-1, -2)) / math.sqrt(D)
    if is_causal:
        s = s.masked_fill(~torch.tril(torch.ones(L, L, dtype=torch.bool)), -torch.inf)
    p = bisect10_entmax(s, alpha, n_iter)
    out = torch.matmul(p, v)
    dv = torch.matmul(p.transpose(-1, -2), do)
    dp = torch.matmul(do, v.transpose(-1, -2))
    ds = entmax_bwd_ref(p, dp, alpha) / math.sqrt(D)
    dq = torch.matmul(ds, k)
    dk = torch.matmul(ds.transpose(-1, -2), q)
    return out, dq, dk, dv, time.perf_counter() - t0


def entmax_attention_rows_ref(q, k, v, do, rows, alpha=1.5, is_causal=False, length=None,
                              work_dtype=torch.float32, round_to=None):
    """The same mathematics as ``entmax_attention_bwd_ref`` for ONE (batch, head) pair and a subset
    of its query rows, so that long sequences can be checked with bounded memory.

    ``q, k, v, do``: [L, D]; ``rows``: 1-D int64 tensor of query rows; ``length``: valid leading
    tokens (``varlen`` of this batch element).  Returns a dict with ``out``, ``dq`` [R, D],
    ``tau`` [R] and the dense row blocks ``p``, ``ds`` [R, L] (rounded to ``round_to`` when given,
    as the second products see them).  dK and dV of a key range are
    ``ds[:, keys].T @ q[rows] / sqrt(D)`` and ``p[:, keys].T @ do[rows]`` once ``rows`` holds every
    row that can see those keys.  Rows at or beyond ``length`` give zeros."""
    L, D = q.shape
    n = L if length is None else int(length)
    kf, vf = k.to(work_dtype), v.to(work_dtype)
    qr, dor = q[rows].to(work_dtype), do[rows].to(work_dtype)
    s = qr @ kf.t() / math.sqrt(D)
    cols = torch.arange(L)
    valid = (cols[None, :] < n).expand(len(rows), L).clone()
    if is_causal:
        valid &= cols[None, :] <= rows[:, None]
    live = (rows < n)[:, None]
    X = s.masked_fill(~valid, -torch.inf) * (alpha - 1.0)
    tau = _tau_bisect(X, alpha, 64)
    p = (X - tau).clamp(min=0).pow(1.0 / (alpha - 1.0))
    p = torch.where(valid & live, p, torch.zeros_like(p))
    dor = dor * live.to(work_dtype)

    def rnd(t):
        return t if round_to is None else t.to(round_to).to(work_dtype)

    out = p.to(q.dtype).to(work_dtype) @ vf
    dp = dor @ vf.t()
    ds = entmax_bwd_ref(p, dp, alpha)
    ds = rnd(torch.where(p > 0, ds, torch.zeros_like(ds)))
    dq = ds @ kf / math.sqrt(D)
    return {"out": out, "dq": dq, "tau": torch.where(live[:, 0], tau[:, 0], torch.zeros_like(tau[:, 0])),
            "p": rnd(p), "ds": ds}
