"""Dense CPU restatement of Lazy Attention (windowed head-wise positional bias +
elastic softmax ``ReLU(softmax + tau/i)``).

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).  PINNED against the
reference's own kernels run through the Triton CPU interpreter; the fixtures and
the script that made them live in ``tests/golden``.

Semantics follow the reference's kernels, ``lazy_attention_triton.py``:
  * scores ``q.k/sqrt(D)`` plus ``bias[h, i-j]`` for ``0 <= i-j < W`` (``:58-73``;
    the window is exclusive at W, the dense restatement of
    ``compare_scratch_flash_repro.py:7-51`` agrees),
  * causal mask and, with ``varlen``, a key-padding mask (``:74-78``),
  * softmax over the valid keys (``:80-88``),
  * ``A = max(P + tau_h/(i+1), 0)`` with i the 0-based absolute row, zero above
    the diagonal (``:158-168``), ``O = A V`` with A rounded to V's dtype (``:172``),
  * rows at or beyond ``varlen`` produce zeros and receive zero gradients
    (``tests/test_lazy_attention_varlen.py:42-45,164-169``).
Gradients come from autograd over this dense graph; ReLU's derivative at 0 is 0,
which is the kernels' strict ``P + tau/i > 0`` test (``:259-262``).
"""
from __future__ import annotations

import math

import torch


def lazy_attention_ref(q, k, v, bias, tau, window_size=None, varlen=None,
                       work_dtype=torch.float64, round_probs=True):
    """Dense forward in ``work_dtype``; differentiable w.r.t. every float input.
    Returns the output in ``work_dtype`` (cast it yourself for dtype parity)."""
    B, H, L, D = q.shape
    W = bias.shape[1] if window_size is None else int(window_size)
    qf, kf, vf = (t.to(work_dtype) for t in (q, k, v))
    bf, tf = bias.to(work_dtype), tau.to(work_dtype)
    s = torch.matmul(qf, kf.transpose(-1, -2)) / math.sqrt(D)
    idx = torch.arange(L)
    dist = idx[:, None] - idx[None, :]
    in_win = (dist >= 0) & (dist < W)
    bias_full = bf[:, dist.clamp(0, max(W - 1, 0)).clamp(max=bf.shape[1] - 1)] * in_win.to(work_dtype)
    s = s + bias_full[None]
    valid = (dist >= 0)[None, None].expand(B, 1, L, L)
    if varlen is not None:
        key_ok = idx[None, :] < varlen.to(torch.int64)[:, None]
        valid = valid & key_ok[:, None, None, :]
    s = s.masked_fill(~valid, -torch.inf)
    p = torch.softmax(s, dim=-1)
    tau_term = tf.view(1, H, 1, 1) / (idx + 1).to(work_dtype).view(1, 1, L, 1)
    a = torch.relu(p + tau_term)
    a = torch.where(valid, a, torch.zeros_like(a))
    if round_probs and q.dtype != work_dtype:
        # straight-through rounding to the input dtype before the PV product
        a = a + (a.detach().to(q.dtype).to(work_dtype) - a.detach())
    out = torch.matmul(a, vf)
    if varlen is not None:
        live = (idx[None, :] < varlen.to(torch.int64)[:, None])[:, None, :, None]
        out = out * live.to(work_dtype)
    return out


def lazy_attention_grads_ref(q, k, v, bias, tau, do, window_size=None, varlen=None,
                             work_dtype=torch.float64):
    """(out, dq, dk, dv, dbias, dtau) of the dense graph, all in ``work_dtype``.
    dbias has the shape of ``bias`` (columns at or beyond the window get 0),
    dtau the shape of ``tau``; both summed over the batch."""
    leaves = [t.detach().to(work_dtype).clone().requires_grad_(True) for t in (q, k, v, bias, tau)]
    out = lazy_attention_ref(*leaves, window_size=window_size, varlen=varlen,
                             work_dtype=work_dtype, round_probs=False)
    grads = torch.autograd.grad(out, leaves, do.to(work_dtype), allow_unused=True)
    grads = [g if g is not None else torch.zeros_like(l) for g, l in zip(grads, leaves)]
    return (out.detach(), *grads)


def lazy_attention_grads_analytic(q, k, v, bias, tau, do, window_size=None, varlen=None,
                                  work_dtype=torch.float64, round_to=None):
    """Same results as ``lazy_attention_grads_ref`` from the closed-form backward the reference's
    kernels evaluate (``lazy_attention_triton.py:253-268, 366-391, 476-494``):
    ``dA = dO V^T``, ``M = [P + tau/i > 0]``, ``delta = sum_j P M dA``, ``dS = P (M dA - delta)``,
    ``dQ = dS K / sqrt(D)``, ``dK = dS^T Q / sqrt(D)``, ``dV = A^T dO``,
    ``dbias[h, w] = sum_{b, i-j=w} dS``, ``dtau_h = sum_{b,i} (sum_j M dA) / i``.

    ``round_to`` (a 16-bit dtype) additionally rounds A and dS to that type before the second
    products, as those kernels do (``:172, :379, :490, :494``); the sums for dbias / dtau stay
    unrounded, as there."""
    B, H, L, D = q.shape
    W = bias.shape[1] if window_size is None else int(window_size)
    qf, kf, vf, dof = (t.to(work_dtype) for t in (q, k, v, do))
    bf, tf = bias.to(work_dtype), tau.to(work_dtype)
    scale = 1.0 / math.sqrt(D)
    idx = torch.arange(L)
    dist = idx[:, None] - idx[None, :]
    in_win = (dist >= 0) & (dist < W)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    s = s + (bf[:, dist.clamp(0, max(W - 1, 0)).clamp(max=bf.shape[1] - 1)] * in_win.to(work_dtype))[None]
    valid = (dist >= 0)[None, None].expand(B, 1, L, L)
    live = torch.ones(B, 1, L, 1, dtype=torch.bool)
    if varlen is not None:
        key_ok = idx[None, :] < varlen.to(torch.int64)[:, None]
        valid = valid & key_ok[:, None, None, :]
        live = key_ok[:, None, :, None]
    p = torch.softmax(s.masked_fill(~valid, -torch.inf), dim=-1)
    tau_term = tf.view(1, H, 1, 1) / (idx + 1).to(work_dtype).view(1, 1, L, 1)
    m = ((p + tau_term) > 0) & valid & live
    a = torch.where(m, p + tau_term, torch.zeros_like(p))

    def rnd(t):
        return t if round_to is None else t.to(round_to).to(work_dtype)

    dof = dof * live.to(work_dtype)
    out = torch.matmul(rnd(a), vf)
    da = torch.matmul(dof, vf.transpose(-1, -2))
    mda = torch.where(m, da, torch.zeros_like(da))
    delta = (p * mda).sum(-1, keepdim=True)
    ds = p * (mda - delta) * (valid & live).to(work_dtype)
    dq = torch.matmul(rnd(ds), kf) * scale
    dk = torch.matmul(rnd(ds).transpose(-1, -2), qf) * scale
    dv = torch.matmul(rnd(a).transpose(-1, -2), dof)
    dbias = torch.zeros_like(bf)
    ds_h = ds.sum(0)                                  # [H, L, L]
    for w in range(min(W, L)):
        dbias[:, w] = torch.diagonal(ds_h, offset=-w, dim1=-2, dim2=-1).sum(-1)
    dtau = (mda.sum(-1) / (idx + 1).to(work_dtype)).sum(dim=(0, 2)).view(tau.shape)
    return out, dq, dk, dv, dbias, dtau


def lazy_attention_rows_ref(q, k, v, do, bias_h, tau_h, rows, window_size, length=None,
                            work_dtype=torch.float32, round_to=None):
    """``lazy_attention_grads_analytic`` for ONE (batch, head) pair and a subset of its query rows
    (bounded memory at long sequences).  ``q, k, v, do``: [L, D]; ``bias_h``: [W'] row of the bias
    table of this head; ``tau_h``: scalar; ``rows``: 1-D int64 tensor.  Returns a dict with
    ``out``, ``dq`` [R, D], the dense row blocks ``a`` (rounded to ``round_to``) and ``ds``
    (``ds`` unrounded for dbias, ``ds_r`` rounded for the products) [R, L], and this block's
    contributions ``dbias`` [W'] and ``dtau`` (scalar).  dK / dV of a key range follow from
    ``ds_r[:, keys].T @ q[rows] / sqrt(D)`` and ``a[:, keys].T @ do[rows]`` once ``rows`` holds
    every row that can see those keys."""
    L, D = q.shape
    n = L if length is None else int(length)
    W = int(window_size)
    kf, vf = k.to(work_dtype), v.to(work_dtype)
    qr, dor = q[rows].to(work_dtype), do[rows].to(work_dtype)
    bf = bias_h.to(work_dtype)
    scale = 1.0 / math.sqrt(D)
    cols = torch.arange(L)
    dist = rows[:, None] - cols[None, :]
    in_win = (dist >= 0) & (dist < W)
    s = qr @ kf.t() * scale
    s = s + bf[dist.clamp(0, max(W - 1, 0)).clamp(max=bf.shape[0] - 1)] * in_win.to(work_dtype)
    valid = (dist >= 0) & (cols[None, :] < n)
    live = (rows < n)[:, None]
    p = torch.softmax(s.masked_fill(~valid, -torch.inf), dim=-1)
    p = torch.where(valid, p, torch.zeros_like(p))
    tau_term = tau_h.to(work_dtype) / (rows + 1).to(work_dtype)[:, None]
    m = ((p + tau_term) > 0) & valid & live
    a = torch.where(m, p + tau_term, torch.zeros_like(p))

    def rnd(t):
        return t if round_to is None else t.to(round_to).to(work_dtype)

    dor = dor * live.to(work_dtype)
    out = rnd(a) @ vf
    da = dor @ vf.t()
    mda = torch.where(m, da, torch.zeros_like(da))
    delta = (p * mda).sum(-1, keepdim=True)
    ds = p * (mda - delta) * (valid & live).to(work_dtype)
    dq = rnd(ds) @ kf * scale
    dbias = torch.zeros_like(bf)
    dbias.index_add_(0, dist.clamp(0, bf.shape[0] - 1).reshape(-1), (ds * in_win.to(work_dtype)).reshape(-1))
    dtau = (mda.sum(-1) / (rows + 1).to(work_dtype)).sum()
    return {"out": out, "dq": dq, "a": rnd(a), "ds": ds, "ds_r": rnd(ds), "dbias": dbias, "dtau": dtau}
