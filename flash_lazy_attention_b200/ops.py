"""Host side of the operator API: PyTorch autograd Functions over the C ABI.

The public functions keep the reference's signatures:
  * ``lazy_attention_triton(q, k, v, bias, tau, window_size=None, varlen=None)``
    (``lazy_attention_triton.py:503-541`` of the reference),
  * ``adasplash(q, k, v, alpha=1.5, niter=10, is_causal=False, varlen=None)`` and
    ``adasplash_no_block_mask(...)`` (``README.md:37-57``; the default ``is_causal=False``
    is what ``tests/test_adasplash.py:109-115`` requires),
  * ``triton_entmax(x, alpha=1.5, n_iter=10, fast_math=True)``
    (``tests/test_triton_entmax.py:27,41``).
PyTorch is used for device memory and streams only; all arithmetic is in libflashlazy.
Work is enqueued on the current stream of the inputs' device without synchronising.
"""
from __future__ import annotations

import os

import torch

from . import _lib
from ._lib import AttnGeom, Tensor4

_DTYPES = {torch.float32: _lib.FLA_F32, torch.float16: _lib.FLA_F16, torch.bfloat16: _lib.FLA_BF16}

# FLA_PATH=simt|tcgen05 pins the kernel family (testing); default lets the library choose.
_PATH_ENV = {"": _lib.PATH_AUTO, "auto": _lib.PATH_AUTO, "simt": _lib.PATH_SIMT, "tcgen05": _lib.PATH_TCGEN05}
_forced_path = None
_flags = 0


def set_flags(flags: int) -> None:
    """fla_attn_geom.flags for the calls that follow (``_lib.FLAG_*``; 0 restores normal operation)."""
    global _flags
    _flags = int(flags)


def set_path(name: str | None) -> None:
    """Pin the kernel family ("simt", "tcgen05") or None/"auto" for the library's choice."""
    global _forced_path
    _forced_path = None if name is None else _PATH_ENV[name]


def _path() -> int:
    if _forced_path is not None:
        return _forced_path
    return _PATH_ENV[os.environ.get("FLA_PATH", "").lower()]


def _check_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: this library has no CPU path")
    if t.dtype not in _DTYPES:
        raise TypeError(f"{name}: unsupported dtype {t.dtype} (float32, float16, bfloat16)")


def _unit_inner(t: torch.Tensor) -> torch.Tensor:
    return t if t.stride(-1) == 1 else t.contiguous()


def _tma_friendly(t: torch.Tensor) -> torch.Tensor:
    """Gradients arrive with whatever strides autograd produced; copy them unless a TMA tensor map
    can describe them (unit inner stride, 16-byte aligned base, outer strides multiples of 8)."""
    ok = (t.stride(-1) == 1 and t.data_ptr() % 16 == 0
          and all(s_ % 8 == 0 for s_ in t.stride()[:-1]))
    return t if ok else t.contiguous()


def _t4(t: torch.Tensor) -> Tensor4:
    r = Tensor4()
    r.ptr = t.data_ptr()
    for i in range(4):
        r.stride[i] = t.stride(i)
    return r


_status_bufs: dict = {}


def _status_buf(device: torch.device) -> torch.Tensor:
    """Per-device int32[32] the tensor-core kernels report into (see fla_attn_geom.status)."""
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    buf = _status_bufs.get(key)
    if buf is None:
        buf = torch.zeros(32, dtype=torch.int32, device=device)
        _status_bufs[key] = buf
    return buf


def read_status(device=None, reset: bool = False) -> dict:
    """Synchronising read of the device status words: {"error", "wait_tag", "block", "tile_mmas",
    "list_ctas", "pass_ctas", "kernel_ms", "cta_ms"}.
    ``tile_mmas`` counts 128x128xD tile products issued by tensor-core kernels since the last reset;
    ``cta_ms`` is the sum of the lifetimes of a kernel's CTAs (one CTA per SM: divided by SMs x kernel_ms it
    is the share of the launch during which the SMs were occupied)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    buf = _status_buf(device)
    vals = buf.cpu().tolist()
    if reset:
        buf.zero_()
    return {"error": vals[0], "wait_tag": vals[1], "block": vals[2],
            "tile_mmas": (vals[4] & 0xFFFFFFFF) | ((vals[5] & 0xFFFFFFFF) << 32),
            "list_ctas": vals[6], "pass_ctas": vals[7], "kernel_ms": _kernel_ms(vals),
            "cta_ms": {name: ((vals[26 + 2 * i] & 0xFFFFFFFF) | ((vals[27 + 2 * i] & 0xFFFFFFFF) << 32)) * 1e-6
                       for i, name in enumerate(("fwd", "dq", "dkdv"))}}


def _kernel_ms(vals) -> dict:
    """Durations the kernels clocked themselves (earliest CTA start to latest CTA end, GPU global timer)
    since the status words were last cleared; None for a kernel that did not run."""
    out = {}
    for i, name in enumerate(("fwd", "dq", "dkdv")):
        w = [(vals[8 + 4 * i + 2 * j] & 0xFFFFFFFF) | ((vals[9 + 4 * i + 2 * j] & 0xFFFFFFFF) << 32) for j in range(2)]
        out[name] = None if w[0] == 0 or w[1] == 0 else (w[1] - ((~w[0]) & 0xFFFFFFFFFFFFFFFF)) * 1e-6
    return out


def check_status(device=None) -> None:
    """Raise if a kernel reported that one of its bounded waits ran out (fla_check_status: waits
    for the device's current stream)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    buf = _status_buf(device)
    with torch.cuda.device(device):
        rc = _lib.load().fla_check_status(buf.data_ptr(), torch.cuda.current_stream(device).cuda_stream)
    _lib.check(rc, "fla_check_status")


def _geom(q: torch.Tensor, causal: bool, varlen32, kv_heads: int = 0) -> AttnGeom:
    B, H, L, D = q.shape
    g = AttnGeom()
    g.B, g.H, g.L, g.D = B, H, L, D
    g.dtype = _DTYPES[q.dtype]
    g.causal = int(bool(causal))
    g.varlen = varlen32.data_ptr() if varlen32 is not None else None
    g.path = _path()
    g.status = _status_buf(q.device).data_ptr()
    g.flags = _flags
    g.Hkv = int(kv_heads)
    return g



def _varlen32(varlen, q):
    if varlen is None:
        return None
    if varlen.numel() != q.shape[0]:
        raise ValueError("varlen must hold one length per batch element")
    return varlen.to(device=q.device, dtype=torch.int32).contiguous()


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _qkv_checked(q, k, v):
    for n, t in (("q", q), ("k", k), ("v", v)):
        _check_cuda(t, n)
        if t.dim() != 4:
            raise ValueError(f"{n} must be [B, H, L, D]")
    if not (k.shape == v.shape and q.dtype == k.dtype == v.dtype):
        raise ValueError("k and v must share their shape, and q, k, v their dtype")
    if q.shape[0] != k.shape[0] or q.shape[2:] != k.shape[2:] or k.shape[1] < 1 or q.shape[1] % k.shape[1] != 0:
        raise ValueError("k, v must be [B, Hkv, L, D] with Hkv dividing the H of q [B, H, L, D]")
    return _unit_inner(q), _unit_inner(k), _unit_inner(v)


def _shared_kv(lib, q, k, v, causal, vl):
    """Grouped-query attention: k, v with fewer heads than q.  The tensor-core kernels read the shared heads
    in place (query head h uses head h // (H // Hkv)); where they cannot take the call, the heads are repeated
    here (what the reference's layers always do, examples/sw_attention_lazy.py:30-41) and autograd sums the
    gradients of the copies.  Returns (k, v, kv_heads for the geometry)."""
    H, Hkv = q.shape[1], k.shape[1]
    if Hkv == H:
        return k, v, 0
    with torch.cuda.device(q.device):
        if lib.fla_attn_uses_tensor_cores(_geom(q, causal, vl, Hkv), _t4(q), _t4(k), _t4(v)):
            return k, v, Hkv
    n_rep = H // Hkv
    return k.repeat_interleave(n_rep, dim=1), v.repeat_interleave(n_rep, dim=1), 0


# ---------------------------------------------------------------------------------------------
# alpha-entmax attention
# ---------------------------------------------------------------------------------------------
class EntmaxAttnFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, alpha, niter, is_causal, varlen, use_block_mask, kv_heads=0):
        lib = _lib.load()
        q, k, v = _qkv_checked(q, k, v)
        B, H, L, D = q.shape
        vl = _varlen32(varlen, q)
        with torch.cuda.device(q.device):
            g = _geom(q, is_causal, vl, kv_heads)
            # only the SIMT family's backward needs the aux buffers
            need_aux = any(ctx.needs_input_grad[:3]) and not lib.fla_attn_uses_tensor_cores(g, _t4(q), _t4(k), _t4(v))
            out = torch.empty((B, H, L, D), dtype=q.dtype, device=q.device)
            tau = torch.empty((B, H, L), dtype=torch.float32, device=q.device)
            aux_o = torch.empty((B, H, L, D), dtype=torch.float32, device=q.device) if need_aux else None
            aux_s = torch.empty((B, H, L), dtype=torch.float32, device=q.device) if need_aux else None
            mask = None
            if use_block_mask:
                words = lib.fla_block_mask_words(L)
                mask = torch.empty((B, H, (L + 127) // 128, words), dtype=torch.int32, device=q.device)
            rc = lib.fla_entmax_attn_fwd(g, _t4(q), _t4(k), _t4(v), _t4(out), float(alpha), int(niter),
                                         tau.data_ptr(), aux_o.data_ptr() if need_aux else None,
                                         aux_s.data_ptr() if need_aux else None,
                                         mask.data_ptr() if mask is not None else None, _stream(q))
            _lib.check(rc, "fla_entmax_attn_fwd")
        ctx.save_for_backward(q, k, v, tau, aux_o, aux_s, mask, vl)
        ctx.alpha, ctx.is_causal, ctx.kv_heads = float(alpha), bool(is_causal), int(kv_heads)
        ctx.block_mask = mask
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, tau, aux_o, aux_s, mask, vl = ctx.saved_tensors
        dq, dk, dv = entmax_attention_backward(q, k, v, do, tau, aux_o, aux_s, mask, vl, ctx.alpha, ctx.is_causal,
                                               ctx.kv_heads)
        return dq, dk, dv, None, None, None, None, None, None


def entmax_attention_backward(q, k, v, do, tau, aux_o, aux_s, mask, vl, alpha, is_causal, kv_heads=0):
    """(dq, dk, dv) from the forward's saved state (tau; aux_o, aux_s on the SIMT family; the block mask or None);
    ``vl``: int32 lengths on q's device or None."""
    lib = _lib.load()
    do = _tma_friendly(do)
    with torch.cuda.device(q.device):
        dq = torch.empty(q.shape, dtype=q.dtype, device=q.device)
        dk, dv = (torch.empty(k.shape, dtype=q.dtype, device=q.device) for _ in range(2))
        g = _geom(q, is_causal, vl, kv_heads)
        nbytes = lib.fla_entmax_attn_bwd_workspace(g)
        ws = torch.empty((nbytes,), dtype=torch.uint8, device=q.device)
        rc = lib.fla_entmax_attn_bwd(g, _t4(q), _t4(k), _t4(v), _t4(do), float(alpha), tau.data_ptr(),
                                     aux_o.data_ptr() if aux_o is not None else None,
                                     aux_s.data_ptr() if aux_s is not None else None,
                                     mask.data_ptr() if mask is not None else None,
                                     _t4(dq), _t4(dk), _t4(dv), ws.data_ptr(), nbytes, _stream(q))
        _lib.check(rc, "fla_entmax_attn_bwd")
    return dq, dk, dv


def _entmax_attn(q, k, v, alpha, niter, is_causal, varlen, use_block_mask):
    if torch.compiler.is_compiling():   # one opaque node in the traced graph (custom_ops.py)
        return torch.ops.flash_lazy.entmax_attn_fwd(q, k, v, float(alpha), int(niter), bool(is_causal), varlen,
                                                    bool(use_block_mask))[0]
    if k.dim() == 4 and q.dim() == 4 and k.shape[1] != q.shape[1] and q.is_cuda:
        q_, k_, v_ = _qkv_checked(q, k, v)
        k, v, kvh = _shared_kv(_lib.load(), q_, k_, v_, is_causal, _varlen32(varlen, q_))
        return EntmaxAttnFunc.apply(q, k, v, alpha, niter, is_causal, varlen, use_block_mask, kvh)
    return EntmaxAttnFunc.apply(q, k, v, alpha, niter, is_causal, varlen, use_block_mask, 0)


def adasplash(q, k, v, alpha=1.5, niter=10, is_causal=False, varlen=None):
    """Block-masked alpha-entmax flash attention, forward + backward.  k, v may have fewer heads than q
    (grouped-query attention: Hkv dividing H)."""
    return _entmax_attn(q, k, v, alpha, niter, is_causal, varlen, True)


def adasplash_no_block_mask(q, k, v, alpha=1.5, niter=10, is_causal=False, varlen=None):
    """Same mathematics without the block bitmask (less memory, every block visited)."""
    return _entmax_attn(q, k, v, alpha, niter, is_causal, varlen, False)


def entmax_attention_forward(q, k, v, alpha=1.5, niter=10, is_causal=False, varlen=None,
                             use_block_mask=True, need_aux=False, kv_heads=0):
    """Forward only, returning every side product: (out, tau, aux_o, aux_s, block_mask).
    The threshold rows ``tau`` are in (alpha-1)*score units; ``block_mask`` is an int32
    [B,H,ceil(L/128),words] bit array, bit J of a row = key block J (64 keys) is non-zero."""
    lib = _lib.load()
    q, k, v = _qkv_checked(q, k, v)
    B, H, L, D = q.shape
    vl = _varlen32(varlen, q)
    with torch.cuda.device(q.device):
        out = torch.empty((B, H, L, D), dtype=q.dtype, device=q.device)
        tau = torch.empty((B, H, L), dtype=torch.float32, device=q.device)
        aux_o = torch.empty((B, H, L, D), dtype=torch.float32, device=q.device) if need_aux else None
        aux_s = torch.empty((B, H, L), dtype=torch.float32, device=q.device) if need_aux else None
        mask = None
        if use_block_mask:
            mask = torch.empty((B, H, (L + 127) // 128, lib.fla_block_mask_words(L)), dtype=torch.int32,
                               device=q.device)
        g = _geom(q, is_causal, vl, kv_heads)
        rc = lib.fla_entmax_attn_fwd(g, _t4(q), _t4(k), _t4(v), _t4(out), float(alpha),
                                     int(niter), tau.data_ptr(), aux_o.data_ptr() if need_aux else None,
                                     aux_s.data_ptr() if need_aux else None,
                                     mask.data_ptr() if mask is not None else None, _stream(q))
        _lib.check(rc, "fla_entmax_attn_fwd")
    return out, tau, aux_o, aux_s, mask


def unpack_block_mask(mask: torch.Tensor, L: int) -> torch.Tensor:
    """int32 bit rows [B,H,Tr,words] -> bool [B,H,Tr,Tc] with Tc = ceil(L/64)."""
    tc = (L + 63) // 64
    bits = torch.arange(32, device=mask.device, dtype=torch.int32)
    expanded = ((mask.unsqueeze(-1) >> bits) & 1).bool().flatten(-2)
    return expanded[..., :tc]


# ---------------------------------------------------------------------------------------------
# Lazy Attention
# ---------------------------------------------------------------------------------------------
def lazy_attention_forward(q, k, v, bias, tau, window, varlen=None, need_aux=False, kv_heads=0):
    """Forward only: (out, lse, aux_o).  ``lse`` is the base-2 log-sum-exp of the rows (saved state of the backward);
    ``aux_o`` (fp32 [B,H,L,2D]) is what the SIMT family's backward needs, None unless asked for."""
    lib = _lib.load()
    q, k, v = _qkv_checked(q, k, v)
    B, H, L, D = q.shape
    if bias.dim() != 2 or bias.shape[0] != H or tau.numel() != H:
        raise ValueError("bias must be [H, W] and tau [H]")
    window = int(window)
    if window > bias.shape[1]:
        raise ValueError(f"window_size {window} exceeds the {bias.shape[1]} bias columns")
    vl = _varlen32(varlen, q)
    bias32 = bias.detach().to(device=q.device, dtype=torch.float32).contiguous()
    tau32 = tau.detach().to(device=q.device, dtype=torch.float32).contiguous().view(-1)
    with torch.cuda.device(q.device):
        g = _geom(q, True, vl, kv_heads)
        out = torch.empty((B, H, L, D), dtype=q.dtype, device=q.device)
        lse = torch.empty((B, H, L), dtype=torch.float32, device=q.device)
        aux_o = torch.empty((B, H, L, 2 * D), dtype=torch.float32, device=q.device) if need_aux else None
        rc = lib.fla_lazy_attn_fwd(g, _t4(q), _t4(k), _t4(v), _t4(out), bias32.data_ptr(),
                                   bias32.stride(0), tau32.data_ptr(), window, lse.data_ptr(),
                                   aux_o.data_ptr() if need_aux else None, _stream(q))
        _lib.check(rc, "fla_lazy_attn_fwd")
    return out, lse, aux_o


def lazy_attention_backward(q, k, v, out, do, bias, tau, window, lse, aux_o, vl, want_params, kv_heads=0):
    """(dq, dk, dv, dbias, dtau); dbias [H, bias columns] and dtau [H] are fp32 like the reference's
    (lazy_attention_triton.py:532-533) and None unless ``want_params``."""
    lib = _lib.load()
    do = _tma_friendly(do)
    H = q.shape[1]
    bias32 = bias.detach().to(device=q.device, dtype=torch.float32).contiguous()
    tau32 = tau.detach().to(device=q.device, dtype=torch.float32).contiguous().view(-1)
    with torch.cuda.device(q.device):
        dq = torch.empty(q.shape, dtype=q.dtype, device=q.device)
        dk, dv = (torch.empty(k.shape, dtype=q.dtype, device=q.device) for _ in range(2))
        dbias = dtau = None
        if want_params:
            dbias = torch.zeros(tuple(bias.shape), dtype=torch.float32, device=q.device)
            dtau = torch.zeros((H,), dtype=torch.float32, device=q.device)
        g = _geom(q, True, vl, kv_heads)
        nbytes = lib.fla_lazy_attn_bwd_workspace(g)
        ws = torch.empty((nbytes,), dtype=torch.uint8, device=q.device)
        rc = lib.fla_lazy_attn_bwd(g, _t4(q), _t4(k), _t4(v), _t4(out), _t4(do), bias32.data_ptr(),
                                   bias32.stride(0), tau32.data_ptr(), int(window), lse.data_ptr(),
                                   aux_o.data_ptr() if aux_o is not None else None, _t4(dq), _t4(dk), _t4(dv),
                                   dbias.data_ptr() if want_params else None,
                                   dbias.stride(0) if want_params else 0,
                                   dtau.data_ptr() if want_params else None,
                                   ws.data_ptr(), nbytes, _stream(q))
        _lib.check(rc, "fla_lazy_attn_bwd")
    return dq, dk, dv, dbias, dtau


class LazyAttentionFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, bias, tau, window_size, varlen=None, kv_heads=0):
        lib = _lib.load()
        q, k, v = _qkv_checked(q, k, v)
        vl = _varlen32(varlen, q)
        with torch.cuda.device(q.device):
            g = _geom(q, True, vl, kv_heads)
            need_aux = any(ctx.needs_input_grad[:5]) and not lib.fla_attn_uses_tensor_cores(g, _t4(q), _t4(k), _t4(v))
        out, lse, aux_o = lazy_attention_forward(q, k, v, bias, tau, window_size, vl, need_aux, kv_heads)
        bias32 = bias.detach().to(device=q.device, dtype=torch.float32).contiguous()
        tau32 = tau.detach().to(device=q.device, dtype=torch.float32).contiguous().view(-1)
        ctx.save_for_backward(q, k, v, out, bias32, tau32, lse, aux_o, vl)
        ctx.window, ctx.kv_heads = int(window_size), int(kv_heads)
        ctx.bias_shape, ctx.tau_shape = tuple(bias.shape), tuple(tau.shape)
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, out, bias32, tau32, lse, aux_o, vl = ctx.saved_tensors
        want_params = ctx.needs_input_grad[3] or ctx.needs_input_grad[4]
        dq, dk, dv, dbias, dtau = lazy_attention_backward(q, k, v, out, do, bias32, tau32, ctx.window, lse, aux_o, vl,
                                                          want_params, ctx.kv_heads)
        if want_params:
            dtau = dtau.view(ctx.tau_shape)
        return dq, dk, dv, dbias, dtau, None, None, None


def lazy_attention_triton(q, k, v, bias, tau, window_size=None, varlen=None):
    """Lazy Attention: scores + windowed head-wise bias, softmax, ReLU(P + tau/i), times V.
    ``window_size`` defaults to ``bias.shape[1]`` (lazy_attention_triton.py:503-507).  k, v may have fewer
    heads than q (grouped-query attention: Hkv dividing H); bias and tau are per query head."""
    if window_size is None:
        window_size = bias.shape[1]
    if torch.compiler.is_compiling():   # one opaque node in the traced graph (custom_ops.py)
        return torch.ops.flash_lazy.lazy_attn_fwd(q, k, v, bias, tau, int(window_size), varlen)[0]
    kvh = 0
    if k.dim() == 4 and q.dim() == 4 and k.shape[1] != q.shape[1] and q.is_cuda:
        q_, k_, v_ = _qkv_checked(q, k, v)
        k, v, kvh = _shared_kv(_lib.load(), q_, k_, v_, True, _varlen32(varlen, q_))
    return LazyAttentionFunc.apply(q, k, v, bias, tau, window_size, varlen, kvh)


# ---------------------------------------------------------------------------------------------
# stand-alone entmax
# ---------------------------------------------------------------------------------------------
def entmax_rows_forward(x, alpha, n_iter, fast_math):
    """y = entmax(x) over the last dimension, in x's dtype (float64 is computed in float32 and returned so)."""
    lib = _lib.load()
    if not x.is_cuda:
        raise RuntimeError("x must be a CUDA tensor: this library has no CPU path")
    xc = x.contiguous()
    if xc.dtype == torch.float64:
        xc = xc.float()
    if xc.dtype not in _DTYPES:
        raise TypeError(f"unsupported dtype {x.dtype}")
    cols = xc.shape[-1] if xc.dim() > 0 else 1
    rows = xc.numel() // max(cols, 1)
    with torch.cuda.device(x.device):
        y = torch.empty_like(xc)
        rc = lib.fla_entmax_fwd(xc.data_ptr(), y.data_ptr(), rows, cols, float(alpha), int(n_iter),
                                int(bool(fast_math)), _DTYPES[xc.dtype], _stream(x))
        _lib.check(rc, "fla_entmax_fwd")
    return y


def entmax_rows_backward(y, dy, alpha):
    lib = _lib.load()
    dyc = dy.contiguous().to(y.dtype)
    cols = y.shape[-1] if y.dim() > 0 else 1
    rows = y.numel() // max(cols, 1)
    with torch.cuda.device(y.device):
        dx = torch.empty_like(y)
        rc = lib.fla_entmax_bwd(y.data_ptr(), dyc.data_ptr(), dx.data_ptr(), rows, cols, float(alpha),
                                _DTYPES[y.dtype], _stream(y))
        _lib.check(rc, "fla_entmax_bwd")
    return dx


class EntmaxFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, alpha, n_iter, fast_math):
        y = entmax_rows_forward(x, alpha, n_iter, fast_math)
        ctx.save_for_backward(y)
        ctx.alpha, ctx.orig_dtype = float(alpha), x.dtype
        return y.to(x.dtype) if x.dtype == torch.float64 else y

    @staticmethod
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        return entmax_rows_backward(y, dy, ctx.alpha).to(ctx.orig_dtype), None, None, None


def triton_entmax(x, alpha=1.5, n_iter=10, fast_math=True):
    """alpha-entmax over the last dimension (Halley/Newton on the threshold, bisection-safeguarded)."""
    if torch.compiler.is_compiling():   # one opaque node in the traced graph (custom_ops.py)
        return torch.ops.flash_lazy.entmax_rows_fwd(x, float(alpha), int(n_iter), bool(fast_math)).to(x.dtype)
    return EntmaxFunc.apply(x, alpha, n_iter, fast_math)


# ---------------------------------------------------------------------------------------------
# rotary position embedding of q and k (the step before the attention operators in the layers)
# ---------------------------------------------------------------------------------------------
def rope_qk_apply(q, k, base=10000.0, offset=0, inverse=False):
    """Rotate-half rotary embedding of q [B,H,L,D] and k [B,Hk,L,D] (views with unit inner stride) in one launch;
    returns new tensors with the inputs' strides.  ``inverse`` rotates back (the gradient of the rotation)."""
    lib = _lib.load()
    for n, t in (("q", q), ("k", k)):
        _check_cuda(t, n)
        if t.dim() != 4:
            raise ValueError(f"{n} must be [B, H, L, D]")
    if q.dtype != k.dtype or q.shape[0] != k.shape[0] or q.shape[2:] != k.shape[2:]:
        raise ValueError("q and k must share dtype, batch, length and head dimension")

    q, k = _unit_inner(q), _unit_inner(k)
    B, H, L, D = q.shape
    with torch.cuda.device(q.device):
        qo, ko = torch.empty_like(q), torch.empty_like(k)
        if qo.stride() != q.stride() or ko.stride() != k.stride():   # (overlapping or exotic views)
            q, k = q.contiguous(), k.contiguous()
            qo, ko = torch.empty_like(q), torch.empty_like(k)
        rc = lib.fla_rope_qk(_t4(q), _t4(qo), H, _t4(k), _t4(ko), k.shape[1], B, L, D, _DTYPES[q.dtype], float(base),
                             int(offset), int(bool(inverse)), _stream(q))
        _lib.check(rc, "fla_rope_qk")
    return qo, ko


def rope_qk(q, k, base=10000.0, offset=0):
    """Differentiable rotary embedding of q and k ([B,H,L,D] views; for ``b l h d`` tensors pass
    ``x.transpose(1, 2)``), one kernel launch for both tensors."""
    return torch.ops.flash_lazy.rope_qk(q, k, float(base), int(offset), False)


def last_call_info() -> dict:
    """Kernel family the calling thread's last attention call ran on."""
    lib = _lib.load()
    return {"path": _lib.PATH_NAMES.get(lib.fla_last_path(), "?")}
