"""The operators as ``torch.library`` custom ops, so that ``torch.compile`` traces them as single opaque nodes
(schema, fake implementation for shape propagation, autograd formula) instead of meeting ctypes calls inside an
``autograd.Function``.  The reference's operators are Triton kernels inside ``autograd.Function``s
(lazy_attention_triton.py:509-541), which ``torch.compile`` can trace; this module gives the same property here.

    torch.ops.flash_lazy.entmax_attn_fwd / entmax_attn_bwd      adasplash, adasplash_no_block_mask
    torch.ops.flash_lazy.lazy_attn_fwd   / lazy_attn_bwd        lazy_attention_triton
    torch.ops.flash_lazy.entmax_rows_fwd / entmax_rows_bwd      triton_entmax
    torch.ops.flash_lazy.rope_qk                                rotary embedding of q and k (its own backward)

The public functions of ``ops`` route here while ``torch.compiler.is_compiling()``; in eager mode they keep using
their ``autograd.Function``s (which allocate the SIMT family's aux buffers only when a backward will follow).
Absent optional outputs are zero-element tensors: an op returns a fixed tuple of tensors.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor

from . import _lib, ops

_16BIT = (torch.float16, torch.bfloat16)


def _none_if_empty(t: Tensor):
    return None if t.numel() == 0 else t


def _tensor_core_shape(q: Tensor, k: Tensor) -> bool:
    """Whether contiguous tensors of this dtype and shape run on the tensor-core family (the rule of
    csrc/tc_attn.cu, eligible(), for views the allocator made: aligned, strides multiples of D).  Decides from
    metadata alone whether the forward must emit the SIMT family's aux buffers, so that the fake implementation
    and the real one agree."""
    B, H, L, D = q.shape
    tiles = (L + 127) // 128
    n_rep = H // max(k.shape[1], 1)
    return (q.dtype in _16BIT and D in (64, 128) and tiles <= 512 and n_rep <= 64 and n_rep * tiles <= 2048
            and ops._path() != _lib.PATH_SIMT)


def _empty(q: Tensor, dtype=torch.float32) -> Tensor:
    return torch.empty((0,), dtype=dtype, device=q.device)


def _kv_heads(q: Tensor, k: Tensor) -> int:
    if k.shape[1] == q.shape[1]:
        return 0
    if not _tensor_core_shape(q, k):
        raise RuntimeError("grouped-query heads need the tensor-core family (fp16/bf16, D in {64, 128}); "
                           "repeat k, v over the group for other inputs")
    return k.shape[1]


# ---------------------------------------------------------------------------------------------
# alpha-entmax attention
# ---------------------------------------------------------------------------------------------
@torch.library.custom_op("flash_lazy::entmax_attn_fwd", mutates_args=(), device_types="cuda")
def entmax_attn_fwd(q: Tensor, k: Tensor, v: Tensor, alpha: float, niter: int, causal: bool,
                    varlen: Optional[Tensor], use_block_mask: bool) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    need_aux = not _tensor_core_shape(q, k)
    out, tau, aux_o, aux_s, mask = ops.entmax_attention_forward(q, k, v, alpha, niter, causal, varlen, use_block_mask,
                                                                need_aux, kv_heads=_kv_heads(q, k))
    return (out, tau, aux_o if need_aux else _empty(q), aux_s if need_aux else _empty(q),
            mask if use_block_mask else _empty(q, torch.int32))


@entmax_attn_fwd.register_fake
def _(q, k, v, alpha, niter, causal, varlen, use_block_mask):
    B, H, L, D = q.shape
    need_aux = not _tensor_core_shape(q, k)
    f32 = dict(dtype=torch.float32, device=q.device)
    words = ((L + 63) // 64 + 31) // 32
    return (q.new_empty((B, H, L, D)), q.new_empty((B, H, L), dtype=torch.float32),
            torch.empty((B, H, L, D) if need_aux else (0,), **f32), torch.empty((B, H, L) if need_aux else (0,), **f32),
            torch.empty((B, H, (L + 127) // 128, words) if use_block_mask else (0,), dtype=torch.int32, device=q.device))


@torch.library.custom_op("flash_lazy::entmax_attn_bwd", mutates_args=(), device_types="cuda")
def entmax_attn_bwd(q: Tensor, k: Tensor, v: Tensor, dout: Tensor, tau: Tensor, aux_o: Tensor, aux_s: Tensor,
                    mask: Tensor, alpha: float, causal: bool, varlen: Optional[Tensor]) -> Tuple[Tensor, Tensor, Tensor]:
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    return ops.entmax_attention_backward(q, k, v, dout, tau, _none_if_empty(aux_o), _none_if_empty(aux_s),
                                         _none_if_empty(mask), ops._varlen32(varlen, q), alpha, causal, _kv_heads(q, k))


@entmax_attn_bwd.register_fake
def _(q, k, v, dout, tau, aux_o, aux_s, mask, alpha, causal, varlen):
    return q.new_empty(q.shape), k.new_empty(k.shape), v.new_empty(v.shape)


def _entmax_attn_setup(ctx, inputs, output):
    q, k, v, alpha, niter, causal, varlen, use_block_mask = inputs
    _, tau, aux_o, aux_s, mask = output
    ctx.save_for_backward(q, k, v, tau, aux_o, aux_s, mask, varlen)
    ctx.alpha, ctx.causal = alpha, causal


def _entmax_attn_backward(ctx, dout, *unused):
    q, k, v, tau, aux_o, aux_s, mask, varlen = ctx.saved_tensors
    dq, dk, dv = entmax_attn_bwd(q, k, v, dout, tau, aux_o, aux_s, mask, ctx.alpha, ctx.causal, varlen)
    return dq, dk, dv, None, None, None, None, None


entmax_attn_fwd.register_autograd(_entmax_attn_backward, setup_context=_entmax_attn_setup)


# ---------------------------------------------------------------------------------------------
# Lazy Attention
# ---------------------------------------------------------------------------------------------
@torch.library.custom_op("flash_lazy::lazy_attn_fwd", mutates_args=(), device_types="cuda")
def lazy_attn_fwd(q: Tensor, k: Tensor, v: Tensor, bias: Tensor, tau: Tensor, window: int,
                  varlen: Optional[Tensor]) -> Tuple[Tensor, Tensor, Tensor]:
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    need_aux = not _tensor_core_shape(q, k)
    out, lse, aux_o = ops.lazy_attention_forward(q, k, v, bias, tau, window, varlen, need_aux, _kv_heads(q, k))
    return out, lse, aux_o if need_aux else _empty(q)


@lazy_attn_fwd.register_fake
def _(q, k, v, bias, tau, window, varlen):
    B, H, L, D = q.shape
    need_aux = not _tensor_core_shape(q, k)
    return (q.new_empty((B, H, L, D)), q.new_empty((B, H, L), dtype=torch.float32),
            torch.empty((B, H, L, 2 * D) if need_aux else (0,), dtype=torch.float32, device=q.device))


@torch.library.custom_op("flash_lazy::lazy_attn_bwd", mutates_args=(), device_types="cuda")
def lazy_attn_bwd(q: Tensor, k: Tensor, v: Tensor, out: Tensor, dout: Tensor, bias: Tensor, tau: Tensor, window: int,
                  lse: Tensor, aux_o: Tensor, varlen: Optional[Tensor],
                  want_params: bool) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    dq, dk, dv, dbias, dtau = ops.lazy_attention_backward(q, k, v, out, dout, bias, tau, window, lse,
                                                          _none_if_empty(aux_o), ops._varlen32(varlen, q), want_params,
                                                          _kv_heads(q, k))
    return dq, dk, dv, dbias if want_params else _empty(q), dtau if want_params else _empty(q)


@lazy_attn_bwd.register_fake
def _(q, k, v, out, dout, bias, tau, window, lse, aux_o, varlen, want_params):
    f32 = dict(dtype=torch.float32, device=q.device)
    return (q.new_empty(q.shape), k.new_empty(k.shape), v.new_empty(v.shape),
            torch.empty(tuple(bias.shape) if want_params else (0,), **f32),
            torch.empty((q.shape[1],) if want_params else (0,), **f32))


def _lazy_attn_setup(ctx, inputs, output):
    q, k, v, bias, tau, window, varlen = inputs
    out, lse, aux_o = output
    ctx.save_for_backward(q, k, v, out, bias, tau, lse, aux_o, varlen)
    ctx.window = window


def _lazy_attn_backward(ctx, dout, *unused):
    q, k, v, out, bias, tau, lse, aux_o, varlen = ctx.saved_tensors
    want_params = bool(ctx.needs_input_grad[3] or ctx.needs_input_grad[4])
    dq, dk, dv, dbias, dtau = lazy_attn_bwd(q, k, v, out, dout, bias, tau, ctx.window, lse, aux_o, varlen, want_params)
    if want_params:   # fp32 like the reference (lazy_attention_triton.py:532-533); autograd casts to the parameter's type
        return dq, dk, dv, dbias, dtau.view(tau.shape), None, None
    return dq, dk, dv, None, None, None, None


lazy_attn_fwd.register_autograd(_lazy_attn_backward, setup_context=_lazy_attn_setup)


# ---------------------------------------------------------------------------------------------
# stand-alone entmax over the last dimension
# ---------------------------------------------------------------------------------------------
@torch.library.custom_op("flash_lazy::entmax_rows_fwd", mutates_args=(), device_types="cuda")
def entmax_rows_fwd(x: Tensor, alpha: float, n_iter: int, fast_math: bool) -> Tensor:
    return ops.entmax_rows_forward(x, alpha, n_iter, fast_math)


@entmax_rows_fwd.register_fake
def _(x, alpha, n_iter, fast_math):
    return torch.empty(x.shape, dtype=torch.float32 if x.dtype == torch.float64 else x.dtype, device=x.device)


@torch.library.custom_op("flash_lazy::entmax_rows_bwd", mutates_args=(), device_types="cuda")
def entmax_rows_bwd(y: Tensor, dy: Tensor, alpha: float) -> Tensor:
    return ops.entmax_rows_backward(y, dy, alpha)


@entmax_rows_bwd.register_fake
def _(y, dy, alpha):
    return torch.empty_like(y)


def _entmax_rows_setup(ctx, inputs, output):
    ctx.save_for_backward(output)
    ctx.alpha, ctx.in_dtype = inputs[1], inputs[0].dtype


def _entmax_rows_backward(ctx, dy):
    (y,) = ctx.saved_tensors
    return entmax_rows_bwd(y, dy, ctx.alpha).to(ctx.in_dtype), None, None, None


entmax_rows_fwd.register_autograd(_entmax_rows_backward, setup_context=_entmax_rows_setup)


# ---------------------------------------------------------------------------------------------
# rotary position embedding of q and k
# ---------------------------------------------------------------------------------------------
@torch.library.custom_op("flash_lazy::rope_qk", mutates_args=(), device_types="cuda")
def rope_qk(q: Tensor, k: Tensor, base: float, offset: int, inverse: bool) -> Tuple[Tensor, Tensor]:
    return ops.rope_qk_apply(q, k, base, offset, inverse)


@rope_qk.register_fake
def _(q, k, base, offset, inverse):
    return torch.empty_like(q), torch.empty_like(k)


def _rope_setup(ctx, inputs, output):
    ctx.base, ctx.offset, ctx.inverse = inputs[2], inputs[3], inputs[4]


def _rope_backward(ctx, dq, dk):
    gq, gk = rope_qk(dq, dk, ctx.base, ctx.offset, not ctx.inverse)   # the rotation is orthogonal
    return gq, gk, None, None, None


rope_qk.register_autograd(_rope_backward, setup_context=_rope_setup)
