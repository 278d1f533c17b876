"""Attention layers over the operators: the shapes of the reference's example layers and of its
``LazyAttention`` module, calling this library's kernels.

* ``LazyAttentionLayer`` mirrors ``examples/lazy_attention_layer.py:34-179`` and
  ``examples/sw_attention_lazy.py:52-193`` of the reference: q/k/v/o projections, optional grouped-query
  heads (``num_kv_heads``), rotary embedding (rotate-half, applied in fp32), fp32 master parameters ``bias``
  [H, max_bias_length] and ``tau`` [H] cast to the activations' dtype for the call
  (``lazy_attention_layer.py:86-89,164-170``), padding given as ``attention_mask`` [B, L] or ``cu_seqlens``
  (``:151-160``).  Differences: the ``b l h d`` projections are handed to the kernels as strided
  ``b h l d`` views (no transpose copy), and shared K/V heads are read in place by the kernels instead of
  being repeated (``sw_attention_lazy.py:30-41,154-157``).  KV caches and qk-RMSNorm are not part of it.
* ``LazyAttention(dim, num_heads, window_size, rope_base)`` has the constructor and the parameter names
  (``tau``, ``attention_biases``) that ``tests/test_lazy_attention.py:5-70`` of the reference pins: biases
  initialised to zero, tau to -1, bias-free projections (tau = -100 gives an all-zero output).  Unlike the
  reference's pure-PyTorch module it has no CPU path: CPU tensors raise, like every operator here.
"""
from __future__ import annotations

import torch
from torch import nn

from .ops import lazy_attention_triton, rope_qk


def rotary(x: torch.Tensor, base: float = 10000.0, offset: int = 0) -> torch.Tensor:
    """Rotate-half rotary embedding of ``x`` [B, L, H, D] (positions offset..offset+L-1), computed in fp32: the
    dense formulation of what ``ops.rope_qk`` does in one kernel (kept as its restatement for the tests)."""
    L, D = x.shape[1], x.shape[-1]
    half = D // 2
    inv = 1.0 / (base ** (torch.arange(half, device=x.device, dtype=torch.float32) / half))
    ang = (torch.arange(L, device=x.device, dtype=torch.float32) + offset)[:, None] * inv[None, :]
    cos = torch.cat([ang.cos(), ang.cos()], -1)[None, :, None, :]
    sin = torch.cat([ang.sin(), ang.sin()], -1)[None, :, None, :]
    xf = x.float()
    rot = torch.cat([-xf[..., half:], xf[..., :half]], -1)
    return (xf * cos + rot * sin).to(x.dtype)


def lengths_from(attention_mask=None, cu_seqlens=None):
    """``varlen`` [B] int32 from a 0/1 padding mask [B, L] (valid tokens first) or from cumulative sequence
    lengths, as the reference's layers derive it (``examples/lazy_attention_layer.py:151-160``)."""
    if attention_mask is not None:
        if attention_mask.dim() != 2:
            raise ValueError("attention_mask must be a 0-1 matrix [batch, seq_len] (0 = padding)")
        return attention_mask.sum(dim=1).to(torch.int32)
    if cu_seqlens is not None:
        return (cu_seqlens[1:] - cu_seqlens[:-1]).to(torch.int32)
    return None


class LazyAttentionLayer(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int | None = None, max_bias_length: int = 512,
                 rope_theta: float = 10000.0, qkv_bias: bool = False):
        super().__init__()
        if hidden_size % num_heads:
            raise ValueError("hidden_size must be a multiple of num_heads")
        self.num_heads = num_heads
        self.num_kv_heads = num_heads if num_kv_heads is None else num_kv_heads
        if num_heads % self.num_kv_heads:
            raise ValueError("num_kv_heads must divide num_heads")
        self.head_dim = hidden_size // num_heads
        self.max_bias_length = max_bias_length
        self.rope_theta = rope_theta
        self.q_proj = nn.Linear(hidden_size, num_heads * self.head_dim, bias=qkv_bias)
        self.k_proj = nn.Linear(hidden_size, self.num_kv_heads * self.head_dim, bias=qkv_bias)
        self.v_proj = nn.Linear(hidden_size, self.num_kv_heads * self.head_dim, bias=qkv_bias)
        self.o_proj = nn.Linear(num_heads * self.head_dim, hidden_size, bias=False)
        # fp32 masters, whatever dtype the rest of the model is cast to
        self.bias = nn.Parameter(torch.zeros(num_heads, max_bias_length, dtype=torch.float32))
        self.tau = nn.Parameter(torch.full((num_heads,), -1.0, dtype=torch.float32))

    def forward(self, hidden_states, attention_mask=None, cu_seqlens=None):
        B, L, _ = hidden_states.shape
        q = self.q_proj(hidden_states).view(B, L, self.num_heads, self.head_dim)
        k = self.k_proj(hidden_states).view(B, L, self.num_kv_heads, self.head_dim)
        v = self.v_proj(hidden_states).view(B, L, self.num_kv_heads, self.head_dim)
        # b l h d -> b h l d as views: the kernels take the strides
        q, k, v = (t.permute(0, 2, 1, 3) for t in (q, k, v))
        q, k = rope_qk(q, k, self.rope_theta)     # one launch for both tensors
        o = lazy_attention_triton(q, k, v, self.bias.to(q.dtype), self.tau.to(q.dtype),
                                  window_size=self.max_bias_length, varlen=lengths_from(attention_mask, cu_seqlens))
        return self.o_proj(o.permute(0, 2, 1, 3).reshape(B, L, self.num_heads * self.head_dim))


class LazyAttention(nn.Module):
    def __init__(self, dim: int, num_heads: int, window_size: int = 512, rope_base: float = 10000.0):
        super().__init__()
        if dim % num_heads:
            raise ValueError("dim must be a multiple of num_heads")
        self.dim, self.num_heads, self.head_dim = dim, num_heads, dim // num_heads
        self.window_size, self.rope_base = window_size, rope_base
        self.q_proj = nn.Linear(dim, dim, bias=False)
        self.k_proj = nn.Linear(dim, dim, bias=False)
        self.v_proj = nn.Linear(dim, dim, bias=False)
        self.out_proj = nn.Linear(dim, dim, bias=False)
        self.tau = nn.Parameter(torch.full((num_heads,), -1.0))
        self.attention_biases = nn.Parameter(torch.zeros(num_heads, window_size))

    def forward(self, x, attention_mask=None):
        B, L, _ = x.shape
        q, k, v = (proj(x).view(B, L, self.num_heads, self.head_dim) for proj in (self.q_proj, self.k_proj, self.v_proj))
        q, k, v = (t.permute(0, 2, 1, 3) for t in (q, k, v))
        q, k = rope_qk(q, k, self.rope_base)
        o = lazy_attention_triton(q, k, v, self.attention_biases, self.tau, window_size=self.window_size,
                                  varlen=lengths_from(attention_mask))
        return self.out_proj(o.permute(0, 2, 1, 3).reshape(B, L, self.dim))
