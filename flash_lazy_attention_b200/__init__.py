"""B200-native (sm_100a) alpha-entmax / Lazy Attention operators behind the reference's API."""
from .ops import (adasplash, adasplash_no_block_mask, check_status, entmax_attention_forward,  # noqa: F401
                  last_call_info, lazy_attention_triton, read_status, rope_qk, set_flags, set_path, triton_entmax,
                  unpack_block_mask)

from . import custom_ops  # noqa: F401,E402  (registers torch.ops.flash_lazy.*)
from .layers import LazyAttention, LazyAttentionLayer  # noqa: F401,E402

__all__ = ["LazyAttention", "LazyAttentionLayer", "adasplash", "adasplash_no_block_mask", "triton_entmax", "lazy_attention_triton",
           "entmax_attention_forward", "unpack_block_mask", "set_path", "last_call_info",
           "read_status", "check_status", "set_flags", "rope_qk"]
