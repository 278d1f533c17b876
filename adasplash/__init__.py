"""Drop-in import names of the reference package (README.md:24,90,110 of the reference):
``from adasplash import adasplash, adasplash_no_block_mask, triton_entmax, lazy_attention_triton, LazyAttention``
(and ``from adasplash.lazy_attention import LazyAttention``, tests/test_lazy_attention.py:3).
Everything resolves to the sm_100a library in ``flash_lazy_attention_b200``."""
# The sub-modules share names with the functions; import them first so that the package
# attributes end up bound to the functions, as in the reference.
from . import adasplash_block_mask as _m1  # noqa: F401
from . import adasplash_no_block_mask as _m2  # noqa: F401
from . import lazy_attention_triton as _m3  # noqa: F401
from . import triton_entmax as _m4  # noqa: F401
from . import lazy_attention as _m5  # noqa: F401
from flash_lazy_attention_b200 import (LazyAttention, adasplash, adasplash_no_block_mask,  # noqa: F401,E402
                                       lazy_attention_triton, triton_entmax)

__all__ = ["adasplash", "adasplash_no_block_mask", "triton_entmax", "lazy_attention_triton", "LazyAttention"]
