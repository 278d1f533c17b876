"""CPU checks of the drop-in boundary: the shared library loads, exports every symbol the
header declares, and rejects bad arguments before touching a GPU."""
import ctypes as C
import os
import re

import pytest

from flash_lazy_attention_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "fla.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fla_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = _declared()
    assert len(names) >= 14
    for n in names:
        assert hasattr(lib, n), n
    assert sorted(_lib.SIGNATURES) == names, "ctypes signature table and header disagree"


def test_version_and_mask_words():
    lib = _lib.load()
    assert lib.fla_version() >= 1100
    assert lib.fla_block_mask_words(64) == 1
    assert lib.fla_block_mask_words(2048) == 1
    assert lib.fla_block_mask_words(2049) == 2
    assert lib.fla_block_mask_words(32768) == 16


def test_invalid_arguments_are_rejected_without_a_gpu():
    lib = _lib.load()
    assert lib.fla_entmax_fwd(None, None, 4, 4, 1.5, 10, 1, 0, None) == 1
    assert b"NULL" in lib.fla_last_error()
    buf = C.create_string_buffer(64)
    p = C.cast(buf, C.c_void_p)
    assert lib.fla_entmax_fwd(p, p, 4, 4, 1.0, 10, 1, 0, None) == 1      # alpha out of (1, 2]
    assert lib.fla_entmax_fwd(p, p, 4, 0, 1.5, 10, 1, 0, None) == 1      # empty rows
    assert lib.fla_entmax_fwd(p, p, 0, 8, 1.5, 10, 1, 0, None) == 0      # no rows: nothing to do
    assert lib.fla_entmax_bwd(p, p, p, 4, 4, 1.5, 7, None) == 1          # dtype
    g = _lib.AttnGeom()
    g.B, g.H, g.L, g.D, g.dtype, g.causal, g.varlen, g.path, g.status = 1, 1, 16, 256, 0, 0, None, 0, None
    t = _lib.Tensor4()
    t.ptr = p.value
    t.stride[0], t.stride[1], t.stride[2], t.stride[3] = 16 * 256, 16 * 256, 256, 1
    assert lib.fla_entmax_attn_fwd(g, t, t, t, t, 1.5, 10, p, None, None, None, None) == 2  # D > 128
    g.D = 16
    assert lib.fla_entmax_attn_fwd(g, t, t, t, t, 1.5, 10, None, None, None, None, None) == 1  # tau NULL
    t2 = _lib.Tensor4()
    t2.ptr = p.value
    t2.stride[0], t2.stride[1], t2.stride[2], t2.stride[3] = 256, 256, 1, 16
    assert lib.fla_entmax_attn_fwd(g, t2, t, t, t, 1.5, 10, p, None, None, None, None) == 1  # inner stride
    assert b"stride" in lib.fla_last_error()
    assert lib.fla_entmax_attn_bwd_workspace(g) == 256
    assert lib.fla_check_status(None, None) == 1
    assert lib.fla_entmax_attn_bwd(g, t, t, t, t, 1.5, p, p, p, None, t, t, t, p, 8, None) == 1  # workspace
    assert lib.fla_lazy_attn_fwd(g, t, t, t, t, p, 4, p, 8, p, None, None) == 1  # window > bias columns


def test_ops_refuse_cpu_tensors():
    import torch
    from flash_lazy_attention_b200 import adasplash, lazy_attention_triton, triton_entmax
    x = torch.randn(1, 1, 8, 16)
    with pytest.raises(RuntimeError, match="CUDA"):
        adasplash(x, x, x)
    with pytest.raises(RuntimeError, match="CUDA"):
        triton_entmax(torch.randn(4, 4))
    with pytest.raises(RuntimeError, match="CUDA"):
        lazy_attention_triton(x, x, x, torch.zeros(1, 4), torch.zeros(1))


def test_drop_in_import_names():
    import adasplash as pkg
    from adasplash.lazy_attention_triton import lazy_attention_triton
    from adasplash.triton_entmax import triton_entmax
    assert callable(pkg.adasplash) and callable(pkg.adasplash_no_block_mask)
    assert pkg.lazy_attention_triton is lazy_attention_triton and pkg.triton_entmax is triton_entmax
