"""The allocation-free backward entry point (fla_entmax_attn_bwd_static) against the regular one.

Some users of the library cannot hand it a workspace: bindings without an allocator, code
running where the framework allocator must not be re-entered, processes with a fixed memory pool.
For them the library keeps the backward's per-row scratch in a built-in device array.  This test
calls both entry points through the C ABI on the same inputs, twice in a row (the array keeps
the previous call's contents), and expects the same gradients; it also checks the size limit.
Collected last on purpose, so that a run stopping at the first failure has run everything else.
"""
import pytest
import torch

from flash_lazy_attention_b200 import _lib
from flash_lazy_attention_b200.ops import _geom, _stream, _t4

from gpu_util import close, randn

pytestmark = pytest.mark.gpu


def _forward(lib, q, k, v, alpha, causal, use_tc):
    B, H, L, D = q.shape
    g = _geom(q, causal, None)
    out = torch.empty_like(q)
    tau = torch.empty((B, H, L), dtype=torch.float32, device=q.device)
    aux_o = aux_s = None
    if not use_tc:
        aux_o = torch.empty((B, H, L, D), dtype=torch.float32, device=q.device)
        aux_s = torch.empty((B, H, L), dtype=torch.float32, device=q.device)
    rc = lib.fla_entmax_attn_fwd(g, _t4(q), _t4(k), _t4(v), _t4(out), alpha, 10, tau.data_ptr(),
                                 aux_o.data_ptr() if aux_o is not None else None,
                                 aux_s.data_ptr() if aux_s is not None else None, None, _stream(q))
    _lib.check(rc, "fla_entmax_attn_fwd")
    return g, tau, aux_o, aux_s


@pytest.mark.parametrize("dtype,D", [(torch.bfloat16, 128), (torch.float32, 64)])
def test_static_scratch_backward_matches_workspace_backward(dtype, D):
    lib = _lib.load()
    alpha, causal = 1.5, True
    for call, (B, H, L) in enumerate([(2, 2, 384), (1, 3, 200)]):      # two calls in a row, different sizes
        q, k, v, do = (randn((B, H, L, D), dtype, 10 * call + s) for s in (1, 2, 3, 4))
        g = _geom(q, causal, None)
        use_tc = bool(lib.fla_attn_uses_tensor_cores(g, _t4(q), _t4(k), _t4(v)))
        g, tau, aux_o, aux_s = _forward(lib, q, k, v, alpha, causal, use_tc)
        ao = aux_o.data_ptr() if aux_o is not None else None
        as_ = aux_s.data_ptr() if aux_s is not None else None

        ref = [torch.empty_like(q) for _ in range(3)]
        nbytes = lib.fla_entmax_attn_bwd_workspace(g)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
        rc = lib.fla_entmax_attn_bwd(g, _t4(q), _t4(k), _t4(v), _t4(do), alpha, tau.data_ptr(), ao, as_, None,
                                     _t4(ref[0]), _t4(ref[1]), _t4(ref[2]), ws.data_ptr(), nbytes, _stream(q))
        _lib.check(rc, "fla_entmax_attn_bwd")

        got = [torch.full_like(q, float("nan")) for _ in range(3)]
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = lib.fla_entmax_attn_bwd_static(g, _t4(q), _t4(k), _t4(v), _t4(do), alpha, tau.data_ptr(), ao, as_,
                                            None, _t4(got[0]), _t4(got[1]), _t4(got[2]), _stream(q))
        _lib.check(rc, "fla_entmax_attn_bwd_static")
        torch.cuda.synchronize()
        if call > 0:   # the array's address was looked up by the first call: this one may not take any device memory
            assert torch.cuda.mem_get_info()[0] == free_before
        for name, a, b in zip(("dq", "dk", "dv"), got, ref):
            assert torch.isfinite(a).all(), name
            assert close(a, b, dtype, atol32=1e-4), (name, call, float((a.float() - b.float()).abs().max()))


def test_static_scratch_accepts_exactly_the_limit():
    """B*H*L equal to the limit runs (one more row is refused, see below)."""
    lib = _lib.load()
    B, H, L, D, dtype = 128, 64, 128, 64, torch.bfloat16
    assert B * H * L == lib.fla_entmax_attn_bwd_static_max_rows()
    q, k, v, do = (randn((B, H, L, D), dtype, s) for s in (1, 2, 3, 4))
    g, tau, _, _ = _forward(lib, q, k, v, 1.5, True, True)
    ref = [torch.empty_like(q) for _ in range(3)]
    nbytes = lib.fla_entmax_attn_bwd_workspace(g)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    _lib.check(lib.fla_entmax_attn_bwd(g, _t4(q), _t4(k), _t4(v), _t4(do), 1.5, tau.data_ptr(), None, None, None,
                                       _t4(ref[0]), _t4(ref[1]), _t4(ref[2]), ws.data_ptr(), nbytes, _stream(q)),
               "fla_entmax_attn_bwd")
    got = [torch.empty_like(q) for _ in range(3)]
    _lib.check(lib.fla_entmax_attn_bwd_static(g, _t4(q), _t4(k), _t4(v), _t4(do), 1.5, tau.data_ptr(), None, None,
                                              None, _t4(got[0]), _t4(got[1]), _t4(got[2]), _stream(q)),
               "fla_entmax_attn_bwd_static")
    torch.cuda.synchronize()
    for a, b in zip(got, ref):
        assert torch.equal(a, b)


def test_static_scratch_rejects_oversized_problems():
    lib = _lib.load()
    limit = lib.fla_entmax_attn_bwd_static_max_rows()
    assert limit == 1 << 20
    q = torch.empty((1, 1, 8, 64), dtype=torch.bfloat16, device="cuda")
    g = _geom(q, True, None)
    g.B, g.H, g.L = 8, 32, 8192                     # 2,097,152 rows: beyond the built-in array
    t = _t4(q)
    tau = torch.empty(8, device="cuda")
    rc = lib.fla_entmax_attn_bwd_static(g, t, t, t, t, 1.5, tau.data_ptr(), None, None, None, t, t, t, _stream(q))
    assert rc == 2 and b"built-in scratch" in lib.fla_last_error()
