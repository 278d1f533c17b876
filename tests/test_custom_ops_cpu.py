"""torch.library registration of the operators, checked without a GPU: schemas, shape propagation through the fake
implementations, and that torch.compile traces the public functions into a single custom-op node each."""
import torch

import flash_lazy_attention_b200 as fla


def _meta(*shape, dtype=torch.bfloat16):
    return torch.empty(*shape, dtype=dtype, device="meta")


def test_ops_are_registered_with_their_schemas():
    ns = torch.ops.flash_lazy
    for name in ("entmax_attn_fwd", "entmax_attn_bwd", "lazy_attn_fwd", "lazy_attn_bwd", "entmax_rows_fwd",
                 "entmax_rows_bwd"):
        schema = str(getattr(ns, name).default._schema)
        assert schema.startswith(f"flash_lazy::{name}("), schema
    assert "Tensor? varlen" in str(ns.entmax_attn_fwd.default._schema)
    assert "Tensor? varlen" in str(ns.lazy_attn_fwd.default._schema)


def test_fake_shapes_tensor_core_and_simt_inputs():
    q, k = _meta(2, 4, 300, 128), _meta(2, 2, 300, 128)          # grouped-query, tensor-core shaped: no aux buffers
    out, tau, aux_o, aux_s, mask = torch.ops.flash_lazy.entmax_attn_fwd(q, k, k, 1.5, 10, True, None, True)
    assert out.shape == q.shape and out.dtype == q.dtype and tau.shape == (2, 4, 300) and tau.dtype == torch.float32
    assert aux_o.numel() == 0 and aux_s.numel() == 0 and mask.shape == (2, 4, 3, 1) and mask.dtype == torch.int32
    dq, dk, dv = torch.ops.flash_lazy.entmax_attn_bwd(q, k, k, out, tau, aux_o, aux_s, mask, 1.5, True, None)
    assert dq.shape == q.shape and dk.shape == k.shape and dv.shape == k.shape
    x = _meta(2, 4, 300, 32, dtype=torch.float32)                # fp32: SIMT family, aux buffers emitted
    out, tau, aux_o, aux_s, mask = torch.ops.flash_lazy.entmax_attn_fwd(x, x, x, 2.0, 10, False, None, False)
    assert aux_o.shape == (2, 4, 300, 32) and aux_s.shape == (2, 4, 300) and mask.numel() == 0
    bias, tau_h = _meta(4, 64, dtype=torch.float32), _meta(4, dtype=torch.float32)
    out, lse, aux = torch.ops.flash_lazy.lazy_attn_fwd(q, k, k, bias, tau_h, 64, None)
    assert out.shape == q.shape and lse.shape == (2, 4, 300) and aux.numel() == 0
    grads = torch.ops.flash_lazy.lazy_attn_bwd(q, k, k, out, out, bias, tau_h, 64, lse, aux, None, True)
    assert [tuple(g.shape) for g in grads] == [(2, 4, 300, 128), (2, 2, 300, 128), (2, 2, 300, 128), (4, 64), (4,)]
    assert grads[3].dtype == torch.float32 and grads[4].dtype == torch.float32
    grads = torch.ops.flash_lazy.lazy_attn_bwd(q, k, k, out, out, bias, tau_h, 64, lse, aux, None, False)
    assert grads[3].numel() == 0 and grads[4].numel() == 0
    y = torch.ops.flash_lazy.entmax_rows_fwd(_meta(5, 7, 100, dtype=torch.float16), 1.5, 10, True)
    assert y.shape == (5, 7, 100) and y.dtype == torch.float16


def _traced_targets(fn, *args):
    seen = []

    def backend(gm, example_inputs):
        seen.extend(str(n.target) for n in gm.graph.nodes if n.op == "call_function")
        return gm.forward

    torch._dynamo.reset()
    out = torch.compile(fn, backend=backend, fullgraph=True)(*args)   # meta tensors: runs the fake implementations
    return out, seen


def test_compile_traces_each_public_function_into_one_node():
    q = _meta(1, 2, 256, 64)
    out, seen = _traced_targets(lambda a, b, c: fla.adasplash(a, b, c, alpha=1.5, is_causal=True), q, q, q)
    assert out.shape == q.shape and any("flash_lazy.entmax_attn_fwd" in t for t in seen), seen
    out, seen = _traced_targets(lambda a, b, c: fla.adasplash_no_block_mask(a, b, c, alpha=2.0), q, q, q)
    assert any("flash_lazy.entmax_attn_fwd" in t for t in seen), seen
    bias, tau = _meta(2, 32, dtype=torch.float32), _meta(2, dtype=torch.float32)
    out, seen = _traced_targets(lambda a, b, c, d, e: fla.lazy_attention_triton(a, b, c, d, e), q, q, q, bias, tau)
    assert out.shape == q.shape and any("flash_lazy.lazy_attn_fwd" in t for t in seen), seen
    x = _meta(8, 100, dtype=torch.float32)
    out, seen = _traced_targets(lambda a: fla.triton_entmax(a, alpha=1.5), x)
    assert out.shape == x.shape and any("flash_lazy.entmax_rows_fwd" in t for t in seen), seen
