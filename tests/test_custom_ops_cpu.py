"""`torch.library` registration: schemas exist and the fake (meta) implementations infer the right
shapes and dtypes without touching a GPU (what `torch.compile` needs to trace through the ops)."""

import torch
from torch._subclasses.fake_tensor import FakeTensorMode

import sageattention_b200.nvfp4.custom_ops as C  # noqa: F401  (registers the ops)


def test_ops_are_registered():
    ns = torch.ops.sageattention_b200
    for name in ("nvfp4_attn_fwd", "nvfp4_attn_bwd", "nvfp4_quant", "nvfp4_decode", "nvfp4_attn_ex_fwd",
                 "nvfp4_attn_ex_bwd", "nvfp4_kv_append", "nvfp4_hybrid_decode"):
        assert hasattr(ns, name)


def test_fake_impls_infer_shapes():
    with FakeTensorMode():
        q = torch.empty(2, 8, 300, 128, dtype=torch.bfloat16)
        k = torch.empty(2, 2, 420, 128, dtype=torch.bfloat16)
        v = torch.empty(2, 2, 420, 128, dtype=torch.bfloat16)
        out, lse = torch.ops.sageattention_b200.nvfp4_attn_fwd(q, k, v, 0.088, True, 4)
        assert out.shape == q.shape and out.dtype == torch.bfloat16
        assert lse.shape == (16, 300) and lse.dtype == torch.float32
        dq, dk, dv = torch.ops.sageattention_b200.nvfp4_attn_bwd(q, k, v, out, lse, out, 0.088, True, 4)
        assert dq.shape == q.shape and dk.shape == k.shape and dv.shape == v.shape
        nib, sc = torch.ops.sageattention_b200.nvfp4_quant(k.reshape(4, 420, 128), True, 512)
        assert nib.shape == (4, 128, 256) and sc.shape == (4, 128, 32) and nib.dtype == torch.uint8
        nib, sc = torch.ops.sageattention_b200.nvfp4_quant(k.reshape(4, 420, 128), False, 0)
        assert nib.shape == (4, 420, 64) and sc.shape == (4, 420, 8)
        qd = torch.empty(2, 8, 1, 128, dtype=torch.bfloat16)
        o = torch.ops.sageattention_b200.nvfp4_decode(qd, nib, sc, nib, sc, 420, 512, 0.088, 4)
        assert o.shape == qd.shape


def test_autograd_formula_is_attached_under_fake_mode():
    with FakeTensorMode():
        q = torch.empty(1, 4, 128, 128, dtype=torch.bfloat16, requires_grad=True)
        k = torch.empty(1, 2, 128, 128, dtype=torch.bfloat16, requires_grad=True)
        v = torch.empty(1, 2, 128, 128, dtype=torch.bfloat16, requires_grad=True)
        out = C.nvfp4_attn(q, k, v, 0.088, True, 2)
        out.sum().backward()
        assert q.grad.shape == q.shape and k.grad.shape == k.shape and v.grad.shape == v.shape


def test_general_attention_and_cache_ops_under_fake_mode():
    """Shapes of the zshd / varlen / bias attention ops, their autograd, and the cache ops."""
    with FakeTensorMode():
        q = torch.empty(1, 4, 256, 128, dtype=torch.bfloat16, requires_grad=True)
        k = torch.empty(1, 2, 256, 128, dtype=torch.bfloat16, requires_grad=True)
        v = torch.empty(1, 2, 256, 128, dtype=torch.bfloat16, requires_grad=True)
        cu = torch.empty(4, dtype=torch.int32)
        bias = torch.empty(1, 256)
        out, lse = torch.ops.sageattention_b200.nvfp4_attn_ex_fwd(q, k, v, 0.088, True, 2, None, cu, True)
        assert out.shape == (1, 256, 4, 128) and lse.shape == (4, 256)
        o2 = C.nvfp4_attn_ex(q, k, v, 0.088, True, 2, key_pad_bias=bias, out_layout="zshd",
                             backward_grad_dots="fp4_rownorm")
        o2.sum().backward()
        assert q.grad.shape == q.shape and k.grad.shape == k.shape and v.grad.shape == v.shape
        knv = torch.empty(4, 1024, 64, dtype=torch.uint8)
        ksc = torch.empty(4, 1024, 8, dtype=torch.float8_e4m3fn)
        vnv = torch.empty(4, 128, 512, dtype=torch.uint8)
        vsc = torch.empty(4, 128, 64, dtype=torch.float8_e4m3fn)
        part = torch.empty(4, 16, 128, dtype=torch.bfloat16)
        rk = torch.empty(2, 2, 80, 128, dtype=torch.bfloat16)
        kn = torch.empty(2, 2, 1, 128, dtype=torch.bfloat16)
        assert torch.ops.sageattention_b200.nvfp4_kv_append(kn, kn, knv, ksc, vnv, vsc, part, rk, rk, 700) is None
        qd = torch.empty(2, 8, 1, 128, dtype=torch.bfloat16)
        o = torch.ops.sageattention_b200.nvfp4_hybrid_decode(qd, knv, ksc, vnv, vsc, rk, rk, 701, 64, 0.088, 4)
        assert o.shape == qd.shape and o.dtype == torch.bfloat16
