"""The registered ops on a GPU: eager op == public API, and a `torch.compile`d function that calls
them (traced through the fake implementations, autograd included) gives the same numbers."""

import pytest
import torch

from gpu_util import seeded_bf16

pytestmark = pytest.mark.gpu


def test_ops_match_public_api_and_compile():
    import sageattention_b200.nvfp4 as nv
    import sageattention_b200.nvfp4.custom_ops as C
    z, h, hk, s, d = 1, 4, 2, 320, 128
    q, _ = seeded_bf16((z, h, s, d), 71)
    k, _ = seeded_bf16((z, hk, s, d), 72)
    v, _ = seeded_bf16((z, hk, s, d), 73)
    do, _ = seeded_bf16((z, h, s, d), 74)
    ref = nv.nvfp4_flash_attention(q, k, v, d ** -0.5, causal=True, num_key_value_groups=h // hk)
    out, lse = torch.ops.sageattention_b200.nvfp4_attn_fwd(q, k, v, d ** -0.5, True, h // hk)
    assert torch.equal(out, ref) and lse.shape == (z * h, s)

    def f(q_, k_, v_):
        return C.nvfp4_attn(q_ * 1.0, k_, v_, d ** -0.5, True, h // hk) * 2.0

    grads = []
    for fn in (f, torch.compile(f, backend="aot_eager", fullgraph=True)):
        qq, kk, vv = (t.clone().requires_grad_(True) for t in (q, k, v))
        o = fn(qq, kk, vv)
        o.backward(do)
        grads.append((o.detach(), qq.grad, kk.grad, vv.grad))
    for a, b in zip(*grads):
        assert torch.equal(a, b)
    # the backward op equals the autograd function of the public API
    qq, kk, vv = (t.clone().requires_grad_(True) for t in (q, k, v))
    o = nv.nvfp4_flash_attn_func(qq, kk, vv, d ** -0.5, causal=True, num_key_value_groups=h // hk,
                                 backward_grad_dots="bf16")
    (o * 2.0).backward(do)
    assert torch.equal(grads[0][1], qq.grad) and torch.equal(grads[0][2], kk.grad) and torch.equal(grads[0][3], vv.grad)
    nib, sc = torch.ops.sageattention_b200.nvfp4_quant(k.reshape(z * hk, s, d), False, 0)
    nib2, sc2 = nv._quant_nvfp4(k.reshape(z * hk, s, d))
    assert torch.equal(nib, nib2) and torch.equal(sc, sc2.view(torch.uint8))
