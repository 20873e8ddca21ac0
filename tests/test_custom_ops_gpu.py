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


@pytest.mark.parametrize("mode", ["bf16", "fp4_rownorm"])
def test_general_attention_op_varlen_bias_zshd(mode):
    """`nvfp4_attn_ex`: the registered ops with key bias / packed varlen rows / zshd output and the
    backward modes give the eager entry's bits, eagerly and under `torch.compile`."""
    import sageattention_b200.nvfp4 as nv
    import sageattention_b200.nvfp4.custom_ops as C
    h, hk, d = 4, 2, 128
    lens = [100, 256, 37, 300]
    s = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    q, _ = seeded_bf16((1, h, s, d), 81)
    k, _ = seeded_bf16((1, hk, s, d), 82)
    v, _ = seeded_bf16((1, hk, s, d), 83)
    do, _ = seeded_bf16((1, s, h, d), 84)
    bias = torch.zeros(1, s, device="cuda")
    bias[0, 5::17] = -2.0

    def eager(q_, k_, v_, use_cu):
        return nv.nvfp4_flash_attn_func(q_, k_, v_, d ** -0.5, causal=True, num_key_value_groups=h // hk,
                                        cu_seqlens=cu if use_cu else None, key_pad_bias=None if use_cu else bias,
                                        out_layout="zshd", backward_grad_dots=mode, stochastic_rounding=False)

    def op(q_, k_, v_, use_cu):
        return C.nvfp4_attn_ex(q_, k_, v_, d ** -0.5, True, h // hk, key_pad_bias=None if use_cu else bias,
                               cu_seqlens=cu if use_cu else None, out_layout="zshd", backward_grad_dots=mode)

    for use_cu in (True, False):
        res = []
        for fn in (eager, op, torch.compile(op, backend="aot_eager", fullgraph=True)):
            qq, kk, vv = (t.clone().requires_grad_(True) for t in (q, k, v))
            o = fn(qq, kk, vv, use_cu)
            assert o.shape == (1, s, h, d)
            o.backward(do)
            res.append((o.detach(), qq.grad, kk.grad, vv.grad))
        for other in res[1:]:
            for a, b in zip(res[0], other):
                assert torch.equal(a, b)


def test_cache_ops_match_cache_methods():
    """`nvfp4_kv_append` / `nvfp4_hybrid_decode` on a cache's buffers do what the methods do (bytes
    and bits), eagerly and under `torch.compile`."""
    import sageattention_b200.nvfp4 as nv
    import sageattention_b200.nvfp4.custom_ops as C  # noqa: F401
    z, hk, g, d, s0, window = 2, 2, 4, 128, 700, 64
    k, _ = seeded_bf16((z, hk, s0 + 40, d), 91)
    v, _ = seeded_bf16((z, hk, s0 + 40, d), 92)
    q, _ = seeded_bf16((z, hk * g, 1, d), 93)
    a = nv.NVFP4KVCache(z, hk, d, 1024, "cuda", recent_window=window)
    b = nv.NVFP4KVCache(z, hk, d, 1024, "cuda", recent_window=window)
    a.prefill(k[:, :, :s0], v[:, :, :s0])
    b.prefill(k[:, :, :s0], v[:, :, :s0])
    ops = torch.ops.sageattention_b200

    def step(k_new, v_new, knv, ksc, vnv, vsc, part, rk, rv, qq, pos: int):
        ops.nvfp4_kv_append(k_new, v_new, knv, ksc, vnv, vsc, part, rk, rv, pos)
        return ops.nvfp4_hybrid_decode(qq, knv, ksc, vnv, vsc, rk, rv, pos + 1, window, d ** -0.5, g)

    cstep = torch.compile(step, backend="aot_eager", fullgraph=True)
    for i in range(40):
        t = s0 + i
        a.append(k[:, :, t:t + 1], v[:, :, t:t + 1])
        want = a.hybrid_decode(q, d ** -0.5, g)
        fn = cstep if i % 2 else step
        got = fn(k[:, :, t:t + 1], v[:, :, t:t + 1], b.knv, b.ksc, b.vnv, b.vsc, b.v_partial_bf16, b.rk, b.rv, q, t)
        b.length = t + 1
        assert torch.equal(got, want)
    for x, y in ((a.knv, b.knv), (a.ksc, b.ksc), (a.vnv, b.vnv), (a.vsc, b.vsc), (a.rk, b.rk), (a.rv, b.rv),
                 (a.v_partial_bf16, b.v_partial_bf16)):
        assert torch.equal(x.view(torch.uint8), y.view(torch.uint8))
