"""Argument checks, backward-mode dispatch and edge behaviour of the differentiable entry
``nvfp4_flash_attn_func``, following the reference's own tests of the same interface
(tests/test_nvfp4_attention.py:558-595 bad arguments, :645-696 tiny-amplitude gradients,
:721-808 AUTO gate and deprecated alias, :811-852 scratch knob, :487-555 external packs)."""

import numpy as np
import pytest
import torch

from gpu_util import cos, seeded_bf16
from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu


def _n():
    import sageattention_b200.nvfp4 as n
    return n


def _status():
    from sageattention_b200 import _lib
    return _lib.read_status("cuda")


def _qkv(z, h, hk, s, d, seed):
    return (seeded_bf16((z, h, s, d), seed), seeded_bf16((z, hk, s, d), seed + 1),
            seeded_bf16((z, hk, s, d), seed + 2))


def test_entry_rejects_bad_arguments():
    f = _n().nvfp4_flash_attn_func
    z, h, s, d = 1, 4, 256, 128
    (q, _), (k, _), (v, _) = _qkv(z, h, h, s, d, 1)
    cu = torch.tensor([0, 100, s], dtype=torch.int32)
    sm = d ** -0.5
    with pytest.raises(AssertionError, match="causal"):
        f(q, k, v, sm, causal=False, cu_seqlens=cu)
    with pytest.raises(AssertionError, match=r"cu_seqlens\[-1\]"):
        f(q, k, v, sm, causal=True, cu_seqlens=torch.tensor([0, 100, s + 1], dtype=torch.int32))
    with pytest.raises(AssertionError, match="Z must be 1"):
        (q2, _), (k2, _), (v2, _) = _qkv(2, h, h, s, d, 4)
        f(q2, k2, v2, sm, causal=True, cu_seqlens=cu)
    with pytest.raises(AssertionError, match="Sq == Skv"):
        f(q[:, :, :128], k, v, sm, causal=True, cu_seqlens=torch.tensor([0, 128], dtype=torch.int32))
    with pytest.raises(AssertionError, match="save_backward_packs"):
        f(q, k, v, sm, causal=True, cu_seqlens=cu, save_backward_packs=True)
    with pytest.raises(ValueError, match="backward_grad_dots"):
        f(q, k, v, sm, causal=True, cu_seqlens=cu, backward_grad_dots="bogus")
    with pytest.raises(AssertionError, match="not both"):
        f(q, k, v, sm, causal=True, cu_seqlens=cu, backward_grad_dots="bf16", backward_bf16_grad_dots=True)
    with pytest.raises(AssertionError, match="fp8_rownorm"):
        f(q, k, v, sm, causal=True, backward_grad_dots="fp8_rownorm", save_backward_packs=True)
    with pytest.raises(AssertionError, match="save_backward_packs"):
        packs = _n()._quant_nvfp4(q.reshape(z * h, s, d))
        f(q, k, v, sm, causal=True, q_packs=packs, save_backward_packs=True)
    with pytest.raises(ValueError, match="out_layout"):
        f(q, k, v, sm, out_layout="szhd")
    with pytest.raises(AssertionError):
        f(q, k, v, sm, num_key_value_groups=2)            # H != Hk * groups
    with pytest.raises(AssertionError):
        f(q[..., :64], k[..., :64], v[..., :64], sm)      # head dim outside {128, 256}
    assert _status() == 0


def test_auto_gate_and_deprecated_alias_dispatch(monkeypatch):
    """``backward_grad_dots=None`` resolves on s_kv (or the mean sample length of a packed row);
    the legacy boolean maps True -> "bf16", False -> "fp4_legacy"."""
    from sageattention_b200.nvfp4 import flash
    calls = []
    real_hp, real_fp4 = flash._run_bwd_hp, flash._run_bwd

    nested = [0]                       # the FP4-mode entry runs on the high-precision kernels here

    def spy_hp(*a, **kw):
        if not nested[0]:
            calls.append("bf16")
        return real_hp(*a, **kw)

    def spy_fp4(*a, **kw):
        calls.append(kw.get("mode", "fp4_legacy"))
        nested[0] += 1
        try:
            return real_fp4(*a, **kw)
        finally:
            nested[0] -= 1

    monkeypatch.setattr(flash, "_run_bwd_hp", spy_hp)
    monkeypatch.setattr(flash, "_run_bwd", spy_fp4)
    d = 128

    def run(s, cu=None, **kw):
        (q, _), (k, _), (v, _) = _qkv(1, 2, 2, s, d, s)
        q, k, v = (t.requires_grad_(True) for t in (q, k, v))
        out = flash.nvfp4_flash_attn_func(q, k, v, d ** -0.5, causal=True, num_key_value_groups=1,
                                          cu_seqlens=cu, stochastic_rounding=False, **kw)
        out.backward(torch.ones_like(out))
        for t in (q.grad, k.grad, v.grad):
            assert t is not None and torch.isfinite(t).all()

    run(256)
    assert calls[-1] == "bf16"
    run(4096)
    assert calls[-1] == "fp4_rownorm"
    cu = torch.tensor([512 * i for i in range(10)], dtype=torch.int32)
    run(4608, cu=cu)                                      # S > 4096, mean sample length 512
    assert calls[-1] == "bf16"
    run(128, backward_bf16_grad_dots=True)
    assert calls[-1] == "bf16"
    run(128, backward_bf16_grad_dots=False)
    assert calls[-1] == "fp4_legacy"
    run(128, save_backward_packs=True)                    # only packs saved: "bf16" downgrades
    assert calls[-1] == "fp4_rownorm"
    assert _status() == 0


@pytest.mark.parametrize("mode", ["bf16", "fp4_rownorm", "fp8_rownorm"])
def test_tiny_amplitude_gradient_survives(mode):
    """A 1e-6-amplitude upstream gradient still yields useful gradients (no scale underflow)."""
    z, h, s, d = 1, 4, 128, 128
    (q, qn), (k, kn), (v, vn) = _qkv(z, h, h, s, d, 50)
    do, don = seeded_bf16((z, h, s, d), 53, scale=1e-6)
    rq, rk, rv = O.attention_grads(qn, kn, vn, don, d ** -0.5, True, 1)
    q, k, v = (t.requires_grad_(True) for t in (q, k, v))
    _n().nvfp4_flash_attn_func(q, k, v, d ** -0.5, causal=True, num_key_value_groups=1,
                               stochastic_rounding=False, backward_grad_dots=mode).backward(do)
    assert _status() == 0
    for got, ref in ((q.grad, rq), (k.grad, rk), (v.grad, rv)):
        assert torch.isfinite(got).all()
        assert float(got.abs().max()) > 0
        assert cos(got.float().cpu().numpy(), ref) > 0.9


def test_tiny_amplitude_pack_has_nonzero_scales():
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(2, 64, 128, generator=g) * 1e-6).to(torch.bfloat16).cuda()
    _, sc = _n()._quant_nvfp4(x)
    sc = sc.float()
    assert torch.isfinite(sc).all() and bool((sc > 0).all())
    assert float(sc.min()) == 2.0 ** -9                   # the e4m3 min-subnormal floor


@pytest.mark.parametrize("d", [128, 256])
def test_scratch_knob_and_external_packs_are_bit_neutral(d):
    """``dkdv_scratch_bf16`` does not change any result, and external packs equal to
    ``_quant_nvfp4`` of the operands give bit-identical outputs and gradients."""
    n = _n()
    z, h, hk, s = 1, 4, 2, 200
    (q, _), (k, _), (v, _) = _qkv(z, h, hk, s, d, 60 + d)
    do, _ = seeded_bf16((z, h, s, d), 70 + d)
    cu = torch.tensor([0, 72, s], dtype=torch.int32)

    def run(**kw):
        qx, kx, vx = (t.clone().requires_grad_(True) for t in (q, k, v))
        out = n.nvfp4_flash_attn_func(qx, kx, vx, d ** -0.5, causal=True, num_key_value_groups=h // hk,
                                      stochastic_rounding=False, **kw)
        out.backward(do)
        return out.detach(), qx.grad, kx.grad, vx.grad

    base = run()
    for other in (run(dkdv_scratch_bf16=False), run(dkdv_scratch_bf16=True),
                  run(q_packs=n._quant_nvfp4(q.reshape(z * h, s, d)),
                      k_packs=n._quant_nvfp4(k.reshape(z * hk, s, d)))):
        for a, b in zip(base, other):
            assert torch.equal(a, b)
    vl = run(cu_seqlens=cu)
    vl_packs = run(cu_seqlens=cu, q_packs=n._quant_nvfp4(q.reshape(z * h, s, d)),
                   k_packs=n._quant_nvfp4(k.reshape(z * hk, s, d)))
    for a, b in zip(vl, vl_packs):
        assert torch.equal(a, b)
    assert _status() == 0


def test_gradients_shape_dtype_and_no_leak_into_inputs():
    """Gradients are finite, shaped and typed like their inputs; inputs are left untouched
    (tests/test_nvfp4_train_backward.py:269-305 of the reference)."""
    z, h, hk, s, d = 2, 8, 2, 160, 128
    (q, _), (k, _), (v, _) = _qkv(z, h, hk, s, d, 90)
    do, _ = seeded_bf16((z, h, s, d), 93)
    q0, k0, v0 = q.clone(), k.clone(), v.clone()
    q, k, v = (t.requires_grad_(True) for t in (q, k, v))
    _n().nvfp4_flash_attn_func(q, k, v, d ** -0.5, causal=True, num_key_value_groups=h // hk).backward(do)
    for t, t0 in ((q, q0), (k, k0), (v, v0)):
        assert t.grad.shape == t.shape and t.grad.dtype == t.dtype
        assert torch.isfinite(t.grad).all()
        assert torch.equal(t.detach(), t0)
    assert _status() == 0
