"""Seeded random shapes through forward, backward and decode against the CPU oracle: ragged
lengths, cross attention, GQA groups, both head dims, packed varlen, forced decode decompositions."""

import numpy as np
import pytest
import torch

from gpu_util import cos, seeded_bf16
from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu


def _status():
    from sageattention_b200 import _lib
    return _lib.read_status("cuda")


def _cases(n, seed):
    rng = np.random.default_rng(seed)
    out = []
    for i in range(n):
        d = int(rng.choice([128, 128, 256]))
        hk = int(rng.choice([1, 2, 3]))
        g = int(rng.choice([1, 2, 4, 8]))
        z = int(rng.choice([1, 2]))
        sq = int(rng.integers(1, 400))
        skv = sq + int(rng.integers(0, 300)) * int(rng.integers(0, 2))
        causal = bool(rng.integers(0, 2))
        out.append((i, z, hk * g, hk, sq, skv, d, causal))
    return out


@pytest.mark.parametrize("i,z,h,hk,sq,skv,d,causal", _cases(14, 2024))
def test_forward_random_shapes(i, z, h, hk, sq, skv, d, causal):
    import sageattention_b200.nvfp4 as nv
    q, qf = seeded_bf16((z, h, sq, d), 3000 + i)
    k, kf = seeded_bf16((z, hk, skv, d), 4000 + i)
    v, vf = seeded_bf16((z, hk, skv, d), 5000 + i)
    out, lse = nv.nvfp4_flash_attention(q, k, v, d ** -0.5, causal=causal, num_key_value_groups=h // hk,
                                        return_lse=True)
    assert _status() == 0
    ref, ref_lse = O.attention_mode_b(qf, kf, vf, d ** -0.5, causal, h // hk)
    o = out.float().cpu().numpy()
    assert np.isfinite(o).all()
    assert cos(o, ref) >= 0.999, cos(o, ref)
    assert np.abs(o - ref).max() <= 2e-2 + 2.0 ** -7
    assert np.abs(lse.cpu().numpy().reshape(-1) - ref_lse.reshape(-1)).max() <= 2e-3


@pytest.mark.parametrize("i,z,h,hk,sq,skv,d,causal", _cases(10, 77))
def test_backward_random_shapes(i, z, h, hk, sq, skv, d, causal):
    import sageattention_b200.nvfp4 as nv
    q, qf = seeded_bf16((z, h, sq, d), 6000 + i)
    k, kf = seeded_bf16((z, hk, skv, d), 7000 + i)
    v, vf = seeded_bf16((z, hk, skv, d), 8000 + i)
    do, dof = seeded_bf16((z, h, sq, d), 9000 + i)
    qq, kk, vv = (t.clone().requires_grad_(True) for t in (q, k, v))
    out = nv.nvfp4_flash_attn_func(qq, kk, vv, d ** -0.5, causal=causal, num_key_value_groups=h // hk,
                                   backward_grad_dots="bf16")
    out.backward(do)
    assert _status() == 0
    rq, rk, rv = O.attention_grads(qf, kf, vf, dof, d ** -0.5, causal, h // hk)
    # the FP4 recompute noise of P is the floor: 0.990 +- 0.002 at a few hundred keys, lower below
    floor = 0.985 if min(sq, skv) >= 256 else 0.97
    for nm, a, b in (("dq", qq.grad, rq), ("dk", kk.grad, rk), ("dv", vv.grad, rv)):
        a = a.float().cpu().numpy()
        assert np.isfinite(a).all(), nm
        if np.abs(b).max() < 1e-6:
            continue                                   # a single visible key: exact gradient is zero
        assert cos(a, b) >= floor, (nm, cos(a, b))


@pytest.mark.parametrize("i", range(8))
def test_decode_random_shapes(i):
    from sageattention_b200.nvfp4 import flash
    rng = np.random.default_rng(500 + i)
    d = int(rng.choice([128, 256]))
    hk, g, z = int(rng.choice([1, 2, 5])), int(rng.choice([1, 4, 8, 16])), int(rng.choice([1, 3, 9]))
    s = int(rng.integers(1, 3000))
    q, qf = seeded_bf16((z, hk * g, 1, d), 100 + i)
    k, kf = seeded_bf16((z, hk, s, d), 200 + i)
    v, vf = seeded_bf16((z, hk, s, d), 300 + i)
    packed = flash.nvfp4_quant_kv_decode(k, v)
    full = -(-s // 128) * 128
    ref, ref_lse = O.decode_prequant(qf, O.quant_kv_decode(kf, vf), d ** -0.5, g, split_kv=full)
    for split in (None, 0, full):
        out, lse = flash._decode_core(q.float(), packed, d ** -0.5, g, True, split_kv=split)
        assert _status() == 0
        o = out.cpu().numpy()
        assert np.isfinite(o).all()
        assert cos(o, ref) >= 0.997 and np.abs(o - ref).max() <= 2e-2, (split, cos(o, ref))
        assert np.abs(lse.cpu().numpy() - ref_lse).max() <= 2e-3
