"""CUDA packer vs the CPU oracle and the reference fixtures: packed bytes must be bit-exact."""

import numpy as np
import pytest
import torch

from conftest import bf16_bits_to_f32 as b2f
from gpu_util import np_u8, seeded_bf16
from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu


def _nvfp4():
    import sageattention_b200.nvfp4 as n
    return n


def _bits_to_cuda(bits):
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).cuda()


def test_golden_pack_bytes(golden):
    g = golden("pack")
    n = _nvfp4()
    nib, sc = n._quant_nvfp4(_bits_to_cuda(g["x"]))
    assert np.array_equal(np_u8(nib), g["nib"]) and np.array_equal(np_u8(sc), g["sc"])
    vn, vs = n._quant_nvfp4(_bits_to_cuda(g["v"]), transpose=True, k_pad=128)
    assert np.array_equal(np_u8(vn), g["vnib"]) and np.array_equal(np_u8(vs), g["vsc"])
    sn, ss = n._quant_nvfp4(_bits_to_cuda(g["xs"]))
    assert np.array_equal(np_u8(sn), g["snib"]) and np.array_equal(np_u8(ss), g["ssc"])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(2, 33, 128), (1, 1, 16), (3, 7, 256), (1, 200, 64)])
def test_rows_pack_matches_oracle(dtype, shape):
    g = torch.Generator().manual_seed(hash((shape, str(dtype))) % 2 ** 31)
    x = (torch.randn(*shape, generator=g) * 1.7).to(dtype)
    nib, sc = _nvfp4()._quant_nvfp4(x.cuda())
    onib, osc = O.pack(x.float().numpy())
    assert np.array_equal(np_u8(nib), onib) and np.array_equal(np_u8(sc), osc)


@pytest.mark.parametrize("s,d,pad", [(45, 128, 128), (1, 128, 16), (300, 256, 384), (129, 64, 256),
                                     (1024, 128, 1024)])
def test_transposed_pack_matches_oracle(s, d, pad):
    x, xf = seeded_bf16((2, s, d), seed=s * 7 + d)
    nib, sc = _nvfp4()._quant_nvfp4(x, transpose=True, k_pad=pad)
    onib, osc = O.pack(xf, transpose=True, k_pad=pad)
    assert np.array_equal(np_u8(nib), onib) and np.array_equal(np_u8(sc), osc)


def test_strided_views_and_zshd_layout():
    # [Z, S, H, D] storage viewed as [Z*H, S, D] heads (non-contiguous rows)
    z, s, h, d = 2, 50, 3, 128
    x, xf = seeded_bf16((z, s, h, d), seed=11)
    view = x.permute(0, 2, 1, 3)[0]          # [H, S, D], row stride H*D
    nib, sc = _nvfp4()._quant_nvfp4(view)
    onib, osc = O.pack(np.transpose(xf, (0, 2, 1, 3))[0])
    assert np.array_equal(np_u8(nib), onib) and np.array_equal(np_u8(sc), osc)
    # unaligned base pointer (offset by one element) falls back to scalar loads
    flat = x.reshape(-1)[1: 1 + 4 * 128].reshape(1, 4, 128)
    nib, sc = _nvfp4()._quant_nvfp4(flat)
    onib, osc = O.pack(xf.reshape(-1)[1: 1 + 4 * 128].reshape(1, 4, 128))
    assert np.array_equal(np_u8(nib), onib) and np.array_equal(np_u8(sc), osc)
    # a base that is 16-byte but not 32-byte aligned: 128-bit loads, one group per thread
    flat = x.reshape(-1)[8: 8 + 40 * 128].reshape(1, 40, 128)
    nib, sc = _nvfp4()._quant_nvfp4(flat)
    onib, osc = O.pack(xf.reshape(-1)[8: 8 + 40 * 128].reshape(1, 40, 128))
    assert np.array_equal(np_u8(nib), onib) and np.array_equal(np_u8(sc), osc)
    # 32-byte aligned rows with a row stride larger than the row (four groups per thread, strided)
    wide = x.reshape(-1)[: 64 * 256].reshape(1, 64, 256)[:, :, :128]
    nib, sc = _nvfp4()._quant_nvfp4(wide)
    onib, osc = O.pack(xf.reshape(-1)[: 64 * 256].reshape(1, 64, 256)[:, :, :128])
    assert np.array_equal(np_u8(nib), onib) and np.array_equal(np_u8(sc), osc)


def test_adversarial_values():
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0], np.float32)
    rows = []
    for e in range(-12, 10):                      # every binade the scale can take
        rows.append(np.concatenate([ties, -ties]) * np.float32(2.0 ** e))
    x = np.stack(rows)[None].astype(np.float32)
    x = np.concatenate([x, np.zeros_like(x), -np.zeros_like(x)], axis=1)
    xt = torch.from_numpy(x).to(torch.bfloat16)
    nib, sc = _nvfp4()._quant_nvfp4(xt.cuda())
    onib, osc = O.pack(xt.float().numpy())
    assert np.array_equal(np_u8(nib), onib) and np.array_equal(np_u8(sc), osc)


def test_exhaustive_bf16_inputs_against_oracle():
    """Every finite bf16 bit pattern as the group's first element, with a fixed partner that
    pins the scale, for a sweep of scales: the element quantiser is checked exhaustively."""
    bits = np.arange(65536, dtype=np.uint16)
    vals = b2f(bits)
    finite = np.isfinite(vals)
    bits = bits[finite]
    n = bits.size
    for partner in (6.0, 0.01171875, 3.0e-3, 448.0 * 6, 1.0e4, 0.7):
        grp = np.zeros((1, n, 16), dtype=np.float32)
        grp[0, :, 0] = b2f(bits)
        grp[0, :, 1] = partner
        xt = torch.from_numpy(grp).to(torch.bfloat16)
        nib, sc = _nvfp4()._quant_nvfp4(xt.cuda())
        onib, osc = O.pack(xt.float().numpy())
        assert np.array_equal(np_u8(sc), osc), partner
        assert np.array_equal(np_u8(nib), onib), partner


def test_scale_floor_exact_and_positive():
    # reference test: tests/test_nvfp4_attention.py:645-659
    x = (torch.randn(1, 8, 128) * 1e-6).to(torch.bfloat16).cuda()
    _, sc = _nvfp4()._quant_nvfp4(x)
    assert float(sc.float().min()) == 2.0 ** -9 and bool((sc.float() > 0).all())


def test_empty_and_errors():
    n = _nvfp4()
    nib, sc = n._quant_nvfp4(torch.empty(0, 4, 128, dtype=torch.bfloat16, device="cuda"))
    assert nib.shape == (0, 4, 64) and sc.shape == (0, 4, 8)
    with pytest.raises(AssertionError, match="multiple of 16"):
        n._quant_nvfp4(torch.zeros(1, 2, 24, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(RuntimeError, match="no CPU path"):
        n._quant_nvfp4(torch.zeros(1, 2, 32, dtype=torch.bfloat16))


def test_large_pack_roundtrip_property():
    """Full-size property (C2's K tensor for one batch): dequantised values stay within half a
    grid step of the input relative to the group scale, and re-packing the dequantised tensor
    reproduces the same bytes (idempotence)."""
    x = torch.randn(8, 8192, 128, device="cuda", dtype=torch.bfloat16)
    n = _nvfp4()
    nib, sc = n._quant_nvfp4(x)
    lut = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], device="cuda")
    codes = torch.stack([nib & 15, nib >> 4], dim=-1).reshape(8, 8192, 128).long()
    deq = lut[codes] * sc.float().repeat_interleave(16, dim=-1)
    err = (deq - x.float()).abs() / sc.float().repeat_interleave(16, dim=-1)
    assert float(err.max()) <= 1.0 + 1e-3      # widest e2m1 gap is 2 (4 -> 6): half of it
    nib2, sc2 = n._quant_nvfp4(deq.to(torch.bfloat16))
    assert torch.equal(nib2, nib) and torch.equal(sc2.view(torch.uint8), sc.view(torch.uint8))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("b,s,d,pad", [(2, 300, 128, 384), (1, 16, 128, 16), (3, 77, 256, 128), (1, 1000, 64, 1008),
                                       (2, 129, 48, None)])
def test_dual_pack_equals_two_single_packs(dtype, b, s, d, pad):
    """One-read dual pack (reference property, tests/test_nvfp4_attention.py:423-447): bytes equal
    the along-D pack and the along-S pack taken separately, and both equal the oracle."""
    g = torch.Generator().manual_seed(s * 13 + d)
    x = (torch.randn(b, s, d, generator=g) * 1.3).to(dtype)
    n = _nvfp4()
    nd, sd, ns, ss = n._quant_nvfp4_dual(x.cuda(), pad)
    sp = pad if pad is not None else ((s + 15) // 16) * 16
    assert ns.shape == (b, d, sp // 2) and ss.shape == (b, d, sp // 16) and sd.dtype == torch.float8_e4m3fn
    od, osd = n._quant_nvfp4(x.cuda())
    ot, ost = n._quant_nvfp4(x.cuda(), transpose=True, k_pad=sp)
    assert torch.equal(nd, od) and torch.equal(sd.view(torch.uint8), osd.view(torch.uint8))
    assert torch.equal(ns, ot) and torch.equal(ss.view(torch.uint8), ost.view(torch.uint8))
    cn, cs = O.pack(x.float().numpy())
    tn, ts = O.pack(x.float().numpy(), transpose=True, k_pad=sp)
    assert np.array_equal(np_u8(nd), cn) and np.array_equal(np_u8(sd), cs)
    assert np.array_equal(np_u8(ns), tn) and np.array_equal(np_u8(ss), ts)


def test_dual_pack_strided_rows():
    z, s, h, d = 2, 70, 3, 128
    x, xf = seeded_bf16((z, s, h, d), seed=21)
    view = x.permute(0, 2, 1, 3)[1]          # [H, S, D] with row stride H*D
    nd, sd, ns, ss = _nvfp4()._quant_nvfp4_dual(view, 128)
    ref = np.transpose(xf, (0, 2, 1, 3))[1]
    cn, cs = O.pack(ref)
    tn, ts = O.pack(ref, transpose=True, k_pad=128)
    assert np.array_equal(np_u8(nd), cn) and np.array_equal(np_u8(sd), cs)
    assert np.array_equal(np_u8(ns), tn) and np.array_equal(np_u8(ss), ts)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("zh,zhk,sq,skv,d", [(4, 2, 200, 200, 128), (2, 2, 1, 300, 128), (6, 3, 130, 257, 256),
                                             (32, 8, 1024, 1024, 128)])
def test_fused_qkv_prepack_equals_three_packs(dtype, zh, zhk, sq, skv, d):
    """One-launch Q/K/V pre-pack (flash.py:579-732): bytes equal three separate packs."""
    g = torch.Generator().manual_seed(zh * 1000 + skv)
    q = torch.randn(zh, sq, d, generator=g).to(dtype).cuda()
    k = (torch.randn(zhk, skv, d, generator=g) * 2.0).to(dtype).cuda()
    v = torch.randn(zhk, skv, d, generator=g).to(dtype).cuda()
    n = _nvfp4()
    sp = ((skv + 127) // 128) * 128
    from sageattention_b200.nvfp4 import flash
    got = flash._quant_qkv_fwd(q, k, v, sp)
    want = (*n._quant_nvfp4(q), *n._quant_nvfp4(k), *n._quant_nvfp4(v, transpose=True, k_pad=sp))
    for a, b in zip(got, want):
        assert a.shape == b.shape and a.dtype == b.dtype
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    # strided operands (a [Z, S, H, D] projection output viewed per head) take the same path
    big = torch.randn(2, skv, zhk, d, generator=g).to(dtype).cuda()
    kv = big.permute(0, 2, 1, 3)[0]          # [zhk, skv, d], unit stride along d only
    got = flash._quant_qkv_fwd(q, kv, kv, sp)
    want = (*n._quant_nvfp4(q), *n._quant_nvfp4(kv), *n._quant_nvfp4(kv, transpose=True, k_pad=sp))
    for a, b in zip(got, want):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))


def test_convert_fp32_to_fp4_packed_pairs():
    """Host-callable stand-in for the reference's device function (_fp4_pack.py:15-56): first
    element of a pair in the low nibble, RTNE to the e2m1 grid, saturating, sign kept on -0."""
    vals = torch.tensor([0.0, -0.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.3, -6.5, 0.5, 1.0, 1.5, 6.0],
                        dtype=torch.float32).cuda()
    lo, hi = vals, vals.flip(0)
    got = _nvfp4().convert_fp32_to_fp4_packed((lo, hi)).cpu().numpy()
    c_lo = O.e2m1_codes(lo.cpu().numpy())
    c_hi = O.e2m1_codes(hi.cpu().numpy())
    assert np.array_equal(got, (c_lo | (c_hi << 4)).astype(np.uint8))
    assert "convert_fp32_to_fp4_packed" in _nvfp4().__all__


def test_gqa_reduce_cast_dkdv():
    """`_gqa_reduce_cast_dkdv` (flash.py:2525-2557): per-query-head planes summed over each group."""
    z, hk, g, s, d = 2, 3, 4, 10, 16
    gen = torch.Generator().manual_seed(3)
    a = torch.randn(z * hk * g, s, d, generator=gen).cuda()
    b = torch.randn(z * hk * g, s, d, generator=gen).cuda()
    dk, dv = _nvfp4()._gqa_reduce_cast_dkdv(a, b, z, hk, g, torch.bfloat16)
    assert dk.shape == (z, hk, s, d) and dk.dtype == torch.bfloat16
    ref = a.reshape(z, hk, g, s, d).double().sum(2)
    assert torch.allclose(dk.double(), ref, atol=2e-2, rtol=1e-2)
    assert torch.allclose(dv.double(), b.reshape(z, hk, g, s, d).double().sum(2), atol=2e-2, rtol=1e-2)


def test_stochastic_pack_keeps_exact_values_and_scales():
    """Stochastic rounding leaves e2m1-representable quotients alone, so on such inputs the bytes of
    both packs equal the round-to-nearest pack whatever the seed (this also pins the nibble order of
    the hardware's four-wide stochastic convert)."""
    g = torch.Generator().manual_seed(5)
    codes = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    b, s, d = 2, 160, 128
    x = codes[torch.randint(0, 8, (b, s, d), generator=g)] * (torch.randint(0, 2, (b, s, d), generator=g) * 2 - 1)
    x[:, :, ::16] = 6.0          # every group along D has amax 6 (scale 1)
    x[:, ::16, :] = 6.0          # and every group along S too
    x = x.to(torch.bfloat16).cuda()
    n = _nvfp4()
    want = n._quant_nvfp4_dual(x, 256)
    for seed in (1, 77):
        got = n._quant_nvfp4_dual(x, 256, _sr=(True, True), _seed=seed)
        for a, w in zip(got, want):
            assert torch.equal(a.view(torch.uint8), w.view(torch.uint8))


def test_stochastic_pack_is_unbiased_and_seeded():
    """flash.py:161-176 (the reference's dithered pack): scale bytes are those of the plain pack,
    the same seed repeats the same bytes, another seed differs, and the mean of the dequantised
    packs over many seeds converges to the input far below the round-to-nearest error."""
    g = torch.Generator().manual_seed(6)
    b, s, d = 1, 256, 128
    x = (torch.randn(b, s, d, generator=g) * 0.7).to(torch.bfloat16).cuda()
    xf = x.float().cpu().numpy()
    n = _nvfp4()
    rn = n._quant_nvfp4_dual(x, 256)
    a1 = n._quant_nvfp4_dual(x, 256, _sr=(True, True), _seed=11)
    a2 = n._quant_nvfp4_dual(x, 256, _sr=(True, True), _seed=11)
    a3 = n._quant_nvfp4_dual(x, 256, _sr=(True, True), _seed=12)
    only_d = n._quant_nvfp4_dual(x, 256, _sr=(True, False), _seed=11)
    for i in range(4):
        assert torch.equal(a1[i].view(torch.uint8), a2[i].view(torch.uint8))
    assert torch.equal(a1[1].view(torch.uint8), rn[1].view(torch.uint8))      # scales: along D
    assert torch.equal(a1[3].view(torch.uint8), rn[3].view(torch.uint8))      # scales: along S
    assert not torch.equal(a1[0], a3[0]) and not torch.equal(a1[2], a3[2])
    assert not torch.equal(a1[0], rn[0]) and not torch.equal(a1[2], rn[2])
    assert torch.equal(only_d[0], a1[0]) and torch.equal(only_d[2], rn[2])
    nseed = 96
    acc_d = np.zeros((b, s, d), np.float64)
    acc_s = np.zeros((b, d, s), np.float64)
    for seed in range(nseed):
        nd, sd, ns, ss = n._quant_nvfp4_dual(x, 256, _sr=(True, True), _seed=1000 + seed)
        acc_d += O.unpack(np_u8(nd), np_u8(sd))
        acc_s += O.unpack(np_u8(ns), np_u8(ss))[:, :, :s]
    err_rn_d = np.abs(O.unpack(np_u8(rn[0]), np_u8(rn[1])) - xf).mean()
    err_sr_d = np.abs(acc_d / nseed - xf).mean()
    err_sr_s = np.abs(acc_s / nseed - np.transpose(xf, (0, 2, 1))).mean()
    print("mean abs error: round-to-nearest", err_rn_d, "mean of", nseed, "stochastic packs", err_sr_d, err_sr_s)
    assert err_sr_d < 0.25 * err_rn_d and err_sr_s < 0.25 * err_rn_d


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("b,s,d,pad", [(2, 300, 128, 384), (1, 32, 64, 32), (3, 77, 256, 128), (1, 1000, 128, 1024)])
def test_mxfp8_transposed_pack_matches_oracle(dtype, b, s, d, pad):
    """MXFP8 pack along the tokens (`_pack_mxfp8_along_k` of the transposed operand,
    flash.py:243-257): bytes and scale exponents equal the CPU restatement, on magnitudes from
    denormal-scale to saturating, zeros included; the dequantised tensor is within e4m3 precision."""
    from sageattention_b200.nvfp4 import flash
    g = torch.Generator().manual_seed(s * 7 + d)
    mag = torch.exp2(torch.randint(-30, 20, (b, s // 8 + 1, 1), generator=g).float()).repeat_interleave(8, dim=1)[:, :s]
    x = (torch.randn(b, s, d, generator=g) * mag).to(dtype)
    x[0, : min(s, 40), 3] = 0.0                      # an all-zero group
    if dtype == torch.float32:
        x[0, 0, 5] = 3.0e38
    q, sc = flash._quant_mxfp8_t(x.cuda(), pad)
    oq, osc = O.pack_mxfp8(x.float().numpy(), transpose=True, k_pad=pad)
    assert np.array_equal(np_u8(sc), osc)
    assert np.array_equal(np_u8(q), oq)
    back = O.unpack_mxfp8(np_u8(q), np_u8(sc))[:, :, :s]
    ref = np.transpose(x.float().numpy(), (0, 2, 1))
    gmax = np.repeat(np.exp2(np_u8(sc).astype(np.float64) - 127.0) * 448.0, 32, axis=-1)[:, :, :s]
    assert np.all(np.abs(back - ref) <= gmax * 2.0 ** -4 + 1e-37)


def test_mxfp8_pack_matches_reference_fixture(golden):
    """The GPU MXFP8 pack against the bytes of the reference's own `_pack_mxfp8_along_k`
    (tests/golden/mxfp8_pack.npz): rows of the fixture are packed along their 128 columns, which is
    the along-S pack of the transposed tensor."""
    from sageattention_b200.nvfp4 import flash
    g = golden("mxfp8_pack")
    x = torch.from_numpy(b2f(g["x"]))                       # [rows, K]
    q, sc = flash._quant_mxfp8_t(x.t().contiguous()[None].to(torch.bfloat16).cuda(), x.shape[1])
    assert np.array_equal(np_u8(sc)[0], g["sc"])
    assert np.array_equal(np_u8(q)[0], g["q"])
