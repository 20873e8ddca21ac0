"""KV cache and split-K decode on the GPU vs the CPU oracle and the reference fixtures."""

import numpy as np
import pytest
import torch

from conftest import bf16_bits_to_f32 as b2f
from gpu_util import cos, np_u8, seeded_bf16
from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu


def _n():
    import sageattention_b200.nvfp4 as n
    return n


def _status():
    from sageattention_b200 import _lib
    return _lib.read_status("cuda")


def _bits_to_cuda(bits):
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).cuda()


def test_append_equals_one_shot_bytes_config1():
    """BASELINE config 1b: K/V one-shot pack vs 1024 single-token appends, whole buffers."""
    z, hk, s, d = 1, 2, 1024, 128
    k, kf = seeded_bf16((z, hk, s, d), 1)
    v, vf = seeded_bf16((z, hk, s, d), 2)
    n = _n()
    cache = n.NVFP4KVCache(z, hk, d, s, "cuda")
    for t in range(s):
        cache.append(k[:, :, t:t + 1], v[:, :, t:t + 1])
    knv, ksc, vnv, vsc, s_kv, s_pad = n.nvfp4_quant_kv_decode(k, v)
    got = cache.get_packed()
    for a, b in zip(got[:4], (knv, ksc, vnv, vsc)):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    oracle = O.quant_kv_decode(kf, vf)
    for a, b in zip(got[:4], oracle[:4]):
        assert np.array_equal(np_u8(a), b)


def test_cache_state_machine_matches_reference_fixture(golden):
    g = golden("decode_cache")
    z, hk, d, gq, pre, n_app, win, length, partial = g["c_meta"].tolist()
    k, v, q = _bits_to_cuda(g["c_k"]), _bits_to_cuda(g["c_v"]), _bits_to_cuda(g["c_q"])
    n = _n()
    c = n.NVFP4KVCache(z, hk, d, 128, "cuda", torch.bfloat16, recent_window=win)
    c.prefill(k[:, :, :pre], v[:, :, :pre])
    for t in range(pre, pre + n_app):
        c.append(k[:, :, t:t + 1], v[:, :, t:t + 1])
    assert (c.length, c.partial_len) == (length, partial)
    for name in ("knv", "ksc", "vnv", "vsc"):
        assert np.array_equal(np_u8(getattr(c, name)), g["c_" + name]), name
    assert np.array_equal(c.rk.float().cpu().numpy(), b2f(g["c_rk"]))
    assert np.array_equal(c.rv.float().cpu().numpy(), b2f(g["c_rv"]))
    out = n.nvfp4_flash_decode_prequant(q.float(), c.get_packed(), d ** -0.5, gq)
    assert _status() == 0
    ref = g["c_out"]
    o = out.cpu().numpy()
    assert cos(o, ref) > 0.9995 and np.abs(o - ref).max() <= 2e-2
    hyb = c.hybrid_decode(q.float(), d ** -0.5, gq).cpu().numpy()
    assert _status() == 0
    assert cos(hyb, g["c_hyb"]) > 0.9995 and np.abs(hyb - g["c_hyb"]).max() <= 2e-2


@pytest.mark.parametrize("z,h,hk,s,d", [(2, 4, 1, 777, 128), (1, 8, 2, 1, 128), (1, 6, 1, 130, 128),
                                         (2, 16, 1, 515, 128), (1, 4, 2, 384, 256), (3, 2, 2, 2049, 256)])
def test_decode_matches_oracle(z, h, hk, s, d):
    g = h // hk
    q, qf = seeded_bf16((z, h, 1, d), 100 + s)
    k, kf = seeded_bf16((z, hk, s, d), 200 + s)
    v, vf = seeded_bf16((z, hk, s, d), 300 + s)
    n = _n()
    packed = n.nvfp4_quant_kv_decode(k, v)
    oracle_packed = O.quant_kv_decode(kf, vf)
    for a, b in zip(packed[:4], oracle_packed[:4]):
        assert np.array_equal(np_u8(a), b)
    from sageattention_b200.nvfp4 import flash
    out, lse = flash._decode_prequant_with_lse(q.float(), packed, d ** -0.5, g)
    assert _status() == 0
    nsplit, split_kv, _ = flash._decode_plan(s, z * hk, d, "cuda")
    if nsplit == 0:      # balanced decomposition: compare with the unsplit walk
        split_kv = -(-s // 128) * 128
    ref, ref_lse = O.decode_prequant(qf, oracle_packed, d ** -0.5, g, split_kv=split_kv)
    o = out.cpu().numpy()
    assert cos(o, ref) >= 0.999, cos(o, ref)
    assert np.abs(o - ref).max() <= 2e-2
    assert np.abs(lse.cpu().numpy() - ref_lse).max() <= 2e-3


@pytest.mark.parametrize("z,h,hk,s,d", [(3, 8, 2, 1100, 128), (37, 4, 4, 700, 128), (2, 16, 1, 5000, 128),
                                         (5, 4, 2, 1300, 256), (1, 4, 1, 130, 128), (150, 2, 2, 100, 128)])
def test_decode_balanced_decomposition(z, h, hk, s, d):
    """Forced balanced decomposition: CTAs own equal shares of the unit-major tile list, so units
    are cut at arbitrary tile boundaries and a CTA may hold pieces of several units."""
    g = h // hk
    q, qf = seeded_bf16((z, h, 1, d), 400 + s)
    k, kf = seeded_bf16((z, hk, s, d), 500 + s)
    v, vf = seeded_bf16((z, hk, s, d), 600 + s)
    from sageattention_b200.nvfp4 import flash
    packed = flash.nvfp4_quant_kv_decode(k, v)
    out, lse = flash._decode_core(q.float(), packed, d ** -0.5, g, True, split_kv=0)
    assert _status() == 0
    fixed, fixed_lse = flash._decode_core(q.float(), packed, d ** -0.5, g, True, split_kv=-(-s // 128) * 128)
    ref, ref_lse = O.decode_prequant(qf, O.quant_kv_decode(kf, vf), d ** -0.5, g, split_kv=-(-s // 128) * 128)
    o = out.cpu().numpy()
    assert np.isfinite(o).all()
    print("balanced vs oracle cos", cos(o, ref), "maxabs", np.abs(o - ref).max(), "vs one split", cos(o, fixed.cpu().numpy()))
    # another (equally valid) P-quantisation schedule than the unsplit walk: FP4-P rounding level
    assert cos(o, ref) >= 0.997 and np.abs(o - ref).max() <= 2e-2, (cos(o, ref), np.abs(o - ref).max())
    assert np.abs(lse.cpu().numpy() - ref_lse).max() <= 2e-3      # the statistics themselves are exact
    assert cos(o, fixed.cpu().numpy()) >= 0.997


def test_decode_multi_split_explicit():
    z, h, hk, s, d = 1, 4, 1, 1500, 128
    q, qf = seeded_bf16((z, h, 1, d), 5)
    k, kf = seeded_bf16((z, hk, s, d), 6)
    v, vf = seeded_bf16((z, hk, s, d), 7)
    from sageattention_b200.nvfp4 import flash
    packed = flash.nvfp4_quant_kv_decode(k, v)
    outs = []
    for split_kv in (128, 256, 512, 1536):
        out, lse = flash._decode_core(q.float(), packed, d ** -0.5, 4, True, split_kv=split_kv)
        assert _status() == 0
        ref, ref_lse = O.decode_prequant(qf, O.quant_kv_decode(kf, vf), d ** -0.5, 4, split_kv=split_kv)
        assert cos(out.cpu().numpy(), ref) >= 0.999
        assert np.abs(out.cpu().numpy() - ref).max() <= 2e-2
        assert np.abs(lse.cpu().numpy() - ref_lse).max() <= 2e-3
        outs.append(out)


def test_decode_reference_fixture(golden):
    g = golden("decode_cache")
    z, h, hk, s, d = g["meta"].tolist()
    q, k, v = _bits_to_cuda(g["q"]), _bits_to_cuda(g["k"]), _bits_to_cuda(g["v"])
    n = _n()
    packed = n.nvfp4_quant_kv_decode(k, v)
    for a, name in zip(packed[:4], ("knv", "ksc", "vnv", "vsc")):
        assert np.array_equal(np_u8(a), g[name])
    # the kernel's own split plan: a different (equally valid) P-quantisation schedule
    out = n.nvfp4_flash_decode_prequant(q.float(), packed, d ** -0.5, h // hk).cpu().numpy()
    assert _status() == 0
    assert cos(out, g["out"]) >= 0.995 and np.abs(out - g["out"]).max() <= 2e-2
    # the reference's split for this shape (flash.py:3255-3262): tile-for-tile comparison
    from sageattention_b200.nvfp4 import flash
    _, ref_split = O.decode_split_plan(s, z * hk)
    out2, _ = flash._decode_core(q.float(), packed, d ** -0.5, h // hk, False, split_kv=ref_split)
    out2 = out2.cpu().numpy()
    assert _status() == 0
    print("decode vs reference fixture: cos", cos(out2, g["out"]), "maxabs", np.abs(out2 - g["out"]).max())
    assert cos(out2, g["out"]) >= 0.999 and np.abs(out2 - g["out"]).max() <= 2e-2


def test_strided_cache_read_equals_contiguous_copy():
    """reference test: tests/test_nvfp4_kv_cache.py:253-289 -- bit-identical outputs."""
    z, hk, d, g = 2, 2, 128, 4
    n = _n()
    cache = n.NVFP4KVCache(z, hk, d, 1024, "cuda")
    k, _ = seeded_bf16((z, hk, 300, d), 9)
    v, _ = seeded_bf16((z, hk, 300, d), 10)
    cache.prefill(k, v)
    q, _ = seeded_bf16((z, hk * g, 1, d), 11)
    views = cache.get_packed()
    assert not views[0].is_contiguous()
    a = n.nvfp4_flash_decode_prequant(q, views, d ** -0.5, g)
    copies = tuple(t.contiguous() for t in views[:4]) + views[4:]
    b = n.nvfp4_flash_decode_prequant(q, copies, d ** -0.5, g)
    assert _status() == 0
    assert torch.equal(a, b)


def test_decode_vs_bf16_sdpa_floor():
    """reference floor: tests/test_nvfp4_attention.py:98,125 (cosine vs bf16 SDPA >= 0.95)."""
    z, h, hk, s, d = 2, 8, 2, 2048, 128
    q, _ = seeded_bf16((z, h, 1, d), 21)
    k, _ = seeded_bf16((z, hk, s, d), 22)
    v, _ = seeded_bf16((z, hk, s, d), 23)
    out = _n().nvfp4_flash_decode(q, k, v, d ** -0.5, 4)
    ref = torch.nn.functional.scaled_dot_product_attention(
        q.float(), k.float().repeat_interleave(4, 1), v.float().repeat_interleave(4, 1))
    assert _status() == 0
    assert cos(out.float().cpu().numpy(), ref.cpu().numpy()) > 0.95


def test_cache_guards_and_accounting():
    n = _n()
    with pytest.raises(AssertionError):
        n.NVFP4KVCache(1, 1, 64, 16, "cuda")
    c = n.NVFP4KVCache(1, 2, 128, 32, "cuda")
    k, _ = seeded_bf16((1, 2, 33, 128), 1)
    with pytest.raises(AssertionError, match="capacity"):
        c.prefill(k, k)
    with pytest.raises(RuntimeError, match="recent_window"):
        c.hybrid_decode(k[:, :, :1].repeat(1, 2, 1, 1), 0.1, 2)
    c2 = n.NVFP4KVCache(1, 2, 128, 32, "cuda", recent_window=8)
    with pytest.raises(RuntimeError, match="at least one token"):
        c2.hybrid_decode(k[:, :, :1].repeat(1, 2, 1, 1), 0.1, 2)
    with pytest.raises(AssertionError, match="multiple of 16"):
        c2._packed_upto(5)
    c.prefill(k[:, :, :32], k[:, :, :32])
    with pytest.raises(AssertionError, match="capacity"):
        c.append(k[:, :, :1], k[:, :, :1])
    big = n.NVFP4KVCache(1, 2, 128, 2048, "cuda")
    kk, _ = seeded_bf16((1, 2, 2048, 128), 3)
    big.prefill(kk, kk)
    assert big.bf16_bytes() / big.fp4_bytes() > 3.2      # tests/test_nvfp4_kv_cache.py:404-427


def test_hybrid_decode_long_matches_oracle():
    z, hk, d, g, win = 1, 2, 128, 4, 64
    s0, steps = 500, 40
    k, kf = seeded_bf16((z, hk, s0 + steps, d), 31)
    v, vf = seeded_bf16((z, hk, s0 + steps, d), 32)
    q, qf = seeded_bf16((z, hk * g, 1, d), 33)
    n = _n()
    c = n.NVFP4KVCache(z, hk, d, 1024, "cuda", recent_window=win)
    oc = O.KVCacheOracle(z, hk, d, 1024, recent_window=win)
    c.prefill(k[:, :, :s0], v[:, :, :s0]); oc.prefill(kf[:, :, :s0], vf[:, :, :s0])
    for t in range(s0, s0 + steps):
        c.append(k[:, :, t:t + 1], v[:, :, t:t + 1]); oc.append(kf[:, :, t:t + 1], vf[:, :, t:t + 1])
    for name in ("knv", "ksc", "vnv", "vsc"):
        assert np.array_equal(np_u8(getattr(c, name)), getattr(oc, name)), name
    out = c.hybrid_decode(q, d ** -0.5, g).float().cpu().numpy()
    assert _status() == 0
    ref = oc.hybrid_decode(qf, d ** -0.5, g)
    assert cos(out, ref) >= 0.999 and np.abs(out - ref).max() <= 2e-2


def test_fp16_cache_cut_zero_hybrid_and_packed_prefix():
    """fp16 operands (tests/test_nvfp4_kv_cache.py:501-524 of the reference), a sequence shorter
    than the recent window (cut == 0: the whole answer comes from the unquantised window,
    :339-364), and a 16-aligned packed prefix decoding like a one-shot pack of K/V[:cut] (:472-495)."""
    n = _n()
    z, hk, g, d, s = 1, 2, 4, 128, 200
    gen = torch.Generator().manual_seed(9)
    k = torch.randn(z, hk, s, d, generator=gen).to(torch.float16).cuda()
    v = torch.randn(z, hk, s, d, generator=gen).to(torch.float16).cuda()
    q = torch.randn(z, hk * g, 1, d, generator=gen).to(torch.float16).cuda()
    c = n.NVFP4KVCache(z, hk, d, 256, "cuda", torch.float16)
    c.prefill(k[:, :, :195], v[:, :, :195])
    for t in range(195, s):
        c.append(k[:, :, t:t + 1], v[:, :, t:t + 1])
    out_c = n.nvfp4_flash_decode_prequant(q, c.get_packed(), d ** -0.5, g)
    out_w = n.nvfp4_flash_decode_prequant(q, n.nvfp4_quant_kv_decode(k, v), d ** -0.5, g)
    assert out_c.dtype == torch.float16
    assert cos(out_c.float().cpu().numpy(), out_w.float().cpu().numpy()) > 0.9999   # same bytes on the valid region
    sdpa = torch.nn.functional.scaled_dot_product_attention(
        q.float(), k.float().repeat_interleave(g, 1), v.float().repeat_interleave(g, 1))
    assert cos(out_c.float().cpu().numpy(), sdpa.cpu().numpy()) > 0.97

    # cut == 0: pure unquantised-window path
    z2, s2, win = 2, 40, 256
    k2, _ = seeded_bf16((z2, hk, s2, d), 4)
    v2, _ = seeded_bf16((z2, hk, s2, d), 5)
    q2, _ = seeded_bf16((z2, hk * g, 1, d), 6)
    ch = n.NVFP4KVCache(z2, hk, d, 512, "cuda", recent_window=win)
    ch.prefill(k2[:, :, :35], v2[:, :, :35])
    for t in range(35, s2):
        ch.append(k2[:, :, t:t + 1], v2[:, :, t:t + 1])
    oh = ch.hybrid_decode(q2, d ** -0.5, g)
    ref = torch.nn.functional.scaled_dot_product_attention(
        q2.float(), k2.float().repeat_interleave(g, 1), v2.float().repeat_interleave(g, 1))
    assert torch.isfinite(oh).all()
    assert cos(oh.float().cpu().numpy(), ref.cpu().numpy()) > 0.999
    assert ch.hybrid_bytes() > ch.fp4_bytes()

    # packed prefix
    s3, cut = 777, 512
    k3, _ = seeded_bf16((z2, hk, s3, d), 7)
    v3, _ = seeded_bf16((z2, hk, s3, d), 8)
    c3 = n.NVFP4KVCache(z2, hk, d, 1024, "cuda")
    c3.prefill(k3, v3)
    a = n.nvfp4_flash_decode_prequant(q2, c3._packed_upto(cut), d ** -0.5, g)
    b = n.nvfp4_flash_decode_prequant(q2, n.nvfp4_quant_kv_decode(k3[:, :, :cut], v3[:, :, :cut]), d ** -0.5, g)
    assert cos(a.float().cpu().numpy(), b.float().cpu().numpy()) > 0.999
    assert _status() == 0


def test_state_dict_roundtrip_resumes_decoding(tmp_path):
    """A cache restored from its state dict (through torch.save / torch.load, into a cache of a
    different capacity) holds the same bytes and keeps appending and decoding bit-identically."""
    n = _n()
    z, hk, g, d, win = 2, 2, 4, 128, 64
    k, _ = seeded_bf16((z, hk, 300, d), 71)
    v, _ = seeded_bf16((z, hk, 300, d), 72)
    q, _ = seeded_bf16((z, hk * g, 1, d), 73)
    a = n.NVFP4KVCache(z, hk, d, 512, "cuda", recent_window=win)
    a.prefill(k[:, :, :250], v[:, :, :250])
    for t in range(250, 275):                               # stops inside a 16-key V group
        a.append(k[:, :, t:t + 1], v[:, :, t:t + 1])
    path = tmp_path / "cache.pt"
    torch.save(a.state_dict(), path)
    b = n.NVFP4KVCache(z, hk, d, 1024, "cuda", recent_window=win)
    b.load_state_dict(torch.load(path))
    assert (b.length, b.partial_len) == (a.length, a.partial_len)
    for t in range(275, 300):
        a.append(k[:, :, t:t + 1], v[:, :, t:t + 1])
        b.append(k[:, :, t:t + 1], v[:, :, t:t + 1])
    pa, pb = a.get_packed(), b.get_packed()
    assert torch.equal(pa[0], pb[0]) and torch.equal(pa[1].view(torch.uint8), pb[1].view(torch.uint8))
    ng = -(-300 // 16)
    assert torch.equal(pa[2][:, :, : ng * 8], pb[2][:, :, : ng * 8])
    assert torch.equal(pa[3].view(torch.uint8)[:, :, :ng], pb[3].view(torch.uint8)[:, :, :ng])
    assert torch.equal(n.nvfp4_flash_decode_prequant(q, pa, d ** -0.5, g),
                       n.nvfp4_flash_decode_prequant(q, pb, d ** -0.5, g))
    assert torch.equal(a.hybrid_decode(q, d ** -0.5, g), b.hybrid_decode(q, d ** -0.5, g))
    with pytest.raises(AssertionError, match="geometry"):
        n.NVFP4KVCache(z, hk, 256, 512, "cuda", recent_window=win).load_state_dict(a.state_dict())
    assert _status() == 0


def test_decode_demo_small_model():
    """The decode demo (random-weight GQA decoder, per-layer caches) tracks its bf16-cache run."""
    from sageattention_b200.nvfp4 import demo_decode
    rep = demo_decode.main(["--layers", "2", "--hidden", "512", "--heads", "4", "--kv-heads", "2",
                            "--vocab", "512", "--batch", "1", "--prompt", "300", "--new", "8", "--window", "64"])
    assert rep["fp4"]["logit_cos"] > 0.97 and rep["hybrid"]["logit_cos"] > 0.97
    assert rep["fp4"]["bf16_bytes"] / rep["fp4"]["bytes"] > 2.5
    assert _status() == 0
