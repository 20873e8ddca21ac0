"""The CPU oracle against fixtures produced by the reference's own kernels.

The fixtures come from ``tests/golden/make_golden.py`` (reference kernels run under the Triton
CPU interpreter).  Packed bytes must match bit for bit; attention outputs, which the reference
stores in bf16, must match to bf16 rounding.
"""

import numpy as np
import pytest

from conftest import bf16_bits_to_f32 as b2f
from oracle import nvfp4_oracle as O


def test_pack_bytes_match_reference(golden):
    g = golden("pack")
    nib, sc = O.pack(b2f(g["x"]))
    assert np.array_equal(nib, g["nib"])
    assert np.array_equal(sc, g["sc"])


def test_pack_transposed_padded_matches_reference(golden):
    g = golden("pack")
    nib, sc = O.pack(b2f(g["v"]), transpose=True, k_pad=128)
    assert np.array_equal(nib, g["vnib"])
    assert np.array_equal(sc, g["vsc"])
    # padded groups: floor scale byte 0x01 and zero nibbles (flash.py:375-376)
    assert np.all(sc[:, :, 3:] == 1) and np.all(nib[:, :, 24:] == 0)


def test_pack_second_shape(golden):
    g = golden("pack")
    nib, sc = O.pack(b2f(g["xs"]))
    assert np.array_equal(nib, g["snib"]) and np.array_equal(sc, g["ssc"])


def test_e4m3_codec_against_torch():
    torch = pytest.importorskip("torch")
    b = np.arange(0, 127, dtype=np.uint8)
    ref = torch.from_numpy(b.copy()).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(O.e4m3_to_f32(b), ref)
    rng = np.random.default_rng(0)
    x = np.exp(rng.uniform(np.log(2.0 ** -9), np.log(448.0), 200000)).astype(np.float32)
    x = np.concatenate([x, ref[1:], (ref[1:-1] + ref[2:]) / 2])  # exact values and exact ties
    x = np.clip(x, 2.0 ** -9, 448.0).astype(np.float32)
    want = torch.from_numpy(x.copy()).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(O.e4m3_bytes_from_f32(x), want)


def test_e2m1_ties_saturation_and_signed_zero():
    y = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.0, -0.1, -6.5, 0.2500001],
                 dtype=np.float32)
    assert O.e2m1_codes(y).tolist() == [0, 2, 2, 4, 4, 6, 6, 7, 8, 8, 15, 1]


def test_scale_floor_and_never_zero():
    # tests/test_nvfp4_attention.py:645-659 of the reference: 1e-6-amplitude input
    x = (np.random.default_rng(1).standard_normal((1, 4, 128)) * 1e-6).astype(np.float32)
    _, sc = O.pack(x)
    assert sc.min() == 1 and O.e4m3_to_f32(sc).min() == 2.0 ** -9


@pytest.mark.parametrize("name", ["causal_d128", "ragged_d128", "cross_d128", "bias_d128",
                                  "varlen_d128", "causal_d256", "causal_d128_t64"])
def test_forward_mode_b_matches_reference(golden, name):
    g = golden("forward")
    z, h, hk, sq, skv, d, causal, bias, bm, bn = g[name + "_meta"].tolist()
    q, k, v = b2f(g[name + "_q"]), b2f(g[name + "_k"]), b2f(g[name + "_v"])
    cu = g[name + "_cu"] if name + "_cu" in g.files else None
    kb = None
    if bias:
        kb = np.zeros((z, skv), np.float32)
        kb[:, skv - 7:] = -np.inf
    out, lse = O.attention_mode_b(q, k, v, d ** -0.5, bool(causal), h // hk, cu, kb, block_n=bn)
    ref = g[name + "_out"]
    # same arithmetic in the same order: only the BLAS summation order may differ
    assert np.max(np.abs(out - ref)) <= 1e-4
    assert O.cosine(out, ref) > 0.9999999
    assert np.allclose(lse, g[name + "_lse"].reshape(lse.shape), atol=2e-5, rtol=1e-5)


def test_decode_matches_reference(golden):
    g = golden("decode_cache")
    z, h, hk, s, d = g["meta"].tolist()
    q, k, v = b2f(g["q"]), b2f(g["k"]), b2f(g["v"])
    packed = O.quant_kv_decode(k, v)
    for a, b in zip(packed[:4], (g["knv"], g["ksc"], g["vnv"], g["vsc"])):
        assert np.array_equal(a, b)
    out, _ = O.decode_prequant(q, packed, d ** -0.5, h // hk)
    ref = g["out"]
    assert np.max(np.abs(out - ref)) <= 1e-4
    assert O.cosine(out, ref) > 0.9999999


def test_cache_state_machine_matches_reference(golden):
    g = golden("decode_cache")
    z, hk, d, gq, pre, n_app, win, length, partial = g["c_meta"].tolist()
    k, v, q = b2f(g["c_k"]), b2f(g["c_v"]), b2f(g["c_q"])
    c = O.KVCacheOracle(z, hk, d, 128, recent_window=win)
    c.prefill(k[:, :, :pre], v[:, :, :pre])
    for t in range(pre, pre + n_app):
        c.append(k[:, :, t:t + 1], v[:, :, t:t + 1])
    assert (c.length, c.partial_len) == (length, partial)
    for name in ("knv", "ksc", "vnv", "vsc"):
        assert np.array_equal(getattr(c, name), g["c_" + name]), name
    assert np.array_equal(c.rk, b2f(g["c_rk"])) and np.array_equal(c.rv, b2f(g["c_rv"]))
    out, _ = O.decode_prequant(q, c.get_packed(), d ** -0.5, gq)
    assert np.max(np.abs(out - g["c_out"])) <= 1e-4
    hyb = c.hybrid_decode(q, d ** -0.5, gq)
    assert np.max(np.abs(hyb - g["c_hyb"])) <= 1e-4


def test_incremental_equals_one_shot_on_valid_region():
    rng = np.random.default_rng(7)
    z, hk, d, s = 1, 2, 128, 53
    k = rng.standard_normal((z, hk, s, d)).astype(np.float32)
    v = rng.standard_normal((z, hk, s, d)).astype(np.float32)
    c = O.KVCacheOracle(z, hk, d, 256)
    for t in range(s):
        c.append(k[:, :, t:t + 1], v[:, :, t:t + 1])
    knv, ksc, vnv, vsc, _, sp = O.quant_kv_decode(k, v)
    ng = -(-s // 16)
    assert np.array_equal(c.knv[:, :s], knv) and np.array_equal(c.ksc[:, :s], ksc)
    assert np.array_equal(c.vnv[:, :, : ng * 8], vnv[:, :, : ng * 8])
    assert np.array_equal(c.vsc[:, :, :ng], vsc[:, :, :ng])
    # beyond the valid groups the two differ by design: zero-initialised cache vs floor scale
    assert np.all(c.vsc[:, :, ng:] == 0) and np.all(vsc[:, :, ng:] == 1)


def test_mxfp8_pack_matches_reference(golden):
    """The oracle's MXFP8 pack against the bytes and scale exponents the reference's own
    `_pack_mxfp8_along_k` (flash.py:243-257) produced: random magnitudes over 2^-20 .. 2^12, an
    all-zero group, a group whose maximum is exactly 448, and a row of 1e-12 values."""
    g = golden("mxfp8_pack")
    q, sc = O.pack_mxfp8(b2f(g["x"])[None])
    assert np.array_equal(sc[0], g["sc"])
    assert np.array_equal(q[0], g["q"])


@pytest.mark.parametrize("name,floor", [("hp_d128", 0.985), ("hp_varlen_d128", 0.985),
                                        ("rownorm_d128", 0.93), ("fp8rn_d128", 0.93)])
def test_reference_grads_close_to_exact_grads(golden, name, floor):
    """The reference's own backward (HP, all-FP4 and MXFP8) against analytic gradients."""
    g = golden("backward_fp8" if name.startswith("fp8") else "backward")
    z, h, hk, s, d = g[name + "_meta"].tolist()
    cu = g[name + "_cu"] if name + "_cu" in g.files else None
    q, k, v, do = (b2f(g[f"{name}_{n}"]) for n in ("q", "k", "v", "do"))
    dq, dk, dv = O.attention_grads(q, k, v, do, d ** -0.5, True, h // hk, cu)
    for mine, nm in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert O.cosine(mine, g[f"{name}_{nm}"]) > floor, nm
