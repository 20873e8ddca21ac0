"""tcgen05 NVFP4 forward vs the CPU oracle, the reference fixtures and the reference's own
bit-identity properties (tests/test_nvfp4_attention.py and test_nvfp4_train_forward.py there)."""

import numpy as np
import pytest
import torch

from conftest import bf16_bits_to_f32 as b2f
from gpu_util import cos, seeded_bf16
from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu

# tolerances of the task statement: forward vs the emulated-FP4 oracle
COS_MIN = 0.995
MAXABS = 2e-2


def _n():
    import sageattention_b200.nvfp4 as n
    return n


def _status():
    from sageattention_b200 import _lib
    return _lib.read_status("cuda")


def _bits_to_cuda(bits):
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).cuda()


@pytest.mark.parametrize("name", ["causal_d128", "ragged_d128", "cross_d128", "bias_d128",
                                  "varlen_d128", "causal_d256"])
def test_forward_matches_reference_fixture(golden, name):
    """Outputs of the reference's own forward kernel (128-key tiles) on the same inputs."""
    g = golden("forward")
    z, h, hk, sq, skv, d, causal, bias, bm, bn = g[name + "_meta"].tolist()
    q, k, v = (_bits_to_cuda(g[f"{name}_{t}"]).float() for t in "qkv")
    cu = torch.from_numpy(g[name + "_cu"]).cuda() if name + "_cu" in g.files else None
    kb = None
    if bias:
        kb = torch.zeros(z, skv, device="cuda")
        kb[:, skv - 7:] = float("-inf")
    out, lse = _n().nvfp4_flash_attention(q, k, v, d ** -0.5, causal=bool(causal),
                                          num_key_value_groups=h // hk, key_pad_bias=kb,
                                          cu_seqlens=cu, return_lse=True)
    assert _status() == 0
    o, ref = out.cpu().numpy(), g[name + "_out"]
    print(name, "cos", cos(o, ref), "maxabs", np.abs(o - ref).max())
    assert cos(o, ref) >= 0.9999 and np.abs(o - ref).max() <= MAXABS
    assert np.abs(lse.cpu().numpy().reshape(-1) - g[name + "_lse"].reshape(-1)).max() <= 2e-3


def test_config1_cpu_reference_path():
    """BASELINE config 1: Z1 H8 Hk2 S1024 D128 causal, seeded N(0,1) bf16."""
    z, h, hk, s, d = 1, 8, 2, 1024, 128
    q, qf = seeded_bf16((z, h, s, d), 1001)
    k, kf = seeded_bf16((z, hk, s, d), 1002)
    v, vf = seeded_bf16((z, hk, s, d), 1003)
    out = _n().nvfp4_flash_attention(q, k, v, d ** -0.5, causal=True, num_key_value_groups=4)
    assert _status() == 0
    o = out.float().cpu().numpy()
    ref_b, _ = O.attention_mode_b(qf, kf, vf, d ** -0.5, True, 4)
    ref_a, _ = O.attention_mode_a(qf, kf, vf, d ** -0.5, True, 4)
    cb, mb = cos(o, ref_b), np.abs(o - ref_b).max()
    ca, ma = cos(o, ref_a), np.abs(o - ref_a).max()
    print(f"C1 vs oracle B (P quantised, the reference's arithmetic): cos {cb:.6f} max-abs {mb:.4f}")
    print(f"C1 vs oracle A (P exact): cos {ca:.6f} max-abs {ma:.4f}")
    assert cb >= 0.9995 and mb <= MAXABS + 2.0 ** -7   # bf16 output rounding on |o| <= 4
    assert ca >= COS_MIN


@pytest.mark.parametrize("s", [1, 16, 17, 33, 128, 200, 256, 777])
@pytest.mark.parametrize("d,g", [(128, 1), (128, 4), (256, 2)])
def test_forward_matches_oracle_shapes(s, d, g):
    z, hk = 1, 2
    h = hk * g
    q, qf = seeded_bf16((z, h, s, d), 7 * s + d)
    k, kf = seeded_bf16((z, hk, s, d), 7 * s + d + 1)
    v, vf = seeded_bf16((z, hk, s, d), 7 * s + d + 2)
    out, lse = _n().nvfp4_flash_attention(q.float(), k.float(), v.float(), d ** -0.5, causal=True,
                                          num_key_value_groups=g, return_lse=True)
    assert _status() == 0
    ref, ref_lse = O.attention_mode_b(qf, kf, vf, d ** -0.5, True, g)
    o = out.cpu().numpy()
    assert cos(o, ref) >= 0.9995, cos(o, ref)
    assert np.abs(o - ref).max() <= MAXABS
    assert np.abs(lse.cpu().numpy().reshape(ref_lse.shape) - ref_lse).max() <= 2e-3


@pytest.mark.parametrize("sq,skv", [(1, 300), (100, 300), (130, 129), (64, 1029)])
def test_cross_attention_noncausal(sq, skv):
    z, h, hk, d = 2, 4, 2, 128
    q, qf = seeded_bf16((z, h, sq, d), sq)
    k, kf = seeded_bf16((z, hk, skv, d), skv)
    v, vf = seeded_bf16((z, hk, skv, d), skv + 1)
    out = _n().nvfp4_flash_attention(q.float(), k.float(), v.float(), d ** -0.5, causal=False,
                                     num_key_value_groups=2)
    assert _status() == 0
    ref, _ = O.attention_mode_b(qf, kf, vf, d ** -0.5, False, 2)
    o = out.cpu().numpy()
    assert cos(o, ref) >= 0.9995 and np.abs(o - ref).max() <= MAXABS


def test_causal_bottom_right_alignment():
    z, h, d, sq, skv = 1, 2, 128, 70, 333
    q, qf = seeded_bf16((z, h, sq, d), 1)
    k, kf = seeded_bf16((z, h, skv, d), 2)
    v, vf = seeded_bf16((z, h, skv, d), 3)
    out = _n().nvfp4_flash_attention(q.float(), k.float(), v.float(), d ** -0.5, causal=True)
    ref, _ = O.attention_mode_b(qf, kf, vf, d ** -0.5, True, 1)
    assert _status() == 0
    assert np.abs(out.cpu().numpy() - ref).max() <= MAXABS


def test_varlen_matches_oracle_and_per_sample_runs():
    d, h, hk = 128, 4, 2
    lens = [1, 255, 17, 128, 300, 64]
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    s = int(cu[-1])
    q, qf = seeded_bf16((1, h, s, d), 41)
    k, kf = seeded_bf16((1, hk, s, d), 42)
    v, vf = seeded_bf16((1, hk, s, d), 43)
    n = _n()
    out = n.nvfp4_flash_attention(q.float(), k.float(), v.float(), d ** -0.5, causal=True,
                                  num_key_value_groups=2, cu_seqlens=torch.from_numpy(cu).cuda())
    assert _status() == 0
    ref, _ = O.attention_mode_b(qf, kf, vf, d ** -0.5, True, 2, cu_seqlens=cu)
    o = out.cpu().numpy()
    assert cos(o, ref) >= 0.9995 and np.abs(o - ref).max() <= MAXABS
    # no leakage across samples: perturbing one sample leaves the others' outputs bit-unchanged
    # (reference test: tests/test_nvfp4_train_forward.py:367-404)
    k2 = k.clone()
    k2[:, :, cu[2]:cu[3]] += 1.0
    out2 = n.nvfp4_flash_attention(q.float(), k2.float(), v.float(), d ** -0.5, causal=True,
                                   num_key_value_groups=2, cu_seqlens=torch.from_numpy(cu).cuda())
    keep = torch.ones(s, dtype=torch.bool)
    keep[cu[2]:cu[3]] = False
    assert torch.equal(out[:, :, keep], out2[:, :, keep])


def test_varlen_single_sample_equals_dense_bitwise():
    """tests/test_nvfp4_attention.py:375-420 of the reference."""
    d, h, s = 128, 2, 300
    q, _ = seeded_bf16((1, h, s, d), 51)
    k, _ = seeded_bf16((1, h, s, d), 52)
    v, _ = seeded_bf16((1, h, s, d), 53)
    n = _n()
    a = n.nvfp4_flash_attention(q, k, v, d ** -0.5, causal=True)
    b = n.nvfp4_flash_attention(q, k, v, d ** -0.5, causal=True,
                                cu_seqlens=torch.tensor([0, s], dtype=torch.int32, device="cuda"))
    assert _status() == 0
    assert torch.equal(a, b)


def test_zshd_equals_zhsd_transposed_and_determinism():
    """tests/test_nvfp4_attention.py:131-159 and test_nvfp4_train_forward.py:250-284."""
    z, h, hk, s, d = 2, 4, 2, 200, 128
    q, _ = seeded_bf16((z, h, s, d), 61)
    k, _ = seeded_bf16((z, hk, s, d), 62)
    v, _ = seeded_bf16((z, hk, s, d), 63)
    n = _n()
    a = n.nvfp4_flash_attention(q, k, v, d ** -0.5, causal=True, num_key_value_groups=2)
    b = n.nvfp4_flash_attention(q, k, v, d ** -0.5, causal=True, num_key_value_groups=2,
                                out_layout="zshd")
    c = n.nvfp4_flash_attention(q, k, v, d ** -0.5, causal=True, num_key_value_groups=2)
    assert _status() == 0
    assert b.shape == (z, s, h, d) and torch.equal(a, b.transpose(1, 2)) and torch.equal(a, c)


def test_prepacked_equals_in_kernel_quant():
    """tests/test_nvfp4_attention.py:423-555: packed entry and external q/k packs are bit-identical."""
    z, h, hk, s, d = 1, 4, 2, 160, 128
    q, _ = seeded_bf16((z, h, s, d), 71)
    k, _ = seeded_bf16((z, hk, s, d), 72)
    v, _ = seeded_bf16((z, hk, s, d), 73)
    n = _n()
    out, packs = n.nvfp4_flash_attention(q, k, v, d ** -0.5, causal=True, num_key_value_groups=2,
                                         return_packs=True)
    qnv, qsc, knv, ksc, vnv, vsc = packs
    out2 = n.nvfp4_flash_attention_packed(qnv, qsc, knv, ksc, vnv, vsc, z, h, hk, s, s, d, d ** -0.5,
                                          q.dtype, causal=True)
    out3 = n.nvfp4_flash_attention(q, k, v, d ** -0.5, causal=True, num_key_value_groups=2,
                                   q_packs=(qnv, qsc), k_packs=(knv, ksc))
    assert _status() == 0
    assert torch.equal(out, out2) and torch.equal(out, out3)
    with pytest.raises(AssertionError, match="q_packs layout"):
        n.nvfp4_flash_attention(q, k, v, d ** -0.5, q_packs=(knv, ksc), num_key_value_groups=2)
    with pytest.raises(ValueError):
        n.nvfp4_flash_attention(q, k, v, d ** -0.5, out_layout="hzsd", num_key_value_groups=2)


def test_forward_vs_bf16_sdpa_floor():
    """Reference floor (tests/test_nvfp4_attention.py:72): cosine vs bf16 SDPA >= 0.95."""
    z, h, hk, s, d = 1, 8, 2, 2048, 128
    q, _ = seeded_bf16((z, h, s, d), 81)
    k, _ = seeded_bf16((z, hk, s, d), 82)
    v, _ = seeded_bf16((z, hk, s, d), 83)
    out = _n().nvfp4_flash_attention(q, k, v, d ** -0.5, causal=True, num_key_value_groups=4)
    ref = torch.nn.functional.scaled_dot_product_attention(
        q.float(), k.float().repeat_interleave(4, 1), v.float().repeat_interleave(4, 1), is_causal=True)
    assert _status() == 0
    c = cos(out.float().cpu().numpy(), ref.cpu().numpy())
    print("fwd vs fp32 SDPA cosine", c)
    assert c > 0.95


def test_full_size_properties_c2_shape():
    """BASELINE config 2 for one batch element (H32 Hk8 S8192 D128 causal, outlier K channels):
    size-independent properties -- finite, deterministic, rows are convex combinations of V
    (|o| <= max|v_deq|), the first row equals dequantised V[0]."""
    z, h, hk, s, d = 1, 32, 8, 8192, 128
    gen = torch.Generator().manual_seed(2)
    q = torch.randn(z, h, s, d, generator=gen).to(torch.bfloat16).cuda()
    k = torch.randn(z, hk, s, d, generator=gen)
    ch = torch.randperm(d, generator=gen)[:8]
    k[..., ch] += torch.randn(8, generator=gen) * 2.0
    k = k.to(torch.bfloat16).cuda()
    v = torch.randn(z, hk, s, d, generator=gen).to(torch.bfloat16).cuda()
    n = _n()
    a = n.nvfp4_flash_attention(q, k, v, d ** -0.5, causal=True, num_key_value_groups=4)
    b = n.nvfp4_flash_attention(q, k, v, d ** -0.5, causal=True, num_key_value_groups=4)
    assert _status() == 0
    assert torch.isfinite(a).all() and torch.equal(a, b)
    assert float(a.float().abs().max()) <= float(v.float().abs().max()) * 1.07 + 1e-3
    ref = torch.nn.functional.scaled_dot_product_attention(
        q[:, :8].float(), k[:, :2].float().repeat_interleave(4, 1),
        v[:, :2].float().repeat_interleave(4, 1), is_causal=True)
    c = cos(a[:, :8].float().cpu().numpy(), ref.cpu().numpy())
    print("C2-shape cosine vs fp32 SDPA (first 8 heads)", c)
    assert c > 0.95
