"""Rotary embedding fused into the packer: bytes equal pack(rope(x)) of the CPU restatement, and the
packs drop into the attention entry points as `q_packs` / `k_packs`."""

import numpy as np
import pytest
import torch

from gpu_util import np_u8, seeded_bf16
from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu


def _tables(p, d, base=10000.0):
    inv = 1.0 / (base ** (np.arange(0, d, 2, dtype=np.float64) / d))
    ang = np.arange(p, dtype=np.float64)[:, None] * inv[None, :]
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


@pytest.mark.parametrize("b,r,d,pos0", [(3, 200, 128, 0), (2, 77, 256, 1000), (1, 1, 64, 5)])
def test_rope_pack_bytes_match_cpu_restatement(b, r, d, pos0):
    import sageattention_b200.nvfp4 as nv
    x, xf = seeded_bf16((b, r, d), 900 + d)
    cos, sin = _tables(pos0 + r + 3, d)
    nib, sc = nv.rope_quant_nvfp4(x, torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda(), pos0=pos0)
    y = O.rope_half_split(xf, cos, sin, pos0=pos0)
    rn, rs = O.pack(y)
    bad = (np_u8(nib) != rn).mean() + (np_u8(sc) != rs).mean()
    assert bad <= 1e-4, bad      # fp64 emulation of the kernel's fma: ties may differ once in a while
    # explicit positions give the same bytes
    pos = torch.arange(pos0, pos0 + r, dtype=torch.int32)
    nib2, sc2 = nv.rope_quant_nvfp4(x, torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda(), positions=pos)
    assert torch.equal(nib, nib2) and torch.equal(sc.view(torch.uint8), sc2.view(torch.uint8))
    # and equal the unfused product path: rotate in fp32 on the GPU, round to bf16, pack
    h = d // 2
    c = torch.from_numpy(cos[pos0:pos0 + r]).cuda()
    s_ = torch.from_numpy(sin[pos0:pos0 + r]).cuda()
    xf32 = x.float()
    lo, hi = xf32[..., :h], xf32[..., h:]
    y_gpu = torch.cat([torch.addcmul(lo * c, -hi, s_), torch.addcmul(hi * c, lo, s_)], dim=-1).to(torch.bfloat16)
    nib3, sc3 = nv._quant_nvfp4(y_gpu)
    assert (nib3 != nib).float().mean().item() <= 1e-3


def test_rope_packs_feed_attention():
    import sageattention_b200.nvfp4 as nv
    z, h, hk, s, d = 1, 4, 2, 384, 128
    q, _ = seeded_bf16((z, h, s, d), 911)
    k, _ = seeded_bf16((z, hk, s, d), 912)
    v, _ = seeded_bf16((z, hk, s, d), 913)
    cos, sin = _tables(s, d)
    c, s_ = torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda()
    qp = nv.rope_quant_nvfp4(q.reshape(z * h, s, d), c, s_)
    kp = nv.rope_quant_nvfp4(k.reshape(z * hk, s, d), c, s_)
    out = nv.nvfp4_flash_attention(q, k, v, d ** -0.5, causal=True, num_key_value_groups=2, q_packs=qp, k_packs=kp)

    def rope(x):
        xf = x.float()
        lo, hi = xf[..., :d // 2], xf[..., d // 2:]
        return torch.cat([lo * c - hi * s_, hi * c + lo * s_], dim=-1).to(torch.bfloat16)

    ref = nv.nvfp4_flash_attention(rope(q), rope(k), v, d ** -0.5, causal=True, num_key_value_groups=2)
    cosv = torch.nn.functional.cosine_similarity(out.float().flatten(), ref.float().flatten(), dim=0).item()
    assert cosv >= 0.9999, cosv
