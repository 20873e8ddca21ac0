"""V projection with the NVFP4 pack as its epilogue: the projected values match a plain fp32
reference of the same product, the packed bytes equal the packer run on those values, and the
packs feed the packed attention entry with the unfused path's bits."""

import pytest
import torch

from gpu_util import seeded_bf16

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("z,s,hidden,hk,d,use_bias", [(2, 300, 512, 2, 128, True), (1, 128, 64, 1, 128, False),
                                                      (1, 1000, 1032, 3, 64, True), (2, 77, 256, 1, 256, False)])
def test_vproj_pack_matches_projection_then_pack(dtype, z, s, hidden, hk, d, use_bias):
    import sageattention_b200.nvfp4 as nv
    from sageattention_b200 import _lib
    g = torch.Generator().manual_seed(z * 100 + s)
    x = (torch.randn(z, s, hidden, generator=g) * 0.5).to(dtype).cuda()
    w = (torch.randn(hk * d, hidden, generator=g) * hidden ** -0.5).to(dtype).cuda()
    b = (torch.randn(hk * d, generator=g) * 0.1).to(dtype).cuda() if use_bias else None
    vnv, vsc, v = nv.vproj_quant_nvfp4(x, w, b, hk, d)
    torch.cuda.synchronize()
    assert _lib.read_status("cuda") == 0
    sp = ((s + 127) // 128) * 128
    assert v.shape == (z, hk, s, d) and vnv.shape == (z * hk, d, sp // 2) and vsc.shape == (z * hk, d, sp // 16)
    # the projection itself: fp32 reference of the same op, rounded once
    ref = torch.nn.functional.linear(x.float(), w.float(), b.float() if b is not None else None)
    ref = ref.view(z, s, hk, d).permute(0, 2, 1, 3)
    err = (v.float() - ref).abs().max().item()
    tol = 2.0 ** (-8 if dtype == torch.bfloat16 else -11) * max(1.0, ref.abs().max().item()) * 1.01
    assert err <= tol, (err, tol)
    # the epilogue pack: bytes of the packer on the very values the kernel stored
    n2, s2 = nv._quant_nvfp4(v.reshape(z * hk, s, d), transpose=True, k_pad=sp)
    assert torch.equal(vnv, n2) and torch.equal(vsc.view(torch.uint8), s2.view(torch.uint8))
    # without the value output, and with another padding, the packs keep their bytes
    vnv2, vsc2, none = nv.vproj_quant_nvfp4(x, w, b, hk, d, s_pad=((s + 15) // 16) * 16, return_value=False)
    assert none is None
    k16 = ((s + 15) // 16) * 16
    assert torch.equal(vnv2, vnv[:, :, : k16 // 2]) and torch.equal(vsc2.view(torch.uint8), vsc.view(torch.uint8)[:, :, : k16 // 16])


def test_vproj_packs_feed_packed_attention():
    import sageattention_b200.nvfp4 as nv
    z, h, hk, s, d, hidden = 1, 4, 2, 384, 128, 256
    q, _ = seeded_bf16((z, h, s, d), 921)
    k, _ = seeded_bf16((z, hk, s, d), 922)
    x, _ = seeded_bf16((z, s, hidden), 923)
    w, _ = seeded_bf16((hk * d, hidden), 924)
    w = (w * hidden ** -0.5).to(torch.bfloat16)
    vnv, vsc, v = nv.vproj_quant_nvfp4(x, w, None, hk, d)
    qnv, qsc = nv._quant_nvfp4(q.reshape(z * h, s, d))
    knv, ksc = nv._quant_nvfp4(k.reshape(z * hk, s, d))
    fused = nv.nvfp4_flash_attention_packed(qnv, qsc, knv, ksc, vnv, vsc, z, h, hk, s, s, d, d ** -0.5,
                                            torch.bfloat16, causal=True)
    plain = nv.nvfp4_flash_attention(q, k, v, d ** -0.5, causal=True, num_key_value_groups=h // hk)
    assert torch.equal(fused, plain)
