"""The allocation-free decode entry point (`nvfp4_decode_static`) against `nvfp4_decode`.

Some callers of this library own all device memory themselves and may not allocate when a request
arrives (a server with a fixed memory plan, a plugin that must not touch its host's allocator).
`nvfp4_decode_static` keeps the split-K partials in a fixed 16 MiB array inside the library
instead of a caller-provided workspace.  This test drives both entry points through the C ABI on
the same inputs, twice in a row (the array is shared and keeps the previous call's contents), and
requires identical outputs.  It is collected last on purpose.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(static, q, packed, z, hk, g, d, s_kv, scaling, nsplit, split_kv):
    from sageattention_b200 import _lib
    L = _lib.lib()
    knv, ksc, vnv, vsc = packed[:4]
    h = hk * g
    out = torch.empty(z, h, d, dtype=q.dtype, device=q.device)
    lse = torch.empty(z, h, dtype=torch.float32, device=q.device)
    common = (q.data_ptr(), _lib.dtype_code(q.dtype), q.stride(0), q.stride(1),
              knv.data_ptr(), knv.stride(0), ksc.data_ptr(), ksc.stride(0),
              vnv.data_ptr(), vnv.stride(0), vnv.stride(1), vsc.data_ptr(), vsc.stride(0), vsc.stride(1),
              z, hk, g, d, s_kv, float(scaling), out.data_ptr(), lse.data_ptr())
    tail = (nsplit, split_kv, _lib.status_word(q.device).data_ptr(), _lib.stream_ptr(q.device))
    if static:
        rc = L.nvfp4_decode_static(*common, *tail)
        ws = None
    else:
        nbytes = z * hk * nsplit * (16 * d + 32) * 4
        ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
        rc = L.nvfp4_decode(*common, ws.data_ptr(), nbytes, *tail)
    _lib.check(rc, "decode")
    torch.cuda.synchronize()
    assert _lib.read_status(q.device) == 0
    return out, lse


def test_static_scratch_decode_matches_workspace_decode_twice():
    import sageattention_b200.nvfp4 as nv
    from sageattention_b200 import _lib
    z, hk, g, d = 2, 2, 4, 128
    gen = torch.Generator(device="cuda").manual_seed(0)
    for s_kv, split_kv in ((1500, 256), (777, 128)):          # two different calls in a row
        k = torch.randn(z, hk, s_kv, d, device="cuda", dtype=torch.bfloat16, generator=gen)
        v = torch.randn(z, hk, s_kv, d, device="cuda", dtype=torch.bfloat16, generator=gen)
        q = torch.randn(z, hk * g, d, device="cuda", dtype=torch.bfloat16, generator=gen)
        packed = nv.nvfp4_quant_kv_decode(k, v)
        nsplit = -(-s_kv // split_kv)
        ref_out, ref_lse = _call(False, q, packed, z, hk, g, d, s_kv, d ** -0.5, nsplit, split_kv)
        out, lse = _call(True, q, packed, z, hk, g, d, s_kv, d ** -0.5, nsplit, split_kv)
        assert torch.equal(out, ref_out) and torch.equal(lse, ref_lse)
        out2, lse2 = _call(True, q, packed, z, hk, g, d, s_kv, d ** -0.5, nsplit, split_kv)
        assert torch.equal(out2, ref_out) and torch.equal(lse2, ref_lse)
    # beyond the fixed capacity: a clear error, nothing launched
    cap = _lib.lib().nvfp4_decode_static_capacity()
    assert cap == 16 << 20
    L = _lib.lib()
    too_many = cap // ((16 * d + 32) * 4) // (z * hk) + 1
    with pytest.raises(RuntimeError, match="static"):
        _call(True, q, packed, z, hk, g, d, 128 * too_many, d ** -0.5, too_many, 128)
