"""Host side of the B200 NVFP4 flash-attention path.

Mirrors the operator surface of the reference module ``sageattention/nvfp4/flash.py`` (same
names, argument order, defaults and error behaviour) so callers and tests written against the
reference run unchanged; each function cites the reference lines it stands in for.  All compute
is in ``libnvfp4_b200.so`` (hand-written sm_100a CUDA behind the C ABI of
``include/nvfp4_b200.h``); torch is used for allocation, streams and autograd plumbing only.
There is no Triton and no CPU fallback: CPU tensors are rejected.

Tile arguments (``block_m``, ``block_n``, ``num_warps``, ``num_stages``) are accepted for
signature compatibility.  The sm_100a kernels always walk 128-key tiles (the reference's own
D=128 default), so ``block_n`` only has to be 128 where it fixes a visible padding
(``nvfp4_quant_kv_decode``); other tile hints are ignored.
"""

from __future__ import annotations

import ctypes
import functools
import os

import torch

from .. import _lib

# --------------------------------------------------------------------------- constants
# (names kept importable: tests and scripts of the reference read them, flash.py:260-273,
#  :993-1037)
_BWD_GRAD_DOTS_MODES = ("bf16", "fp4_rownorm", "fp8_rownorm", "fp4_legacy")
_BWD_AUTO_FP4_MIN_SEQ = 4096
_BWD_RN_DO_ZSHD = True
_FWD_TILE = {256: (128, 128, 8, 2), 128: (128, 128, 8, 2)}
_FWD_TILE_DEFAULT = (64, 128, 8, 3)
_FWD_TILE_VARLEN = {256: (128, 128, 8, 2), 128: (128, 128, 8, 2)}
_FWD_FUSED_QUANT_MAX_SEQ = 3072
_FWD_VARLEN_DENSE_MIN_MEAN = 4096
_KEY_TILE = 128


def _next_mult(n: int, m: int) -> int:
    return ((n + m - 1) // m) * m


def _resolve_fwd_tiles(d, block_m, block_n, num_warps, num_stages, varlen=False, mean_len=None):
    """Tile policy hook of the reference (flash.py:1040-1056).

    Explicit tiles are echoed back, generic defaults resolve to the one tile shape the sm_100a
    forward kernel implements (128 query rows x 128 keys).
    """
    if (block_m, block_n, num_warps, num_stages) == _FWD_TILE_DEFAULT:
        return (_FWD_TILE_VARLEN if varlen else _FWD_TILE).get(d, _FWD_TILE_DEFAULT)
    return block_m, block_n, num_warps, num_stages


def _resolve_backward_grad_dots(mode, eff_seq, save_backward_packs, num_key_value_groups) -> str:
    """Backward-mode resolver, same table as the reference (flash.py:276-302).

    ``None`` = AUTO: "bf16" (high-precision gradient GEMMs) below ``_BWD_AUTO_FP4_MIN_SEQ``
    effective sequence, else "fp4_rownorm"; "bf16" silently downgrades to "fp4_rownorm" when only
    packs are saved or the GQA group exceeds 8.
    """
    if mode is None:
        mode = "bf16" if eff_seq < _BWD_AUTO_FP4_MIN_SEQ else "fp4_rownorm"
    if mode not in _BWD_GRAD_DOTS_MODES:
        raise ValueError(
            f"backward_grad_dots must be one of {_BWD_GRAD_DOTS_MODES} or None (auto), got {mode!r}")
    if mode == "bf16" and (save_backward_packs or num_key_value_groups > 8):
        mode = "fp4_rownorm"
    return mode


# --------------------------------------------------------------------------- packer
def _pack_into(x, nib, sc, transpose=False, k_pad=None):
    """Pack ``x`` ([B,R,K], or [B,K,R] with ``transpose``) into existing (possibly strided) views.

    ``nib`` [B,R,Kp/2] uint8 and ``sc`` [B,R,Kp/16] (uint8 or float8_e4m3fn) must have unit
    stride along their last axis; this is how the KV cache packs straight into its buffers.
    """
    _lib.require_cuda(x, "x")
    if transpose:
        b, k_read, r = x.shape
        sxb, sxk, sxr = x.stride()
    else:
        b, r, k_read = x.shape
        sxb, sxr, sxk = x.stride()
    kp = k_read if k_pad is None else int(k_pad)
    assert kp % 16 == 0, "padded contraction dim must be a multiple of 16"
    assert kp >= k_read, "k_pad must cover the contraction axis"
    assert nib.shape == (b, r, kp // 2) and sc.shape == (b, r, kp // 16), "output view shape mismatch"
    assert nib.stride(2) == 1 and sc.stride(2) == 1
    if b * r * kp == 0:
        return
    _lib.call("nvfp4_pack", _lib.same_device(x, nib, sc),
              x.data_ptr(), _lib.dtype_code(x.dtype), b, r, k_read, kp, sxb, sxr, sxk,
              nib.data_ptr(), nib.stride(0), nib.stride(1), sc.data_ptr(), sc.stride(0), sc.stride(1),
              _lib.stream_ptr(x.device))


def _quant_nvfp4(x: torch.Tensor, transpose: bool = False, k_pad: int | None = None):
    """NVFP4-pack along the contraction axis; stands in for flash.py:363-419.

    ``x`` is ``[B, R, K]`` (quantised along K) or, with ``transpose=True``, ``[B, K, R]`` read
    through its strides to produce the V^T layout.  ``k_pad`` zero-pads the contraction axis
    (padded groups get the floor scale and zero nibbles).  Returns
    ``(uint8 [B, R, Kp/2], float8_e4m3fn [B, R, Kp/16])``.
    """
    if transpose:
        b, k_read, r = x.shape
    else:
        b, r, k_read = x.shape
    kp = k_read if k_pad is None else int(k_pad)
    assert kp % 16 == 0, "padded contraction dim must be a multiple of 16"
    nib = torch.empty(b, r, kp // 2, dtype=torch.uint8, device=x.device)
    sc = torch.empty(b, r, kp // 16, dtype=torch.uint8, device=x.device)
    _pack_into(x, nib, sc, transpose=transpose, k_pad=kp)
    return nib, sc.view(torch.float8_e4m3fn)


def rope_quant_nvfp4(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions=None, pos0: int = 0):
    """Rotary embedding fused into the NVFP4 packer (the producer the reference asks callers to
    fuse before `q_packs` / `k_packs`, flash.py:10-13, 2812-2821).

    ``x`` ``[B, R, D]`` (row r at position ``positions[r]`` or ``pos0 + r``), ``cos`` / ``sin``
    ``[P, D/2]`` fp32, half-split ("rotate_half") convention.  The rotated values are rounded once to
    ``x.dtype`` and packed along D: bit-identical to ``_quant_nvfp4(rope(x).to(x.dtype))`` with the
    rotation in fp32, without writing the rotated tensor.  Returns ``(uint8 [B,R,D/2],
    float8_e4m3fn [B,R,D/16])``, directly usable as ``q_packs`` / ``k_packs``.
    """
    _lib.require_cuda(x, "x")
    b, r, d = x.shape
    assert x.stride(2) == 1, "rows must be contiguous along D"
    assert cos.shape[-1] == d // 2 and sin.shape == cos.shape and cos.dtype == torch.float32
    cos, sin = cos.contiguous(), sin.contiguous()
    if positions is not None:
        positions = positions.to(device=x.device, dtype=torch.int32).contiguous()
        assert positions.numel() == r
    nib = torch.empty(b, r, d // 2, dtype=torch.uint8, device=x.device)
    sc = torch.empty(b, r, d // 16, dtype=torch.uint8, device=x.device)
    _lib.call("nvfp4_rope_pack", _lib.same_device(x, cos, sin, positions),
              x.data_ptr(), _lib.dtype_code(x.dtype), b, r, d, x.stride(0), x.stride(1), cos.data_ptr(), sin.data_ptr(),
              positions.data_ptr() if positions is not None else None, int(pos0), nib.data_ptr(), nib.stride(0),
              nib.stride(1), sc.data_ptr(), sc.stride(0), sc.stride(1), _lib.stream_ptr(x.device))
    return nib, sc.view(torch.float8_e4m3fn)


def _quant_mxfp8_t(x: torch.Tensor, s_pad: int, _prescale_amax: torch.Tensor | None = None):
    """MXFP8 pack of ``x`` [B, S, D] along S: e4m3 bytes [B, D, s_pad] and e8m0 scale bytes
    [B, D, s_pad/32] (one power-of-two scale per 32 tokens); stands in for ``_pack_mxfp8_along_k`` of
    the transposed operand (flash.py:243-257, 1255-1394).  The gradient operands dO^T, Q^T, K^T of the
    ``fp8_rownorm`` backward."""
    _lib.require_cuda(x, "x")
    b, s, d = x.shape
    assert s_pad % 32 == 0 and s_pad >= s, "s_pad must be a multiple of 32 covering S"
    if x.stride(2) != 1:
        x = x.contiguous()
    out = torch.empty(b, d, s_pad, dtype=torch.uint8, device=x.device)
    sc = torch.empty(b, d, s_pad // 32, dtype=torch.uint8, device=x.device)
    if b * s_pad > 0:
        _lib.call("nvfp4_pack_mx8_t", x.device, x.data_ptr(), _lib.dtype_code(x.dtype), b, s, d, s_pad, x.stride(0),
                  x.stride(1), _prescale_amax.data_ptr() if _prescale_amax is not None else None, out.data_ptr(),
                  sc.data_ptr(), _lib.stream_ptr(x.device))
    return out, sc


def vproj_quant_nvfp4(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, num_kv_heads: int,
                      head_dim: int, s_pad: int | None = None, return_value: bool = True):
    """V projection with the NVFP4 pack as its epilogue (the producer the reference asks callers to
    fuse for V, flash.py:10-13, 2812-2821): ``V = x @ weight.T (+ bias)`` on the tensor cores, written
    directly as the V^T pack along the keys, so V is never re-read for quantisation.

    ``x`` ``[Z, S, hidden]`` and ``weight`` ``[Hk*D, hidden]`` in bf16 or fp16.  Returns ``(vnv uint8
    [Z*Hk, D, s_pad/2], vsc float8_e4m3fn [Z*Hk, D, s_pad/16], value)`` where ``value`` is the
    projected tensor as a ``[Z, Hk, S, D]`` view (``None`` with ``return_value=False``); the packs are
    bit-identical to ``_quant_nvfp4(value, transpose=True, k_pad=s_pad)`` and feed
    ``nvfp4_flash_attention_packed`` / ``nvfp4_flash_decode_prequant`` as they are.
    """
    _lib.require_cuda(x, "x")
    z, s, hidden = x.shape
    feats = num_kv_heads * head_dim
    assert weight.shape == (feats, hidden), "weight must be [Hk*D, hidden]"
    assert x.dtype in (torch.bfloat16, torch.float16) and weight.dtype == x.dtype, "operands must be bf16 or fp16"
    assert hidden % 8 == 0 and head_dim % 16 == 0
    if x.stride(2) != 1 or x.stride(0) % 8 or x.stride(1) % 8:
        x = x.contiguous()
    weight = weight.contiguous()
    if bias is not None:
        bias = bias.to(x.dtype).contiguous()
        assert bias.numel() == feats
    sp = _next_mult(s, _KEY_TILE) if s_pad is None else int(s_pad)
    assert sp % 16 == 0 and sp >= s, "s_pad must be a multiple of 16 covering S"
    dev = x.device
    vnv = torch.empty(z * num_kv_heads, head_dim, sp // 2, dtype=torch.uint8, device=dev)
    vsc = torch.empty(z * num_kv_heads, head_dim, sp // 16, dtype=torch.uint8, device=dev)
    v = torch.empty(z, s, num_kv_heads, head_dim, dtype=x.dtype, device=dev) if return_value else None
    _lib.call("nvfp4_vproj_pack", _lib.same_device(x, weight, bias),
              x.data_ptr(), weight.data_ptr(), bias.data_ptr() if bias is not None else None, _lib.dtype_code(x.dtype),
              z, s, hidden, num_kv_heads, head_dim, x.stride(0), x.stride(1), sp, vnv.data_ptr(), vsc.data_ptr(),
              v.data_ptr() if v is not None else None, v.stride(0) if v is not None else 0,
              v.stride(1) if v is not None else 0, _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev))
    return vnv, vsc.view(torch.float8_e4m3fn), (v.permute(0, 2, 1, 3) if v is not None else None)


def _quant_nvfp4_dual(x: torch.Tensor, s_pad: int | None = None, _prescale_amax: torch.Tensor | None = None,
                      _sr: tuple = (False, False), _seed: int = 0):
    """Both layouts of ``x`` [B, S, D] from one read: along D and along S (padded to ``s_pad``).

    Stands in for flash.py:514-561 (one kernel, one pass over ``x``); bytes equal two
    ``_quant_nvfp4`` calls.  Returns ``(nib_d, sc_d, nib_s, sc_s)``.  ``_prescale_amax`` (a device
    float holding max|x|) first divides ``x`` by the smallest power of two >= that value (the global
    normalisation of dO in the all-FP4 backward).  ``_sr`` = (along D, along S): round that pack's
    e2m1 codes stochastically from ``_seed`` (the dO packs of the ``fp4_legacy`` backward).
    """
    _lib.require_cuda(x, "x")
    b, s, d = x.shape
    sp = _next_mult(s, 16) if s_pad is None else int(s_pad)
    assert sp % 16 == 0 and sp >= s, "s_pad must be a multiple of 16 covering S"
    assert d % 16 == 0, "D must be a multiple of 16"
    if x.stride(2) != 1:
        x = x.contiguous()
    dev = x.device
    nd = torch.empty(b, s, d // 2, dtype=torch.uint8, device=dev)
    sd = torch.empty(b, s, d // 16, dtype=torch.uint8, device=dev)
    ns = torch.empty(b, d, sp // 2, dtype=torch.uint8, device=dev)
    ss = torch.empty(b, d, sp // 16, dtype=torch.uint8, device=dev)
    if b * sp > 0:
        _lib.call("nvfp4_pack_dual", dev, x.data_ptr(), _lib.dtype_code(x.dtype), b, s, d, sp, x.stride(0),
                  x.stride(1), _prescale_amax.data_ptr() if _prescale_amax is not None else None,
                  (1 if _sr[0] else 0) | (2 if _sr[1] else 0), int(_seed) & 0xFFFFFFFF, nd.data_ptr(), sd.data_ptr(), ns.data_ptr(), ss.data_ptr(), _lib.stream_ptr(dev))
    return nd, sd.view(torch.float8_e4m3fn), ns, ss.view(torch.float8_e4m3fn)


def _quant_qkv_fwd(q2, k2, v2, s_kv_pad):
    """Q, K along D and V along keys (padded to ``s_kv_pad``) in one launch; stands in for
    flash.py:682-732.  ``q2`` [ZH, Sq, D], ``k2`` / ``v2`` [ZHk, Skv, D].  Operands that are not
    unit-stride along D (or differ in dtype) fall back to one ``_quant_nvfp4`` launch each."""
    bq, s_q, d = q2.shape
    bk, s_kv, _ = k2.shape
    fused = (q2.dtype == k2.dtype == v2.dtype and q2.stride(2) == 1 and k2.stride(2) == 1 and v2.stride(2) == 1
             and v2.shape == k2.shape and d in (64, 128, 256) and s_kv_pad % 16 == 0 and bq * s_q * bk * s_kv > 0)
    if not fused:
        qnv, qsc = _quant_nvfp4(q2)
        knv, ksc = _quant_nvfp4(k2)
        vnv, vsc = _quant_nvfp4(v2, transpose=True, k_pad=s_kv_pad)
        return qnv, qsc, knv, ksc, vnv, vsc
    dev = _lib.same_device(q2, k2, v2)
    u8 = lambda *sh: torch.empty(*sh, dtype=torch.uint8, device=dev)
    qnv, qsc = u8(bq, s_q, d // 2), u8(bq, s_q, d // 16)
    knv, ksc = u8(bk, s_kv, d // 2), u8(bk, s_kv, d // 16)
    vnv, vsc = u8(bk, d, s_kv_pad // 2), u8(bk, d, s_kv_pad // 16)
    _lib.call("nvfp4_pack_qkv", dev, q2.data_ptr(), k2.data_ptr(), v2.data_ptr(), _lib.dtype_code(q2.dtype),
              bq, bk, s_q, s_kv, s_kv_pad, d, q2.stride(0), q2.stride(1), k2.stride(0), k2.stride(1),
              v2.stride(0), v2.stride(1), qnv.data_ptr(), qsc.data_ptr(), knv.data_ptr(), ksc.data_ptr(),
              vnv.data_ptr(), vsc.data_ptr(), _lib.stream_ptr(dev))
    f8 = torch.float8_e4m3fn
    return qnv, qsc.view(f8), knv, ksc.view(f8), vnv, vsc.view(f8)


def convert_fp32_to_fp4_packed(x_pairs):
    """Pairs of fp32 tensors -> one byte per pair (first in the low nibble), e2m1 RTNE.

    The reference exposes this as a Triton device function (_fp4_pack.py:15-56); here it is a
    host-callable helper over the same hardware convert: values are packed with unit scale.
    """
    lo, hi = x_pairs
    x = torch.stack([lo.float(), hi.float()], dim=-1).reshape(1, -1, 2)
    n = x.shape[1]
    # unit scale: pad every pair to a group whose amax is exactly 6 so the group scale is 1
    grp = torch.zeros(1, n, 16, dtype=torch.float32, device=x.device)
    grp[:, :, 0:2] = x.clamp(-6.0, 6.0)
    grp[:, :, 2] = 6.0
    nib, _ = _quant_nvfp4(grp)
    return nib[0, :, 0].reshape(lo.shape)


# --------------------------------------------------------------------------- varlen
def _varlen_seq_arrays(cu_seqlens: torch.Tensor, s: int, device):
    """``cu_seqlens`` [n+1] -> int32 ``[s]`` arrays (seq_id, seq_start, seq_end) on ``device``.

    Same contract and validation messages as flash.py:940-984, including the cache on the
    tensor keyed by (s, device, version) so one host copy serves every layer of a step.
    """
    assert cu_seqlens.ndim == 1 and cu_seqlens.numel() >= 2, (
        f"cu_seqlens must be a 1-D [nseq+1] tensor, got shape {tuple(cu_seqlens.shape)}")
    key = (int(s), str(device), cu_seqlens._version)
    cached = getattr(cu_seqlens, "_nvfp4_seq_arrays", None)
    if cached is not None and cached[0] == key:
        return cached[1]
    cu = cu_seqlens.detach().to("cpu", torch.int64)
    assert int(cu[0]) == 0, f"cu_seqlens[0] must be 0, got {int(cu[0])}"
    assert int(cu[-1]) == s, f"cu_seqlens[-1] ({int(cu[-1])}) must equal the packed seqlen ({s})"
    assert bool((cu[1:] >= cu[:-1]).all()), "cu_seqlens must be nondecreasing"
    lens = (cu[1:] - cu[:-1])
    ids = torch.repeat_interleave(torch.arange(lens.numel(), dtype=torch.int64), lens)
    seq_id = ids.to(torch.int32)
    seq_start = cu[ids].to(torch.int32)
    seq_end = cu[ids + 1].to(torch.int32)
    arrays = tuple(t.to(device).contiguous() for t in (seq_id, seq_start, seq_end))
    try:
        cu_seqlens._nvfp4_seq_arrays = (key, arrays)
    except (AttributeError, RuntimeError):
        pass
    return arrays


# --------------------------------------------------------------------------- decode
def nvfp4_quant_kv_decode(key: torch.Tensor, value: torch.Tensor, block_n: int = 128) -> tuple:
    """One-shot NVFP4 pack of a GQA KV cache (stands in for flash.py:3211-3241).

    ``key``/``value``: ``[Z, Hk, Skv, D]``.  Returns ``(knv, ksc, vnv, vsc, s_kv, s_kv_pad)`` with K
    packed along D and V packed along keys as V^T, the key axis padded to ``block_n``.
    """
    z, hk, s_kv, d = key.shape
    assert d % 16 == 0 and d in (128, 256)
    s_kv_pad = _next_mult(s_kv, block_n)
    knv, ksc = _quant_nvfp4(key.reshape(z * hk, s_kv, d))
    vnv, vsc = _quant_nvfp4(value.reshape(z * hk, s_kv, d), transpose=True, k_pad=s_kv_pad)
    return knv, ksc, vnv, vsc, s_kv, s_kv_pad


@functools.lru_cache(maxsize=64)
def _sm_count_cached(index: int) -> int:
    return torch.cuda.get_device_properties(index).multi_processor_count


def _sm_count(device) -> int:
    dev = device if isinstance(device, torch.device) else torch.device(device)
    return _sm_count_cached(torch.cuda.current_device() if dev.index is None else dev.index)


@functools.lru_cache(maxsize=4096)
def _decode_plan_cached(s_kv: int, zhk: int, d: int, sms: int):
    ns, sk, wb = ctypes.c_int(), ctypes.c_int64(), ctypes.c_size_t()
    _lib.check(_lib.lib().nvfp4_decode_plan(s_kv, zhk, d, sms, ctypes.byref(ns), ctypes.byref(sk), ctypes.byref(wb)),
               "nvfp4_decode_plan")   # host only
    return ns.value, sk.value, wb.value


def _decode_plan(s_kv: int, zhk: int, d: int, device):
    return _decode_plan_cached(int(s_kv), int(zhk), int(d), _sm_count(device))


def _decode_core(query, kv_packed, scaling, g, want_lse, split_kv=None, extra=None):
    """Shared body of the decode entry points: plan, allocate scratch, one C-ABI call.

    ``extra = (n_extra, fill)``: ``n_extra`` more split-K partials per (batch, kv-head) unit are
    reserved behind the kernel's own; ``fill(workspace, total_slots, extra_base)`` is called to
    enqueue whatever writes them (the high-precision window of hybrid decode) before the decode,
    whose combine then merges everything in one pass."""
    _lib.require_cuda(query, "query")
    z, h, s_q, d = query.shape
    assert s_q == 1, "nvfp4_flash_decode is for seqlen_q == 1 (decode)"
    assert d % 16 == 0 and d in (128, 256)
    knv, ksc, vnv, vsc, s_kv, s_kv_pad = kv_packed
    zhk = knv.shape[0]
    assert zhk % z == 0, "packed KV batch must be a multiple of Z"
    hk = zhk // z
    assert h % hk == 0 and h // hk == g, "G mismatch vs packed KV"
    assert g <= 16, f"GQA group {g} must be <= 16"
    assert s_kv >= 1, "decode needs at least one key"
    dev = query.device
    q3 = query.reshape(z, h, d)
    if q3.stride(2) != 1:
        q3 = q3.contiguous()
    slot_bytes = (16 * d + 32) * 4
    if split_kv is None:
        nsplit, split_kv, wbytes = _decode_plan(s_kv, zhk, d, dev)
    elif split_kv == 0:
        # balanced decomposition (every CTA streams an equal share of all key tiles), forced;
        # slots as in `decode_balanced_geometry` of the C library
        tiles = -(-s_kv // 128)
        total = zhk * tiles
        ctas = max(1, min(_sm_count(dev), total // 4 if total // 4 > 0 else 1))
        per = -(-total // ctas)
        nsplit, wbytes = 0, ctas * ((per + tiles - 2) // tiles + 1) * slot_bytes
    else:
        assert split_kv % 128 == 0
        nsplit = -(-s_kv // split_kv)
        wbytes = zhk * nsplit * slot_bytes
    own_slots = wbytes // slot_bytes
    n_extra = 0 if extra is None else int(extra[0])
    wbytes = (own_slots + zhk * n_extra) * slot_bytes
    ws = torch.empty(wbytes, dtype=torch.uint8, device=dev)
    if n_extra:
        extra[1](ws, own_slots + zhk * n_extra, own_slots)
    out = torch.empty(z, h, d, dtype=query.dtype, device=dev)
    lse = torch.empty(z, h, dtype=torch.float32, device=dev) if want_lse else None
    for t in (knv, ksc, vnv, vsc):
        assert t.stride(-1) == 1, "packed cache rows must be contiguous"
    assert knv.stride(1) == d // 2 and ksc.stride(1) == d // 16, "K rows must be dense"
    _lib.call("nvfp4_decode_hybrid", _lib.same_device(q3, knv, ksc, vnv, vsc),
              q3.data_ptr(), _lib.dtype_code(q3.dtype), q3.stride(0), q3.stride(1),
              knv.data_ptr(), knv.stride(0), ksc.data_ptr(), ksc.stride(0),
              vnv.data_ptr(), vnv.stride(0), vnv.stride(1), vsc.data_ptr(), vsc.stride(0), vsc.stride(1),
              z, hk, g, d, s_kv, float(scaling), out.data_ptr(),
              lse.data_ptr() if lse is not None else None, ws.data_ptr(), wbytes, nsplit, split_kv, n_extra,
              _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev))
    return out.reshape(z, h, 1, d), lse


def nvfp4_flash_decode_prequant(query, kv_packed, scaling, num_key_value_groups=1, block_n=128,
                                num_warps=4, num_stages=3, target_programs=256):
    """Decode one query token per head against a pre-packed NVFP4 cache (HBM-bound fast path).

    Stands in for flash.py:3296-3342.  ``query`` ``[Z, H, 1, D]``; ``kv_packed`` is the tuple from
    ``nvfp4_quant_kv_decode`` or ``NVFP4KVCache.get_packed()`` (strided views are read in place).
    The split count follows the device's SM count; ``target_programs`` is accepted and ignored.
    Returns ``[Z, H, 1, D]`` in ``query.dtype``.
    """
    assert block_n == 128, "the B200 decode kernel walks 128-key tiles"
    out, _ = _decode_core(query, kv_packed, scaling, num_key_value_groups, want_lse=False)
    return out


def _decode_prequant_with_lse(query, kv_packed, scaling, g, block_n=128, num_warps=4,
                              num_stages=3, target_programs=256):
    """Decode that also returns the per-head log-sum-exp (kv_cache.py:32-97): ``(out, lse[Z,H])``."""
    return _decode_core(query, kv_packed, scaling, g, want_lse=True)


def nvfp4_flash_decode(query, key, value, scaling, num_key_value_groups=1, block_n=128,
                       num_warps=4, num_stages=3, target_programs=256):
    """Convenience decode that packs K/V from high precision on every call (flash.py:3345-3400)."""
    z, h, s_q, d = query.shape
    _, hk, s_kv, _ = key.shape
    assert s_q == 1, "nvfp4_flash_decode is for seqlen_q == 1 (decode)"
    assert h % hk == 0 and h // hk == num_key_value_groups
    assert d % 16 == 0 and d in (128, 256)
    assert num_key_value_groups <= 16, f"GQA group {num_key_value_groups} must be <= 16"
    packed = nvfp4_quant_kv_decode(key, value, block_n)
    return nvfp4_flash_decode_prequant(query, packed, scaling, num_key_value_groups, block_n)


# --------------------------------------------------------------------------- forward
def _run_flash_packed(qnv, qsc, knv, ksc, vnv, vsc, z, h, hk, s_q, s_kv, d, scaling, out_dtype,
                      causal=False, key_pad_bias=None, cu_seqlens=None, block_m=64, block_n=128,
                      num_warps=8, num_stages=3, out_layout="zhsd", return_lse=False,
                      _varlen_arrays=None):
    """Launch the forward kernel over packed operands (stands in for flash.py:2560-2652)."""
    dev = qnv.device
    _lib.require_cuda(qnv, "qnv")
    if out_layout not in ("zhsd", "zshd"):
        raise ValueError(f"out_layout must be 'zhsd' or 'zshd', got {out_layout!r}")
    assert d in (128, 256), "D must be 128 or 256"
    s_pad = vnv.shape[-1] * 2
    assert s_pad % _KEY_TILE == 0 and s_pad >= s_kv, (
        f"V^T key axis ({s_pad}) must be padded to a multiple of the key tile ({_KEY_TILE})")
    seq_id = seq_start = None
    if cu_seqlens is not None or _varlen_arrays is not None:
        assert z == 1, "cu_seqlens varlen requires Z must be 1 (one packed row)"
        assert s_q == s_kv, "cu_seqlens varlen requires Sq == Skv"
        arrays = _varlen_arrays if _varlen_arrays is not None else _varlen_seq_arrays(cu_seqlens, s_q, dev)
        seq_id, seq_start = arrays[0], arrays[1]
    if out_layout == "zhsd":
        out = torch.empty(z, h, s_q, d, dtype=out_dtype, device=dev)
        so_z, so_h, so_s = out.stride(0), out.stride(1), out.stride(2)
    else:
        out = torch.empty(z, s_q, h, d, dtype=out_dtype, device=dev)
        so_z, so_s, so_h = out.stride(0), out.stride(1), out.stride(2)
    lse = torch.empty(z * h, s_q, dtype=torch.float32, device=dev) if return_lse else None
    bias = None
    if key_pad_bias is not None:
        bias = key_pad_bias.to(device=dev, dtype=torch.float32).contiguous()
        assert bias.shape == (z, s_kv), "key_pad_bias must be [Z, Skv]"
    tensors = [t.contiguous() for t in (qnv, qsc, knv, ksc, vnv, vsc)]
    _lib.call("nvfp4_fwd", _lib.same_device(*tensors, bias, seq_id, seq_start),
              *(t.data_ptr() for t in tensors),
              bias.data_ptr() if bias is not None else None,
              seq_id.data_ptr() if seq_id is not None else None,
              seq_start.data_ptr() if seq_start is not None else None,
              out.data_ptr(), _lib.dtype_code(out_dtype), so_z, so_h, so_s,
              lse.data_ptr() if lse is not None else None, z, h, hk, s_q, s_kv, s_pad, d, float(scaling),
              1 if causal else 0, _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev))
    return (out, lse) if return_lse else out


def nvfp4_flash_attention_packed(qnv, qsc, knv, ksc, vnv, vsc, z, h, hk, s_q, s_kv, d, scaling,
                                 out_dtype, causal=False, key_pad_bias=None, cu_seqlens=None,
                                 block_m=64, block_n=128, num_warps=8, num_stages=3,
                                 out_layout="zhsd", _varlen_arrays=None):
    """Forward over operands the caller already packed (stands in for flash.py:2655-2766)."""
    return _run_flash_packed(qnv, qsc, knv, ksc, vnv, vsc, z, h, hk, s_q, s_kv, d, scaling,
                             out_dtype, causal, key_pad_bias, cu_seqlens, block_m, block_n,
                             num_warps, num_stages, out_layout, False, _varlen_arrays)


def _check_packs(packs, rows_shape, name):
    nv, sc = packs
    assert nv.shape == rows_shape[:-1] + (rows_shape[-1] // 2,) and \
        sc.shape == rows_shape[:-1] + (rows_shape[-1] // 16,), (
            f"{name} layout mismatch: expected along-D packs for shape {rows_shape}")
    return nv, sc


def nvfp4_flash_attention(query, key, value, scaling, causal=False, num_key_value_groups=1,
                          key_pad_bias=None, cu_seqlens=None, block_m=64, block_n=128, num_warps=8,
                          num_stages=3, return_lse=False, return_packs=False, out_layout="zhsd",
                          q_packs=None, k_packs=None, _varlen_arrays=None):
    """NVFP4 flash-attention forward (no autograd); stands in for flash.py:2769-3015.

    ``query`` ``[Z, H, Sq, D]``, ``key``/``value`` ``[Z, Hk, Skv, D]`` (bf16 / fp16 / fp32),
    ``D`` in {128, 256}.  Q and K are packed along D, V along keys, then the block-scaled FP4
    kernel runs.  Causal masking is bottom-right aligned.  Return arity follows the two flags
    exactly as in the reference: ``out`` | ``(out, lse)`` | ``(out, packs)`` |
    ``(out, lse, packs)`` with ``packs = (qnv, qsc, knv, ksc, vnv, vsc)``.
    """
    if out_layout not in ("zhsd", "zshd"):
        raise ValueError(f"out_layout must be 'zhsd' or 'zshd', got {out_layout!r}")
    _lib.require_cuda(query, "query")
    z, h, s_q, d = query.shape
    _, hk, s_kv, _ = key.shape
    g = num_key_value_groups
    assert h == hk * g, "num_key_value_groups must equal H // Hk"
    assert d in (128, 256), "D must be 128 or 256"
    if causal and cu_seqlens is None:
        assert s_kv >= s_q, "causal attention requires Skv >= Sq (bottom-right aligned mask)"
    if cu_seqlens is not None:
        assert z == 1, "cu_seqlens varlen requires Z must be 1 (one packed row)"
        assert s_q == s_kv, "cu_seqlens varlen requires Sq == Skv"
        assert causal, "cu_seqlens varlen is block-diagonal causal: pass causal=True"
    s_pad = _next_mult(s_kv, _KEY_TILE)
    q2 = query.reshape(z * h, s_q, d)
    k2 = key.reshape(z * hk, s_kv, d)
    v2 = value.reshape(z * hk, s_kv, d) if value.dim() == 4 else value
    if q_packs is None and k_packs is None and v2.dim() == 3:
        qnv, qsc, knv, ksc, vnv, vsc = _quant_qkv_fwd(q2, k2, v2, s_pad)     # one launch
    else:
        if q_packs is not None:
            qnv, qsc = _check_packs(q_packs, (z * h, s_q, d), "q_packs layout")
        else:
            qnv, qsc = _quant_nvfp4(q2)
        if k_packs is not None:
            knv, ksc = _check_packs(k_packs, (z * hk, s_kv, d), "k_packs layout")
        else:
            knv, ksc = _quant_nvfp4(k2)
        vnv, vsc = _quant_nvfp4(v2, transpose=True, k_pad=s_pad)
    res = _run_flash_packed(qnv, qsc, knv, ksc, vnv, vsc, z, h, hk, s_q, s_kv, d, scaling,
                            query.dtype, causal, key_pad_bias, cu_seqlens, block_m, block_n,
                            num_warps, num_stages, out_layout, return_lse, _varlen_arrays)
    packs = (qnv, qsc, knv, ksc, vnv, vsc)
    if return_lse and return_packs:
        return res[0], res[1], packs
    if return_packs:
        return res, packs
    return res


# --------------------------------------------------------------------------- backward
def _bwd_prep(x, y=None, want_copy=False, want_amax=False):
    """C-ABI pre-pass on a ``[B1, B2, S, D]`` tensor with unit stride along D (any other strides):
    returns ``(xc [B1*B2, S, D] bf16 | None, delta [B1*B2, S] = rowsum(x*y) | None)``, and with
    ``want_amax`` a third element: a device float holding max|x|."""
    b1, b2, s, d = x.shape
    if x.stride(3) != 1:
        x = x.contiguous()
    dev = x.device
    xc = torch.empty(b1 * b2, s, d, dtype=torch.bfloat16, device=dev) if want_copy else None
    delta = torch.empty(b1 * b2, s, dtype=torch.float32, device=dev) if y is not None else None
    amax = torch.zeros(1, dtype=torch.float32, device=dev) if want_amax else None
    if y is not None:
        if y.dtype != x.dtype:
            y = y.to(x.dtype)
        if y.stride(3) != 1:
            y = y.contiguous()
    _lib.call("nvfp4_bwd_prep", _lib.same_device(x, y),
              x.data_ptr(), _lib.dtype_code(x.dtype), x.stride(0), x.stride(1), x.stride(2), b1, b2,
              y.data_ptr() if y is not None else None,
              y.stride(0) if y is not None else 0, y.stride(1) if y is not None else 0,
              y.stride(2) if y is not None else 0, s, d,
              xc.data_ptr() if xc is not None else None,
              delta.data_ptr() if delta is not None else None,
              amax.data_ptr() if amax is not None else None, _lib.stream_ptr(dev))
    if want_amax:
        return xc, delta, amax
    return xc, delta


def _as_bf16_rows(x):
    """``[B1, B2, S, D]`` -> contiguous bf16 ``[B1*B2, S, D]``; no copy when it already is one."""
    b1, b2, s, d = x.shape
    if x.dtype == torch.bfloat16 and x.is_contiguous():
        return x.view(b1 * b2, s, d)
    return _bwd_prep(x, want_copy=True)[0]


def _run_bwd_hp(q, k, v, out, lse, dout, scaling, causal, g, varlen_arrays=None, out_layout="zhsd",
                q_packs=None, k_packs=None, key_pad_bias=None):
    """High-precision-grad-dots backward (stands in for flash.py:3459-3805).

    ``q`` ``[Z,H,Sq,D]``, ``k``/``v`` ``[Z,Hk,Skv,D]`` (v may be a strided view), ``out``/``dout`` in
    ``out_layout``, ``lse`` ``[Z*H, Sq]``.  Returns ``(dq, dk, dv)`` shaped like q, k, v in
    ``dout.dtype``.  One pre-pass launch for delta (plus a bf16 copy per operand that is not already
    contiguous bf16), then the dK/dV kernel (GQA reduced in-kernel) and the dQ kernel.
    """
    z, h, s_q, d = q.shape
    _, hk, s_kv, _ = k.shape
    assert d in (128, 256), "D must be 128 or 256"
    dev = q.device
    if out_layout == "zshd":          # [Z, Sq, H, D] views as [Z, H, Sq, D] (strided)
        out = out.transpose(1, 2)
        dout = dout.transpose(1, 2)
    need_copy = not (dout.dtype == torch.bfloat16 and dout.is_contiguous())
    doc, delta = _bwd_prep(dout, y=out, want_copy=need_copy)
    if doc is None:
        doc = dout.view(z * h, s_q, d)
    qc, kc, vc = _as_bf16_rows(q), _as_bf16_rows(k), _as_bf16_rows(v)
    # packs handed in by the caller may be strided views (a slice of a fused producer's buffer):
    # the kernels' tensor maps assume dense [rows, D/2] / [rows, D/16] rows
    if q_packs is not None:
        qnv, qsc = (t.contiguous() for t in _check_packs(q_packs, (z * h, s_q, d), "q_packs layout"))
    else:
        qnv, qsc = _quant_nvfp4(q.reshape(z * h, s_q, d))
    if k_packs is not None:
        knv, ksc = (t.contiguous() for t in _check_packs(k_packs, (z * hk, s_kv, d), "k_packs layout"))
    else:
        knv, ksc = _quant_nvfp4(k.reshape(z * hk, s_kv, d))
    gdt = dout.dtype
    dq = torch.empty(z, h, s_q, d, dtype=gdt, device=dev)
    dk = torch.empty(z, hk, s_kv, d, dtype=gdt, device=dev)
    dv = torch.empty(z, hk, s_kv, d, dtype=gdt, device=dev)
    sst = sen = None
    if varlen_arrays is not None:
        _, sst, sen = varlen_arrays
    lse = lse.contiguous()
    bias = None
    if key_pad_bias is not None:
        bias = key_pad_bias.to(device=dev, dtype=torch.float32).contiguous()
        assert bias.shape == (z, s_kv), "key_pad_bias must be [Z, Skv]"
    _lib.call("nvfp4_bwd_hp", _lib.same_device(qnv, qsc, knv, ksc, qc, kc, vc, doc, lse, delta, bias, sst, sen),
              qnv.data_ptr(), qsc.data_ptr(), knv.data_ptr(), ksc.data_ptr(), qc.data_ptr(), kc.data_ptr(),
              vc.data_ptr(), doc.data_ptr(), lse.data_ptr(), delta.data_ptr(),
              bias.data_ptr() if bias is not None else None,
              sst.data_ptr() if sst is not None else None, sen.data_ptr() if sen is not None else None,
              dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), _lib.dtype_code(gdt), z, h, hk, s_q, s_kv, d,
              float(scaling), 1 if causal else 0, _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev))
    return dq, dk, dv


def _run_bwd(q, k, v, out, lse, dout, scaling, causal, g, varlen_arrays=None, out_layout="zhsd",
             mode="fp4_rownorm", q_packs=None, k_packs=None, key_pad_bias=None, sr=False, sr_p_dv=None,
             sr_dot_dv=None, sr_ds_dq=None, seed=None, qt_packs=None, kt_packs=None, vd_packs=None, **_unused):
    """Block-scaled backward for the ``fp4_rownorm`` / ``fp4_legacy`` / ``fp8_rownorm`` modes (stands
    in for flash.py:3811-4265): every GEMM of the backward is a block-scaled tensor-core product.

    Pre-pass (four small launches): delta = rowsum(dO o O) and max|dO|; dO / 2^e packed along D and
    along the tokens from one read; Q^T and K^T packed along the tokens; V packed along D.  Then the
    dK/dV kernel (GQA reduced in tensor memory) and the dQ kernel.  In ``fp8_rownorm`` the operands
    of the three gradient GEMMs (dO^T, Q^T, K^T from the pre-pass; P^T, dS^T, dS packed in the
    kernels) are MXFP8 -- e4m3 with an e8m0 scale per 32 -- while S and dP stay NVFP4 products.

    Stochastic rounding (flash.py:3897-3915): only ``fp4_legacy`` honours the knobs; ``sr`` rounds
    the dO pack along D and the dS^T pack stochastically, ``sr_p_dv`` / ``sr_dot_dv`` / ``sr_ds_dq``
    (default: ``sr``) the P^T pack, the dO^T pack and the dS pack of the dQ kernel.  ``seed`` is drawn
    on the host when not given.

    ``qt_packs`` / ``kt_packs`` / ``vd_packs``: the transposed packs of Q and K (padded to 128
    tokens) and the along-D pack of V saved by the forward under ``save_backward_packs``; given,
    the pre-pass skips those launches (and the re-read of Q, K and V).
    """
    fp8 = mode == "fp8_rownorm"
    z, h, s_q, d = q.shape
    _, hk, s_kv, _ = k.shape
    assert d in (128, 256), "D must be 128 or 256"
    dev = q.device
    if out_layout == "zshd":          # [Z, Sq, H, D] views as [Z, H, Sq, D] (strided)
        out = out.transpose(1, 2)
        dout = dout.transpose(1, 2)
    if mode != "fp4_legacy":         # the normalised modes round to nearest only
        sr = sr_p_dv = sr_dot_dv = sr_ds_dq = False
    sr = bool(sr)
    sr_p_dv = sr if sr_p_dv is None else bool(sr_p_dv)
    sr_dot_dv = sr if sr_dot_dv is None else bool(sr_dot_dv)
    sr_ds_dq = sr if sr_ds_dq is None else bool(sr_ds_dq)
    any_sr = sr or sr_p_dv or sr_dot_dv or sr_ds_dq
    if seed is None:
        seed = int(torch.randint(0, 2 ** 31 - 1, (1,), device="cpu").item()) if any_sr else 0
    _, delta, amax = _bwd_prep(dout, y=out, want_amax=True)       # strided reads: no copy for the pre-pass
    # the dual pack wants one batch stride: a [Z,S,H,D] gradient viewed per head has two (Z > 1)
    do3 = dout.reshape(z * h, s_q, d) if (dout.is_contiguous() or z == 1) else dout.contiguous().view(z * h, s_q, d)
    sq_pad, skv_pad = _next_mult(s_q, _KEY_TILE), _next_mult(s_kv, _KEY_TILE)
    donv, dosc, dotnv, dotsc = _quant_nvfp4_dual(do3, sq_pad, _prescale_amax=amax, _sr=(sr, sr_dot_dv), _seed=seed)
    q3, k3, v3 = q.reshape(z * h, s_q, d), k.reshape(z * hk, s_kv, d), v.reshape(z * hk, s_kv, d)
    if fp8:
        assert qt_packs is None and kt_packs is None, (
            "fp8_rownorm repacks Q^T/K^T as MXFP8; incompatible with saved FP4 transposed packs")
        dotnv, dotsc = _quant_mxfp8_t(do3, sq_pad, _prescale_amax=amax)
        qnv, qsc = ((t.contiguous() for t in _check_packs(q_packs, (z * h, s_q, d), "q_packs layout"))
                    if q_packs is not None else _quant_nvfp4(q3))
        knv, ksc = ((t.contiguous() for t in _check_packs(k_packs, (z * hk, s_kv, d), "k_packs layout"))
                    if k_packs is not None else _quant_nvfp4(k3))
        qtnv, qtsc = _quant_mxfp8_t(q3, sq_pad)
        ktnv, ktsc = _quant_mxfp8_t(k3, skv_pad)
    elif q_packs is not None:
        qnv, qsc = (t.contiguous() for t in _check_packs(q_packs, (z * h, s_q, d), "q_packs layout"))
        qtnv, qtsc = qt_packs if qt_packs is not None else _quant_nvfp4(q3, transpose=True, k_pad=sq_pad)
    else:
        qnv, qsc, qtnv, qtsc = _quant_nvfp4_dual(q3, sq_pad)
    if fp8:
        pass
    elif k_packs is not None:
        knv, ksc = (t.contiguous() for t in _check_packs(k_packs, (z * hk, s_kv, d), "k_packs layout"))
        ktnv, ktsc = kt_packs if kt_packs is not None else _quant_nvfp4(k3, transpose=True, k_pad=skv_pad)
    else:
        knv, ksc, ktnv, ktsc = _quant_nvfp4_dual(k3, skv_pad)
    tb = 1 if fp8 else 2          # elements per byte of a transposed pack
    assert qtnv.shape == (z * h, d, sq_pad // tb) and ktnv.shape == (z * hk, d, skv_pad // tb), "transposed pack layout"
    vdnv, vdsc = vd_packs if vd_packs is not None else _quant_nvfp4(v3)
    gdt = dout.dtype
    dq = torch.empty(z, h, s_q, d, dtype=gdt, device=dev)
    dk = torch.empty(z, hk, s_kv, d, dtype=gdt, device=dev)
    dv = torch.empty(z, hk, s_kv, d, dtype=gdt, device=dev)
    sst = sen = None
    if varlen_arrays is not None:
        _, sst, sen = varlen_arrays
    lse = lse.contiguous()
    bias = None
    if key_pad_bias is not None:
        bias = key_pad_bias.to(device=dev, dtype=torch.float32).contiguous()
        assert bias.shape == (z, s_kv), "key_pad_bias must be [Z, Skv]"
    ptr = lambda t: t.data_ptr() if t is not None else None
    _lib.call("nvfp4_bwd_fp4", _lib.same_device(qnv, knv, vdnv, donv, dotnv, qtnv, ktnv, lse, delta, bias, sst, sen),
              ptr(qnv), ptr(qsc), ptr(knv), ptr(ksc), ptr(vdnv), ptr(vdsc), ptr(donv), ptr(dosc), ptr(dotnv),
              ptr(dotsc), ptr(qtnv), ptr(qtsc), ptr(ktnv), ptr(ktsc), ptr(lse), ptr(delta), ptr(amax), ptr(bias),
              ptr(sst), ptr(sen), ptr(dq), ptr(dk), ptr(dv), _lib.dtype_code(gdt), z, h, hk, s_q, s_kv, sq_pad,
              skv_pad, d, float(scaling), (1 if causal else 0) | (16 if sr else 0) | (32 if sr_p_dv else 0)
              | (64 if sr_ds_dq else 0) | (128 if fp8 else 0), (int(seed) * 2654435761 + 1) & 0xFFFFFFFF,
              _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev))
    return dq, dk, dv


def _gqa_reduce_cast_dkdv(dk_planes: torch.Tensor, dv_planes: torch.Tensor, z: int, hk: int, g: int,
                          out_dtype=None):
    """Sum per-query-head dK/dV planes ``[Z*H, S, D]`` over each GQA group -> ``[Z, Hk, S, D]``.

    Kept for API parity with flash.py:2525-2557; the B200 kernels reduce inside the dK/dV kernel
    and never materialise the planes."""
    zh, s, d = dk_planes.shape
    dt = out_dtype or dk_planes.dtype
    dk = dk_planes.reshape(z, hk, g, s, d).float().sum(dim=2).to(dt)
    dv = dv_planes.reshape(z, hk, g, s, d).float().sum(dim=2).to(dt)
    return dk, dv


class _NVFP4FlashAttn(torch.autograd.Function):
    """Autograd wrapper of the NVFP4 attention (stands in for flash.py:4268-4545).

    ``apply`` takes the reference's 26 positional arguments in the same order (query, key, value,
    scaling, causal, num_key_value_groups, key_pad_bias, sr, save_backward_packs, the three
    backward stochastic-rounding knobs, dkdv_scratch_bf16, backward_grad_dots (resolved mode),
    out_zshd, four tile hints, seq_id / seq_start / seq_end, and the optional Q / K packs) and
    returns gradients for the first three.
    """

    @staticmethod
    def forward(ctx, query, key, value, scaling, causal, num_key_value_groups, key_pad_bias, sr,
                save_backward_packs, backward_p_dv_sr, backward_dot_dv_sr, backward_ds_dq_sr,
                dkdv_scratch_bf16, backward_grad_dots, out_zshd, block_m, block_n, num_warps, num_stages,
                seq_id, seq_start, seq_end, qnv_in, qsc_in, knv_in, ksc_in):
        varlen = (seq_id, seq_start, seq_end) if seq_id is not None else None
        if varlen is not None:
            assert not save_backward_packs, "varlen (cu_seqlens) is incompatible with save_backward_packs"
        # direct callers of the Function may pass None (AUTO on s_kv) or a raw mode
        backward_grad_dots = _resolve_backward_grad_dots(backward_grad_dots, key.shape[2], save_backward_packs,
                                                         num_key_value_groups)
        if backward_grad_dots == "fp8_rownorm":
            assert not save_backward_packs, (
                "backward_grad_dots='fp8_rownorm' is incompatible with the saved forward FP4 "
                "transposed packs (save_backward_packs)")
        if qnv_in is not None or knv_in is not None:
            assert not save_backward_packs, (
                "q_packs/k_packs are incompatible with save_backward_packs "
                "(the saved pack set must come from the same fused HP read)")
        out_layout = "zshd" if out_zshd else "zhsd"
        q_in = (qnv_in, qsc_in) if qnv_in is not None else None
        k_in = (knv_in, ksc_in) if knv_in is not None else None
        extra = ()
        if save_backward_packs and backward_grad_dots in ("fp4_rownorm", "fp4_legacy"):
            # flash.py:4330-4385: everything the all-FP4 backward needs of Q, K and V is packed here,
            # from the one read of each operand (along D for the forward, transposed for the backward)
            z, h, s_q, d = query.shape
            hk, s_kv = key.shape[1], key.shape[2]
            qd = _quant_nvfp4_dual(query.reshape(z * h, s_q, d), _next_mult(s_q, _KEY_TILE))
            kd = _quant_nvfp4_dual(key.reshape(z * hk, s_kv, d), _next_mult(s_kv, _KEY_TILE))
            q_in, k_in = (qd[0], qd[1]), (kd[0], kd[1])
            extra = (qd[2], qd[3], kd[2], kd[3], *_quant_nvfp4(value.reshape(z * hk, s_kv, d)))
        out, lse, packs = nvfp4_flash_attention(
            query, key, value, scaling, causal=causal, num_key_value_groups=num_key_value_groups,
            key_pad_bias=key_pad_bias, return_lse=True, return_packs=True, out_layout=out_layout,
            q_packs=q_in, k_packs=k_in, _varlen_arrays=varlen)
        bias = key_pad_bias if key_pad_bias is not None else torch.empty(0, device=query.device)
        ctx.save_for_backward(query, key, value, out, lse, packs[0], packs[1], packs[2], packs[3], bias, *extra)
        ctx.meta = (float(scaling), bool(causal), int(num_key_value_groups), varlen, out_layout,
                    backward_grad_dots, key_pad_bias is not None,
                    (bool(sr), backward_p_dv_sr, backward_dot_dv_sr, backward_ds_dq_sr))
        return out

    @staticmethod
    def backward(ctx, grad_out):
        query, key, value, out, lse, qnv, qsc, knv, ksc, bias, *extra = ctx.saved_tensors
        scaling, causal, g, varlen, out_layout, mode, has_bias, srk = ctx.meta
        bias = bias if has_bias else None
        if mode == "bf16":
            dq, dk, dv = _run_bwd_hp(query, key, value, out, lse, grad_out, scaling, causal, g, varlen,
                                     out_layout, q_packs=(qnv, qsc), k_packs=(knv, ksc), key_pad_bias=bias)
        else:
            dq, dk, dv = _run_bwd(query, key, value, out, lse, grad_out, scaling, causal, g, varlen,
                                  out_layout, mode=mode, q_packs=(qnv, qsc), k_packs=(knv, ksc),
                                  key_pad_bias=bias, sr=srk[0], sr_p_dv=srk[1], sr_dot_dv=srk[2],
                                  sr_ds_dq=srk[3], qt_packs=tuple(extra[0:2]) if extra else None,
                                  kt_packs=tuple(extra[2:4]) if extra else None,
                                  vd_packs=tuple(extra[4:6]) if extra else None)
        return (dq, dk, dv) + (None,) * 23


def nvfp4_flash_attn_func(query, key, value, scaling, causal=False, num_key_value_groups=1,
                          key_pad_bias=None, cu_seqlens=None, stochastic_rounding=True,
                          save_backward_packs=False, backward_p_dv_stochastic_rounding=None,
                          backward_dot_dv_stochastic_rounding=None,
                          backward_ds_dq_stochastic_rounding=None, dkdv_scratch_bf16=None,
                          backward_grad_dots=None, backward_bf16_grad_dots=None, out_layout="zhsd",
                          block_m=64, block_n=128, num_warps=8, num_stages=3, q_packs=None, k_packs=None):
    """Differentiable NVFP4 flash attention (training entry; stands in for flash.py:4548-4703).

    Same signature as the reference.  ``backward_grad_dots`` in {None (auto), "bf16",
    "fp4_rownorm", "fp8_rownorm", "fp4_legacy"}; ``backward_bf16_grad_dots`` is the legacy boolean
    spelling of "bf16" (not both).  The stochastic-rounding knobs act on the "fp4_legacy" backward
    only (as in the reference, the normalised modes round to nearest); tile hints are accepted and
    ignored.
    """
    z, h, s_q, d = query.shape
    hk, s_kv = key.shape[1], key.shape[2]
    assert h % hk == 0 and h // hk == num_key_value_groups, "H must equal Hk * num_key_value_groups"
    assert d in (128, 256), "head dim must be 128 or 256"
    if out_layout not in ("zhsd", "zshd"):
        raise ValueError(f"out_layout must be 'zhsd' or 'zshd', got {out_layout!r}")
    if backward_bf16_grad_dots is not None:
        assert backward_grad_dots is None, (
            "pass either backward_grad_dots or the deprecated backward_bf16_grad_dots, not both")
        backward_grad_dots = "bf16" if backward_bf16_grad_dots else "fp4_legacy"
    if backward_grad_dots is None:
        # AUTO on the effective sequence: s_kv, or the mean sample length of a packed row
        eff = s_kv if cu_seqlens is None else s_q / max(1, cu_seqlens.numel() - 1)
        backward_grad_dots = _resolve_backward_grad_dots(None, eff, save_backward_packs, num_key_value_groups)
    seq_id = seq_start = seq_end = None
    if cu_seqlens is not None:
        assert causal, "varlen (cu_seqlens) implements block-diagonal causal attention; pass causal=True"
        assert z == 1, f"varlen packs all samples into one flattened row: Z must be 1, got Z={z}"
        assert s_q == s_kv, f"varlen requires packed self-attention (Sq == Skv), got {s_q} vs {s_kv}"
        seq_id, seq_start, seq_end = _varlen_seq_arrays(cu_seqlens, s_q, query.device)
    if q_packs is not None or k_packs is not None:
        assert not save_backward_packs, (
            "q_packs/k_packs are incompatible with save_backward_packs "
            "(the saved pack set must come from the same fused HP read)")
    qnv_in, qsc_in = q_packs if q_packs is not None else (None, None)
    knv_in, ksc_in = k_packs if k_packs is not None else (None, None)
    return _NVFP4FlashAttn.apply(
        query, key, value, scaling, causal, num_key_value_groups, key_pad_bias, stochastic_rounding,
        save_backward_packs, backward_p_dv_stochastic_rounding, backward_dot_dv_stochastic_rounding,
        backward_ds_dq_stochastic_rounding, dkdv_scratch_bf16, backward_grad_dots, out_layout == "zshd", block_m,
        block_n, num_warps, num_stages, seq_id, seq_start, seq_end, qnv_in, qsc_in, knv_in, ksc_in)
