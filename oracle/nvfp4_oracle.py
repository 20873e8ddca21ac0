"""CPU restatement of the reference's NVFP4 attention path (numpy only).

TEST INFRASTRUCTURE, NOT PRODUCT: this module is the checker the CUDA kernels are compared with.
Only the test-suite, the smoke entry and the benchmark's CPU-baseline leg may import it; the
shipped package never does (it fails loudly when the CUDA library is missing).

Pinning: the functions below are checked against fixtures produced by the reference's own
kernels executed under the Triton CPU interpreter (two hardware primitives emulated: the PTX
``cvt.rn.satfinite.e2m1x2.f32`` and the block-scaled MMA, for e2m1 and for e4m3 operands); see
``tests/golden/make_golden.py``.  That covers the NVFP4 pack, the forward, decode, the KV cache,
the three backward modes and the MXFP8 pack (``tests/golden/mxfp8_pack.npz``: bytes and scale
exponents of the reference's ``_pack_mxfp8_along_k``).

All ``file:line`` citations are paths inside the reference project
(thad0ctor/SageAttention), e.g. ``sageattention/nvfp4/flash.py:341-347``.

Arithmetic contract (IEEE fp32 throughout, as a torch CPU path would compute it):
  * per 16 along the contraction axis: ``amax -> sc = e4m3(clamp(amax / 6, 2**-9, 448))``,
    ``y = x / float(sc)``, ``code = e2m1_rtne_satfinite(y)``                (flash.py:341-347)
  * byte j = code[2j] | code[2j+1] << 4                                   (_fp4_pack.py:28-54)
  * padded / masked positions read as +0.0, so padded groups store scale byte 0x01 and
    nibble 0                                                                (flash.py:335-339)
"""

from __future__ import annotations

import numpy as np

GROUP = 16
E4M3_FLOOR = np.float32(2.0 ** -9)  # flash.py:127
E4M3_MAX = np.float32(448.0)        # flash.py:128
F4_MAX = np.float32(6.0)            # flash.py:129
NEG_INF = np.float32(-3.4028234663852886e38)  # flash.py:130 (finite, not -inf)

_E2M1_GRID = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
_E2M1_LUT = np.concatenate([_E2M1_GRID, -_E2M1_GRID]).astype(np.float32)


# --------------------------------------------------------------------------- scalar formats
def e4m3_bytes_from_f32(x: np.ndarray) -> np.ndarray:
    """Round positive finite fp32 values in [2**-9, 448] to float8_e4m3fn bit patterns (RTNE).

    Matches ``.to(tl.float8e4nv)`` on the clamped scale (flash.py:344).  Below 2**-6 the format
    is sub-normal with step 2**-9; a mantissa that rounds up to 8 carries into the exponent,
    which the integer encoding does for free.
    """
    x = np.asarray(x, dtype=np.float32)
    xd = x.astype(np.float64)
    mant, exp = np.frexp(xd)          # xd = mant * 2**exp, mant in [0.5, 1)
    e = exp - 1                       # xd = (2*mant) * 2**e, 2*mant in [1, 2)
    e = np.maximum(e, -6)             # sub-normals share the exponent of the smallest normal
    q = np.rint(xd / np.exp2(e.astype(np.float64) - 3.0))  # units of 2**(e-3); RTNE
    # normal: q in [8, 16]; sub-normal: q in [1, 8].  byte = (e + 6) * 8 + q works for both
    # (q == 16 carries to the next exponent, q == 8 at e == -6 is the smallest normal).
    b = (e + 6) * 8 + q.astype(np.int64)
    return b.astype(np.uint8)


def e4m3_to_f32(b: np.ndarray) -> np.ndarray:
    """Decode float8_e4m3fn bit patterns (sign ignored: scales are non-negative)."""
    b = np.asarray(b, dtype=np.uint8).astype(np.int32)
    e = (b >> 3) & 15
    m = b & 7
    sub = np.ldexp(m.astype(np.float64), -9)
    nrm = np.ldexp(1.0 + m.astype(np.float64) / 8.0, e - 7)
    return np.where(e == 0, sub, nrm).astype(np.float32)


def e2m1_codes(y: np.ndarray) -> np.ndarray:
    """fp32 -> 4-bit e2m1 code, round-to-nearest-even, saturating, sign kept on zero.

    Semantics of PTX ``cvt.rn.satfinite.e2m1x2.f32`` per element (_fp4_pack.py:38-54): ties go
    to the code with an even mantissa bit (0.25->0, 0.75->1, 1.25->1, 1.75->2, 2.5->2, 3.5->4,
    5->4); |y| > 6 -> 6; -0.0 and negatives that round to zero keep bit 3.
    """
    y = np.asarray(y, dtype=np.float32)
    a = np.abs(y)
    c = np.zeros(a.shape, dtype=np.uint8)
    c = np.where(a > 0.25, 1, c)
    c = np.where(a >= 0.75, 2, c)
    c = np.where(a > 1.25, 3, c)
    c = np.where(a >= 1.75, 4, c)
    c = np.where(a > 2.5, 5, c)
    c = np.where(a >= 3.5, 6, c)
    c = np.where(a > 5.0, 7, c)
    return (c.astype(np.uint8) | (np.signbit(y).astype(np.uint8) << 3)).astype(np.uint8)


def e2m1_to_f32(code: np.ndarray) -> np.ndarray:
    return _E2M1_LUT[np.asarray(code, dtype=np.uint8) & 15]


# --------------------------------------------------------------------------- pack / unpack
def _quant_groups(x: np.ndarray):
    """x [..., K] fp32 with K % 16 == 0 -> (codes uint8 [..., K], scale bytes uint8 [..., K/16])."""
    x = np.asarray(x, dtype=np.float32)
    k = x.shape[-1]
    assert k % GROUP == 0
    xb = x.reshape(x.shape[:-1] + (k // GROUP, GROUP))
    amax = np.max(np.abs(xb), axis=-1)
    s32 = np.minimum(np.maximum(amax / F4_MAX, E4M3_FLOOR), E4M3_MAX).astype(np.float32)
    sc_b = e4m3_bytes_from_f32(s32)
    scf = e4m3_to_f32(sc_b)
    y = (xb / scf[..., None]).astype(np.float32)
    return e2m1_codes(y).reshape(x.shape), sc_b


def _nibbles_to_bytes(codes: np.ndarray) -> np.ndarray:
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).astype(np.uint8)


def pack(x: np.ndarray, transpose: bool = False, k_pad: int | None = None):
    """NVFP4-pack along the contraction axis; mirrors ``_quant_nvfp4`` (flash.py:363-419).

    ``x`` is [B, R, K] (or [B, K, R] with ``transpose=True``, producing the V^T layout).
    Returns ``(nibbles uint8 [B, R, Kp/2], scale bytes uint8 [B, R, Kp/16])`` with
    ``Kp = k_pad or K``; the pad region reads as +0.0.
    """
    x = np.asarray(x, dtype=np.float32)
    if transpose:
        x = np.swapaxes(x, 1, 2)
    b, r, k = x.shape
    kp = k if k_pad is None else int(k_pad)
    assert kp % GROUP == 0 and kp >= k, "padded contraction dim must be a multiple of 16"
    if kp != k:
        xp = np.zeros((b, r, kp), dtype=np.float32)
        xp[:, :, :k] = x
        x = xp
    codes, sc = _quant_groups(x)
    return _nibbles_to_bytes(codes), sc


def unpack(nib: np.ndarray, sc: np.ndarray) -> np.ndarray:
    """Inverse view of ``pack``: [.., R, K/2] + [.., R, K/16] -> fp32 [.., R, K]."""
    nib = np.asarray(nib, dtype=np.uint8)
    codes = np.stack([nib & 15, nib >> 4], axis=-1).reshape(nib.shape[:-1] + (nib.shape[-1] * 2,))
    return (e2m1_to_f32(codes) * np.repeat(e4m3_to_f32(sc), GROUP, axis=-1)).astype(np.float32)


# --------------------------------------------------------------------------- MXFP8 (fp8_rownorm)
def e4m3_signed_bytes(x: np.ndarray) -> np.ndarray:
    """fp32 -> float8_e4m3fn bit patterns, round-to-nearest-even, saturating at +-448, signed zero
    (PTX ``cvt.rn.satfinite.e4m3x2.f32`` per element; Triton's ``.to(tl.float8e4nv)``)."""
    x = np.asarray(x, dtype=np.float32)
    a = np.minimum(np.abs(x).astype(np.float64), 448.0)
    mant, exp = np.frexp(a)
    e = np.maximum(exp - 1, -6)
    q = np.rint(a / np.exp2(e.astype(np.float64) - 3.0)).astype(np.int64)
    b = np.where(a == 0.0, 0, (e + 6) * 8 + q)
    b = np.minimum(b, 0x7E)
    return (b.astype(np.uint8) | (np.signbit(x).astype(np.uint8) << 7)).astype(np.uint8)


def e4m3_signed_to_f32(b: np.ndarray) -> np.ndarray:
    b = np.asarray(b, dtype=np.uint8)
    return (e4m3_to_f32(b & 0x7F) * np.where(b & 0x80, -1.0, 1.0)).astype(np.float32)


def pack_mxfp8(x: np.ndarray, transpose: bool = False, k_pad: int | None = None):
    """MXFP8 pack along the contraction axis, group 32; restates ``_pack_mxfp8_along_k``
    (flash.py:243-257): ``e = ceil(log2(max(amax, 1e-30) / 448))`` -- evaluated exactly, as the
    smallest integer with ``amax / 2**e <= 448`` --, bytes = e4m3(x / 2**e), scale byte = e + 127.
    Bit-equal to the reference's own function on the ``mxfp8_pack`` fixture (random magnitudes, an
    all-zero group, a group maximum of exactly 448, 1e-12 values).
    ``x`` [B, R, K] (or [B, K, R] with ``transpose``); returns (uint8 [B, R, Kp], uint8 [B, R, Kp/32])."""
    x = np.asarray(x, dtype=np.float32)
    if transpose:
        x = np.swapaxes(x, 1, 2)
    b, r, k = x.shape
    kp = k if k_pad is None else int(k_pad)
    assert kp % 32 == 0 and kp >= k
    xp = np.zeros((b, r, kp), dtype=np.float32)
    xp[:, :, :k] = x
    xb = xp.reshape(b, r, kp // 32, 32)
    amax = np.maximum(np.max(np.abs(xb), axis=-1), np.float32(1e-30)).astype(np.float32)
    mant, exp = np.frexp(amax.astype(np.float64))        # amax = mant 2^exp, mant in [0.5, 1)
    e = (exp - 1) - 8 + (mant * 2.0 > 1.75)
    q = e4m3_signed_bytes((xb.astype(np.float64) * np.exp2(-e.astype(np.float64))[..., None]).astype(np.float32))
    return q.reshape(b, r, kp), (e + 127).astype(np.uint8)


def unpack_mxfp8(q: np.ndarray, sc: np.ndarray) -> np.ndarray:
    scale = np.exp2(np.asarray(sc, dtype=np.float64) - 127.0)
    return (e4m3_signed_to_f32(q).astype(np.float64) * np.repeat(scale, 32, axis=-1)).astype(np.float32)


def next_mult(n: int, m: int) -> int:
    return ((n + m - 1) // m) * m


def quant_kv_decode(key: np.ndarray, value: np.ndarray, block_n: int = 128):
    """One-shot cache pack; mirrors ``nvfp4_quant_kv_decode`` (flash.py:3211-3241)."""
    z, hk, s, d = key.shape
    sp = next_mult(s, block_n)
    knv, ksc = pack(key.reshape(z * hk, s, d))
    vnv, vsc = pack(value.reshape(z * hk, s, d), transpose=True, k_pad=sp)
    return knv, ksc, vnv, vsc, s, sp


# --------------------------------------------------------------------------- masks
def varlen_arrays(cu_seqlens, s: int):
    """cu_seqlens [n+1] -> per-token (seq_id, seq_start, seq_end); flash.py:940-984."""
    cu = np.asarray(cu_seqlens, dtype=np.int64)
    assert cu.ndim == 1 and cu.size >= 2
    assert cu[0] == 0, f"cu_seqlens[0] must be 0, got {int(cu[0])}"
    assert cu[-1] == s, f"cu_seqlens[-1] ({int(cu[-1])}) must equal the packed seqlen ({s})"
    assert np.all(cu[1:] >= cu[:-1]), "cu_seqlens must be nondecreasing"
    pos = np.arange(s)
    seq_id = np.searchsorted(cu, pos, side="right") - 1
    return seq_id.astype(np.int32), cu[seq_id].astype(np.int32), cu[seq_id + 1].astype(np.int32)


def _visible(sq, skv, causal, seq_id_q=None, seq_id_k=None):
    """Boolean [sq, skv] visibility: causal is bottom-right aligned (flash.py:863-865)."""
    vis = np.ones((sq, skv), dtype=bool)
    if causal:
        i = np.arange(sq)[:, None]
        j = np.arange(skv)[None, :]
        vis &= j <= i + (skv - sq)
    if seq_id_q is not None:
        vis &= seq_id_q[:, None] == seq_id_k[None, :]
    return vis


# --------------------------------------------------------------------------- attention, mode A
def attention_mode_a(q, k, v, scaling, causal=False, g=1, cu_seqlens=None, key_pad_bias=None,
                     block_n: int = 128):
    """Q, K (along D) and V (along keys) quantise->dequantise, then exact fp32 softmax attention.

    q [Z,H,Sq,D], k/v [Z,Hk,Skv,D] as fp32 arrays holding bf16/fp16-representable values.
    Returns (out fp32 [Z,H,Sq,D], lse fp32 [Z,H,Sq]).  P is NOT quantised in this mode.
    """
    q = np.asarray(q, np.float32); k = np.asarray(k, np.float32); v = np.asarray(v, np.float32)
    z, h, sq, d = q.shape
    _, hk, skv, _ = k.shape
    assert h == hk * g
    qd = unpack(*pack(q.reshape(z * h, sq, d))).reshape(z, h, sq, d)
    kd = unpack(*pack(k.reshape(z * hk, skv, d))).reshape(z, hk, skv, d)
    sp = next_mult(skv, block_n)
    vd = unpack(*pack(v.reshape(z * hk, skv, d), transpose=True, k_pad=sp))  # [zhk, d, sp]
    vd = np.swapaxes(vd, 1, 2)[:, :skv].reshape(z, hk, skv, d)
    sid = None
    if cu_seqlens is not None:
        assert z == 1
        sid, _, _ = varlen_arrays(cu_seqlens, sq)
    vis = _visible(sq, skv, causal, sid, sid)
    out = np.zeros((z, h, sq, d), np.float32)
    lse = np.zeros((z, h, sq), np.float32)
    for zi in range(z):
        for hi in range(h):
            kh = hi // g
            s = (qd[zi, hi] @ kd[zi, kh].T).astype(np.float32) * np.float32(scaling)
            if key_pad_bias is not None:
                s = s + np.asarray(key_pad_bias, np.float32)[zi][None, :]
            s = np.where(vis, s, -np.inf)
            m = np.max(s, axis=1, keepdims=True)
            m = np.where(np.isfinite(m), m, 0.0)
            p = np.exp(s - m)
            l = p.sum(axis=1, keepdims=True)
            l_safe = np.where(l == 0, 1.0, l)
            out[zi, hi] = (p @ vd[zi, kh]) / l_safe
            lse[zi, hi] = (m + np.log(l_safe))[:, 0]
    return out, lse


# --------------------------------------------------------------------------- attention, mode B
def _pack_p_dequant(p: np.ndarray) -> np.ndarray:
    """In-kernel P pack per 16 keys, then what the MMA sees (flash.py:890-896)."""
    codes, sc = _quant_groups(p)
    return (e2m1_to_f32(codes) * np.repeat(e4m3_to_f32(sc), GROUP, axis=-1)).astype(np.float32)


def _walk_tiles(qd, kd, vdT, scaling, vis, bias, block_n, n_lo, n_hi):
    """Online-softmax walk over key tiles [n_lo, n_hi) in steps of block_n for one head.

    qd [Sq,D], kd [Skv,D], vdT [D,Sp] (dequantised), vis bool [Sq,Skv].  Follows
    flash.py:841-913: scale after the dot, bias, masks to NEG_INF, running max, natural exp,
    l from the unquantised p, P packed per 16 keys, fp32 accumulate.  A row whose history is
    still empty and whose tile is fully masked is left untouched (flash.py:876-884).
    Returns un-normalised (acc [Sq,D], m [Sq], l [Sq]).
    """
    sq, d = qd.shape
    skv = kd.shape[0]
    m_i = np.full((sq,), NEG_INF, np.float32)
    l_i = np.zeros((sq,), np.float32)
    acc = np.zeros((sq, d), np.float32)
    for n0 in range(n_lo, n_hi, block_n):
        n1 = min(n0 + block_n, skv)
        if n1 <= n0:
            break
        tile_vis = vis[:, n0:n1]
        if not tile_vis.any():
            continue
        s = (qd @ kd[n0:n1].T).astype(np.float32) * np.float32(scaling)
        if bias is not None:
            s = s + bias[None, n0:n1]
        sfull = np.full((sq, block_n), NEG_INF, np.float32)
        sfull[:, : n1 - n0] = np.where(tile_vis, s, NEG_INF)
        m_new = np.maximum(m_i, sfull.max(axis=1))
        m_sf = np.where(m_new == NEG_INF, np.float32(0.0), m_new)
        with np.errstate(over="ignore", under="ignore"):
            alpha = np.exp(m_i - m_sf).astype(np.float32)
            p = np.exp(sfull - m_sf[:, None]).astype(np.float32)
        l_i = (l_i * alpha + p.sum(axis=1, dtype=np.float32)).astype(np.float32)
        acc = acc * alpha[:, None]
        pq = _pack_p_dequant(p)
        vt = vdT[:, n0 : n0 + block_n]  # V^T is padded to a multiple of block_n
        acc = (acc + pq @ vt.T).astype(np.float32)
        m_i = m_new
    return acc, m_i, l_i


def attention_mode_b(q, k, v, scaling, causal=False, g=1, cu_seqlens=None, key_pad_bias=None,
                     block_n: int = 128):
    """Mode A plus the reference's tile walk with P quantised per 16 keys (flash.py:739-933).

    This is what a faithful FP4 kernel computes.  Returns (out fp32, lse fp32).
    """
    q = np.asarray(q, np.float32); k = np.asarray(k, np.float32); v = np.asarray(v, np.float32)
    z, h, sq, d = q.shape
    _, hk, skv, _ = k.shape
    assert h == hk * g
    qd = unpack(*pack(q.reshape(z * h, sq, d))).reshape(z, h, sq, d)
    kd = unpack(*pack(k.reshape(z * hk, skv, d))).reshape(z, hk, skv, d)
    sp = next_mult(skv, block_n)
    vdT = unpack(*pack(v.reshape(z * hk, skv, d), transpose=True, k_pad=sp)).reshape(z, hk, d, sp)
    sid = None
    if cu_seqlens is not None:
        assert z == 1
        sid, _, _ = varlen_arrays(cu_seqlens, sq)
    vis = _visible(sq, skv, causal, sid, sid)
    out = np.zeros((z, h, sq, d), np.float32)
    lse = np.zeros((z, h, sq), np.float32)
    for zi in range(z):
        bias = None if key_pad_bias is None else np.asarray(key_pad_bias, np.float32)[zi]
        for hi in range(h):
            kh = hi // g
            acc, m_i, l_i = _walk_tiles(qd[zi, hi], kd[zi, kh], vdT[zi, kh], scaling, vis, bias,
                                        block_n, 0, skv)
            l_safe = np.where(l_i == 0, np.float32(1.0), l_i)
            out[zi, hi] = acc / l_safe[:, None]
            m_fin = np.where(m_i == NEG_INF, np.float32(0.0), m_i)
            lse[zi, hi] = m_fin + np.log(l_safe)
    return out, lse


def attention_packed_mode_b(qnv, qsc, knv, ksc, vnv, vsc, z, h, hk, sq, skv, d, scaling,
                            causal=False, cu_seqlens=None, key_pad_bias=None, block_n=128):
    """Mode B starting from packs (the ``nvfp4_flash_attention_packed`` entry, flash.py:2655)."""
    g = h // hk
    qd = unpack(qnv, qsc).reshape(z, h, sq, d)
    kd = unpack(knv, ksc).reshape(z, hk, skv, d)
    vdT = unpack(vnv, vsc).reshape(z, hk, d, -1)
    sid = None
    if cu_seqlens is not None:
        sid, _, _ = varlen_arrays(cu_seqlens, sq)
    vis = _visible(sq, skv, causal, sid, sid)
    out = np.zeros((z, h, sq, d), np.float32)
    lse = np.zeros((z, h, sq), np.float32)
    for zi in range(z):
        bias = None if key_pad_bias is None else np.asarray(key_pad_bias, np.float32)[zi]
        for hi in range(h):
            acc, m_i, l_i = _walk_tiles(qd[zi, hi], kd[zi, hi // g], vdT[zi, hi // g], scaling,
                                        vis, bias, block_n, 0, skv)
            l_safe = np.where(l_i == 0, np.float32(1.0), l_i)
            out[zi, hi] = acc / l_safe[:, None]
            lse[zi, hi] = np.where(m_i == NEG_INF, np.float32(0.0), m_i) + np.log(l_safe)
    return out, lse


# --------------------------------------------------------------------------- decode
def decode_split_plan(s_kv: int, zhk: int, block_n: int = 128, target_programs: int = 256):
    """The reference's split heuristic (flash.py:3255-3262): returns (nsplit, split_kv)."""
    n_kblocks = -(-s_kv // block_n)
    want = max(1, target_programs // zhk)
    nsplit = max(1, min(n_kblocks, want))
    split_kv = -(-n_kblocks // nsplit) * block_n
    return -(-s_kv // split_kv), split_kv


def decode_prequant(query, kv_packed, scaling, g=1, block_n=128, split_kv=None,
                    target_programs=256, pieces=None):
    """Split-K decode over packs with exact combine; flash.py:3031-3208 and kv_cache.py:83-97.

    query [Z,H,1,D] fp32; kv_packed as returned by ``quant_kv_decode``.  ``split_kv`` (keys per
    split, multiple of block_n) overrides the reference heuristic so a kernel with a different
    split policy can be checked tile-for-tile.  ``pieces`` (unit index -> list of (lo, hi) key
    ranges, multiples of block_n except the last hi) replaces the equal splits altogether, for
    decompositions that cut units at arbitrary tile boundaries.
    Returns (out fp32 [Z,H,1,D], lse fp32 [Z,H]).
    """
    query = np.asarray(query, np.float32)
    z, h, one, d = query.shape
    assert one == 1
    knv, ksc, vnv, vsc, s_kv, s_pad = kv_packed
    zhk = knv.shape[0]
    hk = zhk // z
    assert h == hk * g and g <= 16
    if split_kv is None:
        _, split_kv = decode_split_plan(s_kv, zhk, block_n, target_programs)
    qd = unpack(*pack(query.reshape(zhk, g, d)))            # [zhk, g, d]
    kd = unpack(knv[:, :s_kv], ksc[:, :s_kv])               # [zhk, s, d]
    vdT = unpack(vnv, vsc)                                  # [zhk, d, sp]
    out = np.zeros((zhk, g, d), np.float32)
    lse = np.zeros((zhk, g), np.float32)
    vis = np.ones((g, s_kv), dtype=bool)
    for u in range(zhk):
        parts = []
        ranges = pieces[u] if pieces is not None else [(st, min(s_kv, st + split_kv))
                                                       for st in range(0, s_kv, split_kv)]
        for start, hi in ranges:
            parts.append(_walk_tiles(qd[u], kd[u], vdT[u], scaling, vis, None, block_n, start, hi))
        ms = np.stack([p[1] for p in parts])                # [nsplit, g]
        gm = ms.max(axis=0)
        with np.errstate(under="ignore"):
            f = np.exp(ms - gm[None]).astype(np.float32)
        f = np.where(ms == NEG_INF, np.float32(0), f)
        acc = sum(f[i][:, None] * parts[i][0] for i in range(len(parts)))
        den = sum(f[i] * parts[i][2] for i in range(len(parts)))
        den = np.where(den == 0, np.float32(1), den)
        out[u] = acc / den[:, None]
        lse[u] = gm + np.log(den)
    return out.reshape(z, h, 1, d), lse.reshape(z, h)


def lse_merge(o1, lse1, o2, lse2):
    """Exact merge of two softmax regions (kv_cache.py:347-350). o [..,D], lse [..]."""
    m = np.maximum(lse1, lse2)
    a = np.exp(lse1 - m)[..., None]
    b = np.exp(lse2 - m)[..., None]
    return ((a * o1 + b * o2) / (a + b)).astype(np.float32)


# --------------------------------------------------------------------------- KV cache
class KVCacheOracle:
    """State machine of ``NVFP4KVCache`` (kv_cache.py:100-373) on numpy arrays.

    Buffers are zero-initialised (scale byte 0x00 in never-written groups, kv_cache.py:141-146),
    the partial V group (< 16 tokens) is re-packed on every append (kv_cache.py:239-247), the
    optional recent ring has ``next16(W + 16)`` slots addressed by ``pos % ring_cap``
    (kv_cache.py:161, 250).
    """

    def __init__(self, z, hk, d, max_seq_len, block_n=128, recent_window=0):
        assert d in (128, 256), "D must be 128 or 256"
        self.z, self.hk, self.d, self.zhk = z, hk, d, z * hk
        self.max_seq_len, self.block_n = max_seq_len, block_n
        self.cap_pad = next_mult(max_seq_len, block_n)
        self.knv = np.zeros((self.zhk, max_seq_len, d // 2), np.uint8)
        self.ksc = np.zeros((self.zhk, max_seq_len, d // 16), np.uint8)
        self.vnv = np.zeros((self.zhk, d, self.cap_pad // 2), np.uint8)
        self.vsc = np.zeros((self.zhk, d, self.cap_pad // 16), np.uint8)
        self.v_partial = np.zeros((self.zhk, GROUP, d), np.float32)
        self.partial_len = 0
        self.length = 0
        self.recent_window = recent_window
        self.ring_cap = next_mult(recent_window + GROUP, GROUP) if recent_window > 0 else 0
        if recent_window > 0:
            self.rk = np.zeros((z, hk, self.ring_cap, d), np.float32)
            self.rv = np.zeros((z, hk, self.ring_cap, d), np.float32)

    def _pack_v_group(self, rows, gidx):
        nv, sc = pack(rows, transpose=True, k_pad=GROUP)
        self.vnv[:, :, gidx * 8 : gidx * 8 + 8] = nv
        self.vsc[:, :, gidx : gidx + 1] = sc

    def prefill(self, key, value):
        key = np.asarray(key, np.float32); value = np.asarray(value, np.float32)
        z, hk, s, d = key.shape
        assert (z, hk, d) == (self.z, self.hk, self.d)
        assert s <= self.max_seq_len, "prefill exceeds capacity"
        k2, v2 = key.reshape(self.zhk, s, d), value.reshape(self.zhk, s, d)
        self.knv[:, :s], self.ksc[:, :s] = pack(k2)
        full = (s // GROUP) * GROUP
        if full:
            nv, sc = pack(v2[:, :full], transpose=True)
            self.vnv[:, :, : full // 2] = nv
            self.vsc[:, :, : full // 16] = sc
        rem = s - full
        self.partial_len = rem
        self.v_partial[:] = 0
        if rem:
            self.v_partial[:, :rem] = v2[:, full:]
            self._pack_v_group(self.v_partial[:, :rem], full // GROUP)
        if self.recent_window > 0:
            for p in range(s - min(self.ring_cap, s), s):
                self.rk[:, :, p % self.ring_cap] = key[:, :, p]
                self.rv[:, :, p % self.ring_cap] = value[:, :, p]
        self.length = s

    def append(self, key_new, value_new):
        key_new = np.asarray(key_new, np.float32); value_new = np.asarray(value_new, np.float32)
        z, hk, one, d = key_new.shape
        assert one == 1 and (z, hk, d) == (self.z, self.hk, self.d)
        t = self.length
        assert t < self.max_seq_len, "append exceeds capacity"
        nv, sc = pack(key_new.reshape(self.zhk, 1, d))
        self.knv[:, t : t + 1], self.ksc[:, t : t + 1] = nv, sc
        gidx, pos = t // GROUP, t % GROUP
        if pos == 0:
            self.v_partial[:] = 0
        self.v_partial[:, pos] = value_new.reshape(self.zhk, d)
        self.partial_len = pos + 1
        self._pack_v_group(self.v_partial[:, : self.partial_len], gidx)
        if self.recent_window > 0:
            self.rk[:, :, t % self.ring_cap] = key_new[:, :, 0]
            self.rv[:, :, t % self.ring_cap] = value_new[:, :, 0]
        self.length = t + 1
        if self.partial_len == GROUP:
            self.partial_len = 0

    def get_packed(self, upto=None):
        s = self.length if upto is None else upto
        sp = next_mult(s, self.block_n)
        return (self.knv[:, :s], self.ksc[:, :s], self.vnv[:, :, : sp // 2],
                self.vsc[:, :, : sp // 16], s, sp)

    def hybrid_decode(self, query, scaling, g, split_kv=None):
        """bf16-recent + FP4-old with exact LSE merge (kv_cache.py:293-351)."""
        if self.recent_window <= 0:
            raise RuntimeError("hybrid_decode needs recent_window > 0")
        if self.length == 0:
            raise RuntimeError("hybrid_decode requires at least one token")
        query = np.asarray(query, np.float32)
        z, h, _, d = query.shape
        s = self.length
        cut = (max(0, s - self.recent_window) // GROUP) * GROUP
        idx = [p % self.ring_cap for p in range(cut, s)]
        kr = np.repeat(self.rk[:, :, idx], g, axis=1)
        vr = np.repeat(self.rv[:, :, idx], g, axis=1)
        sc = np.matmul(query, np.swapaxes(kr, -1, -2)) * np.float32(scaling)   # [Z,H,1,w]
        m = sc.max(axis=-1)
        ex = np.exp(sc - m[..., None])
        den = ex.sum(axis=-1)
        o_rec = np.matmul(ex, vr) / den[..., None]
        lse_rec = (m + np.log(den))[..., 0]
        if cut == 0:
            return o_rec.astype(np.float32)
        o_old, lse_old = decode_prequant(query, self.get_packed(cut), scaling, g,
                                         self.block_n, split_kv=split_kv)
        return lse_merge(o_old[:, :, 0], lse_old, o_rec[:, :, 0], lse_rec)[:, :, None, :]

    def fp4_bytes(self, itemsize=2):
        s, sp = self.length, next_mult(self.length, self.block_n)
        k = self.zhk * s * (self.d // 2 + self.d // 16)
        v = self.zhk * self.d * (sp // 2 + sp // 16)
        return k + v + self.partial_len * self.zhk * self.d * itemsize

    def bf16_bytes(self, itemsize=2):
        return 2 * self.zhk * self.length * self.d * itemsize


# --------------------------------------------------------------------------- exact attention + grads
def attention_exact(q, k, v, scaling, causal=False, g=1, cu_seqlens=None, key_pad_bias=None):
    """Plain fp32 attention on unquantised inputs with its gradients' building blocks.

    Returns (out, p) with p the softmax probabilities [Z,H,Sq,Skv]; used to derive reference
    gradients the way the reference's tests do with autograd of SDPA
    (tests/test_nvfp4_train_backward.py:92-103).
    """
    q = np.asarray(q, np.float64); k = np.asarray(k, np.float64); v = np.asarray(v, np.float64)
    z, h, sq, d = q.shape
    skv = k.shape[2]
    sid = None
    if cu_seqlens is not None:
        sid, _, _ = varlen_arrays(cu_seqlens, sq)
    vis = _visible(sq, skv, causal, sid, sid)
    kk = np.repeat(k, g, axis=1); vv = np.repeat(v, g, axis=1)
    s = np.matmul(q, np.swapaxes(kk, -1, -2)) * scaling
    if key_pad_bias is not None:       # [Z, Skv] additive, after the scaling (flash.py:2098-2100)
        s = s + np.asarray(key_pad_bias, np.float64)[:, None, None, :]
    s = np.where(vis, s, -np.inf)
    m = s.max(axis=-1, keepdims=True)
    p = np.exp(s - m)
    p = p / p.sum(axis=-1, keepdims=True)
    return np.matmul(p, vv), p


def attention_grads(q, k, v, do, scaling, causal=False, g=1, cu_seqlens=None, key_pad_bias=None):
    """Analytic dQ, dK, dV of exact attention (fp64), GQA-reduced to [Z,Hk,Skv,D]."""
    q = np.asarray(q, np.float64); k = np.asarray(k, np.float64); v = np.asarray(v, np.float64)
    do = np.asarray(do, np.float64)
    z, h, sq, d = q.shape
    hk, skv = k.shape[1], k.shape[2]
    out, p = attention_exact(q, k, v, scaling, causal, g, cu_seqlens, key_pad_bias)
    kk = np.repeat(k, g, axis=1); vv = np.repeat(v, g, axis=1)
    dv_h = np.matmul(np.swapaxes(p, -1, -2), do)
    dp = np.matmul(do, np.swapaxes(vv, -1, -2))
    delta = (do * out).sum(axis=-1, keepdims=True)
    ds = p * (dp - delta) * scaling
    dq = np.matmul(ds, kk)
    dk_h = np.matmul(np.swapaxes(ds, -1, -2), q)
    dk = dk_h.reshape(z, hk, g, skv, d).sum(axis=2)
    dv = dv_h.reshape(z, hk, g, skv, d).sum(axis=2)
    return dq, dk, dv


def cosine(a, b) -> float:
    a = np.asarray(a, np.float64).ravel(); b = np.asarray(b, np.float64).ravel()
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-300))


def bf16_round(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 (round to nearest even) -> fp32."""
    u = np.asarray(x, np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)


def rope_half_split(x, cos, sin, positions=None, pos0=0, round_to="bf16"):
    """Rotary embedding, half-split ("rotate_half") convention, fp32 math, one rounding to the
    storage dtype: the arithmetic of the fused rotary + pack producer (no reference counterpart:
    flash.py:10-13 asks callers to fuse one).  x [B, R, D]; cos / sin [P, D/2]."""
    x = np.asarray(x, np.float32)
    b, r, d = x.shape
    h = d // 2
    pos = (np.arange(r) + pos0) if positions is None else np.asarray(positions)
    c, s = np.asarray(cos, np.float32)[pos], np.asarray(sin, np.float32)[pos]
    lo, hi = x[..., :h], x[..., h:]
    # fused multiply-add of the kernel: fma(rot, sin, x * cos) with x * cos rounded to fp32 first
    y_lo = (np.float64(np.float32(lo * c)) + np.float64(-hi) * np.float64(s)).astype(np.float32)
    y_hi = (np.float64(np.float32(hi * c)) + np.float64(lo) * np.float64(s)).astype(np.float32)
    y = np.concatenate([y_lo, y_hi], axis=-1)
    if round_to == "bf16":
        y = bf16_round(y)
    return y
