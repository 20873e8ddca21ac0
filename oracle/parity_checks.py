"""Parity checks of the CUDA kernels at the sizes of the benchmark configurations.

TEST INFRASTRUCTURE, NOT PRODUCT (like everything under ``oracle/``): used by the GPU parity tests
and by the CPU-baseline leg of ``bench.py``, never by the shipped package.  Each check takes the
benchmark's own seeded inputs (numpy, the bf16-representable values the GPU saw) and the kernel's
results for one unit of the configuration, runs the numpy oracle on that unit, and returns the
agreement figures: ``{"cosine": ..., "max_abs": ..., "oracle_seconds": ...}``.

Configurations (sizes as stated in the benchmark):
  2  prefill forward  Z4 H32 Hk8 S8192 D128 causal, K with 8 outlier channels  -> one (batch,
     KV-group) unit = 4 query heads on 1 KV head, oracle mode B (the reference's tile walk)
  3  packed varlen 16384 tokens H32 Hk8 D128 -> the longest segment of one KV group: forward vs
     mode B on the same global 128-key tile alignment, gradients vs analytic fp64 gradients
  4  decode Z16 H32 Hk8 D128 S32768 -> two cache units under the kernel's own decomposition
  5  D=256 long context -> one head at S >= 16384, forward vs mode B
"""

from __future__ import annotations

import time

import numpy as np

from . import nvfp4_oracle as O

def _agree(got, ref, seconds):
    got = np.asarray(got, np.float32); ref = np.asarray(ref, np.float32)
    return {"cosine": O.cosine(got, ref), "max_abs": float(np.abs(got - ref).max()),
            "oracle_seconds": float(seconds)}


# ----------------------------------------------------------------------------- configuration 2 / 5
def forward_unit(out_unit, q_unit, k_unit, v_unit, scaling, causal=True):
    """Kernel output of one (batch, KV-group) unit ``[G, S, D]`` against oracle mode B on the same
    inputs: ``q_unit [G, S, D]``, ``k_unit`` / ``v_unit [S, D]`` (fp32 arrays of bf16 values)."""
    g = q_unit.shape[0]
    t0 = time.perf_counter()
    ref, ref_lse = O.attention_mode_b(q_unit[None], k_unit[None, None], v_unit[None, None], scaling, causal, g)
    dt = time.perf_counter() - t0
    res = _agree(out_unit, ref[0], dt)
    s, d = k_unit.shape
    res["flops"] = g * 4.0 * s * s * d / (2.0 if causal else 1.0)
    return res


# ----------------------------------------------------------------------------- configuration 3
def varlen_segment(lens, which=None):
    """(start, end, aligned_start) of the chosen (default: longest) segment of the packed row;
    aligned_start is the 128-key tile boundary at or below start."""
    cu = np.concatenate([[0], np.cumsum(lens)])
    i = int(np.argmax(lens)) if which is None else which
    a, b = int(cu[i]), int(cu[i + 1])
    return a, b, (a // 128) * 128


def varlen_forward_segment(out_rows, q_rows, k_rows, v_rows, seg_start, scaling):
    """Forward of a packed-row segment against mode B with the kernel's global tile alignment.

    All arrays cover tokens [aligned_start, seg_end) of the packed row (``q_rows [G, n, D]``,
    ``k_rows`` / ``v_rows [n, D]``, ``out_rows [G, n, D]``); ``seg_start`` is the segment's first
    token relative to aligned_start.  The sub-row is itself a packed row of two samples (the tail of
    the previous sample, then the segment), so the oracle walks the same 128-key tiles as the
    kernel did on the full row.  Only the segment's rows are compared."""
    g, n, d = q_rows.shape
    cu = [0, n] if seg_start == 0 else [0, seg_start, n]
    t0 = time.perf_counter()
    ref, _ = O.attention_mode_b(q_rows[None], k_rows[None, None], v_rows[None, None], scaling, True, g,
                                cu_seqlens=np.asarray(cu, np.int32))
    dt = time.perf_counter() - t0
    return _agree(out_rows[:, seg_start:], ref[0][:, seg_start:], dt)


def varlen_grads_segment(dq, dk, dv, q_seg, k_seg, v_seg, do_seg, scaling):
    """Gradients of one segment of one KV group (``dq [G, n, D]``, ``dk`` / ``dv [n, D]``) against
    the analytic fp64 gradients of exact attention on the isolated segment (block-diagonal causal
    attention is exact per segment)."""
    g = q_seg.shape[0]
    t0 = time.perf_counter()
    rq, rk, rv = O.attention_grads(q_seg[None], k_seg[None, None], v_seg[None, None], do_seg[None], scaling,
                                   True, g)
    dt = time.perf_counter() - t0
    return {"dq": O.cosine(dq, rq[0]), "dk": O.cosine(dk, rk[0, 0]), "dv": O.cosine(dv, rv[0, 0]),
            "oracle_seconds": float(dt)}


# ----------------------------------------------------------------------------- configuration 4
def balanced_pieces(zhk: int, s_kv: int, sm_count: int, units):
    """Key ranges each listed unit is cut into by the balanced decode decomposition: the unit-major
    list of 128-key tiles is shared equally by ``n`` persistent CTAs (CTA b owns tiles
    [b*T/n, (b+1)*T/n)), ``n = min(sm_count, T/4)``; a unit's pieces are the intersections."""
    tiles = -(-s_kv // 128)
    total = zhk * tiles
    n = max(1, min(sm_count, total // 4 if total // 4 > 0 else 1))
    bounds = sorted({(b * total) // n for b in range(n + 1)})
    out = {}
    for u in units:
        x0, x1 = u * tiles, (u + 1) * tiles
        cuts = [x0] + [b for b in bounds if x0 < b < x1] + [x1]
        out[u] = [((a - x0) * 128, min(s_kv, (b - x0) * 128)) for a, b in zip(cuts[:-1], cuts[1:])]
    return out


def decode_units(out_units, q_units, packed_units, scaling, g, pieces):
    """Decode outputs ``[U, G, D]`` of U cache units against the oracle's split-K walk over the
    same pieces.  ``packed_units`` = (knv, ksc, vnv, vsc, s_kv, s_pad) holding only those U units;
    ``pieces`` = list (per unit) of key ranges."""
    u, gg, d = q_units.shape
    t0 = time.perf_counter()
    ref, ref_lse = O.decode_prequant(q_units.reshape(1, u * gg, 1, d), packed_units, scaling, g,
                                     pieces={i: p for i, p in enumerate(pieces)})
    dt = time.perf_counter() - t0
    res = _agree(out_units, ref.reshape(u, gg, d), dt)
    res["lse"] = ref_lse.reshape(u, gg)
    return res


def hybrid_units(out_units, q_units, packed_old_units, k_win, v_win, scaling, g, pieces):
    """``hybrid_decode`` outputs ``[U, G, D]`` against: oracle split-K decode of the FP4 prefix over
    the kernel's pieces, exact fp32 attention over the high-precision window ``k_win`` / ``v_win
    [U, W, D]``, merged with the exact log-sum-exp formula."""
    u, gg, d = q_units.shape
    t0 = time.perf_counter()
    o_old, lse_old = O.decode_prequant(q_units.reshape(1, u * gg, 1, d), packed_old_units, scaling, g,
                                       pieces={i: p for i, p in enumerate(pieces)})
    o_old, lse_old = o_old.reshape(u, gg, d), lse_old.reshape(u, gg)
    sc = np.einsum("ugd,uwd->ugw", q_units.astype(np.float32), k_win.astype(np.float32)) * np.float32(scaling)
    m = sc.max(-1)
    ex = np.exp(sc - m[..., None])
    den = ex.sum(-1)
    o_rec = np.einsum("ugw,uwd->ugd", ex, v_win.astype(np.float32)) / den[..., None]
    ref = O.lse_merge(o_old, lse_old, o_rec, m + np.log(den))
    return _agree(out_units, ref, time.perf_counter() - t0)
