"""NVFP4 KV cache for decode, B200-native.

Host-side mirror of ``NVFP4KVCache`` (reference: sageattention/nvfp4/kv_cache.py:100-373): same
constructor, attributes, methods and error behaviour; the work is done by CUDA kernels reached
through the C ABI:

* ``append`` is ONE launch (``nvfp4_kv_append``): K row pack, partial-group V store, re-pack of
  the current 16-key V^T group and the optional ring write, with no host synchronisation
  (the reference issues two Triton launches and about six small torch ops per token);
* ``prefill`` packs K and the full V groups straight into the cache buffers through the strided
  packer (no temporaries), then stashes the trailing < 16 tokens;
* ``hybrid_decode`` runs the split-K FP4 decode over the old prefix, an exact window-attention
  kernel over the bf16 ring, and merges the two on the device by their log-sum-exps.

Buffers (layouts identical to the reference so packed bytes can be compared):
  knv [Z*Hk, cap, D/2] uint8       ksc [Z*Hk, cap, D/16] float8_e4m3fn
  vnv [Z*Hk, D, cap_pad/2] uint8   vsc [Z*Hk, D, cap_pad/16] float8_e4m3fn   (V^T along keys)
  v_partial_bf16 [Z*Hk, 16, D]     rk / rv [Z, Hk, ring_cap, D] (only with recent_window > 0)
"""

from __future__ import annotations

import torch

from .. import _lib
from . import flash as _flash
from .flash import _next_mult, _pack_into


def append_token(key_new, value_new, knv, ksc, vnv, vsc, v_partial, rk, rv, pos: int) -> None:
    """One decode token ([Z, Hk, 1, D] or [Z*Hk, D]) into the cache buffers at position ``pos``: one
    kernel launch (K row pack, V stash and re-pack of the open 16-key V^T group, ring write when
    ``rk`` / ``rv`` are given).  The buffer-level form of ``NVFP4KVCache.append``."""
    zhk, _, half = knv.shape
    d = half * 2
    dtype = v_partial.dtype
    _lib.require_cuda(key_new, "key_new")
    kn = key_new.reshape(zhk, d)
    vn = value_new.reshape(zhk, d)
    if kn.dtype != dtype or kn.stride(1) != 1:
        kn = kn.to(dtype).contiguous()
    if vn.dtype != dtype or vn.stride(1) != 1:
        vn = vn.to(dtype).contiguous()
    if kn.stride(0) != vn.stride(0):
        kn, vn = kn.contiguous(), vn.contiguous()
    ring = rk is not None
    dev = knv.device
    _lib.call("nvfp4_kv_append", _lib.same_device(kn, vn, knv),
              kn.data_ptr(), vn.data_ptr(), _lib.dtype_code(dtype), kn.stride(0), zhk, d, int(pos),
              knv.data_ptr(), knv.stride(0), ksc.data_ptr(), ksc.stride(0),
              vnv.data_ptr(), vnv.stride(0), vnv.stride(1), vsc.data_ptr(), vsc.stride(0), vsc.stride(1),
              v_partial.data_ptr(), rk.data_ptr() if ring else None, rv.data_ptr() if ring else None,
              rk.shape[2] if ring else 0, _lib.stream_ptr(dev))


def hybrid_decode_buffers(query, knv, ksc, vnv, vsc, rk, rv, length: int, recent_window: int, scaling: float,
                          g: int, block_n: int = 128) -> torch.Tensor:
    """``NVFP4KVCache.hybrid_decode`` on the raw buffers of a cache holding ``length`` tokens."""
    z, h, _, d = query.shape
    hk, ring_cap, dtype = rk.shape[1], rk.shape[2], rk.dtype
    s = int(length)
    cut = (max(0, s - recent_window) // 16) * 16
    w = s - cut
    _lib.require_cuda(query, "query")
    qv = query if query.stride(-1) == 1 else query.contiguous()
    if qv.dtype != dtype:
        qv = qv.to(dtype)
    dev = query.device
    if cut == 0:
        # everything is still inside the window: exact attention over the ring alone
        out_rec = torch.empty(z, h, d, dtype=torch.float32, device=dev)
        lse_rec = torch.empty(z, h, dtype=torch.float32, device=dev)
        _lib.call("nvfp4_window_attention", _lib.same_device(qv, rk),
                  qv.data_ptr(), _lib.dtype_code(qv.dtype), qv.stride(0), qv.stride(1), rk.data_ptr(),
                  rv.data_ptr(), z, hk, g, d, ring_cap, cut, w, float(scaling),
                  out_rec.data_ptr(), lse_rec.data_ptr(), _lib.stream_ptr(dev))
        return out_rec.reshape(z, h, 1, d).to(query.dtype)
    # The window is cut into a few key ranges per (batch, kv head); each block stages its rows in
    # shared memory and writes an un-normalised split-K partial behind the FP4 decode's own, and the
    # decode's combine merges prefix and window in one pass (two launches + the combine; no
    # intermediate outputs, no copy of the query).  Pieces of at most 144 keys.
    pieces = max(1, min(64, -(-w // 144)))

    def fill(ws, total_slots, extra_base):
        _lib.call("nvfp4_window_partials", _lib.same_device(qv, rk, ws),
                  qv.data_ptr(), _lib.dtype_code(qv.dtype), qv.stride(0), qv.stride(1), rk.data_ptr(),
                  rv.data_ptr(), z, hk, g, d, ring_cap, cut, w, float(scaling), pieces,
                  ws.data_ptr(), total_slots, extra_base, _lib.stream_ptr(dev))

    s_pad = _next_mult(cut, block_n)
    packed = (knv[:, :cut], ksc[:, :cut], vnv[:, :, : s_pad // 2], vsc[:, :, : s_pad // 16], cut, s_pad)
    out, _ = _flash._decode_core(qv, packed, scaling, g, want_lse=False, extra=(pieces, fill))
    return out.to(query.dtype)


class NVFP4KVCache:
    """One layer's GQA KV cache held in NVFP4 and grown one token at a time.

    Args mirror the reference (kv_cache.py:115-125): ``z`` batch, ``hk`` kv heads, ``d`` head dim
    in {128, 256}, ``max_seq_len`` capacity, ``device``, ``dtype`` of incoming K/V, ``block_n``
    the key tile the V^T axis is padded to, ``recent_window`` > 0 keeps a bf16 ring of the most
    recent tokens for ``hybrid_decode``.
    """

    GROUP = 16

    def __init__(self, z, hk, d, max_seq_len, device, dtype=torch.bfloat16, block_n=128,
                 recent_window=0):
        assert d in (128, 256), "D must be 128 or 256"
        assert block_n == 128, "the B200 decode kernel walks 128-key tiles (block_n must be 128)"
        self.z, self.hk, self.d = z, hk, d
        self.zhk = z * hk
        self.max_seq_len = max_seq_len
        self.device = torch.device(device)
        self.dtype = dtype
        self.block_n = block_n
        self.cap_pad = _next_mult(max_seq_len, block_n)
        dev = self.device
        self.knv = torch.zeros(self.zhk, max_seq_len, d // 2, dtype=torch.uint8, device=dev)
        self.ksc = torch.zeros(self.zhk, max_seq_len, d // 16, dtype=torch.float8_e4m3fn, device=dev)
        self.vnv = torch.zeros(self.zhk, d, self.cap_pad // 2, dtype=torch.uint8, device=dev)
        self.vsc = torch.zeros(self.zhk, d, self.cap_pad // 16, dtype=torch.float8_e4m3fn, device=dev)
        self.v_partial_bf16 = torch.zeros(self.zhk, self.GROUP, d, dtype=dtype, device=dev)
        self.partial_len = 0
        self.length = 0
        self.recent_window = recent_window
        self.ring_cap = _next_mult(recent_window + self.GROUP, self.GROUP) if recent_window > 0 else 0
        if recent_window > 0:
            self.rk = torch.zeros(z, hk, self.ring_cap, d, dtype=dtype, device=dev)
            self.rv = torch.zeros(z, hk, self.ring_cap, d, dtype=dtype, device=dev)

    # ------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill(self, key: torch.Tensor, value: torch.Tensor):
        """Pack a prompt's K/V ([Z, Hk, S, D]) into the cache (kv_cache.py:187-224)."""
        z, hk, s, d = key.shape
        assert (z, hk, d) == (self.z, self.hk, self.d)
        assert s <= self.max_seq_len, "prefill exceeds capacity"
        k2 = key.reshape(self.zhk, s, d)
        v2 = value.reshape(self.zhk, s, d)
        _pack_into(k2, self.knv[:, :s], self.ksc[:, :s])
        full = (s // self.GROUP) * self.GROUP
        if full:
            _pack_into(v2[:, :full], self.vnv[:, :, : full // 2], self.vsc[:, :, : full // 16],
                       transpose=True)
        rem = s - full
        self.partial_len = rem
        self.v_partial_bf16.zero_()
        if rem:
            self.v_partial_bf16[:, :rem] = v2[:, full:]
            g0 = full // self.GROUP
            _pack_into(self.v_partial_bf16[:, :rem], self.vnv[:, :, g0 * 8 : g0 * 8 + 8],
                       self.vsc[:, :, g0 : g0 + 1], transpose=True, k_pad=self.GROUP)
        if self.recent_window > 0:
            w = min(self.ring_cap, s)
            pos = torch.arange(s - w, s, device=self.device)
            slots = pos % self.ring_cap
            self.rk[:, :, slots] = key[:, :, s - w :].to(self.dtype)
            self.rv[:, :, slots] = value[:, :, s - w :].to(self.dtype)
        self.length = s

    # ------------------------------------------------------------------ append
    @torch.no_grad()
    def append(self, key_new: torch.Tensor, value_new: torch.Tensor):
        """Append one decode token ([Z, Hk, 1, D]); a single kernel launch (kv_cache.py:227-257)."""
        z, hk, sq, d = key_new.shape
        assert sq == 1 and (z, hk, d) == (self.z, self.hk, self.d)
        t = self.length
        assert t < self.max_seq_len, "append exceeds capacity"
        ring = self.recent_window > 0
        append_token(key_new, value_new, self.knv, self.ksc, self.vnv, self.vsc, self.v_partial_bf16,
                     self.rk if ring else None, self.rv if ring else None, t)
        self.length = t + 1
        self.partial_len = (t % self.GROUP) + 1
        if self.partial_len == self.GROUP:
            self.partial_len = 0

    # ------------------------------------------------------------------ views
    def get_packed(self) -> tuple:
        """``(knv, ksc, vnv, vsc, s_kv, s_kv_pad)`` views of the live buffers (kv_cache.py:260-275)."""
        return self._packed_upto(self.length, _check=False)

    def _packed_upto(self, cut: int, _check: bool = True) -> tuple:
        if _check:
            assert cut % self.GROUP == 0, "cut must be a multiple of 16"
        s_pad = _next_mult(cut, self.block_n)
        return (self.knv[:, :cut], self.ksc[:, :cut], self.vnv[:, :, : s_pad // 2],
                self.vsc[:, :, : s_pad // 16], cut, s_pad)

    # ------------------------------------------------------------------ hybrid decode
    @torch.no_grad()
    def hybrid_decode(self, query: torch.Tensor, scaling: float, g: int) -> torch.Tensor:
        """Recent-window bf16 attention + FP4 attention over the older prefix, merged by LSE.

        Mirrors kv_cache.py:292-351: the split ``cut`` is rounded down to a 16-key boundary so no
        V group is divided; the recent side covers positions ``[cut, length)``.
        """
        if self.recent_window <= 0:
            raise RuntimeError("hybrid_decode needs recent_window > 0 "
                               "(construct NVFP4KVCache with recent_window>0)")
        if self.length == 0:
            raise RuntimeError("hybrid_decode requires at least one token (call prefill/append first)")
        return hybrid_decode_buffers(query, self.knv, self.ksc, self.vnv, self.vsc, self.rk, self.rv, self.length,
                                     self.recent_window, scaling, g, self.block_n)

    # ------------------------------------------------------------------ checkpoint / resume
    def state_dict(self) -> dict:
        """Everything needed to resume decoding: the packed prefix (only the ``length`` valid
        tokens, so a long-capacity cache checkpoints at its fill level), the bf16 stash of the open
        16-key V group, the recent-window ring and the geometry.  Tensors are clones on the
        cache's device; ``torch.save`` moves them like any other state dict.  (No counterpart in
        the reference; the cache there is rebuilt by re-running the prompt.)"""
        s = self.length
        s_grp = _next_mult(s, self.GROUP)
        sd = {
            "geometry": (self.z, self.hk, self.d, self.max_seq_len, self.block_n, self.recent_window,
                         str(self.dtype)),
            "length": s, "partial_len": self.partial_len,
            "knv": self.knv[:, :s].clone(), "ksc": self.ksc[:, :s].view(torch.uint8).clone(),
            "vnv": self.vnv[:, :, : s_grp // 2].clone(),
            "vsc": self.vsc[:, :, : s_grp // 16].view(torch.uint8).clone(),
            "v_partial": self.v_partial_bf16.clone(),
        }
        if self.recent_window > 0:
            sd["rk"], sd["rv"] = self.rk.clone(), self.rv.clone()
        return sd

    def load_state_dict(self, sd: dict) -> None:
        """Restore a cache saved by ``state_dict`` into this (same-geometry) cache; the capacity
        may differ as long as it holds ``length`` tokens."""
        z, hk, d, _cap, block_n, window, dt = sd["geometry"]
        assert (z, hk, d, block_n, window, dt) == (self.z, self.hk, self.d, self.block_n,
                                                   self.recent_window, str(self.dtype)), "geometry mismatch"
        s = int(sd["length"])
        assert s <= self.max_seq_len, "saved cache exceeds capacity"
        s_grp = _next_mult(s, self.GROUP)
        dev = self.device
        for buf in (self.knv, self.vnv):
            buf.zero_()
        self.ksc.view(torch.uint8).zero_()
        self.vsc.view(torch.uint8).zero_()
        self.knv[:, :s] = sd["knv"].to(dev)
        self.ksc.view(torch.uint8)[:, :s] = sd["ksc"].to(dev)
        self.vnv[:, :, : s_grp // 2] = sd["vnv"].to(dev)
        self.vsc.view(torch.uint8)[:, :, : s_grp // 16] = sd["vsc"].to(dev)
        self.v_partial_bf16.copy_(sd["v_partial"].to(dev))
        if self.recent_window > 0:
            self.rk.copy_(sd["rk"].to(dev))
            self.rv.copy_(sd["rv"].to(dev))
        self.length, self.partial_len = s, int(sd["partial_len"])

    # ------------------------------------------------------------------ accounting
    def fp4_bytes(self) -> int:
        s = self.length
        s_pad = _next_mult(s, self.block_n)
        k = self.zhk * s * (self.d // 2) + self.zhk * s * (self.d // 16)
        v = self.zhk * self.d * (s_pad // 2) + self.zhk * self.d * (s_pad // 16)
        return k + v + self.partial_len * self.zhk * self.d * self.dtype.itemsize

    def bf16_bytes(self) -> int:
        return 2 * self.zhk * self.length * self.d * self.dtype.itemsize

    def hybrid_bytes(self) -> int:
        ring = 2 * self.zhk * self.ring_cap * self.d * self.dtype.itemsize if self.recent_window > 0 else 0
        return self.fp4_bytes() + ring
