"""Multi-GPU use of the NVFP4 attention path: one process per GPU over ``torch.distributed``.

The reference has no distributed code on this path.  Two schemes cover its configurations:

* **(batch, KV-head group) sharding** -- attention is independent per (z, kv-head): each rank
  owns a subset of those units with the G query heads that share each KV head and runs the
  ordinary single-GPU operators on it.  No collective on the data path.  ``unit_partition``
  gives the assignment; ``shard_qkv`` slices tensors accordingly.
* **context-parallel ring attention** for the long-context configuration (few units, very long
  S): every rank owns a contiguous slice of the sequence.  Local K and V are packed to NVFP4 once;
  the packs (nibbles + e4m3 scales, about 9/32 of the bf16 bytes) travel around the ring with
  ``batch_isend_irecv`` while the rank computes on the block it already holds, and the partial
  (out, lse) pairs are merged with the exact log-sum-exp formula.  Received blocks land in the
  rank's own HBM before any kernel reads them.

``ring_attention`` is written against two callables (block attention and merge) so the ring
schedule and the message plumbing are testable with ``gloo`` on CPU; ``ring_flash_attention``
binds them to the CUDA operators.  The backward (``ring_attention_backward`` /
``ring_flash_attention_backward``) walks the same ring: a K/V block travels together with the
fp32 accumulators of its dK/dV, every rank adds the contribution of its own queries (exact
because the probabilities are recomputed against the merged LSE of the forward), and one last hop
brings each accumulator home.  ``ring_flash_attn_func`` ties both into autograd.
"""

from __future__ import annotations

from typing import Callable, List, Sequence, Tuple

import torch
import torch.distributed as dist


# --------------------------------------------------------------------------- unit sharding
def unit_partition(z: int, hk: int, world: int) -> List[List[Tuple[int, int]]]:
    """Round-robin assignment of the z*hk (batch, kv-head) units to ``world`` ranks."""
    units = [(zi, ki) for zi in range(z) for ki in range(hk)]
    return [units[r::world] for r in range(world)]


def shard_qkv(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, rank: int, world: int):
    """Slice ``[Z,H,S,D]`` / ``[Z,Hk,S,D]`` tensors to the units of ``rank``.

    Units are flattened into the batch axis: returns ``q [U,G,Sq,D]``, ``k, v [U,1,Skv,D]`` so the
    ordinary operators run unchanged with ``num_key_value_groups = G``.
    """
    z, h, sq, d = q.shape
    hk = k.shape[1]
    g = h // hk
    mine = unit_partition(z, hk, world)[rank]
    qs = torch.stack([q[zi, ki * g:(ki + 1) * g] for zi, ki in mine]) if mine else q.new_empty(0, g, sq, d)
    ks = torch.stack([k[zi, ki:ki + 1] for zi, ki in mine]) if mine else k.new_empty(0, 1, k.shape[2], d)
    vs = torch.stack([v[zi, ki:ki + 1] for zi, ki in mine]) if mine else v.new_empty(0, 1, v.shape[2], d)
    return qs, ks, vs, mine


def unshard_out(parts: Sequence[torch.Tensor], z: int, hk: int, world: int) -> torch.Tensor:
    """Inverse of ``shard_qkv`` for outputs ``[U,G,Sq,D]`` gathered from all ranks."""
    g, sq, d = parts[0].shape[1:]
    out = parts[0].new_empty(z, hk * g, sq, d)
    assign = unit_partition(z, hk, world)
    for r, part in enumerate(parts):
        for u, (zi, ki) in enumerate(assign[r]):
            out[zi, ki * g:(ki + 1) * g] = part[u]
    return out


# --------------------------------------------------------------------------- ring attention
def ring_steps(rank: int, world: int, causal: bool) -> List[Tuple[int, str]]:
    """Key/value blocks rank ``rank`` meets, in order, and how to mask each.

    Step t holds the block that originated on rank ``(rank - t) mod world``.  With causal
    masking and contiguous sequence slices a block from a later rank is invisible ("skip"), the
    rank's own block is causal ("causal") and earlier blocks are fully visible ("full").
    """
    steps = []
    for t in range(world):
        src = (rank - t) % world
        if not causal or src < rank:
            steps.append((src, "full"))
        elif src == rank:
            steps.append((src, "causal"))
        else:
            steps.append((src, "skip"))
    return steps


def ring_steps_zigzag(rank: int, world: int) -> List[Tuple[int, str]]:
    """Causal schedule for the zigzag layout: the sequence is cut into ``2*world`` chunks and rank
    r owns chunks r and ``2*world-1-r`` (concatenated in that order), which balances causal work.

    With the block of rank ``src`` in hand: "causal" = the rank's own block (a plain causal mask
    over the local concatenation is the global mask); "lo_kv" (src < rank) = every local query sees
    the block's first chunk and nothing of its second; "hi_q" (src > rank) = only the local second
    chunk sees the block, all of it.  Every step costs half a full block on every rank.
    """
    steps = []
    for t in range(world):
        src = (rank - t) % world
        steps.append((src, "causal" if src == rank else ("lo_kv" if src < rank else "hi_q")))
    return steps


def zigzag_split(x: torch.Tensor, rank: int, world: int, dim: int = 2) -> torch.Tensor:
    """This rank's slice of a full-sequence tensor in the zigzag layout (chunks r and 2W-1-r)."""
    chunks = x.chunk(2 * world, dim=dim)
    return torch.cat([chunks[rank], chunks[2 * world - 1 - rank]], dim=dim)


def zigzag_merge(parts: Sequence[torch.Tensor], dim: int = 2) -> torch.Tensor:
    """Inverse of ``zigzag_split`` over the per-rank slices (rank order)."""
    world = len(parts)
    chunks = [None] * (2 * world)
    for r, p in enumerate(parts):
        lo, hi = p.chunk(2, dim=dim)
        chunks[r], chunks[2 * world - 1 - r] = lo, hi
    return torch.cat(chunks, dim=dim)


def _steps(rank: int, world: int, causal: bool, schedule: str):
    if schedule not in ("contiguous", "zigzag"):
        raise ValueError(f"schedule must be 'contiguous' or 'zigzag', got {schedule!r}")
    if schedule == "zigzag" and causal:
        return ring_steps_zigzag(rank, world)
    return ring_steps(rank, world, causal)


def _exchange(tensors: Sequence[torch.Tensor], recv: Sequence[torch.Tensor], group, rank: int, world: int,
              communicate: bool = True):
    """Post sends of ``tensors`` to rank+1 and receives into ``recv`` from rank-1 (non-blocking).

    ``communicate=False`` (a measurement aid) copies the local tensors instead of exchanging
    messages: the same kernels run on the same schedule without any communication."""
    if not communicate:
        for t, r in zip(tensors, recv):
            r.copy_(t)
        return []
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    ops = []
    for t, r in zip(tensors, recv):
        ops.append(dist.P2POp(dist.isend, t, dist.get_global_rank(group, nxt) if group else nxt, group))
        ops.append(dist.P2POp(dist.irecv, r, dist.get_global_rank(group, prv) if group else prv, group))
    return dist.batch_isend_irecv(ops)


class RingPeerTimeout(RuntimeError):
    """A neighbour of the ring did not deliver (or accept) a block within the allowed time."""


def _wait_all(reqs, timeout_s, what: str):
    """Wait for posted sends / receives.  With ``timeout_s`` the wait is bounded on the host: a
    peer that died, never joined the step or never posted its send surfaces here as
    ``RingPeerTimeout`` instead of blocking this rank forever (the backends report an expired wait
    as an exception or a False return)."""
    if timeout_s is None:
        for r in reqs:
            r.wait()
        return
    import datetime
    limit = datetime.timedelta(seconds=float(timeout_s))
    for r in reqs:
        try:
            ok = r.wait(limit)
        except Exception as exc:        # gloo: RuntimeError "Timed out waiting ..."; nccl: DistBackendError
            raise RingPeerTimeout(f"ring attention: {what} not completed within {timeout_s} s ({exc})") from exc
        if ok is False:
            raise RingPeerTimeout(f"ring attention: {what} not completed within {timeout_s} s")


def ring_attention(q_local, kv_block: Sequence[torch.Tensor],
                   block_attention: Callable, merge: Callable, causal: bool, group=None,
                   schedule: str = "contiguous", _communicate: bool = True, timeout_s=None):
    """Context-parallel attention of the local queries against every rank's K/V block.

    ``timeout_s`` bounds every wait on a neighbour (``RingPeerTimeout`` on expiry); None waits as
    long as the process group allows.

    ``kv_block``: the tensors describing the local K/V block (anything with a fixed shape across
    ranks, e.g. the six pack tensors).  ``block_attention(q_local, block, mode)`` returns
    ``(out, lse)`` for mode "full" or "causal" (with ``schedule="zigzag"`` also "lo_kv" / "hi_q",
    see ``ring_steps_zigzag``; rows a step does not touch carry lse = -inf);
    ``merge(out_a, lse_a, out_b, lse_b)`` returns the combined ``(out, lse)``.  Communication of
    step t+1 overlaps the compute of step t.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    cur = list(kv_block)
    out = lse = None
    for t, (src, mode) in enumerate(_steps(rank, world, causal, schedule)):
        reqs, nxt_bufs = [], None
        if t + 1 < world:
            nxt_bufs = [torch.empty_like(x) for x in cur]
            reqs = _exchange(cur, nxt_bufs, group, rank, world, _communicate)
        if mode != "skip":
            o, l = block_attention(q_local, cur, mode)
            out, lse = (o, l) if out is None else merge(out, lse, o, l)
        _wait_all(reqs, timeout_s, f"K/V block exchange of step {t}")
        if nxt_bufs is not None:
            cur = nxt_bufs
    return out, lse


def ring_attention_backward(kv_block: Sequence[torch.Tensor], grad_like: Sequence[torch.Tensor],
                            block_backward: Callable, causal: bool, group=None,
                            schedule: str = "contiguous", _communicate: bool = True, timeout_s=None):
    """Gradients of ``ring_attention``.  ``timeout_s`` as in ``ring_attention``.

    ``kv_block``: the tensors that describe the local K/V block for the backward (fixed shapes
    across ranks).  ``grad_like``: two tensors shaped like the local dK and dV (fp32 accumulators are
    allocated like them).  ``block_backward(block, mode)`` returns ``(dq, dk, dv)`` of the local
    queries against that block for mode "full" or "causal" (dq of the local queries, dk/dv of the
    block's keys).  Returns ``(dq, dk, dv)`` for the local slices; dk/dv in fp32.

    Step t works on the block that originated on rank ``rank - t``; the block's accumulators arrive
    one step behind the block itself, so their transfer overlaps the next block computation.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    cur = list(kv_block)
    acc = [torch.zeros_like(g, dtype=torch.float32) for g in grad_like]
    acc_recv, acc_reqs = None, []
    dq = None
    for t, (src, mode) in enumerate(_steps(rank, world, causal, schedule)):
        reqs, nxt_bufs = [], None
        if t + 1 < world:
            nxt_bufs = [torch.empty_like(x) for x in cur]
            reqs = _exchange(cur, nxt_bufs, group, rank, world, _communicate)
        part = block_backward(cur, mode) if mode != "skip" else None
        if t > 0:                       # accumulators of the block held now, sent after step t-1
            _wait_all(acc_reqs, timeout_s, f"dK/dV accumulator hop before step {t}")
            acc = acc_recv
        if part is not None:
            dq = part[0].float() if dq is None else dq + part[0].float()
            acc[0] += part[1].float()
            acc[1] += part[2].float()
        _wait_all(reqs, timeout_s, f"K/V block exchange of step {t}")
        if world > 1:                   # forward the accumulators (last step: the hop back home)
            acc_recv = [torch.empty_like(a) for a in acc]
            acc_reqs = _exchange(acc, acc_recv, group, rank, world, _communicate)
        if nxt_bufs is not None:
            cur = nxt_bufs
    if world > 1:
        _wait_all(acc_reqs, timeout_s, "last dK/dV accumulator hop")
        acc = acc_recv
    if dq is None:
        dq = torch.zeros_like(grad_like[0][:0])
    return dq, acc[0], acc[1]


def ring_flash_attention(query, key, value, scaling, causal=True, num_key_value_groups=1, group=None,
                         schedule="contiguous", _communicate=True):
    """NVFP4 ring attention on CUDA: ``query [Z,H,S_loc,D]``, ``key/value [Z,Hk,S_loc,D]`` are this
    rank's slice of the sequence: one contiguous piece (``schedule="contiguous"``, length a multiple
    of 128) or the two zigzag chunks (``schedule="zigzag"``, each a multiple of 128; see
    ``zigzag_split``).  Returns ``(out [Z,H,S_loc,D], lse [Z*H, S_loc])``.
    """
    from .. import _lib
    from . import flash

    z, h, s_loc, d = query.shape
    hk = key.shape[1]
    zig = schedule == "zigzag" and causal
    c = s_loc // 2
    assert s_loc % (256 if zig else 128) == 0, "ring attention needs 128-multiple slices (per chunk)"
    knv, ksc = flash._quant_nvfp4(key.reshape(z * hk, s_loc, d))
    vnv, vsc = flash._quant_nvfp4(value.reshape(z * hk, s_loc, d), transpose=True, k_pad=s_loc)
    qnv, qsc = flash._quant_nvfp4(query.reshape(z * h, s_loc, d))
    block = [knv, ksc.view(torch.uint8), vnv, vsc.view(torch.uint8)]
    if zig:
        qnv_hi, qsc_hi = qnv[:, c:].contiguous(), qsc[:, c:].contiguous()

    def run(qn, qs, blk, sq, skv, is_causal):
        return flash._run_flash_packed(qn, qs, blk[0], blk[1], blk[2], blk[3], z, h, hk, sq, skv, d,
                                       scaling, torch.float32, causal=is_causal, return_lse=True)

    def block_attention(_q, blk, mode):
        if mode in ("full", "causal"):
            return run(qnv, qsc, blk, s_loc, s_loc, mode == "causal")
        if mode == "lo_kv":          # all local queries x the block's first chunk
            lo = [blk[0][:, :c].contiguous(), blk[1][:, :c].contiguous(),
                  blk[2][:, :, :c // 2].contiguous(), blk[3][:, :, :c // 16].contiguous()]
            return run(qnv, qsc, lo, s_loc, c, False)
        o_hi, l_hi = run(qnv_hi, qsc_hi, blk, c, s_loc, False)      # "hi_q": second local chunk x whole block
        o = torch.zeros(z, h, s_loc, d, dtype=torch.float32, device=o_hi.device)
        l = torch.full((z * h, s_loc), float("-inf"), dtype=torch.float32, device=o_hi.device)
        o[:, :, c:] = o_hi
        l[:, c:] = l_hi
        return o, l

    def merge(o1, l1, o2, l2):
        rows = z * h * s_loc
        out, lse = torch.empty_like(o1), torch.empty_like(l1)
        _lib.call("nvfp4_lse_merge", _lib.same_device(o1, l1, o2, l2),
                  o1.data_ptr(), l1.data_ptr(), o2.data_ptr(), l2.data_ptr(),
                  out.data_ptr(), lse.data_ptr(), _lib.DT_FP32, rows, d, _lib.stream_ptr(o1.device))
        return out, lse

    out, lse = ring_attention(query, block, block_attention, merge, causal, group, schedule, _communicate)
    return out.to(query.dtype), lse


def ring_flash_attention_backward(query, key, value, out, lse, dout, scaling, causal=True,
                                  num_key_value_groups=1, group=None, schedule="contiguous",
                                  _communicate=True, backward_grad_dots="bf16"):
    """NVFP4 ring-attention backward on CUDA for the local sequence slices (bf16 tensors).

    ``out`` / ``lse`` are the merged results of ``ring_flash_attention``; with them every block's
    probabilities are the globally normalised ones, so the per-block backward kernels give exact
    contributions.  ``backward_grad_dots``: "bf16" (high-precision gradient GEMMs, the default),
    "fp4_rownorm" or "fp8_rownorm" (the block-scaled kernels, faster at head dim 256; the
    transposed packs of a block's K and the along-D pack of its V are made by the rank that holds
    the block, so the messages stay the same).  Returns ``(dq, dk, dv)`` in ``dout.dtype``.
    """
    from .. import _lib
    from . import flash

    z, h, s_loc, d = query.shape
    hk = key.shape[1]
    dev = query.device
    zig = schedule == "zigzag" and causal
    c = s_loc // 2
    qc, kc, vc = flash._as_bf16_rows(query), flash._as_bf16_rows(key), flash._as_bf16_rows(value)
    need_copy = not (dout.dtype == torch.bfloat16 and dout.is_contiguous())
    doc, delta = flash._bwd_prep(dout, y=out.to(dout.dtype), want_copy=need_copy)
    if doc is None:
        doc = dout.view(z * h, s_loc, d)
    qnv, qsc = flash._quant_nvfp4(query.reshape(z * h, s_loc, d))
    knv, ksc = flash._quant_nvfp4(key.reshape(z * hk, s_loc, d))
    lse = lse.contiguous()
    block = [kc, vc, knv, ksc.view(torch.uint8)]
    q_side = (qnv, qsc, qc, doc, lse, delta)
    if zig:   # the second local chunk as contiguous tensors of its own
        q_side_hi = tuple(t[:, c:].contiguous() for t in q_side)

    def run(qs, blk, sq, skv, is_causal):
        dq = torch.empty(z, h, sq, d, dtype=torch.float32, device=dev)
        dk = torch.empty(z, hk, skv, d, dtype=torch.float32, device=dev)
        dv = torch.empty(z, hk, skv, d, dtype=torch.float32, device=dev)
        _lib.call("nvfp4_bwd_hp", _lib.same_device(*qs, *blk),
            qs[0].data_ptr(), qs[1].data_ptr(), blk[2].data_ptr(), blk[3].data_ptr(), qs[2].data_ptr(),
            blk[0].data_ptr(), blk[1].data_ptr(), qs[3].data_ptr(), qs[4].data_ptr(), qs[5].data_ptr(), None, None, None,
            dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), _lib.DT_FP32, z, h, hk, sq, skv, d, float(scaling),
            1 if is_causal else 0, _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev))
        return dq, dk, dv

    def block_backward(blk, mode):
        if mode in ("full", "causal"):
            return run(q_side, blk, s_loc, s_loc, mode == "causal")
        if mode == "lo_kv":
            lo = [t[:, :c].contiguous() for t in blk]
            dq, dk_lo, dv_lo = run(q_side, lo, s_loc, c, False)
            dk = torch.zeros(z, hk, s_loc, d, dtype=torch.float32, device=dev)
            dv = torch.zeros(z, hk, s_loc, d, dtype=torch.float32, device=dev)
            dk[:, :, :c] = dk_lo
            dv[:, :, :c] = dv_lo
            return dq, dk, dv
        dq_hi, dk, dv = run(q_side_hi, blk, c, s_loc, False)      # "hi_q"
        dq = torch.zeros(z, h, s_loc, d, dtype=torch.float32, device=dev)
        dq[:, :, c:] = dq_hi
        return dq, dk, dv

    if backward_grad_dots != "bf16":
        assert backward_grad_dots in ("fp4_rownorm", "fp8_rownorm"), backward_grad_dots
        assert s_loc % 128 == 0 and (not zig or c % 128 == 0), (
            "the block-scaled ring backward wants local slices (and zigzag chunks) of a multiple of 128 tokens")
        fp8 = backward_grad_dots == "fp8_rownorm"
        tpack = (lambda x, pad: flash._quant_mxfp8_t(x, pad)) if fp8 else \
                (lambda x, pad: flash._quant_nvfp4(x, transpose=True, k_pad=pad))

        def q_side_packs(qt, dot, ot, lse_t):
            """Everything the block-scaled kernels need of a set of local query rows."""
            sq = qt.shape[2]
            _, dl, amax = flash._bwd_prep(dot, y=ot.to(dot.dtype), want_amax=True)
            do3 = dot.reshape(z * h, sq, d) if dot.is_contiguous() or z == 1 else dot.contiguous().view(z * h, sq, d)
            donv, dosc, dotnv, dotsc = flash._quant_nvfp4_dual(do3, sq, _prescale_amax=amax)
            if fp8:
                dotnv, dotsc = flash._quant_mxfp8_t(do3, sq, _prescale_amax=amax)
            q3 = qt.reshape(z * h, sq, d)
            qn, qs_ = flash._quant_nvfp4(q3)
            qtn, qts = tpack(q3, sq)
            return (qn, qs_, donv, dosc, dotnv, dotsc, qtn, qts, lse_t.contiguous(), dl, amax)

        qf = q_side_packs(query, dout, out, lse)
        if zig:
            qf_hi = q_side_packs(query[:, :, c:], dout[:, :, c:], out[:, :, c:], lse[:, c:])

        def run4(qs, blk, sq, skv, is_causal):
            kb, vb = blk[0][:, :skv], blk[1][:, :skv]
            ktn, kts = tpack(kb, skv)
            vdn, vds = flash._quant_nvfp4(vb)
            knv_b = blk[2][:, :skv].contiguous()
            ksc_b = blk[3][:, :skv].contiguous()
            dq = torch.empty(z, h, sq, d, dtype=torch.float32, device=dev)
            dk = torch.empty(z, hk, skv, d, dtype=torch.float32, device=dev)
            dv = torch.empty(z, hk, skv, d, dtype=torch.float32, device=dev)
            ptr = lambda t: t.data_ptr()
            _lib.call("nvfp4_bwd_fp4", _lib.same_device(qs[0], kb, vb),
                      ptr(qs[0]), ptr(qs[1]), ptr(knv_b), ptr(ksc_b), ptr(vdn), ptr(vds), ptr(qs[2]), ptr(qs[3]),
                      ptr(qs[4]), ptr(qs[5]), ptr(qs[6]), ptr(qs[7]), ptr(ktn), ptr(kts), ptr(qs[8]), ptr(qs[9]),
                      ptr(qs[10]), None, None, None, ptr(dq), ptr(dk), ptr(dv), _lib.DT_FP32, z, h, hk, sq, skv, sq,
                      skv, d, float(scaling), (1 if is_causal else 0) | (128 if fp8 else 0), 0,
                      _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev))
            return dq, dk, dv

        def block_backward(blk, mode):      # noqa: F811  (the block-scaled twin of the function above)
            if mode in ("full", "causal"):
                return run4(qf, blk, s_loc, s_loc, mode == "causal")
            if mode == "lo_kv":
                dq, dk_lo, dv_lo = run4(qf, blk, s_loc, c, False)
                dk = torch.zeros(z, hk, s_loc, d, dtype=torch.float32, device=dev)
                dv = torch.zeros(z, hk, s_loc, d, dtype=torch.float32, device=dev)
                dk[:, :, :c] = dk_lo
                dv[:, :, :c] = dv_lo
                return dq, dk, dv
            dq_hi, dk, dv = run4(qf_hi, blk, c, s_loc, False)      # "hi_q"
            dq = torch.zeros(z, h, s_loc, d, dtype=torch.float32, device=dev)
            dq[:, :, c:] = dq_hi
            return dq, dk, dv

    like = torch.empty(z, hk, s_loc, d, dtype=torch.float32, device=dev)
    dq, dk, dv = ring_attention_backward(block, [like, like], block_backward, causal, group, schedule,
                                         _communicate)
    gdt = dout.dtype
    return dq.to(gdt), dk.to(gdt), dv.to(gdt)


class _RingFlashAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, query, key, value, scaling, causal, g, group, schedule, communicate, grad_dots="bf16"):
        out, lse = ring_flash_attention(query, key, value, scaling, causal, g, group, schedule, communicate)
        ctx.save_for_backward(query, key, value, out, lse)
        ctx.meta = (float(scaling), bool(causal), int(g), group, schedule, communicate, grad_dots)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        query, key, value, out, lse = ctx.saved_tensors
        scaling, causal, g, group, schedule, communicate, grad_dots = ctx.meta
        dq, dk, dv = ring_flash_attention_backward(query, key, value, out, lse, grad_out, scaling, causal, g,
                                                   group, schedule, communicate, grad_dots)
        return dq, dk, dv, None, None, None, None, None, None, None


def ring_flash_attn_func(query, key, value, scaling, causal=True, num_key_value_groups=1, group=None,
                         schedule="zigzag", _communicate=True, backward_grad_dots="bf16"):
    """Differentiable context-parallel NVFP4 attention over this rank's slice of the sequence.

    ``schedule="zigzag"`` (default, causal only): the slice is chunks r and 2W-1-r of the sequence
    (``zigzag_split``), every rank does the same work per ring step.  ``"contiguous"``: one piece per
    rank; with a causal mask the last rank works on every step and the first on one.
    """
    return _RingFlashAttn.apply(query, key, value, scaling, causal, num_key_value_groups, group, schedule,
                                _communicate, backward_grad_dots)
