"""Host-side multi-GPU logic on CPU with two `gloo` ranks: unit sharding and the ring schedule.

The ring driver is exercised with CPU stand-ins for the two CUDA callables (block attention and
LSE merge are the numpy oracle here), so what is tested is the partitioning, the message
plumbing (`batch_isend_irecv` around the ring) and the order of merges: the 2-rank result must
equal single-process attention over the whole sequence.
"""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import nvfp4_oracle as O
from sageattention_b200.nvfp4 import distributed as D


def test_unit_partition_covers_every_unit_once():
    for z, hk, world in ((4, 8, 8), (1, 8, 8), (16, 8, 4), (1, 4, 8), (3, 5, 2)):
        parts = D.unit_partition(z, hk, world)
        flat = [u for p in parts for u in p]
        assert sorted(flat) == [(a, b) for a in range(z) for b in range(hk)]
        assert max(len(p) for p in parts) - min(len(p) for p in parts) <= 1


def test_shard_and_unshard_roundtrip():
    z, h, hk, s, d = 2, 8, 4, 5, 16
    q = torch.arange(z * h * s * d, dtype=torch.float32).reshape(z, h, s, d)
    k = torch.randn(z, hk, s, d); v = torch.randn(z, hk, s, d)
    world = 3
    outs = []
    for r in range(world):
        qs, ks, vs, mine = D.shard_qkv(q, k, v, r, world)
        assert qs.shape[1] == h // hk and ks.shape[1] == 1 and len(mine) == qs.shape[0]
        outs.append(qs)            # identity "attention": output = the query shard
    assert torch.equal(D.unshard_out(outs, z, hk, world), q)


def test_ring_steps_causal_and_full():
    assert D.ring_steps(0, 4, True) == [(0, "causal"), (3, "skip"), (2, "skip"), (1, "skip")]
    assert D.ring_steps(2, 4, True) == [(2, "causal"), (1, "full"), (0, "full"), (3, "skip")]
    assert [m for _, m in D.ring_steps(1, 4, False)] == ["full"] * 4


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _ring_worker(rank, world, port, causal, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        z, h, hk, s_loc, d = 1, 2, 1, 32, 16
        g = torch.Generator().manual_seed(0)
        q = torch.randn(z, h, s_loc * world, d, generator=g)
        k = torch.randn(z, hk, s_loc * world, d, generator=g)
        v = torch.randn(z, hk, s_loc * world, d, generator=g)
        sl = slice(rank * s_loc, (rank + 1) * s_loc)
        ql, kl, vl = q[:, :, sl].contiguous(), k[:, :, sl].contiguous(), v[:, :, sl].contiguous()

        def block_attention(q_loc, blk, mode):
            kb, vb = blk
            sc = torch.matmul(q_loc, kb.repeat_interleave(h // hk, 1).transpose(-1, -2)) * d ** -0.5
            if mode == "causal":
                mask = torch.ones(s_loc, s_loc, dtype=torch.bool).tril()
                sc = sc.masked_fill(~mask, float("-inf"))
            m = sc.max(-1, keepdim=True).values
            p = torch.exp(sc - m)
            l = p.sum(-1, keepdim=True)
            return torch.matmul(p / l, vb.repeat_interleave(h // hk, 1)), (m + torch.log(l)).squeeze(-1)

        def merge(o1, l1, o2, l2):
            o = torch.from_numpy(O.lse_merge(o1.numpy(), l1.numpy(), o2.numpy(), l2.numpy()))
            m = torch.maximum(l1, l2)
            return o, m + torch.log(torch.exp(l1 - m) + torch.exp(l2 - m))

        out, lse = D.ring_attention(ql, [kl, vl], block_attention, merge, causal)
        ref, _ = O.attention_exact(q.numpy(), k.numpy(), v.numpy(), d ** -0.5, causal, h // hk)
        err = float(np.abs(out.numpy() - ref[:, :, sl]).max())
        ret[rank] = err
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("causal", [True, False])
def test_ring_attention_two_gloo_ranks_equals_single_process(causal):
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_ring_worker, args=(r, world, port, causal, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert len(ret) == world and max(ret.values()) < 1e-5, dict(ret)


def _ring_bwd_worker(rank, world, port, causal, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        z, h, hk, s_loc, d = 1, 4, 2, 16, 8
        g_ = h // hk
        gen = torch.Generator().manual_seed(1)
        q = torch.randn(z, h, s_loc * world, d, generator=gen)
        k = torch.randn(z, hk, s_loc * world, d, generator=gen)
        v = torch.randn(z, hk, s_loc * world, d, generator=gen)
        do = torch.randn(z, h, s_loc * world, d, generator=gen)
        sl = slice(rank * s_loc, (rank + 1) * s_loc)
        ql, kl, vl, dol = (t[:, :, sl].contiguous() for t in (q, k, v, do))
        rq, rk, rv = O.attention_grads(q.numpy(), k.numpy(), v.numpy(), do.numpy(), d ** -0.5, causal, g_)
        out_full, p_full = O.attention_exact(q.numpy(), k.numpy(), v.numpy(), d ** -0.5, causal, g_)
        out_l = torch.from_numpy(out_full[:, :, sl]).float()
        # merged LSE of the forward for the local rows
        sc = torch.matmul(q, k.repeat_interleave(g_, 1).transpose(-1, -2)) * d ** -0.5
        if causal:
            n = s_loc * world
            sc = sc.masked_fill(~torch.ones(n, n, dtype=torch.bool).tril(), float("-inf"))
        lse_l = torch.logsumexp(sc, dim=-1)[:, :, sl]
        delta_l = (dol * out_l).sum(-1)

        def block_backward(blk, mode):
            kb, vb = blk
            kk, vv = kb.repeat_interleave(g_, 1), vb.repeat_interleave(g_, 1)
            s_ = torch.matmul(ql, kk.transpose(-1, -2)) * d ** -0.5
            if mode == "causal":
                s_ = s_.masked_fill(~torch.ones(s_loc, s_loc, dtype=torch.bool).tril(), float("-inf"))
            p_ = torch.exp(s_ - lse_l[..., None])
            dp = torch.matmul(dol, vv.transpose(-1, -2))
            ds = p_ * (dp - delta_l[..., None]) * d ** -0.5
            dq = torch.matmul(ds, kk)
            dk = torch.matmul(ds.transpose(-1, -2), ql).reshape(z, hk, g_, s_loc, d).sum(2)
            dv = torch.matmul(p_.transpose(-1, -2), dol).reshape(z, hk, g_, s_loc, d).sum(2)
            return dq, dk, dv

        dq, dk, dv = D.ring_attention_backward([kl, vl], [kl, vl], block_backward, causal)
        err = max(float(np.abs(dq.numpy() - rq[:, :, sl]).max()), float(np.abs(dk.numpy() - rk[:, :, sl]).max()),
                  float(np.abs(dv.numpy() - rv[:, :, sl]).max()))
        ret[rank] = err
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("causal,world", [(True, 2), (False, 2), (True, 3)])
def test_ring_backward_gloo_ranks_equal_single_process(causal, world):
    """dK/dV accumulators travel with their block and come home after the last hop."""
    port = _free_port()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_ring_bwd_worker, args=(r, world, port, causal, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert len(ret) == world and max(ret.values()) < 1e-4, dict(ret)


def test_zigzag_split_merge_roundtrip_and_steps():
    x = torch.arange(2 * 3 * 16 * 4, dtype=torch.float32).reshape(2, 3, 16, 4)
    for world in (1, 2, 4):
        parts = [D.zigzag_split(x, r, world) for r in range(world)]
        assert torch.equal(D.zigzag_merge(parts), x)
    assert D.ring_steps_zigzag(1, 4) == [(1, "causal"), (0, "lo_kv"), (3, "hi_q"), (2, "hi_q")]


def _mode_mask(mode, n):
    c = n // 2
    m = torch.zeros(n, n, dtype=torch.bool)
    if mode == "causal":
        m = torch.ones(n, n, dtype=torch.bool).tril()
    elif mode == "lo_kv":
        m[:, :c] = True
    elif mode == "hi_q":
        m[c:, :] = True
    elif mode == "full":
        m[:] = True
    return m


def _zigzag_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        z, h, hk, c, d = 1, 2, 1, 8, 8
        g_ = h // hk
        s = 2 * c * world
        n = 2 * c
        gen = torch.Generator().manual_seed(2)
        q = torch.randn(z, h, s, d, generator=gen)
        k = torch.randn(z, hk, s, d, generator=gen)
        v = torch.randn(z, hk, s, d, generator=gen)
        do = torch.randn(z, h, s, d, generator=gen)
        pos = torch.arange(s, dtype=torch.float32).reshape(1, 1, s, 1)
        ql, kl, vl, dol, pl = (D.zigzag_split(t, rank, world) for t in (q, k, v, do, pos))
        pos_q = pl.reshape(-1)

        def scores(blk, mode):
            kb, vb, pk = blk
            # the mode's mask must be exactly the global causal mask between these positions
            assert torch.equal(_mode_mask(mode, n), pk.reshape(1, -1) <= pos_q.reshape(-1, 1)), mode
            sc = torch.matmul(ql, kb.repeat_interleave(g_, 1).transpose(-1, -2)) * d ** -0.5
            return sc.masked_fill(~_mode_mask(mode, n), float("-inf")), vb.repeat_interleave(g_, 1)

        def block_attention(q_loc, blk, mode):
            sc, vv = scores(blk, mode)
            m = sc.max(-1, keepdim=True).values
            m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
            p = torch.exp(sc - m_safe)
            l = p.sum(-1, keepdim=True)
            o = torch.matmul(p, vv) / torch.where(l == 0, torch.ones_like(l), l)
            return o, (m_safe + torch.log(l)).squeeze(-1)      # rows without keys: lse = -inf

        def merge(o1, l1, o2, l2):
            m = torch.maximum(l1, l2)
            w1, w2 = torch.exp(l1 - m)[..., None], torch.exp(l2 - m)[..., None]
            return (w1 * o1 + w2 * o2) / (w1 + w2), m + torch.log(torch.exp(l1 - m) + torch.exp(l2 - m))

        out, lse = D.ring_attention(ql, [kl, vl, pl], block_attention, merge, True, schedule="zigzag")
        ref, _ = O.attention_exact(q.numpy(), k.numpy(), v.numpy(), d ** -0.5, True, g_)
        ref_l = D.zigzag_split(torch.from_numpy(ref).float(), rank, world)
        err_f = float((out - ref_l).abs().max())
        delta = (dol * out).sum(-1)

        def block_backward(blk, mode):
            sc, vv = scores(blk, mode)
            kk = blk[0].repeat_interleave(g_, 1)
            p_ = torch.exp(sc - lse[..., None])
            dp = torch.matmul(dol, vv.transpose(-1, -2))
            ds = p_ * (dp - delta[..., None]) * d ** -0.5
            dq = torch.matmul(ds, kk)
            dk = torch.matmul(ds.transpose(-1, -2), ql).reshape(z, hk, g_, n, d).sum(2)
            dv = torch.matmul(p_.transpose(-1, -2), dol).reshape(z, hk, g_, n, d).sum(2)
            return dq, dk, dv

        dq, dk, dv = D.ring_attention_backward([kl, vl, pl], [kl, vl], block_backward, True, schedule="zigzag")
        rq, rk, rv = O.attention_grads(q.numpy(), k.numpy(), v.numpy(), do.numpy(), d ** -0.5, True, g_)
        errs = [float((a - D.zigzag_split(torch.from_numpy(b).float(), rank, world)).abs().max())
                for a, b in ((dq, rq), (dk, rk), (dv, rv))]
        ret[rank] = max([err_f] + errs)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_zigzag_ring_forward_backward_gloo(world):
    """Zigzag layout: every step's mode mask equals the global causal mask, results equal the
    single-process attention and its gradients."""
    port = _free_port()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_zigzag_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert len(ret) == world and max(ret.values()) < 1e-4, dict(ret)
