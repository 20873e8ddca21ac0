"""Failure detection without faulting anything.

* Host side (CPU, `gloo`): a ring-attention rank whose neighbour never posts its send must give up
  with an error instead of blocking forever.
* Device side (marked gpu): a kernel wait that can never be satisfied must run out of its probe
  budget, return by itself and report through the status word; the context stays usable.
"""

import os
import socket
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sageattention_b200.nvfp4 import distributed as D


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _withholding_worker(rank, world, port, ret, done):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    z, h, s_loc, d = 1, 2, 8, 4
    g = torch.Generator().manual_seed(rank)
    q, k, v = (torch.randn(z, h, s_loc, d, generator=g) for _ in range(3))

    def block_attention(q_loc, blk, mode):
        sc = torch.matmul(q_loc, blk[0].transpose(-1, -2))
        return torch.matmul(torch.softmax(sc, -1), blk[1]), torch.logsumexp(sc, -1)

    def merge(o1, l1, o2, l2):
        m = torch.maximum(l1, l2)
        w1, w2 = torch.exp(l1 - m)[..., None], torch.exp(l2 - m)[..., None]
        return (w1 * o1 + w2 * o2) / (w1 + w2), m + torch.log(torch.exp(l1 - m) + torch.exp(l2 - m))

    if rank == 0:
        t0 = time.time()
        try:
            D.ring_attention(q, [k, v], block_attention, merge, causal=False, timeout_s=2.0)
            ret[rank] = ("no error", time.time() - t0)
        except D.RingPeerTimeout as exc:
            ret[rank] = ("timeout", time.time() - t0, str(exc))
        except Exception as exc:          # any other failure is reported as such
            ret[rank] = (type(exc).__name__, time.time() - t0, str(exc))
        done.set()
    else:
        # this rank joined the group but never enters the step: its block is never sent
        done.wait(50)
        ret[rank] = ("withheld",)
    os._exit(0)     # the group holds an operation that can no longer complete; leave without a collective shutdown


def test_ring_rank_gives_up_when_peer_withholds_its_block():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager()
    ret, done = mgr.dict(), mgr.Event()
    procs = [ctx.Process(target=_withholding_worker, args=(r, world, port, ret, done)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        for p in procs:
            p.join(90)
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(10)
                if p.is_alive():
                    p.kill()
    assert ret.get(1) == ("withheld",)
    kind, dt = ret[0][0], ret[0][1]
    assert kind == "timeout", ret[0]
    assert 1.0 <= dt <= 30.0, dt
    assert "K/V block exchange of step 0" in ret[0][2]


def test_wait_helper_passes_completed_requests():
    class Done:
        def wait(self, timeout=None):
            return True

    class Late:
        def wait(self, timeout=None):
            return False

    D._wait_all([Done(), Done()], 0.1, "x")
    D._wait_all([Done()], None, "x")
    with pytest.raises(D.RingPeerTimeout, match="dK/dV"):
        D._wait_all([Done(), Late()], 0.1, "dK/dV accumulator hop")


@pytest.mark.gpu
def test_expired_device_wait_reports_status_and_context_survives(monkeypatch):
    from sageattention_b200 import _lib
    import sageattention_b200.nvfp4 as nv
    dev = torch.device("cuda", torch.cuda.current_device())
    assert _lib.read_status(dev) == 0
    w = _lib.status_word(dev)
    t0 = time.time()
    _lib.call("nvfp4_selftest_wait_timeout", dev, 37, 64, w.data_ptr(), _lib.stream_ptr(dev))
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0                       # the kernel gave up by itself
    assert _lib.read_status(dev) == (0x100 | 37)        # the first role's site, not the second's
    assert _lib.read_status(dev) == 0                   # read-and-clear
    # the context is healthy: a real kernel runs and leaves the status word clean
    x = torch.randn(2, 8, 128, device=dev, dtype=torch.bfloat16)
    nib, sc = nv._quant_nvfp4(x)
    torch.cuda.synchronize()
    assert nib.shape == (2, 8, 64) and _lib.read_status(dev) == 0
    # checked mode: the same expiry raises at the call site
    monkeypatch.setenv("NVFP4_CHECK_STATUS", "1")
    with pytest.raises(RuntimeError, match="bounded in-kernel wait expired"):
        _lib.call("nvfp4_selftest_wait_timeout", dev, 5, 64, w.data_ptr(), _lib.stream_ptr(dev))
    assert _lib.read_status(dev) == 0
    nv._quant_nvfp4(x)                                  # and a healthy call passes in checked mode
