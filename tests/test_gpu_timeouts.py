"""Bounded waits: a peer that never arrives ends the peer-to-peer all_reduce with a status code, not a hang.

The failure is made on the host side — a loopback communicator whose other "ranks" do not exist — never by faulting or
trapping the GPU: the kernel notices after its wait limit (about one second) that a flag is not coming, records where
it gave up and returns; the context stays usable and the next launches work.
"""
import time

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("algo_name", ["one_shot", "two_shot"])
def test_missing_peer_times_out_cleanly(pkg, dev, algo_name):
    comm = pkg.Comm.loopback(0, 2, 1 << 20)
    op = pkg.AllReduce(comm)
    op.set_algo(pkg.ALL_REDUCE_P2P_ONE_SHOT if algo_name == "one_shot" else pkg.ALL_REDUCE_P2P_TWO_SHOT)
    x = torch.ones(64, 4096, dtype=torch.float16, device=dev)
    assert comm.p2p_status() == 0
    t0 = time.time()
    op.launch(pkg.AllReduceArgs.of(x, x))
    torch.cuda.synchronize()  # returns: the wait is bounded
    waited = time.time() - t0
    assert 0.5 < waited < 10.0, waited
    code = comm.p2p_status()
    assert code != 0 and code % 16 in (1, 2, 3), code  # phase of the wait that ran out; code // 16 - 1 = the rank waited for
    assert code // 16 - 1 == 1
    # the context is intact: an ordinary operator still runs and is correct
    y = torch.empty(8, 256, dtype=torch.float16, device=dev)
    w = torch.ones(256, dtype=torch.float16, device=dev)
    pkg.RmsNorm(0).launch(pkg.RmsNormArgs.of(y, torch.full((8, 256), 2.0, dtype=torch.float16, device=dev), w, 0.0))
    torch.cuda.synchronize()
    np.testing.assert_allclose(y.float().cpu().numpy(), 1.0, atol=1e-3)
    # the first failure sticks until the communicator is reset; after the reset a new time-out is reported afresh
    comm.p2p_reset()
    assert comm.p2p_status() == 0
    op.launch(pkg.AllReduceArgs.of(x, x))
    torch.cuda.synchronize()
    assert comm.p2p_status() == code
    del op
    comm.destroy()


def test_status_reset_keeps_handles_usable(pkg, dev):
    # the reset entry points clear the status word and the internal arrival counters; a handle that was never in trouble
    # must come out of them unchanged (the time-out itself cannot be provoked for these kernels without faulting a GPU)
    mm, att = pkg.MatMul(0), pkg.Attention(0)
    a = torch.randn(300, 8192, device=dev).half()
    b = (torch.randn(8192, 700, device=dev) * 0.01).half()
    c = torch.empty(300, 700, dtype=torch.float16, device=dev)
    mm.launch(pkg.MatMulArgs.of(c, 0.0, a, b, 1.0))
    torch.cuda.synchronize()
    first = c.clone()
    mm.status_reset()
    att.status_reset()
    assert mm.status() == 0 and att.status() == 0
    mm.launch(pkg.MatMulArgs.of(c, 0.0, a, b, 1.0))
    torch.cuda.synchronize()
    assert torch.equal(first, c) and mm.status() == 0


def test_nvls_attach_needs_attached_staging(pkg, dev):
    # The in-switch all_reduce synchronises its ranks through the flags of the peer-to-peer staging buffer: a communicator
    # without attached peers refuses a multicast buffer (argument error, nothing launched), and detaching is always allowed.
    comm = pkg.Comm.loopback(0, 2, 1 << 20)
    buf = torch.zeros(1 << 20, dtype=torch.uint8, device=dev)
    with pytest.raises(pkg.SchemeError):
        comm.nvls_attach(buf.data_ptr(), buf)  # not a multicast address either, but the check comes first
    comm.nvls_detach()
    comm.destroy()
