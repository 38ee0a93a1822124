"""The bounded flag wait of the peer exchange, made to run out on one GPU.

tq_peer_merge waits for a flag per rank; here the exchange claims two ranks but only rank 0 ever
publishes, with the wait bound set to 5 ms.  The kernel gives up, records status 1 and finishes;
nothing faults or spins on, the context stays usable and the next, complete exchange is correct."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_peer_merge_wait_runs_out_and_the_context_survives(tq):
    dev = torch.device("cuda:0")
    hq, h, rows = 8, 2, 16
    gen = torch.Generator(device=dev)
    gen.manual_seed(3)
    local = torch.randn(rows, 130, device=dev, generator=gen)
    local[:, 129] = local[:, 129].abs() + 1.0  # a positive softmax denominator
    out = torch.zeros(rows, 128, dtype=torch.float16, device=dev)
    tq.peer_clear_status()
    assert tq.peer_status() == 0
    try:
        tq.peer_set_wait_ns(5_000_000)
        buf = torch.zeros(tq.peer_buffer_bytes(2, rows), dtype=torch.uint8, device=dev)
        ptrs = (C.c_void_p * 2)(buf.data_ptr(), buf.data_ptr())
        tq.peer_publish(local, ptrs, 0, 2, rows, rows, 1)  # rank 0 publishes; rank 1 never does
        tq.peer_merge(buf, 2, rows, rows, 1, out, hq, h)
        torch.cuda.synchronize()                          # returns: the wait gave up after 5 ms
        assert tq.peer_status() == 1
    finally:
        tq.peer_set_wait_ns(0)
        tq.peer_clear_status()
    # a complete exchange afterwards (one rank) gives the merge of its single record
    buf1 = torch.zeros(tq.peer_buffer_bytes(1, rows), dtype=torch.uint8, device=dev)
    ptrs1 = (C.c_void_p * 1)(buf1.data_ptr())
    tq.peer_publish(local, ptrs1, 0, 1, rows, rows, 1)
    tq.peer_merge(buf1, 1, rows, rows, 1, out, hq, h)
    want = torch.zeros_like(out)
    tq.merge_partials(local.view(1, rows, 130), want, hq, h)
    torch.cuda.synchronize()
    assert tq.peer_status() == 0
    assert torch.equal(out, want)
