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


def test_fused_exchange_with_one_rank_equals_plain_decode(tq, oracle):
    """tq_decode_paged_exchange (decode, publish, wait, final merge in two launches) with a world of one
    rank: the same bits as tq_decode_paged, twice in a row (both buffer parities, the self-resetting
    ticket)."""
    import numpy as np

    from tests.test_zz_no_alloc import _case
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(8)
    lens, hq, h = [900, 333], 28, 4
    pool, tables = _case(oracle, "turbo_prod", rng, lens, h)
    cfg = tq.default_config()
    cfg.num_kv_heads = h
    lay = tq.make_layout_for(cfg)
    q = torch.from_numpy(rng.standard_normal((2, hq, 128)).astype(np.float16).view(np.int16)).to(dev).view(torch.float16)
    args = ("turbo_prod", q, torch.from_numpy(pool).to(dev), torch.from_numpy(tables).to(dev),
            torch.tensor(lens, dtype=torch.int32, device=dev), lay, cfg)
    want = tq.decode_paged(*args, max_kv_tokens=max(lens))
    rows = 2 * hq
    buf = torch.zeros(tq.peer_buffer_bytes(1, rows), dtype=torch.uint8, device=dev)
    ptrs = (C.c_void_p * 1)(buf.data_ptr())
    tq.peer_clear_status()
    for exchange in (1, 2, 3):
        out = torch.full_like(want, 5.0)
        tq.decode_paged_exchange(*args, ptrs, 0, 1, rows, exchange, max(lens), 0, max(lens), out)
        torch.cuda.synchronize()
        assert torch.equal(out, want)
    assert tq.peer_status() == 0
