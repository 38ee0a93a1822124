"""The allocation-free decode entry point (tq_decode_paged_static), through the C ABI.

It exists for hosts that may not allocate device memory on the decode path (a serving
engine whose own pool owns the whole GPU, a loop that cannot risk an allocation's implicit
synchronisation): its split-KV scratch is a fixed array inside
the library.  Checked here against the regular entry point on two calls in a row (the array
is shared and keeps the previous call's bytes), and that a shape beyond the array is refused.
This file is collected last so that every other test has already run if it fails."""
import ctypes as C

import numpy as np
import pytest
import torch

from tests.conftest import rowwise_rel_err
from tests.golden.cases import make_kv

pytestmark = pytest.mark.gpu


def _case(oracle, scheme, rng, lens, h):
    maxpages = (max(lens) + 15) // 16
    b = len(lens)
    tables = rng.permutation(b * maxpages + 2).astype(np.int32)[:b * maxpages].reshape(b, maxpages)
    ocfg = oracle.make_config(h)
    lay = oracle.layout_for(scheme, ocfg)
    pool = np.zeros((b * maxpages + 2) * lay.page_size_bytes, np.uint8)
    for i, n in enumerate(lens):
        k, v = make_kv(rng, n, h)
        t = np.arange(n)
        oracle.pack(scheme, k, v, (tables[i][t // 16] * 16 + t % 16).astype(np.int32), ocfg, pool=pool)
    return pool, tables


@pytest.mark.parametrize("scheme", ["turbo_prod", "turbo_mse"])
def test_static_scratch_decode_matches_regular_entry_point(tq, oracle, scheme):
    assert torch.cuda.is_available()
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(2718)
    cfg = tq.default_config()
    cfg.num_kv_heads = 2
    lay = tq.layout_for_scheme(scheme, cfg)
    # two different shapes back to back: the second call finds the first call's bytes in the array
    for lens, hq in (([1500, 700, 33], 16), ([4000], 4)):
        pool, tables = _case(oracle, scheme, rng, lens, 2)
        query = rng.standard_normal((len(lens), hq, 128)).astype(np.float16)
        q = torch.from_numpy(query.view(np.int16)).to(dev).view(torch.float16)
        args = (scheme, q, torch.from_numpy(pool).to(dev), torch.from_numpy(tables).to(dev),
                torch.tensor(lens, dtype=torch.int32, device=dev), lay, cfg)
        regular = tq.decode_paged(*args, max_kv_tokens=max(lens))
        static = tq.decode_paged_static(*args, max_kv_tokens=max(lens))
        torch.cuda.synchronize()
        # same kernels, same split count, same arithmetic: identical bits
        assert torch.equal(regular, static)
        ref = oracle.decode_paged(scheme, query, pool, tables, lens, oracle.make_config(2))
        assert rowwise_rel_err(static.cpu().numpy(), ref) < 2e-3


def test_static_scratch_rejects_oversized_shape(tq):
    dev = torch.device("cuda:0")
    cfg = tq.default_config()
    cfg.num_kv_heads = 8
    lay = tq.make_layout_for(cfg)
    b, hq, n = 512, 64, 4096  # 512 x 64 rows x 130 floats already exceed 8 MiB
    need = tq.decode_workspace_bytes(b, hq, n, cfg)
    assert need > 8 << 20
    q = torch.zeros(b, hq, 128, dtype=torch.float16, device=dev)
    tables = torch.zeros(b, n // 16, dtype=torch.int32, device=dev)
    lens = torch.zeros(b, dtype=torch.int32, device=dev)
    pool = torch.zeros(lay.page_size_bytes, dtype=torch.uint8, device=dev)
    with pytest.raises(RuntimeError, match="built-in array holds"):
        tq.decode_paged_static("turbo_prod", q, pool, tables, lens, lay, cfg, max_kv_tokens=n)


def test_static_scratch_leaves_device_memory_alone(tq, oracle):
    """The device's free memory (driver view: every allocation of any pool in this process counts)
    is the same after a series of static calls as before it, with the output tensor made
    beforehand -- whereas the regular entry point without a workspace draws on the library's
    stream-ordered pool, which shows as less free memory once that pool has grown."""
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(5)
    cfg = tq.default_config()
    cfg.num_kv_heads = 2
    lay = tq.make_layout_for(cfg)
    lens = [2500, 900]
    pool, tables = _case(oracle, "turbo_prod", rng, lens, 2)
    q = torch.from_numpy(rng.standard_normal((2, 16, 128)).astype(np.float16).view(np.int16)).to(dev).view(torch.float16)
    out = torch.empty_like(q)
    args = ("turbo_prod", q, torch.from_numpy(pool).to(dev), torch.from_numpy(tables).to(dev),
            torch.tensor(lens, dtype=torch.int32, device=dev), lay, cfg)
    tq.decode_paged_static(*args, output=out, max_kv_tokens=max(lens))  # first call: symbol address lookup
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info(dev)
    for _ in range(8):
        tq.decode_paged_static(*args, output=out, max_kv_tokens=max(lens))
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info(dev)
    assert free1 == free0
