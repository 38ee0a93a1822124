"""KV-sequence split across ranks (world_size 2, gloo, CPU): every rank computes the
(acc, m, l) partial of its page-aligned token range with the oracle, the package's
gather helper all-gathers them, and a log-sum-exp merge reproduces full-range attention."""
import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.golden.cases import make_kv


def lse_merge(parts):
    """parts [P, rows, 130] -> normalised rotated-domain accumulators [rows, 128]."""
    m = parts[:, :, 128].max(axis=0)
    w = np.exp(parts[:, :, 128] - m[None])
    acc = (parts[:, :, :128] * w[:, :, None]).sum(0)
    l = (parts[:, :, 129] * w).sum(0)
    return acc / l[:, None]


def _worker(rank, world, port, q):
    import os
    import sys
    from pathlib import Path
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    from oracle import oracle as O
    from turborag_b200.parallel import gather_partials, kv_token_range, shard_range
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(123)  # same data on every rank
        H, n, nq = 2, 203, 3
        cfg = O.make_config(H)
        key, value = make_kv(rng, n, H)
        query = rng.standard_normal((nq, H, 128)).astype(np.float16)
        slots = np.arange(n, dtype=np.int32)
        res = {}
        for scheme in ("turbo_prod", "turbo_mse"):
            pool = O.pack(scheme, key, value, slots, cfg)
            b, e = kv_token_range(n, rank, world, 16)
            part = O.attn_state(scheme, query, pool, slots[b:e], cfg).reshape(nq * H, 130)
            allp = gather_partials(torch.from_numpy(part)).numpy()
            full = O.attn_state(scheme, query, pool, slots, cfg).reshape(nq * H, 130)
            merged = lse_merge(allp)
            ref = full[:, :128] / full[:, 129:130]
            res[scheme] = float(np.abs(merged - ref).max() / np.abs(ref).max())
        res["ranges"] = [kv_token_range(n, r, world, 16) for r in range(world)]
        res["units"] = [list(shard_range(7, r, world)) for r in range(world)]
        if rank == 0:
            q.put(res)
    finally:
        dist.destroy_process_group()


def test_kv_split_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + int(np.random.default_rng().integers(0, 2000))
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res["turbo_prod"] < 1e-5 and res["turbo_mse"] < 1e-5
    assert res["ranges"] == [(0, 112), (112, 203)]
    assert res["units"] == [[0, 1, 2, 3], [4, 5, 6]]


def test_shard_helpers():
    from turborag_b200.parallel import kv_token_range, shard_range
    for n in (0, 1, 7, 64, 2304):
        for w in (1, 2, 4, 8):
            got = [i for r in range(w) for i in shard_range(n, r, w)]
            assert got == list(range(n))
    for n in (0, 5, 16, 17, 131072):
        for w in (1, 2, 8):
            rs = [kv_token_range(n, r, w) for r in range(w)]
            assert rs[0][0] == 0 and rs[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(rs, rs[1:]))
            assert all(a % 16 == 0 or a == n for a, _ in rs)
