"""Parity at the sizes the benchmark runs, through the C ABI, against the CPU oracle.

The small-shape tests in test_gpu_parity.py cover the edge cases; these cover what only shows at
size: the split counts, row tiles and stream lengths of the benchmark shapes, and the spread of the
attention error over seeds.  Pools are packed on the GPU (pack parity is held bit-exact elsewhere)
and read by both sides; tolerance 2e-3 of the row maximum, as everywhere."""
import numpy as np
import pytest
import torch

from tests.conftest import rowwise_rel_err

pytestmark = pytest.mark.gpu

ATTN_TOL = 2e-3
OUTLIERS = (3, 17, 64, 101)


def synth_kv(n, h, dev, gen):
    scale = torch.ones(128, device=dev)
    scale[list(OUTLIERS)] = 8.0
    k = (torch.randn(n, h, 128, device=dev, generator=gen) * scale).to(torch.float16)
    v = torch.randn(n, h, 128, device=dev, generator=gen).to(torch.float16)
    return k, v


def build_pool(tq, scheme, batch, n, h, dev, gen):
    """`batch` sequences of `n` tokens in one pool, pages permuted over the whole pool."""
    cfg = tq.default_config()
    cfg.num_kv_heads = h
    lay = tq.layout_for_scheme(scheme, cfg)
    pages = batch * (n // 16)
    pool = torch.zeros(pages * lay.page_size_bytes, dtype=torch.uint8, device=dev)
    tables = torch.randperm(pages, device=dev, generator=gen).to(torch.int32).view(batch, n // 16).contiguous()
    t = torch.arange(n, device=dev)
    pack = tq.pack if scheme == "turbo_prod" else tq.mse_pack
    for b in range(batch):
        k, v = synth_kv(n, h, dev, gen)
        pack(k, v, (tables[b][t // 16].to(torch.int64) * 16 + t % 16).to(torch.int32), pool, lay, cfg)
    return pool, tables, lay, cfg


def test_decode_benchmark_shape_over_seeds(tq, oracle):
    """Config 3 (32 sequences x 32768 tokens, 16 q / 2 kv heads, turbo_prod), 8 seeds: the worst row
    over all seeds stays inside the tolerance (printed, so the margin is on record)."""
    dev = torch.device("cuda:0")
    b, n, hq, h = 32, 32768, 16, 2
    ocfg = oracle.make_config(h)
    worst = []
    for seed in range(8):
        gen = torch.Generator(device=dev)
        gen.manual_seed(1000 + seed)
        pool, tables, lay, cfg = build_pool(tq, "turbo_prod", b, n, h, dev, gen)
        q = torch.randn(b, hq, 128, device=dev, generator=gen).to(torch.float16)
        lens = torch.full((b,), n, dtype=torch.int32, device=dev)
        out = tq.decode_paged("turbo_prod", q, pool, tables, lens, lay, cfg, max_kv_tokens=n)
        torch.cuda.synchronize()
        ref = oracle.decode_paged("turbo_prod", q.cpu().numpy(), pool.cpu().numpy(), tables.cpu().numpy(),
                                  [n] * b, ocfg)
        worst.append(rowwise_rel_err(out.cpu().numpy(), ref))
        del pool
    print("decode 32x32768, worst row error per seed:", " ".join(f"{e:.2e}" for e in worst))
    assert max(worst) < ATTN_TOL


def test_long_context_shape_whole_and_as_eight_ranges(tq, oracle):
    """Config 5's per-sequence shape: 131072 cached tokens, 28 q / 4 kv heads, turbo_prod -- decoded
    whole, and as eight contiguous token ranges (what eight ranks hold) merged by tq_merge_partials."""
    from turborag_b200.parallel import kv_token_range
    dev = torch.device("cuda:0")
    n, hq, h, world = 131072, 28, 4, 8
    gen = torch.Generator(device=dev)
    gen.manual_seed(77)
    pool, tables, lay, cfg = build_pool(tq, "turbo_prod", 1, n, h, dev, gen)
    q = torch.randn(1, hq, 128, device=dev, generator=gen).to(torch.float16)
    lens = torch.tensor([n], dtype=torch.int32, device=dev)
    whole = tq.decode_paged("turbo_prod", q, pool, tables, lens, lay, cfg, max_kv_tokens=n)
    parts = torch.zeros(world, hq, 130, dtype=torch.float32, device=dev)
    for r in range(world):
        lo, hi = kv_token_range(n, r, world, 16)
        tq.decode_paged("turbo_prod", q, pool, tables, lens, lay, cfg, partials_out=parts[r].view(1, hq, 130),
                        max_kv_tokens=n, kv_begin=lo, kv_end=hi)
    merged = torch.zeros(hq, 128, dtype=torch.float16, device=dev)
    tq.merge_partials(parts, merged, hq, h)
    torch.cuda.synchronize()
    ref = oracle.decode_paged("turbo_prod", q.cpu().numpy(), pool.cpu().numpy(), tables.cpu().numpy(), [n],
                              oracle.make_config(h))
    e_whole = rowwise_rel_err(whole.cpu().numpy(), ref)
    e_split = rowwise_rel_err(merged.cpu().numpy()[None], ref)
    print(f"131072 tokens, 28q/4kv: whole {e_whole:.2e}, eight ranges merged {e_split:.2e}")
    assert e_whole < ATTN_TOL and e_split < ATTN_TOL


def test_prefill_benchmark_shape_sampled_rows(tq, oracle):
    """Config 4 (8 sequences x 256 query tokens over a 32768-token turbo_mse prefix, 16 q / 2 kv heads):
    64 query tokens per sequence -- four in every 16-token row tile, all 16 query heads of each, so
    both kv heads and every row tile of every sequence -- against the oracle's fp32 attention over
    [prefix ; causal chunk]."""
    dev = torch.device("cuda:0")
    b, nq, n, hq, h = 8, 256, 32768, 16, 2
    gen = torch.Generator(device=dev)
    gen.manual_seed(4)
    pool, tables, lay, cfg = build_pool(tq, "turbo_mse", b, n, h, dev, gen)
    q = torch.randn(b, nq, hq, 128, device=dev, generator=gen).to(torch.float16)
    ck, cv = synth_kv(b * nq, h, dev, gen)
    ck, cv = ck.view(b, nq, h, 128), cv.view(b, nq, h, 128)
    lens = torch.full((b,), n, dtype=torch.int32, device=dev)
    out = torch.full((b, nq, hq, 128), 3.0, dtype=torch.float16, device=dev)
    tq.mse_prefill_paged(q, pool, tables, lens, ck, cv, out, lay, cfg)
    torch.cuda.synchronize()
    assert tq.mse_prefill_status() == 0, "a bounded wait inside the prefill kernel ran out"
    pool_h, tab_h = pool.cpu().numpy(), tables.cpu().numpy()
    q_h, ck_h, cv_h, out_h = q.cpu().numpy(), ck.cpu().numpy(), cv.cpu().numpy(), out.cpu().numpy()
    rng = np.random.default_rng(9)
    ocfg = oracle.make_config(h)
    t = np.arange(n)
    worst = 0.0
    for i in range(b):
        rows = np.sort(np.concatenate([16 * tile + rng.choice(16, 4, replace=False) for tile in range(nq // 16)]))
        rows[0], rows[-1] = 0, nq - 1  # first row sees one chunk token, last row all of them
        slots = (tab_h[i][t // 16].astype(np.int64) * 16 + t % 16).astype(np.int32)
        ref = oracle.mse_prefill(q_h[i], pool_h, slots, ck_h[i], cv_h[i], ocfg, rows=rows)
        worst = max(worst, rowwise_rel_err(out_h[i][rows], ref))
    print(f"prefill 8x256x32768: worst sampled row error {worst:.2e}")
    assert worst < ATTN_TOL


@pytest.mark.parametrize("scheme", ["turbo_prod", "turbo_mse"])
def test_attention_with_sixteen_kv_heads(tq, oracle, scheme):
    """More kv heads than one CTA serves (8): the reference-API attention and the paged decode run one
    launch per group of 8 heads and give the oracle's result for every head."""
    dev = torch.device("cuda:0")
    n, h, nq = 700, 16, 3
    rng = np.random.default_rng(16)
    key = rng.standard_normal((n, h, 128)).astype(np.float16)
    value = rng.standard_normal((n, h, 128)).astype(np.float16)
    query = rng.standard_normal((nq, h, 128)).astype(np.float16)
    slots = (rng.permutation(-(-n // 16) + 2)[:-(-n // 16)].repeat(16)[:n] * 16 + np.arange(n) % 16).astype(np.int32)
    ocfg = oracle.make_config(h)
    pool = oracle.pack(scheme, key, value, slots, ocfg)
    cfg = tq.default_config()
    cfg.num_kv_heads = h
    lay = tq.layout_for_scheme(scheme, cfg)
    out = torch.full((nq, h, 128), 9.0, dtype=torch.float16, device=dev)
    fn = tq.fused_attn_output if scheme == "turbo_prod" else tq.mse_fused_attn_output
    qd = torch.from_numpy(query.view(np.int16)).to(dev).view(torch.float16)
    fn(qd, torch.from_numpy(pool).to(dev), torch.from_numpy(slots).to(dev), out, lay, cfg, nq, n)
    torch.cuda.synchronize()
    assert rowwise_rel_err(out.cpu().numpy(), oracle.attn(scheme, query, pool, slots, ocfg)) < ATTN_TOL
    if scheme == "turbo_prod":
        lg = torch.zeros(nq * h * n, dtype=torch.float32, device=dev)
        tq.fused_attn_logits(qd, torch.from_numpy(pool).to(dev), torch.from_numpy(slots).to(dev), lg, lay, cfg, nq, n)
        torch.cuda.synchronize()
        ref = oracle.prod_logits(query, pool, slots, ocfg)
        assert np.abs(lg.cpu().numpy().reshape(nq, h, n) - ref).max() < 2e-3 * np.abs(ref).max()
