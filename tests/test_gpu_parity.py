"""Parity of the sm_100a kernels with the CPU oracle and with the reference-made
fixtures, through the C ABI (turborag_b200.TurboQuantWrapper -> libturboquant.so).

Bars: packed codes, sign bits and fp16 scales bit-exact (mismatches are counted and each
must lie within 1 ulp of a decision boundary); dequant output bit-exact; attention
outputs within 2e-3 (max |a-b| over a row / max |b| of the row); logits within 2e-3 of
the largest logit."""
import numpy as np
import pytest
import torch

from tests.conftest import load_golden, rowwise_rel_err
from tests.golden.cases import CASES, make_inputs, make_kv, make_slots
from tests.parity_check import assert_pool_parity

pytestmark = pytest.mark.gpu

ATTN_TOL = 2e-3
SCHEMES = [("turbo_prod", "prod"), ("turbo_mse", "mse")]


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch.device("cuda:0")


def h16(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).to(dev).view(torch.float16)


def cfg_for(tq, h, bs=16):
    cfg = tq.default_config()
    cfg.num_kv_heads, cfg.head_dim, cfg.block_size = h, 128, bs
    return cfg


def gpu_pack(tq, scheme, key, value, slots, cfg, dev, pool_np=None, offset=0):
    lay = tq.layout_for_scheme(scheme, cfg)
    pages = int(slots.max()) // cfg.block_size + 1
    if pool_np is None:
        pool_np = np.zeros(pages * lay.page_size_bytes, np.uint8)
    buf = torch.zeros(pool_np.size + 64, dtype=torch.uint8, device=dev)
    pool = buf[offset:offset + pool_np.size]
    pool.copy_(torch.from_numpy(pool_np))
    fn = tq.pack if scheme == "turbo_prod" else tq.mse_pack
    fn(h16(key, dev), h16(value, dev), torch.from_numpy(slots).to(dev), pool, lay, cfg)
    torch.cuda.synchronize()
    return pool.cpu().numpy()


# ---------------------------------------------------------------------------------
# quantize + pack
# ---------------------------------------------------------------------------------

@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
@pytest.mark.parametrize("scheme,tag", SCHEMES)
def test_pack_matches_reference_fixture_and_oracle(tq, oracle, dev, case, scheme, tag):
    key, value, query, slots = make_inputs(case)
    cfg, ocfg = cfg_for(tq, case["h"]), oracle.make_config(case["h"])
    mine = gpu_pack(tq, scheme, key, value, slots, cfg, dev)
    ref = load_golden(case["name"])[f"{tag}_pool"]
    r = assert_pool_parity(oracle, scheme, mine, ref, key, value, slots, ocfg, case["name"])
    assert r["code_mismatches"] == 0 and r["scale_ulp_max"] == 0  # in fact identical
    assert int((mine != oracle.pack(scheme, key, value, slots, ocfg)).sum()) == 0


@pytest.mark.parametrize("scheme,tag", SCHEMES)
@pytest.mark.parametrize("n,h", [(1, 1), (15, 2), (16, 2), (17, 2), (333, 3), (100, 4), (65, 8), (40, 32)])
def test_pack_ragged_sizes_permuted_slots_untouched_bytes(tq, oracle, dev, scheme, tag, n, h):
    rng = np.random.default_rng(1000 * n + h)
    key, value = make_kv(rng, n, h)
    slots = make_slots(rng, n, True, extra_pages=2)
    cfg, ocfg = cfg_for(tq, h), oracle.make_config(h)
    lay = oracle.layout_for(scheme, ocfg)
    pages = int(slots.max()) // 16 + 1
    canary = np.full(pages * lay.page_size_bytes, 0xA5, np.uint8)
    mine = gpu_pack(tq, scheme, key, value, slots, cfg, dev, pool_np=canary.copy())
    ref = oracle.pack(scheme, key, value, slots, ocfg, pool=canary.copy())
    assert int((mine != ref).sum()) == 0  # includes every byte no token maps to


@pytest.mark.parametrize("scheme,tag", SCHEMES)
def test_pack_pool_not_8_byte_aligned(tq, oracle, dev, scheme, tag):
    rng = np.random.default_rng(5)
    key, value = make_kv(rng, 50, 2)
    slots = make_slots(rng, 50, True)
    mine = gpu_pack(tq, scheme, key, value, slots, cfg_for(tq, 2), dev, offset=2)
    assert int((mine != oracle.pack(scheme, key, value, slots, oracle.make_config(2))).sum()) == 0


@pytest.mark.parametrize("scheme,tag", SCHEMES)
def test_pack_special_values(tq, oracle, dev, scheme, tag):
    """All-zero rows (RMS floor 1e-8), fp16 subnormals, large magnitudes, exact ties at 0."""
    rng = np.random.default_rng(8)
    key, value = make_kv(rng, 32, 2)
    key[0] = 0
    value[1] = 0
    key[2] = np.float16(6e-8)
    value[3] = np.float16(60000.0)
    key[4, :, ::2] = 0
    value[5] = np.float16(1.0)
    slots = np.arange(32, dtype=np.int32)
    mine = gpu_pack(tq, scheme, key, value, slots, cfg_for(tq, 2), dev)
    assert int((mine != oracle.pack(scheme, key, value, slots, oracle.make_config(2))).sum()) == 0


@pytest.mark.parametrize("scheme,tag", SCHEMES)
def test_pack_full_store_unit(tq, oracle, dev, scheme, tag):
    """One (layer, document) unit of the offline store build: 8192 tokens x 2 kv heads."""
    rng = np.random.default_rng(2024)
    key, value = make_kv(rng, 8192, 2)
    slots = make_slots(rng, 8192, True)
    mine = gpu_pack(tq, scheme, key, value, slots, cfg_for(tq, 2), dev)
    ref = oracle.pack(scheme, key, value, slots, oracle.make_config(2))
    r = assert_pool_parity(oracle, scheme, mine, ref, key, value, slots, oracle.make_config(2), "8192x2x128")
    assert r["code_mismatches"] == 0


@pytest.mark.parametrize("scheme,tag", SCHEMES)
def test_pack_large_outlier_rows_identical_pool(tq, oracle, dev, scheme, tag):
    """32768 tokens x 2 kv heads with two outlier channels: every byte of the pool, the fp16 scales
    included, equals the oracle's.  Sums of squares that are off in their last fp32 bit (a fused
    multiply-add where the reference multiplies and adds) show up here as a handful of scale
    bytes, which smaller cases miss."""
    rng = np.random.default_rng(32768)
    key, value = make_kv(rng, 32768, 2)
    key[:, :, [5, 77]] *= 6
    slots = make_slots(rng, 32768, True)
    mine = gpu_pack(tq, scheme, key, value, slots, cfg_for(tq, 2), dev)
    ref = oracle.pack(scheme, key, value, slots, oracle.make_config(2))
    assert int((mine != ref).sum()) == 0


def test_pack_block_size_other_than_16(tq, oracle, dev):
    rng = np.random.default_rng(77)
    key, value = make_kv(rng, 40, 2)
    for bs in (8, 32, 5):
        cfg, ocfg = cfg_for(tq, 2, bs), oracle.make_config(2)
        ocfg.block_size = bs
        slots = make_slots(rng, 40, True, block=bs)
        for scheme, _ in SCHEMES:
            mine = gpu_pack(tq, scheme, key, value, slots, cfg, dev)
            assert int((mine != oracle.pack(scheme, key, value, slots, ocfg)).sum()) == 0


def test_pack_rejects_misaligned_input(tq, dev):
    cfg = cfg_for(tq, 2)
    lay = tq.make_layout_for(cfg)
    raw = torch.zeros(4 * 2 * 128 + 8, dtype=torch.float16, device=dev)
    key = raw[1:1 + 4 * 2 * 128].view(4, 2, 128)  # 2-byte aligned only
    good = torch.zeros(4, 2, 128, dtype=torch.float16, device=dev)
    pool = torch.zeros(lay.page_size_bytes, dtype=torch.uint8, device=dev)
    with pytest.raises(RuntimeError, match="16-byte aligned"):
        tq.pack(key, good, torch.arange(4, dtype=torch.int32, device=dev), pool, lay, cfg)


# ---------------------------------------------------------------------------------
# dequant
# ---------------------------------------------------------------------------------

def gpu_dequant(tq, scheme, pool_np, slots, cfg, dev, hnd=False):
    lay = tq.layout_for_scheme(scheme, cfg)
    n, h = slots.shape[0], cfg.num_kv_heads
    shape = (h, n, 128) if hnd else (n, h, 128)
    ok = torch.full(shape, 7.0, dtype=torch.float16, device=dev)
    ov = torch.full(shape, 7.0, dtype=torch.float16, device=dev)
    pool = torch.from_numpy(pool_np).to(dev)
    s = torch.from_numpy(slots).to(dev)
    if hnd:
        tq.dequant_hnd(scheme, pool, s, ok, ov, lay, cfg)
    else:
        (tq.dequant if scheme == "turbo_prod" else tq.mse_dequant)(pool, s, ok, ov, lay, cfg)
    torch.cuda.synchronize()
    return ok.cpu().numpy(), ov.cpu().numpy()


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
@pytest.mark.parametrize("scheme,tag", SCHEMES)
def test_dequant_bit_exact(tq, oracle, dev, case, scheme, tag):
    key, value, query, slots = make_inputs(case)
    z = load_golden(case["name"])
    cfg, ocfg = cfg_for(tq, case["h"]), oracle.make_config(case["h"])
    k, v = gpu_dequant(tq, scheme, z[f"{tag}_pool"], slots, cfg, dev)
    rk, rv = oracle.dequant(scheme, z[f"{tag}_pool"], slots, ocfg)
    assert (k.view(np.uint16) == rk.view(np.uint16)).all() and (v.view(np.uint16) == rv.view(np.uint16)).all()
    keep = z[f"{tag}_dequant_key_head"].shape[0]
    assert (k.view(np.uint16)[:keep] == z[f"{tag}_dequant_key_head"]).all()  # the reference's own output
    assert (v.view(np.uint16)[:keep] == z[f"{tag}_dequant_value_head"]).all()
    hk, hv = gpu_dequant(tq, scheme, z[f"{tag}_pool"], slots, cfg, dev, hnd=True)
    assert (hk.transpose(1, 0, 2) == k).all() and (hv.transpose(1, 0, 2) == v).all()


@pytest.mark.parametrize("scheme,tag", SCHEMES)
@pytest.mark.parametrize("n,h", [(1, 1), (17, 3), (333, 4), (8192, 2)])
def test_dequant_random_pages_and_roundtrip_quality(tq, oracle, dev, scheme, tag, n, h):
    rng = np.random.default_rng(31 * n + h)
    key, value = make_kv(rng, n, h)
    slots = make_slots(rng, n, True, extra_pages=1)
    cfg, ocfg = cfg_for(tq, h), oracle.make_config(h)
    pool = gpu_pack(tq, scheme, key, value, slots, cfg, dev)
    k, v = gpu_dequant(tq, scheme, pool, slots, cfg, dev)
    rk, rv = oracle.dequant(scheme, pool, slots, ocfg)
    assert (k.view(np.uint16) == rk.view(np.uint16)).all() and (v.view(np.uint16) == rv.view(np.uint16)).all()
    # the reference suite's own acceptance bound (tests/test_cag.py:212-246) and a tight one
    for a, b in ((key, k), (value, v)):
        rel = np.mean((a.astype(np.float32) - b.astype(np.float32)) ** 2) / (np.var(a.astype(np.float32)) + 1e-8)
        assert rel < (0.35 if scheme == "turbo_prod" else 0.25) and (n < 16 or rel < 0.02)


def test_debug_pack_dumps_the_oracle_intermediates(tq, oracle, dev):
    """tq_debug_turbo_prod_pack_kv: the pool of the regular pack, plus the normalised values the
    oracle traces (bit-identical) and level indices that are the packed nibbles."""
    rng = np.random.default_rng(21)
    n, h = 77, 2
    key, value = make_kv(rng, n, h)
    slots = make_slots(rng, n, True, extra_pages=1)
    cfg, ocfg = cfg_for(tq, h), oracle.make_config(h)
    lay = tq.make_layout_for(cfg)
    pool_o, kn_o, vn_o = oracle.pack("turbo_prod", key, value, slots, ocfg, trace=True)
    pool = torch.zeros(pool_o.size, dtype=torch.uint8, device=dev)
    d = tq.debug_pack(h16(key, dev), h16(value, dev), torch.from_numpy(slots).to(dev), pool, lay, cfg)
    torch.cuda.synchronize()
    assert np.array_equal(pool.cpu().numpy(), pool_o)
    assert np.array_equal(d["kn"].cpu().numpy(), np.clip(kn_o, -2.5, 2.5))
    assert np.array_equal(d["vn"].cpu().numpy(), np.clip(vn_o, -2.75, 2.75))
    # indices against the levels: nearest level of the normalised value
    cb3, cb4 = oracle.cb3(), oracle.cb4()
    assert np.array_equal(d["kidx"].cpu().numpy(), np.abs(np.clip(kn_o, -2.5, 2.5)[..., None] - cb3).argmin(-1))
    assert np.array_equal(d["vidx"].cpu().numpy(), np.abs(np.clip(vn_o, -2.75, 2.75)[..., None] - cb4).argmin(-1))
    # rotated values: the oracle's normalised value times the stored scale reproduces them to fp16 precision of the scale
    assert np.isfinite(d["k_rot"].cpu().numpy()).all() and np.isfinite(d["v_rot"].cpu().numpy()).all()


# ---------------------------------------------------------------------------------
# fused attention, reference API (one sequence, per-token slots, query [Q, H, D])
# ---------------------------------------------------------------------------------

def gpu_attn(tq, scheme, query, pool_np, slots, cfg, dev):
    lay = tq.layout_for_scheme(scheme, cfg)
    nq = query.shape[0]
    out = torch.full(query.shape, 9.0, dtype=torch.float16, device=dev)
    fn = tq.fused_attn_output if scheme == "turbo_prod" else tq.mse_fused_attn_output
    fn(h16(query, dev), torch.from_numpy(pool_np).to(dev), torch.from_numpy(slots).to(dev), out, lay,
       cfg, nq, slots.shape[0])
    torch.cuda.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
@pytest.mark.parametrize("scheme,tag", SCHEMES)
def test_fused_attention_vs_oracle_and_reference(tq, oracle, dev, case, scheme, tag):
    key, value, query, slots = make_inputs(case)
    z = load_golden(case["name"])
    cfg, ocfg = cfg_for(tq, case["h"]), oracle.make_config(case["h"])
    out = gpu_attn(tq, scheme, query, z[f"{tag}_pool"], slots, cfg, dev)
    e_or = rowwise_rel_err(out, oracle.attn(scheme, query, z[f"{tag}_pool"], slots, ocfg))
    e_ref = rowwise_rel_err(out, z[f"{tag}_attn"].view(np.float16))
    print(f"{case['name']} {scheme}: rel err vs oracle {e_or:.2e}, vs reference kernel {e_ref:.2e}")
    assert e_or < ATTN_TOL and e_ref < ATTN_TOL


@pytest.mark.parametrize("scheme,tag", SCHEMES)
@pytest.mark.parametrize("n,h,nq", [(1, 2, 1), (16, 2, 1), (17, 1, 2), (700, 4, 7), (300, 2, 11), (5000, 2, 8), (64, 8, 3)])
def test_fused_attention_shapes(tq, oracle, dev, scheme, tag, n, h, nq):
    rng = np.random.default_rng(17 * n + nq)
    key, value = make_kv(rng, n, h)
    query = rng.standard_normal((nq, h, 128)).astype(np.float16)
    slots = make_slots(rng, n, True, extra_pages=1)
    ocfg = oracle.make_config(h)
    pool = oracle.pack(scheme, key, value, slots, ocfg)
    out = gpu_attn(tq, scheme, query, pool, slots, cfg_for(tq, h), dev)
    assert rowwise_rel_err(out, oracle.attn(scheme, query, pool, slots, ocfg)) < ATTN_TOL


def test_fused_attention_token_order_scattered_slots(tq, oracle, dev):
    """slot_mapping is per token: tokens of one sequence may sit in any slot of any page."""
    rng = np.random.default_rng(99)
    n, h = 100, 2
    key, value = make_kv(rng, n, h)
    slots = rng.permutation(16 * 9)[:n].astype(np.int32)
    query = rng.standard_normal((2, h, 128)).astype(np.float16)
    ocfg = oracle.make_config(h)
    for scheme, _ in SCHEMES:
        pool = gpu_pack(tq, scheme, key, value, slots, cfg_for(tq, h), dev)
        assert int((pool != oracle.pack(scheme, key, value, slots, ocfg)).sum()) == 0
        out = gpu_attn(tq, scheme, query, pool, slots, cfg_for(tq, h), dev)
        assert rowwise_rel_err(out, oracle.attn(scheme, query, pool, slots, ocfg)) < ATTN_TOL


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_logits_vs_oracle_and_reference(tq, oracle, dev, case):
    key, value, query, slots = make_inputs(case)
    z = load_golden(case["name"])
    cfg = cfg_for(tq, case["h"])
    lay = tq.make_layout_for(cfg)
    n, nq, h = case["n"], case["nq"], case["h"]
    lg = torch.full((nq * h * n,), 5.0, dtype=torch.float32, device=dev)
    tq.fused_attn_logits(h16(query, dev), torch.from_numpy(z["prod_pool"]).to(dev),
                         torch.from_numpy(slots).to(dev), lg, lay, cfg, nq, n)
    torch.cuda.synchronize()
    mine = lg.cpu().numpy().reshape(nq, h, n)
    ref = oracle.prod_logits(query, z["prod_pool"], slots, oracle.make_config(h))
    scale = np.abs(ref).max()
    assert np.abs(mine - ref).max() < 2e-3 * scale
    assert np.abs(mine - z["prod_logits"]).max() < 2e-3 * scale


# ---------------------------------------------------------------------------------
# batched paged GQA decode, split-KV partials and merge
# ---------------------------------------------------------------------------------

def build_paged(oracle, scheme, rng, lens, h, extra=3):
    maxpages = max(1, (max(lens) + 15) // 16)
    b = len(lens)
    total = b * maxpages + extra
    tables = rng.permutation(total).astype(np.int32)[:b * maxpages].reshape(b, maxpages)
    ocfg = oracle.make_config(h)
    lay = oracle.layout_for(scheme, ocfg)
    pool = np.zeros(total * lay.page_size_bytes, np.uint8)
    for i, n in enumerate(lens):
        if n:
            k, v = make_kv(rng, n, h)
            t = np.arange(n)
            oracle.pack(scheme, k, v, (tables[i][t // 16] * 16 + t % 16).astype(np.int32), ocfg, pool=pool)
    return pool, tables


@pytest.mark.parametrize("scheme,tag", SCHEMES)
@pytest.mark.parametrize("hq,h,lens", [(16, 2, [1143, 16, 700, 1]), (28, 4, [333, 64]), (8, 8, [100, 5]),
                                       (4, 2, [0, 40]), (32, 2, [257]), (2, 2, [4096, 4095, 31]),
                                       (8, 1, [77, 300, 2049])])
def test_decode_paged_vs_oracle(tq, oracle, dev, scheme, tag, hq, h, lens):
    rng = np.random.default_rng(sum(lens) + hq)
    pool, tables = build_paged(oracle, scheme, rng, lens, h)
    b = len(lens)
    query = rng.standard_normal((b, hq, 128)).astype(np.float16)
    cfg = cfg_for(tq, h)
    lay = tq.layout_for_scheme(scheme, cfg)
    out = tq.decode_paged(scheme, h16(query, dev), torch.from_numpy(pool).to(dev),
                          torch.from_numpy(tables).to(dev), torch.tensor(lens, dtype=torch.int32, device=dev),
                          lay, cfg, max_kv_tokens=max(max(lens), 1))
    torch.cuda.synchronize()
    mine = out.cpu().numpy()
    ref = oracle.decode_paged(scheme, query, pool, tables, lens, oracle.make_config(h))
    for i, n in enumerate(lens):
        if n == 0:
            assert (mine[i] == 0).all()  # l == 0 -> zeros (tq_turbo_prod_kernels.cu:561-564)
        else:
            assert rowwise_rel_err(mine[i], ref[i]) < ATTN_TOL


@pytest.mark.parametrize("scheme,tag", SCHEMES)
def test_partials_of_token_ranges_merge_to_full_attention(tq, oracle, dev, scheme, tag):
    """What the multi-GPU KV split does, on one device: partials of disjoint token ranges,
    stacked like an all-gather result, merged by tq_merge_partials."""
    rng = np.random.default_rng(4242)
    lens, hq, h = [1000, 517], 14, 2
    pool, tables = build_paged(oracle, scheme, rng, lens, h)
    b = len(lens)
    query = rng.standard_normal((b, hq, 128)).astype(np.float16)
    cfg = cfg_for(tq, h)
    lay = tq.layout_for_scheme(scheme, cfg)
    args = (h16(query, dev), torch.from_numpy(pool).to(dev), torch.from_numpy(tables).to(dev),
            torch.tensor(lens, dtype=torch.int32, device=dev), lay, cfg)
    from turborag_b200.parallel import kv_token_range
    world = 3
    parts = torch.zeros(world, b * hq, 130, dtype=torch.float32, device=dev)
    for r in range(world):
        lo, hi = kv_token_range(max(lens), r, world, 16)
        tq.decode_paged(scheme, *args, partials_out=parts[r].view(b, hq, 130), max_kv_tokens=max(lens),
                        kv_begin=lo, kv_end=hi)
    out = torch.zeros(b * hq, 128, dtype=torch.float16, device=dev)
    tq.merge_partials(parts, out, hq, h)
    full = tq.decode_paged(scheme, *args, max_kv_tokens=max(lens))
    torch.cuda.synchronize()
    ref = oracle.decode_paged(scheme, query, pool, tables, lens, oracle.make_config(h))
    assert rowwise_rel_err(out.cpu().numpy().reshape(b, hq, 128), ref) < ATTN_TOL
    assert rowwise_rel_err(full.cpu().numpy(), ref) < ATTN_TOL
    # a partial is (acc, m, l) in the rotated domain: compare one range with the oracle's state
    lo, hi = kv_token_range(max(lens), 0, world, 16)
    t = np.arange(lo, min(hi, lens[0]))
    st = oracle.attn_state(scheme, oracle.gqa_to_ref_query(query[0], h), pool,
                           (tables[0][t // 16] * 16 + t % 16).astype(np.int32), oracle.make_config(h))
    mine = parts[0].view(b, hq, 130)[0].cpu().numpy()  # rows h*G+g
    g = hq // h
    for hh in range(h):
        for gg in range(g):
            a, r_ = mine[hh * g + gg], st[gg, hh]
            # the reference m of a record may sit up to 1.5 ln 2 below the largest logit (the kernel
            # keeps it while a block stays within 2^1.5 of it); m + log(l) does not depend on it
            tol_m = 2e-3 * max(1.0, abs(r_[128]))
            assert -tol_m < r_[128] - a[128] < 1.5 * np.log(2) + tol_m
            lse_a, lse_r = a[128] + np.log(a[129]), r_[128] + np.log(r_[129])
            assert abs(lse_a - lse_r) < 2e-3 * max(1.0, abs(lse_r))
            na, nr = a[:128] / a[129], r_[:128] / r_[129]
            assert np.abs(na - nr).max() < ATTN_TOL * np.abs(nr).max()


def test_decode_long_sequence_full_size(tq, oracle, dev):
    """One sequence of the decode benchmark shape: 32768 cached tokens, 16 q heads / 2 kv heads."""
    rng = np.random.default_rng(32768)
    n, hq, h = 32768, 16, 2
    cfg, ocfg = cfg_for(tq, h), oracle.make_config(h)
    lay = tq.make_layout_for(cfg)
    key, value = make_kv(rng, n, h)
    tables = rng.permutation(n // 16).astype(np.int32)[None, :]
    t = np.arange(n)
    slots = (tables[0][t // 16] * 16 + t % 16).astype(np.int32)
    pool = gpu_pack(tq, "turbo_prod", key, value, slots, cfg, dev)
    query = rng.standard_normal((1, hq, 128)).astype(np.float16)
    out = tq.decode_paged("turbo_prod", h16(query, dev), torch.from_numpy(pool).to(dev),
                          torch.from_numpy(tables).to(dev), torch.tensor([n], dtype=torch.int32, device=dev),
                          lay, cfg, max_kv_tokens=n)
    torch.cuda.synchronize()
    ref = oracle.decode_paged("turbo_prod", query, pool, tables, [n], ocfg)
    err = rowwise_rel_err(out.cpu().numpy(), ref)
    print(f"32768-token decode: rel err {err:.2e}")
    assert err < ATTN_TOL


def test_decode_workspace_argument(tq, oracle, dev):
    rng = np.random.default_rng(3)
    lens, hq, h = [600, 900], 8, 2
    pool, tables = build_paged(oracle, "turbo_prod", rng, lens, h)
    query = rng.standard_normal((2, hq, 128)).astype(np.float16)
    cfg = cfg_for(tq, h)
    lay = tq.make_layout_for(cfg)
    args = ("turbo_prod", h16(query, dev), torch.from_numpy(pool).to(dev), torch.from_numpy(tables).to(dev),
            torch.tensor(lens, dtype=torch.int32, device=dev), lay, cfg)
    ws = torch.empty(tq.decode_workspace_bytes(2, hq, 900, cfg), dtype=torch.uint8, device=dev)
    a = tq.decode_paged(*args, max_kv_tokens=900, workspace=ws)
    b = tq.decode_paged(*args, max_kv_tokens=900)
    torch.cuda.synchronize()
    assert (a == b).all()
    with pytest.raises(RuntimeError, match="workspace too small"):
        tq.decode_paged(*args, max_kv_tokens=900, workspace=ws[:128])
    with pytest.raises(RuntimeError, match="narrower"):
        tq.decode_paged(*args, max_kv_tokens=16 * tables.shape[1] + 1)


# ---------------------------------------------------------------------------------
# chunked query prefill over a turbo_mse prefix + causal fp16 chunk
# ---------------------------------------------------------------------------------

@pytest.mark.parametrize("hq,h,nq,lens,with_chunk", [
    (16, 2, 1, [100, 37], True), (16, 2, 20, [333, 64], True), (16, 2, 70, [1000], True),
    (8, 4, 33, [129, 5], True), (16, 2, 24, [500, 17], False), (4, 2, 130, [64], True),
    (8, 8, 9, [40], True), (16, 2, 16, [0, 50], True)])
def test_mse_prefill_vs_oracle(tq, oracle, dev, hq, h, nq, lens, with_chunk):
    rng = np.random.default_rng(1000 * nq + sum(lens) + hq)
    pool, tables = build_paged(oracle, "turbo_mse", rng, lens, h)
    b = len(lens)
    query = rng.standard_normal((b, nq, hq, 128)).astype(np.float16)
    ck = rng.standard_normal((b, nq, h, 128)).astype(np.float16) if with_chunk else None
    cv = rng.standard_normal((b, nq, h, 128)).astype(np.float16) if with_chunk else None
    if with_chunk:
        ck[:, :, :, [3, 17]] *= 8
    cfg, ocfg = cfg_for(tq, h), oracle.make_config(h)
    lay = tq.make_mse_layout_for(cfg)
    out = torch.full((b, nq, hq, 128), 3.0, dtype=torch.float16, device=dev)
    tq.mse_prefill_paged(h16(query, dev), torch.from_numpy(pool).to(dev), torch.from_numpy(tables).to(dev),
                         torch.tensor(lens, dtype=torch.int32, device=dev),
                         None if ck is None else h16(ck, dev), None if cv is None else h16(cv, dev),
                         out, lay, cfg)
    torch.cuda.synchronize()
    mine = out.cpu().numpy()
    for i, n in enumerate(lens):
        t = np.arange(n)
        slots = (tables[i][t // 16] * 16 + t % 16).astype(np.int32)
        if n == 0 and not with_chunk:
            continue
        ref = oracle.mse_prefill(query[i], pool, slots, None if ck is None else ck[i],
                                 None if cv is None else cv[i], ocfg)
        err = rowwise_rel_err(mine[i], ref)
        print(f"prefill b={i} n={n} nq={nq}: rel err {err:.2e}")
        assert err < ATTN_TOL
    assert tq.mse_prefill_status() == 0, "a bounded wait inside the prefill kernel ran out"
