"""The CPU oracle against (1) fixtures produced by the reference's own kernels on a
B200 (tests/golden/*.npz, made by tests/golden/make_golden.py), (2) the reference's
host code where oracle/_ref was built, (3) known answers derived from the reference
sources.  No GPU needed."""
import ctypes as C
import hashlib
import re
from pathlib import Path

import numpy as np
import pytest

from tests.conftest import load_golden, rowwise_rel_err
from tests.golden.cases import CASES, make_inputs

ROOT = Path(__file__).resolve().parent.parent
CASE_IDS = [c["name"] for c in CASES]


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.fixture(params=CASES, ids=CASE_IDS)
def case(request):
    c = request.param
    z = load_golden(c["name"])
    key, value, query, slots = make_inputs(c)
    # the seeded generator must reproduce the inputs the fixture was made from
    assert sha(key) == str(z["key_sha"]) and sha(value) == str(z["value_sha"])
    assert sha(query) == str(z["query_sha"]) and (slots == z["slots"]).all()
    return c, z, key, value, query, slots


@pytest.mark.parametrize("scheme,tag", [("turbo_prod", "prod"), ("turbo_mse", "mse")])
def test_pack_bit_exact_vs_reference(oracle, case, scheme, tag):
    c, z, key, value, query, slots = case
    pool = oracle.pack(scheme, key, value, slots, oracle.make_config(c["h"]))
    ref = z[f"{tag}_pool"]
    assert pool.shape == ref.shape
    assert int((pool != ref).sum()) == 0  # codes, sign bits and fp16 scales, padding untouched


@pytest.mark.parametrize("scheme,tag", [("turbo_prod", "prod"), ("turbo_mse", "mse")])
def test_dequant_bit_exact_vs_reference(oracle, case, scheme, tag):
    c, z, key, value, query, slots = case
    k, v = oracle.dequant(scheme, z[f"{tag}_pool"], slots, oracle.make_config(c["h"]))
    keep = z[f"{tag}_dequant_key_head"].shape[0]
    assert (k.view(np.uint16)[:keep] == z[f"{tag}_dequant_key_head"]).all()
    assert (v.view(np.uint16)[:keep] == z[f"{tag}_dequant_value_head"]).all()
    assert sha(k.view(np.uint16)) == str(z[f"{tag}_dequant_sha"][0])
    assert sha(v.view(np.uint16)) == str(z[f"{tag}_dequant_sha"][1])


@pytest.mark.parametrize("scheme,tag", [("turbo_prod", "prod"), ("turbo_mse", "mse")])
def test_fused_attention_vs_reference(oracle, case, scheme, tag):
    c, z, key, value, query, slots = case
    out = oracle.attn(scheme, query, z[f"{tag}_pool"], slots, oracle.make_config(c["h"]))
    ref = z[f"{tag}_attn"].view(np.float16)
    # same fp32 algorithm; the GPU's expf and fused multiply-adds leave at most a
    # couple of fp16 last-place differences
    assert rowwise_rel_err(out, ref) < 5e-4
    assert (out.view(np.uint16) != ref.view(np.uint16)).mean() < 0.02


def test_logits_vs_reference(oracle, case):
    c, z, key, value, query, slots = case
    lg = oracle.prod_logits(query, z["prod_pool"], slots, oracle.make_config(c["h"]))
    ref = z["prod_logits"]
    assert np.abs(lg - ref).max() <= 4e-6 * max(1.0, np.abs(ref).max())


def test_rsqrt_constant_matches_gpu(oracle):
    z = load_golden("small_h2")
    assert int(z["rsqrt128_bits"][0]) == oracle.lib().orc_inv_sqrt_d_bits() == 0x3DB504F2


# ---- layouts -------------------------------------------------------------------

def test_layout_known_numbers(oracle):
    # values measured from the built reference (src/tq_turbo_prod.cpp, tq_turbo_mse_layout.cpp)
    p = oracle.prod_layout(oracle.make_config(2))
    assert (p.page_size_bytes, p.k4_codes_offset, p.k_residual_scales_offset, p.k_scales_offset,
            p.v4_codes_offset, p.v_scales_offset) == (4288, 0, 2048, 2112, 2176, 4224)
    assert (p.k4_bytes_per_token_head, p.v4_bytes_per_token_head, p.scale_bytes_per_token_head) == (64, 64, 2)
    p4 = oracle.prod_layout(oracle.make_config(4))
    assert (p4.page_size_bytes, p4.k_residual_scales_offset, p4.k_scales_offset, p4.v4_codes_offset,
            p4.v_scales_offset) == (8576, 4096, 4224, 4352, 8448)
    m = oracle.mse_layout(oracle.make_config(2))
    assert (m.page_size_bytes, m.k_codes_offset, m.v_codes_offset, m.k_norms_offset,
            m.v_norms_offset) == (4608, 0, 2048, 4096, 4352)
    m4 = oracle.mse_layout(oracle.make_config(4))
    assert (m4.page_size_bytes, m4.v_codes_offset, m4.k_norms_offset, m4.v_norms_offset) == (8704, 4096, 8192, 8448)
    assert C.sizeof(oracle.Config) == 32 and C.sizeof(oracle.ProdLayout) == 64 and C.sizeof(oracle.MseLayout) == 56


def test_layouts_vs_reference_host_code(oracle):
    ref = oracle.ref_host()
    if ref is None:
        pytest.skip("oracle/_ref not built (reference tree absent)")
    for h in (1, 2, 3, 4, 8, 32):
        for bs in (1, 8, 16, 32):
            for d in (64, 128):
                cfg = oracle.make_config(h, d)
                cfg.block_size = bs
                a, b = oracle.ProdLayout(), oracle.MseLayout()
                ref.ref_prod_layout(C.byref(cfg), C.byref(a))
                ref.ref_mse_layout(C.byref(cfg), C.byref(b))
                assert bytes(a)[:60] == bytes(oracle.prod_layout(cfg))[:60]
                assert bytes(b) == bytes(oracle.mse_layout(cfg))


def test_attention_ref_vs_reference_host_code(oracle):
    if oracle.ref_host() is None:
        pytest.skip("oracle/_ref not built (reference tree absent)")
    rng = np.random.default_rng(5)
    for n in (1, 7, 300):
        q = rng.standard_normal(128).astype(np.float16)
        k = rng.standard_normal((n, 128)).astype(np.float16)
        v = rng.standard_normal((n, 128)).astype(np.float16)
        assert (oracle.attention_ref_single_head(q, k, v) == oracle.ref_attention_single_head(q, k, v)).all()


# ---- known answers ---------------------------------------------------------------

def test_sign_pattern(oracle):
    L = oracle.lib()
    for h in range(16):
        for i in range(256):
            assert L.orc_sign_flip(i, h) == (1.0 if (i + h) % 2 == 0 else -1.0)


def test_fwht_known_answers(oracle):
    e = np.zeros(128, np.float32)
    e[0] = 1.0
    assert (oracle.fwht(e) == 1.0).all()
    e[:] = 0
    e[5] = 1.0
    y = oracle.fwht(e)
    # Sylvester ordering: H[i, j] = (-1)^popcount(i & j)
    exp = np.array([(-1.0) ** bin(i & 5).count("1") for i in range(128)], np.float32)
    assert (y == exp).all()
    x = np.random.default_rng(0).standard_normal(128).astype(np.float32)
    assert np.allclose(oracle.fwht(oracle.fwht(x)) / 128.0, x, atol=1e-5)


def test_codebooks(oracle):
    c3, c4 = oracle.cb3(), oracle.cb4()
    assert (c3 == -c3[::-1]).all() and (c4 == -c4[::-1]).all()
    assert (np.diff(c3) > 0).all() and (np.diff(c4) > 0).all()
    # Lloyd-Max 8-level design for N(0,1) (what src/gaussian_codebook.cpp prints)
    assert np.allclose(c3[4:], [0.244919, 0.755526, 1.34326, 2.1513], atol=2e-6)
    assert np.float32(c4[8]) == np.float32(0.1284) and np.float32(c4[15]) == np.float32(2.7326)


def test_nibble_order_and_pack_roundtrip(oracle):
    # even element -> low nibble (include/tq_shared_device.cuh:61-64)
    rng = np.random.default_rng(11)
    cfg = oracle.make_config(1)
    key = rng.standard_normal((1, 1, 128)).astype(np.float16)
    val = rng.standard_normal((1, 1, 128)).astype(np.float16)
    pool, kn, vn = oracle.pack("turbo_prod", key, val, np.zeros(1, np.int32), cfg, trace=True)
    lay = oracle.prod_layout(cfg)
    kb = pool[lay.k4_codes_offset:lay.k4_codes_offset + 64]
    L = oracle.lib()
    for i in (0, 1, 2, 77, 126, 127):
        nib = (kb[i // 2] >> (4 * (i % 2))) & 0xF
        assert (nib & 7) == L.orc_nearest_k3(C.c_float(kn[0, 0, i]))
        e = np.float32(kn[0, 0, i]) - oracle.cb3()[nib & 7]
        assert (nib >> 3) == (1 if e >= 0 else 0)


def test_roundtrip_quality(oracle):
    rng = np.random.default_rng(3)
    cfg = oracle.make_config(2)
    key = rng.standard_normal((64, 2, 128)).astype(np.float16)
    val = rng.standard_normal((64, 2, 128)).astype(np.float16)
    slots = np.arange(64, dtype=np.int32)
    for scheme, tol in (("turbo_prod", 0.35), ("turbo_mse", 0.25)):  # tests/test_cag.py:212-215
        k2, v2 = oracle.dequant(scheme, oracle.pack(scheme, key, val, slots, cfg), slots, cfg)
        for a, b in ((key, k2), (val, v2)):
            rel = np.mean((a.astype(np.float32) - b.astype(np.float32)) ** 2) / np.var(a.astype(np.float32))
            assert rel < tol and rel < 0.02


def test_zero_and_tiny_rows(oracle):
    cfg = oracle.make_config(2)
    key = np.zeros((3, 2, 128), np.float16)
    val = np.zeros((3, 2, 128), np.float16)
    val[1] = np.float16(6e-8)  # fp16 subnormal
    slots = np.arange(3, dtype=np.int32)
    pool = oracle.pack("turbo_prod", key, val, slots, cfg)
    k2, v2 = oracle.dequant("turbo_prod", pool, slots, cfg)
    assert np.isfinite(k2.astype(np.float32)).all() and np.abs(k2.astype(np.float32)).max() < 1e-6


# ---- the kernels' threshold tables ----------------------------------------------------

def _thresholds(fn, cb):
    def key(x):
        i = int(np.float32(x).view(np.uint32))
        return (i ^ 0x80000000) if i < 0x80000000 else (~i & 0xFFFFFFFF)

    def unkey(k):
        i = (k ^ 0x80000000) if k >= 0x80000000 else (~k & 0xFFFFFFFF)
        return np.uint32(i).view(np.float32)

    out = []
    for i in range(len(cb) - 1):
        lo, hi = key(cb[i]), key(cb[i + 1])
        while hi - lo > 1:
            mid = (lo + hi) // 2
            if fn(C.c_float(unkey(mid))) >= i + 1:
                hi = mid
            else:
                lo = mid
        out.append(int(unkey(hi).view(np.uint32)))
    return out


def test_kernel_threshold_tables_match_reference_scan(oracle):
    """tq_common.cuh holds the decision thresholds of the reference's nearest-level scan
    as fp32 bit patterns; recompute them from the restated scan."""
    src = (ROOT / "turborag_b200" / "csrc" / "tq_common.cuh").read_text()
    consts = {m.group(1): int(m.group(2), 16)
              for m in re.finditer(r"#define (TQ_\w+) TQF\(0x([0-9a-fA-F]+)\)", src)}
    L = oracle.lib()
    for name, fn, cb, mid in (("K3", L.orc_nearest_k3, oracle.cb3(), 3), ("V4", L.orc_nearest_v4, oracle.cb4(), 7)):
        t = _thresholds(fn, cb)
        assert t[mid] == consts["TQ_TMID"]
        for j in range(1, mid + 1):
            assert consts[f"TQ_{name}_M{j}"] == t[mid + j]
            neg = int(np.float32(-np.uint32(t[mid - j]).view(np.float32)).view(np.uint32))
            assert consts[f"TQ_{name}_N{j}"] == neg + 1  # |x| > A  <=>  |x| >= nextup(A)


def test_nearest_is_monotone_near_thresholds(oracle):
    L = oracle.lib()
    for fn, cb in ((L.orc_nearest_k3, oracle.cb3()), (L.orc_nearest_v4, oracle.cb4())):
        for t in _thresholds(fn, cb):
            base = np.uint32(t).view(np.float32)
            xs = [np.nextafter(base, np.float32(-10)), base, np.nextafter(base, np.float32(10))]
            for _ in range(6):
                xs.insert(0, np.nextafter(xs[0], np.float32(-10)))
                xs.append(np.nextafter(xs[-1], np.float32(10)))
            codes = [fn(C.c_float(x)) for x in xs]
            assert codes == sorted(codes) and codes[-1] - codes[0] == 1


def test_exact_division_sequence():
    """q0 = x*r, rem = fma(-q0, d, x), q = fma(rem, r, q0) with r = RN(1/d) equals x/d."""
    rng = np.random.default_rng(9)
    x = (rng.standard_normal(200000) * rng.choice([1e-3, 1.0, 30.0], 200000)).astype(np.float32)
    d = np.abs(rng.standard_normal(200000)).astype(np.float32) + np.float32(1e-3)
    r = (np.float32(1.0) / d).astype(np.float32)
    q0 = (x * r).astype(np.float32)
    rem = (x.astype(np.float64) - q0.astype(np.float64) * d.astype(np.float64)).astype(np.float32)
    q = (q0.astype(np.float64) + rem.astype(np.float64) * r.astype(np.float64)).astype(np.float32)
    assert (q == (x / d).astype(np.float32)).all()
