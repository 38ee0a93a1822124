"""QJL-1bit scheme (K = one sign bit per rotated dimension + fp16 RMS, V = 4-bit codes + fp16
RMS; src/cuda/tq_qjl_kernels.cu of the reference, which compiles the kernels but does not export
them through its C API).

CPU: layout numbers, the oracle against fixtures made by the reference's own kernels
(tests/golden/qjl_*.npz, ``make_golden.py --qjl``), properties of the format.
GPU: the sm_100a kernels through the C ABI against the oracle and the fixtures -- pools and
dequantised tensors bit-exact, attention within 2e-3.
"""
import ctypes as C
import hashlib
from pathlib import Path

import numpy as np
import pytest

from tests.conftest import GOLDEN, rowwise_rel_err
from tests.golden.cases import CASES, make_inputs, make_kv, make_slots

ROOT = Path(__file__).resolve().parent.parent
ATTN_TOL = 2e-3


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def golden(name):
    path = GOLDEN / f"qjl_{name}.npz"
    if not path.exists():
        pytest.skip(f"{path.name} not generated")
    return np.load(path)


# ---------------------------------------------------------------------------------------------
# CPU
# ---------------------------------------------------------------------------------------------

def test_layout_known_numbers(oracle, tq):
    # 16 + 2 + 64 + 2 = 84 bytes per token-head (include/tq_qjl.cuh:14-19)
    cfg = oracle.make_config(2)
    lay = oracle.qjl_layout(cfg)
    assert (lay.k1_codes_offset, lay.k_scales_offset, lay.v4_codes_offset, lay.v_scales_offset,
            lay.page_size_bytes) == (0, 512, 576, 2624, 2688)
    assert (lay.k1_bytes_per_token_head, lay.v4_bytes_per_token_head, lay.scale_bytes_per_token_head) == (16, 64, 2)
    for h in (1, 2, 3, 4, 8, 32):
        for bs in (1, 8, 16, 32):
            for d in (64, 128):
                ocfg = oracle.make_config(h, d)
                ocfg.block_size = bs
                tcfg = tq.default_config()
                tcfg.num_kv_heads, tcfg.block_size, tcfg.head_dim = h, bs, d
                assert bytes(tq.make_qjl_layout_for(tcfg))[:52] == bytes(oracle.qjl_layout(ocfg))[:52]


def test_layout_vs_reference_host_code(oracle):
    ref = ROOT / "oracle" / "_ref" / "libturboquant_ref.so"
    if not ref.exists():
        pytest.skip("oracle/_ref not built (reference tree absent)")
    try:
        lib = C.CDLL(str(ref))
    except OSError as e:
        pytest.skip(f"reference library does not load here: {e}")
    for h in (1, 2, 3, 8):
        for bs in (1, 16, 32):
            cfg = oracle.make_config(h)
            cfg.block_size = bs
            out = oracle.QjlLayout()
            assert lib.tq_make_qjl_layout(C.byref(cfg), C.byref(out)) == 0
            assert bytes(out)[:52] == bytes(oracle.qjl_layout(cfg))[:52]


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_oracle_vs_reference_fixture(oracle, case):
    z = golden(case["name"])
    key, value, query, slots = make_inputs(case)
    assert sha(key) == str(z["key_sha"]) and sha(value) == str(z["value_sha"]) and (slots == z["slots"]).all()
    cfg = oracle.make_config(case["h"])
    assert oracle.qjl_layout(cfg).page_size_bytes == int(z["page_size_bytes"][0])
    pool = oracle.pack("qjl", key, value, slots, cfg)
    assert np.array_equal(pool, z["qjl_pool"]), "oracle pool differs from the reference kernels' pool"
    dk, dv = oracle.dequant("qjl", z["qjl_pool"], slots, cfg)
    assert sha(dk.view(np.uint16)) == str(z["qjl_dequant_sha"][0])
    assert sha(dv.view(np.uint16)) == str(z["qjl_dequant_sha"][1])
    keep = z["qjl_dequant_key_head"].shape[0]
    assert np.array_equal(dk.view(np.uint16)[:keep], z["qjl_dequant_key_head"])
    out = oracle.attn("qjl", query, z["qjl_pool"], slots, cfg)
    assert rowwise_rel_err(out, z["qjl_attn"].view(np.float16)) < ATTN_TOL


def test_format_properties(oracle):
    rng = np.random.default_rng(5)
    key, value = make_kv(rng, 40, 2)
    slots = make_slots(rng, 40, True, extra_pages=1)
    cfg = oracle.make_config(2)
    lay = oracle.qjl_layout(cfg)
    pool = oracle.pack("qjl", key, value, slots, cfg)
    # sign bits = signs of the rotated key (no head term in the rotation), bit i of byte i/8
    sign = np.where(np.arange(128) % 2 == 0, 1.0, -1.0).astype(np.float32)
    for t in (0, 17, 39):
        for h in (0, 1):
            rot = oracle.fwht(key[t, h].astype(np.float32) * sign)
            page = (slots[t] // 16) * lay.page_size_bytes
            th = (slots[t] % 16) * 2 + h
            bits = np.unpackbits(pool[page + th * 16: page + th * 16 + 16], bitorder="little")
            assert np.array_equal(bits.astype(bool), rot >= 0)
    # dequantised K: every rotated coordinate has magnitude ks, so |k|^2 = 128 ks^2 / ... = D * ks^2
    dk, dv = oracle.dequant("qjl", pool, slots, cfg)
    ks = pool[lay.k_scales_offset: lay.k_scales_offset + 2].view(np.float16)[0].astype(np.float32)
    t0 = int(np.flatnonzero(slots == 0)[0])
    assert abs(np.square(dk[t0, 0].astype(np.float32)).sum() - 128 * ks * ks) < 0.02 * 128 * ks * ks
    # V goes through the turbo_prod V quantiser: relative error of the 4-bit codebook
    rel = np.square(dv.astype(np.float32) - value.astype(np.float32)).mean() / np.square(value.astype(np.float32)).mean()
    assert rel < 0.02
    # untouched cells (the spare page, the ragged tail) stay zero
    used = np.zeros(pool.size, bool)
    for s in slots:
        page, tib = (s // 16) * lay.page_size_bytes, s % 16
        for h in (0, 1):
            th = tib * 2 + h
            for off, nb in ((lay.k1_codes_offset, 16), (lay.k_scales_offset, 2), (lay.v4_codes_offset, 64),
                            (lay.v_scales_offset, 2)):
                used[page + off + th * nb: page + off + th * nb + nb] = True
    assert not pool[~used].any()


# ---------------------------------------------------------------------------------------------
# GPU
# ---------------------------------------------------------------------------------------------

def _gpu(tq, key, value, query, slots, h, pool_offset=0):
    import torch
    dev = torch.device("cuda:0")
    cfg = tq.default_config()
    cfg.num_kv_heads, cfg.head_dim = h, 128
    lay = tq.make_qjl_layout_for(cfg)
    pages = int(slots.max()) // 16 + 1
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).to(dev).view(torch.float16)  # noqa: E731
    buf = torch.zeros(pages * lay.page_size_bytes + 64, dtype=torch.uint8, device=dev)
    pool = buf[pool_offset: pool_offset + pages * lay.page_size_bytes]
    ds = torch.from_numpy(slots).to(dev)
    n = key.shape[0]
    tq.qjl_pack(t(key), t(value), ds, pool, lay, cfg)
    ok = torch.zeros(n, h, 128, dtype=torch.float16, device=dev)
    ov = torch.zeros_like(ok)
    tq.qjl_dequant(pool, ds, ok, ov, lay, cfg)
    out = None
    if query is not None:
        out = torch.zeros(query.shape[0], h, 128, dtype=torch.float16, device=dev)
        tq.qjl_fused_attn_output(t(query), pool, ds, out, lay, cfg, query.shape[0], n)
        out = out.cpu().numpy()
    torch.cuda.synchronize()
    return pool.cpu().numpy(), ok.cpu().numpy(), ov.cpu().numpy(), out


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_kernels_vs_oracle_and_fixture(tq, oracle, case):
    key, value, query, slots = make_inputs(case)
    cfg = oracle.make_config(case["h"])
    pool, dk, dv, out = _gpu(tq, key, value, query, slots, case["h"])
    want = oracle.pack("qjl", key, value, slots, cfg)
    assert np.array_equal(pool, want)
    ok, ov = oracle.dequant("qjl", want, slots, cfg)
    assert np.array_equal(dk.view(np.uint16), ok.view(np.uint16)) and np.array_equal(dv.view(np.uint16), ov.view(np.uint16))
    assert rowwise_rel_err(out, oracle.attn("qjl", query, want, slots, cfg)) < ATTN_TOL
    z = golden(case["name"])
    assert np.array_equal(pool, z["qjl_pool"])
    assert sha(dk.view(np.uint16)) == str(z["qjl_dequant_sha"][0]) and sha(dv.view(np.uint16)) == str(z["qjl_dequant_sha"][1])
    assert rowwise_rel_err(out, z["qjl_attn"].view(np.float16)) < ATTN_TOL


@pytest.mark.gpu
@pytest.mark.parametrize("n,h,nq,offset", [(1, 1, 1, 0), (17, 3, 5, 0), (333, 2, 9, 0), (4099, 8, 2, 0), (50, 4, 3, 4)])
def test_kernels_ragged_permuted_misaligned(tq, oracle, n, h, nq, offset):
    rng = np.random.default_rng(n * 31 + h)
    key, value = make_kv(rng, n, h)
    query = rng.standard_normal((nq, h, 128)).astype(np.float16)
    slots = make_slots(rng, n, True, extra_pages=2)
    cfg = oracle.make_config(h)
    pool, dk, dv, out = _gpu(tq, key, value, query, slots, h, pool_offset=offset)
    want = oracle.pack("qjl", key, value, slots, cfg)
    assert np.array_equal(pool, want)  # includes the bytes no token maps to
    ok, ov = oracle.dequant("qjl", want, slots, cfg)
    assert np.array_equal(dk.view(np.uint16), ok.view(np.uint16)) and np.array_equal(dv.view(np.uint16), ov.view(np.uint16))
    assert rowwise_rel_err(out, oracle.attn("qjl", query, want, slots, cfg)) < ATTN_TOL


@pytest.mark.gpu
def test_special_rows(tq, oracle):
    rng = np.random.default_rng(0)
    key, value = make_kv(rng, 20, 2)
    key[0] = 0
    value[1] = 0
    key[2] = np.float16(6e-8)      # denormal inputs
    key[3, :, ::2] = np.float16(-0.0)
    key[4] = np.float16(60000.0)
    slots = np.arange(20, dtype=np.int32)
    pool, dk, dv, _ = _gpu(tq, key, value, None, slots, 2)
    cfg = oracle.make_config(2)
    want = oracle.pack("qjl", key, value, slots, cfg)
    assert np.array_equal(pool, want)
    ok, ov = oracle.dequant("qjl", want, slots, cfg)
    assert np.array_equal(dk.view(np.uint16), ok.view(np.uint16)) and np.array_equal(dv.view(np.uint16), ov.view(np.uint16))


@pytest.mark.gpu
def test_paged_gqa_decode(tq, oracle):
    import torch
    dev = torch.device("cuda:0")
    h, hq, lens = 2, 16, [77, 300, 2049]
    rng = np.random.default_rng(12)
    cfg = tq.default_config()
    cfg.num_kv_heads, cfg.head_dim = h, 128
    lay = tq.make_qjl_layout_for(cfg)
    ocfg = oracle.make_config(h)
    width = max((n + 15) // 16 for n in lens)
    total = sum((n + 15) // 16 for n in lens)
    order = rng.permutation(total)
    pool = torch.zeros(total * lay.page_size_bytes, dtype=torch.uint8, device=dev)
    tables = np.zeros((len(lens), width), np.int32)
    q = rng.standard_normal((len(lens), hq, 128)).astype(np.float16)
    t16 = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).to(dev).view(torch.float16)  # noqa: E731
    want, first = [], 0
    for b, n in enumerate(lens):
        pages = (n + 15) // 16
        tables[b, :pages] = order[first:first + pages]
        first += pages
        key, value = make_kv(rng, n, h)
        tt = np.arange(n)
        slots = (tables[b, tt // 16] * 16 + tt % 16).astype(np.int32)
        tq.qjl_pack(t16(key), t16(value), torch.from_numpy(slots).to(dev), pool, lay, cfg)
        # query head j belongs to kv head j // 8: reference rows are [g][h]
        qref = q[b].reshape(h, 8, 128).transpose(1, 0, 2)
        o = oracle.attn("qjl", qref, oracle.pack("qjl", key, value, slots, ocfg,
                                                 pool=np.zeros(total * lay.page_size_bytes, np.uint8)), slots, ocfg)
        want.append(o.transpose(1, 0, 2).reshape(hq, 128))
    out = tq.decode_paged("qjl", t16(q), pool, torch.from_numpy(tables).to(dev),
                          torch.tensor(lens, dtype=torch.int32, device=dev), lay, cfg)
    torch.cuda.synchronize()
    assert rowwise_rel_err(out.cpu().numpy(), np.stack(want)) < ATTN_TOL
    # records of this scheme are not handed out (the stand-alone merges assume the per-head sign)
    with pytest.raises(RuntimeError):
        tq.decode_paged("qjl", t16(q), pool, torch.from_numpy(tables).to(dev),
                        torch.tensor(lens, dtype=torch.int32, device=dev), lay, cfg,
                        partials_out=torch.zeros(len(lens), hq, 130, device=dev))
