"""numpy front-end to the CPU oracle (``liboracle.so``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the
CPU-baseline leg of ``bench.py``; the shipped package never imports it.

Arrays are numpy: fp16 tensors as ``float16`` (or their ``uint16`` views),
pools as ``uint8``, slot maps as ``int32``.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "liboracle.so"
REF_HOST_PATH = HERE / "_ref" / "libtq_ref_host.so"
REF_GPU_PATH = HERE / "_ref" / "libturboquant_ref.so"


class Config(C.Structure):
    """include/tq_config.h:4-13"""
    _fields_ = [(n, C.c_int) for n in (
        "block_size", "num_kv_heads", "head_dim", "nbits", "group_size",
        "page_alignment", "scale_type", "quant_mode")]


class ProdLayout(C.Structure):
    """include/tq_turbo_prod.cuh:15-28"""
    _fields_ = [(n, C.c_size_t) for n in (
        "page_size_bytes", "k4_codes_offset", "k_residual_scales_offset",
        "k_scales_offset", "v4_codes_offset", "v_scales_offset")] + [
        (n, C.c_int) for n in (
            "k4_bytes_per_token_head", "v4_bytes_per_token_head",
            "scale_bytes_per_token_head")]


class MseLayout(C.Structure):
    """include/tq_turbo_mse_layout.h:5-15"""
    _fields_ = [(n, C.c_size_t) for n in (
        "code_bytes_per_token_head", "norm_bytes_per_token_head",
        "k_codes_offset", "v_codes_offset", "k_norms_offset", "v_norms_offset",
        "page_size_bytes")]


def build(force: bool = False) -> Path:
    """Compile liboracle.so with gcc if it is missing or stale."""
    src = HERE / "tq_oracle.c"
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "liboracle.so"], check=True,
                       capture_output=True)
    return LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(str(LIB_PATH))
        _lib.orc_sign_flip.restype = C.c_float
        _lib.orc_sign_flip.argtypes = [C.c_int, C.c_int]
        _lib.orc_nearest_k3.argtypes = [C.c_float]
        _lib.orc_nearest_v4.argtypes = [C.c_float]
        _lib.orc_inv_sqrt_d_bits.restype = C.c_uint32
        _lib.orc_cb3.restype = C.POINTER(C.c_float)
        _lib.orc_cb4.restype = C.POINTER(C.c_float)
        _lib.orc_attention_ref_single_head.restype = C.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _u16(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a)
    if a.dtype == np.float16:
        return a.view(np.uint16)
    assert a.dtype == np.uint16, a.dtype
    return a


def make_config(num_kv_heads: int, head_dim: int = 128) -> Config:
    cfg = Config()
    lib().orc_default_config(C.byref(cfg))
    cfg.num_kv_heads = num_kv_heads
    cfg.head_dim = head_dim
    return cfg


def prod_layout(cfg: Config) -> ProdLayout:
    out = ProdLayout()
    lib().orc_prod_layout(C.byref(cfg), C.byref(out))
    return out


def mse_layout(cfg: Config) -> MseLayout:
    out = MseLayout()
    lib().orc_mse_layout(C.byref(cfg), C.byref(out))
    return out


class QjlLayout(C.Structure):
    """include/tq_qjl.cuh:22-35"""
    _fields_ = [(n, C.c_size_t) for n in ("page_size_bytes", "k1_codes_offset", "k_scales_offset",
                                          "v4_codes_offset", "v_scales_offset")] + \
               [(n, C.c_int) for n in ("k1_bytes_per_token_head", "v4_bytes_per_token_head",
                                       "scale_bytes_per_token_head")]


def qjl_layout(cfg: Config) -> QjlLayout:
    out = QjlLayout()
    lib().orc_qjl_layout(C.byref(cfg), C.byref(out))
    return out


def layout_for(scheme: str, cfg: Config):
    if scheme == "qjl":
        return qjl_layout(cfg)
    return prod_layout(cfg) if scheme == "turbo_prod" else mse_layout(cfg)


def _fn(scheme: str, op: str):
    return getattr(lib(), {"turbo_prod": "orc_prod_", "turbo_mse": "orc_mse_", "qjl": "orc_qjl_"}[scheme] + op)


def cb3() -> np.ndarray:
    return np.ctypeslib.as_array(lib().orc_cb3(), (8,)).copy()


def cb4() -> np.ndarray:
    return np.ctypeslib.as_array(lib().orc_cb4(), (16,)).copy()


def set_threads(n: int) -> None:
    lib().orc_set_threads(int(n))


def fwht(x: np.ndarray) -> np.ndarray:
    y = np.ascontiguousarray(x, dtype=np.float32).copy()
    lib().orc_fwht128(_p(y), C.c_int(y.shape[-1]))
    return y


def num_pages(slots: np.ndarray, block_size: int = 16) -> int:
    return int(slots.max()) // block_size + 1 if slots.size else 0


def pack(scheme: str, key, value, slots, cfg: Config, pool: np.ndarray | None = None,
         trace: bool = False):
    """Quantise+pack into a (zero-initialised unless given) pool.

    Returns pool, or (pool, kn, vn) with the normalised pre-quantisation values
    when ``trace`` is set (used for the 1-ulp boundary accounting)."""
    k, v = _u16(key), _u16(value)
    slots = np.ascontiguousarray(slots, dtype=np.int32)
    n = k.shape[0]
    lay = layout_for(scheme, cfg)
    if pool is None:
        pool = np.zeros(num_pages(slots, cfg.block_size) * lay.page_size_bytes, np.uint8)
    kn = np.zeros(k.shape, np.float32) if trace else None
    vn = np.zeros(k.shape, np.float32) if trace else None
    fn = _fn(scheme, "pack")
    fn(_p(k), _p(v), _p(slots), _p(pool), C.byref(lay), C.byref(cfg), C.c_int(n),
       _p(kn), _p(vn))
    return (pool, kn, vn) if trace else pool


def dequant(scheme: str, pool, slots, cfg: Config):
    slots = np.ascontiguousarray(slots, dtype=np.int32)
    n = slots.shape[0]
    lay = layout_for(scheme, cfg)
    shape = (n, cfg.num_kv_heads, cfg.head_dim)
    ok, ov = np.zeros(shape, np.uint16), np.zeros(shape, np.uint16)
    fn = _fn(scheme, "dequant")
    fn(_p(pool), _p(slots), _p(ok), _p(ov), C.byref(lay), C.byref(cfg), C.c_int(n))
    return ok.view(np.float16), ov.view(np.float16)


def prod_logits(query, pool, slots, cfg: Config):
    q = _u16(query)
    slots = np.ascontiguousarray(slots, dtype=np.int32)
    nq, nkv = q.shape[0], slots.shape[0]
    lay = prod_layout(cfg)
    out = np.zeros((nq, cfg.num_kv_heads, nkv), np.float32)
    lib().orc_prod_logits(_p(q), _p(pool), _p(slots), _p(out), C.byref(lay),
                          C.byref(cfg), C.c_int(nq), C.c_int(nkv))
    return out


def attn(scheme: str, query, pool, slots, cfg: Config):
    """Reference-API fused attention: query [nq, H, D] -> fp16 [nq, H, D]."""
    q = _u16(query)
    slots = np.ascontiguousarray(slots, dtype=np.int32)
    nq, nkv = q.shape[0], slots.shape[0]
    lay = layout_for(scheme, cfg)
    out = np.zeros(q.shape, np.uint16)
    fn = _fn(scheme, "attn")
    fn(_p(q), _p(pool), _p(slots), _p(out), C.byref(lay), C.byref(cfg),
       C.c_int(nq), C.c_int(nkv))
    return out.view(np.float16)


def attn_state(scheme: str, query, pool, slots, cfg: Config):
    """Rotated-domain fp32 (acc[D], m, l) per (query, head): [nq, H, D+2]."""
    q = _u16(query)
    slots = np.ascontiguousarray(slots, dtype=np.int32)
    nq, nkv = q.shape[0], slots.shape[0]
    lay = layout_for(scheme, cfg)
    out = np.zeros((nq, cfg.num_kv_heads, cfg.head_dim + 2), np.float32)
    fn = _fn(scheme, "attn_f32")
    fn(_p(q), _p(pool), _p(slots), _p(out), C.byref(lay), C.byref(cfg),
       C.c_int(nq), C.c_int(nkv))
    return out


def gqa_to_ref_query(q: np.ndarray, num_kv_heads: int) -> np.ndarray:
    """[Hq, D] (HF head order) -> reference layout [G, H, D], row g of kv-head h
    being query head h*G+g."""
    hq, d = q.shape
    g = hq // num_kv_heads
    return np.ascontiguousarray(q.reshape(num_kv_heads, g, d).transpose(1, 0, 2))


def ref_to_gqa_out(o: np.ndarray) -> np.ndarray:
    g, h, d = o.shape
    return np.ascontiguousarray(o.transpose(1, 0, 2)).reshape(h * g, d)


def decode_paged(scheme: str, query, pool, block_tables, seq_lens, cfg: Config):
    """Batched paged GQA decode: query [B, Hq, D] fp16 -> fp16 [B, Hq, D].
    block_tables int32 [B, max_pages]; token t of sequence b lives in slot
    block_tables[b, t // 16] * 16 + t % 16 (src/tq_block_table.cpp:24-39)."""
    q = _u16(query)
    b, hq, d = q.shape
    tables = np.ascontiguousarray(block_tables, dtype=np.int32)
    lens = np.ascontiguousarray(seq_lens, dtype=np.int32)
    lay = layout_for(scheme, cfg)
    out = np.zeros((b, hq, d), np.uint16)
    lib().orc_decode_paged(C.c_int(0 if scheme == "turbo_prod" else 1), _p(q), _p(pool), _p(tables),
                           C.c_int(tables.shape[1]), _p(lens), _p(out), C.byref(lay), C.byref(cfg),
                           C.c_int(b), C.c_int(hq))
    return out.view(np.float16)


def attention_ref_single_head(q, k_all, v_all):
    """src/tq_attention_ref.cpp:10-56 restated: q [D], k/v [N, D] fp16 -> fp32 [D]."""
    q, k, v = _u16(q), _u16(k_all), _u16(v_all)
    n, d = k.shape
    out = np.zeros(d, np.float32)
    rc = lib().orc_attention_ref_single_head(_p(q), _p(k), _p(v), C.c_int(n), C.c_int(d), _p(out))
    if rc != 0:
        raise RuntimeError("size mismatch")
    return out


def mse_prefill(query, pool, slots, chunk_k, chunk_v, cfg: Config, rows=None):
    """query [nq, Hq, D]; prefix = turbo_mse pool via slots; optional causal
    fp16 chunk [nq, H, D]. Returns fp32 [nq, Hq, D], or [len(rows), Hq, D] for the listed
    query rows only (a row's index inside the chunk decides how much of the chunk it sees)."""
    q = _u16(query)
    slots = np.ascontiguousarray(slots, dtype=np.int32)
    nq, hq, d = q.shape
    lay = mse_layout(cfg)
    ck = None if chunk_k is None else _u16(chunk_k)
    cv = None if chunk_v is None else _u16(chunk_v)
    rows_a = None if rows is None else np.ascontiguousarray(rows, dtype=np.int32)
    nrows = nq if rows_a is None else int(rows_a.shape[0])
    out = np.zeros((nrows, hq, d), np.float32)
    lib().orc_mse_prefill_rows(_p(q), _p(pool), _p(slots), C.c_int(slots.shape[0]), _p(ck),
                               _p(cv), C.c_int(nq), C.c_int(hq), _p(rows_a), C.c_int(nrows),
                               _p(out), C.byref(lay), C.byref(cfg))
    return out


# --------------------------------------------------------------------------- #
# the reference's own host code (present only where oracle/_ref was built)    #
# --------------------------------------------------------------------------- #

_ref_host = None


def ref_host():
    """libtq_ref_host.so or None."""
    global _ref_host
    if _ref_host is None and REF_HOST_PATH.exists():
        _ref_host = C.CDLL(str(REF_HOST_PATH))
    return _ref_host


def ref_attention_single_head(q, k_all, v_all):
    r = ref_host()
    q, k, v = _u16(q), _u16(k_all), _u16(v_all)
    n, d = k.shape
    out = np.zeros(d, np.float32)
    if r.ref_attention_single_head(_p(q), _p(k), _p(v), C.c_int(n), C.c_int(d), _p(out)) != 0:
        raise RuntimeError("reference threw")
    return out
