"""ctypes front-end to libturboquant.so, interface-compatible with the reference's
``tq_backend/turboquant_wrapper.py :: TurboQuantWrapper`` (same class, method and
argument names, same error behaviour: ``RuntimeError`` on a non-zero return code,
``FileNotFoundError`` when the library is missing), plus the additions of
``include/turboquant.h`` part 2.

There is no CPU path: every compute method needs the CUDA library and CUDA
tensors, and raises if either is missing.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

PKG = Path(__file__).resolve().parent
DEFAULT_LIB_PATH = PKG / "lib" / "libturboquant.so"

SCHEME_ID = {"turbo_prod": 0, "turbo_mse": 1, "qjl": 2}
PARTIAL_STRIDE = 130
INT32_MAX = 2**31 - 1


def _struct(name, doc, fields):
    return type(name, (C.Structure,), {"_fields_": fields, "__doc__": doc})


TQConfig = _struct("TQConfig", "include/tq_config.h:4-13", [(n, C.c_int) for n in (
    "block_size", "num_kv_heads", "head_dim", "nbits", "group_size", "page_alignment",
    "scale_type", "quant_mode")])

TQTurboProdPageLayout = _struct(
    "TQTurboProdPageLayout", "include/tq_turbo_prod.cuh:15-28",
    [(n, C.c_size_t) for n in (
        "page_size_bytes", "k4_codes_offset", "k_residual_scales_offset", "k_scales_offset",
        "v4_codes_offset", "v_scales_offset")] +
    [(n, C.c_int) for n in (
        "k4_bytes_per_token_head", "v4_bytes_per_token_head", "scale_bytes_per_token_head")])

TQTurbomsePageLayout = _struct(
    "TQTurbomsePageLayout", "include/tq_turbo_mse_layout.h:5-15",
    [(n, C.c_size_t) for n in (
        "code_bytes_per_token_head", "norm_bytes_per_token_head", "k_codes_offset",
        "v_codes_offset", "k_norms_offset", "v_norms_offset", "page_size_bytes")])

TQQJLPageLayout = _struct(
    "TQQJLPageLayout", "include/tq_qjl.cuh:22-35",
    [(n, C.c_size_t) for n in (
        "page_size_bytes", "k1_codes_offset", "k_scales_offset", "v4_codes_offset", "v_scales_offset")] +
    [(n, C.c_int) for n in (
        "k1_bytes_per_token_head", "v4_bytes_per_token_head", "scale_bytes_per_token_head")])

_P = C.c_void_p
_CFG = C.POINTER(TQConfig)
_PROD = C.POINTER(TQTurboProdPageLayout)
_MSE = C.POINTER(TQTurbomsePageLayout)
_QJL = C.POINTER(TQQJLPageLayout)

# symbol -> (restype, argtypes); every symbol declared in include/turboquant.h
SIGNATURES = {
    "tq_last_error": (C.c_char_p, []),
    "tq_make_default_config": (C.c_int, [_CFG]),
    "tq_make_turbo_prod_layout": (C.c_int, [_CFG, _PROD]),
    "tq_make_turbo_mse_layout": (C.c_int, [_CFG, _MSE]),
    "tq_launch_turbo_prod_pack_kv": (C.c_int, [_P, _P, _P, _P, _PROD, _CFG, C.c_int, _P]),
    "tq_launch_turbo_prod_dequant_kv": (C.c_int, [_P, _P, _P, _P, _PROD, _CFG, C.c_int, _P]),
    "tq_launch_turbo_prod_fused_attention_logits":
        (C.c_int, [_P, _P, _P, _P, _PROD, _CFG, C.c_int, C.c_int, _P]),
    "tq_launch_turbo_prod_fused_attention_output":
        (C.c_int, [_P, _P, _P, _P, _PROD, _CFG, C.c_int, C.c_int, _P]),
    "tq_launch_turbo_mse_pack_kv": (C.c_int, [_P, _P, _P, _P, _MSE, _CFG, C.c_int, _P]),
    "tq_launch_turbo_mse_dequant_kv": (C.c_int, [_P, _P, _P, _P, _MSE, _CFG, C.c_int, _P]),
    "tq_launch_turbo_mse_fused_attention_output":
        (C.c_int, [_P, _P, _P, _P, _MSE, _CFG, C.c_int, C.c_int, _P]),
    "tq_make_qjl_layout": (C.c_int, [_CFG, _QJL]),
    "tq_launch_qjl_pack_kv": (C.c_int, [_P, _P, _P, _P, _QJL, _CFG, C.c_int, _P]),
    "tq_launch_qjl_dequant_kv": (C.c_int, [_P, _P, _P, _P, _QJL, _CFG, C.c_int, _P]),
    "tq_launch_qjl_fused_attention_output": (C.c_int, [_P, _P, _P, _P, _QJL, _CFG, C.c_int, C.c_int, _P]),
    "tq_decode_num_splits": (C.c_int, [C.c_int] * 4),
    "tq_decode_workspace_bytes": (C.c_size_t, [C.c_int] * 3),
    "tq_decode_paged": (C.c_int, [C.c_int, _P, _P, _P, C.c_int, _P, _P, _P, _P, _CFG, C.c_int,
                                  C.c_int, C.c_int, C.c_int, C.c_int, _P, C.c_size_t, _P]),
    "tq_decode_paged_static": (C.c_int, [C.c_int, _P, _P, _P, C.c_int, _P, _P, _P, _CFG, C.c_int,
                                         C.c_int, C.c_int, _P]),
    "tq_merge_partials": (C.c_int, [_P, C.c_int, _P, C.c_int, C.c_int, C.c_int, _P]),
    "tq_dequant_kv_hnd": (C.c_int, [C.c_int, _P, _P, _P, _P, _P, _CFG, C.c_int, _P]),
    "tq_debug_turbo_prod_pack_kv": (C.c_int, [_P, _P, _P, _P, _PROD, _CFG, C.c_int, _P, _P, _P, _P, _P, _P, _P]),
    "tq_mse_prefill_paged": (C.c_int, [_P, _P, _P, C.c_int, _P, _P, _P, _P, _MSE, _CFG, C.c_int,
                                       C.c_int, C.c_int, _P]),
    "tq_mse_prefill_status": (C.c_int, []),
    "tq_peer_buffer_bytes": (C.c_size_t, [C.c_int, C.c_int]),
    "tq_decode_paged_publish": (C.c_int, [C.c_int, _P, _P, _P, C.c_int, _P, _P, _CFG, C.c_int, C.c_int,
                                          C.c_int, C.c_int, C.c_int, _P, C.c_size_t, _P, C.c_int, C.c_int,
                                          C.c_int, C.c_uint, _P]),
    "tq_decode_paged_exchange": (C.c_int, [C.c_int, _P, _P, _P, C.c_int, _P, _P, _CFG, C.c_int, C.c_int,
                                           C.c_int, C.c_int, C.c_int, _P, C.c_size_t, _P, C.c_int, C.c_int,
                                           C.c_int, C.c_uint, _P, _P]),
    "tq_peer_publish": (C.c_int, [_P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint, _P]),
    "tq_peer_merge": (C.c_int, [_P, C.c_int, C.c_int, C.c_int, C.c_uint, _P, C.c_int, C.c_int, C.c_int, _P]),
    "tq_peer_status": (C.c_int, []),
    "tq_peer_clear_status": (C.c_int, []),
    "tq_peer_set_wait_ns": (C.c_int, [C.c_ulonglong]),
    "tq_block_table_create": (_P, [C.c_int, C.c_int]),
    "tq_block_table_destroy": (None, [_P]),
    "tq_block_table_free_pages": (C.c_int, [_P]),
    "tq_block_table_append": (C.c_int, [_P, C.c_int, C.c_int, _P]),
    "tq_block_table_num_tokens": (C.c_int, [_P, C.c_int]),
    "tq_block_table_pages": (C.c_int, [_P, C.c_int, _P, C.c_int]),
    "tq_block_table_release": (C.c_int, [_P, C.c_int]),
}


def load_library(lib_path: str | Path | None = None) -> C.CDLL:
    path = Path(lib_path) if lib_path else DEFAULT_LIB_PATH
    if not path.exists():
        raise FileNotFoundError(
            f"libturboquant.so not found at {path}. Run:  python -m turborag_b200.build  first.")
    lib = C.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype, fn.argtypes = res, args
    return lib


def _ptr(t: torch.Tensor | None) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


def _cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("libturboquant has no CPU path: tensors must live on a CUDA device")
        if t is not None and not t.is_contiguous():
            raise RuntimeError("tensors must be contiguous")


class TurboQuantWrapper:
    """turbo_prod — K = 3-bit Lloyd-Max code + 1-bit residual sign, V = 4-bit;
    turbo_mse — 4-bit K and V.  Tensors in, tensors out; pointers handled here."""

    def __init__(self, lib_path: str | Path | None = None) -> None:
        self._lib = load_library(lib_path)
        self.lib_path = Path(lib_path) if lib_path else DEFAULT_LIB_PATH

    # -- errors ---------------------------------------------------------------
    def _last_cuda_error(self) -> str:
        raw = self._lib.tq_last_error()
        return raw.decode() if raw else ""

    def _kernel_raise(self, rc: int, scheme: str, op: str) -> None:
        if rc == -2:
            raise RuntimeError(f"{scheme} {op} CUDA error: {self._last_cuda_error()}")
        raise RuntimeError(f"{scheme} {op} failed (rc={rc})")

    def _call(self, scheme: str, op: str, fn, *args) -> None:
        rc = fn(*args)
        if rc != 0:
            self._kernel_raise(rc, scheme, op)

    # -- config / layouts -------------------------------------------------------
    def default_config(self) -> TQConfig:
        cfg = TQConfig()
        if self._lib.tq_make_default_config(C.byref(cfg)) != 0:
            raise RuntimeError("tq_make_default_config failed")
        return cfg

    def make_layout_for(self, cfg: TQConfig) -> TQTurboProdPageLayout:
        layout = TQTurboProdPageLayout()
        if self._lib.tq_make_turbo_prod_layout(C.byref(cfg), C.byref(layout)) != 0:
            raise RuntimeError("tq_make_turbo_prod_layout failed")
        return layout

    def make_mse_layout_for(self, cfg: TQConfig) -> TQTurbomsePageLayout:
        layout = TQTurbomsePageLayout()
        if self._lib.tq_make_turbo_mse_layout(C.byref(cfg), C.byref(layout)) != 0:
            raise RuntimeError("tq_make_turbo_mse_layout failed")
        return layout

    def make_qjl_layout_for(self, cfg: TQConfig) -> TQQJLPageLayout:
        layout = TQQJLPageLayout()
        if self._lib.tq_make_qjl_layout(C.byref(cfg), C.byref(layout)) != 0:
            raise RuntimeError("Failed to build the QJL layout.")
        return layout

    def layout_for_scheme(self, scheme: str, cfg: TQConfig):
        if scheme == "qjl":
            return self.make_qjl_layout_for(cfg)
        return self.make_layout_for(cfg) if scheme == "turbo_prod" else self.make_mse_layout_for(cfg)

    # -- turbo_prod ---------------------------------------------------------------
    def pack(self, key, value, slot_mapping, page_pool, layout, cfg, stream: int = 0) -> None:
        _cuda(key, value, slot_mapping, page_pool)
        self._call("turbo_prod", "pack_kv", self._lib.tq_launch_turbo_prod_pack_kv,
                   _ptr(key), _ptr(value), _ptr(slot_mapping), _ptr(page_pool),
                   C.byref(layout), C.byref(cfg), key.shape[0], C.c_void_p(stream))

    def dequant(self, page_pool, slot_mapping, out_key, out_value, layout, cfg,
                stream: int = 0) -> None:
        _cuda(page_pool, slot_mapping, out_key, out_value)
        self._call("turbo_prod", "dequant_kv", self._lib.tq_launch_turbo_prod_dequant_kv,
                   _ptr(page_pool), _ptr(slot_mapping), _ptr(out_key), _ptr(out_value),
                   C.byref(layout), C.byref(cfg), out_key.shape[0], C.c_void_p(stream))

    def fused_attn_logits(self, query, page_pool, slot_mapping, logits, layout, cfg,
                          num_queries: int, num_kv_tokens: int, stream: int = 0) -> None:
        """logits[(q*H + h)*num_kv_tokens + t] = <q, k_t> / sqrt(D) (fp32)."""
        _cuda(query, page_pool, slot_mapping, logits)
        self._call("turbo_prod", "fused_attn_logits",
                   self._lib.tq_launch_turbo_prod_fused_attention_logits,
                   _ptr(query), _ptr(page_pool), _ptr(slot_mapping), _ptr(logits),
                   C.byref(layout), C.byref(cfg), num_queries, num_kv_tokens, C.c_void_p(stream))

    def fused_attn_output(self, query, page_pool, slot_mapping, output, layout, cfg,
                          num_queries: int, num_kv_tokens: int, stream: int = 0) -> None:
        _cuda(query, page_pool, slot_mapping, output)
        self._call("turbo_prod", "fused_attn_output",
                   self._lib.tq_launch_turbo_prod_fused_attention_output,
                   _ptr(query), _ptr(page_pool), _ptr(slot_mapping), _ptr(output),
                   C.byref(layout), C.byref(cfg), num_queries, num_kv_tokens, C.c_void_p(stream))

    # -- turbo_mse ----------------------------------------------------------------
    def mse_pack(self, key, value, slot_mapping, page_pool, layout, cfg, stream: int = 0) -> None:
        _cuda(key, value, slot_mapping, page_pool)
        self._call("turbo_mse", "pack_kv", self._lib.tq_launch_turbo_mse_pack_kv,
                   _ptr(key), _ptr(value), _ptr(slot_mapping), _ptr(page_pool),
                   C.byref(layout), C.byref(cfg), key.shape[0], C.c_void_p(stream))

    def mse_dequant(self, page_pool, slot_mapping, out_key, out_value, layout, cfg,
                    stream: int = 0) -> None:
        _cuda(page_pool, slot_mapping, out_key, out_value)
        self._call("turbo_mse", "dequant_kv", self._lib.tq_launch_turbo_mse_dequant_kv,
                   _ptr(page_pool), _ptr(slot_mapping), _ptr(out_key), _ptr(out_value),
                   C.byref(layout), C.byref(cfg), out_key.shape[0], C.c_void_p(stream))

    def mse_fused_attn_output(self, query, page_pool, slot_mapping, output, layout, cfg,
                              num_queries: int, num_kv_tokens: int, stream: int = 0) -> None:
        _cuda(query, page_pool, slot_mapping, output)
        self._call("turbo_mse", "fused_attn_output",
                   self._lib.tq_launch_turbo_mse_fused_attention_output,
                   _ptr(query), _ptr(page_pool), _ptr(slot_mapping), _ptr(output),
                   C.byref(layout), C.byref(cfg), num_queries, num_kv_tokens, C.c_void_p(stream))

    # -- QJL-1bit (src/cuda/tq_qjl_kernels.cu; not bound by the reference's wrapper) --------------
    def qjl_pack(self, key, value, slot_mapping, page_pool, layout, cfg, stream: int = 0) -> None:
        _cuda(key, value, slot_mapping, page_pool)
        self._call("qjl", "pack_kv", self._lib.tq_launch_qjl_pack_kv,
                   _ptr(key), _ptr(value), _ptr(slot_mapping), _ptr(page_pool),
                   C.byref(layout), C.byref(cfg), key.shape[0], C.c_void_p(stream))

    def qjl_dequant(self, page_pool, slot_mapping, out_key, out_value, layout, cfg,
                    stream: int = 0) -> None:
        _cuda(page_pool, slot_mapping, out_key, out_value)
        self._call("qjl", "dequant_kv", self._lib.tq_launch_qjl_dequant_kv,
                   _ptr(page_pool), _ptr(slot_mapping), _ptr(out_key), _ptr(out_value),
                   C.byref(layout), C.byref(cfg), out_key.shape[0], C.c_void_p(stream))

    def qjl_fused_attn_output(self, query, page_pool, slot_mapping, output, layout, cfg,
                              num_queries: int, num_kv_tokens: int, stream: int = 0) -> None:
        """Logits are <q', k'> without 1/sqrt(head_dim) (tq_qjl_kernels.cu:335)."""
        _cuda(query, page_pool, slot_mapping, output)
        self._call("qjl", "fused_attn_output", self._lib.tq_launch_qjl_fused_attention_output,
                   _ptr(query), _ptr(page_pool), _ptr(slot_mapping), _ptr(output),
                   C.byref(layout), C.byref(cfg), num_queries, num_kv_tokens, C.c_void_p(stream))

    # -- pools and sizes ----------------------------------------------------------
    @staticmethod
    def _pages(num_tokens: int, cfg: TQConfig) -> int:
        return (num_tokens + cfg.block_size - 1) // cfg.block_size

    def alloc_page_pool(self, num_tokens: int, layout, cfg: TQConfig) -> torch.Tensor:
        return torch.zeros(self._pages(num_tokens, cfg) * layout.page_size_bytes,
                           device="cuda", dtype=torch.uint8)

    alloc_mse_pool = alloc_page_pool

    def fp16_bytes(self, num_tokens: int, cfg: TQConfig) -> int:
        return num_tokens * cfg.num_kv_heads * cfg.head_dim * 2 * 2

    def quant_bytes(self, num_tokens: int, layout, cfg: TQConfig) -> int:
        return self._pages(num_tokens, cfg) * layout.page_size_bytes

    mse_bytes = quant_bytes

    @staticmethod
    def compute_mse(a: torch.Tensor, b: torch.Tensor) -> float:
        return torch.mean((a.float() - b.float()) ** 2).item()

    def summary(self) -> dict:
        cfg = self.default_config()
        fp16_page = cfg.block_size * cfg.num_kv_heads * cfg.head_dim * 2 * 2
        return {
            "lib_path": str(self.lib_path),
            "config": {k: getattr(cfg, k) for k in ("block_size", "num_kv_heads", "head_dim", "nbits")},
            "turbo_prod_compression_ratio_vs_fp16":
                round(fp16_page / self.make_layout_for(cfg).page_size_bytes, 2),
            "turbo_mse_compression_ratio_vs_fp16":
                round(fp16_page / self.make_mse_layout_for(cfg).page_size_bytes, 2),
        }

    # -- additions (include/turboquant.h part 2) ------------------------------------
    def decode_num_splits(self, batch: int, max_kv_tokens: int, cfg: TQConfig) -> int:
        return self._lib.tq_decode_num_splits(batch, max_kv_tokens, cfg.num_kv_heads, cfg.block_size)

    def decode_workspace_bytes(self, batch: int, num_q_heads: int, max_kv_tokens: int,
                               cfg: TQConfig) -> int:
        groups = -(-(num_q_heads // cfg.num_kv_heads) // 8)
        splits = self.decode_num_splits(batch * groups, max_kv_tokens, cfg)
        return self._lib.tq_decode_workspace_bytes(batch, num_q_heads, splits)

    def decode_paged(self, scheme: str, query, page_pool, block_tables, seq_lens, layout, cfg,
                     output=None, partials_out=None, max_kv_tokens: int | None = None,
                     kv_begin: int = 0, kv_end: int = INT32_MAX, workspace=None,
                     stream: int = 0):
        """Batched paged GQA decode.  query [B, Hq, 128] fp16, block_tables int32
        [B, max_pages], seq_lens int32 [B].  Returns ``output`` (fp16 [B, Hq, 128]) unless
        only ``partials_out`` (fp32 [B, Hq, 130]) was asked for."""
        _cuda(query, page_pool, block_tables, seq_lens, output, partials_out, workspace)
        b, hq, _ = query.shape
        if output is None and partials_out is None:
            output = torch.empty_like(query)
        if max_kv_tokens is None:
            max_kv_tokens = block_tables.shape[1] * cfg.block_size
        self._call(scheme, "decode_paged", self._lib.tq_decode_paged,
                   SCHEME_ID[scheme], _ptr(query), _ptr(page_pool), _ptr(block_tables),
                   block_tables.shape[1], _ptr(seq_lens), _ptr(output), _ptr(partials_out),
                   C.cast(C.byref(layout), C.c_void_p), C.byref(cfg), b, hq, max_kv_tokens,
                   kv_begin, kv_end, _ptr(workspace),
                   0 if workspace is None else workspace.numel() * workspace.element_size(),
                   C.c_void_p(stream))
        return output if output is not None else partials_out

    def decode_paged_static(self, scheme: str, query, page_pool, block_tables, seq_lens, layout,
                            cfg, output=None, max_kv_tokens: int | None = None, stream: int = 0):
        """``decode_paged`` for hosts that cannot allocate device memory while decoding (an
        engine whose own pool owns the GPU, a loop that cannot risk an allocation's implicit
        synchronisation): the split-KV scratch is a
        fixed 8 MiB array inside the library, nothing is allocated or freed.  Shapes that need
        more scratch raise; calls that may overlap on one GPU must be ordered by the caller."""
        _cuda(query, page_pool, block_tables, seq_lens, output)
        b, hq, _ = query.shape
        if output is None:
            output = torch.empty_like(query)
        if max_kv_tokens is None:
            max_kv_tokens = block_tables.shape[1] * cfg.block_size
        self._call(scheme, "decode_paged_static", self._lib.tq_decode_paged_static,
                   SCHEME_ID[scheme], _ptr(query), _ptr(page_pool), _ptr(block_tables),
                   block_tables.shape[1], _ptr(seq_lens), _ptr(output),
                   C.cast(C.byref(layout), C.c_void_p), C.byref(cfg), b, hq, max_kv_tokens,
                   C.c_void_p(stream))
        return output

    def merge_partials(self, partials, output, num_q_heads: int, num_kv_heads: int,
                       stream: int = 0):
        """partials fp32 [num_parts, rows, 130] -> output fp16 [rows, 128]."""
        _cuda(partials, output)
        parts, rows, _ = partials.shape
        self._call("merge", "partials", self._lib.tq_merge_partials, _ptr(partials), parts,
                   _ptr(output), rows, num_q_heads, num_kv_heads, C.c_void_p(stream))
        return output

    def debug_pack(self, key, value, slot_mapping, page_pool, layout, cfg, stream: int = 0) -> dict:
        """turbo_prod pack that also returns the kernel's intermediates (fp32 / int32 tensors shaped
        like ``key``): rotated K / V, clamped normalised values, level indices."""
        _cuda(key, value, slot_mapping, page_pool)
        f = lambda dt: torch.zeros(key.shape, dtype=dt, device=key.device)  # noqa: E731
        out = {"k_rot": f(torch.float32), "v_rot": f(torch.float32), "kn": f(torch.float32),
               "vn": f(torch.float32), "kidx": f(torch.int32), "vidx": f(torch.int32)}
        self._call("turbo_prod", "debug_pack_kv", self._lib.tq_debug_turbo_prod_pack_kv, _ptr(key), _ptr(value),
                   _ptr(slot_mapping), _ptr(page_pool), C.byref(layout), C.byref(cfg), key.shape[0],
                   _ptr(out["k_rot"]), _ptr(out["v_rot"]), _ptr(out["kn"]), _ptr(out["vn"]), _ptr(out["kidx"]),
                   _ptr(out["vidx"]), C.c_void_p(stream))
        return out

    def dequant_hnd(self, scheme: str, page_pool, slot_mapping, out_key, out_value, layout, cfg,
                    stream: int = 0) -> None:
        """Dequant into [H, N, 128] (the order a Hugging Face cache wants)."""
        _cuda(page_pool, slot_mapping, out_key, out_value)
        self._call(scheme, "dequant_kv_hnd", self._lib.tq_dequant_kv_hnd, SCHEME_ID[scheme],
                   _ptr(page_pool), _ptr(slot_mapping), _ptr(out_key), _ptr(out_value),
                   C.cast(C.byref(layout), C.c_void_p), C.byref(cfg), slot_mapping.shape[0],
                   C.c_void_p(stream))

    def mse_prefill_paged(self, query, page_pool, block_tables, seq_lens, chunk_key, chunk_value,
                          output, layout, cfg, stream: int = 0):
        _cuda(query, page_pool, block_tables, seq_lens, chunk_key, chunk_value, output)
        b, nq, hq, _ = query.shape
        self._call("turbo_mse", "prefill_paged", self._lib.tq_mse_prefill_paged,
                   _ptr(query), _ptr(page_pool), _ptr(block_tables), block_tables.shape[1],
                   _ptr(seq_lens), _ptr(chunk_key), _ptr(chunk_value), _ptr(output),
                   C.byref(layout), C.byref(cfg), b, nq, hq, C.c_void_p(stream))
        return output

    # -- peer exchange of split-KV partials (see turborag_b200/parallel.py: PeerExchange) --------
    def peer_buffer_bytes(self, world: int, rows_cap: int) -> int:
        return int(self._lib.tq_peer_buffer_bytes(world, rows_cap))

    def peer_publish(self, local_partials, peer_ptrs, rank: int, world: int, rows: int, rows_cap: int,
                     exchange: int, stream: int = 0) -> None:
        """``peer_ptrs``: ctypes array of ``world`` device pointers (own buffer included)."""
        _cuda(local_partials)
        self._call("kv split", "peer_publish", self._lib.tq_peer_publish, _ptr(local_partials),
                   C.cast(peer_ptrs, C.c_void_p), rank, world, rows, rows_cap, exchange, C.c_void_p(stream))

    def decode_paged_publish(self, scheme, query, page_pool, block_tables, seq_lens, layout, cfg, peer_ptrs,
                             rank: int, world: int, rows_cap: int, exchange: int, max_kv_tokens: int,
                             kv_begin: int, kv_end: int, workspace=None, stream: int = 0) -> None:
        """Decode this rank's token range and store the merged records into every peer's buffer."""
        _cuda(query, page_pool, block_tables, seq_lens, workspace)
        b, hq, _ = query.shape
        self._call(scheme, "decode_paged_publish", self._lib.tq_decode_paged_publish, SCHEME_ID[scheme],
                   _ptr(query), _ptr(page_pool), _ptr(block_tables), block_tables.shape[1], _ptr(seq_lens),
                   C.cast(C.byref(layout), C.c_void_p), C.byref(cfg), b, hq, max_kv_tokens, kv_begin, kv_end,
                   _ptr(workspace), 0 if workspace is None else workspace.numel() * workspace.element_size(),
                   C.cast(peer_ptrs, C.c_void_p), rank, world, rows_cap, exchange, C.c_void_p(stream))

    def decode_paged_exchange(self, scheme, query, page_pool, block_tables, seq_lens, layout, cfg, peer_ptrs,
                              rank: int, world: int, rows_cap: int, exchange: int, max_kv_tokens: int,
                              kv_begin: int, kv_end: int, output, workspace=None, stream: int = 0) -> None:
        """Decode this rank's token range, publish the records to every peer and merge all ranks'
        records into ``output`` ([B, Hq, 128] fp16) -- the publishing kernel finishes the exchange
        itself when the batch is small enough for its grid to be resident at once."""
        _cuda(query, page_pool, block_tables, seq_lens, workspace, output)
        b, hq, _ = query.shape
        self._call(scheme, "decode_paged_exchange", self._lib.tq_decode_paged_exchange, SCHEME_ID[scheme],
                   _ptr(query), _ptr(page_pool), _ptr(block_tables), block_tables.shape[1], _ptr(seq_lens),
                   C.cast(C.byref(layout), C.c_void_p), C.byref(cfg), b, hq, max_kv_tokens, kv_begin, kv_end,
                   _ptr(workspace), 0 if workspace is None else workspace.numel() * workspace.element_size(),
                   C.cast(peer_ptrs, C.c_void_p), rank, world, rows_cap, exchange, _ptr(output), C.c_void_p(stream))

    def peer_merge(self, my_buffer, world: int, rows: int, rows_cap: int, exchange: int, output,
                   num_q_heads: int, num_kv_heads: int, stream: int = 0) -> None:
        _cuda(my_buffer, output)
        self._call("kv split", "peer_merge", self._lib.tq_peer_merge, _ptr(my_buffer), world, rows,
                   rows_cap, exchange, _ptr(output), num_q_heads, num_kv_heads, 128, C.c_void_p(stream))

    def peer_status(self) -> int:
        return int(self._lib.tq_peer_status())

    def peer_clear_status(self) -> None:
        if self._lib.tq_peer_clear_status() != 0:
            raise RuntimeError("tq_peer_clear_status failed")

    def peer_set_wait_ns(self, ns: int) -> None:
        """Bound of the flag wait in later ``peer_merge`` calls (0 = the default 2 s)."""
        self._lib.tq_peer_set_wait_ns(int(ns))

    def mse_prefill_status(self) -> int:
        """0 when every bounded wait inside the prefill kernel was satisfied (synchronises)."""
        return int(self._lib.tq_mse_prefill_status())


class BlockTable:
    """Host page allocator + per-sequence block table (LIFO free list; slot =
    page*block_size + token_in_page, as src/tq_block_table.cpp:24-39)."""

    def __init__(self, num_pages: int, block_size: int = 16, lib: C.CDLL | None = None) -> None:
        self._lib = lib or load_library()
        self._h = self._lib.tq_block_table_create(num_pages, block_size)
        if not self._h:
            raise RuntimeError("tq_block_table_create failed")
        self.block_size = block_size

    def close(self) -> None:
        if self._h:
            self._lib.tq_block_table_destroy(self._h)
            self._h = None

    __del__ = close

    @property
    def free_pages(self) -> int:
        return self._lib.tq_block_table_free_pages(self._h)

    def append(self, seq_id: int, num_tokens: int) -> torch.Tensor:
        """Slot map (int32, CPU) for ``num_tokens`` new tokens of ``seq_id``."""
        slots = torch.empty(num_tokens, dtype=torch.int32)
        rc = self._lib.tq_block_table_append(self._h, seq_id, num_tokens,
                                             C.c_void_p(slots.data_ptr()))
        if rc != 0:
            msg = self._lib.tq_last_error()
            raise RuntimeError(msg.decode() if rc == -2 and msg else f"append failed (rc={rc})")
        return slots

    def num_tokens(self, seq_id: int) -> int:
        return self._lib.tq_block_table_num_tokens(self._h, seq_id)

    def pages(self, seq_id: int) -> torch.Tensor:
        n = -(-self.num_tokens(seq_id) // self.block_size)
        out = torch.empty(n, dtype=torch.int32)
        got = self._lib.tq_block_table_pages(self._h, seq_id, C.c_void_p(out.data_ptr()), n)
        if got < 0:
            raise RuntimeError("tq_block_table_pages failed")
        return out[:got]

    def release(self, seq_id: int) -> None:
        self._lib.tq_block_table_release(self._h, seq_id)
