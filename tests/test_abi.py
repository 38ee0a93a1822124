"""The C-ABI library: loads, exports every symbol include/turboquant.h declares, keeps the
reference's struct layouts and error conventions, and its host-only entry points (layouts,
block table) agree with the oracle.  No GPU: nothing here launches a kernel."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    src = (ROOT / "include" / "turboquant.h").read_text()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(tq_[a-z0-9_]+)\s*\(", src)))


def test_every_declared_symbol_is_exported(lib_path):
    lib = C.CDLL(str(lib_path))
    names = declared_symbols()
    assert len(names) >= 24 and "tq_launch_turbo_prod_pack_kv" in names
    for n in names:
        assert hasattr(lib, n), n
    from turborag_b200.wrapper import SIGNATURES
    assert sorted(SIGNATURES) == names


def test_reference_symbol_set(lib_path):
    # the 11 entry points + tq_last_error bound by tq_backend/turboquant_wrapper.py:92-173
    ref = ["tq_make_default_config", "tq_make_turbo_prod_layout", "tq_make_turbo_mse_layout",
           "tq_launch_turbo_prod_pack_kv", "tq_launch_turbo_prod_dequant_kv",
           "tq_launch_turbo_prod_fused_attention_logits", "tq_launch_turbo_prod_fused_attention_output",
           "tq_launch_turbo_mse_pack_kv", "tq_launch_turbo_mse_dequant_kv",
           "tq_launch_turbo_mse_fused_attention_output", "tq_last_error"]
    lib = C.CDLL(str(lib_path))
    for n in ref:
        assert hasattr(lib, n)


def test_struct_sizes_and_default_config(tq):
    from turborag_b200 import TQConfig, TQTurbomsePageLayout, TQTurboProdPageLayout
    assert C.sizeof(TQConfig) == 32 and C.sizeof(TQTurboProdPageLayout) == 64
    assert C.sizeof(TQTurbomsePageLayout) == 56
    cfg = tq.default_config()
    assert [getattr(cfg, f) for f, _ in cfg._fields_] == [16, 8, 128, 4, 128, 256, 0, 0]
    assert tq.summary()["turbo_prod_compression_ratio_vs_fp16"] == 3.82


def test_layouts_match_oracle(tq, oracle):
    for h in (1, 2, 3, 4, 8, 32):
        for bs in (1, 8, 16, 32):
            for d in (64, 128):
                cfg = tq.default_config()
                cfg.num_kv_heads, cfg.block_size, cfg.head_dim = h, bs, d
                ocfg = oracle.make_config(h, d)
                ocfg.block_size = bs
                assert bytes(tq.make_layout_for(cfg))[:60] == bytes(oracle.prod_layout(ocfg))[:60]
                assert bytes(tq.make_mse_layout_for(cfg)) == bytes(oracle.mse_layout(ocfg))


def test_null_arguments_return_minus_one(tq):
    L = tq._lib
    cfg = tq.default_config()
    lay = tq.make_layout_for(cfg)
    assert L.tq_make_default_config(None) == -1
    assert L.tq_make_turbo_prod_layout(None, C.byref(lay)) == -1
    assert L.tq_make_turbo_mse_layout(C.byref(cfg), None) == -1
    one = C.c_void_p(16)
    assert L.tq_launch_turbo_prod_pack_kv(None, one, one, one, C.byref(lay), C.byref(cfg), 1, None) == -1
    assert L.tq_launch_turbo_prod_dequant_kv(one, one, one, None, C.byref(lay), C.byref(cfg), 1, None) == -1
    assert L.tq_launch_turbo_prod_fused_attention_output(one, one, one, one, None, C.byref(cfg), 1, 1, None) == -1
    mlay = tq.make_mse_layout_for(cfg)
    assert L.tq_launch_turbo_mse_pack_kv(one, one, None, one, C.byref(mlay), C.byref(cfg), 1, None) == -1
    assert L.tq_merge_partials(None, 1, one, 1, 1, 1, None) == -1


def test_unsupported_shape_is_minus_two_with_message(tq):
    L = tq._lib
    cfg = tq.default_config()
    cfg.head_dim = 256
    lay = tq.make_layout_for(cfg)
    p = C.c_void_p(256)
    assert L.tq_launch_turbo_prod_pack_kv(p, p, p, p, C.byref(lay), C.byref(cfg), 4, None) == -2
    assert b"head_dim > 128" in L.tq_last_error()  # src/cuda/tq_turbo_prod_kernels.cu:595-596
    cfg.head_dim = 64
    lay = tq.make_layout_for(cfg)
    assert L.tq_launch_turbo_prod_dequant_kv(p, p, p, p, C.byref(lay), C.byref(cfg), 4, None) == -2
    assert b"head_dim" in L.tq_last_error()
    with pytest.raises(RuntimeError, match="CUDA error"):
        tq._kernel_raise(-2, "turbo_prod", "pack_kv")
    with pytest.raises(RuntimeError, match="rc=-1"):
        tq._kernel_raise(-1, "turbo_prod", "pack_kv")


def test_missing_library_raises():
    import turborag_b200
    with pytest.raises(FileNotFoundError):
        turborag_b200.TurboQuantWrapper("/nonexistent/libturboquant.so")


def test_no_cpu_path(tq):
    import torch
    cfg = tq.default_config()
    cfg.num_kv_heads = 2
    lay = tq.make_layout_for(cfg)
    k = torch.zeros(4, 2, 128, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        tq.pack(k, k, torch.zeros(4, dtype=torch.int32), torch.zeros(4288, dtype=torch.uint8), lay, cfg)


def test_block_table_matches_reference_formula(tq, oracle):
    from turborag_b200 import BlockTable
    bt = BlockTable(10, 16)
    s0 = bt.append(0, 20).numpy()
    s1 = bt.append(1, 5).numpy()
    s0b = bt.append(0, 30).numpy()
    # LIFO free list hands out pages 0,1,2,... (src/tq_allocator.cpp:5-31)
    assert bt.pages(0).tolist() == [0, 1, 3, 4] and bt.pages(1).tolist() == [2]
    exp = np.zeros(50, np.int32)
    oracle.lib().orc_build_slot_map(np.array([0, 1, 3, 4], np.int32).ctypes.data_as(C.c_void_p),
                                    0, 50, 16, exp.ctypes.data_as(C.c_void_p))
    assert (np.concatenate([s0, s0b]) == exp).all()
    assert (s1 == 2 * 16 + np.arange(5)).all()
    assert bt.num_tokens(0) == 50 and bt.free_pages == 5
    with pytest.raises(RuntimeError, match="out of blocks"):  # src/tq_block_table.cpp:17-19
        bt.append(2, 16 * 6)
    assert bt.free_pages == 5
    bt.release(0)
    assert bt.free_pages == 9 and bt.num_tokens(0) == 0
    assert bt.append(3, 1).tolist() == [0]  # most recently freed page first


def test_decode_split_heuristic(tq):
    cfg = tq.default_config()
    cfg.num_kv_heads = 2
    s = tq.decode_num_splits(32, 32768, cfg)
    assert 1 <= s <= 64
    assert tq.decode_num_splits(32, 16, cfg) == 1
    assert tq._lib.tq_decode_workspace_bytes(32, 16, s) == 32 * 16 * s * 130 * 4
