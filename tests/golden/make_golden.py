"""Generate the golden fixtures in this folder from the REFERENCE's own kernels.

Needs a CUDA GPU and ``oracle/_ref/libturboquant_ref.so`` (the unmodified
reference sources compiled for sm_100 by ``make -C oracle ref``).  Run once:

    python tests/golden/make_golden.py [out_dir]          # turbo_prod / turbo_mse: <case>.npz
    python tests/golden/make_golden.py --qjl [out_dir]    # QJL-1bit: qjl_<case>.npz

For every case it draws seeded inputs with numpy, runs the reference's
pack / dequant / logits / fused-attention entry points through its C API
(src/tq_capi.cpp) and stores inputs' hashes and the reference outputs.  The
fixtures pin the CPU oracle (tests/test_oracle_golden.py); nothing here is
needed at test time except the .npz files.
"""
from __future__ import annotations

import ctypes as C
import hashlib
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
from tests.golden.cases import CASES, make_inputs  # noqa: E402


class Cfg(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("block_size", "num_kv_heads", "head_dim", "nbits",
                                       "group_size", "page_alignment", "scale_type", "quant_mode")]


class Prod(C.Structure):
    _fields_ = [(n, C.c_size_t) for n in ("page_size_bytes", "k4", "kres", "ks", "v4", "vs")] + \
               [(n, C.c_int) for n in ("kb", "vb", "sb")]


class Mse(C.Structure):
    _fields_ = [(n, C.c_size_t) for n in ("cb", "nb", "kc", "vc", "kn", "vn", "page_size_bytes")]


def p(t):
    return C.c_void_p(t.data_ptr())


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


class Qjl(C.Structure):
    _fields_ = [(n, C.c_size_t) for n in ("page_size_bytes", "k1", "ks", "v4", "vs")] + \
               [(n, C.c_int) for n in ("kb", "vb", "sb")]


def main_qjl(out_dir: Path) -> None:
    """QJL-1bit: the reference compiles the kernels (src/cuda/tq_qjl_kernels.cu) but does not
    export them; oracle/ref_qjl_shim.cu, built into the same library, forwards to its launchers."""
    out_dir.mkdir(parents=True, exist_ok=True)
    lib = C.CDLL(str(ROOT / "oracle" / "_ref" / "libturboquant_ref.so"))
    dev = torch.device("cuda:0")
    for case in CASES:
        name, n, h, nq = case["name"], case["n"], case["h"], case["nq"]
        key, value, query, slots = make_inputs(case)
        cfg, lay = Cfg(), Qjl()
        lib.tq_make_default_config(C.byref(cfg))
        cfg.num_kv_heads, cfg.head_dim = h, 128
        assert lib.tq_make_qjl_layout(C.byref(cfg), C.byref(lay)) == 0
        npages = int(slots.max()) // 16 + 1
        dk = torch.from_numpy(key.view(np.int16)).to(dev)
        dv = torch.from_numpy(value.view(np.int16)).to(dev)
        dq = torch.from_numpy(query.view(np.int16)).to(dev)
        ds = torch.from_numpy(slots).to(dev)
        pool = torch.zeros(npages * lay.page_size_bytes, dtype=torch.uint8, device=dev)
        ok = torch.zeros(n, h, 128, dtype=torch.int16, device=dev)
        ov = torch.zeros_like(ok)
        oa = torch.zeros(nq, h, 128, dtype=torch.int16, device=dev)
        assert lib.tq_launch_qjl_pack_kv(p(dk), p(dv), p(ds), p(pool), C.byref(lay), C.byref(cfg), n, None) == 0
        assert lib.tq_launch_qjl_dequant_kv(p(pool), p(ds), p(ok), p(ov), C.byref(lay), C.byref(cfg), n, None) == 0
        assert lib.tq_launch_qjl_fused_attention_output(p(dq), p(pool), p(ds), p(oa), C.byref(lay), C.byref(cfg),
                                                        nq, n, None) == 0
        torch.cuda.synchronize()
        k_np, v_np = ok.cpu().numpy().view(np.uint16), ov.cpu().numpy().view(np.uint16)
        keep = n if case.get("store_inputs") else min(n, 48)
        out = {"key_sha": sha(key), "value_sha": sha(value), "query_sha": sha(query), "slots": slots,
               "page_size_bytes": np.array([lay.page_size_bytes]), "qjl_pool": pool.cpu().numpy(),
               "qjl_dequant_sha": np.array([sha(k_np), sha(v_np)]),
               "qjl_dequant_key_head": k_np[:keep], "qjl_dequant_value_head": v_np[:keep],
               "qjl_attn": oa.cpu().numpy().view(np.uint16)}
        np.savez_compressed(out_dir / f"qjl_{name}.npz", **out)
        print("wrote", f"qjl_{name}", {k: getattr(v, "shape", None) for k, v in out.items()})


def main() -> None:
    if len(sys.argv) > 1 and sys.argv[1] == "--qjl":
        return main_qjl(Path(sys.argv[2]) if len(sys.argv) > 2 else HERE)
    out_dir = Path(sys.argv[1]) if len(sys.argv) > 1 else HERE
    out_dir.mkdir(parents=True, exist_ok=True)
    lib = C.CDLL(str(ROOT / "oracle" / "_ref" / "libturboquant_ref.so"))
    lib.tq_last_error.restype = C.c_char_p
    dev = torch.device("cuda:0")
    for case in CASES:
        name, n, h, nq = case["name"], case["n"], case["h"], case["nq"]
        key, value, query, slots = make_inputs(case)
        cfg = Cfg()
        lib.tq_make_default_config(C.byref(cfg))
        cfg.num_kv_heads, cfg.head_dim = h, 128
        prod, mse = Prod(), Mse()
        lib.tq_make_turbo_prod_layout(C.byref(cfg), C.byref(prod))
        lib.tq_make_turbo_mse_layout(C.byref(cfg), C.byref(mse))
        npages = int(slots.max()) // 16 + 1
        dk = torch.from_numpy(key.view(np.int16)).to(dev)
        dv = torch.from_numpy(value.view(np.int16)).to(dev)
        dq = torch.from_numpy(query.view(np.int16)).to(dev)
        ds = torch.from_numpy(slots).to(dev)
        out = {"key_sha": sha(key), "value_sha": sha(value), "query_sha": sha(query),
               "slots": slots}
        if case.get("store_inputs"):
            out.update(key=key.view(np.uint16), value=value.view(np.uint16),
                       query=query.view(np.uint16))
        for scheme, lay in (("prod", prod), ("mse", mse)):
            pool = torch.zeros(npages * lay.page_size_bytes, dtype=torch.uint8, device=dev)
            ok = torch.zeros(n, h, 128, dtype=torch.int16, device=dev)
            ov = torch.zeros_like(ok)
            oa = torch.zeros(nq, h, 128, dtype=torch.int16, device=dev)
            pack = getattr(lib, f"tq_launch_turbo_{scheme}_pack_kv")
            deq = getattr(lib, f"tq_launch_turbo_{scheme}_dequant_kv")
            att = getattr(lib, f"tq_launch_turbo_{scheme}_fused_attention_output")
            rc = pack(p(dk), p(dv), p(ds), p(pool), C.byref(lay), C.byref(cfg), n, None)
            assert rc == 0, lib.tq_last_error()
            rc = deq(p(pool), p(ds), p(ok), p(ov), C.byref(lay), C.byref(cfg), n, None)
            assert rc == 0, lib.tq_last_error()
            rc = att(p(dq), p(pool), p(ds), p(oa), C.byref(lay), C.byref(cfg), nq, n, None)
            assert rc == 0, lib.tq_last_error()
            torch.cuda.synchronize()
            out[f"{scheme}_pool"] = pool.cpu().numpy()
            k_np = ok.cpu().numpy().view(np.uint16)
            v_np = ov.cpu().numpy().view(np.uint16)
            out[f"{scheme}_dequant_sha"] = np.array([sha(k_np), sha(v_np)])
            keep = n if case.get("store_inputs") else min(n, 48)
            out[f"{scheme}_dequant_key_head"] = k_np[:keep]
            out[f"{scheme}_dequant_value_head"] = v_np[:keep]
            out[f"{scheme}_attn"] = oa.cpu().numpy().view(np.uint16)
            if scheme == "prod":
                lg = torch.zeros(nq * h * n, dtype=torch.float32, device=dev)
                rc = lib.tq_launch_turbo_prod_fused_attention_logits(
                    p(dq), p(pool), p(ds), p(lg), C.byref(lay), C.byref(cfg), nq, n, None)
                assert rc == 0, lib.tq_last_error()
                torch.cuda.synchronize()
                out["prod_logits"] = lg.cpu().numpy().reshape(nq, h, n)
        out["rsqrt128_bits"] = np.array(
            [int(torch.rsqrt(torch.tensor([128.0], device=dev)).cpu().numpy().view(np.uint32)[0])],
            dtype=np.uint32)
        np.savez_compressed(out_dir / f"{name}.npz", **out)
        print("wrote", name, {k: getattr(v, "shape", None) for k, v in out.items()})


if __name__ == "__main__":
    main()
