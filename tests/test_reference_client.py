"""Drop-in acceptance on a GPU: the reference's own client code, unmodified, on this library.

`make -C oracle ref` byte-compiles the reference's ctypes wrapper and disk store
(tq_backend/turboquant_wrapper.py, tq_backend/cag_store.py) into oracle/_ref/tq_backend/; here they
are loaded from there (oracle/ref_client.py), given this library as `lib_path`, and taken through the checks of the
reference's own GPU round-trip test (tests/test_cag.py:218-252: pack a document, load and
dequantise it, shapes, dtypes, relative MSE below 0.35 / 0.25, manifest entry).  The files they
wrote are then read by this package's store, and the other way round: same bytes, same tensors."""
import json

import pytest
import torch

from oracle import ref_client

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref_client.available(),
                                 reason="oracle/_ref/tq_backend was not built (make -C oracle ref)")]

ROUNDTRIP_TOL = {"turbo_prod": 0.35, "turbo_mse": 0.25}  # tests/test_cag.py:212-215


def reference_store_class():
    return ref_client.load()[1].CAGStore


@pytest.mark.parametrize("scheme", ["turbo_prod", "turbo_mse"])
@pytest.mark.parametrize("n", [16, 1143])
def test_reference_client_round_trip_on_this_library(tmp_path, lib_path, scheme, n):
    from turborag_b200.store import CAGStore as MyStore
    RefStore = reference_store_class()
    ref = RefStore(tmp_path / "ref", lib_path=str(lib_path))
    h, d = 2, 128
    gen = torch.Generator(device="cuda")
    gen.manual_seed(n)
    key = torch.randn(n, h, d, device="cuda", generator=gen).to(torch.float16)
    val = torch.randn(n, h, d, device="cuda", generator=gen).to(torch.float16)
    ref.pack_document("rt_doc", layer=0, key=key, value=val, scheme=scheme, overwrite=True)
    assert ref.exists("rt_doc", layer=0, scheme=scheme)
    k_out, v_out = ref.load_as_kv_fp16("rt_doc", layer=0, scheme=scheme, head_shape=(h, d))
    assert k_out.shape == (n, h, d) and v_out.shape == (n, h, d)
    assert k_out.dtype == torch.float16 and v_out.dtype == torch.float16
    for x, y in ((key, k_out), (val, v_out)):
        mse = torch.mean((x.float() - y.float()) ** 2).item()
        assert mse / (torch.var(x.float()).item() + 1e-8) < ROUNDTRIP_TOL[scheme]
    manifest = json.loads((tmp_path / "ref" / "manifest.json").read_text())
    assert f"0::{scheme}" in manifest["entries"]["rt_doc"]["layers"]

    # fused attention through the reference's wrapper (its one query row per kv head)
    pool, slots, n_loaded = ref.load_document("rt_doc", layer=0, scheme=scheme, head_shape=(h, d))
    assert n_loaded == n
    q = torch.randn(1, h, d, device="cuda", generator=gen).to(torch.float16)
    out = ref.fused_attention(q, pool, slots, n, scheme, head_shape=(h, d))
    want = torch.softmax(torch.einsum("qhd,nhd->hqn", q.float(), k_out.float()) * d ** -0.5, dim=-1)
    want = torch.einsum("hqn,nhd->qhd", want, v_out.float())
    assert ((out.float() - want).abs().amax(-1) / want.abs().amax(-1)).max().item() < 5e-3

    # the two stores read each other's files: same pool bytes, same dequantised bits
    mine = MyStore(tmp_path / "mine", lib_path)
    mine.pack_document("rt_doc", 0, key, val, scheme)
    name = ref._pool_path("rt_doc", 0, scheme).name
    assert (tmp_path / "ref" / name).read_bytes() == (tmp_path / "mine" / name).read_bytes()
    cross = MyStore(tmp_path / "ref", lib_path)
    k2, v2 = cross.load_as_kv_fp16("rt_doc", 0, scheme, (h, d))
    assert torch.equal(k2, k_out) and torch.equal(v2, v_out)
    k3, v3 = ref.__class__(tmp_path / "mine", lib_path=str(lib_path)).load_as_kv_fp16(
        "rt_doc", layer=0, scheme=scheme, head_shape=(h, d))
    assert torch.equal(k3, k_out) and torch.equal(v3, v_out)
