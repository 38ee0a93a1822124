"""Byte-level comparison of two page pools with the boundary accounting the parity bar
asks for: a differing code nibble is excused only if the element's normalised value lies
within one ulp of the decision boundary it crossed (midpoint of two adjacent levels for a
code, the chosen level for the residual-sign bit); fp16 scales may differ by one ulp.  Any
other differing byte (padding, cells no token maps to) is an error."""
from __future__ import annotations

import numpy as np


def _cell_offsets(scheme, lay, h_count, tib, h):
    th = tib * h_count + h
    if scheme == "turbo_prod":
        return {"k_codes": lay.k4_codes_offset + th * 64, "v_codes": lay.v4_codes_offset + th * 64,
                "scales": [lay.k_scales_offset + th * 2, lay.v_scales_offset + th * 2,
                           lay.k_residual_scales_offset + th * 2]}
    return {"k_codes": lay.k_codes_offset + th * 64, "v_codes": lay.v_codes_offset + th * 64,
            "scales": [lay.k_norms_offset + th * 2, lay.v_norms_offset + th * 2]}


def _near(x, bounds):
    x = np.float32(x)
    return bool((np.abs(x - bounds) <= np.spacing(np.abs(x))).any())


def compare_pools(oracle, scheme, mine, ref, key, value, slots, cfg):
    """Returns dict(code_mismatches, excused, unexcused, scale_ulp_max, stray_bytes)."""
    res = dict(code_mismatches=0, excused=0, unexcused=0, scale_ulp_max=0, stray_bytes=0)
    diff = mine != ref
    if not diff.any():
        return res
    lay = oracle.layout_for(scheme, cfg)
    _, kn, vn = oracle.pack(scheme, key, value, slots, cfg, trace=True)
    cb3, cb4 = oracle.cb3(), oracle.cb4()
    mid3, mid4 = (cb3[1:] + cb3[:-1]) / 2, (cb4[1:] + cb4[:-1]) / 2
    seen = np.zeros(mine.size, bool)
    H, bs = cfg.num_kv_heads, cfg.block_size
    for t, slot in enumerate(slots):
        page = (int(slot) // bs) * lay.page_size_bytes
        for h in range(H):
            off = _cell_offsets(scheme, lay, H, int(slot) % bs, h)
            for which, norm in (("k_codes", kn), ("v_codes", vn)):
                a = page + off[which]
                seen[a:a + 64] = True
                for j in np.flatnonzero(diff[a:a + 64]):
                    for half in (0, 1):
                        na = (int(mine[a + j]) >> (4 * half)) & 15
                        nb = (int(ref[a + j]) >> (4 * half)) & 15
                        if na == nb:
                            continue
                        res["code_mismatches"] += 1
                        x = norm[t, h, 2 * j + half]
                        if scheme == "turbo_prod" and which == "k_codes":
                            ok = _near(x, mid3) if (na & 7) != (nb & 7) else _near(x, cb3)
                        else:
                            ok = _near(x, mid4)
                        res["excused" if ok else "unexcused"] += 1
            for s in off["scales"]:
                a = page + s
                seen[a:a + 2] = True
                d = abs(int(mine[a:a + 2].view(np.uint16)[0]) - int(ref[a:a + 2].view(np.uint16)[0]))
                res["scale_ulp_max"] = max(res["scale_ulp_max"], d)
    res["stray_bytes"] = int((diff & ~seen).sum())
    return res


def assert_pool_parity(oracle, scheme, mine, ref, key, value, slots, cfg, label=""):
    r = compare_pools(oracle, scheme, mine, ref, key, value, slots, cfg)
    print(f"{label} {scheme}: {r}")
    assert r["unexcused"] == 0 and r["stray_bytes"] == 0 and r["scale_ulp_max"] <= 1, r
    return r
