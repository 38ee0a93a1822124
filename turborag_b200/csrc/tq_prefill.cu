// Chunked query prefill over a turbo_mse-compressed prefix plus a causal fp16 chunk, sm_100a.
//
// The reference has no such kernel: its fused kernel (src/cuda/tq_turbo_mse_kernels.cu:302-417)
// takes one query row per kv head and walks the tokens serially, so a 256-token chunk with 16
// query heads would mean 2048 independent passes over the prefix.  Here the 2048 rows
// (token, query head) that share a kv head form the M dimension of a flash-attention style
// tile loop: a CTA owns 128 rows, the compressed K/V pages of 64 tokens are unpacked ONCE per
// CTA into swizzled fp16 tiles in shared memory (nibble -> fp16 by byte-permute lookups, as
// in the decode kernel), and QK^T / PV run on the tensor cores with fp32 accumulation.
// Arithmetic follows the rotated-domain formulation of the reference: q' = R(q), logits
// <q', k'>/sqrt(D), V accumulated in the rotated domain, inverse rotation at the end.  The
// chunk's own K/V (fp16) are rotated by a small pre-pass so that prefix and chunk tiles look
// the same to the main loop; a row (token i, head j) sees the whole prefix and chunk tokens
// 0..i.  Results leave as split partials (acc, m, l) and go through the decode path's merge
// kernel, which normalises, applies the inverse rotation and stores fp16.
#include <climits>
#include <cstring>

#include "tq_common.cuh"
#include "tq_launch.h"

namespace tq {
namespace {

#define TQ_ALPHA4P TQF(0x404c9252)  // table scale of the 4-bit levels (see tq_decode.cu)
constexpr float kLog2eP = 1.4426950408889634f;
constexpr float kLn2P = 0.6931471805599453f;
constexpr int kTileTokens = 64;
constexpr int kTileBytes = kTileTokens * 256;  // 64 rows x 128 fp16
constexpr int kStageBytesP = 2 * kTileBytes + 2 * kTileTokens * 4;  // K tile, V tile, two scale rows
constexpr int kQTileOff = 2 * kStageBytesP;  // Q tile after the two K/V stages
constexpr int kPrefillWarps = 8;
constexpr int kRowsPerCta = kPrefillWarps * 16;

__device__ __forceinline__ uint32_t prmt_p(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ void mma_p(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                      uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ float ex2_p(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

struct Pools {
    uint32_t hi_a, hi_b, lo_a, lo_b;
};
__device__ __forceinline__ Pools mag_pools() {
    const float t[8] = {TQ_C4_0 * TQ_ALPHA4P, TQ_C4_1 * TQ_ALPHA4P, TQ_C4_2 * TQ_ALPHA4P,
                        TQ_C4_3 * TQ_ALPHA4P, TQ_C4_4 * TQ_ALPHA4P, TQ_C4_5 * TQ_ALPHA4P,
                        TQ_C4_6 * TQ_ALPHA4P, TQ_C4_7 * TQ_ALPHA4P};
    Pools p = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const uint32_t a = __half_as_ushort(__float2half_rn(t[e]));
        const uint32_t b = __half_as_ushort(__float2half_rn(t[e + 4]));
        p.hi_a |= (a >> 8) << (8 * e);
        p.lo_a |= (a & 0xFFu) << (8 * e);
        p.hi_b |= (b >> 8) << (8 * e);
        p.lo_b |= (b & 0xFFu) << (8 * e);
    }
    return p;
}

// Eight 4-bit codes of one token -> eight fp16 levels (times alpha) in the stored order
// [0,4,1,5,2,6,3,7] of the 8-dim group (position p holds dim (p>>1) + 4(p&1)).
__device__ __forceinline__ uint4 unpack_word(uint32_t w, const Pools& t) {
    const uint32_t neg = ~w & 0x88888888u;
    uint32_t flip;
    asm("mul.hi.u32 %0, %1, %2;" : "=r"(flip) : "r"(neg), "r"(0xE0000000u));
    const uint32_t sel = (w ^ flip) & 0x77777777u;
    const uint32_t y = prmt_p(sel, sel, 0x3120u);
    const uint32_t yh = y >> 16;
    const uint32_t h0 = prmt_p(t.hi_a, t.hi_b, y), l0 = prmt_p(t.lo_a, t.lo_b, y);
    const uint32_t h1 = prmt_p(t.hi_a, t.hi_b, yh), l1 = prmt_p(t.lo_a, t.lo_b, yh);
    uint4 o;
    o.x = ((neg << 12) & 0x80008000u) ^ prmt_p(l0, h0, 0x6240u);
    o.y = ((neg << 8) & 0x80008000u) ^ prmt_p(l0, h0, 0x7351u);
    o.z = ((neg << 4) & 0x80008000u) ^ prmt_p(l1, h1, 0x6240u);
    o.w = (neg & 0x80008000u) ^ prmt_p(l1, h1, 0x7351u);
    return o;
}

// ---- pre-pass: rotate fp16 rows, R(x) * scale, stored in the permuted dim order ---------------
// rows of 128; head of row r is (r % heads_per_row_group) / group  (group = 1 for K/V rows).
__global__ void __launch_bounds__(128)
rotate_rows_kernel(const __half* __restrict__ src, __half* __restrict__ dst, long long rows,
                   int heads_mod, int group, float scale, int head_dim) {
    const int lane = threadIdx.x & 31;
    const long long row = static_cast<long long>(blockIdx.x) * 4 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int h = static_cast<int>(row % heads_mod) / group;
    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(src + row * kHeadDim) + lane);
    const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
    const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
    float x[4];
    const float a0 = f0.x - f0.y, a1 = f0.x + f0.y, a2 = f1.x - f1.y, a3 = f1.x + f1.y;
    x[0] = a0 + a2; x[2] = a0 - a2; x[1] = a1 + a3; x[3] = a1 - a3;
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float o = __shfl_xor_sync(0xffffffffu, x[e], m);
            x[e] = (lane & m) ? o - x[e] : x[e] + o;
        }
    }
    const float c = inv_sqrt_dim(head_dim);
    const float sc = ((h & 1) ? -c : c) * scale;
    // element i = 4 lane + e sits at position 8 (i/8) + perm(i%8), perm(d) = 2 (d%4) + d/4
    __half* out = dst + row * kHeadDim + 8 * (lane >> 1);
    const int d0 = 4 * (lane & 1);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const int d = d0 + e;
        out[2 * (d & 3) + (d >> 2)] = __float2half_rn(x[e] * sc);
    }
}

struct PrefillParams {
    const __half* q_rot;      // [B, Nq, Hq, 128] rotated, scaled, permuted
    const __half* ck_rot;     // [B, Nq, H, 128] or nullptr
    const __half* cv_rot;
    const uint8_t* pool;
    const int32_t* block_tables;
    const int32_t* seq_lens;
    float* partials;          // [B*Nq, splits, Hq, 130]
    PageGeom geo;
    int table_stride, nq, hq, groups, splits;
};

// Tile addressing: row = token (256 B), sixteen 16-byte units, unit index XORed with token&7.
__device__ __forceinline__ uint32_t tile_off(int token, int unit) {
    return static_cast<uint32_t>(token * 256 + ((unit ^ (token & 7)) << 4));
}

__global__ void __launch_bounds__(kPrefillWarps * 32, 1)
prefill_kernel(PrefillParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    // two stages of {K tile, V tile, K scales, V scales}
    const uint32_t smem_addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, tig = lane & 3;
    const int H = p.geo.num_kv_heads, G = p.groups;
    const int mt = blockIdx.x;
    const int h = blockIdx.y % H, split = blockIdx.y / H;
    const int b = blockIdx.z;
    const int rows_total = p.nq * G;                 // rows of this (sequence, kv head)
    const int row0 = mt * kRowsPerCta + warp * 16;   // this warp's first row
    const Pools pools = mag_pools();

    // ---- Q tile: the CTA's 128 rows (row r = token r / G, query head h*G + r % G), 32 KB, swizzled
    // like the K/V tiles; A fragments come from it with ldmatrix, one per k-step
    {
        const int r = tid >> 1, half = tid & 1;
        const int rg = min(mt * kRowsPerCta + r, rows_total - 1);
        const uint4* src = reinterpret_cast<const uint4*>(
            p.q_rot + ((static_cast<long long>(b) * p.nq + rg / G) * p.hq + h * G + rg % G) * kHeadDim) + 8 * half;
#pragma unroll
        for (int u = 0; u < 8; ++u)
            *reinterpret_cast<uint4*>(smem + kQTileOff + tile_off(r, 8 * half + u)) = __ldg(src + u);
    }
    // Per-lane ldmatrix bases.  Every matrix row this lane addresses has (row & 7) == (lane & 7), so the
    // swizzled unit (u ^ (row & 7)) only needs four pre-XORed offsets per operand; the rest of an address
    // is an immediate.
    const int lrow = lane & 7, lmat = lane >> 3;
    uint32_t offA[4], offB[4];  // offA: unit parity from bit 1 of the matrix index, offB: from bit 0
#pragma unroll
    for (int qd = 0; qd < 4; ++qd) {
        offA[qd] = static_cast<uint32_t>(((2 * qd + (lmat >> 1)) ^ lrow) << 4);
        offB[qd] = static_cast<uint32_t>(((2 * qd + (lmat & 1)) ^ lrow) << 4);
    }
    const uint32_t q_base = smem_addr + kQTileOff + (warp * 16 + lrow + 8 * (lmat & 1)) * 256;  // + offA
    const uint32_t k_row = (lrow + 8 * (lmat >> 1)) * 256;                                   // + offB
    const uint32_t v_row = (lrow + 8 * (lmat & 1)) * 256;                                    // + offA
    const int tok_a = (row0 + g) / G, tok_b = (row0 + g + 8) / G;  // chunk positions of the two rows

    float o[16][4];
#pragma unroll
    for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
    float m_run[2] = {kInitMaxLogit, kInitMaxLogit}, l_run[2] = {0.0f, 0.0f};

    // ---- this CTA's share of the prefix: tiles of 64 tokens; the last split also takes the chunk ----
    const int n_prefix = __ldg(p.seq_lens + b);
    const int prefix_tiles = (n_prefix + kTileTokens - 1) / kTileTokens;
    const int per = (prefix_tiles + p.splits - 1) / p.splits;
    const int tile_lo = split * per, tile_hi = min(prefix_tiles, tile_lo + per);
    // chunk tiles visible to this M tile: tokens 0 .. last row's token
    const int last_tok = min((mt * kRowsPerCta + kRowsPerCta - 1) / G, p.nq - 1);
    const int chunk_tiles = (p.ck_rot && split == p.splits - 1) ? last_tok / kTileTokens + 1 : 0;
    const int n_tiles = max(tile_hi - tile_lo, 0) + chunk_tiles;

    const int ut = tid & 63, uh = tid >> 6;  // unpack role: token ut of the tile, 16-byte code chunk uh (of 4)
    const int32_t* table = p.block_tables + static_cast<long long>(b) * p.table_stride;
    const int n_pref = max(tile_hi - tile_lo, 0);

    // Raw codes of one prefix tile for this thread, fetched one tile ahead of their use.
    struct Raw {
        uint4 kc, vc;
        float ks, vs;
    };
    auto fetch = [&](int it, Raw& r) {
        if (it >= n_pref) return;  // chunk tiles are copied directly in fill()
        const int t = min((tile_lo + it) * kTileTokens + ut, n_prefix - 1);
        const int page = __ldg(table + (t >> 4));
        const uint8_t* pg = p.pool + static_cast<unsigned long long>(page) * p.geo.page_size;
        const unsigned th = static_cast<unsigned>((t & 15) * H + h);
        r.kc = __ldg(reinterpret_cast<const uint4*>(pg + p.geo.k_codes + th * 64 + 16 * uh));
        r.vc = __ldg(reinterpret_cast<const uint4*>(pg + p.geo.v_codes + th * 64 + 16 * uh));
        if (uh == 0) {
            r.ks = __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short*>(pg + p.geo.k_scales + th * 2))));
            r.vs = __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short*>(pg + p.geo.v_scales + th * 2))));
        }
    };
    // Unpack (prefix) or copy (chunk) tile `it` into stage `st`.
    auto fill = [&](int it, int st, const Raw& r) {
        uint8_t* ktile = smem + st * kStageBytesP;
        uint8_t* vtile = ktile + kTileBytes;
        float* kscale = reinterpret_cast<float*>(ktile + 2 * kTileBytes);
        float* vscale = kscale + kTileTokens;
        if (it < n_pref) {
            const int t0 = (tile_lo + it) * kTileTokens;
            const uint32_t kw[4] = {r.kc.x, r.kc.y, r.kc.z, r.kc.w}, vw[4] = {r.vc.x, r.vc.y, r.vc.z, r.vc.w};
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
                *reinterpret_cast<uint4*>(ktile + tile_off(ut, 4 * uh + wi)) = unpack_word(kw[wi], pools);
                *reinterpret_cast<uint4*>(vtile + tile_off(ut, 4 * uh + wi)) = unpack_word(vw[wi], pools);
            }
            if (uh == 0) {
                const bool ok = t0 + ut < n_prefix;
                kscale[ut] = ok ? r.ks : 0.0f;
                vscale[ut] = ok ? r.vs * (1.0f / TQ_ALPHA4P) : 0.0f;
            }
        } else {
            const int t0 = (it - n_pref) * kTileTokens;
            const int t = min(t0 + ut, p.nq - 1);
            const long long rowi = (static_cast<long long>(b) * p.nq + t) * H + h;
            const uint4* ks = reinterpret_cast<const uint4*>(p.ck_rot + rowi * kHeadDim) + 4 * uh;
            const uint4* vs = reinterpret_cast<const uint4*>(p.cv_rot + rowi * kHeadDim) + 4 * uh;
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
                *reinterpret_cast<uint4*>(ktile + tile_off(ut, 4 * uh + wi)) = __ldg(ks + wi);
                *reinterpret_cast<uint4*>(vtile + tile_off(ut, 4 * uh + wi)) = __ldg(vs + wi);
            }
            if (uh == 0) {
                const bool ok = t0 + ut < p.nq;
                kscale[ut] = ok ? 1.0f : 0.0f;
                vscale[ut] = ok ? 1.0f / TQ_ALPHA4P : 0.0f;
            }
        }
    };

    Raw raw;
    raw.ks = raw.vs = 0.0f;
    raw.kc = raw.vc = make_uint4(0u, 0u, 0u, 0u);
    if (n_tiles > 0) {
        fetch(0, raw);
        fill(0, 0, raw);
        fetch(1, raw);
    }
    __syncthreads();

    for (int it = 0; it < n_tiles; ++it) {
        const int st = it & 1;
        // next tile: unpack into the other stage (ALU work that overlaps other warps' MMAs), then
        // start the loads of the tile after it; they stay in flight during the MMAs below
        if (it + 1 < n_tiles) fill(it + 1, st ^ 1, raw);
        if (it + 2 < n_tiles) fetch(it + 2, raw);

        const bool is_chunk = it >= n_pref;
        const int t0 = is_chunk ? (it - n_pref) * kTileTokens : (tile_lo + it) * kTileTokens;
        const uint32_t ktile_addr = smem_addr + st * kStageBytesP;
        const uint32_t vtile_addr = ktile_addr + kTileBytes;
        const float* kscale = reinterpret_cast<const float*>(smem + st * kStageBytesP + 2 * kTileBytes);
        const float* vscale = kscale + kTileTokens;

        // ---- S = Q K^T: 8 n-tiles of 8 tokens ----
        float s[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
        {
            uint32_t kb[4];
#pragma unroll
            for (int qd = 0; qd < 4; ++qd) kb[qd] = ktile_addr + k_row + offB[qd];
            uint32_t bf[2][4], af[4];
            ldsm4(bf[0], kb[0]);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                // A: (rows 0-7, unit 2ks), (rows 8-15, 2ks), (rows 0-7, 2ks+1), (rows 8-15, 2ks+1)
                ldsm4(af, q_base + offA[ks & 3] + 128 * (ks >> 2));
#pragma unroll
                for (int np = 0; np < 4; ++np) {
                    // B: (tokens 16np..+7, unit 2ks), (same, 2ks+1), (tokens +8.., 2ks), (+8.., 2ks+1)
                    const int idx = 4 * ks + np, nx = idx + 1;
                    if (nx < 32)
                        ldsm4(bf[nx & 1], kb[(nx >> 2) & 3] + 128 * (nx >> 4) + 4096 * (nx & 3));
                    mma_p(s[2 * np], af[0], af[1], af[2], af[3], bf[idx & 1][0], bf[idx & 1][1]);
                    mma_p(s[2 * np + 1], af[0], af[1], af[2], af[3], bf[idx & 1][2], bf[idx & 1][3]);
                }
            }
        }
        // ---- scale by the per-token K scale, mask, online softmax ----
        const int n_valid = is_chunk ? p.nq : n_prefix;
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            const float2 ksc = *reinterpret_cast<const float2*>(kscale + 8 * n + 2 * tig);
            s[n][0] *= ksc.x;
            s[n][1] *= ksc.y;
            s[n][2] *= ksc.x;
            s[n][3] *= ksc.y;
        }
        if (is_chunk || t0 + kTileTokens > n_valid) {  // only ragged or causal tiles need masks
#pragma unroll
            for (int n = 0; n < 8; ++n) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int t = t0 + 8 * n + 2 * tig + e;
                    bool va = t < n_valid, vb = va;
                    if (is_chunk) {
                        va = va && t <= tok_a;
                        vb = vb && t <= tok_b;
                    }
                    if (!va) s[n][e] = -INFINITY;
                    if (!vb) s[n][2 + e] = -INFINITY;
                }
            }
        }
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
            mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
        const float al0 = ex2_p(m_run[0] - mn0), al1 = ex2_p(m_run[1] - mn1);
        m_run[0] = mn0;
        m_run[1] = mn1;
        float ls0 = 0.0f, ls1 = 0.0f;
        uint32_t pa[4][4];  // A fragments of P (times the V scale) for the 4 k-steps of 16 tokens
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            const float p0 = ex2_p(s[n][0] - mn0), p1 = ex2_p(s[n][1] - mn0);
            const float p2 = ex2_p(s[n][2] - mn1), p3 = ex2_p(s[n][3] - mn1);
            ls0 += p0 + p1;
            ls1 += p2 + p3;
            const float2 vsc = *reinterpret_cast<const float2*>(vscale + 8 * n + 2 * tig);
            pa[n >> 1][(n & 1) * 2 + 0] = pack2(p0 * vsc.x, p1 * vsc.y);
            pa[n >> 1][(n & 1) * 2 + 1] = pack2(p2 * vsc.x, p3 * vsc.y);
        }
        l_run[0] = fmaf(l_run[0], al0, ls0);
        l_run[1] = fmaf(l_run[1], al1, ls1);
        if (__any_sync(0xffffffffu, (al0 != 1.0f) | (al1 != 1.0f))) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                o[j][0] *= al0;
                o[j][1] *= al0;
                o[j][2] *= al1;
                o[j][3] *= al1;
            }
        }
        // ---- O += P V: 16 n-tiles of 8 dims (one 16-byte unit each), 4 k-steps of 16 tokens ----
        {
            uint32_t vb[4];
#pragma unroll
            for (int qd = 0; qd < 4; ++qd) vb[qd] = vtile_addr + v_row + offA[qd];
            uint32_t bf[2][4];
            ldsm4_t(bf[0], vb[0]);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
                for (int up = 0; up < 8; ++up) {
                    // B: (tokens 16kk..+7, unit 2up), (tokens +8.., 2up), (tokens 16kk.., 2up+1), (+8.., 2up+1)
                    const int idx = 8 * kk + up, nx = idx + 1;
                    if (nx < 32)
                        ldsm4_t(bf[nx & 1], vb[nx & 3] + 128 * ((nx >> 2) & 1) + 4096 * (nx >> 3));
                    mma_p(o[2 * up], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], bf[idx & 1][0], bf[idx & 1][1]);
                    mma_p(o[2 * up + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], bf[idx & 1][2], bf[idx & 1][3]);
                }
            }
        }
        __syncthreads();  // stage st is free again, stage st^1 is complete
    }

    // ---- write the split partial of every live row: acc (natural dim order), m (natural log), l ----
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 1);
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 2);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 1);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 2);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = row0 + g + 8 * half;
        if (r >= rows_total) continue;
        // layout [sequence = (b, token)][split][query head][130], as the decode kernels write it
        const long long seq = static_cast<long long>(b) * p.nq + r / G;
        float* out = p.partials + ((seq * p.splits + split) * p.hq + h * G + r % G) * TQ_PARTIAL_STRIDE;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int pos = 2 * tig + e;  // stored position inside 8-dim group j
                out[8 * j + (pos >> 1) + 4 * (pos & 1)] = o[j][2 * half + e];
            }
        }
        if (tig == 0) {
            out[128] = m_run[half] * kLn2P;
            out[129] = l_run[half];
        }
    }
}

}  // namespace

void launch_prefill(const void* query, const uint8_t* pool, const int32_t* block_tables,
                    int table_stride, const int32_t* seq_lens, const void* chunk_key,
                    const void* chunk_value, void* output, const PageGeom& geo, int head_dim,
                    int batch, int nq, int hq, int max_prefix_tokens, cudaStream_t stream) {
    const int H = geo.num_kv_heads;
    if (batch <= 0 || nq <= 0) return;
    if (hq % H != 0) throw std::runtime_error("prefill: num_q_heads must be a multiple of num_kv_heads");
    if (geo.block_size != 16) throw std::runtime_error("prefill: block_size must be 16");
    if ((reinterpret_cast<uintptr_t>(pool) & 15) || (geo.page_size & 15) || (geo.k_codes & 15) ||
        (geo.v_codes & 15))
        throw std::runtime_error("prefill: page pool must be 16-byte aligned");
    const int G = hq / H;
    const long long q_rows = static_cast<long long>(batch) * nq * hq;
    const long long kv_rows = chunk_key ? static_cast<long long>(batch) * nq * H : 0;
    const int rows_total = nq * G;
    const int mtiles = (rows_total + kRowsPerCta - 1) / kRowsPerCta;
    const int prefix_tiles = (max_prefix_tokens + kTileTokens - 1) / kTileTokens;
    // one CTA per SM: pick the split count (up to 8) that fills whole waves best
    const int base = mtiles * H * batch, sms = sm_count();
    int splits = 1;
    double best = 0.0;
    for (int sp = 1; sp <= 8 && sp <= (prefix_tiles + 7) / 8; ++sp) {
        const double waves = static_cast<double>(base) * sp / sms;
        const double eff = waves / static_cast<double>(static_cast<long long>(waves + 0.999999));
        if (eff > best + 0.02) {
            best = eff;
            splits = sp;
        }
    }

    // workspace: rotated q, rotated chunk k/v, partials
    const size_t q_bytes = static_cast<size_t>(q_rows) * kHeadDim * 2;
    const size_t kv_bytes = static_cast<size_t>(kv_rows) * kHeadDim * 2;
    const size_t part_bytes = static_cast<size_t>(q_rows) * splits * TQ_PARTIAL_STRIDE * sizeof(float);
    auto up = [](size_t x) { return (x + 255) / 256 * 256; };
    uint8_t* ws = nullptr;
    ws = static_cast<decltype(ws)>(scratch_alloc(up(q_bytes) + 2 * up(kv_bytes) + part_bytes, stream,
                                                 "scratch_alloc(prefill workspace)"));
    __half* q_rot = reinterpret_cast<__half*>(ws);
    __half* ck_rot = reinterpret_cast<__half*>(ws + up(q_bytes));
    __half* cv_rot = reinterpret_cast<__half*>(ws + up(q_bytes) + up(kv_bytes));
    float* partials = reinterpret_cast<float*>(ws + up(q_bytes) + 2 * up(kv_bytes));

    const uint32_t alpha_bits = 0x404c9252u;
    float alpha;
    std::memcpy(&alpha, &alpha_bits, sizeof alpha);
    // q' = R(q) * (1/sqrt(D)) * log2(e) / alpha: the rotation's own 1/sqrt(D) is applied in the
    // kernel (rsqrtf), the attention scale, log2(e) and the table scale ride in `scale`
    rotate_rows_kernel<<<static_cast<unsigned>((q_rows + 3) / 4), 128, 0, stream>>>(
        static_cast<const __half*>(query), q_rot, q_rows, hq, G,
        kLog2eP / alpha * 0.08838834764831845f, head_dim);
    check_launch("prefill rotate q");
    if (chunk_key) {
        rotate_rows_kernel<<<static_cast<unsigned>((kv_rows + 3) / 4), 128, 0, stream>>>(
            static_cast<const __half*>(chunk_key), ck_rot, kv_rows, H, 1, alpha, head_dim);
        rotate_rows_kernel<<<static_cast<unsigned>((kv_rows + 3) / 4), 128, 0, stream>>>(
            static_cast<const __half*>(chunk_value), cv_rot, kv_rows, H, 1, alpha, head_dim);
        check_launch("prefill rotate chunk");
    }

    PrefillParams p{};
    p.q_rot = q_rot;
    p.ck_rot = chunk_key ? ck_rot : nullptr;
    p.cv_rot = chunk_key ? cv_rot : nullptr;
    p.pool = pool;
    p.block_tables = block_tables;
    p.seq_lens = seq_lens;
    p.partials = partials;
    p.geo = geo;
    p.table_stride = table_stride;
    p.nq = nq;
    p.hq = hq;
    p.groups = G;
    p.splits = splits;
    const size_t smem = 2 * kStageBytesP + kRowsPerCta * 256;
    static bool attr[64] = {};
    int dev = 0;
    check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (dev >= 0 && dev < 64 && !attr[dev]) {
        check_cuda(cudaFuncSetAttribute(prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(smem)), "prefill smem attr");
        attr[dev] = true;
    }
    prefill_kernel<<<dim3(mtiles, H * splits, batch), kPrefillWarps * 32, smem, stream>>>(p);
    check_launch("turbo_mse prefill");
    // rows = (b, token, q head): one "sequence" per (b, token) with hq rows; parts = splits
    launch_merge_splits(partials, splits, output, static_cast<int>(q_rows), hq, H, head_dim, stream);
    scratch_free(ws, stream, "scratch_free(prefill workspace)");
}

}  // namespace tq
