// Dequant kernels (compressed pages -> fp16 K/V) for sm_100a.
//
// Replaces turbo_prod_dequant_kv_kernel (src/cuda/tq_turbo_prod_kernels.cu:265-341)
// and turbo_mse_dequant_kv_kernel (src/cuda/tq_turbo_mse_kernels.cu:239-287).  Same
// register-resident transform as the pack kernels, run in the inverse
// direction: 8 code bytes per lane are expanded through a bank-replicated
// shared-memory codebook, stages 1..8 run in registers, one re-deal, stages
// 16..64, then every lane stores eight half2 values; the eight lanes of a row
// cover one 32-byte sector per store.  Output is bit-identical to the
// reference.  An [H, N, D] output order is available for Hugging Face caches.
// The QJL-1bit scheme (qjl_dequant_kv_kernel, src/cuda/tq_qjl_kernels.cu:172-244) is the third
// instance: K is one sign bit per dimension times the row's RMS, V as in turbo_prod, and the
// rotation has no per-head sign.
#include <climits>
#include <stdexcept>
#include <type_traits>
#include "tq_common.cuh"
#include "tq_launch.h"

namespace tq {
namespace {

constexpr int kDqWarps = 8;

__constant__ float kLevels3[8] = {-2.1513f,  -1.34326f, -0.755526f, -0.244919f,
                                  0.244919f, 0.755526f, 1.34326f,   2.1513f};
__constant__ float kLevels4[16] = {-2.7326f, -2.0690f, -1.6180f, -1.2562f, -0.9423f, -0.6568f,
                                   -0.3880f, -0.1284f, 0.1284f,  0.3880f,  0.6568f,  0.9423f,
                                   1.2562f,  1.6180f,  2.0690f,  2.7326f};

// (a & b) | c and (a & b) ^ c as one three-input logic instruction each.
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t lop3_and_xor(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ uint2 load_codes(const uint8_t* p, bool aligned8) {
    if (aligned8) return __ldcs(reinterpret_cast<const uint2*>(p));
    uint2 v = make_uint2(0u, 0u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v.x |= static_cast<uint32_t>(p[i]) << (8 * i);
        v.y |= static_cast<uint32_t>(p[4 + i]) << (8 * i);
    }
    return v;
}

// Inverse rotation of 16 rotated-domain values per lane and fp16 store.
__device__ __forceinline__ void inverse_and_store(float2 (&x)[8], float* buf, int lane, float c,
                                                  int h, __half* dst_row, bool valid) {
    float2 y[8];
    fwht_phase1(x);
    redeal(x, y, buf, lane);
    fwht_phase2(y);
    const int l = lane & 7;
    // element 2l+b+16j has sign +1 iff (b+h) is even; (y*c)*s == y*(c*s) exactly
    const float s0 = (h & 1) ? -c : c;
    const float2 cs = make_float2(s0, -s0);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float2 v = mul2(y[j], cs);
        if (valid)
            *reinterpret_cast<__half2*>(dst_row + 2 * l + 16 * j) = __floats2half2_rn(v.x, v.y);
    }
}

// S: 0 turbo_prod, 1 turbo_mse, 2 QJL-1bit.  ALIGNED8: pool base and page size are multiples of
// 8 bytes, so a lane's 8 code bytes are one load.  It is a template argument because as a run-time
// flag both load sequences end up in the instruction stream, predicated.
// POW2: kv head count and tokens per page are powers of two, so the index divisions are shifts.
template <int S, bool ALIGNED8, bool POW2>
__global__ void __launch_bounds__(kDqWarps * 32)
dequant_kv_kernel(const uint8_t* __restrict__ page_pool, const int32_t* __restrict__ slot_mapping,
                  __half* __restrict__ out_key, __half* __restrict__ out_value, PageGeom geo,
                  IndexDiv div_heads, IndexDiv div_block, int head_dim, int num_rows,
                  int num_tokens, int hnd) {
    __shared__ __align__(16) float xchg[kDqWarps][kXchgWarpFloats];
    __shared__ float lut3[8 * 32];
    __shared__ float lut4[16 * 32];
    constexpr bool PROD = S == 0, QJL = S == 2;
    for (int i = threadIdx.x; i < 8 * 32; i += blockDim.x) lut3[i] = kLevels3[i >> 5];
    for (int i = threadIdx.x; i < 16 * 32; i += blockDim.x) lut4[i] = kLevels4[i >> 5];
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rr = lane >> 3, l = lane & 7;
    float* buf = xchg[warp];
    const int H = geo.num_kv_heads;
    const float c = inv_sqrt_dim(head_dim);
    const int groups = (num_rows + 3) >> 2;  // rows are counted in 32 bits (checked by the launcher)
    const int warps_total = static_cast<int>(gridDim.x) * kDqWarps;
    constexpr bool al = ALIGNED8;
    const unsigned long long slots64 = reinterpret_cast<unsigned long long>(slot_mapping);
    const unsigned long long pool64 = reinterpret_cast<unsigned long long>(page_pool);
    const unsigned int page_size32 = static_cast<unsigned int>(geo.page_size);

    // Packed inputs of one row group for this lane, software-pipelined two deep so that neither
    // link of the dependent chain slot -> page -> codes is waited for: iteration i loads the slot of
    // group i + 2, issues the page loads of group i + 1 (whose slot arrived during iteration i - 1)
    // and expands group i.  Scales stay raw fp16 bits until they are used: a conversion placed next to
    // its load would wait for the load inside the prefetch.
    struct Raw {
        uint2 kc, vc;
        unsigned short ks, vs, re;
        int out_row;
        int h;
        bool valid;
    };
    struct Slot {
        int row, tok;
        int slot;
        bool valid;
    };
    auto fetch_slot = [&](int g, Slot& sl) {
        const int row_raw = g * 4 + rr;
        sl.valid = row_raw < num_rows;
        sl.row = sl.valid ? row_raw : num_rows - 1;
        sl.tok = POW2 ? (sl.row >> div_heads.shift) : sl.row / H;
        sl.slot = __ldg(reinterpret_cast<const int32_t*>(mad_wide(sl.tok, 4u, slots64)));
    };
    auto fetch = [&](const Slot& sl, Raw& r) {
        r.valid = sl.valid;
        r.h = sl.row - sl.tok * H;
        const int blk = POW2 ? (sl.slot >> div_block.shift) : sl.slot / geo.block_size;
        const int tib = sl.slot - blk * geo.block_size;
        const uint8_t* page = reinterpret_cast<const uint8_t*>(mad_wide(blk, page_size32, pool64));
        const unsigned int th = static_cast<unsigned int>(tib * H + r.h);
        if (QJL)  // 16 sign bits: dims 16l .. 16l+15
            r.kc = make_uint2(__ldg(reinterpret_cast<const unsigned short*>(page + geo.k_codes + th * 16 + 2 * l)), 0u);
        else
            r.kc = load_codes(page + geo.k_codes + th * 64 + 8 * l, al);
        r.vc = load_codes(page + geo.v_codes + th * 64 + 8 * l, al);
        r.ks = __ldg(reinterpret_cast<const unsigned short*>(page + geo.k_scales + th * 2));
        r.vs = __ldg(reinterpret_cast<const unsigned short*>(page + geo.v_scales + th * 2));
        r.re = PROD ? __ldg(reinterpret_cast<const unsigned short*>(page + geo.k_res + th * 2)) : static_cast<unsigned short>(0);
        r.out_row = hnd ? r.h * num_tokens + sl.tok : sl.row;
    };
    auto widen = [](unsigned short bits) { return __half2float(__ushort_as_half(bits)); };

    int g = blockIdx.x * kDqWarps + warp;
    Raw cur{}, nxt{};
    Slot s1{}, s2{};
    if (g < groups) {
        fetch_slot(g, s1);
        fetch(s1, cur);
    }
    if (g + warps_total < groups) {
        fetch_slot(g + warps_total, s1);
        fetch(s1, nxt);
    }
    if (g + 2 * warps_total < groups) fetch_slot(g + 2 * warps_total, s2);
    for (; g < groups; g += warps_total) {
        // group i + 2: its slot was loaded an iteration ago, its page loads start now; group i + 3: slot
        Raw nn = nxt;
        if (g + 2 * warps_total < groups) fetch(s2, nn);
        if (g + 3 * warps_total < groups) fetch_slot(g + 3 * warps_total, s2);

        const float re = widen(cur.re), ks = widen(cur.ks), vs = widen(cur.vs);
        const int h = QJL ? 0 : cur.h;  // the QJL rotation has no head term (tq_qjl_kernels.cu:18-21)
        float2 x[8];
        // Level of nibble J of code word w: the table row (128 bytes of replicas) is nibble * 128, this lane's
        // replica lane * 4 -- one shift and one and-or form the byte address.  turbo_prod K: 3-bit code, and the
        // residual term +-re takes its sign from bit 3 of the nibble (set = +) by one shift and one and-xor.
        const uint32_t lane4 = lane * 4u;
        const uint32_t re_neg = __float_as_uint(re) | 0x80000000u;
        auto level4 = [&](uint32_t w, auto jc) {
            constexpr int J = decltype(jc)::value;
            const uint32_t t = J >= 2 ? (w >> (4 * J - 7)) : (w << (7 - 4 * J));
            return *reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(lut4) + lop3_and_or(t, 0x780u, lane4));
        };
        auto level_k = [&](uint32_t w, auto jc) {
            constexpr int J = decltype(jc)::value;
            if (!PROD) return level4(w, jc);
            const uint32_t t = J >= 2 ? (w >> (4 * J - 7)) : (w << (7 - 4 * J));
            const float lv = *reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(lut3) + lop3_and_or(t, 0x380u, lane4));
            const uint32_t sg = J == 7 ? w : (w << (28 - 4 * J));  // bit 3 of the nibble at bit 31
            return __fadd_rn(lv, __uint_as_float(lop3_and_xor(sg, 0x80000000u, re_neg)));
        };
        // K: rotated-domain values (tq_turbo_prod_kernels.cu:315-330 /
        // tq_turbo_mse_kernels.cu:150-156)
        const float2 ks2 = make_float2(ks, ks), vs2 = make_float2(vs, vs);
#define TQ_DQ_PAIR(FN, W, K) make_float2(FN(W, std::integral_constant<int, 2 * ((K) & 3)>{}), \
                                         FN(W, std::integral_constant<int, 2 * ((K) & 3) + 1>{}))
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (QJL) {  // (bit ? +1 : -1) * ks   (tq_qjl_kernels.cu:235)
                x[k] = make_float2((cur.kc.x >> (2 * k)) & 1u ? ks : -ks,
                                   (cur.kc.x >> (2 * k + 1)) & 1u ? ks : -ks);
            }
        }
        if (!QJL) {
            x[0] = mul2(TQ_DQ_PAIR(level_k, cur.kc.x, 0), ks2);
            x[1] = mul2(TQ_DQ_PAIR(level_k, cur.kc.x, 1), ks2);
            x[2] = mul2(TQ_DQ_PAIR(level_k, cur.kc.x, 2), ks2);
            x[3] = mul2(TQ_DQ_PAIR(level_k, cur.kc.x, 3), ks2);
            x[4] = mul2(TQ_DQ_PAIR(level_k, cur.kc.y, 0), ks2);
            x[5] = mul2(TQ_DQ_PAIR(level_k, cur.kc.y, 1), ks2);
            x[6] = mul2(TQ_DQ_PAIR(level_k, cur.kc.y, 2), ks2);
            x[7] = mul2(TQ_DQ_PAIR(level_k, cur.kc.y, 3), ks2);
        }
        inverse_and_store(x, buf, lane, c, h, out_key + static_cast<long long>(cur.out_row) * kHeadDim, cur.valid);

        x[0] = mul2(TQ_DQ_PAIR(level4, cur.vc.x, 0), vs2);
        x[1] = mul2(TQ_DQ_PAIR(level4, cur.vc.x, 1), vs2);
        x[2] = mul2(TQ_DQ_PAIR(level4, cur.vc.x, 2), vs2);
        x[3] = mul2(TQ_DQ_PAIR(level4, cur.vc.x, 3), vs2);
        x[4] = mul2(TQ_DQ_PAIR(level4, cur.vc.y, 0), vs2);
        x[5] = mul2(TQ_DQ_PAIR(level4, cur.vc.y, 1), vs2);
        x[6] = mul2(TQ_DQ_PAIR(level4, cur.vc.y, 2), vs2);
        x[7] = mul2(TQ_DQ_PAIR(level4, cur.vc.y, 3), vs2);
#undef TQ_DQ_PAIR
        inverse_and_store(x, buf, lane, c, h, out_value + static_cast<long long>(cur.out_row) * kHeadDim, cur.valid);
        cur = nxt;
        nxt = nn;
    }
}

}  // namespace

void launch_dequant(int scheme, const uint8_t* pool, const int32_t* slots, void* out_key,
                    void* out_value, const PageGeom& geo, int head_dim, int num_tokens, bool hnd,
                    cudaStream_t stream) {
    if (num_tokens <= 0) return;
    const long long rows = static_cast<long long>(num_tokens) * geo.num_kv_heads;
    const long long groups = (rows + 3) / 4;
    long long blocks = (groups + kDqWarps - 1) / kDqWarps;
    const long long cap = static_cast<long long>(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    const bool aligned = (reinterpret_cast<uintptr_t>(pool) & 7) == 0 && (geo.page_size & 7) == 0;
    if (rows > INT_MAX) throw std::runtime_error("dequant: more than 2^31 - 1 token-heads in one call");
    const IndexDiv dh = make_index_div(geo.num_kv_heads), db = make_index_div(geo.block_size);
    const bool pow2 = dh.shift >= 0 && db.shift >= 0;
#define TQ_DEQUANT_LAUNCH2(SV, AL, P2)                                                            \
    dequant_kv_kernel<SV, AL, P2><<<static_cast<unsigned>(blocks), kDqWarps * 32, 0, stream>>>(     \
        pool, slots, static_cast<__half*>(out_key), static_cast<__half*>(out_value), geo, dh, db,  \
        head_dim, static_cast<int>(rows), num_tokens, hnd ? 1 : 0)
#define TQ_DEQUANT_LAUNCH(SV)                                                                     \
    do {                                                                                          \
        if (aligned && pow2) TQ_DEQUANT_LAUNCH2(SV, true, true);                                  \
        else if (aligned) TQ_DEQUANT_LAUNCH2(SV, true, false);                                    \
        else if (pow2) TQ_DEQUANT_LAUNCH2(SV, false, true);                                       \
        else TQ_DEQUANT_LAUNCH2(SV, false, false);                                                \
    } while (0)
    if (scheme == TQ_SCHEME_TURBO_PROD) TQ_DEQUANT_LAUNCH(0);
    else if (scheme == TQ_SCHEME_TURBO_MSE) TQ_DEQUANT_LAUNCH(1);
    else TQ_DEQUANT_LAUNCH(2);
#undef TQ_DEQUANT_LAUNCH
#undef TQ_DEQUANT_LAUNCH2
    check_launch(scheme == TQ_SCHEME_TURBO_PROD ? "turbo_prod dequant_kv"
                 : scheme == TQ_SCHEME_TURBO_MSE ? "turbo_mse dequant_kv" : "qjl dequant_kv");
}

}  // namespace tq
