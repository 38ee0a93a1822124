// Quantize + pack kernels (turbo_prod and turbo_mse) for sm_100a.
//
// Replaces turbo_prod_pack_kv_kernel (src/cuda/tq_turbo_prod_kernels.cu:110-260)
// and turbo_mse_pack_kv_kernel (src/cuda/tq_turbo_mse_kernels.cu:186-237) of the
// reference with one register-resident design: a warp owns four token-heads at
// a time (8 lanes x 16 elements each), inputs arrive as 16-byte vector loads,
// the 128-point transform runs in registers around one shared-memory re-deal,
// and code bytes leave as 8-byte stores (64 contiguous bytes per token-head).
// Results are bit-identical to the reference's arithmetic; see tq_common.cuh.
#include "tq_common.cuh"
#include "tq_launch.h"

namespace tq {
namespace {

constexpr int kPackWarps = 8;
constexpr int kCodeRowBytes = 72;  // 64 code bytes + pad: rows land on distinct banks

__device__ __forceinline__ uint4 ld_stream(const uint4* p) { return __ldcs(p); }

// ---- nearest-level search through bank-replicated shared tables ---------------------------
// The threshold search is the kernel's largest cost and runs on the half-rate integer/compare
// pipe, while the load/store pipe is mostly idle.  |x| (clamped) is cut into 16 cells of
// width 3/16; each cell holds at most one decision threshold, so a table entry (threshold
// inside the cell or +inf, code below it) plus ONE compare gives the exact code.  Entries
// exist per sign class (the thresholds of the negative half differ by an ulp where an exact
// fp32 tie exists) and are replicated over the 32 lanes, so lookups never conflict.
constexpr float kCellScale = 16.0f / 3.0f;
constexpr float kCellMagic = 8388608.0f;  // 2^23: the fma's low mantissa bits are round(|x| * scale)
constexpr float kCellClamp = 2.8125f;     // 15 cells

struct CellInfo {
    float t;   // threshold inside the cell, +inf if none
    int base;  // thresholds below the cell
};
template <int N>
__device__ __forceinline__ CellInfo cell_info(const float (&thr)[N], int cell) {
    CellInfo c{__int_as_float(0x7f800000), 0};
#pragma unroll
    for (int j = 0; j < N; ++j) {
        const int cj = __float2int_rn(thr[j] * kCellScale);
        if (cj < cell) ++c.base;
        if (cj == cell) c.t = thr[j];
    }
    return c;
}

// lutV[(sign*16 + cell)*32 + lane] = (threshold, code if below it; +1 when (above == positive))
// lutK[...]                       = (threshold, level below, level above, code as for lutV)
__device__ void build_luts(float4* lutK, float2* lutV, bool need_k) {
    const float k3m[3] = {TQ_K3_M1, TQ_K3_M2, TQ_K3_M3}, k3n[3] = {TQ_K3_N1, TQ_K3_N2, TQ_K3_N3};
    const float v4m[7] = {TQ_V4_M1, TQ_V4_M2, TQ_V4_M3, TQ_V4_M4, TQ_V4_M5, TQ_V4_M6, TQ_V4_M7};
    const float v4n[7] = {TQ_V4_N1, TQ_V4_N2, TQ_V4_N3, TQ_V4_N4, TQ_V4_N5, TQ_V4_N6, TQ_V4_N7};
    const float lv3[4] = {TQ_C3_0, TQ_C3_1, TQ_C3_2, TQ_C3_3};
    for (int i = threadIdx.x; i < 2 * 16 * 32; i += blockDim.x) {
        const int cell = (i >> 5) & 15;
        const bool neg = (i >> 9) != 0;
        const CellInfo v = neg ? cell_info(v4n, cell) : cell_info(v4m, cell);
        lutV[i] = make_float2(v.t, __int_as_float(neg ? 6 - v.base : 8 + v.base));
        if (need_k) {
            const CellInfo k = neg ? cell_info(k3n, cell) : cell_info(k3m, cell);
            const int hi = k.base < 3 ? k.base + 1 : 3;
            lutK[i] = make_float4(k.t, lv3[k.base], lv3[hi], __int_as_float(neg ? 2 - k.base : 4 + k.base));
        }
    }
}

__device__ __forceinline__ uint32_t cell_index(float a, float x) {
    const float u = __fmaf_rn(a, kCellScale, kCellMagic);
    return (__float_as_uint(u) & 31u) + (x >= TQ_TMID ? 0u : 16u);
}

// 4-bit code (nearest_v4_idx / nearest_codebook_idx of the reference), exact.
__device__ __forceinline__ uint32_t quant_v4_lut(float x, const float2* lutV, int lane) {
    const float a = fabsf(x);
    const bool pos = x >= TQ_TMID;
    const float2 e = lutV[cell_index(fminf(a, kCellClamp), x) * 32 + lane];
    return __float_as_uint(e.y) + (((a >= e.x) == pos) ? 1u : 0u);
}

// K nibble = residual sign << 3 | 3-bit code, and the residual e = clamp(kn) - level.
__device__ __forceinline__ uint32_t quant_k3_lut(float kn, const float4* lutK, int lane, float& e) {
    const float a = fminf(fabsf(kn), 2.5f);  // |clamp(kn, -2.5, 2.5)|
    const bool pos = kn >= TQ_TMID;
    const float4 t = lutK[cell_index(a, kn) * 32 + lane];
    const bool above = a >= t.x;
    const float lvl = above ? t.z : t.y;
    e = __fadd_rn(copysignf(a, kn), pos ? -lvl : lvl);
    return (__float_as_uint(t.w) + ((above == pos) ? 1u : 0u)) | (e >= 0.0f ? 8u : 0u);
}

// Move a row's 64 code bytes from "lane l' holds byte l'+8j" to "lane l holds
// bytes 8l..8l+7" through a per-warp byte buffer, then store them.
__device__ __forceinline__ void store_codes(const uint32_t (&byte_j)[8], uint8_t* code_buf,
                                            uint8_t* dst, int lane, bool valid, bool aligned8) {
    const int rr = lane >> 3, l = lane & 7;
    uint8_t* row = code_buf + rr * kCodeRowBytes;
#pragma unroll
    for (int j = 0; j < 8; ++j) row[l + 8 * j] = static_cast<uint8_t>(byte_j[j]);
    __syncwarp();
    const uint2 v = *reinterpret_cast<const uint2*>(row + 8 * l);
    __syncwarp();
    if (!valid) return;
    if (aligned8) {
        *reinterpret_cast<uint2*>(dst + 8 * l) = v;
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            dst[8 * l + i] = static_cast<uint8_t>(v.x >> (8 * i));
            dst[8 * l + 4 + i] = static_cast<uint8_t>(v.y >> (8 * i));
        }
    }
}

template <bool PROD>
__global__ void __launch_bounds__(kPackWarps * 32)
pack_kv_kernel(const uint4* __restrict__ key, const uint4* __restrict__ value,
               const int32_t* __restrict__ slot_mapping, uint8_t* __restrict__ page_pool,
               PageGeom geo, int head_dim, long long num_rows, int pool_aligned8) {
    __shared__ __align__(16) float xchg[kPackWarps][kXchgWarpFloats];
    __shared__ __align__(16) float4 lutK[PROD ? 2 * 16 * 32 : 1];
    __shared__ __align__(16) float2 lutV[2 * 16 * 32];
    build_luts(lutK, lutV, PROD);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rr = lane >> 3, l = lane & 7;
    float* buf = xchg[warp];
    uint8_t* code_buf = reinterpret_cast<uint8_t*>(buf);
    const int H = geo.num_kv_heads;
    const float c = inv_sqrt_dim(head_dim);
    const long long groups = (num_rows + 3) >> 2;
    const long long warps_total = static_cast<long long>(gridDim.x) * kPackWarps;

    for (long long g = static_cast<long long>(blockIdx.x) * kPackWarps + warp; g < groups;
         g += warps_total) {
        const long long row_raw = g * 4 + rr;
        const bool valid = row_raw < num_rows;
        const long long row = valid ? row_raw : num_rows - 1;  // keep all lanes converged
        const long long tok = row / H;
        const int h = static_cast<int>(row - tok * H);
        const float cs = (h & 1) ? -c : c;  // odd heads: the whole rotated row is negated

        const uint4* kp = key + row * 16 + 2 * l;
        const uint4* vp = value + row * 16 + 2 * l;
        const uint4 k_lo = ld_stream(kp), k_hi = ld_stream(kp + 1);
        const uint4 v_lo = ld_stream(vp), v_hi = ld_stream(vp + 1);
        const int slot = __ldg(slot_mapping + tok);

        const int blk = slot / geo.block_size;
        const int tib = slot - blk * geo.block_size;
        uint8_t* page = page_pool + static_cast<unsigned long long>(blk) * geo.page_size;
        const unsigned int th = static_cast<unsigned int>(tib * H + h);

        float2 x[8], y[8];

        // ---------------- K ----------------
        fwht_phase1_from_half(k_lo, k_hi, x);
        redeal(x, y, buf, lane);
        fwht_phase2(y);
        const float2 cs2 = make_float2(cs, cs);
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = mul2(y[j], cs2);

        uint32_t kbytes[8];
        if (PROD) {
            float2 sq[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) sq[j] = mul2(y[j], y[j]);
            const float krms = rms_from_sum(tree128(sq));
            const float kr = __frcp_rn(krms);
            float2 e2[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float e0, e1;
                const float2 kn = div_by2(y[j], krms, kr);
                const uint32_t n0 = quant_k3_lut(kn.x, lutK, lane, e0);
                const uint32_t n1 = quant_k3_lut(kn.y, lutK, lane, e1);
                kbytes[j] = n0 | (n1 << 4);
                const float2 e = make_float2(e0, e1);
                e2[j] = mul2(e, e);
            }
            const float rms_e = rms_from_sum(tree128(e2));
            if (valid && l == 0) {
                *reinterpret_cast<__half*>(page + geo.k_scales + th * 2) = __float2half_rn(krms);
                *reinterpret_cast<__half*>(page + geo.k_res + th * 2) = __float2half_rn(rms_e);
            }
        } else {
            float pr[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                pr[j] = __fmaf_rn(y[j].x, y[j].x, __fmul_rn(y[j].y, y[j].y));
            const float krms = rms_from_sum(tree64(pr));
            const float kr = __frcp_rn(krms);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float2 kn = div_by2(y[j], krms, kr);
                kbytes[j] = quant_v4_lut(kn.x, lutV, lane) | (quant_v4_lut(kn.y, lutV, lane) << 4);
            }
            if (valid && l == 0)
                *reinterpret_cast<__half*>(page + geo.k_scales + th * 2) = __float2half_rn(krms);
        }
        store_codes(kbytes, code_buf, page + geo.k_codes + th * 64, lane, valid,
                    pool_aligned8 != 0);

        // ---------------- V ----------------
        fwht_phase1_from_half(v_lo, v_hi, x);
        redeal(x, y, buf, lane);
        fwht_phase2(y);
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = mul2(y[j], cs2);
        float vrms;
        if (PROD) {
            float2 sq[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) sq[j] = mul2(y[j], y[j]);
            vrms = rms_from_sum(tree128(sq));
        } else {
            float pr[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                pr[j] = __fmaf_rn(y[j].x, y[j].x, __fmul_rn(y[j].y, y[j].y));
            vrms = rms_from_sum(tree64(pr));
        }
        const float vr = __frcp_rn(vrms);
        uint32_t vbytes[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float2 vn = div_by2(y[j], vrms, vr);
            vbytes[j] = quant_v4_lut(vn.x, lutV, lane) | (quant_v4_lut(vn.y, lutV, lane) << 4);
        }
        if (valid && l == 0)
            *reinterpret_cast<__half*>(page + geo.v_scales + th * 2) = __float2half_rn(vrms);
        store_codes(vbytes, code_buf, page + geo.v_codes + th * 64, lane, valid,
                    pool_aligned8 != 0);
    }
}

}  // namespace

void launch_pack(bool prod, const void* key, const void* value, const int32_t* slots,
                 uint8_t* pool, const PageGeom& geo, int head_dim, int num_tokens,
                 cudaStream_t stream) {
    if (num_tokens <= 0) return;
    const long long rows = static_cast<long long>(num_tokens) * geo.num_kv_heads;
    const long long groups = (rows + 3) / 4;
    long long blocks = (groups + kPackWarps - 1) / kPackWarps;
    const long long cap = static_cast<long long>(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    const int aligned = (reinterpret_cast<uintptr_t>(pool) & 7) == 0 && (geo.page_size & 7) == 0;
    if (prod)
        pack_kv_kernel<true><<<static_cast<unsigned>(blocks), kPackWarps * 32, 0, stream>>>(
            static_cast<const uint4*>(key), static_cast<const uint4*>(value), slots, pool, geo,
            head_dim, rows, aligned);
    else
        pack_kv_kernel<false><<<static_cast<unsigned>(blocks), kPackWarps * 32, 0, stream>>>(
            static_cast<const uint4*>(key), static_cast<const uint4*>(value), slots, pool, geo,
            head_dim, rows, aligned);
    check_launch(prod ? "turbo_prod pack_kv" : "turbo_mse pack_kv");
}

}  // namespace tq
