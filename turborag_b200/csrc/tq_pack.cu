// Quantize + pack kernels (turbo_prod and turbo_mse) for sm_100a.
//
// Replaces turbo_prod_pack_kv_kernel (src/cuda/tq_turbo_prod_kernels.cu:110-260)
// and turbo_mse_pack_kv_kernel (src/cuda/tq_turbo_mse_kernels.cu:186-237) of the
// reference with one register-resident design: a warp owns four token-heads at
// a time (8 lanes x 16 elements each), inputs arrive as 16-byte vector loads,
// the 128-point transform runs in registers around one shared-memory re-deal,
// and code bytes leave as 8-byte stores (64 contiguous bytes per token-head).
// Results are bit-identical to the reference's arithmetic; see tq_common.cuh.
// The QJL-1bit scheme (qjl_pack_kv_kernel, src/cuda/tq_qjl_kernels.cu:69-170) is the third
// instance of the same kernel: K keeps one sign bit per rotated dimension and the row's RMS, V
// is quantised as in turbo_prod, and the rotation has no per-head sign.
#include <climits>
#include <stdexcept>
#include "tq_common.cuh"
#include "tq_launch.h"

namespace tq {
namespace {

constexpr int kPackWarps = 8;
constexpr int kCodeRowBytes = 72;  // 64 code bytes + pad: rows land on distinct banks

__device__ __forceinline__ uint4 ld_stream(const uint4* p) { return __ldcs(p); }

// ---- nearest-level search through replicated shared tables --------------------------------
// The reference scans the levels for the smallest distance (first index wins ties).  That is
// the same as counting the decision thresholds that are <= x, where the thresholds are exact
// fp32 numbers: M_j on the positive side, TMID at the centre and, on the negative side, the
// float just above -N_j (there the scan moves up for x > -N_j).  x * 16/3 + magic maps x to
// a cell of width 3/16 (any monotonic map would do); thresholds are further apart than that,
// so a cell holds at most one.  The magic constant's exponent puts the cell number at mantissa
// bits 7.. , which is the byte offset of a 128-byte table row: the row address is one and-or of
// the fma's result.  A table row per cell gives (threshold in the cell or +inf, number
// of thresholds below the cell): code = base + (x >= threshold) -- one fma, one logic op,
// one load, one compare, one add, and no sign handling.  Rows are 128 bytes of replicas: 16
// x 8 bytes for the 4-bit table (the two half-warps of a 64-bit load are separate wavefronts),
// 8 x 16 bytes for the 3-bit table, so no lookup ever conflicts.
constexpr float kCellScale = 16.0f / 3.0f;
constexpr int kCellsV = 128, kCellsK = 32;          // |x| <= sqrt(128) -> |cell| <= 61; K is clamped to 2.5
constexpr float kMagicV = 65536.0f + 64.5f;         // ulp 2^-7: mantissa bits 7..13 = floor(x*16/3 + 64.5)
constexpr float kMagicK = 65536.0f + 16.5f;         // mantissa bits 7..11 = floor(x*16/3 + 16.5)
constexpr int kLutRowBytes = 128;
constexpr uint32_t kRowMaskV = (kCellsV - 1) * kLutRowBytes, kRowMaskK = (kCellsK - 1) * kLutRowBytes;

__device__ __forceinline__ uint32_t cell_v(float x) {
    return (__float_as_uint(__fmaf_rn(x, kCellScale, kMagicV)) & kRowMaskV) / kLutRowBytes;
}
__device__ __forceinline__ uint32_t cell_k(float x) {
    return (__float_as_uint(__fmaf_rn(x, kCellScale, kMagicK)) & kRowMaskK) / kLutRowBytes;
}
__device__ __forceinline__ float next_up_of_negated(float n) {  // smallest float above -n, n > 0
    return -__uint_as_float(__float_as_uint(n) - 1u);
}

// (a & b) | c as one three-input logic instruction (table row addresses).
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// lutV row c: 16 x (threshold, code below it).
// The K nibble (residual sign << 3 | 3-bit code) is a step function of the clamped value with 15
// thresholds: the 7 decision thresholds of the code and the 8 levels themselves (the residual
// e = x - level is >= 0 exactly when x >= level).  They are at least 0.2449 apart, so a cell of
// width 3/16 still holds at most one.  lutK1 row c: 16 x (threshold in the cell or +inf, byte
// offset into lutK2 of the interval below it, this replica's offset included); lutK2: for interval
// i (0..15 = number of thresholds <= x) a pair of 128-byte rows, the second one serving "x >= the
// cell's threshold", each 16 x (level, nibble).
__device__ void build_luts(uint8_t* lutK1, uint8_t* lutK2, uint8_t* lutV, bool need_k) {
    const float v4[15] = {next_up_of_negated(TQ_V4_N7), next_up_of_negated(TQ_V4_N6),
                          next_up_of_negated(TQ_V4_N5), next_up_of_negated(TQ_V4_N4),
                          next_up_of_negated(TQ_V4_N3), next_up_of_negated(TQ_V4_N2),
                          next_up_of_negated(TQ_V4_N1), TQ_TMID, TQ_V4_M1, TQ_V4_M2, TQ_V4_M3,
                          TQ_V4_M4, TQ_V4_M5, TQ_V4_M6, TQ_V4_M7};
    const float k3[7] = {next_up_of_negated(TQ_K3_N3), next_up_of_negated(TQ_K3_N2),
                         next_up_of_negated(TQ_K3_N1), TQ_TMID, TQ_K3_M1, TQ_K3_M2, TQ_K3_M3};
    const float lv3[8] = {-TQ_C3_3, -TQ_C3_2, -TQ_C3_1, -TQ_C3_0, TQ_C3_0, TQ_C3_1, TQ_C3_2, TQ_C3_3};
    const float inf = __int_as_float(0x7f800000);
    for (int c = threadIdx.x; c < kCellsV; c += blockDim.x) {
        float t = inf;
        int base = 0;
#pragma unroll
        for (int j = 0; j < 15; ++j) {
            const int cj = static_cast<int>(cell_v(v4[j]));
            if (cj < c) ++base;
            if (cj == c) t = v4[j];
        }
        float2* row = reinterpret_cast<float2*>(lutV + c * kLutRowBytes);
        for (int r = 0; r < 16; ++r) row[r] = make_float2(t, __int_as_float(base));
    }
    if (!need_k) return;
    // all 15 thresholds in ascending order: level j sits between code thresholds j - 1 and j
    float th[15];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        th[2 * j] = lv3[j];
        if (j < 7) th[2 * j + 1] = k3[j];
    }
    for (int c = threadIdx.x; c < kCellsK; c += blockDim.x) {
        float t = inf;
        int below = 0;
#pragma unroll
        for (int j = 0; j < 15; ++j) {
            const int cj = static_cast<int>(cell_k(th[j]));
            if (cj < c) ++below;
            if (cj == c) t = th[j];
        }
        float2* row = reinterpret_cast<float2*>(lutK1 + c * kLutRowBytes);
        for (int r = 0; r < 16; ++r) row[r] = make_float2(t, __int_as_float(below * 256 + r * 8));
    }
    for (int i = threadIdx.x; i < 32; i += blockDim.x) {
        // interval i / 2 + i % 2 (the last pair's second row is never addressed: no threshold above th[14])
        const int iv = min((i >> 1) + (i & 1), 15);
        // interval iv lies in [th[iv - 1], th[iv]): its code is the number of code thresholds at or below it,
        // its residual is non-negative when its lower end is the level itself (odd number of thresholds below)
        const int code = iv >> 1;
        const int nibble = code | ((iv & 1) ? 8 : 0);
        float2* row = reinterpret_cast<float2*>(lutK2 + i * kLutRowBytes);
        for (int r = 0; r < 16; ++r) row[r] = make_float2(lv3[code], __int_as_float(nibble));
    }
}

// 4-bit code (nearest_v4_idx / nearest_codebook_idx of the reference), exact.
// `rep` = (lane % 16) * 8, this lane's replica inside a row.
__device__ __forceinline__ uint32_t quant_v4_lut(float x, const uint8_t* lutV, uint32_t rep) {
    const uint32_t u = __float_as_uint(__fmaf_rn(x, kCellScale, kMagicV));
    const float2 e = *reinterpret_cast<const float2*>(lutV + lop3_and_or(u, kRowMaskV, rep));
    return __float_as_uint(e.y) + (x >= e.x ? 1u : 0u);
}

// K nibble = residual sign << 3 | 3-bit code, and the residual e = clamp(kn) - level: two table
// steps, the comparison result (all ones or zero) picks the second row of the interval pair.
// `rep` = (lane % 16) * 8.
__device__ __forceinline__ uint32_t quant_k3_lut(float kn, const uint8_t* lutK1, const uint8_t* lutK2, uint32_t rep,
                                                 float& e) {
    const float xc = fminf(fmaxf(kn, -2.5f), 2.5f);
    const uint32_t u = __float_as_uint(__fmaf_rn(xc, kCellScale, kMagicK));
    const float2 c = *reinterpret_cast<const float2*>(lutK1 + lop3_and_or(u, kRowMaskK, rep));
    uint32_t ge;
    asm("set.ge.u32.f32 %0, %1, %2;" : "=r"(ge) : "f"(xc), "f"(c.x));
    const float2 r = *reinterpret_cast<const float2*>(lutK2 + lop3_and_or(ge, 128u, __float_as_uint(c.y)));
    e = __fsub_rn(xc, r.x);
    return __float_as_uint(r.y);
}

// Squares that feed the reference's summation tree.  A packed mul.rn.f32x2 whose only consumer
// is a packed add gets contracted by the assembler (observed: the first tree level came out as
// fma(x, x, y*y)), which changes the sum in its last bit for about half of the rows.  A packed
// fma with a zero addend rounds the same product once (x*x + 0 == RN(x*x)), is a single
// instruction for two squares, and an fma feeding an add is never contracted.  The zero is a
// kernel argument so that the fma cannot be simplified back into a multiply at compile time.
__device__ __forceinline__ float2 square2(const float2& v, const float2& zero) {
    return fma2(v, v, zero);
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
    if (aligned8) {
        st_global_v2_if(reinterpret_cast<unsigned long long>(dst) + 8 * l, v, valid);
    } else {
        if (!valid) return;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            dst[8 * l + i] = static_cast<uint8_t>(v.x >> (8 * i));
            dst[8 * l + 4 + i] = static_cast<uint8_t>(v.y >> (8 * i));
        }
    }
}

// Intermediate values of the turbo_prod pack for parity triage, each [num_tokens, num_kv_heads, 128]
// or null (the reference kernel's debug_* arguments, tq_turbo_prod_kernels.cu:119-124, 216-217,
// 243-246): rotated K / V, the clamped normalised values, the 3-bit / 4-bit level indices.
struct PackDump {
    float *k_rot, *v_rot, *kn, *vn;
    int *kidx, *vidx;
};

// S: 0 turbo_prod, 1 turbo_mse, 2 QJL-1bit.  ALIGNED8: pool base and page size are multiples of
// 8 bytes (code rows leave as 8-byte stores); a template argument so that the byte-store sequence
// of the other case is not part of this kernel's instruction stream.  DUMP: the debug instance of
// the turbo_prod kernel, which also writes its intermediates (never launched by the pack entry points).
// POW2: the kv head count and the tokens per page are powers of two (every layout in use), so
// token = row / H and page = slot / block_size are shifts; the other instance divides.
template <int S, bool ALIGNED8, bool DUMP = false, bool POW2 = false>
__global__ void __launch_bounds__(kPackWarps * 32, (DUMP || S == 0) ? 0 : 4)
pack_kv_kernel(const uint4* __restrict__ key, const uint4* __restrict__ value,
               const int32_t* __restrict__ slot_mapping, uint8_t* __restrict__ page_pool,
               PageGeom geo, IndexDiv div_heads, IndexDiv div_block, int head_dim,
               int num_rows, float zero, PackDump dump) {
    constexpr bool PROD = S == 0, QJL = S == 2;
    constexpr bool TREE128 = PROD || QJL;  // sum of squares: 128-leaf tree (prod, QJL) or 64 pair leaves (mse)
    __shared__ __align__(16) float xchg[kPackWarps][kXchgWarpFloats];
    __shared__ __align__(128) uint8_t lutK1[PROD ? kCellsK * kLutRowBytes : 16];
    __shared__ __align__(128) uint8_t lutK2[PROD ? 32 * kLutRowBytes : 16];
    __shared__ __align__(128) uint8_t lutV[kCellsV * kLutRowBytes];
    build_luts(lutK1, lutK2, lutV, PROD);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rr = lane >> 3, l = lane & 7;
    const uint32_t rep_v = (lane & 15) * 8;
    float* buf = xchg[warp];
    uint8_t* code_buf = reinterpret_cast<uint8_t*>(buf);
    const int H = geo.num_kv_heads;
    const float c = inv_sqrt_dim(head_dim);
    const float2 zero2 = make_float2(zero, zero);
    const int groups = (num_rows + 3) >> 2;  // rows are counted in 32 bits (checked by the launcher)
    const int warps_total = static_cast<int>(gridDim.x) * kPackWarps;
    // loop-invariant halves of the addresses: a row is 256 bytes of fp16, this lane's part starts at 32 l
    const unsigned long long key64 = reinterpret_cast<unsigned long long>(key) + 32 * l;
    const unsigned long long val64 = reinterpret_cast<unsigned long long>(value) + 32 * l;
    const unsigned long long slots64 = reinterpret_cast<unsigned long long>(slot_mapping);
    const unsigned long long pool64 = reinterpret_cast<unsigned long long>(page_pool);
    const unsigned int page_size32 = static_cast<unsigned int>(geo.page_size);

    for (int g = blockIdx.x * kPackWarps + warp; g < groups; g += warps_total) {
        const int row_raw = g * 4 + rr;
        const bool valid = row_raw < num_rows;
        const int row = valid ? row_raw : num_rows - 1;  // keep all lanes converged
        const int tok = POW2 ? (row >> div_heads.shift) : row / H;
        const int h = row - tok * H;
        // odd heads: the whole rotated row is negated; the QJL sign hash has no head term
        // (tq_qjl_kernels.cu:18-21)
        const float cs = (!QJL && (h & 1)) ? -c : c;

        const uint4* kp = reinterpret_cast<const uint4*>(mad_wide(row, 256u, key64));
        const uint4* vp = reinterpret_cast<const uint4*>(mad_wide(row, 256u, val64));
        const uint4 k_lo = ld_stream(kp), k_hi = ld_stream(kp + 1);
        const uint4 v_lo = ld_stream(vp), v_hi = ld_stream(vp + 1);
        const int slot = __ldg(reinterpret_cast<const int32_t*>(mad_wide(tok, 4u, slots64)));

        const int blk = POW2 ? (slot >> div_block.shift) : slot / geo.block_size;
        const int tib = slot - blk * geo.block_size;
        const unsigned long long page64 = mad_wide(blk, page_size32, pool64);
        uint8_t* page = reinterpret_cast<uint8_t*>(page64);
        const unsigned int th = static_cast<unsigned int>(tib * H + h);
        const bool head_lane = valid && l == 0;  // the lane that writes the row's scales

        float2 x[8], y[8];

        // ---------------- K ----------------
        fwht_phase1_from_half(k_lo, k_hi, x);
        redeal(x, y, buf, lane);
        fwht_phase2(y);
        const float2 cs2 = make_float2(cs, cs);
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = mul2(y[j], cs2);

        uint32_t kbytes[8];
        if (QJL) {
            float2 sq[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) sq[j] = square2(y[j], zero2);
            const float krms = rms_from_sum(tree128(sq));
            // bit = (k / krms >= 0) (tq_qjl_kernels.cu:155): krms > 0 and the quotient of a rotated
            // fp16 row cannot underflow, so this is the sign of k itself (-0 counts as >= 0)
            uint32_t w0 = 0u, w1 = 0u;  // byte j & 3 of w(j >> 2): this lane's 2 bits of sign byte 2j + (l >> 2)
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t two = (y[j].x >= 0.0f ? 1u : 0u) | (y[j].y >= 0.0f ? 2u : 0u);
                const uint32_t at = two << (2 * (l & 3) + 8 * (j & 3));
                if (j < 4) w0 |= at; else w1 |= at;
            }
#pragma unroll
            for (int m = 1; m <= 2; m <<= 1) {
                w0 |= __shfl_xor_sync(0xffffffffu, w0, m);
                w1 |= __shfl_xor_sync(0xffffffffu, w1, m);
            }
            // lanes 0-3 hold the even sign bytes, lanes 4-7 the odd ones
            const uint32_t o0 = __shfl_xor_sync(0xffffffffu, w0, 4), o1 = __shfl_xor_sync(0xffffffffu, w1, 4);
            if (valid && l == 0) {
                const uint4 bits = make_uint4(__byte_perm(w0, o0, 0x5140), __byte_perm(w0, o0, 0x7362),
                                              __byte_perm(w1, o1, 0x5140), __byte_perm(w1, o1, 0x7362));
                uint8_t* dst = page + geo.k_codes + th * 16;
                if (ALIGNED8) {
                    reinterpret_cast<uint2*>(dst)[0] = make_uint2(bits.x, bits.y);
                    reinterpret_cast<uint2*>(dst)[1] = make_uint2(bits.z, bits.w);
                } else {
                    const uint32_t wds[4] = {bits.x, bits.y, bits.z, bits.w};
#pragma unroll
                    for (int i = 0; i < 16; ++i) dst[i] = static_cast<uint8_t>(wds[i >> 2] >> (8 * (i & 3)));
                }
                *reinterpret_cast<__half*>(page + geo.k_scales + th * 2) = __float2half_rn(krms);
            }
        } else if (PROD) {
            float2 sq[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) sq[j] = square2(y[j], zero2);
            const float krms = rms_from_sum(tree128(sq));
            const float kr = __frcp_rn(krms);
            float2 e2[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float e0, e1;
                const float2 kn = div_by2(y[j], krms, kr);
                const uint32_t n0 = quant_k3_lut(kn.x, lutK1, lutK2, rep_v, e0);
                const uint32_t n1 = quant_k3_lut(kn.y, lutK1, lutK2, rep_v, e1);
                kbytes[j] = n0 | (n1 << 4);
                e2[j] = square2(make_float2(e0, e1), zero2);
                if (DUMP && valid) {  // element 2l + b + 16j of the row
                    const long long at = static_cast<long long>(row) * kHeadDim + 2 * l + 16 * j;
                    if (dump.k_rot) { dump.k_rot[at] = y[j].x; dump.k_rot[at + 1] = y[j].y; }
                    if (dump.kn) {
                        dump.kn[at] = fminf(fmaxf(kn.x, -2.5f), 2.5f);
                        dump.kn[at + 1] = fminf(fmaxf(kn.y, -2.5f), 2.5f);
                    }
                    if (dump.kidx) { dump.kidx[at] = static_cast<int>(n0 & 7u); dump.kidx[at + 1] = static_cast<int>(n1 & 7u); }
                }
            }
            const float rms_e = rms_from_sum(tree128(e2));
            st_global_u16_if(mad_wide(geo.k_scales + th * 2, 1u, page64), __half_as_ushort(__float2half_rn(krms)), head_lane);
            st_global_u16_if(mad_wide(geo.k_res + th * 2, 1u, page64), __half_as_ushort(__float2half_rn(rms_e)), head_lane);
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
                kbytes[j] = quant_v4_lut(kn.x, lutV, rep_v) | (quant_v4_lut(kn.y, lutV, rep_v) << 4);
            }
            st_global_u16_if(mad_wide(geo.k_scales + th * 2, 1u, page64), __half_as_ushort(__float2half_rn(krms)), head_lane);
        }
        if (!QJL)
            store_codes(kbytes, code_buf, reinterpret_cast<uint8_t*>(mad_wide(geo.k_codes + th * 64, 1u, page64)), lane,
                        valid, ALIGNED8);

        // ---------------- V ----------------
        fwht_phase1_from_half(v_lo, v_hi, x);
        redeal(x, y, buf, lane);
        fwht_phase2(y);
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = mul2(y[j], cs2);
        float vrms;
        if (TREE128) {
            float2 sq[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) sq[j] = square2(y[j], zero2);
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
            const uint32_t c0 = quant_v4_lut(vn.x, lutV, rep_v), c1 = quant_v4_lut(vn.y, lutV, rep_v);
            vbytes[j] = c0 | (c1 << 4);
            if (DUMP && valid) {
                const long long at = static_cast<long long>(row) * kHeadDim + 2 * l + 16 * j;
                if (dump.v_rot) { dump.v_rot[at] = y[j].x; dump.v_rot[at + 1] = y[j].y; }
                if (dump.vn) {
                    dump.vn[at] = fminf(fmaxf(vn.x, -2.75f), 2.75f);
                    dump.vn[at + 1] = fminf(fmaxf(vn.y, -2.75f), 2.75f);
                }
                if (dump.vidx) { dump.vidx[at] = static_cast<int>(c0); dump.vidx[at + 1] = static_cast<int>(c1); }
            }
        }
        st_global_u16_if(mad_wide(geo.v_scales + th * 2, 1u, page64), __half_as_ushort(__float2half_rn(vrms)), head_lane);
        store_codes(vbytes, code_buf, reinterpret_cast<uint8_t*>(mad_wide(geo.v_codes + th * 64, 1u, page64)), lane,
                    valid, ALIGNED8);
    }
}

}  // namespace

void launch_pack(int scheme, const void* key, const void* value, const int32_t* slots,
                 uint8_t* pool, const PageGeom& geo, int head_dim, int num_tokens,
                 cudaStream_t stream) {
    if (num_tokens <= 0) return;
    const long long rows = static_cast<long long>(num_tokens) * geo.num_kv_heads;
    const long long groups = (rows + 3) / 4;
    long long blocks = (groups + kPackWarps - 1) / kPackWarps;
    const long long cap = static_cast<long long>(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    const bool aligned = (reinterpret_cast<uintptr_t>(pool) & 7) == 0 && (geo.page_size & 7) == 0;
    if (rows > INT_MAX) throw std::runtime_error("pack: more than 2^31 - 1 token-heads in one call");
    const IndexDiv dh = make_index_div(geo.num_kv_heads), db = make_index_div(geo.block_size);
    const bool pow2 = dh.shift >= 0 && db.shift >= 0;
#define TQ_PACK_LAUNCH2(SV, AL, P2)                                                            \
    pack_kv_kernel<SV, AL, false, P2><<<static_cast<unsigned>(blocks), kPackWarps * 32, 0, stream>>>( \
        static_cast<const uint4*>(key), static_cast<const uint4*>(value), slots, pool, geo, dh, db, head_dim, \
        static_cast<int>(rows), 0.0f, PackDump{})
#define TQ_PACK_LAUNCH1(SV, AL) do { if (pow2) TQ_PACK_LAUNCH2(SV, AL, true); else TQ_PACK_LAUNCH2(SV, AL, false); } while (0)
#define TQ_PACK_LAUNCH(SV) do { if (aligned) TQ_PACK_LAUNCH1(SV, true); else TQ_PACK_LAUNCH1(SV, false); } while (0)
    if (scheme == TQ_SCHEME_TURBO_PROD) TQ_PACK_LAUNCH(0);
    else if (scheme == TQ_SCHEME_TURBO_MSE) TQ_PACK_LAUNCH(1);
    else TQ_PACK_LAUNCH(2);
#undef TQ_PACK_LAUNCH
#undef TQ_PACK_LAUNCH1
#undef TQ_PACK_LAUNCH2
    check_launch(scheme == TQ_SCHEME_TURBO_PROD ? "turbo_prod pack_kv"
                 : scheme == TQ_SCHEME_TURBO_MSE ? "turbo_mse pack_kv" : "qjl pack_kv");
}

void launch_pack_debug(const void* key, const void* value, const int32_t* slots, uint8_t* pool,
                       const PageGeom& geo, int head_dim, int num_tokens, float* k_rot, float* v_rot, float* kn,
                       float* vn, int* kidx, int* vidx, cudaStream_t stream) {
    if (num_tokens <= 0) return;
    const long long rows = static_cast<long long>(num_tokens) * geo.num_kv_heads;
    const long long groups = (rows + 3) / 4;
    long long blocks = (groups + kPackWarps - 1) / kPackWarps;
    const long long cap = static_cast<long long>(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    const PackDump dump{k_rot, v_rot, kn, vn, kidx, vidx};
    // the byte-store instance: any pool alignment, this entry point is not a hot path
    if (rows > INT_MAX) throw std::runtime_error("pack: more than 2^31 - 1 token-heads in one call");
    pack_kv_kernel<0, false, true, false><<<static_cast<unsigned>(blocks), kPackWarps * 32, 0, stream>>>(
        static_cast<const uint4*>(key), static_cast<const uint4*>(value), slots, pool, geo,
        make_index_div(geo.num_kv_heads), make_index_div(geo.block_size), head_dim, static_cast<int>(rows), 0.0f, dump);
    check_launch("turbo_prod pack_kv (debug)");
}

}  // namespace tq
