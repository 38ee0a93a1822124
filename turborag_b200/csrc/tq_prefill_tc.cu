// Chunked query prefill over a turbo_mse-compressed prefix plus a causal fp16 chunk on the
// 5th-generation tensor cores (tcgen05 + TMEM), sm_100a.
//
// The reference has no such kernel: its fused kernel (src/cuda/tq_turbo_mse_kernels.cu:302-417)
// takes one query row per kv head and walks the tokens serially.  Here the rows (token, query
// head) that share a kv head form the M dimension of a flash-attention tile loop; arithmetic
// follows the reference's rotated-domain formulation (q' = R(q), logits <q', k'>/sqrt(D), V
// accumulated in the rotated domain, inverse rotation in the merge kernel).
//
// One CTA = 128 query rows of one (sequence, kv head, prefix split), 17 warps in three roles:
//   warps 0-3, 8-11  softmax: two threads per row (tokens 0-31 / 32-63 of a 64-token tile); a row
//              is TMEM lane i, which warps w and w + 8 may both touch.  Per tile a thread reads
//              its 32 scores from TMEM (tcgen05.ld), applies the per-token K scale and the causal /
//              length mask, agrees with its partner on the row maximum (shared memory + a 64-thread
//              named barrier), and writes P * (V scale) as fp16 pairs into TMEM (tcgen05.st), where
//              it is the A operand of the second product.  The maximum in use only follows the true one when
//              that runs ahead by more than 2^8; then the O accumulator (TMEM) is rescaled in place
//              (tcgen05.ld / st).  Elementwise work uses packed fp32 pairs.
//   warps 4-7, 13-16  unpack: page bytes travel global -> shared with cp.async two tiles ahead (a
//              thread copies exactly the bytes it reads back, so wait_group is the only
//              synchronisation); every code byte becomes two fp16 operands with one shared-memory
//              table lookup; K and V tiles are stored in the 128-byte-swizzled canonical operand
//              layout (three stages); chunk tiles (fp16, rotated by a pre-pass) are copied instead.
//   warp 12    one thread issues tcgen05.mma: S = Q K^T (M 128, N 64, K 128, A = Q from TMEM, K-major
//              B; 16 instructions: the rotated query rows live in tensor memory as two fp16 parts,
//              q' = hi + lo, so S carries no fp16 rounding of q' and the tensor core never reads Q
//              from shared memory) into one of two TMEM buffers, and O += P V (M 128, N 128, K 64: 4
//              instructions, A = P from TMEM, V as MN-major B operand) into TMEM; tcgen05.commit arrives on
//              mbarriers.  It issues whichever product has its operands ready, S up to two tiles
//              ahead, so the tensor pipe works on the next scores during the current softmax.
// Synchronisation is all mbarriers (K/V stages full / empty, S full, P full, P V done); every wait
// is bounded: after kWaitLimit polls a warp records a status code, stops waiting (it keeps
// walking its loop so that no partner blocks) and the kernel ends through the common exit, where
// the TMEM allocation is released.  tq_mse_prefill_status() reports the code.
// Measured bound: the shared-memory port (operand tiles are written once by the unpack warps and
// read by the tensor core, plus table lookups and the raw ring) and the softmax chain's latency.
#include <climits>
#include <cstring>

#include "tq_common.cuh"
#include "tq_launch.h"

namespace tq {
namespace {

constexpr float kLog2eT = 1.4426950408889634f;
constexpr float kLn2T = 0.6931471805599453f;
constexpr int kTileTok = 64;
constexpr int kRowsCta = 128;
constexpr int kThreadsTc = 544;  // warps: softmax 0-3, unpack 4-7, softmax 8-11, MMA issue 12, unpack 13-16
constexpr int kWaitLimit = 1 << 20;
constexpr float kRescaleLag = 8.0f;  // log2 units a row maximum may run ahead of the one in use

// shared-memory map (bytes); every operand tile starts on a 1024-byte boundary
constexpr int kOffLut = 0;                      // 256 rows of 256 B: 32 replicas x half2 in the first 128 B of a row,
                                                // so that a lookup address is one byte permute (byte << 8 | lane * 4)
constexpr int kKvStages = 3;
constexpr int kOffKV = 65536;                   // stage s: K [2][64][128 B] at +32768 s, V behind it
constexpr int kOffScale = kOffKV + kKvStages * 32768;  // per K/V stage: kscale[64], vscale[64] (fp32)
constexpr int kOffBar = kOffScale + 2048;       // mbarriers, TMEM base
constexpr int kRawStages = 3;
constexpr int kRawStage = 8704;                 // K codes 4 KB, V codes 4 KB, 64 x (K scale word, V scale word)
constexpr int kOffXch = kOffBar + 128;          // row maxima exchanged by the two threads of a row
constexpr int kOffRaw = kOffXch + 2048;
constexpr int kSmemTc = kOffRaw + kRawStages * kRawStage;
static_assert(kSmemTc <= 232448, "shared memory of one SM");

// fp16(alpha4 * |level|) of the 4-bit codebook as byte pools (entries 0-3 | 4-7), and alpha4
#define TQ_ALPHA4T TQF(0x404c9252)
constexpr uint32_t kMagHiA = 0x42403c36u, kMagHiB = 0x48464544u, kMagLoA = 0x0633f691u, kMagLoB = 0x5e9d2c04u;

__device__ __forceinline__ uint32_t level4_half_bits(uint32_t n) {
    const uint32_t mag = n >= 8u ? n - 8u : 7u - n;
    const uint32_t sh = 8u * (mag & 3u);
    const uint32_t hi = ((mag < 4u ? kMagHiA : kMagHiB) >> sh) & 0xFFu;
    const uint32_t lo = ((mag < 4u ? kMagLoA : kMagLoB) >> sh) & 0xFFu;
    return (hi << 8) | lo | (n >= 8u ? 0u : 0x8000u);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint32_t prmt_t(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ float ex2_t(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Byte offset of 16-byte unit `unit` (0..7) of row `row` inside a [rows][128 B] operand chunk:
// groups of 8 rows are 1024 bytes, the unit index is XOR-ed with row % 8 (128-byte swizzle).
__device__ __forceinline__ uint32_t sw128(int row, int unit) {
    return static_cast<uint32_t>((row >> 3) * 1024 + (row & 7) * 128 + ((unit ^ (row & 7)) << 4));
}
// Shared-memory matrix descriptor: start address, leading / stride byte offsets (16-byte units),
// descriptor version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t make_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return static_cast<uint64_t>((addr >> 4) & 0x3FFFu) |
           (static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           (static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptors (kind::f16): fp32 accumulate, fp16 A/B, M = 128.
constexpr uint32_t kIdescS = (1u << 4) | (8u << 17) | (8u << 24);                // N = 64, A and B K-major
constexpr uint32_t kIdescPV = (1u << 4) | (1u << 16) | (16u << 17) | (8u << 24);  // N = 128, B MN-major

__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}\n"
        ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// A operand in tensor memory (lane = row, packed 16-bit pairs along K), B through a descriptor.
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// The same with the descriptor handed over as its two 32-bit words and the accumulate flag as a
// template argument.  One thread issues every MMA of a CTA and waits until the tensor pipe takes each
// one; whatever it computes between two MMAs is added to that.  The words of a descriptor differ
// between k-steps only by a constant in the low one (start address >> 4).
template <bool ACCUMULATE>
__device__ __forceinline__ void mma_f16_ts_words(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi,
                                                 uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 bd;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 bd, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], bd, %4, {%6, %6, %6, %6}, p;\n\t}\n"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "n"(ACCUMULATE ? 1 : 0), "r"(0u) : "memory");
}
// Low and high word of make_desc(addr, lbo, sbo).
__device__ __forceinline__ uint32_t desc_lo(uint32_t addr, uint32_t lbo_bytes) {
    return ((addr >> 4) & 0x3FFFu) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}
__host__ __device__ constexpr uint32_t desc_hi(uint32_t sbo_bytes) {
    return ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait for the phase with the given parity to complete.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (int i = 0; i < kWaitLimit; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}\n" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
// One poll that the hardware may suspend for up to `ns` nanoseconds while the phase is incomplete.
__device__ __forceinline__ bool mbar_try_wait_for(uint32_t bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n" : "=r"(ok) : "r"(bar), "r"(parity), "r"(ns) : "memory");
    return ok != 0;
}
// Non-blocking test of the same condition.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// The same for a whole warp: every lane gets the same answer, so warp-collective instructions
// that follow are executed by all lanes or by none.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity) {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity)) != 0;
}
__device__ __forceinline__ void cp_async16_t(uint32_t dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4_t(uint32_t dst_smem, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
    uint32_t r[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(v[j]);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// Status word of the last prefill launches on this device: 0 = every wait was satisfied.
__device__ int g_prefill_tc_status = 0;

// ---- pre-pass: R(x) * scale for fp16 rows of 128, natural dim order --------------------------
__global__ void __launch_bounds__(128)
rotate_rows_tc_kernel(const __half* __restrict__ src, __half* __restrict__ dst, __half* __restrict__ dst_lo,
                      long long rows, int heads_mod, int group, float scale, int head_dim) {
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
    __half2* out = reinterpret_cast<__half2*>(dst + row * kHeadDim + 4 * lane);
    const __half2 h0 = __floats2half2_rn(x[0] * sc, x[1] * sc), h1 = __floats2half2_rn(x[2] * sc, x[3] * sc);
    out[0] = h0;
    out[1] = h1;
    if (dst_lo) {
        // what the fp16 rounding dropped, as a second fp16 row: value = hi + lo to ~22 bits
        const float2 f0h = __half22float2(h0), f1h = __half22float2(h1);
        __half2* lo = reinterpret_cast<__half2*>(dst_lo + row * kHeadDim + 4 * lane);
        lo[0] = __floats2half2_rn(x[0] * sc - f0h.x, x[1] * sc - f0h.y);
        lo[1] = __floats2half2_rn(x[2] * sc - f1h.x, x[3] * sc - f1h.y);
    }
}

struct PrefillTcParams {
    const __half* q_rot;      // [B, Nq, Hq, 128] rotated, scaled: fp16 part
    const __half* q_rot_lo;   // the same rows: remainder of the fp16 rounding
    const __half* ck_rot;     // [B, Nq, H, 128] or nullptr
    const __half* cv_rot;
    const uint8_t* pool;
    const int32_t* block_tables;
    const int32_t* seq_lens;
    float* partials;          // [B*Nq, splits, Hq, 130]
    PageGeom geo;
    int table_stride, nq, hq, groups, splits;
};

__global__ void __launch_bounds__(kThreadsTc, 1)
prefill_tc_kernel(PrefillTcParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int H = p.geo.num_kv_heads, G = p.groups;
    const int mt = blockIdx.x;
    const int h = blockIdx.y % H, split = blockIdx.y / H;
    const int b = blockIdx.z;
    const int rows_total = p.nq * G;

    // barriers: kv_full[3] (128 arrivals) / kv_empty[3] (1): barrier j % 3 serves tile j, phase j / 3;
    // s_full[2] (1), p_full[2] (128), pv_done[2] (1): barrier j % 2 serves tile j, phase j / 2
    const uint32_t bar0 = sbase + kOffBar;
    const uint32_t bar_kv_full = bar0, bar_kv_empty = bar0 + 24, bar_s_full = bar0 + 48, bar_p_full = bar0 + 64,
                   bar_pv_done = bar0 + 80;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kOffBar + 112);

    // ---- tile schedule of this CTA (identical in every role) ----
    const int n_prefix = __ldg(p.seq_lens + b);
    const int prefix_tiles = (n_prefix + kTileTok - 1) / kTileTok;
    const int per = (prefix_tiles + p.splits - 1) / p.splits;
    const int tile_lo = split * per, tile_hi = min(prefix_tiles, tile_lo + per);
    const int n_pref = max(tile_hi - tile_lo, 0);
    const int last_tok = min((mt * kRowsCta + kRowsCta - 1) / G, p.nq - 1);
    const int chunk_tiles = (p.ck_rot && split == p.splits - 1) ? last_tok / kTileTok + 1 : 0;
    const int n_tiles = n_pref + chunk_tiles;

    // ---- set-up: table, Q tile, barriers, TMEM ----
    for (int i = tid; i < 256 * 8; i += kThreadsTc) {
        const uint32_t row = i >> 3, n0 = row & 15u, n1 = row >> 4;
        const uint32_t e = level4_half_bits(n0) | (level4_half_bits(n1) << 16);
        *reinterpret_cast<uint4*>(smem + kOffLut + row * 256 + (i & 7) * 16) = make_uint4(e, e, e, e);
    }
    fence_async_smem();
    if (tid == 0) {
        for (int k = 0; k < kKvStages; ++k) {
            mbar_init(bar_kv_full + 8 * k, 256);
            mbar_init(bar_kv_empty + 8 * k, 1);
        }
        mbar_init(bar_s_full, 1);
        mbar_init(bar_s_full + 8, 1);
        mbar_init(bar_p_full, 256);
        mbar_init(bar_p_full + 8, 256);
        mbar_init(bar_pv_done, 1);
        mbar_init(bar_pv_done + 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;          // columns 0-63 / 64-127: S buffers, 128-255: O
    const uint32_t tmem_o = tmem + 128;
    const uint32_t tmem_p = tmem + 256;        // columns 256-287 / 288-319: P buffers (fp16 pairs)
    const uint32_t tmem_q = tmem + 320;        // columns 320-383: Q hi, 384-447: Q lo (fp16 pairs along dims)
    int fail = 0;

    // ---- the CTA's 128 query rows go to tensor memory once: lane = row, 32-bit column c = dims 2c, 2c+1.
    // Warps 0-3 write the fp16 part of their 32 rows, warps 8-11 the remainder part of the same rows.
    if (warp < 4 || (warp >= 8 && warp < 12)) {
        const int r = (warp & 3) * 32 + lane;
        const int rg = min(mt * kRowsCta + r, rows_total - 1);
        const __half* src = (warp < 4 ? p.q_rot : p.q_rot_lo) +
                            ((static_cast<long long>(b) * p.nq + rg / G) * p.hq + h * G + rg % G) * kHeadDim;
        const uint32_t dst = tmem_q + (warp < 4 ? 0u : 64u) + (static_cast<uint32_t>((warp & 3) * 32) << 16);
#pragma unroll 1
        for (int c0 = 0; c0 < 64; c0 += 32) {
            float v[32];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const uint4 w = __ldg(reinterpret_cast<const uint4*>(src + 2 * c0) + u);
                v[4 * u] = __uint_as_float(w.x);
                v[4 * u + 1] = __uint_as_float(w.y);
                v[4 * u + 2] = __uint_as_float(w.z);
                v[4 * u + 3] = __uint_as_float(w.w);
            }
            tmem_st32(dst + c0, v);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    if ((warp >= 4 && warp < 8) || warp >= 13) {
        // =========================== unpack warps ===========================
        const int u = warp < 8 ? tid - 128 : tid - 288;   // 0..255
        const int ut = u & 63, uq = u >> 6;   // token of the tile, 16-byte quarter of its 64 code bytes
        const int uh = uq >> 1;               // dim chunk (64 dims) the quarter belongs to
        const uint32_t lane_v = static_cast<uint32_t>(lane) * 4u;  // table address = byte << 8 | lane * 4
        const int32_t* table = p.block_tables + static_cast<long long>(b) * p.table_stride;
        // Page bytes travel global -> shared with cp.async, two tiles ahead, into a ring of
        // three raw stages (an HBM round trip is longer than a tile takes, and loads parked in
        // registers would share scoreboards with younger loads).  A thread copies exactly the bytes
        // it will read itself (16 code bytes of K and of V, and the two words holding its scales),
        // so cp.async.wait_group is the only synchronisation the raw ring needs.
        const uint32_t raw_base = sbase + kOffRaw;
        // 16-byte piece uq of token ut sits at an XOR-ed position, so the 16-byte reads of eight
        // neighbouring tokens cover all banks
        const uint32_t code_off = static_cast<uint32_t>(ut * 64 + ((uq ^ ((ut >> 1) & 3)) << 4));
        // Source addresses: a thread always copies the same in-page bytes (token ut % 16 of its page, quarter
        // uq), so everything but the page is loop-invariant and an address is one wide multiply-add of the
        // page id.  Tokens past the end of the prefix read the prefix's last page (any finite bytes do: their
        // scales are written as zero and their scores masked).  The page id of tile it + 2 is loaded while
        // tile it + 1 is prefetched: one 4-byte load per thread and tile, no shuffles.
        const uint32_t page_size32 = static_cast<uint32_t>(p.geo.page_size);
        const unsigned th = static_cast<unsigned>((ut & 15) * H + h);
        const unsigned long long pool64 = reinterpret_cast<unsigned long long>(p.pool);
        const unsigned long long k_src = pool64 + p.geo.k_codes + th * 64 + 16 * uq;
        const unsigned long long v_src = pool64 + p.geo.v_codes + th * 64 + 16 * uq;
        const unsigned long long ks_src = pool64 + p.geo.k_scales + ((th * 2) & ~3u);
        const unsigned long long vs_src = pool64 + p.geo.v_scales + ((th * 2) & ~3u);
        const int last_page = (n_prefix - 1) >> 4;
        const int page0 = tile_lo * (kTileTok / 16) + (ut >> 4);  // index of this thread's page of tile 0
        auto load_id = [&](int it) {
            return it < n_pref ? __ldg(table + min(page0 + (kTileTok / 16) * it, last_page)) : 0;
        };
        int pf_it = 0, pf_id = load_id(0), pf_id_next = load_id(1);
        uint32_t pf_dst = raw_base;  // stage of tile pf_it
        auto prefetch_next = [&]() {
            if (pf_it < n_pref) {
                const uint32_t page = static_cast<uint32_t>(pf_id);
                cp_async16_t(pf_dst + code_off, reinterpret_cast<const void*>(mad_wide(page, page_size32, k_src)));
                cp_async16_t(pf_dst + 4096 + code_off, reinterpret_cast<const void*>(mad_wide(page, page_size32, v_src)));
                if (uq == 0) {  // the aligned 4-byte words that hold this token-head's two fp16 scales
                    cp_async4_t(pf_dst + 8192 + ut * 8, reinterpret_cast<const void*>(mad_wide(page, page_size32, ks_src)));
                    cp_async4_t(pf_dst + 8192 + ut * 8 + 4, reinterpret_cast<const void*>(mad_wide(page, page_size32, vs_src)));
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");  // one group per tile, empty or not
            pf_id = pf_id_next;
            pf_id_next = load_id(pf_it + 2);
            ++pf_it;
            pf_dst = pf_dst == raw_base + (kRawStages - 1) * kRawStage ? raw_base : pf_dst + kRawStage;
        };
        // four code words (32 codes) -> four 16-byte units of fp16 operands.  All table loads are
        // issued before the first store: shared-memory stores and loads through unrelated pointers
        // keep their program order, so alternating them would serialise on the load latency.
        auto unpack_row = [&](const uint4& c, uint8_t* dst_chunk) {
            const uint32_t w[4] = {c.x, c.y, c.z, c.w};
            uint32_t o[16];
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
                o[4 * wi + 0] = *reinterpret_cast<const uint32_t*>(smem + kOffLut + prmt_t(w[wi], lane_v, 0x5504u));
                o[4 * wi + 1] = *reinterpret_cast<const uint32_t*>(smem + kOffLut + prmt_t(w[wi], lane_v, 0x5514u));
                o[4 * wi + 2] = *reinterpret_cast<const uint32_t*>(smem + kOffLut + prmt_t(w[wi], lane_v, 0x5524u));
                o[4 * wi + 3] = *reinterpret_cast<const uint32_t*>(smem + kOffLut + prmt_t(w[wi], lane_v, 0x5534u));
            }
#pragma unroll
            for (int wi = 0; wi < 4; ++wi)
                *reinterpret_cast<uint4*>(dst_chunk + sw128(ut, 4 * (uq & 1) + wi)) =
                    make_uint4(o[4 * wi], o[4 * wi + 1], o[4 * wi + 2], o[4 * wi + 3]);
        };
        // one tile: its raw bytes have landed -> start the copies of tile it + 2 -> wait for the
        // operand stage -> unpack (or copy a chunk tile)
        int st = 0, kv_round = 0;        // operand stage of the tile in hand (it % kKvStages), it / kKvStages
        uint32_t raw_rd = kOffRaw;       // raw stage of the tile in hand
        const uint32_t sc_rd = 8192u + ut * 8u + ((th * 2u) & 2u);
        auto do_tile = [&](int it) {
            asm volatile("cp.async.wait_group 1;" ::: "memory");  // every byte a thread reads it copied itself
            prefetch_next();  // tile it + 2
            if (kv_round > 0 && !warp_wait(bar_kv_empty + 8 * st, (kv_round - 1) & 1)) { fail = 1; return; }
            uint8_t* ktile = smem + kOffKV + st * 32768;
            uint8_t* vtile = ktile + 16384;
            float* kscale = reinterpret_cast<float*>(smem + kOffScale) + st * 128;
            float* vscale = kscale + 64;
            if (it < n_pref) {
                const uint8_t* rawst = smem + raw_rd;
                const uint4 kc = *reinterpret_cast<const uint4*>(rawst + code_off);
                const uint4 vc = *reinterpret_cast<const uint4*>(rawst + 4096 + code_off);
                const int t0 = (tile_lo + it) * kTileTok;
                const unsigned short ks_bits = *reinterpret_cast<const unsigned short*>(rawst + sc_rd);
                const unsigned short vs_bits = *reinterpret_cast<const unsigned short*>(rawst + sc_rd + 4);
                // this thread's 32 dims: dim chunk uh of the tile, units 4 (uq % 2) .. + 3 inside it
                unpack_row(kc, ktile + uh * 8192);
                unpack_row(vc, vtile + uh * 8192);
                if (uq == 0) {
                    const bool ok = t0 + ut < n_prefix;
                    kscale[ut] = ok ? __half2float(__ushort_as_half(ks_bits)) : 0.0f;
                    vscale[ut] = ok ? __half2float(__ushort_as_half(vs_bits)) * (1.0f / TQ_ALPHA4T) : 0.0f;
                }
            } else {
                const int t0 = (it - n_pref) * kTileTok;
                const int t = min(t0 + ut, p.nq - 1);
                const long long rowi = (static_cast<long long>(b) * p.nq + t) * H + h;
                const uint4* ks = reinterpret_cast<const uint4*>(p.ck_rot + rowi * kHeadDim) + 4 * uq;
                const uint4* vs = reinterpret_cast<const uint4*>(p.cv_rot + rowi * kHeadDim) + 4 * uq;
                uint4 kq[4], vq[4];
#pragma unroll
                for (int wi = 0; wi < 4; ++wi) {
                    kq[wi] = __ldg(ks + wi);
                    vq[wi] = __ldg(vs + wi);
                }
#pragma unroll
                for (int wi = 0; wi < 4; ++wi) {
                    *reinterpret_cast<uint4*>(ktile + uh * 8192 + sw128(ut, 4 * (uq & 1) + wi)) = kq[wi];
                    *reinterpret_cast<uint4*>(vtile + uh * 8192 + sw128(ut, 4 * (uq & 1) + wi)) = vq[wi];
                }
                if (uq == 0) {
                    const bool ok = t0 + ut < p.nq;
                    kscale[ut] = ok ? 1.0f : 0.0f;
                    vscale[ut] = ok ? 1.0f / TQ_ALPHA4T : 0.0f;
                }
            }
            fence_async_smem();
            mbar_arrive(bar_kv_full + 8 * st);
            if (++st == kKvStages) {
                st = 0;
                ++kv_round;
            }
            raw_rd = raw_rd == kOffRaw + (kRawStages - 1) * kRawStage ? kOffRaw : raw_rd + kRawStage;
        };
        prefetch_next();
        prefetch_next();
        for (int it = 0; it < n_tiles && !fail; ++it) do_tile(it);
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else if (warp == 12) {
        // =========================== MMA issuer ===========================
        if (lane == 0) {
            // Two counters: S tiles issued, P V tiles issued.  Whichever operand set is ready first
            // is issued first; S may run at most two tiles ahead of P V (two S buffers).
            int next_s = 0, next_pv = 0, idle = 0;
            int s_stage = 0, pv_stage = 0;   // next_s % kKvStages, next_pv % kKvStages
            uint32_t s_phase = 0;            // (next_s / kKvStages) & 1
            while (next_pv < n_tiles) {
                bool progress = false;
                if (next_s < n_tiles && next_s <= next_pv + 1 &&
                    mbar_test(bar_kv_full + 8 * s_stage, s_phase)) {
                    tc_fence_after();
                    const uint32_t k_lo = desc_lo(sbase + kOffKV + s_stage * 32768, 16);
                    const uint32_t s_tmem = tmem + 64 * (next_s & 1);
                    // k-steps 0-7: Q hi, 8-15: Q lo against the same K tile (dim chunk (ks & 7) / 4, 32 bytes per step)
                    mma_f16_ts_words<false>(s_tmem, tmem_q, k_lo, desc_hi(1024), kIdescS);
#pragma unroll
                    for (int ks = 1; ks < 16; ++ks)
                        mma_f16_ts_words<true>(s_tmem, tmem_q + 8 * ks,
                                               k_lo + ((((ks & 7) >> 2) * 8192 + (ks & 3) * 32) >> 4), desc_hi(1024), kIdescS);
                    mma_commit(bar_s_full + 8 * (next_s & 1));
                    ++next_s;
                    if (++s_stage == kKvStages) {
                        s_stage = 0;
                        s_phase ^= 1u;
                    }
                    progress = true;
                }
                if (next_pv < next_s && mbar_test(bar_p_full + 8 * (next_pv & 1), (next_pv >> 1) & 1)) {
                    tc_fence_after();
                    const uint32_t v_lo = desc_lo(sbase + kOffKV + pv_stage * 32768 + 16384, 8192);
                    const uint32_t p_tmem = tmem_p + 32 * (next_pv & 1);
                    // 16 tokens = 8 TMEM columns of P per instruction
                    if (next_pv > 0) mma_f16_ts_words<true>(tmem_o, p_tmem, v_lo, desc_hi(1024), kIdescPV);
                    else mma_f16_ts_words<false>(tmem_o, p_tmem, v_lo, desc_hi(1024), kIdescPV);
#pragma unroll
                    for (int ks = 1; ks < 4; ++ks)
                        mma_f16_ts_words<true>(tmem_o, p_tmem + 8 * ks, v_lo + ks * (2048 >> 4), desc_hi(1024), kIdescPV);
                    mma_commit(bar_pv_done + 8 * (next_pv & 1));
                    mma_commit(bar_kv_empty + 8 * pv_stage);
                    ++next_pv;
                    if (++pv_stage == kKvStages) pv_stage = 0;
                    progress = true;
                }
                if (progress) {
                    idle = 0;
                } else {
                    // a tight polling loop would take issue slots from the warps of this scheduler: sleep in
                    // the barrier unit on the condition that comes first in a steady pipeline (the P tile of
                    // the oldest open product, else the next K/V tile), at most a microsecond at a time
                    if (next_pv < next_s)
                        mbar_try_wait_for(bar_p_full + 8 * (next_pv & 1), (next_pv >> 1) & 1, 1000u);
                    else
                        mbar_try_wait_for(bar_kv_full + 8 * s_stage, s_phase, 1000u);
                    if (++idle > kWaitLimit) {
                        fail = 2;
                        break;
                    }
                }
            }
        }
    } else {
        // =========================== softmax warps ===========================
        // Two threads per row: warps 0-3 take the tile's tokens 0-31, warps 8-11 tokens 32-63 (both
        // sets may touch TMEM lanes 32 (warp % 4) ..).  The two threads of a row agree on the
        // row maximum through shared memory and a 64-thread named barrier per warp pair.  After a
        // failed wait a warp keeps walking the loop (without waiting) so its partner never blocks.
        const int half = warp >> 3;                       // 0: tokens 0-31 of a tile, 1: tokens 32-63
        const int r = (warp & 3) * 32 + lane;             // row of the tile = TMEM lane
        const int rg = mt * kRowsCta + r;                 // row of this (sequence, kv head)
        const int tok = min(rg, rows_total - 1) / G;      // chunk position of the row's token
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const int pair_bar = 1 + (warp & 3);
        float* xch = reinterpret_cast<float*>(smem + kOffXch);  // [2 buffers][2 halves][128 rows]
        float m_use = kInitMaxLogit, l_run = 0.0f;
        for (int it = 0; it < n_tiles; ++it) {
            const int st = it & 1;
            const bool is_chunk = it >= n_pref;
            const int t0 = (is_chunk ? (it - n_pref) * kTileTok : (tile_lo + it) * kTileTok) + 32 * half;
            const int n_valid = is_chunk ? p.nq : n_prefix;
            if (!fail && !warp_wait(bar_s_full + 8 * st, (it >> 1) & 1)) fail = 4;
            tc_fence_after();
            const float* kscale = reinterpret_cast<const float*>(smem + kOffScale) + (it % kKvStages) * 128 + 32 * half;
            const float* vscale = kscale + 64;
            // the row's 32 scores as 16 packed pairs: scale, mask, maximum (packed fp32 arithmetic)
            float2 s2[16];
            {
                float s[32];
                tmem_ld32(tmem + lane_base + 64 * st + 32 * half, s);
#pragma unroll
                for (int j = 0; j < 16; j += 2) {
                    const float4 kc = *reinterpret_cast<const float4*>(kscale + 2 * j);
                    s2[j] = mul2(make_float2(s[2 * j], s[2 * j + 1]), make_float2(kc.x, kc.y));
                    s2[j + 1] = mul2(make_float2(s[2 * j + 2], s[2 * j + 3]), make_float2(kc.z, kc.w));
                }
            }
            const bool need_mask = is_chunk || t0 + 32 > n_valid;
            if (need_mask) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int t = t0 + 2 * j;
                    if (!(t < n_valid && (!is_chunk || t <= tok))) s2[j].x = -INFINITY;
                    if (!(t + 1 < n_valid && (!is_chunk || t + 1 <= tok))) s2[j].y = -INFINITY;
                }
            }
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 16; ++j) mx = fmaxf(mx, fmaxf(s2[j].x, s2[j].y));
            // exchange the half-row maxima
            xch[(st * 2 + half) * 128 + r] = mx;
            asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
            mx = fmaxf(mx, xch[(st * 2 + (half ^ 1)) * 128 + r]);
            // keep the maximum in use until the true one runs ahead by more than kRescaleLag
            const float m_true = fmaxf(m_use, mx);
            const bool grow = m_true > m_use + kRescaleLag || (it == 0);
            const float m_new = grow ? m_true : m_use;
            if (it > 0 && __any_sync(0xffffffffu, grow)) {
                // O *= 2^(m_use - m_new) on this thread's 64 columns: the previous P V must have landed
                if (!fail && !warp_wait(bar_pv_done + 8 * ((it - 1) & 1), ((it - 1) >> 1) & 1)) fail = 5;
                tc_fence_after();
                const float al = ex2_t(m_use - m_new);
                l_run *= al;
#pragma unroll 1
                for (int c0 = 64 * half; c0 < 64 * half + 64; c0 += 32) {
                    float o[32];
                    tmem_ld32(tmem_o + lane_base + c0, o);
#pragma unroll
                    for (int j = 0; j < 32; ++j) o[j] *= al;
                    tmem_st32(tmem_o + lane_base + c0, o);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            }
            m_use = m_new;
            float2 vs2[16];
#pragma unroll
            for (int j = 0; j < 16; j += 2) {
                const float4 vc = *reinterpret_cast<const float4*>(vscale + 2 * j);
                vs2[j] = make_float2(vc.x, vc.y);
                vs2[j + 1] = make_float2(vc.z, vc.w);
            }
            const float2 neg_m = make_float2(-m_use, -m_use);
            float2 ls2 = make_float2(0.0f, 0.0f);
            uint32_t pw[16];  // P * (V scale) of this thread's 32 tokens as 16 fp16 pairs
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float2 a = add2(s2[j], neg_m);
                const float2 pp = make_float2(ex2_t(a.x), ex2_t(a.y));
                ls2 = add2(ls2, pp);
                const float2 pv = mul2(pp, vs2[j]);
                const __half2 hh = __floats2half2_rn(pv.x, pv.y);
                pw[j] = *reinterpret_cast<const uint32_t*>(&hh);
            }
            l_run += ls2.x + ls2.y;
            // P goes to TMEM as the A operand of the second product: lane = row, 32-bit column c of
            // the buffer holds tokens 2c, 2c+1 of the tile (this thread: columns 16 half .. + 15)
            tmem_st16(tmem_p + lane_base + 32 * st + 16 * half, pw);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            mbar_arrive(bar_p_full + 8 * st);
        }
        // ---- epilogue: the row's partial (acc, m in natural-log units, l); each thread 64 dims ----
        {
            float* out = nullptr;
            if (rg < rows_total) {
                const long long seq = static_cast<long long>(b) * p.nq + rg / G;
                out = p.partials + ((seq * p.splits + split) * p.hq + h * G + rg % G) * TQ_PARTIAL_STRIDE;
            }
            if (n_tiles > 0) {
                if (!fail && !warp_wait(bar_pv_done + 8 * ((n_tiles - 1) & 1), ((n_tiles - 1) >> 1) & 1)) fail = 6;
                tc_fence_after();
            }
            if (half == 1) xch[r] = l_run;
            asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
            if (half == 0) l_run += xch[r];
#pragma unroll 1
            for (int c0 = 64 * half; c0 < 64 * half + 64; c0 += 32) {
                float o[32];
                if (n_tiles > 0) {
                    tmem_ld32(tmem_o + lane_base + c0, o);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) o[j] = 0.0f;
                }
                if (out && !fail) {
#pragma unroll
                    for (int j = 0; j < 32; j += 2)  // records are 520 bytes apart: 8-byte aligned only
                        *reinterpret_cast<float2*>(out + c0 + j) = make_float2(o[j], o[j + 1]);
                }
            }
            if (out && !fail && half == 0) {
                out[128] = m_use * kLn2T;
                out[129] = l_run;
            }
        }
    }
    if (fail) atomicMax(&g_prefill_tc_status, fail);
    tc_fence_before();
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
}

}  // namespace

int prefill_tc_status() {
    int v = 0;
    check_cuda(cudaMemcpyFromSymbol(&v, g_prefill_tc_status, sizeof v), "cudaMemcpyFromSymbol(prefill status)");
    return v;
}

void launch_prefill_tc(const void* query, const uint8_t* pool, const int32_t* block_tables,
                       int table_stride, const int32_t* seq_lens, const void* chunk_key,
                       const void* chunk_value, void* output, const PageGeom& geo, int head_dim,
                       int batch, int nq, int hq, int max_prefix_tokens, cudaStream_t stream) {
    const int H = geo.num_kv_heads;
    if (batch <= 0 || nq <= 0) return;
    if (hq % H != 0) throw std::runtime_error("prefill: num_q_heads must be a multiple of num_kv_heads");
    if (geo.block_size != 16) throw std::runtime_error("prefill: block_size must be 16");
    if ((reinterpret_cast<uintptr_t>(pool) & 15) || (geo.page_size & 15) || (geo.k_codes & 15) ||
        (geo.v_codes & 15) || (geo.k_scales & 3) || (geo.v_scales & 3))
        throw std::runtime_error("prefill: page pool must be 16-byte aligned");
    const int G = hq / H;
    const long long q_rows = static_cast<long long>(batch) * nq * hq;
    const long long kv_rows = chunk_key ? static_cast<long long>(batch) * nq * H : 0;
    const int rows_total = nq * G;
    const int mtiles = (rows_total + kRowsCta - 1) / kRowsCta;
    const int prefix_tiles = (max_prefix_tokens + kTileTok - 1) / kTileTok;
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
    const size_t q_bytes = static_cast<size_t>(q_rows) * kHeadDim * 2;
    const size_t kv_bytes = static_cast<size_t>(kv_rows) * kHeadDim * 2;
    const size_t part_bytes = static_cast<size_t>(q_rows) * splits * TQ_PARTIAL_STRIDE * sizeof(float);
    auto up = [](size_t x) { return (x + 255) / 256 * 256; };
    uint8_t* ws = nullptr;
    ws = static_cast<decltype(ws)>(scratch_alloc(2 * up(q_bytes) + 2 * up(kv_bytes) + part_bytes, stream,
                                                 "scratch_alloc(prefill workspace)"));
    __half* q_rot = reinterpret_cast<__half*>(ws);
    __half* q_rot_lo = reinterpret_cast<__half*>(ws + up(q_bytes));
    __half* ck_rot = reinterpret_cast<__half*>(ws + 2 * up(q_bytes));
    __half* cv_rot = reinterpret_cast<__half*>(ws + 2 * up(q_bytes) + up(kv_bytes));
    float* partials = reinterpret_cast<float*>(ws + 2 * up(q_bytes) + 2 * up(kv_bytes));

    const uint32_t alpha_bits = 0x404c9252u;
    float alpha;
    std::memcpy(&alpha, &alpha_bits, sizeof alpha);
    // q' = R(q) / sqrt(D) * log2(e) / alpha: the rotation's own 1/sqrt(D) is applied in the kernel
    rotate_rows_tc_kernel<<<static_cast<unsigned>((q_rows + 3) / 4), 128, 0, stream>>>(
        static_cast<const __half*>(query), q_rot, q_rot_lo, q_rows, hq, G, kLog2eT / alpha * 0.08838834764831845f,
        head_dim);
    check_launch("prefill rotate q");
    if (chunk_key) {
        rotate_rows_tc_kernel<<<static_cast<unsigned>((kv_rows + 3) / 4), 128, 0, stream>>>(
            static_cast<const __half*>(chunk_key), ck_rot, nullptr, kv_rows, H, 1, alpha, head_dim);
        rotate_rows_tc_kernel<<<static_cast<unsigned>((kv_rows + 3) / 4), 128, 0, stream>>>(
            static_cast<const __half*>(chunk_value), cv_rot, nullptr, kv_rows, H, 1, alpha, head_dim);
        check_launch("prefill rotate chunk");
    }
    PrefillTcParams p{};
    p.q_rot = q_rot;
    p.q_rot_lo = q_rot_lo;
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
    static bool attr[64] = {};
    int dev = 0;
    check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (dev >= 0 && dev < 64 && !attr[dev]) {
        check_cuda(cudaFuncSetAttribute(prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTc),
                   "prefill smem attr");
        attr[dev] = true;
    }
    prefill_tc_kernel<<<dim3(mtiles, H * splits, batch), kThreadsTc, kSmemTc, stream>>>(p);
    check_launch("turbo_mse prefill (tcgen05)");
    launch_merge_splits(partials, splits, output, static_cast<int>(q_rows), hq, H, head_dim, stream);
    scratch_free(ws, stream, "scratch_free(prefill workspace)");
}

}  // namespace tq
