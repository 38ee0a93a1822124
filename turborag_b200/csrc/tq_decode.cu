// Fused decode attention over compressed pages (turbo_prod and turbo_mse), sm_100a.
//
// Replaces turbo_prod_fused_attention_logits_kernel / turbo_prod_fused_attn_online_kernel
// (src/cuda/tq_turbo_prod_kernels.cu:346-571) and turbo_mse_fused_attn_online_kernel
// (src/cuda/tq_turbo_mse_kernels.cu:302-417).  The reference walks the KV tokens
// serially inside one 128-thread CTA per (query, kv-head); here
//   * the KV range of every sequence is cut into splits (one CTA each) and, inside
//     a CTA, into per-warp streams of 16-token blocks; (acc, m, l) partials are
//     merged by log-sum-exp (second kernel, also the multi-GPU reducer);
//   * a warp owns one kv-head of a block: the 16x128 code tile is the A operand
//     of mma.sync m16n8k16 (rows = tokens), the up-to-8 query heads that share the
//     kv-head are the 8 columns, so GQA costs no extra code traffic or unpack work;
//   * a code byte (two 4-bit fields) becomes two fp16 operands either by one lookup in a
//     byte-indexed, lane-replicated shared-memory table (paged fast path) or by byte-permute
//     lookups in registers (general kernel: 8-entry signed table for the 3-bit K code, 8-entry
//     magnitude table plus a sign XOR for the 4-bit codes); the 1-bit residual sign is a second
//     MMA with +-1 operands, scaled per token column (ks*re) afterwards;
//   * V^T is the A operand of the second product; its k index runs over tokens, so a fragment
//     register pairs the same dim of two adjacent tokens: built in registers, by looking up an
//     index byte made of the two tokens' nibbles (fast path) or by paired permutes (general
//     kernel); no shared-memory transpose.
// Arithmetic: rotated-domain dot products in fp16 x fp16 -> fp32, softmax state
// and accumulators in fp32 (within 2e-3 of the reference's fp32 path).
#include <climits>
#include <type_traits>
#include <mutex>

#include "tq_common.cuh"
#include "tq_launch.h"

namespace tq {
namespace {

// ---- programmatic dependent launch -------------------------------------------------------
// The paged decode kernel and the merge kernel are launched with the programmatic stream
// serialisation attribute: each lets the next kernel in the stream start while it is still
// running (pdl_launch_dependents at its top) and waits for everything before it in the stream
// to complete (pdl_wait) before it reads an input or writes an output.  What overlaps is only
// work that depends on nothing -- the next decode launch's operand-table build and block
// scheduling run under this launch's tail and merge instead of after them.  Both instructions
// do nothing in a kernel that was launched the ordinary way.
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
void launch_after_wait(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                       cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    check_cuda(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...), "cudaLaunchKernelEx");
}

constexpr int kMaxHeads = 8;          // kv heads per CTA
constexpr int kWarpSmemBytes = 4608;  // per-warp merge record: 36 floats x 32 lanes
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
// The fp16 lookup tables hold alpha * level: alpha is chosen so that every
// scaled level lands within 1.4e-5 (3-bit table) / 9.3e-5 (4-bit table) of an
// fp16 value, against 4.2e-4 / 3.1e-4 unscaled; 1/alpha is folded into the fp32
// query scale (K side) and into the per-token V scale.
#define TQ_ALPHA3 TQF(0x3fa55cec)
#define TQ_ALPHA4 TQF(0x404c9252)
#define TQ_POOL3_HI_A 0xb5bbbec1u
#define TQ_POOL3_HI_B 0x413e3b35u
#define TQ_POOL3_LO_A 0x10cff18fu
#define TQ_POOL3_LO_B 0x8ff1cf10u
#define TQ_MAG4_HI_A 0x42403c36u
#define TQ_MAG4_HI_B 0x48464544u
#define TQ_MAG4_LO_A 0x0633f691u
#define TQ_MAG4_LO_B 0x5e9d2c04u

struct DecodeParams {
    const __half* query;
    const uint8_t* pool;
    const int32_t* slot_mapping;
    const int32_t* block_tables;
    const int32_t* seq_lens;
    float* partials;  // [batch, splits, rows_per_seq, 130]
    float* logits;
    PageGeom geo;
    int table_stride;
    int head_dim;
    int groups;        // query heads per kv head
    int ref_layout;    // query row of (g, h): g*H+h if set, else h*G+g
    int max_kv_tokens;
    int kv_begin, kv_end;
    int splits;
    int batch;
    int streams;       // warps per kv head inside a group
    int bs_shift;      // log2(block_size) or -1
    int aligned16;     // every code row starts on a 16-byte boundary
    int head0, heads;  // kv heads [head0, head0 + heads) are served by this launch (heads <= 8)
};

// ---- small PTX wrappers ------------------------------------------------------

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
// (a & b) ^ c and (a & m) | (b & ~m) as ONE three-input logic instruction each.  Written as the
// instruction: left to the compiler, expressions of this kind with two constant operands came out
// as two or more operations (measured: 72 logic instructions per 16-token block for the residual
// signs where 32 suffice).
__device__ __forceinline__ uint32_t lop3_and_xor(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t lop3_select(uint32_t a, uint32_t b, uint32_t m) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xE4;" : "=r"(d) : "r"(a), "r"(b), "r"(m));
    return d;
}
// x >> N as the high word of x * 2^(32-N): runs on the multiply-add pipe, which the unpack
// leaves idle, instead of the half-rate integer/logic pipe that limits this kernel.
template <int N>
__device__ __forceinline__ uint32_t shr_mul(uint32_t x) {
    uint32_t d;
    asm("mul.hi.u32 %0, %1, %2;" : "=r"(d) : "r"(x), "r"(1u << (32 - N)));
    return d;
}
// x << N on the same pipe.
template <int N>
__device__ __forceinline__ uint32_t shl_mul(uint32_t x) {
    uint32_t d;
    asm("mul.lo.u32 %0, %1, %2;" : "=r"(d) : "r"(x), "r"(1u << N));
    return d;
}
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// Byte pools for the permute lookups: entry e of an 8-entry fp16 table is split
// into its high byte (pool hi.x/hi.y) and low byte (pool lo.x/lo.y).
struct BytePools {
    uint32_t hi_a, hi_b, lo_a, lo_b;
};

// Eight 3-bit selectors (one per nibble, bit 3 of every nibble clear) -> four
// half2 registers holding the table values of nibble pairs (0,4) (1,5) (2,6) (3,7).
__device__ __forceinline__ void lookup8(uint32_t sel, const BytePools& t, uint32_t (&out)[4]) {
    const uint32_t y = prmt(sel, sel, 0x3120u);  // nibbles 0,1,4,5 | 2,3,6,7
    const uint32_t yh = shr_mul<16>(y);
    const uint32_t h_lo = prmt(t.hi_a, t.hi_b, y), l_lo = prmt(t.lo_a, t.lo_b, y);
    const uint32_t h_hi = prmt(t.hi_a, t.hi_b, yh), l_hi = prmt(t.lo_a, t.lo_b, yh);
    out[0] = prmt(l_lo, h_lo, 0x6240u);
    out[1] = prmt(l_lo, h_lo, 0x7351u);
    out[2] = prmt(l_hi, h_hi, 0x6240u);
    out[3] = prmt(l_hi, h_hi, 0x7351u);
}

// turbo_prod K word: 3-bit code -> signed level (nibble bit 3 masked off).
__device__ __forceinline__ void unpack_k3(uint32_t w, const BytePools& t, uint32_t (&out)[4]) {
    lookup8(w & 0x77777777u, t, out);
}
// Residual sign bits (bit 3 of every nibble) -> +-1.0 halves, same pairing.
__device__ __forceinline__ void unpack_sign(uint32_t w, uint32_t (&out)[4]) {
    out[0] = lop3_and_xor(shl_mul<12>(w), 0x80008000u, 0xBC00BC00u);
    out[1] = lop3_and_xor(shl_mul<8>(w), 0x80008000u, 0xBC00BC00u);
    out[2] = lop3_and_xor(shl_mul<4>(w), 0x80008000u, 0xBC00BC00u);
    out[3] = lop3_and_xor(w, 0x80008000u, 0xBC00BC00u);
}
// 4-bit code n -> cb4[n]: magnitude index is n-8 for n >= 8 and 7-n below, the sign bit is
// set when bit 3 of the nibble is clear.  `neg` gets bit 3 of every negative nibble,
// `sel` the 3-bit magnitude selectors.
__device__ __forceinline__ void c4_selectors(uint32_t w, uint32_t& sel, uint32_t& neg) {
    neg = ~w & 0x88888888u;
    uint32_t flip;  // 7 in every negative nibble: (neg * 7) >> 3 as one high multiply
    asm("mul.hi.u32 %0, %1, %2;" : "=r"(flip) : "r"(neg), "r"(0xE0000000u));
    sel = (w ^ flip) & 0x77777777u;
}
// One word of one token: pairs are nibbles (0,4) (1,5) (2,6) (3,7) (K operand of turbo_mse).
__device__ __forceinline__ void unpack_c4(uint32_t w, const BytePools& mag, uint32_t (&out)[4]) {
    uint32_t sel, neg;
    c4_selectors(w, sel, neg);
    lookup8(sel, mag, out);
    out[0] = lop3_and_xor(shl_mul<12>(neg), 0x80008000u, out[0]);
    out[1] = lop3_and_xor(shl_mul<8>(neg), 0x80008000u, out[1]);
    out[2] = lop3_and_xor(shl_mul<4>(neg), 0x80008000u, out[2]);
    out[3] = lop3_and_xor(neg, 0x80008000u, out[3]);
}
// The same word of two tokens A and B: out[d] = half2(level of A's nibble d, level of B's
// nibble d), d = 0..7 -- pairs run along tokens, which is what the k index of the V^T
// operand needs, so V never goes through a shared-memory transpose.
__device__ __forceinline__ void unpack_c4_token_pair(uint32_t wa, uint32_t wb, const BytePools& t,
                                                     uint32_t (&out)[8]) {
    uint32_t sa, sb, na, nb;
    c4_selectors(wa, sa, na);
    c4_selectors(wb, sb, nb);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        // bytes [A.b(2h), B.b(2h), A.b(2h+1), B.b(2h+1)]: 16 selector bits per nibble pair
        const uint32_t y = prmt(sa, sb, half ? 0x7362u : 0x5140u);
        const uint32_t yh = shr_mul<16>(y);
        const uint32_t h0 = prmt(t.hi_a, t.hi_b, y), l0 = prmt(t.lo_a, t.lo_b, y);
        const uint32_t h1 = prmt(t.hi_a, t.hi_b, yh), l1 = prmt(t.lo_a, t.lo_b, yh);
        // sign bits of A's nibbles 4h..4h+3 in the low half-word, of B's in the high one
        const uint32_t z = prmt(na, nb, half ? 0x7632u : 0x5410u);
        out[4 * half + 0] = lop3_and_xor(shl_mul<12>(z), 0x80008000u, prmt(l0, h0, 0x6240u));
        out[4 * half + 1] = lop3_and_xor(shl_mul<8>(z), 0x80008000u, prmt(l0, h0, 0x7351u));
        out[4 * half + 2] = lop3_and_xor(shl_mul<4>(z), 0x80008000u, prmt(l1, h1, 0x6240u));
        out[4 * half + 3] = lop3_and_xor(z, 0x80008000u, prmt(l1, h1, 0x7351u));
    }
}

// Slot of token t of sequence b.
__device__ __forceinline__ int token_slot(const DecodeParams& p, int b, int t) {
    if (p.slot_mapping) return __ldg(p.slot_mapping + t);
    const int bs = p.geo.block_size;
    const int pg = p.bs_shift >= 0 ? (t >> p.bs_shift) : t / bs;
    return __ldg(p.block_tables + static_cast<long long>(b) * p.table_stride + pg) * bs +
           (t - pg * bs);
}

struct Cell {
    const uint8_t* page;
    unsigned int th;
};
__device__ __forceinline__ Cell token_cell(const DecodeParams& p, int slot, int h) {
    const int bs = p.geo.block_size;
    const int blk = p.bs_shift >= 0 ? (slot >> p.bs_shift) : slot / bs;
    Cell c;
    c.page = p.pool + static_cast<unsigned long long>(blk) * p.geo.page_size;
    c.th = static_cast<unsigned int>((slot - blk * bs) * p.geo.num_kv_heads + h);
    return c;
}

__device__ __forceinline__ uint4 ld16(const uint8_t* p, bool aligned) {
    if (aligned) return __ldg(reinterpret_cast<const uint4*>(p));
    uint32_t v[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i >> 2] |= static_cast<uint32_t>(p[i]) << (8 * (i & 3));
    return make_uint4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ float ld_scale(const uint8_t* p) {
    return __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short*>(p))));
}

__device__ __forceinline__ uint2 ld8(const uint8_t* p, bool aligned) {
    if (aligned) return __ldg(reinterpret_cast<const uint2*>(p));
    uint32_t v[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i >> 2] |= static_cast<uint32_t>(p[i]) << (8 * (i & 3));
    return make_uint2(v[0], v[1]);
}

// Raw (still packed) data of one 16-token block for one lane (g = lane/4, tig = lane%4).
struct BlockRaw {
    uint4 k0, k1;  // K codes of token rows g and g+8, bytes [16 tig, 16 tig + 16)
    uint2 v[4];    // V codes of token rows 2tig, 2tig+1, 2tig+8, 2tig+9, bytes [8g, 8g+8)
    float ks0, ks1, re0, re1, vs0, vs1;  // scales of token rows g and g+8
};

// QJL-1bit rows are 16 bytes of sign bits: the lane's 32 dims are word tig of the row.
__device__ __forceinline__ uint32_t ld4(const uint8_t* p, bool aligned) {
    if (aligned) return __ldg(reinterpret_cast<const uint32_t*>(p));
    uint32_t v = 0u;
#pragma unroll
    for (int i = 0; i < 4; ++i) v |= static_cast<uint32_t>(p[i]) << (8 * i);
    return v;
}

template <bool PROD, bool QJL = false>
__device__ __forceinline__ void load_block(const DecodeParams& p, int b, int h, int tb, int t_end,
                                           int lane, bool aligned, BlockRaw& r) {
    const int g = lane >> 2, tig = lane & 3;
    const int last = t_end - 1;  // rows past the end re-read the last token (masked later)
    const Cell c0 = token_cell(p, token_slot(p, b, min(tb + g, last)), h);
    const Cell c1 = token_cell(p, token_slot(p, b, min(tb + g + 8, last)), h);
    if (QJL) {
        r.k0 = make_uint4(ld4(c0.page + p.geo.k_codes + c0.th * 16 + 4 * tig, aligned), 0u, 0u, 0u);
        r.k1 = make_uint4(ld4(c1.page + p.geo.k_codes + c1.th * 16 + 4 * tig, aligned), 0u, 0u, 0u);
    } else {
        r.k0 = ld16(c0.page + p.geo.k_codes + c0.th * 64 + 16 * tig, aligned);
        r.k1 = ld16(c1.page + p.geo.k_codes + c1.th * 64 + 16 * tig, aligned);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t = tb + 2 * tig + (i & 1) + 8 * (i >> 1);
        const Cell cv = token_cell(p, token_slot(p, b, min(t, last)), h);
        r.v[i] = ld8(cv.page + p.geo.v_codes + cv.th * 64 + 8 * g, aligned);
    }
    r.ks0 = ld_scale(c0.page + p.geo.k_scales + c0.th * 2);
    r.ks1 = ld_scale(c1.page + p.geo.k_scales + c1.th * 2);
    r.vs0 = ld_scale(c0.page + p.geo.v_scales + c0.th * 2);
    r.vs1 = ld_scale(c1.page + p.geo.v_scales + c1.th * 2);
    if (PROD) {
        r.re0 = ld_scale(c0.page + p.geo.k_res + c0.th * 2);
        r.re1 = ld_scale(c1.page + p.geo.k_res + c1.th * 2);
    } else {
        r.re0 = r.re1 = 0.0f;
    }
}

// Everything a warp keeps across the blocks of its stream.
struct WarpState {
    float o[8][4];      // O^T accumulators: 8 tiles of 16 dims x 8 queries
    float m_run[2], l_run[2];
};

struct BlockCtx {
    uint32_t qf[8][2];  // B fragments of the rotated, pre-scaled queries
    uint32_t qlo[8][2];  // QJL only: fp16 remainders of the same values
    const uint4* qsign;  // fast path, turbo_prod: this head's query fragments in the (d, d+4) pairing, [4][32]
    BytePools pool3, mag4;
    float inv_alpha_v;
    uint8_t* warp_smem;   // per-warp shared region (merge record at the end; fast path: ring)
    uint32_t warp_smem_addr;
    const uint8_t* lut;   // byte -> operand tables in shared memory (fast path only)
    uint32_t lane_k, lane_v;  // this lane's replica offsets inside a table row
    uint8_t* group_smem;  // first per-warp region of this warp's group (merge records)
    int bar_id, bar_threads;  // barrier shared by the warps that work on one (sequence, split)
    int lane, g, tig, h, H, nq, gq0;  // h: kv head (global index), H: kv heads of the page layout
    int hl, Hl;                       // head index inside this launch, heads of this launch
};

// ---- shared-memory operand tables (paged fast path) -----------------------------------
// Turning a code byte (two 4-bit fields) into MMA operands with byte permutes costs about two
// integer-pipe instructions per element, and that pipe bounds the kernel.  The fast path looks
// the byte up instead: row r (256 bytes) of the table belongs to byte value r,
//   bytes   0..127: 32 replicas of the half2 levels of the two 3-bit K codes of turbo_prod,
//   bytes 128..255: 32 replicas of the half2 levels of the two 4-bit codes;
// lane l reads replica l with a 4-byte load, so every lookup is one conflict-free wavefront.
// Shared-memory bandwidth is 4 operand bytes per lane per wavefront whatever the access width,
// which is why the +-1 residual-sign operands are not looked up: they cost two logic-pipe
// operations per pair (see sign_pairs), a lookup would double the K lookups' wavefronts.
// The address is one byte permute: byte 1 = the code byte, byte 0 = the lane's replica offset.
constexpr int kLutBytes = 256 * 256;

__device__ __forceinline__ uint32_t pool_entry(uint32_t hi_a, uint32_t hi_b, uint32_t lo_a,
                                               uint32_t lo_b, uint32_t e) {
    const uint32_t sh = 8u * (e & 3u);
    const uint32_t hi = ((e < 4u ? hi_a : hi_b) >> sh) & 0xFFu;
    const uint32_t lo = ((e < 4u ? lo_a : lo_b) >> sh) & 0xFFu;
    return (hi << 8) | lo;
}
// fp16 bits of alpha3 * (signed 3-bit level), alpha4 * (signed 4-bit level)
__device__ __forceinline__ uint32_t level3_bits(uint32_t code) {
    return pool_entry(TQ_POOL3_HI_A, TQ_POOL3_HI_B, TQ_POOL3_LO_A, TQ_POOL3_LO_B, code & 7u);
}
__device__ __forceinline__ uint32_t level4_bits(uint32_t n) {
    const uint32_t mag = n >= 8u ? n - 8u : 7u - n;
    return pool_entry(TQ_MAG4_HI_A, TQ_MAG4_HI_B, TQ_MAG4_LO_A, TQ_MAG4_LO_B, mag) |
           (n >= 8u ? 0u : 0x8000u);
}
// All threads of the CTA; the caller synchronises afterwards.
__device__ __forceinline__ void build_operand_lut(uint8_t* lut) {
    for (int i = threadIdx.x; i < 512; i += blockDim.x) {
        const uint32_t row = i >> 1, part = i & 1;
        const uint32_t n0 = row & 15u, n1 = row >> 4;
        const uint32_t lv3 = level3_bits(n0) | (level3_bits(n1) << 16);
        const uint32_t lv4 = level4_bits(n0) | (level4_bits(n1) << 16);
        uint4* dk = reinterpret_cast<uint4*>(lut + row * 256 + part * 64);
        uint4* dv = reinterpret_cast<uint4*>(lut + row * 256 + 128 + part * 64);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            dk[k] = make_uint4(lv3, lv3, lv3, lv3);
            dv[k] = make_uint4(lv4, lv4, lv4, lv4);
        }
    }
}
// Residual-sign bits of one code word (bit 3 of every nibble) -> four half2 of +-1.0, pair p =
// nibbles 2p, 2p+1 (the pairing of the table lookups): a permute puts byte p of w << 4 under
// bit 15 and byte p of w under bit 31, one logic op keeps those two bits and adds 1.0.
__device__ __forceinline__ void sign_pairs(uint32_t w, uint32_t (&out)[4]) {
    const uint32_t ws = shl_mul<4>(w);
    out[0] = lop3_and_xor(prmt(ws, w, 0x4400u), 0x80008000u, 0xBC00BC00u);
    out[1] = lop3_and_xor(prmt(ws, w, 0x5511u), 0x80008000u, 0xBC00BC00u);
    out[2] = lop3_and_xor(prmt(ws, w, 0x6622u), 0x80008000u, 0xBC00BC00u);
    out[3] = lop3_and_xor(prmt(ws, w, 0x7733u), 0x80008000u, 0xBC00BC00u);
}
__device__ __forceinline__ uint32_t lut_v(const uint8_t* lut, uint32_t word, uint32_t lane_v, uint32_t sel) {
    return *reinterpret_cast<const uint32_t*>(lut + prmt(word, lane_v, sel));
}
__device__ __forceinline__ void group_sync(int bar_id, int nthreads) {
    if (bar_id == 0) __syncthreads();
    else asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(nthreads) : "memory");
}

// One 16-token block for one kv head: QK^T (+ residual-sign product), online softmax, PV.
// MODE 1 writes logits instead.
// half2(bit I of ~nw ? -1 : +1, bit J ...) from the complemented sign word: a set sign bit is +1.0
// (tq_qjl_kernels.cu:235, 298), so a set bit of nw = ~w puts the fp16 sign bit on top of 1.0.
template <int I, int J>
__device__ __forceinline__ uint32_t sign_half2(uint32_t nw) {
    uint32_t lo;
    if constexpr (I <= 15) lo = nw << (15 - I);
    else lo = nw >> (I - 15);
    const uint32_t hi = nw << (31 - J);
    return (lo & 0x8000u) | (hi & 0x80000000u) | 0x3C003C00u;
}

template <bool PROD, int MODE, bool LUT = false, bool QJL = false, bool SIGNQ = false, bool RAGGED = true>
__device__ __forceinline__ void process_block(const DecodeParams& p, const BlockCtx& c,
                                              const BlockRaw& cur, int tb, int t_end,
                                              WarpState& st) {
    const int g = c.g, tig = c.tig, h = c.h, H = c.H;
    const int nq = c.nq, gq0 = c.gq0;
    const BytePools pool3 = {TQ_POOL3_HI_A, TQ_POOL3_HI_B, TQ_POOL3_LO_A, TQ_POOL3_LO_B};
    const BytePools mag4 = {TQ_MAG4_HI_A, TQ_MAG4_HI_B, TQ_MAG4_LO_A, TQ_MAG4_LO_B};
    const float inv_alpha_v = c.inv_alpha_v;
    float (&o)[8][4] = st.o;
    float (&m_run)[2] = st.m_run;
    float (&l_run)[2] = st.l_run;
    const uint32_t (&qf)[8][2] = c.qf;
    // ---- S = K_hat Q'^T (rows = tokens g, g+8; cols = queries 2tig, 2tig+1) ----
    float s1[4] = {0.f, 0.f, 0.f, 0.f}, s2[4] = {0.f, 0.f, 0.f, 0.f};
    const uint32_t kw0[4] = {cur.k0.x, cur.k0.y, cur.k0.z, cur.k0.w};
    const uint32_t kw1[4] = {cur.k1.x, cur.k1.y, cur.k1.z, cur.k1.w};
    if constexpr (LUT) {
        // MMA n covers bytes 2n, 2n+1 of this lane's 16 code bytes: dims 32 tig + 4n + {0,1 | 2,3}
        uint32_t sg0[4], sg1[4];
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            const int wi = n >> 1;
            const uint32_t sa = (n & 1) ? 0x5524u : 0x5504u, sb = (n & 1) ? 0x5534u : 0x5514u;
            if (PROD) {
                const uint32_t e00 = lut_v(c.lut, kw0[wi], c.lane_k, sa);
                const uint32_t e10 = lut_v(c.lut, kw1[wi], c.lane_k, sa);
                const uint32_t e01 = lut_v(c.lut, kw0[wi], c.lane_k, sb);
                const uint32_t e11 = lut_v(c.lut, kw1[wi], c.lane_k, sb);
                mma16816(s1, e00, e10, e01, e11, qf[n][0], qf[n][1]);
                if constexpr (SIGNQ) {
                    // Residual signs paired (d, d+4): one shift on the multiplier pipe and one logic
                    // op per register (the table's (d, d+1) pairing costs a permute more, and the
                    // logic pipe is the busiest one).  The matching query fragments are not kept in
                    // registers: one 16-byte shared load per code word fetches them.
                    if ((n & 1) == 0) {
                        const uint4 qs = c.qsign[wi * 32 + c.lane];
                        unpack_sign(kw0[wi], sg0);
                        unpack_sign(kw1[wi], sg1);
                        mma16816(s2, sg0[0], sg1[0], sg0[1], sg1[1], qs.x, qs.y);
                        mma16816(s2, sg0[2], sg1[2], sg0[3], sg1[3], qs.z, qs.w);
                    }
                } else {
                    if ((n & 1) == 0) {
                        sign_pairs(kw0[wi], sg0);
                        sign_pairs(kw1[wi], sg1);
                    }
                    mma16816(s2, sg0[2 * (n & 1)], sg1[2 * (n & 1)], sg0[2 * (n & 1) + 1],
                             sg1[2 * (n & 1) + 1], qf[n][0], qf[n][1]);
                }
            } else {
                const uint32_t e00 = lut_v(c.lut, kw0[wi], c.lane_v, sa);
                const uint32_t e10 = lut_v(c.lut, kw1[wi], c.lane_v, sa);
                const uint32_t e01 = lut_v(c.lut, kw0[wi], c.lane_v, sb);
                const uint32_t e11 = lut_v(c.lut, kw1[wi], c.lane_v, sb);
                mma16816(s1, e00, e10, e01, e11, qf[n][0], qf[n][1]);
            }
        }
    } else if constexpr (QJL) {
        // MMA s = 2wi + hf takes dims 8wi + {2hf, 2hf+4 | 2hf+1, 2hf+5} of the lane's 32 (the
        // pairing of the query fragments): operands are +-1.0 straight from the sign bits
        const uint32_t n0 = ~kw0[0], n1 = ~kw1[0];
#define TQ_QJL_STEP(SV)                                                                                  \
    {                                                                                                    \
        const uint32_t a0 = sign_half2<8 * (SV >> 1) + 2 * (SV & 1), 8 * (SV >> 1) + 2 * (SV & 1) + 4>(n0);     \
        const uint32_t a1 = sign_half2<8 * (SV >> 1) + 2 * (SV & 1), 8 * (SV >> 1) + 2 * (SV & 1) + 4>(n1);     \
        const uint32_t a2 = sign_half2<8 * (SV >> 1) + 2 * (SV & 1) + 1, 8 * (SV >> 1) + 2 * (SV & 1) + 5>(n0); \
        const uint32_t a3 = sign_half2<8 * (SV >> 1) + 2 * (SV & 1) + 1, 8 * (SV >> 1) + 2 * (SV & 1) + 5>(n1); \
        mma16816(s1, a0, a1, a2, a3, qf[SV][0], qf[SV][1]);                                              \
        mma16816(s2, a0, a1, a2, a3, c.qlo[SV][0], c.qlo[SV][1]);                                        \
    }
        TQ_QJL_STEP(0); TQ_QJL_STEP(1); TQ_QJL_STEP(2); TQ_QJL_STEP(3);
        TQ_QJL_STEP(4); TQ_QJL_STEP(5); TQ_QJL_STEP(6); TQ_QJL_STEP(7);
#undef TQ_QJL_STEP
#pragma unroll
        for (int e = 0; e < 4; ++e) s1[e] += s2[e];  // hi and lo parts of the query
    } else {
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
        uint32_t a[4], bq[4];
        if (PROD) {
            unpack_k3(kw0[wi], pool3, a);
            unpack_k3(kw1[wi], pool3, bq);
        } else {
            unpack_c4(kw0[wi], mag4, a);
            unpack_c4(kw1[wi], mag4, bq);
        }
        mma16816(s1, a[0], bq[0], a[1], bq[1], qf[2 * wi][0], qf[2 * wi][1]);
        mma16816(s1, a[2], bq[2], a[3], bq[3], qf[2 * wi + 1][0], qf[2 * wi + 1][1]);
        if (PROD) {
            unpack_sign(kw0[wi], a);
            unpack_sign(kw1[wi], bq);
            mma16816(s2, a[0], bq[0], a[1], bq[1], qf[2 * wi][0], qf[2 * wi][1]);
            mma16816(s2, a[2], bq[2], a[3], bq[3], qf[2 * wi + 1][0], qf[2 * wi + 1][1]);
        }
    }
    }
    const bool ok0 = tb + g < t_end, ok1 = tb + g + 8 < t_end;
    // per-token scaling on packed fp32 pairs (the two query columns of a row are a register pair)
    float lg[4];
    {
        float2 lo = mul2(make_float2(s1[0], s1[1]), make_float2(cur.ks0, cur.ks0));
        float2 hi = mul2(make_float2(s1[2], s1[3]), make_float2(cur.ks1, cur.ks1));
        if (PROD) {
            // the sign product shares the 1/alpha-scaled query fragments
            const float2 rr = mul2(mul2(make_float2(cur.ks0, cur.ks1), make_float2(cur.re0, cur.re1)),
                                   make_float2(TQ_ALPHA3, TQ_ALPHA3));
            lo = fma2(make_float2(s2[0], s2[1]), make_float2(rr.x, rr.x), lo);
            hi = fma2(make_float2(s2[2], s2[3]), make_float2(rr.y, rr.y), hi);
        }
        lg[0] = lo.x;
        lg[1] = lo.y;
        lg[2] = hi.x;
        lg[3] = hi.y;
    }

    if (MODE == 1) {
        // logits[(q*H + h)*N + t]  (tq_turbo_prod_kernels.cu:428-431)
        const long long nkv = p.max_kv_tokens;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int col = 2 * tig + (e & 1);
            const int t = tb + g + 8 * (e >> 1);
            if (col < nq && t < t_end)
                p.logits[(static_cast<long long>(gq0 + col) * H + h) * nkv + t] = lg[e];
        }
        return;
    }

    if (RAGGED && tb + 16 > t_end) {  // only the last block of a sequence can be ragged
        if (!ok0) lg[0] = lg[1] = -INFINITY;
        if (!ok1) lg[2] = lg[3] = -INFINITY;
    }

    // ---- online softmax over the 16 tokens of the block ---------------------
    // The reference m of exp2(logit - m) is the running maximum, which only has to stay within
    // 2^kLazyBits of the true one: a block whose logits do not exceed m by more than that keeps
    // m (p <= 2^kLazyBits, no cross-lane maximum, no rescale).  Otherwise -- the first blocks of
    // a range and the occasional larger logit -- the whole warp reduces the block maximum
    // over the token lanes and rescales its sums, as a plain online softmax does every block.
    // 2^1.5 stays below the V table scale (TQ_ALPHA4 = 3.2), so the fp16 operand p * vs / alpha
    // is never larger than the row scale vs itself: no new overflow case for any fp16 input.
    constexpr float kLazyBits = 1.5f;
    static_assert(2.8285f < 3.19f, "2^kLazyBits must stay below TQ_ALPHA4");
    float mx0 = fmaxf(lg[0], lg[2]), mx1 = fmaxf(lg[1], lg[3]);
    if (__any_sync(0xffffffffu, (mx0 > m_run[0] + kLazyBits) | (mx1 > m_run[1] + kLazyBits))) {
#pragma unroll
        for (int msk = 4; msk < 32; msk <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, msk));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, msk));
        }
        const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
        const float2 dm = add2(make_float2(m_run[0], m_run[1]), make_float2(-mn0, -mn1));
        const float2 al = make_float2(ex2(dm.x), ex2(dm.y));
        m_run[0] = mn0;
        m_run[1] = mn1;
        const float2 ls = mul2(make_float2(l_run[0], l_run[1]), al);
        l_run[0] = ls.x;
        l_run[1] = ls.y;
        // packed multiplies: an accumulator tile's (col 2tig, col 2tig+1) pairs are register pairs
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float2 a = mul2(make_float2(o[j][0], o[j][1]), al);
            const float2 b = mul2(make_float2(o[j][2], o[j][3]), al);
            o[j][0] = a.x;
            o[j][1] = a.y;
            o[j][2] = b.x;
            o[j][3] = b.y;
        }
    }
    const float2 neg_mn = make_float2(-m_run[0], -m_run[1]);
    const float2 d01 = add2(make_float2(lg[0], lg[1]), neg_mn), d23 = add2(make_float2(lg[2], lg[3]), neg_mn);
    const float p0 = ex2(d01.x), p1 = ex2(d01.y);
    const float p2 = ex2(d23.x), p3 = ex2(d23.y);
    {
        const float2 ls = add2(make_float2(l_run[0], l_run[1]), add2(make_float2(p0, p1), make_float2(p2, p3)));
        l_run[0] = ls.x;
        l_run[1] = ls.y;
    }
    // P^T (k = token, n = query), V scale folded in
    const float2 wv = mul2(make_float2(cur.vs0, cur.vs1), make_float2(inv_alpha_v, inv_alpha_v));
    const float w0 = wv.x, w1 = wv.y;
    const float2 pw0 = mul2(make_float2(p0, p1), make_float2(w0, w0));
    const float2 pw1 = mul2(make_float2(p2, p3), make_float2(w1, w1));
    const uint32_t pb0 = movmatrix_trans(pack_half2(pw0.x, pw0.y));
    const uint32_t pb1 = movmatrix_trans(pack_half2(pw1.x, pw1.y));

    // ---- O^T += V^T P^T: A = V^T (rows = this lane's dims 16g + 2j + {0,1}, k = tokens) ----
    if constexpr (LUT) {
        // The A fragment pairs the same dim of two adjacent tokens.  The table row of byte
        // (nibble_lo | nibble_hi << 4) holds half2(level(lo), level(hi)), so an index byte made of
        // the two TOKENS' nibbles of one dim returns the fragment register itself: per code word of
        // a token pair, two logic ops build the index bytes of its even dims (lo) and odd dims (hi).
        constexpr uint32_t kLoNib = 0x0F0F0F0Fu;
        uint32_t ilo[2][2], ihi[2][2];  // [token pair][word]
#pragma unroll
        for (int pr = 0; pr < 2; ++pr) {
#pragma unroll
            for (int w = 0; w < 2; ++w) {
                const uint32_t wa = w ? cur.v[2 * pr].y : cur.v[2 * pr].x;          // token 2tig (+8)
                const uint32_t wb = w ? cur.v[2 * pr + 1].y : cur.v[2 * pr + 1].x;  // token 2tig+1 (+8)
                ilo[pr][w] = lop3_select(wa, shl_mul<4>(wb), kLoNib);
                ihi[pr][w] = lop3_select(shr_mul<4>(wa), wb, kLoNib);
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {  // tile j = byte j of the lane's 8 V bytes: dims 2j (row g), 2j+1 (row g+8)
            const uint32_t sel = 0x5504u | (static_cast<uint32_t>(j & 3) << 4);
            const int w = j >> 2;
            mma16816(o[j], lut_v(c.lut, ilo[0][w], c.lane_v, sel), lut_v(c.lut, ihi[0][w], c.lane_v, sel),
                     lut_v(c.lut, ilo[1][w], c.lane_v, sel), lut_v(c.lut, ihi[1][w], c.lane_v, sel), pb0, pb1);
        }
    } else {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        uint32_t ab[8], cd[8];
        unpack_c4_token_pair(i ? cur.v[0].y : cur.v[0].x, i ? cur.v[1].y : cur.v[1].x, mag4, ab);
        unpack_c4_token_pair(i ? cur.v[2].y : cur.v[2].x, i ? cur.v[3].y : cur.v[3].x, mag4, cd);
#pragma unroll
        for (int dd = 0; dd < 4; ++dd)
            mma16816(o[4 * i + dd], ab[2 * dd], ab[2 * dd + 1], cd[2 * dd], cd[2 * dd + 1], pb0, pb1);
    }
    }
}

// Per-CTA geometry shared by both kernels.
struct CtaRange {
    int split, b, G, rows_per_seq, stream, t_begin, t_end, blk_lo, blk_hi;
};

// Prologue: rotate this pass's queries (q' = FWHT(s .* q) * rsqrt(D), pre-scaled), build the
// B fragments and the lookup pools, and work out the CTA's block range.
// A "group" is the set of warps (H kv heads x p.streams streams) that works on one (sequence,
// split): the whole CTA in the general kernel, one half of the CTA in the paged fast path.
// `group_smem` is the group's first per-warp region, `qsm` a scratch of H*8*128 halves that is
// dead once the fragments are built, `warp` the warp's index inside the group.
template <bool PROD, int MODE, bool LUT = false, bool QJL = false>
__device__ __forceinline__ void decode_prologue(const DecodeParams& p, uint8_t* group_smem,
                                                int warp_bytes, __half* qsm, int warp, int seq,
                                                int split, int bar_id, int bar_threads,
                                                BlockCtx& ctx, CtaRange& r, uint4* qsign_group = nullptr) {
    const int lane = threadIdx.x & 31;
    const int H = p.geo.num_kv_heads;
    const int Hl = p.heads;
    const int hl = warp % Hl, stream = warp / Hl;
    const int h = p.head0 + hl;
    const int g = lane >> 2, tig = lane & 3;
    const int qg = blockIdx.z;
    r.split = split;
    r.b = seq;
    r.G = p.groups;
    r.rows_per_seq = r.G * H;
    r.stream = stream;
    const int gq0 = qg * 8;                  // first query of this pass within the group
    const int nq = min(8, r.G - gq0);        // live columns

    uint8_t* warp_smem = group_smem + warp * warp_bytes;

    // one warp per (kv head, column); lane holds 4 consecutive elements
    const float c = inv_sqrt_dim(p.head_dim);
    const float alpha_k = PROD ? TQ_ALPHA3 : TQ_ALPHA4;
    // QJL: +-1 operands (no table scale), logits <q', k'> without 1/sqrt(D) (tq_qjl_kernels.cu:335),
    // rotation sign without a head term (:18-21)
    const float qscale = QJL ? c * kLog2e : ((MODE == 0) ? c * c * kLog2e : c * c) / alpha_k;
    for (int col = stream; col < 8; col += p.streams) {
        float x[4] = {0.f, 0.f, 0.f, 0.f};
        if (col < nq) {
            const int gq = gq0 + col;
            const long long qrow = static_cast<long long>(r.b) * r.rows_per_seq +
                                   (p.ref_layout ? gq * H + h : h * r.G + gq);
            const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p.query + qrow * kHeadDim) + lane);
            const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
            const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
            // even-head sign pattern (+,-,+,-); odd heads negate the result
            float a0 = f0.x - f0.y, a1 = f0.x + f0.y, a2 = f1.x - f1.y, a3 = f1.x + f1.y;
            x[0] = a0 + a2; x[2] = a0 - a2; x[1] = a1 + a3; x[3] = a1 - a3;
#pragma unroll
            for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float o = __shfl_xor_sync(0xffffffffu, x[e], m);
                    x[e] = (lane & m) ? o - x[e] : x[e] + o;
                }
            }
            const float sc = (!QJL && (h & 1)) ? -qscale : qscale;
#pragma unroll
            for (int e = 0; e < 4; ++e) x[e] *= sc;
        }
        __half2* dst = reinterpret_cast<__half2*>(qsm + (hl * 8 + col) * kHeadDim + 4 * lane);
        const __half2 hi0 = __floats2half2_rn(x[0], x[1]), hi1 = __floats2half2_rn(x[2], x[3]);
        dst[0] = hi0;
        dst[1] = hi1;
        if (QJL) {
            // the fp16 rounding of q' that the other schemes tolerate is 11 times larger against
            // unscaled logits: keep the remainder as a second fp16 fragment set (q' = hi + lo)
            const float2 h0 = __half22float2(hi0), h1 = __half22float2(hi1);
            __half2* dlo = dst + (Hl * 8 * kHeadDim) / 2;
            dlo[0] = __floats2half2_rn(x[0] - h0.x, x[1] - h0.y);
            dlo[1] = __floats2half2_rn(x[2] - h1.x, x[3] - h1.y);
        }
    }
    group_sync(bar_id, bar_threads);

    {
        const __half* qrow = qsm + (hl * 8 + g) * kHeadDim + 32 * tig;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            if (LUT) {
                // B fragments: column g, dims 32*tig + 4*s + {0,1 | 2,3}
                const uint2 q4 = *reinterpret_cast<const uint2*>(qrow + 4 * s);
                ctx.qf[s][0] = q4.x;
                ctx.qf[s][1] = q4.y;
            } else {
                // B fragments: column g, dims 32*tig + 8*wi + {2hf, 2hf+4 | 2hf+1, 2hf+5}
                const int base = 8 * (s >> 1) + 2 * (s & 1);
                const __half2 b01 = __halves2half2(qrow[base], qrow[base + 4]);
                const __half2 b23 = __halves2half2(qrow[base + 1], qrow[base + 5]);
                ctx.qf[s][0] = *reinterpret_cast<const uint32_t*>(&b01);
                ctx.qf[s][1] = *reinterpret_cast<const uint32_t*>(&b23);
                if (QJL) {
                    const __half* qlo = qrow + Hl * 8 * kHeadDim;
                    const __half2 l01 = __halves2half2(qlo[base], qlo[base + 4]);
                    const __half2 l23 = __halves2half2(qlo[base + 1], qlo[base + 5]);
                    ctx.qlo[s][0] = *reinterpret_cast<const uint32_t*>(&l01);
                    ctx.qlo[s][1] = *reinterpret_cast<const uint32_t*>(&l23);
                }
            }
        }
    }
    ctx.qsign = nullptr;
    if (qsign_group) {
        // fragments in the (d, d+4) pairing for the residual-sign MMAs: word wi of the lane's 32 dims
        // -> (q[0],q[4]) (q[1],q[5]) | (q[2],q[6]) (q[3],q[7]); written once per kv head
        const __half* qrow = qsm + (hl * 8 + g) * kHeadDim + 32 * tig;
        if (stream == 0) {
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
                const __half* q8 = qrow + 8 * wi;
                const __half2 f0 = __halves2half2(q8[0], q8[4]), f1 = __halves2half2(q8[1], q8[5]);
                const __half2 f2 = __halves2half2(q8[2], q8[6]), f3 = __halves2half2(q8[3], q8[7]);
                qsign_group[(hl * 4 + wi) * 32 + lane] =
                    make_uint4(*reinterpret_cast<const uint32_t*>(&f0), *reinterpret_cast<const uint32_t*>(&f1),
                               *reinterpret_cast<const uint32_t*>(&f2), *reinterpret_cast<const uint32_t*>(&f3));
            }
        }
        ctx.qsign = qsign_group + hl * 4 * 32;
    }
    // fp16(alpha * level) split into high-byte and low-byte pools, entries 0-3 | 4-7
    // (tests/test_abi.py recomputes them from the level tables)
    ctx.pool3 = BytePools{TQ_POOL3_HI_A, TQ_POOL3_HI_B, TQ_POOL3_LO_A, TQ_POOL3_LO_B};
    ctx.mag4 = BytePools{TQ_MAG4_HI_A, TQ_MAG4_HI_B, TQ_MAG4_LO_A, TQ_MAG4_LO_B};
    ctx.inv_alpha_v = 1.0f / TQ_ALPHA4;
    ctx.warp_smem = warp_smem;
    ctx.warp_smem_addr = static_cast<uint32_t>(__cvta_generic_to_shared(warp_smem));
    ctx.lut = nullptr;
    ctx.lane_k = static_cast<uint32_t>(lane) * 4u;
    ctx.lane_v = 128u + static_cast<uint32_t>(lane) * 4u;
    ctx.group_smem = group_smem;
    ctx.bar_id = bar_id;
    ctx.bar_threads = bar_threads;
    ctx.lane = lane;
    ctx.g = g;
    ctx.tig = tig;
    ctx.h = h;
    ctx.H = H;
    ctx.hl = hl;
    ctx.Hl = Hl;
    ctx.nq = nq;
    ctx.gq0 = gq0;

    const int n = p.seq_lens ? min(__ldg(p.seq_lens + r.b), p.max_kv_tokens) : p.max_kv_tokens;
    r.t_begin = max(p.kv_begin, 0);
    r.t_end = min(n, p.kv_end);
    const int nblk = r.t_end > r.t_begin ? (r.t_end - r.t_begin + 15) >> 4 : 0;
    const int per = (nblk + p.splits - 1) / p.splits;
    r.blk_lo = r.split * per;
    r.blk_hi = min(nblk, r.blk_lo + per);
}

__device__ __forceinline__ void init_state(WarpState& st) {
#pragma unroll
    for (int j = 0; j < 8; ++j) st.o[j][0] = st.o[j][1] = st.o[j][2] = st.o[j][3] = 0.0f;
    st.m_run[0] = st.m_run[1] = kInitMaxLogit;
    st.l_run[0] = st.l_run[1] = 0.0f;
}

// Epilogue: combine the streams of a kv head through shared memory (the per-warp regions
// are dead by now and are reused as records), then write the split partial.
__device__ __forceinline__ void decode_epilogue(const DecodeParams& p, int warp_bytes,
                                                const BlockCtx& c, const CtaRange& r,
                                                WarpState& st) {
    uint8_t* smem_raw = c.group_smem;
    const int lane = c.lane, g = c.g, tig = c.tig, h = c.h, H = c.H;
    float (&o)[8][4] = st.o;
    float (&m_run)[2] = st.m_run;
    float (&l_run)[2] = st.l_run;
#pragma unroll
    for (int msk = 4; msk < 32; msk <<= 1) {
        l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], msk);
        l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], msk);
    }
    group_sync(c.bar_id, c.bar_threads);
    float* rec = reinterpret_cast<float*>(c.warp_smem);
    if (r.stream > 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) rec[(4 * j + e) * 32 + lane] = o[j][e];
        rec[32 * 32 + lane] = m_run[0];
        rec[33 * 32 + lane] = m_run[1];
        rec[34 * 32 + lane] = l_run[0];
        rec[35 * 32 + lane] = l_run[1];
    }
    group_sync(c.bar_id, c.bar_threads);
    if (r.stream > 0) return;
    for (int s = 1; s < p.streams; ++s) {
        const float* q = reinterpret_cast<const float*>(smem_raw + (s * c.Hl + c.hl) * warp_bytes);
        const float ms0 = q[32 * 32 + lane], ms1 = q[33 * 32 + lane];
        const float mn0 = fmaxf(m_run[0], ms0), mn1 = fmaxf(m_run[1], ms1);
        const float a0 = ex2(m_run[0] - mn0), a1 = ex2(m_run[1] - mn1);
        const float b0 = ex2(ms0 - mn0), b1 = ex2(ms1 - mn1);
        l_run[0] = l_run[0] * a0 + q[34 * 32 + lane] * b0;
        l_run[1] = l_run[1] * a1 + q[35 * 32 + lane] * b1;
        m_run[0] = mn0;
        m_run[1] = mn1;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            o[j][0] = o[j][0] * a0 + q[(4 * j + 0) * 32 + lane] * b0;
            o[j][1] = o[j][1] * a1 + q[(4 * j + 1) * 32 + lane] * b1;
            o[j][2] = o[j][2] * a0 + q[(4 * j + 2) * 32 + lane] * b0;
            o[j][3] = o[j][3] * a1 + q[(4 * j + 3) * 32 + lane] * b1;
        }
    }
    // partial record: acc[128] (natural dim order), m in natural-log units, l
    float* out = p.partials + (static_cast<long long>(r.b) * p.splits + r.split) * r.rows_per_seq *
                                  TQ_PARTIAL_STRIDE;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int col = 2 * tig + e;
        if (col >= c.nq) continue;
        float* row = out + static_cast<long long>(h * r.G + c.gq0 + col) * TQ_PARTIAL_STRIDE;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            // accumulator rows g and g+8 of tile j are dims 16g + 2j and 16g + 2j + 1
            row[16 * g + 2 * j] = o[j][e];
            row[16 * g + 2 * j + 1] = o[j][2 + e];
        }
        if (g == 0) {
            row[128] = m_run[e] * kLn2;
            row[129] = l_run[e];
        }
    }
}

// General kernel: any slot mapping / block size / alignment; one block of register prefetch.
// MODE 0: attention partials, MODE 1: logits only (turbo_prod).
template <bool PROD, int MODE, bool QJL = false>
__global__ void __launch_bounds__(256, 2)
decode_kernel(DecodeParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    BlockCtx ctx;
    CtaRange r;
    decode_prologue<PROD, MODE, false, QJL>(p, smem_raw, kWarpSmemBytes,
                                reinterpret_cast<__half*>(smem_raw + (blockDim.x >> 5) * kWarpSmemBytes),
                                threadIdx.x >> 5, blockIdx.y, blockIdx.x, 0, 0, ctx, r);
    WarpState st;
    init_state(st);
    const bool aligned = p.aligned16 != 0;

    BlockRaw cur;
    int blk = r.blk_lo + r.stream;
    if (blk < r.blk_hi)
        load_block<PROD, QJL>(p, r.b, ctx.h, r.t_begin + 16 * blk, r.t_end, ctx.lane, aligned, cur);
    for (; blk < r.blk_hi; blk += p.streams) {
        const int tb = r.t_begin + 16 * blk;
        BlockRaw nxt = cur;
        if (blk + p.streams < r.blk_hi)
            load_block<PROD, QJL>(p, r.b, ctx.h, r.t_begin + 16 * (blk + p.streams), r.t_end, ctx.lane,
                             aligned, nxt);
        process_block<PROD, MODE, false, QJL>(p, ctx, cur, tb, r.t_end, st);
        cur = nxt;
    }
    if (MODE == 1) return;
    decode_epilogue(p, kWarpSmemBytes, ctx, r, st);
}

// ---- paged fast path ----------------------------------------------------------------
// Block tables with 16-token pages, 16-byte aligned pool, H in {1,2,4,8}: a 16-token block IS
// a page, so every lane's source offsets inside the page are loop constants (and, with H a
// template argument, the distances between a lane's rows are immediates).  Code bytes and
// scales travel global -> shared with cp.async (no registers held while in flight) into a
// per-warp ring of kStages stages; cp.async.wait_group paces the consumer.
constexpr int kStages = 3;
constexpr int kStageCodeBytes = 2 * 32 * 16 + 2 * 32 * 16;  // K and V: two 16-byte pieces per lane each
constexpr int kStageScaleBytes = 3 * 256;                   // three regions of 16*H fp16, H <= 8
constexpr int kStageBytes = kStageCodeBytes + kStageScaleBytes;
constexpr int kFastWarpBytes = kStages * kStageBytes;       // 8448 >= kWarpSmemBytes (merge record)
static_assert(kFastWarpBytes >= kWarpSmemBytes, "the merge record reuses the ring");

__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
// The same with immediate byte offsets on both addresses.
template <int DST_OFF, int SRC_OFF>
__device__ __forceinline__ void cp_async16_at(uint32_t dst_smem, unsigned long long src) {
    asm volatile("cp.async.cg.shared.global [%0 + %2], [%1 + %3], 16;" ::"r"(dst_smem), "l"(src), "n"(DST_OFF),
                 "n"(SRC_OFF) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// One CTA per SM, 16 warps = two groups of 8; each group works on its own (sequence, split)
// exactly like an 8-warp CTA would, the two share the operand tables.
constexpr int kFastGroupWarps = 8;
constexpr int kFastGroups = 2;
constexpr int kFastGroupBytes = kFastGroupWarps * kFastWarpBytes;
constexpr int kFastSmemBytes = kLutBytes + kFastGroups * kFastGroupBytes;
// turbo_prod, up to 4 kv heads: the residual-sign query fragments of each group (2 KB per head) sit
// behind the rings; with 8 heads they would not fit and the table pairing serves the signs too
constexpr int kSignFragBytesPerHead = 4 * 32 * 16;
__host__ __device__ constexpr bool sign_frags(bool prod, int heads) { return prod && heads <= 4; }
__host__ __device__ constexpr int fast_smem_bytes(bool prod, int heads) {
    return kFastSmemBytes + (sign_frags(prod, heads) ? kFastGroups * heads * kSignFragBytesPerHead : 0);
}
static_assert(kFastGroupBytes >= kMaxHeads * 8 * kHeadDim * 2, "the query scratch reuses the ring");

template <bool PROD, int H>
__global__ void __launch_bounds__(kFastGroups * kFastGroupWarps * 32, 1)
decode_paged16_kernel(DecodeParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr int kStreams = kFastGroupWarps / H;
    pdl_launch_dependents();
    build_operand_lut(smem_raw);  // constants only: may run before the previous kernel is done
    __syncthreads();
    pdl_wait();
    // work items (sequence, split) are numbered sequence-major; a CTA takes two neighbours
    const int group = threadIdx.x / (kFastGroupWarps * 32);
    const int item = blockIdx.x * kFastGroups + group;
    if (item >= p.batch * p.splits) return;  // odd item count: the last CTA runs one group
    const int seq = item / p.splits, split = item - seq * p.splits;
    uint8_t* group_smem = smem_raw + kLutBytes + group * kFastGroupBytes;
    const int bar_id = 1 + group, bar_threads = kFastGroupWarps * 32;
    BlockCtx ctx;
    CtaRange r;
    constexpr bool kSignQ = sign_frags(PROD, H);
    uint4* qsign_group = kSignQ ? reinterpret_cast<uint4*>(smem_raw + kFastSmemBytes +
                                                           group * H * kSignFragBytesPerHead)
                                : nullptr;
    decode_prologue<PROD, 0, true>(p, group_smem, kFastWarpBytes, reinterpret_cast<__half*>(group_smem),
                                   (threadIdx.x >> 5) % kFastGroupWarps, seq, split, bar_id,
                                   bar_threads, ctx, r, qsign_group);
    ctx.lut = smem_raw;
    group_sync(bar_id, bar_threads);  // the query scratch is dead: the ring may be filled
    WarpState st;
    init_state(st);
    const int lane = ctx.lane, g = ctx.g, tig = ctx.tig, h = ctx.h;

    uint8_t* ring = ctx.warp_smem;
    const uint32_t ring_addr = ctx.warp_smem_addr;
    // loop-constant source offsets inside a page
    const uint32_t k_off = p.geo.k_codes + ((g * H + h) << 6) + (tig << 4);          // row g; row g+8: +512H
    // V travels in 16-byte pieces (token t, chunk c of 4): an 8-byte copy costs the load/store
    // unit as many wavefronts as a 16-byte one.  Piece (t, c) lands where the later 8-byte
    // fragment reads (lane (g, tig): chunk g/2, half g%2 of tokens 2tig + {0, 1, 8, 9}) are
    // conflict-free: the four tokens of one read instruction differ in (t >> 1) & 3.
    auto v_piece = [](int t, int c) {
        return 1024 + 128 * ((t & 1) + 2 * (t >> 3) + 4 * (c >> 1)) + 32 * ((t >> 1) & 3) + 16 * (c & 1);
    };
    // the lane's two V pieces are tokens t and t + 8 of chunk c: 512*H bytes apart in the page, 256 in the stage
    uint32_t v_rd[4];
    const uint32_t v_off = p.geo.v_codes + (((lane >> 2) * H + h) << 6) + ((lane & 3) << 4);
    const uint32_t v_dst = v_piece(lane >> 2, lane & 3);
#pragma unroll
    for (int j = 0; j < 4; ++j)
        v_rd[j] = v_piece(2 * tig + (j & 1) + 8 * (j >> 1), g >> 1) + 8 * (g & 1);
    // scale regions (16*H fp16 each) are copied in 16-byte pieces spread over the lanes
    constexpr int kPiecesPerRegion = 2 * H;
    constexpr int kRegions = PROD ? 3 : 2;
    uint32_t sc_src[2], sc_dst[2];
    bool sc_on[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int i = lane + 32 * k;
        const int reg = i / kPiecesPerRegion, j = i - reg * kPiecesPerRegion;
        sc_on[k] = reg < kRegions;
        const uint32_t base = reg == 0 ? p.geo.k_scales : (reg == 1 ? p.geo.v_scales : p.geo.k_res);
        sc_src[k] = base + 16 * j;
        sc_dst[k] = kStageCodeBytes + reg * 256 + 16 * j;
    }
    const uint32_t s_idx = 2 * (g * H + h);  // this lane's row-g scale inside a region; row g+8: +16H

    const int32_t* table = p.block_tables + static_cast<long long>(r.b) * p.table_stride +
                           (r.t_begin >> 4) + r.blk_lo + r.stream;
    const int n_iter = r.blk_hi > r.blk_lo + r.stream
                           ? (r.blk_hi - r.blk_lo - r.stream + kStreams - 1) / kStreams : 0;

    // page ids of 32 consecutive iterations, one per lane
    int ids = 0, ids_base = 0;
    auto refill = [&](int it0) {
        const int it = it0 + lane;
        ids = it < n_iter ? __ldg(table + it * kStreams) : 0;
        ids_base = it0;
    };
    // Address arithmetic of a fill, spelled out: one wide multiply-add gives the page's address, one
    // more per distinct in-page offset adds the lane's 32-bit offset, the second piece of a pair is an
    // immediate offset of the copy instruction (written as generic 64-bit pointer arithmetic the fill
    // of one block cost ~90 instructions).
    const uint32_t page_size32 = static_cast<uint32_t>(p.geo.page_size);
    const unsigned long long pool64 = reinterpret_cast<unsigned long long>(p.pool);
    const uint32_t lane16 = lane * 16;
    auto issue = [&](int it, uint32_t dst) {
        if (it < n_iter) {
            if (it - ids_base >= 32) refill(it);
            const uint32_t page = static_cast<uint32_t>(__shfl_sync(0xffffffffu, ids, it - ids_base));
            const unsigned long long src = mad_wide(page, page_size32, pool64);
            const unsigned long long ks = mad_wide(k_off, 1u, src);
            cp_async16_at<0, 0>(dst + lane16, ks);
            cp_async16_at<512, 512 * H>(dst + lane16, ks);
            const unsigned long long vs = mad_wide(v_off, 1u, src);
            cp_async16_at<0, 0>(dst + v_dst, vs);
            cp_async16_at<256, 512 * H>(dst + v_dst, vs);
            if (sc_on[0]) cp_async16_at<0, 0>(dst + sc_dst[0], mad_wide(sc_src[0], 1u, src));
            if (kRegions * kPiecesPerRegion > 32 && sc_on[1])
                cp_async16_at<0, 0>(dst + sc_dst[1], mad_wide(sc_src[1], 1u, src));
        }
        cp_async_commit();  // one group per iteration, empty or not, keeps the count uniform
    };

    refill(0);
#pragma unroll
    for (int s = 0; s < kStages - 1; ++s) issue(s, ring_addr + s * kStageBytes);

    int stage = 0;  // stage holding the iteration in hand
    int tb = r.t_begin + 16 * (r.blk_lo + r.stream);
    // One ring step and one block.  `ragged` is a compile-time tag: only the last block of the token
    // range can end inside its 16 tokens, so the loop proper runs without the masking code and that
    // block, if this warp owns it, runs once through a second copy.
    auto step = [&](int it, auto ragged) {
        constexpr bool kRagged = decltype(ragged)::value;
        const int fill = stage == 0 ? kStages - 1 : stage - 1;  // (it + kStages - 1) % kStages
        // Two orders of the same ring step.  turbo_mse pages (less arithmetic per byte) want the
        // refill in flight before the warp waits for block `it`.  turbo_prod pages are served
        // better by waiting first: the barrier that publishes block `it` is then also behind every
        // lane's reads of block it-1, so that block's stage is refilled right after it and the
        // second barrier of the iteration goes away (measured: +0.9 % on turbo_prod pages, -15 %
        // on turbo_mse pages, hence the switch).
        constexpr bool kRefillAfterWait = PROD;
        if constexpr (!kRefillAfterWait) issue(it + kStages - 1, ring_addr + fill * kStageBytes);
        cp_async_wait<kRefillAfterWait ? kStages - 2 : kStages - 1>();
        __syncwarp();  // pieces are copied by other lanes
        if constexpr (kRefillAfterWait) issue(it + kStages - 1, ring_addr + fill * kStageBytes);
        const uint8_t* stg = ring + stage * kStageBytes;
        BlockRaw cur;
        cur.k0 = *reinterpret_cast<const uint4*>(stg + lane * 16);
        cur.k1 = *reinterpret_cast<const uint4*>(stg + 512 + lane * 16);
#pragma unroll
        for (int i = 0; i < 4; ++i)
            cur.v[i] = *reinterpret_cast<const uint2*>(stg + v_rd[i]);
        const uint8_t* sc = stg + kStageCodeBytes + s_idx;
        auto ld = [&](uint32_t off) {
            return __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(sc + off)));
        };
        cur.ks0 = ld(0);
        cur.ks1 = ld(16 * H);
        cur.vs0 = ld(256);
        cur.vs1 = ld(256 + 16 * H);
        cur.re0 = PROD ? ld(512) : 0.0f;
        cur.re1 = PROD ? ld(512 + 16 * H) : 0.0f;
        if (kRagged && tb + 16 > r.t_end) {
            // rows past the end of the sequence may hold anything: zero their scales so that
            // P * vs stays finite (their logits are masked to -inf in process_block)
            if (tb + g >= r.t_end) cur.ks0 = cur.vs0 = cur.re0 = 0.0f;
            if (tb + g + 8 >= r.t_end) cur.ks1 = cur.vs1 = cur.re1 = 0.0f;
        }
        process_block<PROD, 0, true, false, kSignQ, kRagged>(p, ctx, cur, tb, r.t_end, st);
        if constexpr (!kRefillAfterWait) __syncwarp();  // every lane is done reading this stage before it is refilled
        stage = stage == kStages - 1 ? 0 : stage + 1;
        tb += 16 * kStreams;
    };
    // (turbo_mse pages: the single loop with the run-time check measured 3635 GB/s against 3215 with
    // the second copy, turbo_prod pages 3228 against 3330 -- hence per scheme.)
    constexpr bool kPeelRagged = PROD;
    if constexpr (kPeelRagged) {
        const bool last_ragged = n_iter > 0 && tb + 16 * kStreams * (n_iter - 1) + 16 > r.t_end;
        const int n_full = last_ragged ? n_iter - 1 : n_iter;
        for (int it = 0; it < n_full; ++it) step(it, std::false_type{});
        if (last_ragged) step(n_full, std::true_type{});
    } else {
        for (int it = 0; it < n_iter; ++it) step(it, std::true_type{});
    }
    cp_async_wait<0>();
    decode_epilogue(p, kFastWarpBytes, ctx, r, st);
}

// WPR warps merge the parts of one (sequence, query head) row; lane holds dims 4*lane..4*lane+3.
// With WPR == 1 a warp walks all parts itself (many rows, few parts: the serving shape).  With
// WPR > 1 the CTA owns one row, warp `sub` takes parts sub, sub + WPR, .. and the warps' maxima
// and weighted sums meet in `xchg` (WPR * kMergeXchgFloats floats of shared memory) -- one long
// sequence split hundreds of ways would otherwise be a serial walk of hundreds of records.
constexpr int kMergeXchgFloats = 132;
template <int WPR>
__device__ __forceinline__ void merge_row(const float* __restrict__ partials, int num_parts,
                                          long long part_stride, long long seq_stride, int rows_per_seq,
                                          __half* __restrict__ output, float* __restrict__ partials_out,
                                          int row, int num_q_heads, int num_kv_heads, int ref_layout,
                                          int head_dim, int lane, const PeerOut* peer, int head_sign = 1,
                                          int sub = 0, float* xchg = nullptr) {
    const int seq = row / rows_per_seq, r = row - seq * rows_per_seq;
    const float* base = partials + seq * seq_stride + static_cast<long long>(r) * TQ_PARTIAL_STRIDE;
    float mmax = kInitMaxLogit;
    for (int s = sub; s < num_parts; s += WPR) mmax = fmaxf(mmax, __ldg(base + s * part_stride + 128));
    if (WPR > 1) {
        if (lane == 0) xchg[sub] = mmax;
        __syncthreads();
#pragma unroll
        for (int w = 0; w < WPR; ++w) mmax = fmaxf(mmax, xchg[w]);
        __syncthreads();  // the maxima are read before the sums overwrite them
    }
    float acc[4] = {0.f, 0.f, 0.f, 0.f}, l = 0.f;
#pragma unroll 4
    for (int s = sub; s < num_parts; s += WPR) {
        const float* ps = base + s * part_stride;
        const float w = __expf(__ldg(ps + 128) - mmax);
        l = fmaf(__ldg(ps + 129), w, l);
        const float2 v0 = __ldg(reinterpret_cast<const float2*>(ps + 4 * lane));
        const float2 v1 = __ldg(reinterpret_cast<const float2*>(ps + 4 * lane + 2));
        acc[0] = fmaf(v0.x, w, acc[0]);
        acc[1] = fmaf(v0.y, w, acc[1]);
        acc[2] = fmaf(v1.x, w, acc[2]);
        acc[3] = fmaf(v1.y, w, acc[3]);
    }
    if (WPR > 1) {
        float* mine = xchg + sub * kMergeXchgFloats;
        *reinterpret_cast<float4*>(mine + 4 * lane) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        if (lane == 0) mine[128] = l;
        __syncthreads();
        if (sub != 0) return;  // warp 0 adds the warps' sums in a fixed order and finishes the row
        l = xchg[128];
#pragma unroll
        for (int w = 1; w < WPR; ++w) {
            const float4 o = *reinterpret_cast<const float4*>(xchg + w * kMergeXchgFloats + 4 * lane);
            acc[0] += o.x;
            acc[1] += o.y;
            acc[2] += o.z;
            acc[3] += o.w;
            l += xchg[w * kMergeXchgFloats + 128];
        }
    }
    if (partials_out) {
        float* po = partials_out + static_cast<long long>(row) * TQ_PARTIAL_STRIDE;
#pragma unroll
        for (int e = 0; e < 4; ++e) po[4 * lane + e] = acc[e];
        if (lane == 0) {
            po[128] = mmax;
            po[129] = l;
        }
    }
    if (peer) {
        const long long at = ((static_cast<long long>(peer->exchange & 1u) * peer->world + peer->rank) *
                                  peer->rows_cap + row) * TQ_PARTIAL_STRIDE;
        for (int q = 0; q < peer->world; ++q) {
            float* po = peer->records[q] + at;
            *reinterpret_cast<float2*>(po + 4 * lane) = make_float2(acc[0], acc[1]);
            *reinterpret_cast<float2*>(po + 4 * lane + 2) = make_float2(acc[2], acc[3]);
            if (lane == 0) *reinterpret_cast<float2*>(po + 128) = make_float2(mmax, l);
        }
    }
    if (!output) return;
    const int G = num_q_heads / num_kv_heads;
    const int h = r / G, gq = r - h * G;
    const float inv_l = l > 0.0f ? 1.0f / l : 1.0f;  // tq_turbo_prod_kernels.cu:561-564
    float x[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) x[e] = acc[e] * inv_l;
    // inverse rotation: FWHT, * rsqrt(D), * s(i, h)   (tq_turbo_prod_kernels.cu:566-570)
    float a0 = x[0] + x[1], a1 = x[0] - x[1], a2 = x[2] + x[3], a3 = x[2] - x[3];
    x[0] = a0 + a2; x[2] = a0 - a2; x[1] = a1 + a3; x[3] = a1 - a3;
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float ov = __shfl_xor_sync(0xffffffffu, x[e], m);
            x[e] = (lane & m) ? ov - x[e] : x[e] + ov;
        }
    }
    const float c = inv_sqrt_dim(head_dim);
    const float s0 = (head_sign && (h & 1)) ? -c : c;  // element 4*lane+e: sign + iff (e+h) even (QJL: e even)
    const long long orow = static_cast<long long>(seq) * rows_per_seq +
                           (ref_layout ? gq * num_kv_heads + h : r);
    __half2* dst = reinterpret_cast<__half2*>(output + orow * kHeadDim + 4 * lane);
    dst[0] = __floats2half2_rn(x[0] * s0, x[1] * -s0);
    dst[1] = __floats2half2_rn(x[2] * s0, x[3] * -s0);
}

// ---- merge: log-sum-exp over parts, normalise, inverse rotation, fp16 store ----
// One warp per (sequence, query head) row; lane holds dims 4*lane..4*lane+3.
template <int WPR>
__global__ void __launch_bounds__(WPR == 1 ? 128 : WPR * 32)
merge_kernel(const float* __restrict__ partials, int num_parts, long long part_stride,
             long long seq_stride, int rows_per_seq, __half* __restrict__ output,
             float* __restrict__ partials_out, int rows, int num_q_heads, int num_kv_heads,
             int ref_layout, int head_dim, PeerOut peer, int head_sign) {
    __shared__ __align__(16) float xchg[WPR == 1 ? 4 : WPR * kMergeXchgFloats];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    // WPR == 1: four rows per CTA, a warp each; otherwise the CTA's warps share one row
    const int row = WPR == 1 ? blockIdx.x * (blockDim.x >> 5) + warp : blockIdx.x;
    const int sub = WPR == 1 ? 0 : warp;
    pdl_launch_dependents();
    pdl_wait();
    if (peer.world > 0) {
        // Publishing variant: the row's merged record goes straight into slot `rank` of every
        // peer's buffer; the last CTA to finish raises this rank's flag on every peer.
        if (row < rows) merge_row<WPR>(partials, num_parts, part_stride, seq_stride, rows_per_seq, nullptr, nullptr,
                                       row, num_q_heads, num_kv_heads, ref_layout, head_dim, lane, &peer, 1, sub, xchg);
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0) {
            const unsigned int done = atomicAdd(peer.ticket, 1u);
            if (done == gridDim.x - 1) {
                *peer.ticket = 0u;
                __threadfence_system();
                for (int q = 0; q < peer.world; ++q)
                    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peer.flags[q] + (peer.exchange & 1u) * peer.world + peer.rank),
                                 "r"(peer.exchange) : "memory");
            }
        }
        if (!peer.final_out) return;
        // Finish the exchange here: wait (bounded) until every rank's records of this exchange have
        // landed in this rank's own buffer, then merge them for this CTA's rows.  The host only asks for
        // this when the whole grid is resident at once (the own flag is raised by the last CTA).
        if (threadIdx.x == 0) {
            const unsigned int* mine = peer.flags[peer.rank] + (peer.exchange & 1u) * peer.world;
            unsigned long long t0;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
            bool bad = false;
            for (int q = 0; q < peer.world && !bad; ++q) {
                while (true) {
                    unsigned int v;
                    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine + q) : "memory");
                    if (v == peer.exchange) break;
                    unsigned long long t1;
                    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
                    if (t1 - t0 > peer.wait_ns) {
                        bad = true;
                        break;
                    }
                    __nanosleep(100);
                }
            }
            if (bad) atomicMax(peer.status, 1);
        }
        __syncthreads();
        if (row >= rows || sub != 0) return;
        {
            // the arithmetic of the stand-alone peer merge: records read through L2 (peer stores do not
            // pass this GPU's L1), ranks in order
            const long long part_stride_w = static_cast<long long>(peer.rows_cap) * TQ_PARTIAL_STRIDE;
            const float* base = peer.records[peer.rank] +
                                static_cast<long long>(peer.exchange & 1u) * peer.world * part_stride_w +
                                static_cast<long long>(row) * TQ_PARTIAL_STRIDE;
            float mmax = kInitMaxLogit;
            for (int s = 0; s < peer.world; ++s) mmax = fmaxf(mmax, __ldcg(base + s * part_stride_w + 128));
            float acc[4] = {0.f, 0.f, 0.f, 0.f}, l = 0.f;
            for (int s = 0; s < peer.world; ++s) {
                const float* ps = base + s * part_stride_w;
                const float w = __expf(__ldcg(ps + 128) - mmax);
                l = fmaf(__ldcg(ps + 129), w, l);
                const float2 v0 = __ldcg(reinterpret_cast<const float2*>(ps + 4 * lane));
                const float2 v1 = __ldcg(reinterpret_cast<const float2*>(ps + 4 * lane + 2));
                acc[0] = fmaf(v0.x, w, acc[0]);
                acc[1] = fmaf(v0.y, w, acc[1]);
                acc[2] = fmaf(v1.x, w, acc[2]);
                acc[3] = fmaf(v1.y, w, acc[3]);
            }
            const int G = num_q_heads / num_kv_heads;
            const int h = (row % rows_per_seq) / G;
            const float inv_l = l > 0.0f ? 1.0f / l : 1.0f;  // tq_turbo_prod_kernels.cu:561-564
            float x[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) x[e] = acc[e] * inv_l;
            const float a0 = x[0] + x[1], a1 = x[0] - x[1], a2 = x[2] + x[3], a3 = x[2] - x[3];
            x[0] = a0 + a2; x[2] = a0 - a2; x[1] = a1 + a3; x[3] = a1 - a3;
#pragma unroll
            for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float ov = __shfl_xor_sync(0xffffffffu, x[e], m);
                    x[e] = (lane & m) ? ov - x[e] : x[e] + ov;
                }
            }
            const float c = inv_sqrt_dim(head_dim);
            const float s0 = (h & 1) ? -c : c;
            __half2* dst = reinterpret_cast<__half2*>(static_cast<__half*>(peer.final_out) +
                                                      static_cast<long long>(row) * kHeadDim + 4 * lane);
            dst[0] = __floats2half2_rn(x[0] * s0, x[1] * -s0);
            dst[1] = __floats2half2_rn(x[2] * s0, x[3] * -s0);
        }
        return;
    }
    if (row >= rows) return;
    merge_row<WPR>(partials, num_parts, part_stride, seq_stride, rows_per_seq, output, partials_out, row,
                   num_q_heads, num_kv_heads, ref_layout, head_dim, lane, nullptr, head_sign, sub, xchg);
}

// Rows with many parts get a CTA of eight warps each, the others a warp each.
constexpr int kMergeWideParts = 16, kMergeWideWarps = 8;
template <bool PDL, typename... Args>
void launch_merge_kernel(int rows, int num_parts, cudaStream_t stream, Args... args) {
    const bool wide = num_parts >= kMergeWideParts;
    const dim3 grid(wide ? rows : (rows + 3) / 4), block(wide ? kMergeWideWarps * 32 : 128);
    if (PDL) {
        if (wide) launch_after_wait(merge_kernel<kMergeWideWarps>, grid, block, 0, stream, args...);
        else launch_after_wait(merge_kernel<1>, grid, block, 0, stream, args...);
    } else {
        if (wide) merge_kernel<kMergeWideWarps><<<grid, block, 0, stream>>>(args...);
        else merge_kernel<1><<<grid, block, 0, stream>>>(args...);
    }
}

// Dynamic shared memory above 48 KB has to be opted into once per device.
void set_smem_attr_once() {
    static bool done[64] = {};
    int dev = 0;
    check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (dev < 0 || dev >= 64 || done[dev]) return;
    const int bytes = 65536;
    check_cuda(cudaFuncSetAttribute(decode_kernel<true, 0>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, bytes), "smem attr");
    check_cuda(cudaFuncSetAttribute(decode_kernel<false, 0>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, bytes), "smem attr");
    check_cuda(cudaFuncSetAttribute(decode_kernel<true, 1>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, bytes), "smem attr");
    check_cuda(cudaFuncSetAttribute(decode_kernel<false, 0, true>,  // two query scratches: 8 heads need 68 KB
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, 73728), "smem attr");
#define TQ_FAST_ATTR(PRODV, HV)                                                               \
    check_cuda(cudaFuncSetAttribute(decode_paged16_kernel<PRODV, HV>,                         \
                                    cudaFuncAttributeMaxDynamicSharedMemorySize,              \
                                    fast_smem_bytes(PRODV, HV)),                              \
               "smem attr")
    TQ_FAST_ATTR(true, 1); TQ_FAST_ATTR(true, 2); TQ_FAST_ATTR(true, 4); TQ_FAST_ATTR(true, 8);
    TQ_FAST_ATTR(false, 1); TQ_FAST_ATTR(false, 2); TQ_FAST_ATTR(false, 4); TQ_FAST_ATTR(false, 8);
#undef TQ_FAST_ATTR
    done[dev] = true;
}

}  // namespace

int decode_num_splits(int batch, int max_kv_tokens, int num_kv_heads, int block_size) {
    (void)block_size;
    if (batch <= 0 || max_kv_tokens <= 0) return 1;
    const int streams = (num_kv_heads <= 8 && 8 % num_kv_heads == 0) ? 8 / num_kv_heads : 1;
    const int slots = 2 * sm_count();
    int splits = slots / batch;
    const int nblk = (max_kv_tokens + 15) / 16;
    const int cap = nblk / (streams * 4);
    if (splits > cap) splits = cap;
    if (splits < 1) splits = 1;
    return splits;
}

size_t decode_workspace_bytes(int batch, int num_q_heads, int num_splits) {
    return static_cast<size_t>(batch) * num_splits * num_q_heads * TQ_PARTIAL_STRIDE * sizeof(float);
}

void launch_merge(const float* partials, int num_parts, void* output, float* partials_out,
                  int rows, int num_q_heads, int num_kv_heads, int ref_query_layout,
                  int head_dim, cudaStream_t stream, int head_sign) {
    if (rows <= 0) return;
    // parts laid out [num_parts, rows, 130]
    const long long part_stride = static_cast<long long>(rows) * TQ_PARTIAL_STRIDE;
    launch_merge_kernel<false>(rows, num_parts, stream,
        partials, num_parts, part_stride, static_cast<long long>(num_q_heads) * TQ_PARTIAL_STRIDE,
        num_q_heads, static_cast<__half*>(output), partials_out, rows, num_q_heads, num_kv_heads,
        ref_query_layout, head_dim, PeerOut{}, head_sign);
    check_launch("merge_partials");
}

void launch_merge_splits(const float* partials, int splits, void* output, int rows, int num_q_heads,
                         int num_kv_heads, int head_dim, cudaStream_t stream) {
    if (rows <= 0) return;
    const long long part_stride = static_cast<long long>(num_q_heads) * TQ_PARTIAL_STRIDE;
    launch_merge_kernel<false>(rows, splits, stream, partials, splits, part_stride, part_stride * splits,
                               num_q_heads, static_cast<__half*>(output), static_cast<float*>(nullptr),
                               rows, num_q_heads, num_kv_heads, 0, head_dim, PeerOut{}, 1);
    check_launch("merge splits");
}

void launch_decode(const DecodeArgs& a, cudaStream_t stream) {
    const int H = a.geo.num_kv_heads;
    if (H < 1) throw std::runtime_error("decode: num_kv_heads must be positive");
    if (a.num_q_heads % H != 0)
        throw std::runtime_error("decode: num_q_heads must be a multiple of num_kv_heads");
    if (a.batch <= 0 || a.num_q_heads <= 0) return;
    const bool prod = a.scheme == TQ_SCHEME_TURBO_PROD;
    const bool qjl = a.scheme == TQ_SCHEME_QJL;
    // records of the QJL scheme live in a rotation without the per-head sign; the stand-alone merges
    // (tq_merge_partials, the peer exchange) apply that sign, so QJL partials are not handed out
    if (qjl && (a.peer.world > 0 || a.partials_out || a.logits_out))
        throw std::runtime_error("decode: partials, logits and the peer exchange serve turbo_prod and turbo_mse only");
    const int G = a.num_q_heads / H;
    const int qgroups = (G + 7) / 8;
    // A CTA serves at most kMaxHeads kv heads; layouts with more heads are served by one launch per
    // group of kMaxHeads heads (same grid, same splits, the partial records of all heads meet in one merge).
    const int heads_per_launch = H <= kMaxHeads ? H : kMaxHeads;
    const int streams = (H <= kMaxHeads && 8 % H == 0) ? 8 / H : 1;
    const int warps = heads_per_launch * streams;
    // per-warp regions, then the query scratch (QJL: a second one for the fp16 remainders)
    const size_t smem = static_cast<size_t>(warps) * kWarpSmemBytes +
                        (a.scheme == TQ_SCHEME_QJL ? 2 : 1) * heads_per_launch * 8 * kHeadDim * sizeof(__half);

    DecodeParams p{};
    p.query = static_cast<const __half*>(a.query);
    p.pool = a.pool;
    p.slot_mapping = a.slot_mapping;
    p.block_tables = a.block_tables;
    p.seq_lens = a.seq_lens;
    p.logits = a.logits_out;
    p.geo = a.geo;
    p.table_stride = a.table_stride;
    p.head_dim = a.head_dim;
    p.groups = G;
    p.ref_layout = a.ref_query_layout;
    p.max_kv_tokens = a.max_kv_tokens;
    p.kv_begin = a.kv_begin;
    p.kv_end = a.kv_end;
    p.streams = streams;
    p.batch = a.batch;
    p.head0 = 0;
    p.heads = heads_per_launch;
    {
        const int bs = a.geo.block_size;
        p.bs_shift = -1;
        if (bs > 0 && (bs & (bs - 1)) == 0)
            for (int sft = 0; sft < 31; ++sft)
                if ((1 << sft) == bs) p.bs_shift = sft;
        // (QJL pages, 1344 H bytes with 16-byte K rows and 64-byte V rows, satisfy the same test)
        p.aligned16 = (reinterpret_cast<uintptr_t>(a.pool) & 15) == 0 && (a.geo.page_size & 15) == 0 &&
                      (a.geo.k_codes & 15) == 0 && (a.geo.v_codes & 15) == 0;
    }
    set_smem_attr_once();

    if (a.logits_out) {
        if (!prod) throw std::runtime_error("logits: turbo_prod only");
        int splits = decode_num_splits(a.batch * qgroups, a.max_kv_tokens, H, a.geo.block_size);
        p.splits = splits;
        for (int h0 = 0; h0 < H; h0 += kMaxHeads) {
            p.head0 = h0;
            p.heads = H - h0 < kMaxHeads ? H - h0 : kMaxHeads;
            decode_kernel<true, 1><<<dim3(splits, a.batch, qgroups), p.heads * streams * 32, smem, stream>>>(p);
            check_launch("turbo_prod fused_attention_logits");
        }
        return;
    }

    const int splits = decode_num_splits(a.batch * qgroups, a.max_kv_tokens, H, a.geo.block_size);
    const size_t need = decode_workspace_bytes(a.batch, a.num_q_heads, splits);
    float* ws = static_cast<float*>(a.workspace);
    bool owned = false;
    if (!ws) {
        ws = static_cast<float*>(scratch_alloc(need, stream, "scratch_alloc(decode workspace)"));
        owned = true;
    } else if (a.workspace_bytes < need) {
        throw std::runtime_error("decode: workspace too small, need " + std::to_string(need) + " bytes");
    }
    p.partials = ws;
    p.splits = splits;

    const dim3 grid(splits, a.batch, qgroups);
    const bool fast = !qjl && a.block_tables && !a.slot_mapping && a.geo.block_size == 16 && p.aligned16 &&
                      (H == 1 || H == 2 || H == 4 || H == 8) && (a.geo.k_scales & 15) == 0 &&
                      (a.geo.v_scales & 15) == 0 && (!prod || (a.geo.k_res & 15) == 0) &&
                      a.kv_begin >= 0 && (a.kv_begin & 15) == 0;
    if (fast) {
        const dim3 fgrid((a.batch * splits + kFastGroups - 1) / kFastGroups, 1, qgroups);
#define TQ_FAST_LAUNCH(PRODV, HV)                                                                \
    launch_after_wait(decode_paged16_kernel<PRODV, HV>, fgrid, dim3(kFastGroups * kFastGroupWarps * 32), \
                      fast_smem_bytes(PRODV, HV), stream, p)
        if (prod) {
            if (H == 1) TQ_FAST_LAUNCH(true, 1);
            else if (H == 2) TQ_FAST_LAUNCH(true, 2);
            else if (H == 4) TQ_FAST_LAUNCH(true, 4);
            else TQ_FAST_LAUNCH(true, 8);
        } else {
            if (H == 1) TQ_FAST_LAUNCH(false, 1);
            else if (H == 2) TQ_FAST_LAUNCH(false, 2);
            else if (H == 4) TQ_FAST_LAUNCH(false, 4);
            else TQ_FAST_LAUNCH(false, 8);
        }
#undef TQ_FAST_LAUNCH
    } else {
        for (int h0 = 0; h0 < H; h0 += kMaxHeads) {
            p.head0 = h0;
            p.heads = H - h0 < kMaxHeads ? H - h0 : kMaxHeads;
            const int threads = p.heads * streams * 32;
            if (prod) decode_kernel<true, 0><<<grid, threads, smem, stream>>>(p);
            else if (qjl) decode_kernel<false, 0, true><<<grid, threads, smem, stream>>>(p);
            else decode_kernel<false, 0><<<grid, threads, smem, stream>>>(p);
            check_launch(prod ? "turbo_prod decode" : qjl ? "qjl decode" : "turbo_mse decode");
        }
    }

    // merge the splits of every (sequence, query head) row
    const int rows = a.batch * a.num_q_heads;
    const long long part_stride = static_cast<long long>(a.num_q_heads) * TQ_PARTIAL_STRIDE;
    launch_merge_kernel<true>(rows, splits, stream,
                      static_cast<const float*>(ws), splits, part_stride, part_stride * splits, a.num_q_heads,
                      static_cast<__half*>(a.output), a.partials_out, rows, a.num_q_heads, H,
                      a.ref_query_layout, a.head_dim, a.peer, qjl ? 0 : 1);
    check_launch("decode merge");
    if (owned) scratch_free(ws, stream, "scratch_free(decode workspace)");
}

// ---------------------------------------------------------------------------------------
// Decode without any allocation: the split-KV scratch lives in the library image.
// ---------------------------------------------------------------------------------------
//
// Some hosts of this library must not allocate device memory on the decode path: a serving
// engine that has handed the whole GPU to its own pool at start-up (any later driver
// allocation can fail or fragment it), or a real-time loop that cannot afford the implicit
// synchronisation an allocation may cause.  tq_decode_paged_static serves them: same arithmetic as tq_decode_paged, but the
// split-KV partials go to the fixed array below instead of a caller buffer or the library's stream-ordered scratch pool.
//
// The array is part of the loaded module: every GPU that loads the library holds these
// bytes until the process exits.  All calls on a device share it, and it keeps whatever the
// previous call wrote.  Nothing in it has to be zero at entry: the decode kernel writes the
// (acc, m, l) record of every (sequence, split, query head) before the merge kernel reads it.
// Two calls whose kernels can overlap on the same GPU (different streams, different threads)
// race on it; serialise them.
namespace {
constexpr size_t kStaticScratchBytes = size_t(8) << 20;  // 8 MiB per device
static __device__ __align__(256) unsigned char g_decode_scratch[kStaticScratchBytes];

// Device address of g_decode_scratch for the current device.  In host code the symbol's
// name is only a handle, not an address a kernel can use; the address comes from
// cudaGetSymbolAddress, asked once per device with that device current.
void* static_scratch_for_current_device() {
    static void* ptrs[64] = {};
    static std::mutex mu;
    int dev = 0;
    check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (dev < 0 || dev >= 64) throw std::runtime_error("decode_paged_static: device index out of range");
    std::lock_guard<std::mutex> lock(mu);
    if (!ptrs[dev]) {
        void* p = nullptr;
        check_cuda(cudaGetSymbolAddress(&p, g_decode_scratch), "cudaGetSymbolAddress(decode scratch)");
        if (!p) throw std::runtime_error("decode_paged_static: scratch symbol has no device address");
        ptrs[dev] = p;
    }
    return ptrs[dev];
}
}  // namespace
}  // namespace tq

static_assert(tq::kStaticScratchBytes == TQ_DECODE_STATIC_SCRATCH_BYTES, "header and array disagree");

extern "C" int tq_decode_paged_static(int scheme, const tq_half* query, const uint8_t* page_pool,
                                      const int32_t* block_tables, int table_stride,
                                      const int32_t* seq_lens, tq_half* output, const void* layout,
                                      const TQConfig* cfg, int batch, int num_q_heads,
                                      int max_kv_tokens, tq_stream_t stream) {
    if (!query || !page_pool || !block_tables || !seq_lens || !output || !layout || !cfg) return -1;
    try {
        if (cfg->head_dim != 128 || cfg->block_size < 1 || cfg->num_kv_heads < 1)
            throw std::runtime_error("decode_paged_static: only head_dim == 128 is supported");
        if (batch < 0 || num_q_heads < 1 || max_kv_tokens < 0 || table_stride < 0 ||
            static_cast<long long>(table_stride) * cfg->block_size < max_kv_tokens)
            throw std::runtime_error("decode_paged_static: bad sizes");
        if ((reinterpret_cast<uintptr_t>(query) & 7) || (reinterpret_cast<uintptr_t>(output) & 3))
            throw std::runtime_error("decode_paged_static: query must be 8-byte and output 4-byte aligned");
        const int H = cfg->num_kv_heads;
        if (H > 8 || num_q_heads % H != 0)
            throw std::runtime_error("decode_paged_static: num_kv_heads must be 1..8 and divide num_q_heads");
        const int qgroups = (num_q_heads / H + 7) / 8;
        const int splits = tq::decode_num_splits(batch * qgroups, max_kv_tokens, H, cfg->block_size);
        const size_t need = tq::decode_workspace_bytes(batch, num_q_heads, splits);
        if (need > tq::kStaticScratchBytes)
            throw std::runtime_error(
                "decode_paged_static: this shape needs " + std::to_string(need) +
                " bytes of split-KV scratch, the built-in array holds " +
                std::to_string(tq::kStaticScratchBytes) + "; use tq_decode_paged with a workspace");
        tq::DecodeArgs a{};
        a.scheme = scheme;
        a.query = query;
        a.pool = page_pool;
        a.block_tables = block_tables;
        a.table_stride = table_stride;
        a.seq_lens = seq_lens;
        a.output = output;
        a.geo = tq::geom_from_layout(scheme, layout, *cfg);
        a.head_dim = cfg->head_dim;
        a.batch = batch;
        a.num_q_heads = num_q_heads;
        a.ref_query_layout = 0;
        a.max_kv_tokens = max_kv_tokens;
        a.kv_begin = 0;
        a.kv_end = INT_MAX;
        a.workspace = tq::static_scratch_for_current_device();
        a.workspace_bytes = tq::kStaticScratchBytes;
        tq::launch_decode(a, static_cast<cudaStream_t>(stream));
        return 0;
    } catch (const std::exception& e) {
        tq::set_last_error(e.what());
        return -2;
    } catch (...) {
        tq::set_last_error("unknown error");
        return -2;
    }
}
