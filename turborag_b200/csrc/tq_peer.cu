// Exchange of split-KV partials between the GPUs of one NVLink domain without a collective
// library call: every rank stores its (acc, m, l) records straight into every peer's buffer
// (plain peer stores over NVLink; no multimem, no TMA), raises a flag there, and merges the
// records that arrive in its own buffer.
//
// The reference has no multi-GPU path; this replaces the all-gather + merge pair of the
// long-context decode (one launch to publish, one to merge, against a collective launch whose
// latency dominates a 100-microsecond layer).
//
// Buffers (allocated and exchanged by the host side, zero-initialised once):
//   records: 2 x [world][rows_cap][130] fp32 -- slot [e % 2][r] of rank q's buffer is written
//            only by rank r, for exchange number e;
//   flags:   2 x [world] u32 -- flag [e % 2][r] of rank q's buffer is set to e by rank r after
//            its records for exchange e are visible system-wide;
//   ticket:  one u32, counts the CTAs of the local publish kernel (self-resetting).
// Double buffering by exchange parity is enough: rank r can only publish exchange e + 2 after
// it merged e + 1, which needed q's records of e + 1, which q sent after it had finished
// reading the buffers of e.
// The merge kernel's wait for the flags is bounded by wall-clock time (2 s unless
// tq_peer_set_wait_ns chose another bound); when it runs out the kernel records a status code,
// skips the wait and finishes (results of that call are then undefined, the context stays usable).
#include "tq_common.cuh"
#include "tq_launch.h"

namespace tq {
namespace {

constexpr int kMaxPeers = 8;
constexpr unsigned long long kDefaultWaitNs = 2000000000ull;  // 2 s
// bound of the flag wait, handed to every merge launch as an argument (tq_peer_set_wait_ns)
unsigned long long g_wait_ns = kDefaultWaitNs;

struct PeerPtrs {
    float* records[kMaxPeers];
    unsigned int* flags[kMaxPeers];
};

__device__ int g_peer_status = 0;

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Copy this rank's records into slot `rank` of every peer's buffer, then let the last CTA raise
// the flags.  `local` is [rows][130] fp32.
__global__ void __launch_bounds__(256)
publish_kernel(const float* __restrict__ local, PeerPtrs peers, unsigned int* ticket, int rank,
               int world, int rows, int rows_cap, unsigned int exchange) {
    const long long n2 = static_cast<long long>(rows) * (TQ_PARTIAL_STRIDE / 2);  // float2 units
    const long long slot = (static_cast<long long>(exchange & 1u) * world + rank) * rows_cap *
                           (TQ_PARTIAL_STRIDE / 2);
    const float2* src = reinterpret_cast<const float2*>(local);
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n2;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const float2 v = __ldg(src + i);
        for (int q = 0; q < world; ++q) reinterpret_cast<float2*>(peers.records[q])[slot + i] = v;
    }
    __threadfence_system();  // this thread's peer stores are visible before the ticket moves
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int done = atomicAdd(ticket, 1u);
        if (done == gridDim.x - 1) {
            *ticket = 0u;  // ready for the next call
            __threadfence_system();
            for (int q = 0; q < world; ++q)
                st_release_sys(peers.flags[q] + (exchange & 1u) * world + rank, exchange);
        }
    }
}

// One warp per (sequence, query head) row: wait until every rank's flag shows `exchange`, then
// log-sum-exp merge of the world records, normalise, inverse rotation, fp16 store (the
// arithmetic of the decode path's merge kernel).
__global__ void __launch_bounds__(128)
peer_merge_kernel(const float* __restrict__ records, const unsigned int* __restrict__ flags, int world,
                  int rows, int rows_cap, unsigned int exchange, __half* __restrict__ output,
                  int num_q_heads, int num_kv_heads, int head_dim, unsigned long long wait_ns) {
    __shared__ int timed_out;
    if (threadIdx.x == 0) {
        int bad = 0;
        const unsigned long long t0 = global_ns();
        for (int q = 0; q < world && !bad; ++q) {
            const unsigned int* f = flags + (exchange & 1u) * world + q;
            while (ld_acquire_sys(f) != exchange) {
                if (global_ns() - t0 > wait_ns) {
                    bad = 1;
                    break;
                }
                __nanosleep(200);
            }
        }
        timed_out = bad;
        if (bad) atomicMax(&g_peer_status, 1);
    }
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const long long part_stride = static_cast<long long>(rows_cap) * TQ_PARTIAL_STRIDE;
    const float* base = records + static_cast<long long>(exchange & 1u) * world * part_stride +
                        static_cast<long long>(row) * TQ_PARTIAL_STRIDE;
    // peer stores bypass this GPU's L1: read through L2 (ld.global.cg)
    float mmax = kInitMaxLogit;
    for (int s = 0; s < world; ++s) mmax = fmaxf(mmax, __ldcg(base + s * part_stride + 128));
    float acc[4] = {0.f, 0.f, 0.f, 0.f}, l = 0.f;
    for (int s = 0; s < world; ++s) {
        const float* ps = base + s * part_stride;
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
    const int r = row % num_q_heads;
    const int h = r / G;
    const float inv_l = l > 0.0f ? 1.0f / l : 1.0f;  // tq_turbo_prod_kernels.cu:561-564
    float x[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) x[e] = acc[e] * inv_l;
    // inverse rotation: FWHT, * rsqrt(D), * s(i, h)   (tq_turbo_prod_kernels.cu:566-570)
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
    __half2* dst = reinterpret_cast<__half2*>(output + static_cast<long long>(row) * kHeadDim + 4 * lane);
    dst[0] = __floats2half2_rn(x[0] * s0, x[1] * -s0);
    dst[1] = __floats2half2_rn(x[2] * s0, x[3] * -s0);
    (void)timed_out;
}

}  // namespace

unsigned long long peer_wait_ns() { return g_wait_ns; }

void launch_peer_merge(const void* my_buffer, int world, int rows, int rows_cap, unsigned int exchange, void* output,
                       int num_q_heads, int num_kv_heads, int head_dim, cudaStream_t stream) {
    if (rows == 0) return;
    const size_t rec = (size_t(2) * world * rows_cap * TQ_PARTIAL_STRIDE * sizeof(float) + 255) / 256 * 256;
    const float* records = static_cast<const float*>(my_buffer);
    const unsigned int* flags =
        reinterpret_cast<const unsigned int*>(static_cast<const unsigned char*>(my_buffer) + rec);
    peer_merge_kernel<<<(rows + 3) / 4, 128, 0, stream>>>(records, flags, world, rows, rows_cap, exchange,
                                                          static_cast<__half*>(output), num_q_heads, num_kv_heads,
                                                          head_dim, g_wait_ns);
    check_launch("peer merge");
}

int* peer_status_ptr() {
    static int* ptrs[64] = {};
    int dev = 0;
    check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (dev < 0 || dev >= 64) throw std::runtime_error("peer exchange: device index out of range");
    if (!ptrs[dev]) {
        void* p = nullptr;
        check_cuda(cudaGetSymbolAddress(&p, g_peer_status), "cudaGetSymbolAddress(peer status)");
        ptrs[dev] = static_cast<int*>(p);
    }
    return ptrs[dev];
}
}  // namespace tq

extern "C" size_t tq_peer_buffer_bytes(int world, int rows_cap) {
    if (world < 1 || rows_cap < 1) return 0;
    const size_t rec = size_t(2) * world * rows_cap * TQ_PARTIAL_STRIDE * sizeof(float);
    return (rec + 255) / 256 * 256 + 256;  // records, then 2 x world flags and the ticket
}

extern "C" int tq_peer_publish(const float* local_partials, void* const* peer_buffers, int rank, int world,
                               int rows, int rows_cap, unsigned int exchange, tq_stream_t stream) {
    if (!local_partials || !peer_buffers) return -1;
    try {
        if (world < 1 || world > tq::kMaxPeers || rank < 0 || rank >= world || rows < 0 || rows > rows_cap)
            throw std::runtime_error("peer_publish: bad rank / world / rows");
        if (rows == 0) return 0;
        const size_t rec = (size_t(2) * world * rows_cap * TQ_PARTIAL_STRIDE * sizeof(float) + 255) / 256 * 256;
        tq::PeerPtrs p{};
        for (int q = 0; q < world; ++q) {
            if (!peer_buffers[q]) throw std::runtime_error("peer_publish: null peer buffer");
            p.records[q] = static_cast<float*>(peer_buffers[q]);
            p.flags[q] = reinterpret_cast<unsigned int*>(static_cast<unsigned char*>(peer_buffers[q]) + rec);
        }
        unsigned int* ticket = p.flags[rank] + 2 * world;
        const long long n2 = static_cast<long long>(rows) * (TQ_PARTIAL_STRIDE / 2);
        int blocks = static_cast<int>((n2 + 255) / 256);
        if (blocks > 64) blocks = 64;
        tq::publish_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
            local_partials, p, ticket, rank, world, rows, rows_cap, exchange);
        tq::check_launch("peer publish");
        return 0;
    } catch (const std::exception& e) {
        tq::set_last_error(e.what());
        return -2;
    }
}

extern "C" int tq_peer_merge(const void* my_buffer, int world, int rows, int rows_cap, unsigned int exchange,
                             tq_half* output, int num_q_heads, int num_kv_heads, int head_dim,
                             tq_stream_t stream) {
    if (!my_buffer || !output) return -1;
    try {
        if (world < 1 || world > tq::kMaxPeers || rows < 0 || rows > rows_cap || head_dim != 128 ||
            num_kv_heads < 1 || num_q_heads % num_kv_heads != 0 || rows % num_q_heads != 0)
            throw std::runtime_error("peer_merge: bad shape");
        tq::launch_peer_merge(my_buffer, world, rows, rows_cap, exchange, output, num_q_heads, num_kv_heads,
                              head_dim, static_cast<cudaStream_t>(stream));
        return 0;
    } catch (const std::exception& e) {
        tq::set_last_error(e.what());
        return -2;
    }
}

extern "C" int tq_peer_status(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, tq::g_peer_status, sizeof v) != cudaSuccess) return -2;
    return v;
}

extern "C" int tq_peer_set_wait_ns(unsigned long long ns) {
    tq::g_wait_ns = ns ? ns : tq::kDefaultWaitNs;
    return 0;
}

extern "C" int tq_peer_clear_status(void) {
    const int zero = 0;
    return cudaMemcpyToSymbol(tq::g_peer_status, &zero, sizeof zero) == cudaSuccess ? 0 : -2;
}
