// extern "C" surface of libturboquant (see include/turboquant.h).
//
// Part 1 mirrors src/tq_capi.cpp of the reference symbol for symbol: null
// arguments -> -1, any failure in a launch helper -> -2 with the text kept in a
// thread-local buffer returned by tq_last_error(), no C++ exception ever
// crosses the boundary, no synchronisation.
#include <cuda_runtime.h>

#include <climits>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "tq_launch.h"
#include "turboquant.h"

static_assert(sizeof(TQConfig) == 32, "TQConfig ABI");
static_assert(sizeof(TQTurboProdPageLayout) == 64, "TQTurboProdPageLayout ABI");
static_assert(sizeof(TQTurbomsePageLayout) == 56, "TQTurbomsePageLayout ABI");

namespace tq {

void check_cuda(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

void check_launch(const char* name) {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) throw std::runtime_error(std::string(name) + ": " + cudaGetErrorString(e));
#ifdef TQ_DEBUG_SYNC
    const cudaError_t s = cudaDeviceSynchronize();
    if (s != cudaSuccess)
        throw std::runtime_error(std::string("async kernel error: ") + cudaGetErrorString(s));
#endif
}

int sm_count() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace tq

namespace {

thread_local char g_last_error[512] = "";

void set_error(const char* msg) { std::snprintf(g_last_error, sizeof g_last_error, "%.511s", msg); }

template <typename F>
int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        set_error(e.what());
        return -2;
    } catch (...) {
        set_error("unknown error");
        return -2;
    }
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

void check_shape(const TQConfig& cfg, const char* who) {
    if (cfg.head_dim > 128) throw std::runtime_error(std::string(who) + ": head_dim > 128 is not supported");
    if (cfg.head_dim != 128)
        throw std::runtime_error(std::string(who) + ": only head_dim == 128 is supported by the sm_100a kernels");
    if (cfg.block_size < 1 || cfg.num_kv_heads < 1)
        throw std::runtime_error(std::string(who) + ": block_size and num_kv_heads must be positive");
}

void check_align(const void* p, size_t a, const char* what) {
    if (reinterpret_cast<uintptr_t>(p) % a != 0)
        throw std::runtime_error(std::string(what) + " must be " + std::to_string(a) + "-byte aligned");
}

tq::PageGeom geom_prod(const TQTurboProdPageLayout& l, const TQConfig& cfg) {
    if (l.k4_bytes_per_token_head != 64 || l.v4_bytes_per_token_head != 64 ||
        l.scale_bytes_per_token_head != 2)
        throw std::runtime_error("turbo_prod: layout does not match head_dim 128");
    tq::PageGeom g{};
    g.page_size = l.page_size_bytes;
    g.k_codes = static_cast<unsigned>(l.k4_codes_offset);
    g.v_codes = static_cast<unsigned>(l.v4_codes_offset);
    g.k_scales = static_cast<unsigned>(l.k_scales_offset);
    g.v_scales = static_cast<unsigned>(l.v_scales_offset);
    g.k_res = static_cast<unsigned>(l.k_residual_scales_offset);
    g.block_size = cfg.block_size;
    g.num_kv_heads = cfg.num_kv_heads;
    return g;
}

tq::PageGeom geom_mse(const TQTurbomsePageLayout& l, const TQConfig& cfg) {
    if (l.code_bytes_per_token_head != 64 || l.norm_bytes_per_token_head != 2)
        throw std::runtime_error("turbo_mse: layout does not match head_dim 128 / 4 bits");
    tq::PageGeom g{};
    g.page_size = l.page_size_bytes;
    g.k_codes = static_cast<unsigned>(l.k_codes_offset);
    g.v_codes = static_cast<unsigned>(l.v_codes_offset);
    g.k_scales = static_cast<unsigned>(l.k_norms_offset);
    g.v_scales = static_cast<unsigned>(l.v_norms_offset);
    g.k_res = 0;
    g.block_size = cfg.block_size;
    g.num_kv_heads = cfg.num_kv_heads;
    return g;
}

tq::PageGeom geom_qjl(const TQQJLPageLayout& l, const TQConfig& cfg) {
    if (l.k1_bytes_per_token_head != 16 || l.v4_bytes_per_token_head != 64 ||
        l.scale_bytes_per_token_head != 2)
        throw std::runtime_error("qjl: layout does not match head_dim 128");
    tq::PageGeom g{};
    g.page_size = l.page_size_bytes;
    g.k_codes = static_cast<unsigned>(l.k1_codes_offset);
    g.v_codes = static_cast<unsigned>(l.v4_codes_offset);
    g.k_scales = static_cast<unsigned>(l.k_scales_offset);
    g.v_scales = static_cast<unsigned>(l.v_scales_offset);
    g.k_res = 0;
    g.block_size = cfg.block_size;
    g.num_kv_heads = cfg.num_kv_heads;
    return g;
}

tq::PageGeom geom_for(int scheme, const void* layout, const TQConfig& cfg) {
    if (scheme == TQ_SCHEME_QJL) return geom_qjl(*static_cast<const TQQJLPageLayout*>(layout), cfg);
    if (scheme == TQ_SCHEME_TURBO_PROD)
        return geom_prod(*static_cast<const TQTurboProdPageLayout*>(layout), cfg);
    if (scheme == TQ_SCHEME_TURBO_MSE)
        return geom_mse(*static_cast<const TQTurbomsePageLayout*>(layout), cfg);
    throw std::runtime_error("unknown scheme");
}

// Reference-API fused attention: one sequence, per-token slots, query rows [q][h].
void ref_attention(int scheme, const void* query, const uint8_t* pool, const int32_t* slots,
                   void* output, float* logits, const tq::PageGeom& geo, const TQConfig& cfg,
                   int num_queries, int num_kv_tokens, cudaStream_t stream) {
    if (num_queries <= 0) return;
    if (num_kv_tokens < 0) throw std::runtime_error("num_kv_tokens < 0");
    check_align(query, 8, "query");
    if (output) check_align(output, 4, "output");
    tq::DecodeArgs a{};
    a.scheme = scheme;
    a.query = query;
    a.pool = pool;
    a.slot_mapping = slots;
    a.output = output;
    a.logits_out = logits;
    a.geo = geo;
    a.head_dim = cfg.head_dim;
    a.batch = 1;
    a.num_q_heads = num_queries * cfg.num_kv_heads;
    a.ref_query_layout = 1;
    a.max_kv_tokens = num_kv_tokens;
    a.kv_begin = 0;
    a.kv_end = INT_MAX;
    tq::launch_decode(a, stream);
}

}  // namespace

namespace tq {
void* scratch_alloc(size_t bytes, cudaStream_t stream, const char* what) {
    static cudaMemPool_t pools[64] = {};
    static std::mutex mu;
    int dev = 0;
    check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (dev < 0 || dev >= 64) throw std::runtime_error("scratch: device index out of range");
    cudaMemPool_t pool;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!pools[dev]) {
            cudaMemPoolProps props{};
            props.allocType = cudaMemAllocationTypePinned;
            props.handleTypes = cudaMemHandleTypeNone;
            props.location.type = cudaMemLocationTypeDevice;
            props.location.id = dev;
            check_cuda(cudaMemPoolCreate(&pools[dev], &props), "cudaMemPoolCreate(scratch)");
            unsigned long long keep = 1ull << 30;
            check_cuda(cudaMemPoolSetAttribute(pools[dev], cudaMemPoolAttrReleaseThreshold, &keep),
                       "cudaMemPoolSetAttribute(release threshold)");
        }
        pool = pools[dev];
    }
    void* p = nullptr;
    check_cuda(cudaMallocFromPoolAsync(&p, bytes, pool, stream), what);
    return p;
}
void scratch_free(void* p, cudaStream_t stream, const char* what) { check_cuda(cudaFreeAsync(p, stream), what); }

void set_last_error(const char* msg) { set_error(msg); }
PageGeom geom_from_layout(int scheme, const void* layout, const TQConfig& cfg) {
    return geom_for(scheme, layout, cfg);
}
}  // namespace tq

// ---------------------------------------------------------------------------
// Part 1 — reference surface
// ---------------------------------------------------------------------------

extern "C" const char* tq_last_error(void) { return g_last_error; }

extern "C" int tq_make_default_config(TQConfig* out_cfg) {
    if (!out_cfg) return -1;
    *out_cfg = TQConfig{16, 8, 128, 4, 128, 256, 0, 0};
    return 0;
}

extern "C" int tq_make_turbo_prod_layout(const TQConfig* cfg, TQTurboProdPageLayout* out) {
    if (!cfg || !out) return -1;
    TQTurboProdPageLayout l{};
    l.k4_bytes_per_token_head = (cfg->head_dim + 1) / 2;
    l.v4_bytes_per_token_head = (cfg->head_dim * 4 + 7) / 8;
    l.scale_bytes_per_token_head = 2;
    const size_t cells = static_cast<size_t>(cfg->block_size) * cfg->num_kv_heads;
    size_t at = 0;
    l.k4_codes_offset = at;
    at = align_up(at + cells * l.k4_bytes_per_token_head, 2);
    l.k_residual_scales_offset = at;
    at += cells * 2;
    l.k_scales_offset = at;
    at += cells * 2;
    l.v4_codes_offset = at;
    at = align_up(at + cells * l.v4_bytes_per_token_head, 2);
    l.v_scales_offset = at;
    at += cells * 2;
    l.page_size_bytes = align_up(at, 2);
    *out = l;
    return 0;
}

extern "C" int tq_make_turbo_mse_layout(const TQConfig* cfg, TQTurbomsePageLayout* out) {
    if (!cfg || !out) return -1;
    TQTurbomsePageLayout l{};
    l.code_bytes_per_token_head = static_cast<size_t>((cfg->head_dim * cfg->nbits + 7) / 8);
    l.norm_bytes_per_token_head = 2;
    const size_t cells = static_cast<size_t>(cfg->block_size) * cfg->num_kv_heads;
    const size_t al = static_cast<size_t>(cfg->page_alignment > 0 ? cfg->page_alignment : 1);
    const size_t codes = cells * l.code_bytes_per_token_head, norms = cells * 2;
    l.k_codes_offset = 0;
    l.v_codes_offset = align_up(codes, al);
    l.k_norms_offset = align_up(l.v_codes_offset + codes, al);
    l.v_norms_offset = align_up(l.k_norms_offset + norms, al);
    l.page_size_bytes = align_up(l.v_norms_offset + norms, al);
    *out = l;
    return 0;
}

extern "C" int tq_launch_turbo_prod_pack_kv(const tq_half* key, const tq_half* value,
                                            const int32_t* slot_mapping, uint8_t* page_pool,
                                            const TQTurboProdPageLayout* layout, const TQConfig* cfg,
                                            int num_tokens, tq_stream_t stream) {
    if (!key || !value || !slot_mapping || !page_pool || !layout || !cfg) return -1;
    return guarded([&] {
        check_shape(*cfg, "turbo_prod");
        check_align(key, 16, "key");
        check_align(value, 16, "value");
        tq::launch_pack(TQ_SCHEME_TURBO_PROD, key, value, slot_mapping, page_pool, geom_prod(*layout, *cfg),
                        cfg->head_dim, num_tokens, static_cast<cudaStream_t>(stream));
    });
}

extern "C" int tq_debug_turbo_prod_pack_kv(const tq_half* key, const tq_half* value, const int32_t* slot_mapping,
                                           uint8_t* page_pool, const TQTurboProdPageLayout* layout,
                                           const TQConfig* cfg, int num_tokens, float* debug_k_rot,
                                           float* debug_v_rot, float* debug_kn, float* debug_vn,
                                           int* debug_kidx, int* debug_vidx, tq_stream_t stream) {
    if (!key || !value || !slot_mapping || !page_pool || !layout || !cfg) return -1;
    return guarded([&] {
        check_shape(*cfg, "turbo_prod");
        check_align(key, 16, "key");
        check_align(value, 16, "value");
        tq::launch_pack_debug(key, value, slot_mapping, page_pool, geom_prod(*layout, *cfg), cfg->head_dim,
                              num_tokens, debug_k_rot, debug_v_rot, debug_kn, debug_vn, debug_kidx, debug_vidx,
                              static_cast<cudaStream_t>(stream));
    });
}

extern "C" int tq_launch_turbo_prod_dequant_kv(const uint8_t* page_pool, const int32_t* slot_mapping,
                                               tq_half* out_key, tq_half* out_value,
                                               const TQTurboProdPageLayout* layout,
                                               const TQConfig* cfg, int num_tokens,
                                               tq_stream_t stream) {
    if (!page_pool || !slot_mapping || !out_key || !out_value || !layout || !cfg) return -1;
    return guarded([&] {
        check_shape(*cfg, "turbo_prod");
        check_align(out_key, 4, "out_key");
        check_align(out_value, 4, "out_value");
        tq::launch_dequant(TQ_SCHEME_TURBO_PROD, page_pool, slot_mapping, out_key, out_value,
                           geom_prod(*layout, *cfg), cfg->head_dim, num_tokens, false,
                           static_cast<cudaStream_t>(stream));
    });
}

extern "C" int tq_launch_turbo_prod_fused_attention_logits(
    const tq_half* query, const uint8_t* page_pool, const int32_t* slot_mapping, float* logits,
    const TQTurboProdPageLayout* layout, const TQConfig* cfg, int num_queries, int num_kv_tokens,
    tq_stream_t stream) {
    if (!query || !page_pool || !slot_mapping || !logits || !layout || !cfg) return -1;
    return guarded([&] {
        check_shape(*cfg, "turbo_prod");
        ref_attention(TQ_SCHEME_TURBO_PROD, query, page_pool, slot_mapping, nullptr, logits,
                      geom_prod(*layout, *cfg), *cfg, num_queries, num_kv_tokens,
                      static_cast<cudaStream_t>(stream));
    });
}

extern "C" int tq_launch_turbo_prod_fused_attention_output(
    const tq_half* query, const uint8_t* page_pool, const int32_t* slot_mapping, tq_half* output,
    const TQTurboProdPageLayout* layout, const TQConfig* cfg, int num_queries, int num_kv_tokens,
    tq_stream_t stream) {
    if (!query || !page_pool || !slot_mapping || !output || !layout || !cfg) return -1;
    return guarded([&] {
        check_shape(*cfg, "turbo_prod");
        ref_attention(TQ_SCHEME_TURBO_PROD, query, page_pool, slot_mapping, output, nullptr,
                      geom_prod(*layout, *cfg), *cfg, num_queries, num_kv_tokens,
                      static_cast<cudaStream_t>(stream));
    });
}

extern "C" int tq_launch_turbo_mse_pack_kv(const tq_half* key, const tq_half* value,
                                           const int32_t* slot_mapping, uint8_t* page_pool,
                                           const TQTurbomsePageLayout* layout, const TQConfig* cfg,
                                           int num_tokens, tq_stream_t stream) {
    if (!key || !value || !slot_mapping || !page_pool || !layout || !cfg) return -1;
    return guarded([&] {
        check_shape(*cfg, "turbo_mse pack");
        check_align(key, 16, "key");
        check_align(value, 16, "value");
        tq::launch_pack(TQ_SCHEME_TURBO_MSE, key, value, slot_mapping, page_pool, geom_mse(*layout, *cfg),
                        cfg->head_dim, num_tokens, static_cast<cudaStream_t>(stream));
    });
}

extern "C" int tq_launch_turbo_mse_dequant_kv(const uint8_t* page_pool, const int32_t* slot_mapping,
                                              tq_half* out_key, tq_half* out_value,
                                              const TQTurbomsePageLayout* layout, const TQConfig* cfg,
                                              int num_tokens, tq_stream_t stream) {
    if (!page_pool || !slot_mapping || !out_key || !out_value || !layout || !cfg) return -1;
    return guarded([&] {
        check_shape(*cfg, "turbo_mse dequant");
        check_align(out_key, 4, "out_key");
        check_align(out_value, 4, "out_value");
        tq::launch_dequant(TQ_SCHEME_TURBO_MSE, page_pool, slot_mapping, out_key, out_value,
                           geom_mse(*layout, *cfg), cfg->head_dim, num_tokens, false,
                           static_cast<cudaStream_t>(stream));
    });
}

extern "C" int tq_launch_turbo_mse_fused_attention_output(
    const tq_half* query, const uint8_t* page_pool, const int32_t* slot_mapping, tq_half* output,
    const TQTurbomsePageLayout* layout, const TQConfig* cfg, int num_queries, int num_kv_tokens,
    tq_stream_t stream) {
    if (!query || !page_pool || !slot_mapping || !output || !layout || !cfg) return -1;
    return guarded([&] {
        check_shape(*cfg, "turbo_mse fused attn");
        ref_attention(TQ_SCHEME_TURBO_MSE, query, page_pool, slot_mapping, output, nullptr,
                      geom_mse(*layout, *cfg), *cfg, num_queries, num_kv_tokens,
                      static_cast<cudaStream_t>(stream));
    });
}

// ---- QJL-1bit (compiled but unexported in the reference: src/cuda/tq_qjl_kernels.cu) -------

extern "C" int tq_make_qjl_layout(const TQConfig* cfg, TQQJLPageLayout* out) {
    if (!cfg || !out) return -1;
    TQQJLPageLayout l{};
    l.k1_bytes_per_token_head = (cfg->head_dim + 7) / 8;
    l.v4_bytes_per_token_head = (cfg->head_dim * 4 + 7) / 8;
    l.scale_bytes_per_token_head = 2;
    const size_t cells = static_cast<size_t>(cfg->block_size) * cfg->num_kv_heads;
    size_t at = 0;
    l.k1_codes_offset = at;
    at = align_up(at + cells * l.k1_bytes_per_token_head, 2);
    l.k_scales_offset = at;
    at += cells * 2;
    l.v4_codes_offset = at;
    at = align_up(at + cells * l.v4_bytes_per_token_head, 2);
    l.v_scales_offset = at;
    at += cells * 2;
    l.page_size_bytes = align_up(at, 2);
    *out = l;
    return 0;
}

extern "C" int tq_launch_qjl_pack_kv(const tq_half* key, const tq_half* value, const int32_t* slot_mapping,
                                     uint8_t* page_pool, const TQQJLPageLayout* layout, const TQConfig* cfg,
                                     int num_tokens, tq_stream_t stream) {
    if (!key || !value || !slot_mapping || !page_pool || !layout || !cfg) return -1;
    return guarded([&] {
        check_shape(*cfg, "QJL");
        check_align(key, 16, "key");
        check_align(value, 16, "value");
        tq::launch_pack(TQ_SCHEME_QJL, key, value, slot_mapping, page_pool, geom_qjl(*layout, *cfg),
                        cfg->head_dim, num_tokens, static_cast<cudaStream_t>(stream));
    });
}

extern "C" int tq_launch_qjl_dequant_kv(const uint8_t* page_pool, const int32_t* slot_mapping,
                                        tq_half* out_key, tq_half* out_value, const TQQJLPageLayout* layout,
                                        const TQConfig* cfg, int num_tokens, tq_stream_t stream) {
    if (!page_pool || !slot_mapping || !out_key || !out_value || !layout || !cfg) return -1;
    return guarded([&] {
        check_shape(*cfg, "QJL");
        check_align(out_key, 4, "out_key");
        check_align(out_value, 4, "out_value");
        tq::launch_dequant(TQ_SCHEME_QJL, page_pool, slot_mapping, out_key, out_value, geom_qjl(*layout, *cfg),
                           cfg->head_dim, num_tokens, false, static_cast<cudaStream_t>(stream));
    });
}

extern "C" int tq_launch_qjl_fused_attention_output(const tq_half* query, const uint8_t* page_pool,
                                                    const int32_t* slot_mapping, tq_half* output,
                                                    const TQQJLPageLayout* layout, const TQConfig* cfg,
                                                    int num_queries, int num_kv_tokens, tq_stream_t stream) {
    if (!query || !page_pool || !slot_mapping || !output || !layout || !cfg) return -1;
    return guarded([&] {
        check_shape(*cfg, "QJL");
        ref_attention(TQ_SCHEME_QJL, query, page_pool, slot_mapping, output, nullptr, geom_qjl(*layout, *cfg),
                      *cfg, num_queries, num_kv_tokens, static_cast<cudaStream_t>(stream));
    });
}

// ---------------------------------------------------------------------------
// Part 2 — additions
// ---------------------------------------------------------------------------

extern "C" int tq_decode_num_splits(int batch, int max_kv_tokens, int num_kv_heads, int block_size) {
    if (num_kv_heads < 1) return 1;
    return tq::decode_num_splits(batch, max_kv_tokens, num_kv_heads, block_size);
}

extern "C" size_t tq_decode_workspace_bytes(int batch, int num_q_heads, int num_splits) {
    if (batch < 0 || num_q_heads < 0 || num_splits < 0) return 0;
    return tq::decode_workspace_bytes(batch, num_q_heads, num_splits);
}

extern "C" int tq_decode_paged(int scheme, const tq_half* query, const uint8_t* page_pool,
                               const int32_t* block_tables, int table_stride,
                               const int32_t* seq_lens, tq_half* output, float* partials_out,
                               const void* layout, const TQConfig* cfg, int batch, int num_q_heads,
                               int max_kv_tokens, int kv_begin, int kv_end, void* workspace,
                               size_t workspace_bytes, tq_stream_t stream) {
    if (!query || !page_pool || !block_tables || !seq_lens || !layout || !cfg) return -1;
    if (!output && !partials_out) return -1;
    return guarded([&] {
        check_shape(*cfg, "decode_paged");
        check_align(query, 8, "query");
        if (output) check_align(output, 4, "output");
        if (batch < 0 || num_q_heads < 1 || max_kv_tokens < 0 || table_stride < 0)
            throw std::runtime_error("decode_paged: negative size");
        if (static_cast<long long>(table_stride) * cfg->block_size < max_kv_tokens)
            throw std::runtime_error("decode_paged: block table narrower than max_kv_tokens");
        tq::DecodeArgs a{};
        a.scheme = scheme;
        a.query = query;
        a.pool = page_pool;
        a.block_tables = block_tables;
        a.table_stride = table_stride;
        a.seq_lens = seq_lens;
        a.output = output;
        a.partials_out = partials_out;
        a.geo = geom_for(scheme, layout, *cfg);
        a.head_dim = cfg->head_dim;
        a.batch = batch;
        a.num_q_heads = num_q_heads;
        a.ref_query_layout = 0;
        a.max_kv_tokens = max_kv_tokens;
        a.kv_begin = kv_begin;
        a.kv_end = kv_end;
        a.workspace = workspace;
        a.workspace_bytes = workspace_bytes;
        tq::launch_decode(a, static_cast<cudaStream_t>(stream));
    });
}

extern "C" int tq_decode_paged_publish(int scheme, const tq_half* query, const uint8_t* page_pool,
                                       const int32_t* block_tables, int table_stride,
                                       const int32_t* seq_lens, const void* layout, const TQConfig* cfg,
                                       int batch, int num_q_heads, int max_kv_tokens, int kv_begin,
                                       int kv_end, void* workspace, size_t workspace_bytes,
                                       void* const* peer_buffers, int rank, int world, int rows_cap,
                                       unsigned int exchange, tq_stream_t stream) {
    if (!query || !page_pool || !block_tables || !seq_lens || !layout || !cfg || !peer_buffers) return -1;
    return guarded([&] {
        check_shape(*cfg, "decode_paged_publish");
        check_align(query, 8, "query");
        if (batch < 0 || num_q_heads < 1 || max_kv_tokens < 0 || table_stride < 0)
            throw std::runtime_error("decode_paged_publish: negative size");
        if (static_cast<long long>(table_stride) * cfg->block_size < max_kv_tokens)
            throw std::runtime_error("decode_paged_publish: block table narrower than max_kv_tokens");
        const long long rows = static_cast<long long>(batch) * num_q_heads;
        if (world < 1 || world > 8 || rank < 0 || rank >= world || rows > rows_cap)
            throw std::runtime_error("decode_paged_publish: bad rank / world / rows_cap");
        tq::DecodeArgs a{};
        a.scheme = scheme;
        a.query = query;
        a.pool = page_pool;
        a.block_tables = block_tables;
        a.table_stride = table_stride;
        a.seq_lens = seq_lens;
        a.geo = geom_for(scheme, layout, *cfg);
        a.head_dim = cfg->head_dim;
        a.batch = batch;
        a.num_q_heads = num_q_heads;
        a.ref_query_layout = 0;
        a.max_kv_tokens = max_kv_tokens;
        a.kv_begin = kv_begin;
        a.kv_end = kv_end;
        a.workspace = workspace;
        a.workspace_bytes = workspace_bytes;
        const size_t rec = (size_t(2) * world * rows_cap * TQ_PARTIAL_STRIDE * sizeof(float) + 255) / 256 * 256;
        for (int q = 0; q < world; ++q) {
            if (!peer_buffers[q]) throw std::runtime_error("decode_paged_publish: null peer buffer");
            a.peer.records[q] = static_cast<float*>(peer_buffers[q]);
            a.peer.flags[q] = reinterpret_cast<unsigned int*>(static_cast<unsigned char*>(peer_buffers[q]) + rec);
        }
        a.peer.ticket = a.peer.flags[rank] + 2 * world;
        a.peer.world = world;
        a.peer.rank = rank;
        a.peer.rows_cap = rows_cap;
        a.peer.exchange = exchange;
        tq::launch_decode(a, static_cast<cudaStream_t>(stream));
    });
}

extern "C" int tq_decode_paged_exchange(int scheme, const tq_half* query, const uint8_t* page_pool,
                                        const int32_t* block_tables, int table_stride,
                                        const int32_t* seq_lens, const void* layout, const TQConfig* cfg,
                                        int batch, int num_q_heads, int max_kv_tokens, int kv_begin,
                                        int kv_end, void* workspace, size_t workspace_bytes,
                                        void* const* peer_buffers, int rank, int world, int rows_cap,
                                        unsigned int exchange, tq_half* output, tq_stream_t stream) {
    if (!query || !page_pool || !block_tables || !seq_lens || !layout || !cfg || !peer_buffers || !output) return -1;
    return guarded([&] {
        check_shape(*cfg, "decode_paged_exchange");
        check_align(query, 8, "query");
        check_align(output, 4, "output");
        if (batch < 0 || num_q_heads < 1 || max_kv_tokens < 0 || table_stride < 0)
            throw std::runtime_error("decode_paged_exchange: negative size");
        if (static_cast<long long>(table_stride) * cfg->block_size < max_kv_tokens)
            throw std::runtime_error("decode_paged_exchange: block table narrower than max_kv_tokens");
        const long long rows = static_cast<long long>(batch) * num_q_heads;
        if (world < 1 || world > 8 || rank < 0 || rank >= world || rows > rows_cap)
            throw std::runtime_error("decode_paged_exchange: bad rank / world / rows_cap");
        if (rows == 0) return;
        tq::DecodeArgs a{};
        a.scheme = scheme;
        a.query = query;
        a.pool = page_pool;
        a.block_tables = block_tables;
        a.table_stride = table_stride;
        a.seq_lens = seq_lens;
        a.geo = geom_for(scheme, layout, *cfg);
        a.head_dim = cfg->head_dim;
        a.batch = batch;
        a.num_q_heads = num_q_heads;
        a.ref_query_layout = 0;
        a.max_kv_tokens = max_kv_tokens;
        a.kv_begin = kv_begin;
        a.kv_end = kv_end;
        a.workspace = workspace;
        a.workspace_bytes = workspace_bytes;
        const size_t rec = (size_t(2) * world * rows_cap * TQ_PARTIAL_STRIDE * sizeof(float) + 255) / 256 * 256;
        for (int q = 0; q < world; ++q) {
            if (!peer_buffers[q]) throw std::runtime_error("decode_paged_exchange: null peer buffer");
            a.peer.records[q] = static_cast<float*>(peer_buffers[q]);
            a.peer.flags[q] = reinterpret_cast<unsigned int*>(static_cast<unsigned char*>(peer_buffers[q]) + rec);
        }
        a.peer.ticket = a.peer.flags[rank] + 2 * world;
        a.peer.world = world;
        a.peer.rank = rank;
        a.peer.rows_cap = rows_cap;
        a.peer.exchange = exchange;
        // The publishing kernel finishes the exchange itself when all of its CTAs are resident at once
        // (they wait for a flag that its own last CTA raises): at most one CTA per row, eight warps each.
        const bool fused = rows <= 4ll * tq::sm_count();
        if (fused) {
            a.peer.final_out = output;
            a.peer.wait_ns = tq::peer_wait_ns();
            a.peer.status = tq::peer_status_ptr();
        }
        tq::launch_decode(a, static_cast<cudaStream_t>(stream));
        if (!fused)
            tq::launch_peer_merge(peer_buffers[rank], world, static_cast<int>(rows), rows_cap, exchange, output,
                                  num_q_heads, cfg->num_kv_heads, cfg->head_dim, static_cast<cudaStream_t>(stream));
    });
}

extern "C" int tq_merge_partials(const float* partials, int num_parts, tq_half* output, int rows,
                                 int num_q_heads, int num_kv_heads, tq_stream_t stream) {
    if (!partials || !output) return -1;
    return guarded([&] {
        if (num_parts < 1 || rows < 0 || num_q_heads < 1 || num_kv_heads < 1 ||
            num_q_heads % num_kv_heads != 0 || rows % num_q_heads != 0)
            throw std::runtime_error("merge_partials: bad sizes");
        check_align(partials, 8, "partials");
        check_align(output, 4, "output");
        tq::launch_merge(partials, num_parts, output, nullptr, rows, num_q_heads, num_kv_heads, 0,
                         128, static_cast<cudaStream_t>(stream));
    });
}

extern "C" int tq_dequant_kv_hnd(int scheme, const uint8_t* page_pool, const int32_t* slot_mapping,
                                 tq_half* out_key, tq_half* out_value, const void* layout,
                                 const TQConfig* cfg, int num_tokens, tq_stream_t stream) {
    if (!page_pool || !slot_mapping || !out_key || !out_value || !layout || !cfg) return -1;
    return guarded([&] {
        check_shape(*cfg, "dequant_kv_hnd");
        check_align(out_key, 4, "out_key");
        check_align(out_value, 4, "out_value");
        tq::launch_dequant(scheme, page_pool, slot_mapping, out_key, out_value,
                           geom_for(scheme, layout, *cfg), cfg->head_dim, num_tokens, true,
                           static_cast<cudaStream_t>(stream));
    });
}

extern "C" int tq_mse_prefill_paged(const tq_half* query, const uint8_t* page_pool,
                                    const int32_t* block_tables, int table_stride,
                                    const int32_t* seq_lens, const tq_half* chunk_key,
                                    const tq_half* chunk_value, tq_half* output,
                                    const TQTurbomsePageLayout* layout, const TQConfig* cfg,
                                    int batch, int num_q_tokens, int num_q_heads,
                                    tq_stream_t stream) {
    if (!query || !page_pool || !block_tables || !seq_lens || !output || !layout || !cfg) return -1;
    if ((chunk_key == nullptr) != (chunk_value == nullptr)) return -1;
    return guarded([&] {
        check_shape(*cfg, "mse_prefill_paged");
        check_align(query, 8, "query");
        check_align(output, 4, "output");
        if (chunk_key) {
            check_align(chunk_key, 8, "chunk_key");
            check_align(chunk_value, 8, "chunk_value");
        }
        if (batch < 0 || num_q_tokens < 0 || num_q_heads < 1 || table_stride < 0)
            throw std::runtime_error("mse_prefill_paged: negative size");
        if (cfg->num_kv_heads > 8) throw std::runtime_error("mse_prefill_paged: num_kv_heads must be 1..8");
        tq::launch_prefill_tc(
            query, page_pool, block_tables, table_stride, seq_lens, chunk_key, chunk_value, output,
            geom_mse(*layout, *cfg), cfg->head_dim, batch, num_q_tokens, num_q_heads,
            table_stride * cfg->block_size, static_cast<cudaStream_t>(stream));
    });
}

extern "C" int tq_mse_prefill_status(void) {
    int v = -1;
    const int rc = guarded([&] { v = tq::prefill_tc_status(); });
    return rc != 0 ? rc : v;
}

// ---- host page allocator + block table -------------------------------------

struct TQBlockTableHandle {
    int block_size = 16;
    std::vector<int32_t> free_list;  // LIFO: back() is handed out next
    struct Seq {
        std::vector<int32_t> pages;
        int num_tokens = 0;
    };
    std::unordered_map<int, Seq> seqs;
    std::mutex mu;
};

extern "C" TQBlockTableHandle* tq_block_table_create(int num_pages, int block_size) {
    if (num_pages < 0 || block_size < 1) return nullptr;
    try {
        auto* h = new TQBlockTableHandle();
        h->block_size = block_size;
        h->free_list.reserve(static_cast<size_t>(num_pages));
        // page 0 is handed out first, as in the reference's free list
        for (int i = num_pages - 1; i >= 0; --i) h->free_list.push_back(i);
        return h;
    } catch (...) {
        return nullptr;
    }
}

extern "C" void tq_block_table_destroy(TQBlockTableHandle* h) { delete h; }

extern "C" int tq_block_table_free_pages(const TQBlockTableHandle* h) {
    if (!h) return -1;
    std::lock_guard<std::mutex> lock(const_cast<TQBlockTableHandle*>(h)->mu);
    return static_cast<int>(h->free_list.size());
}

extern "C" int tq_block_table_append(TQBlockTableHandle* h, int seq_id, int append_tokens,
                                     int32_t* slots_out) {
    if (!h || append_tokens < 0 || (append_tokens > 0 && !slots_out)) return -1;
    return guarded([&] {
        std::lock_guard<std::mutex> lock(h->mu);
        auto& s = h->seqs[seq_id];
        const int bs = h->block_size;
        const int need = (s.num_tokens + append_tokens + bs - 1) / bs;
        if (need - static_cast<int>(s.pages.size()) > static_cast<int>(h->free_list.size()))
            throw std::runtime_error("out of blocks");
        while (static_cast<int>(s.pages.size()) < need) {
            s.pages.push_back(h->free_list.back());
            h->free_list.pop_back();
        }
        for (int i = 0; i < append_tokens; ++i) {
            const int t = s.num_tokens + i;
            slots_out[i] = s.pages[static_cast<size_t>(t / bs)] * bs + t % bs;
        }
        s.num_tokens += append_tokens;
    });
}

extern "C" int tq_block_table_num_tokens(const TQBlockTableHandle* h, int seq_id) {
    if (!h) return -1;
    std::lock_guard<std::mutex> lock(const_cast<TQBlockTableHandle*>(h)->mu);
    const auto it = h->seqs.find(seq_id);
    return it == h->seqs.end() ? 0 : it->second.num_tokens;
}

extern "C" int tq_block_table_pages(const TQBlockTableHandle* h, int seq_id, int32_t* pages_out,
                                    int max_pages) {
    if (!h || (!pages_out && max_pages > 0)) return -1;
    std::lock_guard<std::mutex> lock(const_cast<TQBlockTableHandle*>(h)->mu);
    const auto it = h->seqs.find(seq_id);
    if (it == h->seqs.end()) return 0;
    const int n = static_cast<int>(it->second.pages.size());
    if (n > max_pages) return -1;
    for (int i = 0; i < n; ++i) pages_out[i] = it->second.pages[static_cast<size_t>(i)];
    return n;
}

extern "C" int tq_block_table_release(TQBlockTableHandle* h, int seq_id) {
    if (!h) return -1;
    std::lock_guard<std::mutex> lock(h->mu);
    const auto it = h->seqs.find(seq_id);
    if (it == h->seqs.end()) return 0;
    for (auto pg = it->second.pages.rbegin(); pg != it->second.pages.rend(); ++pg)
        h->free_list.push_back(*pg);
    h->seqs.erase(it);
    return 0;
}
