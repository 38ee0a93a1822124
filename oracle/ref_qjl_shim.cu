// C entry points for the reference's QJL-1bit launchers.  TEST INFRASTRUCTURE ONLY.
//
// The reference compiles src/cuda/tq_qjl_kernels.cu and src/tq_qjl.cpp into its library but its
// C API (src/tq_capi.cpp) does not export them, so a ctypes client cannot reach them.  This file
// is compiled TOGETHER WITH the reference's unmodified sources into oracle/_ref/ (see the
// Makefile) and forwards to the reference's own C++ functions declared in include/tq_qjl.cuh;
// the symbol names are the ones this repository's library exports for the scheme, so the same
// test code drives both.
#include <stdexcept>

#include "tq_qjl.cuh"

extern "C" int tq_make_qjl_layout(const TQConfig* cfg, TQQJLPageLayout* out) {
    if (!cfg || !out) return -1;
    *out = make_tq_qjl_page_layout(*cfg);
    return 0;
}

extern "C" int tq_launch_qjl_pack_kv(const half* key, const half* value, const int32_t* slot_mapping,
                                     uint8_t* page_pool, const TQQJLPageLayout* layout, const TQConfig* cfg,
                                     int num_tokens, cudaStream_t stream) {
    if (!key || !value || !slot_mapping || !page_pool || !layout || !cfg) return -1;
    try {
        launch_tq_qjl_pack_kv(key, value, slot_mapping, page_pool, *layout, *cfg, num_tokens, stream);
    } catch (const std::exception&) {
        return -2;
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int tq_launch_qjl_dequant_kv(const uint8_t* page_pool, const int32_t* slot_mapping, half* out_key,
                                        half* out_value, const TQQJLPageLayout* layout, const TQConfig* cfg,
                                        int num_tokens, cudaStream_t stream) {
    if (!page_pool || !slot_mapping || !out_key || !out_value || !layout || !cfg) return -1;
    try {
        launch_tq_qjl_dequant_kv(page_pool, slot_mapping, out_key, out_value, *layout, *cfg, num_tokens, stream);
    } catch (const std::exception&) {
        return -2;
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int tq_launch_qjl_fused_attention_output(const half* query, const uint8_t* page_pool,
                                                    const int32_t* slot_mapping, half* output,
                                                    const TQQJLPageLayout* layout, const TQConfig* cfg,
                                                    int num_queries, int num_kv_tokens, cudaStream_t stream) {
    if (!query || !page_pool || !slot_mapping || !output || !layout || !cfg) return -1;
    try {
        launch_tq_qjl_fused_attention_output(query, page_pool, slot_mapping, output, *layout, *cfg, num_queries,
                                             num_kv_tokens, stream);
    } catch (const std::exception&) {
        return -2;
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
