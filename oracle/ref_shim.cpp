// C shim over the reference's own host code, compiled together with the
// reference sources where they lie (see Makefile, target `ref`).  TEST
// INFRASTRUCTURE ONLY.  Exposes attention_ref_single_head
// (src/tq_attention_ref.cpp:10-56) and the two page-layout builders
// (src/tq_turbo_prod.cpp:7-39, src/tq_turbo_mse_layout.cpp:7-28) through a C
// ABI so the oracle restatement can be checked against them.
#include <cstdint>
#include <cstring>
#include <vector>

#include "tq_attention_ref.h"
#include "tq_turbo_mse_layout.h"
#include "tq_turbo_prod.cuh"

extern "C" int ref_attention_single_head(const uint16_t* q, const uint16_t* k,
                                         const uint16_t* v, int n, int d,
                                         float* out) {
    try {
        std::vector<half> qv(d), kv((size_t)n * d), vv((size_t)n * d);
        std::memcpy(qv.data(), q, sizeof(half) * d);
        std::memcpy(kv.data(), k, sizeof(half) * (size_t)n * d);
        std::memcpy(vv.data(), v, sizeof(half) * (size_t)n * d);
        std::vector<float> o = attention_ref_single_head(qv, kv, vv, n, d);
        std::memcpy(out, o.data(), sizeof(float) * d);
        return 0;
    } catch (...) {
        return -1;
    }
}

extern "C" void ref_prod_layout(const TQConfig* cfg, TQTurboProdPageLayout* out) {
    *out = make_tq_turbo_prod_page_layout(*cfg);
}

extern "C" void ref_mse_layout(const TQConfig* cfg, TQTurbomsePageLayout* out) {
    *out = make_tq_turbo_mse_page_layout(*cfg);
}

extern "C" void ref_default_config(TQConfig* cfg) { *cfg = TQConfig{}; }
