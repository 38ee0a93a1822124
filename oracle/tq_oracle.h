/*
 * CPU oracle for the TurboCAG compressed-KV hot path.  TEST INFRASTRUCTURE ONLY:
 * it is linked or loaded by the test-suite, by the smoke check and by the
 * CPU-baseline leg of the benchmark, never by the shipped library.
 *
 * Every function restates, in plain C, the arithmetic of one reference CUDA
 * kernel (the reference has no host quantiser of its own).  Citations are
 * relative to the reference project root.
 *
 * Parity status: pinned.  The restatement is checked against fixtures under
 * tests/golden/ that were produced by running the reference's own kernels
 * (compiled unmodified for sm_100) on a B200; see tests/golden/make_golden.py.
 */
#ifndef TQ_ORACLE_H
#define TQ_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* include/tq_config.h:4-13 — eight 32-bit ints. */
typedef struct {
    int block_size, num_kv_heads, head_dim, nbits, group_size, page_alignment,
        scale_type, quant_mode;
} OrcConfig;

/* include/tq_turbo_prod.cuh:15-28 */
typedef struct {
    size_t page_size_bytes, k4_codes_offset, k_residual_scales_offset,
        k_scales_offset, v4_codes_offset, v_scales_offset;
    int k4_bytes_per_token_head, v4_bytes_per_token_head,
        scale_bytes_per_token_head;
} OrcProdLayout;

/* include/tq_turbo_mse_layout.h:5-15 */
typedef struct {
    size_t code_bytes_per_token_head, norm_bytes_per_token_head, k_codes_offset,
        v_codes_offset, k_norms_offset, v_norms_offset, page_size_bytes;
} OrcMseLayout;

/* include/tq_qjl.cuh:22-35 */
typedef struct {
    size_t page_size_bytes, k1_codes_offset, k_scales_offset, v4_codes_offset,
        v_scales_offset;
    int k1_bytes_per_token_head, v4_bytes_per_token_head,
        scale_bytes_per_token_head;
} OrcQjlLayout;

void orc_default_config(OrcConfig* cfg);
void orc_qjl_layout(const OrcConfig* cfg, OrcQjlLayout* out);
void orc_prod_layout(const OrcConfig* cfg, OrcProdLayout* out);
void orc_mse_layout(const OrcConfig* cfg, OrcMseLayout* out);

/* Bit pattern of the fp32 constant the kernels multiply by after the
 * butterflies (the value rsqrtf(128.f) takes on the GPU). */
uint32_t orc_inv_sqrt_d_bits(void);
void orc_set_inv_sqrt_d_bits(uint32_t bits);
/* Selects how a*a+b*b is contracted in the turbo_mse RMS (0: two products and
 * an add, 1: fma(a,a,b*b), 2: fma(b,b,a*a)). */
void orc_set_mse_pair_fma(int mode);
void orc_set_threads(int n);

float orc_sign_flip(int idx, int head);
void orc_fwht128(float* x, int d);
int orc_nearest_k3(float x);
int orc_nearest_v4(float x);
const float* orc_cb3(void);
const float* orc_cb4(void);
float orc_h2f(uint16_t h);
uint16_t orc_f2h(float f);

/* turbo_prod: src/cuda/tq_turbo_prod_kernels.cu */
void orc_prod_pack(const uint16_t* key, const uint16_t* value,
                   const int32_t* slots, uint8_t* pool,
                   const OrcProdLayout* lay, const OrcConfig* cfg, int n,
                   float* dbg_kn, float* dbg_vn);
void orc_prod_dequant(const uint8_t* pool, const int32_t* slots,
                      uint16_t* out_key, uint16_t* out_value,
                      const OrcProdLayout* lay, const OrcConfig* cfg, int n);
void orc_prod_logits(const uint16_t* query, const uint8_t* pool,
                     const int32_t* slots, float* logits,
                     const OrcProdLayout* lay, const OrcConfig* cfg, int nq,
                     int nkv);
void orc_prod_attn(const uint16_t* query, const uint8_t* pool,
                   const int32_t* slots, uint16_t* out,
                   const OrcProdLayout* lay, const OrcConfig* cfg, int nq,
                   int nkv);
/* Same arithmetic, fp32 rotated-domain partials (o[D], m, l) before the final
 * normalise / inverse rotation; used to check split-KV partials. */
void orc_prod_attn_f32(const uint16_t* query, const uint8_t* pool,
                       const int32_t* slots, float* out_f32,
                       const OrcProdLayout* lay, const OrcConfig* cfg, int nq,
                       int nkv);

/* turbo_mse: src/cuda/tq_turbo_mse_kernels.cu */
void orc_mse_pack(const uint16_t* key, const uint16_t* value,
                  const int32_t* slots, uint8_t* pool, const OrcMseLayout* lay,
                  const OrcConfig* cfg, int n, float* dbg_kn, float* dbg_vn);
void orc_mse_dequant(const uint8_t* pool, const int32_t* slots,
                     uint16_t* out_key, uint16_t* out_value,
                     const OrcMseLayout* lay, const OrcConfig* cfg, int n);
void orc_mse_attn(const uint16_t* query, const uint8_t* pool,
                  const int32_t* slots, uint16_t* out, const OrcMseLayout* lay,
                  const OrcConfig* cfg, int nq, int nkv);
void orc_mse_attn_f32(const uint16_t* query, const uint8_t* pool,
                      const int32_t* slots, float* out_f32,
                      const OrcMseLayout* lay, const OrcConfig* cfg, int nq,
                      int nkv);

/* Batched paged GQA decode (scheme 0 = turbo_prod, 1 = turbo_mse). */
void orc_decode_paged(int scheme, const uint16_t* query, const uint8_t* pool,
                      const int32_t* tables, int table_stride,
                      const int32_t* seq_lens, uint16_t* out, const void* lay,
                      const OrcConfig* cfg, int batch, int hq);

/* src/tq_attention_ref.cpp:10-56 — dense fp32 attention for one head. */
int orc_attention_ref_single_head(const uint16_t* q, const uint16_t* k_all,
                                  const uint16_t* v_all, int num_tokens,
                                  int head_dim, float* out);

/* Chunked query prefill over a turbo_mse prefix followed by a causal fp16
 * chunk (extension; arithmetic = restated dequant + dense fp32 softmax).
 * query [nq, hq, d] fp16, chunk_k/chunk_v [nq, h, d] fp16 (may be NULL),
 * out [nq, hq, d] fp32. Query head j uses kv head j / (hq / h). */
/* The same for the listed query rows only (rows[r] = index of the row inside the chunk, which
 * decides how much of the chunk it sees); out is [nrows, hq, head_dim].  rows == NULL: rows 0..nrows-1. */
void orc_mse_prefill_rows(const uint16_t* query, const uint8_t* pool,
                          const int32_t* slots, int nkv, const uint16_t* chunk_k,
                          const uint16_t* chunk_v, int nq, int hq, const int32_t* rows,
                          int nrows, float* out, const OrcMseLayout* lay,
                          const OrcConfig* cfg);
void orc_mse_prefill(const uint16_t* query, const uint8_t* pool,
                     const int32_t* slots, int nkv, const uint16_t* chunk_k,
                     const uint16_t* chunk_v, int nq, int hq, float* out,
                     const OrcMseLayout* lay, const OrcConfig* cfg);

/* src/tq_block_table.cpp:24-39 — slot = physical_block*block_size + t. */
void orc_build_slot_map(const int32_t* blocks, int num_tokens_before,
                        int append_tokens, int block_size, int32_t* slots);

/* QJL-1bit (src/cuda/tq_qjl_kernels.cu): pack :69-170, dequant :172-244, fused
 * attention :256-373 (logits <q', k'> without 1/sqrt(D)). */
void orc_qjl_pack(const uint16_t* key, const uint16_t* value,
                  const int32_t* slots, uint8_t* pool, const OrcQjlLayout* lay,
                  const OrcConfig* cfg, int n, float* dbg_kn, float* dbg_vn);
void orc_qjl_dequant(const uint8_t* pool, const int32_t* slots,
                     uint16_t* out_key, uint16_t* out_value,
                     const OrcQjlLayout* lay, const OrcConfig* cfg, int n);
void orc_qjl_attn(const uint16_t* query, const uint8_t* pool,
                  const int32_t* slots, uint16_t* out, const OrcQjlLayout* lay,
                  const OrcConfig* cfg, int nq, int nkv);
void orc_qjl_attn_f32(const uint16_t* query, const uint8_t* pool,
                      const int32_t* slots, float* out_f32,
                      const OrcQjlLayout* lay, const OrcConfig* cfg, int nq,
                      int nkv);

#ifdef __cplusplus
}
#endif
#endif
