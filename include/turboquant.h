/*
 * libturboquant — C ABI of the B200 (sm_100a) compressed-KV library.
 *
 * Part 1 re-exports, with identical names, argument order, struct layouts and
 * return codes, the `extern "C"` surface of the reference project
 * (src/tq_capi.cpp), so its ctypes bindings (tq_backend/turboquant_wrapper.py)
 * load this library unchanged.  Part 2 adds entry points the reference does
 * not have (batched paged GQA decode, split-KV partials and their merge,
 * [H,N,D] dequant, chunk prefill, host page allocator / block table).
 *
 * Conventions (all from the reference):
 *   return 0 ok, -1 null/invalid argument, -2 CUDA or shape error with the
 *   text available from tq_last_error() (thread-local).
 *   Every pointer except structs is DEVICE memory owned by the caller.
 *   Launches are asynchronous on `stream`; the library never synchronises.
 *   key/value/out_key/out_value: fp16 [num_tokens, num_kv_heads, head_dim].
 *   slot_mapping: int32 [num_tokens]; slot = physical_block*block_size + t.
 *   query/output: fp16 [num_queries, num_kv_heads, head_dim] — one query row
 *   per KV head (GQA group member g of kv-head h is row g).
 * Supported shapes: head_dim == 128, block_size >= 1, any num_kv_heads >= 1 (attention serves
 * layouts with more than 8 kv heads by one launch per group of 8 heads; tq_mse_prefill_paged and
 * tq_decode_paged_static take 1..8 kv heads).
 */
#ifndef TURBOQUANT_H
#define TURBOQUANT_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* tq_stream_t; /* cudaStream_t */
typedef uint16_t tq_half;  /* IEEE binary16 bits (`half` in the reference) */

/* include/tq_config.h:4-13 (32 bytes) */
typedef struct TQConfig {
    int block_size;     /* 16 */
    int num_kv_heads;   /* 8 */
    int head_dim;       /* 128 */
    int nbits;          /* 4 */
    int group_size;     /* 128 */
    int page_alignment; /* 256 */
    int scale_type;     /* TQScaleType::FP16 = 0 */
    int quant_mode;     /* TQQuantMode::MSE_INT4 = 0 */
} TQConfig;

/* include/tq_turbo_prod.cuh:15-28 (64 bytes) */
typedef struct TQTurboProdPageLayout {
    size_t page_size_bytes;
    size_t k4_codes_offset;
    size_t k_residual_scales_offset;
    size_t k_scales_offset;
    size_t v4_codes_offset;
    size_t v_scales_offset;
    int k4_bytes_per_token_head;
    int v4_bytes_per_token_head;
    int scale_bytes_per_token_head;
} TQTurboProdPageLayout;

/* include/tq_turbo_mse_layout.h:5-15 (56 bytes) */
typedef struct TQTurbomsePageLayout {
    size_t code_bytes_per_token_head;
    size_t norm_bytes_per_token_head;
    size_t k_codes_offset;
    size_t v_codes_offset;
    size_t k_norms_offset;
    size_t v_norms_offset;
    size_t page_size_bytes;
} TQTurbomsePageLayout;

/* include/tq_qjl.cuh:22-35 (48 bytes).  The QJL-1bit scheme is compiled into the reference
 * library but not exported through its C API; the entry points below give it one. */
typedef struct TQQJLPageLayout {
    size_t page_size_bytes;
    size_t k1_codes_offset; /* 1 sign bit per dimension */
    size_t k_scales_offset; /* fp16 RMS per token-head */
    size_t v4_codes_offset; /* 4-bit codes, the turbo_prod V codebook */
    size_t v_scales_offset;
    int k1_bytes_per_token_head;
    int v4_bytes_per_token_head;
    int scale_bytes_per_token_head;
} TQQJLPageLayout;

/* ------------------------------------------------------------------------ */
/* Part 1 — the reference surface                                           */
/* ------------------------------------------------------------------------ */

/* src/tq_capi.cpp:17-19 */
const char* tq_last_error(void);
/* src/tq_capi.cpp:35-39 */
int tq_make_default_config(TQConfig* out_cfg);
/* src/tq_capi.cpp:41-47 -> src/tq_turbo_prod.cpp:7-39 */
int tq_make_turbo_prod_layout(const TQConfig* cfg, TQTurboProdPageLayout* out_layout);
/* src/tq_capi.cpp:118-124 -> src/tq_turbo_mse_layout.cpp:7-28 */
int tq_make_turbo_mse_layout(const TQConfig* cfg, TQTurbomsePageLayout* out_layout);

/* src/tq_capi.cpp:49-64 -> src/cuda/tq_turbo_prod_kernels.cu:110-260 */
int tq_launch_turbo_prod_pack_kv(const tq_half* key, const tq_half* value,
                                 const int32_t* slot_mapping, uint8_t* page_pool,
                                 const TQTurboProdPageLayout* layout, const TQConfig* cfg,
                                 int num_tokens, tq_stream_t stream);
/* src/tq_capi.cpp:66-80 -> tq_turbo_prod_kernels.cu:265-341 */
int tq_launch_turbo_prod_dequant_kv(const uint8_t* page_pool, const int32_t* slot_mapping,
                                    tq_half* out_key, tq_half* out_value,
                                    const TQTurboProdPageLayout* layout, const TQConfig* cfg,
                                    int num_tokens, tq_stream_t stream);
/* src/tq_capi.cpp:82-97 -> tq_turbo_prod_kernels.cu:346-434; logits fp32
 * [(q*H + h)*num_kv_tokens + t], scaled by 1/sqrt(head_dim). */
int tq_launch_turbo_prod_fused_attention_logits(const tq_half* query, const uint8_t* page_pool,
                                                const int32_t* slot_mapping, float* logits,
                                                const TQTurboProdPageLayout* layout,
                                                const TQConfig* cfg, int num_queries,
                                                int num_kv_tokens, tq_stream_t stream);
/* src/tq_capi.cpp:99-114 -> tq_turbo_prod_kernels.cu:439-571 */
int tq_launch_turbo_prod_fused_attention_output(const tq_half* query, const uint8_t* page_pool,
                                                const int32_t* slot_mapping, tq_half* output,
                                                const TQTurboProdPageLayout* layout,
                                                const TQConfig* cfg, int num_queries,
                                                int num_kv_tokens, tq_stream_t stream);
/* src/tq_capi.cpp:126-141 -> src/cuda/tq_turbo_mse_kernels.cu:186-237 */
int tq_launch_turbo_mse_pack_kv(const tq_half* key, const tq_half* value,
                                const int32_t* slot_mapping, uint8_t* page_pool,
                                const TQTurbomsePageLayout* layout, const TQConfig* cfg,
                                int num_tokens, tq_stream_t stream);
/* src/tq_capi.cpp:143-157 -> tq_turbo_mse_kernels.cu:239-287 */
int tq_launch_turbo_mse_dequant_kv(const uint8_t* page_pool, const int32_t* slot_mapping,
                                   tq_half* out_key, tq_half* out_value,
                                   const TQTurbomsePageLayout* layout, const TQConfig* cfg,
                                   int num_tokens, tq_stream_t stream);
/* src/tq_capi.cpp:159-174 -> tq_turbo_mse_kernels.cu:302-417 */
int tq_launch_turbo_mse_fused_attention_output(const tq_half* query, const uint8_t* page_pool,
                                               const int32_t* slot_mapping, tq_half* output,
                                               const TQTurbomsePageLayout* layout,
                                               const TQConfig* cfg, int num_queries,
                                               int num_kv_tokens, tq_stream_t stream);

/* ------------------------------------------------------------------------ */
/* Part 2 — additions (no counterpart in the reference's C API)             */
/* ------------------------------------------------------------------------ */

#define TQ_SCHEME_TURBO_PROD 0
#define TQ_SCHEME_TURBO_MSE 1
#define TQ_SCHEME_QJL 2 /* layout argument: TQQJLPageLayout*; logits are <q', k'> without 1/sqrt(head_dim) */

/* QJL-1bit: K = sign bit per rotated dimension + fp16 RMS (18 bytes per token-head at head_dim
 * 128), V = 4-bit codes + fp16 RMS (66 bytes); the rotation's sign pattern has no per-head
 * term and the attention logits are not scaled by 1/sqrt(head_dim).  Same argument meaning as
 * the turbo_prod entry points.
 * src/tq_qjl.cpp:7-34 (layout), src/cuda/tq_qjl_kernels.cu:69-170 (pack), :172-244 (dequant),
 * :256-373 (fused attention), launchers :380-438. */
int tq_make_qjl_layout(const TQConfig* cfg, TQQJLPageLayout* out_layout);
int tq_launch_qjl_pack_kv(const tq_half* key, const tq_half* value, const int32_t* slot_mapping,
                          uint8_t* page_pool, const TQQJLPageLayout* layout, const TQConfig* cfg,
                          int num_tokens, tq_stream_t stream);
int tq_launch_qjl_dequant_kv(const uint8_t* page_pool, const int32_t* slot_mapping, tq_half* out_key,
                             tq_half* out_value, const TQQJLPageLayout* layout, const TQConfig* cfg,
                             int num_tokens, tq_stream_t stream);
int tq_launch_qjl_fused_attention_output(const tq_half* query, const uint8_t* page_pool,
                                         const int32_t* slot_mapping, tq_half* output,
                                         const TQQJLPageLayout* layout, const TQConfig* cfg,
                                         int num_queries, int num_kv_tokens, tq_stream_t stream);

/* Floats per (sequence, query head) in a split-KV partial: the rotated-domain
 * unnormalised accumulator acc[128], then the softmax reference m (natural-log
 * logit units) and the denominator l: acc = sum_t exp(logit_t - m) v_t,
 * l = sum_t exp(logit_t - m).  Same triple the reference's fused kernel
 * carries in sh_m / sh_l / vaccum (tq_turbo_prod_kernels.cu:463-470), except
 * that m is only guaranteed to lie within 1.5 ln 2 below the largest logit, not
 * to equal it; m + log(l) and acc / l do not depend on that choice, and they
 * are all a merge uses. */
#define TQ_PARTIAL_STRIDE 130

/* Number of KV splits the decode kernels use for `batch` sequences of at most
 * `max_kv_tokens` tokens on the current device, and the scratch bytes a call
 * needs (partials for every split). */
int tq_decode_num_splits(int batch, int max_kv_tokens, int num_kv_heads, int block_size);
size_t tq_decode_workspace_bytes(int batch, int num_q_heads, int num_splits);

/* Batched paged GQA decode over compressed pages (generalises
 * tq_turbo_prod_kernels.cu:439-571 / tq_turbo_mse_kernels.cu:302-417 to many
 * sequences, block tables and grouped query heads).
 *   query/output : fp16 [batch, num_q_heads, 128]; query head j reads kv head
 *                  j / (num_q_heads / num_kv_heads).
 *   block_tables : int32 [batch, table_stride]; token t of sequence b lives in
 *                  slot block_tables[b][t / block_size]*block_size + t % block_size
 *                  (src/tq_block_table.cpp:24-39).
 *   seq_lens     : int32 [batch] cached tokens per sequence (0 allowed: zeros out).
 *   kv_begin/kv_end : token range of every sequence this call attends to
 *                  (clamped to seq_lens; pass 0 and INT32_MAX for all).
 *   workspace    : device scratch of tq_decode_workspace_bytes(...) bytes, or
 *                  NULL to use a per-device cache the library grows on demand.
 *   partials_out : if non-NULL, fp32 [batch, num_q_heads, TQ_PARTIAL_STRIDE]
 *                  receives the merged (acc, m, l) of this call's range and
 *                  `output` may be NULL (used for multi-GPU KV splits).
 * `layout` is a TQTurboProdPageLayout* or TQTurbomsePageLayout* per `scheme`. */
int tq_decode_paged(int scheme, const tq_half* query, const uint8_t* page_pool,
                    const int32_t* block_tables, int table_stride, const int32_t* seq_lens,
                    tq_half* output, float* partials_out, const void* layout,
                    const TQConfig* cfg, int batch, int num_q_heads, int max_kv_tokens,
                    int kv_begin, int kv_end, void* workspace, size_t workspace_bytes,
                    tq_stream_t stream);

/* Has no counterpart in the reference.  tq_decode_paged for callers that must not allocate
 * device memory: a serving engine that gave the whole GPU to its own memory pool when it
 * started, or a latency-critical loop that cannot risk the synchronisation an allocation may
 * bring.  Same inputs, outputs and results as
 * tq_decode_paged(..., workspace = NULL) over the whole sequence, but the split-KV scratch is
 * a fixed array inside the library (TQ_DECODE_STATIC_SCRATCH_BYTES per GPU, held from the
 * moment the library is loaded on that GPU until the process ends) and the call performs no
 * cudaMalloc / cudaFree / stream-ordered allocation.
 *   - A shape whose scratch need, tq_decode_workspace_bytes(batch, num_q_heads,
 *     tq_decode_num_splits(batch * ceil(group/8), max_kv_tokens, ..)), exceeds the array is
 *     rejected with -2 and a message; use tq_decode_paged with your own workspace then.
 *   - The first call on each device looks up the array's device address; make that call
 *     before starting any stream capture on the device.
 *   - Every call on a device uses the same array (it keeps the previous call's bytes; no
 *     part needs clearing, each call rewrites all it reads).  Calls whose kernels may run at
 *     the same time on one GPU race on it: issue them on one stream or order them yourself. */
#define TQ_DECODE_STATIC_SCRATCH_BYTES (8u << 20)
int tq_decode_paged_static(int scheme, const tq_half* query, const uint8_t* page_pool,
                           const int32_t* block_tables, int table_stride,
                           const int32_t* seq_lens, tq_half* output, const void* layout,
                           const TQConfig* cfg, int batch, int num_q_heads, int max_kv_tokens,
                           tq_stream_t stream);

/* Log-sum-exp merge of `num_parts` partial sets laid out
 * [num_parts, rows, TQ_PARTIAL_STRIDE] (e.g. an all-gather over ranks), then
 * normalise, inverse rotation and fp16 store: output [rows, 128] with
 * rows = batch*num_q_heads.  Query head of row r is r % num_q_heads. */
int tq_merge_partials(const float* partials, int num_parts, tq_half* output, int rows,
                      int num_q_heads, int num_kv_heads, tq_stream_t stream);

/* turbo_prod quantize+pack that also writes the kernel's intermediates, for parity triage: the
 * debug_* arguments of the reference's pack kernel (src/cuda/tq_turbo_prod_kernels.cu:119-124,
 * 216-217, 243-246), which its C API always passes as null (src/tq_capi.cpp:59-62).  Each is device
 * memory [num_tokens, num_kv_heads, 128] or NULL: rotated K / V, the clamped normalised values
 * (+-2.5 / +-2.75), the 3-bit K and 4-bit V level indices.  The pool receives the same bytes as from
 * tq_launch_turbo_prod_pack_kv. */
int tq_debug_turbo_prod_pack_kv(const tq_half* key, const tq_half* value, const int32_t* slot_mapping,
                                uint8_t* page_pool, const TQTurboProdPageLayout* layout,
                                const TQConfig* cfg, int num_tokens, float* debug_k_rot,
                                float* debug_v_rot, float* debug_kn, float* debug_vn, int* debug_kidx,
                                int* debug_vidx, tq_stream_t stream);

/* Dequant straight into the [num_kv_heads, num_tokens, 128] layout a Hugging
 * Face cache wants (fuses the permute().contiguous() of
 * tq_backend/cag_store.py:250-251). */
int tq_dequant_kv_hnd(int scheme, const uint8_t* page_pool, const int32_t* slot_mapping,
                      tq_half* out_key, tq_half* out_value, const void* layout,
                      const TQConfig* cfg, int num_tokens, tq_stream_t stream);

/* Chunked query prefill over a turbo_mse prefix plus an optional causal fp16
 * chunk.  query/output fp16 [batch, num_q_tokens, num_q_heads, 128];
 * chunk_key/chunk_value fp16 [batch, num_q_tokens, num_kv_heads, 128] or NULL. */
int tq_mse_prefill_paged(const tq_half* query, const uint8_t* page_pool,
                         const int32_t* block_tables, int table_stride,
                         const int32_t* seq_lens, const tq_half* chunk_key,
                         const tq_half* chunk_value, tq_half* output,
                         const TQTurbomsePageLayout* layout, const TQConfig* cfg, int batch,
                         int num_q_tokens, int num_q_heads, tq_stream_t stream);
/* Status word of the prefill kernel on the current device (synchronises it): 0 when no bounded
 * wait inside the kernel ever ran out, else the code of the wait that did (results of that
 * launch are then undefined); negative on a CUDA error.  No reference counterpart. */
int tq_mse_prefill_status(void);

/* Exchange of split-KV partials between the GPUs of one NVLink domain by plain peer stores (no
 * collective library call).  No reference counterpart (the reference is single-GPU).
 * Every rank owns one buffer of tq_peer_buffer_bytes(world, rows_cap) bytes, zero-initialised
 * once, mapped into every peer (CUDA IPC or symmetric memory; the host side does that).
 * Per exchange (numbered 1, 2, 3, ... identically on all ranks):
 *   tq_peer_publish: stores this rank's records local_partials[rows][130] into slot `rank` of
 *     every buffer in peer_buffers[world] (device pointers valid on this GPU, own buffer
 *     included) and raises this rank's flag there;
 *   tq_peer_merge: waits (at most 2 s) until every rank's flag in my_buffer shows `exchange`, then
 *     merges the world records per row (log-sum-exp), normalises, applies the inverse rotation and
 *     writes fp16 output[rows][128]; rows = sequences * num_q_heads, rows ordered (sequence, q head).
 * tq_peer_status(): 0, or 1 if a wait ever ran out on the current device (synchronises);
 * tq_peer_clear_status() sets it back to 0.  tq_peer_set_wait_ns(ns) changes the bound of the waits of
 * later tq_peer_merge calls of this process (0 = back to the default 2 s); a wait that runs out makes
 * the kernel give up on the missing records and finish, the context stays usable.
 * tq_decode_paged_publish = tq_decode_paged restricted to [kv_begin, kv_end) whose split merge
 * writes the records straight into the peers' buffers (decode + publish in two launches). */
size_t tq_peer_buffer_bytes(int world, int rows_cap);
int tq_decode_paged_publish(int scheme, const tq_half* query, const uint8_t* page_pool,
                            const int32_t* block_tables, int table_stride, const int32_t* seq_lens,
                            const void* layout, const TQConfig* cfg, int batch, int num_q_heads,
                            int max_kv_tokens, int kv_begin, int kv_end, void* workspace,
                            size_t workspace_bytes, void* const* peer_buffers, int rank, int world,
                            int rows_cap, unsigned int exchange, tq_stream_t stream);
/* tq_decode_paged_publish followed by tq_peer_merge as one call: this rank's token range is decoded,
 * its records are stored into every peer's buffer, and output[rows][128] receives the merge of all
 * ranks' records.  With at most 4 x (SM count) rows the publishing kernel waits for the peers' flags
 * itself and finishes the merge (two launches per call instead of three); with more rows the
 * stand-alone merge is launched behind it. */
int tq_decode_paged_exchange(int scheme, const tq_half* query, const uint8_t* page_pool,
                             const int32_t* block_tables, int table_stride, const int32_t* seq_lens,
                             const void* layout, const TQConfig* cfg, int batch, int num_q_heads,
                             int max_kv_tokens, int kv_begin, int kv_end, void* workspace,
                             size_t workspace_bytes, void* const* peer_buffers, int rank, int world,
                             int rows_cap, unsigned int exchange, tq_half* output, tq_stream_t stream);
int tq_peer_publish(const float* local_partials, void* const* peer_buffers, int rank, int world,
                    int rows, int rows_cap, unsigned int exchange, tq_stream_t stream);
int tq_peer_merge(const void* my_buffer, int world, int rows, int rows_cap, unsigned int exchange,
                  tq_half* output, int num_q_heads, int num_kv_heads, int head_dim, tq_stream_t stream);
int tq_peer_status(void);
int tq_peer_clear_status(void);
int tq_peer_set_wait_ns(unsigned long long ns);

/* Host-side page allocator and block table (LIFO free list and the slot
 * formula of src/tq_allocator.cpp:5-31, src/tq_block_table.cpp:7-39; the pool
 * memory itself stays with the caller). */
typedef struct TQBlockTableHandle TQBlockTableHandle;
TQBlockTableHandle* tq_block_table_create(int num_pages, int block_size);
void tq_block_table_destroy(TQBlockTableHandle* h);
int tq_block_table_free_pages(const TQBlockTableHandle* h);
/* Appends `append_tokens` to sequence `seq_id`, allocating pages as needed,
 * and writes their slots to slots_out[append_tokens] (host). -2 "out of blocks". */
int tq_block_table_append(TQBlockTableHandle* h, int seq_id, int append_tokens,
                          int32_t* slots_out);
int tq_block_table_num_tokens(const TQBlockTableHandle* h, int seq_id);
/* Copies the sequence's page ids to pages_out (host, capacity max_pages);
 * returns the page count or -1. */
int tq_block_table_pages(const TQBlockTableHandle* h, int seq_id, int32_t* pages_out,
                         int max_pages);
int tq_block_table_release(TQBlockTableHandle* h, int seq_id);

#ifdef __cplusplus
}
#endif
#endif /* TURBOQUANT_H */
