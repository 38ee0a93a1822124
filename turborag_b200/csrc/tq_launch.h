// Host-side launch helpers shared by the kernel translation units and the C API.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <stdexcept>
#include <string>

#include "tq_common.cuh"

namespace tq {

// Throws std::runtime_error("<name>: <cuda error>") when the preceding launch
// was rejected (same contract as TQ_CHECK_LAUNCH, include/tq_cuda_check.h:18-24).
// With -DTQ_DEBUG_SYNC also synchronises the device and reports execution errors
// (include/tq_cuda_check.h:26-37).
void check_launch(const char* name);
void check_cuda(cudaError_t e, const char* what);
int sm_count();
// Stream-ordered scratch memory for calls that were not given a workspace.  It comes from a
// memory pool the library owns (one per device, created on first use) whose release threshold
// keeps up to 1 GiB cached across synchronisations: the driver's default pool returns its
// memory to the system at every synchronise, and the next call then pays milliseconds to map it
// again.  Nothing here touches the process-wide default pool.
void* scratch_alloc(size_t bytes, cudaStream_t stream, const char* what);
void scratch_free(void* p, cudaStream_t stream, const char* what);
// Stores a message for tq_last_error() of the calling thread.
void set_last_error(const char* msg);
// Page geometry from a TQTurboProdPageLayout* / TQTurbomsePageLayout* (throws on a layout that
// does not belong to head_dim 128).
PageGeom geom_from_layout(int scheme, const void* layout, const TQConfig& cfg);

void launch_pack(int scheme, const void* key, const void* value, const int32_t* slots,
                 uint8_t* pool, const PageGeom& geo, int head_dim, int num_tokens,
                 cudaStream_t stream);

// turbo_prod pack that also writes its intermediates (each [num_tokens, H, 128] or null), for parity
// triage; same pool bytes as launch_pack.
void launch_pack_debug(const void* key, const void* value, const int32_t* slots, uint8_t* pool,
                       const PageGeom& geo, int head_dim, int num_tokens, float* k_rot, float* v_rot, float* kn,
                       float* vn, int* kidx, int* vidx, cudaStream_t stream);

// hnd: write [H, N, D] instead of [N, H, D].
void launch_dequant(int scheme, const uint8_t* pool, const int32_t* slots, void* out_key,
                    void* out_value, const PageGeom& geo, int head_dim, int num_tokens, bool hnd,
                    cudaStream_t stream);

// Where the merged (acc, m, l) record of every row goes when the partials are published to the
// GPUs of an NVLink domain (see tq_peer.cu for the buffer layout); world == 0 turns it off.
struct PeerOut {
    float* records[8];
    unsigned int* flags[8];
    unsigned int* ticket;
    int world, rank, rows_cap;
    unsigned int exchange;
    // Optional: finish the exchange in the publishing kernel itself.  After a CTA has stored its rows'
    // records it waits (at most wait_ns) until every rank's flag in this rank's own buffer shows
    // `exchange`, merges the world records of its rows and writes fp16 final_out[row][128]; a wait that
    // runs out sets *status to 1.  Null final_out: the caller merges with tq_peer_merge.
    void* final_out;
    unsigned long long wait_ns;
    int* status;
};
// Bound of the peer flag waits (tq_peer_set_wait_ns) and the device address of the status word
// tq_peer_status reads, for launches outside tq_peer.cu that wait for peers.
unsigned long long peer_wait_ns();
int* peer_status_ptr();
// Stand-alone merge of the records that arrived in this rank's buffer (what tq_peer_merge launches).
void launch_peer_merge(const void* my_buffer, int world, int rows, int rows_cap, unsigned int exchange, void* output,
                       int num_q_heads, int num_kv_heads, int head_dim, cudaStream_t stream);

struct DecodeArgs {
    int scheme;                   // TQ_SCHEME_*
    const void* query;            // fp16
    const uint8_t* pool;
    const int32_t* slot_mapping;  // per-token slots (reference API) or nullptr
    const int32_t* block_tables;  // [batch, table_stride] or nullptr
    int table_stride;
    const int32_t* seq_lens;      // [batch] or nullptr (then every sequence has max_kv_tokens)
    void* output;                 // fp16 or nullptr
    float* partials_out;          // or nullptr
    float* logits_out;            // turbo_prod logits entry point, or nullptr
    PageGeom geo;
    int head_dim;
    int batch;
    int num_q_heads;              // query rows per sequence = groups * num_kv_heads
    int ref_query_layout;         // 1: query/output rows are [g][h] (reference), 0: [h*G+g]
    int max_kv_tokens;
    int kv_begin, kv_end;
    void* workspace;
    size_t workspace_bytes;
    PeerOut peer;                 // optional: publish the merged records to every peer
};
void launch_decode(const DecodeArgs& a, cudaStream_t stream);
int decode_num_splits(int batch, int max_kv_tokens, int num_kv_heads, int block_size);
size_t decode_workspace_bytes(int batch, int num_q_heads, int num_splits);
// head_sign: 1 when the rotation's sign pattern alternates with the kv head (turbo_prod,
// turbo_mse), 0 when it does not (QJL).
void launch_merge(const float* partials, int num_parts, void* output, float* partials_out,
                  int rows, int num_q_heads, int num_kv_heads, int ref_query_layout,
                  int head_dim, cudaStream_t stream, int head_sign = 1);

// Merge of split partials laid out [sequence][split][num_q_heads][130] (what the decode and
// prefill kernels write), rows = sequences * num_q_heads.
void launch_merge_splits(const float* partials, int splits, void* output, int rows, int num_q_heads,
                         int num_kv_heads, int head_dim, cudaStream_t stream);

// Chunk prefill over a turbo_mse prefix on the tcgen05 tensor cores: `nq` query tokens per sequence
// attend to the paged prefix and, causally, to their own fp16 chunk (chunk_key / chunk_value may be
// null: prefix only).  prefill_tc_status() returns the device status word of that kernel (0 = no
// bounded wait ever ran out; synchronises the device).
void launch_prefill_tc(const void* query, const uint8_t* pool, const int32_t* block_tables,
                       int table_stride, const int32_t* seq_lens, const void* chunk_key,
                       const void* chunk_value, void* output, const PageGeom& geo, int head_dim,
                       int batch, int nq, int hq, int max_prefix_tokens, cudaStream_t stream);
int prefill_tc_status();

}  // namespace tq
