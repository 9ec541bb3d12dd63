// Internal launch functions of liboxi_kv (one per kernel file).  Every function
// only enqueues work on `stream` and returns the launch's cudaError_t.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace oxi {

struct DecodeWorkspace {
    float* partial_acc;     // [max_batch][max_chunks][16][128]
    float* partial_stats;   // [max_batch][max_chunks][16][2]  (running max in log2 units, sum)
    uint32_t* status;       // device status word (OR of DEV_* bits)
    uint32_t* work_counter; // items claimed beyond the first per CTA; zero between launches
    float* merge_acc;       // decode_merge_scratch_bytes(): slice sums of rows longer than 16 key ranges (null: none)
    uint32_t* merge_count;  // [max_batch][4] arrival counters of the merge, zero between launches
    uint32_t max_chunks;    // partial slots per row
    uint32_t max_seq_len;
    int num_sms;
    WaitFault fault;        // test support (a stage of CTA 0 goes missing); zero on every normal launch
};

cudaError_t launch_append(cudaStream_t stream, void* q_io, const void* k_in, const void* v_in,
                          const void* q_norm_w, const void* k_norm_w, const void* cos_t,
                          const void* sin_t, const uint32_t* pos_ids, const uint64_t* k_ptrs,
                          const uint64_t* v_ptrs, uint32_t batch, float eps, uint32_t* status);
cudaError_t launch_advance_step(cudaStream_t stream, uint32_t* pos_ids, uint32_t* seq_lens, uint32_t batch,
                                uint32_t delta);
cudaError_t launch_len_from_pos(cudaStream_t stream, const uint32_t* pos_ids, uint32_t* seq_lens, uint32_t batch);
cudaError_t launch_qk_rmsnorm(cudaStream_t stream, void* x_io, const void* w, float eps,
                              uint32_t heads, uint32_t batch);
cudaError_t launch_rope(cudaStream_t stream, void* x_io, const void* cos_t, const void* sin_t,
                        const uint32_t* pos_ids, uint32_t heads, uint32_t batch);
cudaError_t launch_kv_copy(cudaStream_t stream, const uint64_t* dst_ptrs, const void* src,
                           const uint32_t* pos_ids, uint32_t batch, uint32_t* status);
cudaError_t launch_sigmoid_gate(cudaStream_t stream, void* ctx_io, const void* gate,
                                uint32_t batch);

cudaError_t decode_attn_init();  // one-time function attributes (dynamic shared memory)
cudaError_t launch_decode_attn(cudaStream_t stream, const DecodeWorkspace& ws, void* ctx_out,
                               const void* q, const void* gate, const uint64_t* k_ptrs,
                               const uint64_t* v_ptrs, const uint32_t* seq_lens, uint32_t batch,
                               uint32_t window);
// Fused RMSNorm + RoPE + KV append + gated decode attention (positions are seq_lens - 1).
cudaError_t launch_append_decode(cudaStream_t stream, const DecodeWorkspace& ws, void* ctx_out, const void* q_io,
                                 const void* k_in, const void* v_in, const void* gate, const void* q_norm_w,
                                 const void* k_norm_w, const void* cos_t, const void* sin_t,
                                 const uint32_t* seq_lens, const uint64_t* k_ptrs, const uint64_t* v_ptrs,
                                 uint32_t batch, uint32_t window, float eps);
uint32_t decode_chunk_keys();    // keys per split-KV work item
uint32_t decode_max_rows();      // rows one launch can take
size_t decode_merge_scratch_bytes(uint32_t max_batch, uint32_t max_chunks);

// A K/V slab registered for TMA loads in prefill attention: a tiled tensor map (128 bytes, opaque to
// everything but the driver and the TMA unit) over rows of 1024 bytes starting at `base`.
struct alignas(64) TmaDesc {
    uint64_t opaque[16];
};
struct PrefillSlab {
    TmaDesc map;     // 2-D f16 tensor {512 elements, rows}, box {64, 64}, 128-byte swizzle
    uint64_t base;   // device address of row 0
    uint32_t rows;   // 0: no slab registered
};

// Workspace of the key-range split of prefill attention (small waves of long prompts).
struct PrefillSplitWs {
    uint32_t* units;     // prefill_split_table_bytes(): unit, slot and block tables
    float* part;         // max_slots * prefill_split_slot_bytes(): partial O rows, then (max, sum) pairs
    uint32_t max_slots;  // 0: not reserved
};
cudaError_t prefill_attn_init();
cudaError_t launch_prefill_attn(cudaStream_t stream, void* ctx_out, const void* q,
                                const void* gate, const uint64_t* k_ptrs, const uint64_t* v_ptrs,
                                const uint32_t* seq_lens, uint32_t rows, uint32_t window,
                                uint32_t* status, int num_sms,
                                uint32_t* order /* [ceil(rows/32)] block order scratch */,
                                uint32_t* counter /* item claim counter */,
                                const PagedMap* pm = nullptr /* paged K/V: k_ptrs / v_ptrs unused */,
                                const uint32_t* row_seq = nullptr /* paged: table row of each wave row */,
                                const PrefillSplitWs* split = nullptr /* key-range split of small waves */,
                                uint32_t part_keys = 0 /* keys per part; 0: no split */,
                                const PrefillSlab* slab = nullptr /* K/V rows inside it are loaded by TMA */,
                                const WaitFault* fault = nullptr /* test support: a K tile of CTA 0 goes missing */);
size_t prefill_split_slot_bytes();   // partial-result bytes per slot of PrefillSplitWs::part
size_t prefill_split_table_bytes();  // bytes of PrefillSplitWs::units

cudaError_t launch_conv_decode(cudaStream_t stream, void* y_out, const uint64_t* conv_ptrs,
                               const void* bcx, const void* conv_w, uint32_t batch,
                               uint32_t* status);
cudaError_t launch_conv_prefill(cudaStream_t stream, void* y_out, const uint64_t* carry_ptrs,
                                const uint32_t* origin, const uint32_t* local_pos,
                                const void* bcx, const void* conv_w, uint32_t rows,
                                void* stage /* [rows][2048][6] f16 */, uint32_t* status);

// Paged K/V layout (block tables instead of one contiguous lease per sequence).
cudaError_t launch_append_paged(cudaStream_t stream, void* q_io, const void* k_in, const void* v_in,
                                const void* q_norm_w, const void* k_norm_w, const void* cos_t,
                                const void* sin_t, const uint32_t* pos_ids, const PagedMap& pm,
                                uint32_t batch, float eps, uint32_t* status);
cudaError_t launch_decode_attn_paged(cudaStream_t stream, const DecodeWorkspace& ws, void* ctx_out, const void* q,
                                     const void* gate, const PagedMap& pm, const uint32_t* seq_lens, uint32_t batch,
                                     uint32_t window);
cudaError_t launch_append_decode_paged(cudaStream_t stream, const DecodeWorkspace& ws, void* ctx_out, const void* q_io,
                                       const void* k_in, const void* v_in, const void* gate, const void* q_norm_w,
                                       const void* k_norm_w, const void* cos_t, const void* sin_t,
                                       const uint32_t* seq_lens, const PagedMap& pm, uint32_t batch, uint32_t window,
                                       float eps);

// Projection GEMM (tcgen05) with the append operator as its epilogue, and the same GEMM as a plain linear layer.
cudaError_t proj_gemm_init();
int proj_encode_map(TmaDesc* out, const void* base, uint64_t rows, uint32_t box_rows);  // tiled map over [rows][2048] f16; 0 = ok
// w_maps: tensor maps of the four weight matrices (q, k, v, gate), boxes of 128 rows
cudaError_t launch_project_append(cudaStream_t stream, const TmaDesc* w_maps, int num_sms, const void* x, uint32_t rows,
                                  void* q_out, void* gate_out, void* raw_out, const void* q_norm_w, const void* k_norm_w,
                                  const void* cos_t, const void* sin_t, const uint32_t* pos_ids, const uint64_t* k_ptrs,
                                  const uint64_t* v_ptrs, float eps, uint32_t* status, const WaitFault* fault);
// w_map: tensor map of the weight matrix, boxes of 128 rows
cudaError_t launch_linear(cudaStream_t stream, const TmaDesc* w_map, int num_sms, uint32_t out_features, const void* x,
                          uint32_t rows, void* y, uint32_t* status, const WaitFault* fault);

// Read-only streaming probe (bench and tests): the decode kernel's copy pipeline without arithmetic.
cudaError_t stream_probe_init();
cudaError_t launch_stream_read(cudaStream_t stream, const void* src, uint64_t bytes, uint32_t copy_bytes, int num_sms,
                               uint32_t* sink, uint32_t* status);
uint32_t stream_probe_stage_bytes();

// Sampling-side table kernels.
cudaError_t launch_embed_lookup(cudaStream_t stream, void* out, const void* table,
                                const uint32_t* token_ids, uint32_t hidden, uint32_t table_rows,
                                uint32_t batch, uint32_t* status);
cudaError_t launch_argmax(cudaStream_t stream, uint32_t* tokens_out, const void* logits, uint32_t vocab,
                          uint32_t batch, int num_sms,
                          void* cand_scratch /* [batch][argmax_max_splits()][256] (float, uint32) */,
                          uint32_t* counters /* [batch], zero between launches */);
uint32_t argmax_max_splits();

}  // namespace oxi
