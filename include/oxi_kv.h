/*
 * liboxi_kv — B200 (sm_100a) kernels for the pointer-table KV-cache path of
 * oxide-infer's batched engine, behind a C ABI.
 *
 * The reference has no C ABI of its own on this path: its Rust engine calls
 * cuda_core::launch_kernel_on_stream() on PTX entry points looked up by name
 * (crates/oxide-infer-kernels/src/ptx.rs:13-26,
 *  crates/oxide-infer-server/src/batch_engine.rs:387-404).  Every function
 * below therefore cites the PTX entry point(s) and the engine launch site it
 * replaces; a Rust `extern "C"` block binding these symbols is the only change
 * the engine needs.
 *
 * Conventions (same as the reference's launch sites):
 *   - every tensor argument is a DEVICE pointer owned by the caller; fp16
 *     storage, fp32 arithmetic; geometry is LFM's: 16 query heads, 4 KV heads,
 *     head_dim 128, conv hidden 2048 with 7 taps (6 live state slots);
 *   - k_ptrs / v_ptrs / conv_ptrs are device arrays of per-sequence device
 *     pointers, already offset to the layer (batch_engine.rs:709-740);
 *     each K or V cache is row-major [token][kv_head 4][128] f16 (1024 B per
 *     token) and must be 16-byte aligned;
 *   - seq_lens[b] counts the token appended in this step
 *     (batch_engine.rs:689-691), pos_ids[b] = seq_lens[b] - 1;
 *   - `stream` is the caller's CUstream / cudaStream_t; calls only enqueue
 *     work, never synchronise and never allocate after oxi_create();
 *   - return value: 0 = ok, negative = OXI_ERR_* argument error detected on the
 *     host before anything was enqueued, positive = cudaError_t passed through.
 *     No exceptions cross the ABI and nothing aborts.
 *   - a handle may be used by one thread at a time (the reference drives the
 *     path from one worker thread owning one stream, server.rs:319-321).
 */
#ifndef OXI_KV_H
#define OXI_KV_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OXI_VERSION 100 /* major*10000 + minor*100 + patch */

enum {
    OXI_OK = 0,
    OXI_ERR_NULL = -1,      /* a required pointer (or the handle) is null   */
    OXI_ERR_BATCH = -2,     /* batch/rows is 0 or exceeds the handle limit  */
    OXI_ERR_ARG = -3,       /* a scalar argument is out of range            */
    OXI_ERR_WORKSPACE = -4, /* the handle's workspace cannot hold the call  */
    OXI_ERR_NO_DEVICE = -5  /* no usable CUDA device / wrong architecture   */
};

/* Bits of the device-side status word (oxi_device_status). */
enum {
    OXI_DEV_MISALIGNED_PTR = 1u, /* a K/V/state pointer was not 16-byte aligned; row skipped */
    OXI_DEV_BAD_SEQ_LEN = 2u,    /* seq_len 0 or beyond the handle's max_seq_len; row skipped */
    OXI_DEV_WAIT_TIMEOUT = 4u,   /* an in-kernel pipeline wait gave up (internal error)       */
    OXI_DEV_BAD_TOKEN = 8u,      /* a token id was beyond the embedding table; row zero-filled */
    OXI_DEV_BAD_BLOCK = 16u,     /* a block id in a paged layout's table was >= num_blocks      */
    OXI_DEV_OUT_OF_BOUNDS = 32u  /* raised only by libraries built with -DOXI_BOUNDS: a table-driven
                                    index was out of range; the access was not performed         */
};

typedef struct oxi_handle oxi_handle;

int32_t oxi_version(void);
const char* oxi_status_string(int32_t status);
/* Text of the last error raised on the calling thread ("" if none). */
const char* oxi_last_error_string(void);

/* Creates the per-device workspace (split-KV partials, conv staging,
 * host-entry staging, argmax candidates and, when max_prefill_rows > 0, the
 * partial results of the prefill key-range split, see
 * oxi_prefill_split_configure).  Replaces the scratch half of
 * BatchEngine::new (batch_engine.rs:320-364).  max_batch <= 1024.
 * Calls on one handle use that workspace: they must be ordered on the device
 * (one stream, or events between streams), as the engine's single decode stream
 * orders them; independent streams take one handle each. */
int32_t oxi_create(oxi_handle** out, int32_t device, uint32_t max_batch, uint32_t max_seq_len,
                   uint32_t max_prefill_rows);
int32_t oxi_destroy(oxi_handle* h);
/* Bytes of device memory the handle owns. */
size_t oxi_workspace_bytes(const oxi_handle* h);
/* Synchronises `stream`, returns and clears the OR of OXI_DEV_* bits raised by
 * kernels since the last call.  For tests and debugging; not on the hot path. */
int32_t oxi_device_status(oxi_handle* h, void* stream, uint32_t* bits_out);

/* ---- fused operators (the product path) -------------------------------- */

/* Per-head Q/K RMSNorm + RoPE + KV append in ONE launch.
 * Replaces batched_qk_rmsnorm_fp16 x2, batched_rope_fp16 x2 and
 * batched_kv_copy_fp16 x2 (batched_attn.rs:13-118, 128-219, 233-287; launched
 * at batch_engine.rs:941-1014).
 *   q_io  [B][16][128]  in: projected q; out: normed + rotated q
 *   k_in  [B][4][128], v_in [B][4][128]  projected k, v (not modified)
 *   q_norm_w, k_norm_w [128]; cos, sin [max_pos][128] f16 tables (rope.rs:158-201)
 *   pos_ids [B] u32; row pos_ids[b] of k_ptrs[b] / v_ptrs[b] receives the
 *   normed + rotated k and the copied v.
 * K/V/q bytes are bit-identical to the reference kernels' on the same GPU. */
int32_t oxi_append(oxi_handle* h, void* stream, void* q_io, const void* k_in, const void* v_in,
                   const void* q_norm_w, const void* k_norm_w, const void* cos_table,
                   const void* sin_table, const uint32_t* pos_ids, const uint64_t* k_ptrs,
                   const uint64_t* v_ptrs, uint32_t batch, float eps);

/* Batched GQA decode attention with the per-head sigmoid output gate:
 * split-KV flash-decode streaming kernel + a small merge kernel that also
 * applies the gate (rows covered by one key range finish in the first kernel).
 * Replaces batched_gqa_attention_split4_fp16 + batched_gqa_attn_combine_fp16
 * (or batched_gqa_attention_online_fp16) + batched_sigmoid_gate_fp16
 * (batched_attn.rs:2665-3035, 1597-1717, 1194-1370, 583-655; launched at
 * batch_engine.rs:1154-1239).
 *   ctx_out [B][16][128]; q [B][16][128]; gate [B][16] or NULL (no gating);
 *   window: 0 = full attention, else key t is masked iff (seq_len-1) - t >= window. */
int32_t oxi_decode_attn(oxi_handle* h, void* stream, void* ctx_out, const void* q,
                        const void* gate, const uint64_t* k_ptrs, const uint64_t* v_ptrs,
                        const uint32_t* seq_lens, uint32_t batch, uint32_t window);

/* The whole attention-layer hot path of one decode step (batch_engine.rs:941-1239)
 * as ONE streaming kernel plus the merge kernel: RMSNorm + RoPE + KV append are
 * fused into the decode-attention kernel, so q is normalised on chip and never
 * makes a round trip through HBM.  Cache rows and ctx_out are byte-identical to
 * oxi_append followed by oxi_decode_attn.  Differences from that pair: q_io is
 * NOT modified (it is read as the raw projected q), and the position of the
 * appended token is taken as seq_lens[b] - 1 (pos_ids must agree, as the engine
 * guarantees, batch_engine.rs:689-691).  cos/sin tables, k_in and v_in must be
 * 16-byte aligned. */
int32_t oxi_append_decode(oxi_handle* h, void* stream, void* ctx_out, void* q_io, const void* k_in,
                          const void* v_in, const void* gate, const void* q_norm_w,
                          const void* k_norm_w, const void* cos_table, const void* sin_table,
                          const uint32_t* pos_ids, const uint32_t* seq_lens,
                          const uint64_t* k_ptrs, const uint64_t* v_ptrs, uint32_t batch,
                          uint32_t window, float eps);

/* Chunked-prefill causal GQA attention with the gate, over per-row tables:
 * row r attends keys [window start, seq_lens[r]) of its own cache.  All rows'
 * K/V must already be appended (batch_engine.rs:1011-1014).  One fused kernel;
 * scores and weights never touch HBM.
 * Replaces BatchEngine::gemm_attention_chunk (batch_engine.rs:439-592:
 * batched_attn_pack_q_fp16, cuBLASLt QK^T, batched_attn_softmax_mask_fp16,
 * cuBLASLt PV, batched_attn_gate_scatter_fp16) and the online-kernel fallback
 * (batch_engine.rs:1214-1239). */
int32_t oxi_prefill_attn(oxi_handle* h, void* stream, void* ctx_out, const void* q,
                         const void* gate, const uint64_t* k_ptrs, const uint64_t* v_ptrs,
                         const uint32_t* seq_lens, uint32_t rows, uint32_t window);

/* Key-range split for small prefill waves (a few long prompts; the reference's
 * PREFILL_MAX_CONCURRENT = 32 admission limit, batch_engine.rs:93, keeps waves
 * small).  One work item of oxi_prefill_attn is a 64-row block on one KV head;
 * a wave with fewer items than the GPU has SMs would leave SMs idle for as long
 * as its longest block scans its keys.  Such waves cut their long blocks into
 * parts of equal key ranges - as many as fill the SMs once, at most 32 per
 * block, none shorter than min_part_keys - and merge the parts' partial results
 * (unnormalised sums, row maximum, row sum, f32) in a second kernel.  `slots`
 * partial results of oxi_prefill_split_slot_bytes() each are reserved on the
 * handle, one per part of a split block; a wave that would need more runs
 * unsplit, and so does every wave with at least as many items as SMs.
 * oxi_create turns the split on for handles with max_prefill_rows > 0, with
 * min_part_keys = OXI_PREFILL_SPLIT_DEFAULT_MIN_PART_KEYS and SMs / 4 + 3 slots
 * (a split wave never has more parts than that); this call changes the setting.
 * Results stay within the attention tolerance of the unsplit path (not
 * bit-identical to it: the order of the sums changes) and are reproducible from
 * launch to launch.  min_part_keys = 0 or slots = 0 turns the split off and
 * frees the reservation; otherwise min_part_keys >= 256 and slots <= 4096.
 * Synchronises the device; call it with no work of this handle in flight.
 * Applies to oxi_prefill_attn and oxi_prefill_attn_paged. */
#define OXI_PREFILL_SPLIT_DEFAULT_MIN_PART_KEYS 512u
int32_t oxi_prefill_split_configure(oxi_handle* h, uint32_t min_part_keys, uint32_t slots);
uint64_t oxi_prefill_split_slot_bytes(void);

/* Registers the slab that holds the K/V caches (the reference keeps every
 * sequence's K and V rows of all layers in one slab, kv_pool.rs:31-61).  Rows of
 * oxi_prefill_attn whose k_ptrs / v_ptrs entry lies a whole number of 1024-byte
 * rows from `base` and inside the slab are then loaded by the TMA unit (tiled
 * tensor copies with the 128-byte swizzle) instead of by per-thread 16-byte
 * copies; other rows, and the ragged last tile of a sequence, keep the
 * per-thread path, so any table stays legal and the results are bit-identical
 * either way.  One slab per handle; base = NULL or bytes = 0 unregisters.
 * Host-side only (encodes a tensor map), nothing is enqueued. */
int32_t oxi_register_kv_slab(oxi_handle* h, const void* base, uint64_t bytes);

/* One-token causal conv1d + gating with the 6-slot carry state, one launch.
 * Replaces batched_fused_causal_conv1d_gating_ptr_fp16 (batched_attn.rs:727-881,
 * launched at batch_engine.rs:840-899).
 *   y_out [B][2048]; conv_ptrs [B] -> state [2048][6] f16, updated in place;
 *   bcx [B][6144] = [B | C | x]; conv_w [2048][7].  y and state bit-exact. */
int32_t oxi_conv_decode(oxi_handle* h, void* stream, void* y_out, const uint64_t* conv_ptrs,
                        const void* bcx, const void* conv_w, uint32_t batch);

/* Prefill conv for one wave: every row's 7-tap window is read from the wave's
 * own B*x history or the request's carry state, y is written for every row and
 * each chunk's final 6-slot state replaces the request's persistent state.
 * Replaces conv_state_prefill_fp16 + the conv kernel on pool rows + the
 * per-chunk device copies (batched_attn.rs:1049-1176, batch_engine.rs:847-899,
 * server.rs:1192-1224).
 *   carry_ptrs [rows] u64 (row's request state for this layer, [2048][6]);
 *   origin [rows] u32 wave row where the row's chunk starts; local_pos [rows]
 *   u32 position inside the chunk (as PrefillMeta, batch_engine.rs:156-160). */
int32_t oxi_conv_prefill(oxi_handle* h, void* stream, void* y_out, const uint64_t* carry_ptrs,
                         const uint32_t* origin, const uint32_t* local_pos, const void* bcx,
                         const void* conv_w, uint32_t rows);

/* ---- the linear layers on either side of the path -------------------------- */

/* Tensor maps over a layer's projection weights (host object, no device memory, nothing is copied: the
 * weights stay where the caller keeps them and must outlive the object).  Weight layout is the
 * engine's: [out_features][2048] f16 row-major, y = W x (lt.gemm(m = out_features, k = 2048, n = rows,
 * W, x, y), lt_gemm.rs:828-900), 16-byte aligned. */
typedef struct oxi_linear oxi_linear;
/* q_proj [2048][2048], k_proj [512][2048], v_proj [512][2048], gate_proj [16][2048] of one attention layer. */
int32_t oxi_qkvg_create(oxi_linear** out, const void* wq, const void* wk, const void* wv, const void* wg);
int32_t oxi_linear_create(oxi_linear** out, const void* w, uint32_t out_features);
int32_t oxi_linear_destroy(oxi_linear* w);

/* The four projection GEMMs in front of the path and the append operator in ONE kernel: x [rows][2048]
 * (the layer's normed hidden state) times q/k/v/gate weights on the tensor cores (tcgen05, f32
 * accumulate, results rounded to f16 as the reference's GEMMs round them), and in the epilogue per
 * token and head the Q/K RMSNorm + RoPE + KV append of oxi_append on those f16 values: K and V go
 * straight to row pos_ids[b] of k_ptrs[b] / v_ptrs[b], q_out [rows][16][128] receives the normalised +
 * rotated q and gate_out [rows][16] the gate for oxi_decode_attn / oxi_prefill_attn.
 * Replaces lt.gemm x4 (batch_engine.rs:914-926) + batched_qk_rmsnorm_fp16 x2 + batched_rope_fp16 x2 +
 * batched_kv_copy_fp16 x2 (batch_engine.rs:941-1014): ten launches and the q/k/v round trip through
 * HBM.  raw_out (nullable) [rows][3088] receives the f16 projections [q | k | v | gate] themselves.
 * Given those projections, q_out and the cache rows are byte-identical to oxi_append's; the projections
 * are within one f16 step of an fp32-accumulated matmul (the summation order inside a GEMM is not
 * specified by the reference either).  rows <= max(max_batch, max_prefill_rows). */
int32_t oxi_project_append(oxi_handle* h, void* stream, const oxi_linear* qkvg, const void* x, void* q_out, void* gate_out,
                           void* raw_out, const void* q_norm_w, const void* k_norm_w, const void* cos_table,
                           const void* sin_table, const uint32_t* pos_ids, const uint64_t* k_ptrs, const uint64_t* v_ptrs,
                           uint32_t rows, float eps);
/* y [rows][out_features] = x [rows][2048] W^T, the same GEMM without epilogue arithmetic: o_proj on the far
 * side of the path (lt.gemm(2048, 2048, b, o_proj, ctx, layer), batch_engine.rs:1241-1245). */
int32_t oxi_linear_forward(oxi_handle* h, void* stream, const oxi_linear* w, const void* x, void* y, uint32_t rows);

/* ---- step tables that advance on the device ----------------------------- */
/* pos_ids[b] += delta and seq_lens[b] += delta in place (either pointer may be
 * null).  The engine rebuilds and uploads its tables for every step
 * (batch_engine.rs:709-740); while the batch membership is unchanged only the
 * positions move, so with this call a captured CUDA graph of the whole decode
 * step (all layers + this call) can be replayed token after token without any
 * host-to-device copy.  No counterpart in the reference. */
int32_t oxi_advance_step(oxi_handle* h, void* stream, uint32_t* pos_ids, uint32_t* seq_lens, uint32_t batch,
                         uint32_t delta);

/* ---- paged K/V layout: block tables instead of one contiguous lease ---- */
/* The reference's stated next milestone (docs/SCALE_AND_OPTIMIZATION_ROADMAP.md:42-43):
 * its PagedKvPool (core/src/paged_pool.rs:10-25), PagedBlockManager
 * (scheduler/src/block_manager.rs, block_size 16) and the argument list of its
 * paged_attention_decode_v1 stub (kernels/src/attention.rs:9-27: k_cache,
 * v_cache, block_tables [batch][max_blocks], context_lens, max_blocks,
 * block_size) exist, the kernel body does not.  The three entry points below
 * are the pointer-table path's operators over that layout; heads, head dim and
 * scale are the path's constants.  Token t of row b lives in block
 * block_tables[b][t / block_size] at slot t % block_size; block i's rows start
 * at pool + i * block_stride_bytes, one row = 4 KV heads x 128 f16 (1024 bytes)
 * - with block_stride_bytes the reference's pool (all layers, K and V inside a
 * block) is addressed by pointing k_pool / v_pool at the layer's K / V rows of
 * block 0.  Results are bit-identical to the contiguous entry points on the
 * same keys.  A block id >= num_blocks sets OXI_DEV_BAD_BLOCK (block 0 is read
 * instead, nothing is written); a row that needs more than max_blocks blocks
 * sets OXI_DEV_BAD_SEQ_LEN and is skipped. */
typedef struct oxi_paged_layout {
    const void* k_pool;            /* device, 16-byte aligned */
    const void* v_pool;
    const uint32_t* block_tables;  /* device [batch][max_blocks] */
    uint64_t block_stride_bytes;   /* multiple of 16, >= block_size * 1024 */
    uint32_t max_blocks;
    uint32_t block_size;           /* tokens per block: 16, 32, 64, 128 or 256 */
    uint32_t num_blocks;
} oxi_paged_layout;
int32_t oxi_append_paged(oxi_handle* h, void* stream, void* q_io, const void* k_in, const void* v_in,
                         const void* q_norm_w, const void* k_norm_w, const void* cos_table,
                         const void* sin_table, const uint32_t* pos_ids, const oxi_paged_layout* layout,
                         uint32_t batch, float eps);
int32_t oxi_decode_attn_paged(oxi_handle* h, void* stream, void* ctx_out, const void* q, const void* gate,
                              const oxi_paged_layout* layout, const uint32_t* seq_lens, uint32_t batch,
                              uint32_t window);
/* Chunked-prefill attention over the paged layout: wave row r reads the keys of
 * table row row_seq[r] (consecutive rows with equal row_seq form one request's
 * chunk, as equal k_ptrs / v_ptrs do for oxi_prefill_attn); the rows' K/V were
 * appended before (oxi_append_paged).  Bit-identical to oxi_prefill_attn on the
 * same keys. */
int32_t oxi_prefill_attn_paged(oxi_handle* h, void* stream, void* ctx_out, const void* q, const void* gate,
                               const oxi_paged_layout* layout, const uint32_t* row_seq, const uint32_t* seq_lens,
                               uint32_t rows, uint32_t window);
int32_t oxi_append_decode_paged(oxi_handle* h, void* stream, void* ctx_out, void* q_io, const void* k_in,
                                const void* v_in, const void* gate, const void* q_norm_w,
                                const void* k_norm_w, const void* cos_table, const void* sin_table,
                                const uint32_t* seq_lens, const oxi_paged_layout* layout, uint32_t batch,
                                uint32_t window, float eps);

/* ---- the sampling side of a decode step: the file's two other table kernels */
/* out[b][:] = table[token_ids[b]][:] (f16 rows of `hidden` elements).
 * Replaces batched_embed_lookup_fp16 (batched_attn.rs:664-714, launched at
 * batch_engine.rs:765-779).  The reference does not check the ids; here an id
 * >= table_rows zero-fills the row and sets OXI_DEV_BAD_TOKEN. */
int32_t oxi_embed_lookup(oxi_handle* h, void* stream, void* out, const void* table,
                         const uint32_t* token_ids, uint32_t hidden, uint32_t table_rows,
                         uint32_t batch);
/* tokens_out[b] = argmax_v logits[b][v], logits [batch][vocab] f16, batch <= max_batch.
 * Replaces batched_argmax_direct_f16 (batched_attn.rs:890-1023, launched with
 * 256 threads per row at batch_engine.rs:1367-1378) and returns the same index
 * as that launch for every input, ties included: the reference resolves equal
 * maxima by its scan order and reduction tree (not by the lowest index), NaN
 * never wins, a row without any value above -1e30 yields 0. */
int32_t oxi_argmax(oxi_handle* h, void* stream, uint32_t* tokens_out, const void* logits,
                   uint32_t vocab, uint32_t batch);

/* ---- unfused operators with the reference's exact semantics ------------ */
/* Same contract as the PTX entry of the same name, so a harness can swap the
 * reference kernels for these one by one and localise a mismatch. */
int32_t oxi_qk_rmsnorm(oxi_handle* h, void* stream, void* x_io, const void* weight, float eps,
                       uint32_t num_heads, uint32_t batch); /* batched_attn.rs:13-118   */
int32_t oxi_rope(oxi_handle* h, void* stream, void* x_io, const void* cos_table,
                 const void* sin_table, const uint32_t* pos_ids, uint32_t num_heads,
                 uint32_t batch);                           /* batched_attn.rs:128-219  */
int32_t oxi_kv_copy(oxi_handle* h, void* stream, const uint64_t* dst_ptrs, const void* src,
                    const uint32_t* pos_ids, uint32_t batch); /* batched_attn.rs:233-287 */
int32_t oxi_sigmoid_gate(oxi_handle* h, void* stream, void* ctx_io, const void* gate,
                         uint32_t batch);                   /* batched_attn.rs:583-655  */

/* ---- host-buffer entry (what an engine without device staging calls) --- */

/* One decode step of `layers` attention layers driven from HOST memory: per
 * layer l the call uploads q/k/v/gate [l][B][...], the layer's pointer tables
 * and the step's pos_ids (seq_lens = pos_ids + 1), runs oxi_append +
 * oxi_decode_attn, and downloads ctx [l][B][16][128].  Mirrors the metadata
 * uploads of forward_step_with_embeds (batch_engine.rs:681-740).  All host
 * buffers should be pinned; the call returns after enqueueing (the caller
 * synchronises the stream before reading ctx_host).  K/V caches stay on the
 * device.  norm weights: [layers][128]; tables: [layers*B]. */
int32_t oxi_decode_step_host(oxi_handle* h, void* stream, void* ctx_host, const void* q_host,
                             const void* k_host, const void* v_host, const void* gate_host,
                             const void* q_norm_w_dev, const void* k_norm_w_dev,
                             const void* cos_table_dev, const void* sin_table_dev,
                             const uint32_t* pos_ids_host, const uint64_t* k_ptrs_host,
                             const uint64_t* v_ptrs_host, uint32_t batch, uint32_t layers,
                             uint32_t window, float eps);

/* ---- host side of the path as a C API: slab pool, leases, step tables ---- */

/* The reference keeps every sequence's K/V rows and conv states in two slabs and
 * hands each request a lease: a contiguous range of token rows plus a conv slot
 * (KvPool / KvLayout / KvLease, kv_pool.rs:31-251).  K of attention layer a lives
 * in plane 2a of the KV slab, V in plane 2a+1, each capacity_tokens rows of 1024
 * bytes (kv_pool.rs:46-61); the conv state of (slot, conv layer c) is a
 * [2048][6] f16 block.  These entry points restate that pool and the per-step
 * table build + upload of the engine (batch_engine.rs:709-740) so that a host
 * without the Rust engine can drive the operators above; a host that has its own
 * pool ignores them.  oxi_host_last_error_string() gives the text of the last
 * error of these functions on the calling thread. */
typedef struct oxi_kv_pool oxi_kv_pool;
typedef struct oxi_step_tables oxi_step_tables;
typedef struct oxi_lease {
    uint64_t tok_off; /* first token row of the lease inside every K / V plane */
    uint64_t tokens;  /* rows leased: the sequence may grow to this many tokens */
    uint64_t slot;    /* conv-state slot */
} oxi_lease;
const char* oxi_host_last_error_string(void);

/* Allocates both slabs on the current device (KvPool::new, kv_pool.rs:82-150):
 * layer_is_conv[l] != 0 marks conv layers; the token capacity is halved until the
 * KV slab fits (never below 4096 tokens), as the reference does. */
int32_t oxi_pool_create(oxi_kv_pool** out, const uint8_t* layer_is_conv, uint32_t num_layers, uint32_t max_batch,
                        uint64_t capacity_tokens);
int32_t oxi_pool_destroy(oxi_kv_pool* pool);
uint64_t oxi_pool_capacity_tokens(const oxi_kv_pool* pool);
uint64_t oxi_pool_free_tokens(const oxi_kv_pool* pool);
uint32_t oxi_pool_free_slots(const oxi_kv_pool* pool);
/* First-fit lease of `tokens` contiguous rows and a conv slot whose states are
 * zeroed on `stream` (KvPool::acquire, kv_pool.rs:175-218).  OXI_ERR_WORKSPACE
 * when no slot or no range of that size is free (the reference returns None). */
int32_t oxi_pool_acquire(oxi_kv_pool* pool, void* stream, uint64_t tokens, oxi_lease* out);
/* Returns the rows (coalescing with free neighbours) and the slot (kv_pool.rs:220-246). */
int32_t oxi_pool_release(oxi_kv_pool* pool, const oxi_lease* lease);
/* Device addresses the BatchSequence trait hands the engine (batch_engine.rs:78-87);
 * 0 when the layer is not of that kind. */
uint64_t oxi_pool_k_ptr(const oxi_kv_pool* pool, uint32_t layer, const oxi_lease* lease);
uint64_t oxi_pool_v_ptr(const oxi_kv_pool* pool, uint32_t layer, const oxi_lease* lease);
uint64_t oxi_pool_conv_ptr(const oxi_kv_pool* pool, uint32_t layer, const oxi_lease* lease);

/* One decode step's tables (batch_engine.rs:709-740): layer-major pointer tables
 * tbl[layer * batch + i] for K, V and conv state, positions and seq_lens =
 * position + 1.  set_row fills row i of the host image from a lease and the
 * position of the token appended in this step; upload copies rows 0..batch-1
 * to the device on `stream` from pinned memory (a ring of staging blocks: uploads
 * may be enqueued back to back without a sync).  The accessors return DEVICE
 * addresses, valid after the first upload and stable for the life of the object,
 * to be passed to oxi_append_decode, oxi_conv_decode, ...; advance moves every
 * row delta tokens ahead on the device (oxi_advance_step) and in the host image,
 * so that steps with unchanged membership need no upload. */
int32_t oxi_tables_create(oxi_step_tables** out, const oxi_kv_pool* pool, uint32_t max_batch);
int32_t oxi_tables_destroy(oxi_step_tables* tables);
int32_t oxi_tables_set_row(oxi_step_tables* tables, uint32_t row, const oxi_lease* lease, uint32_t position);
int32_t oxi_tables_upload(oxi_step_tables* tables, void* stream, uint32_t batch);
int32_t oxi_tables_advance(oxi_handle* h, oxi_step_tables* tables, void* stream, uint32_t delta);
uint32_t oxi_tables_batch(const oxi_step_tables* tables);
const uint64_t* oxi_tables_k_ptrs(const oxi_step_tables* tables, uint32_t layer);
const uint64_t* oxi_tables_v_ptrs(const oxi_step_tables* tables, uint32_t layer);
const uint64_t* oxi_tables_conv_ptrs(const oxi_step_tables* tables, uint32_t layer);
const uint32_t* oxi_tables_pos_ids(const oxi_step_tables* tables);
const uint32_t* oxi_tables_seq_lens(const oxi_step_tables* tables);

/* ---- test support ------------------------------------------------------- */

/* Every in-kernel pipeline wait (a consumer waiting for a stage of K/V rows, the
 * tensor-core warps waiting for a tile) is bounded: after about one second it
 * gives up, the CTA finishes without writing output and OXI_DEV_WAIT_TIMEOUT is
 * raised.  Nothing in normal operation makes a wait run out, so this call exists
 * to exercise that path without faulting or hanging the GPU: it arms the NEXT
 * launch of this handle's decode-attention kernel (which = 0), prefill-attention
 * kernel (which = 1; oxi_prefill_attn only, the armed wave runs unsplit and without
 * a registered slab) or projection GEMM (which = 2: oxi_project_append or
 * oxi_linear_forward, whichever kernel the row count selects) so that CTA 0
 * withholds its stage-th pipeline stage (decode and projection: no copy is issued
 * for it; prefill: the K tile is copied but never published) and all waits of that
 * launch last limit_us microseconds instead of a second.  The armed launch returns
 * normally with OXI_DEV_WAIT_TIMEOUT set and with the outputs of CTA 0's work
 * (projection: of its cluster's tile) unwritten; later launches are unaffected.
 * No counterpart in the reference. */
int32_t oxi_debug_arm_wait_fault(oxi_handle* h, uint32_t which, uint32_t stage, uint32_t limit_us);

/* Measurement support: streams `bytes` (rounded down to whole 64 KB stages) from
 * `src` through the decode-attention kernel's memory pipeline - one persistent CTA
 * per SM, 1-D bulk copies of copy_bytes each into a 3-stage ring of 64 KB stages,
 * mbarrier hand-over to four consumer warps - with no arithmetic.  Timed by the
 * caller (events on `stream`), it gives the read-only bandwidth ceiling of that
 * pipeline, the yardstick beside the read+write copy bandwidth.  copy_bytes is a
 * power of two in 16 .. 65536 (the decode kernel copies 4096).  No counterpart in
 * the reference. */
int32_t oxi_debug_stream_read(oxi_handle* h, void* stream, const void* src, uint64_t bytes, uint32_t copy_bytes);

/* ---- entry point that allocates nothing -------------------------------- */

#define OXI_STATIC_MAX_BATCH 16u      /* rows per call                         */
#define OXI_STATIC_MAX_SEQ_LEN 4096u  /* keys per row, the appended one included */

/* oxi_decode_attn for callers that cannot allocate device memory (and hence
 * cannot call oxi_create): plugins inside a foreign memory budget, callbacks
 * that run while the application's allocator is locked, processes that gave
 * all device memory to their own pool.  It has no counterpart in the
 * reference, whose engine allocates all scratch in BatchEngine::new.
 *
 * Same inputs, outputs and arithmetic as oxi_decode_attn, no handle.  The
 * split-KV partials, the work counter and the status word live in a ~2.1 MB
 * array inside the library image (held by every GPU that loads the library
 * until the process exits); the call performs no cudaMalloc / cudaFree and
 * calls no allocating library routine.
 *   - batch <= OXI_STATIC_MAX_BATCH, else OXI_ERR_BATCH; max_seq_len (the
 *     caller's bound on every seq_lens[b]) <= OXI_STATIC_MAX_SEQ_LEN, else
 *     OXI_ERR_ARG.  A row whose seq_len exceeds max_seq_len is skipped.
 *   - The device current on the calling thread is used.  The FIRST call on a
 *     device also resolves the array's device address and sets the kernel's
 *     shared-memory attribute; make that first call outside any stream capture.
 *   - All calls on one device share the array: calls whose kernels can overlap
 *     on the GPU (different streams without ordering between them) race.  Calls
 *     on one stream are ordered and safe. */
int32_t oxi_decode_attn_static(void* stream, void* ctx_out, const void* q, const void* gate,
                               const uint64_t* k_ptrs, const uint64_t* v_ptrs,
                               const uint32_t* seq_lens, uint32_t batch, uint32_t max_seq_len,
                               uint32_t window);
/* oxi_device_status for the path above: synchronises `stream`, returns and clears
 * the OXI_DEV_* bits raised by oxi_decode_attn_static calls on the current device
 * since the last read (a skipped row - bad seq_len, misaligned pointer - is
 * otherwise invisible to a caller without a handle).  The word lives in the same
 * array; oxi_decode_attn_static never clears it.  Allocates nothing. */
int32_t oxi_static_device_status(void* stream, uint32_t* bits_out);

#ifdef __cplusplus
}
#endif
#endif /* OXI_KV_H */
