// C ABI of liboxi_kv: handle/workspace management, host-side argument
// validation, and the launch sequences behind each exported operator.
#include "../../include/oxi_kv.h"

#include <cuda.h>  // CUtensorMap and its enums only; the encoder is fetched through the runtime

#include <cstdio>
#include <cstring>
#include <new>

#include "common.cuh"
#include "kernels.h"

using namespace oxi;

struct oxi_handle {
    int device;
    int num_sms;
    uint32_t max_batch, max_seq_len, max_prefill_rows;
    DecodeWorkspace dws;
    void* conv_stage;     // [max_prefill_rows][2048][6] f16
    uint32_t* pf_order;   // [ceil(max_prefill_rows/32)] prefill block order
    void* am_cand;        // [max_batch][argmax_max_splits()][256] argmax candidates of the row splits
    uint32_t* am_count;   // [max_batch] arrival counters, zero between launches
    PrefillSplitWs pf_split;  // reserved by oxi_prefill_split_configure
    uint32_t pf_part_keys;    // keys per part of a split block; 0: off
    PrefillSlab pf_slab;      // registered by oxi_register_kv_slab; rows == 0: none
    WaitFault dbg_decode, dbg_prefill, dbg_proj;  // armed by oxi_debug_arm_wait_fault for the next launch only
    // staging for the host-buffer entry: one contiguous buffer per kind holding a group of up to STG_MAX layers
    // (layer-major, compact for the call's batch), so that a group's inputs arrive with one copy per kind
    static constexpr int STG_MAX = 16;
    uint32_t stg_sets;    // layers per group: 16 for handles of up to 256 rows, else 8
    char* stg_q;          // [stg_sets][max_batch][16][128] f16
    char* stg_k;          // [stg_sets][max_batch][4][128]
    char* stg_v;
    char* stg_gate;       // [stg_sets][max_batch][16]
    char* stg_ctx;        // [stg_sets][max_batch][16][128]
    char* stg_kp;         // [stg_sets][max_batch] u64
    char* stg_vp;
    uint32_t* stg_pos;    // [max_batch]
    uint32_t* stg_len;    // [max_batch]
    // copy streams and events of the host-buffer entry: the uploads of a group's later layers and the
    // downloads of its earlier layers overlap the kernels
    cudaStream_t h2d, d2h;
    cudaEvent_t ev_start, ev_up[6], ev_comp[STG_MAX], ev_down_last;  // ev_up: one per upload chunk of a group
    size_t bytes;
};

static thread_local char g_err[256] = "";

static int32_t fail(int32_t code, const char* msg) {
    snprintf(g_err, sizeof(g_err), "%s", msg);
    return code;
}
static int32_t cuda_fail(cudaError_t e, const char* where) {
    snprintf(g_err, sizeof(g_err), "%s: %s", where, cudaGetErrorString(e));
    return (int32_t)e;
}
#define OXI_CUDA(call, where)                          \
    do {                                               \
        cudaError_t e__ = (call);                      \
        if (e__ != cudaSuccess) return cuda_fail(e__, where); \
    } while (0)

extern "C" {

int32_t oxi_version(void) { return OXI_VERSION; }

const char* oxi_status_string(int32_t s) {
    switch (s) {
        case OXI_OK: return "ok";
        case OXI_ERR_NULL: return "null pointer or handle";
        case OXI_ERR_BATCH: return "batch/rows is zero or exceeds the handle limit";
        case OXI_ERR_ARG: return "scalar argument out of range";
        case OXI_ERR_WORKSPACE: return "workspace too small for this call";
        case OXI_ERR_NO_DEVICE: return "no usable CUDA device";
        default: return s > 0 ? cudaGetErrorString((cudaError_t)s) : "unknown status";
    }
}

const char* oxi_last_error_string(void) { return g_err; }

static int32_t dev_alloc(oxi_handle* h, void** p, size_t bytes) {
    cudaError_t e = cudaMalloc(p, bytes);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc");
    h->bytes += bytes;
    return OXI_OK;
}

int32_t oxi_create(oxi_handle** out, int32_t device, uint32_t max_batch, uint32_t max_seq_len,
                   uint32_t max_prefill_rows) {
    if (!out) return fail(OXI_ERR_NULL, "oxi_create: out is null");
    *out = nullptr;
    if (max_batch == 0 || max_batch > decode_max_rows())
        return fail(OXI_ERR_BATCH, "oxi_create: max_batch must be 1..1024");
    if (max_seq_len == 0 || max_seq_len > (1u << 22)) return fail(OXI_ERR_ARG, "oxi_create: max_seq_len out of range");
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || device < 0 || device >= ndev) {
        cudaGetLastError();
        return fail(OXI_ERR_NO_DEVICE, "oxi_create: no such CUDA device");
    }
    cudaDeviceProp prop;
    OXI_CUDA(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties");
    if (prop.major != 10) return fail(OXI_ERR_NO_DEVICE, "oxi_create: device is not sm_100 (B200)");
    OXI_CUDA(cudaSetDevice(device), "cudaSetDevice");

    oxi_handle* h = new (std::nothrow) oxi_handle();
    if (!h) return fail(OXI_ERR_WORKSPACE, "oxi_create: host allocation failed");
    memset(h, 0, sizeof(*h));
    h->device = device;
    h->num_sms = prop.multiProcessorCount;
    h->max_batch = max_batch;
    h->max_seq_len = max_seq_len;
    h->max_prefill_rows = max_prefill_rows;

    const uint32_t chunk = decode_chunk_keys();
    const uint32_t max_chunks = (max_seq_len + chunk - 1) / chunk;
    h->dws.max_chunks = max_chunks;
    h->dws.max_seq_len = max_seq_len;
    h->dws.num_sms = h->num_sms;
    int32_t rc = OXI_OK;
    const size_t slots = (size_t)max_batch * max_chunks * NQ;
    if ((rc = dev_alloc(h, (void**)&h->dws.partial_acc, slots * HD * sizeof(float)))) goto bad;
    if ((rc = dev_alloc(h, (void**)&h->dws.partial_stats, slots * 2 * sizeof(float)))) goto bad;
    if ((rc = dev_alloc(h, (void**)&h->dws.status, 256))) goto bad;
    h->dws.work_counter = h->dws.status + 32;  // same zero-initialised 256-byte block, own 128-byte line
    if (const size_t mb = decode_merge_scratch_bytes(max_batch, max_chunks)) {
        if ((rc = dev_alloc(h, (void**)&h->dws.merge_acc, mb))) goto bad;
    }
    if ((rc = dev_alloc(h, (void**)&h->dws.merge_count, (size_t)max_batch * NKV * 4))) goto bad;
    if (cudaMemset(h->dws.merge_count, 0, (size_t)max_batch * NKV * 4) != cudaSuccess) {
        rc = cuda_fail(cudaGetLastError(), "cudaMemset");
        goto bad;
    }
    if ((rc = dev_alloc(h, &h->am_cand, (size_t)max_batch * argmax_max_splits() * 256 * 8))) goto bad;
    if ((rc = dev_alloc(h, (void**)&h->am_count, (size_t)max_batch * 4))) goto bad;
    if (cudaMemset(h->am_count, 0, (size_t)max_batch * 4) != cudaSuccess) {
        rc = cuda_fail(cudaGetLastError(), "cudaMemset");
        goto bad;
    }
    if (max_prefill_rows) {
        if ((rc = dev_alloc(h, &h->conv_stage, (size_t)max_prefill_rows * HIDDEN * CONV_S * 2))) goto bad;
        if ((rc = dev_alloc(h, (void**)&h->pf_order, ((size_t)max_prefill_rows / 32 + 1) * sizeof(uint32_t)))) goto bad;
    }
    h->stg_sets = max_batch <= 256u ? 16u : 8u;
    {
        const size_t n = (size_t)h->stg_sets * max_batch;
        if ((rc = dev_alloc(h, (void**)&h->stg_q, n * NQ * HD * 2))) goto bad;
        if ((rc = dev_alloc(h, (void**)&h->stg_k, n * NKV * HD * 2))) goto bad;
        if ((rc = dev_alloc(h, (void**)&h->stg_v, n * NKV * HD * 2))) goto bad;
        if ((rc = dev_alloc(h, (void**)&h->stg_gate, n * NQ * 2))) goto bad;
        if ((rc = dev_alloc(h, (void**)&h->stg_ctx, n * NQ * HD * 2))) goto bad;
        if ((rc = dev_alloc(h, (void**)&h->stg_kp, n * 8))) goto bad;
        if ((rc = dev_alloc(h, (void**)&h->stg_vp, n * 8))) goto bad;
    }
    if ((rc = dev_alloc(h, (void**)&h->stg_pos, (size_t)max_batch * 4))) goto bad;
    if ((rc = dev_alloc(h, (void**)&h->stg_len, (size_t)max_batch * 4))) goto bad;
    {
        cudaError_t e = cudaStreamCreateWithFlags(&h->h2d, cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&h->d2h, cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->ev_start, cudaEventDisableTiming);
        for (int i = 0; i < 6 && e == cudaSuccess; i++) e = cudaEventCreateWithFlags(&h->ev_up[i], cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->ev_down_last, cudaEventDisableTiming);
        for (int i = 0; i < oxi_handle::STG_MAX && e == cudaSuccess; i++)
            e = cudaEventCreateWithFlags(&h->ev_comp[i], cudaEventDisableTiming);
        if (e != cudaSuccess) { rc = cuda_fail(e, "stream/event creation"); goto bad; }
    }
    if (cudaMemset(h->dws.status, 0, 256) != cudaSuccess) {
        rc = cuda_fail(cudaGetLastError(), "cudaMemset");
        goto bad;
    }
    {
        cudaError_t e = decode_attn_init();
        if (e == cudaSuccess) e = prefill_attn_init();
        if (e == cudaSuccess) e = stream_probe_init();
        if (e == cudaSuccess) e = proj_gemm_init();
        if (e != cudaSuccess) { rc = cuda_fail(e, "cudaFuncSetAttribute"); goto bad; }
    }
    if (cudaDeviceSynchronize() != cudaSuccess) {
        rc = cuda_fail(cudaGetLastError(), "oxi_create sync");
        goto bad;
    }
    // Small prefill waves spread their long blocks over idle SMs by default: a split wave has at most
    // one (block part, KV head) item per SM, hence at most num_sms / 4 parts in flight.
    if (max_prefill_rows && (rc = oxi_prefill_split_configure(h, OXI_PREFILL_SPLIT_DEFAULT_MIN_PART_KEYS,
                                                              (uint32_t)h->num_sms / NKV + 3u)))
        goto bad;
    *out = h;
    return OXI_OK;
bad:
    oxi_destroy(h);
    return rc;
}

int32_t oxi_destroy(oxi_handle* h) {
    if (!h) return OXI_OK;
    cudaSetDevice(h->device);
    cudaFree(h->dws.partial_acc);
    cudaFree(h->dws.partial_stats);
    cudaFree(h->dws.status);
    cudaFree(h->dws.merge_acc);
    cudaFree(h->dws.merge_count);
    cudaFree(h->conv_stage);
    cudaFree(h->pf_order);
    cudaFree(h->am_cand);
    cudaFree(h->am_count);
    cudaFree(h->pf_split.units);
    cudaFree(h->pf_split.part);
    cudaFree(h->stg_q); cudaFree(h->stg_k); cudaFree(h->stg_v); cudaFree(h->stg_gate);
    cudaFree(h->stg_ctx); cudaFree(h->stg_kp); cudaFree(h->stg_vp);
    cudaFree(h->stg_pos);
    cudaFree(h->stg_len);
    if (h->h2d) cudaStreamDestroy(h->h2d);
    if (h->d2h) cudaStreamDestroy(h->d2h);
    if (h->ev_start) cudaEventDestroy(h->ev_start);
    for (int i = 0; i < 6; i++)
        if (h->ev_up[i]) cudaEventDestroy(h->ev_up[i]);
    if (h->ev_down_last) cudaEventDestroy(h->ev_down_last);
    for (int i = 0; i < oxi_handle::STG_MAX; i++)
        if (h->ev_comp[i]) cudaEventDestroy(h->ev_comp[i]);
    cudaGetLastError();
    delete h;
    return OXI_OK;
}

size_t oxi_workspace_bytes(const oxi_handle* h) { return h ? h->bytes : 0; }

int32_t oxi_device_status(oxi_handle* h, void* stream, uint32_t* bits_out) {
    if (!h || !bits_out) return fail(OXI_ERR_NULL, "oxi_device_status: null argument");
    cudaStream_t s = (cudaStream_t)stream;
    uint32_t bits = 0;
    OXI_CUDA(cudaMemcpyAsync(&bits, h->dws.status, 4, cudaMemcpyDeviceToHost, s), "status copy");
    OXI_CUDA(cudaMemsetAsync(h->dws.status, 0, 4, s), "status clear");
    OXI_CUDA(cudaStreamSynchronize(s), "status sync");
    *bits_out = bits;
    return OXI_OK;
}

// The decode workspace for one launch; an armed test fault applies to this launch only.
static DecodeWorkspace take_dws(oxi_handle* h) {
    DecodeWorkspace ws = h->dws;
    ws.fault = h->dbg_decode;
    h->dbg_decode = WaitFault{};
    return ws;
}
static WaitFault take_prefill_fault(oxi_handle* h) {
    const WaitFault f = h->dbg_prefill;
    h->dbg_prefill = WaitFault{};
    return f;
}
static WaitFault take_proj_fault(oxi_handle* h) {
    const WaitFault f = h->dbg_proj;
    h->dbg_proj = WaitFault{};
    return f;
}

int32_t oxi_debug_arm_wait_fault(oxi_handle* h, uint32_t which, uint32_t stage, uint32_t limit_us) {
    if (!h) return fail(OXI_ERR_NULL, "oxi_debug_arm_wait_fault: handle is null");
    if (which > 2u || limit_us == 0u || limit_us > 1000000u || stage >= 0x7fffffffu)
        return fail(OXI_ERR_ARG, "oxi_debug_arm_wait_fault: which is 0, 1 or 2, limit_us 1..1000000");
    WaitFault f;
    f.skip_plus1 = stage + 1u;
    f.limit_us = limit_us;
    (which == 0u ? h->dbg_decode : which == 1u ? h->dbg_prefill : h->dbg_proj) = f;
    return OXI_OK;
}

int32_t oxi_debug_stream_read(oxi_handle* h, void* stream, const void* src, uint64_t bytes, uint32_t copy_bytes) {
    if (!h || !src) return fail(OXI_ERR_NULL, "oxi_debug_stream_read: null argument");
    const uint32_t stage = stream_probe_stage_bytes();
    if (copy_bytes < 16u || copy_bytes > stage || (copy_bytes & (copy_bytes - 1u)) != 0u)
        return fail(OXI_ERR_ARG, "oxi_debug_stream_read: copy_bytes must be a power of two, 16 .. 65536");
    if (bytes < stage || ((uintptr_t)src & 15u) != 0u)
        return fail(OXI_ERR_ARG, "oxi_debug_stream_read: at least 64 KB from a 16-byte aligned address");
    OXI_CUDA(launch_stream_read((cudaStream_t)stream, src, bytes, copy_bytes, h->num_sms, h->dws.status + 8, h->dws.status),
             "stream_read launch");
    return OXI_OK;
}

#define REQ_HANDLE(name) \
    if (!h) return fail(OXI_ERR_NULL, name ": handle is null")
#define REQ_PTR(p, name) \
    if (!(p)) return fail(OXI_ERR_NULL, name ": required pointer is null")
#define REQ_BATCH(n, lim, name) \
    if ((n) == 0 || (n) > (lim)) return fail(OXI_ERR_BATCH, name ": batch/rows is 0 or exceeds the handle limit")

int32_t oxi_append(oxi_handle* h, void* stream, void* q_io, const void* k_in, const void* v_in,
                   const void* q_norm_w, const void* k_norm_w, const void* cos_table,
                   const void* sin_table, const uint32_t* pos_ids, const uint64_t* k_ptrs,
                   const uint64_t* v_ptrs, uint32_t batch, float eps) {
    REQ_HANDLE("oxi_append");
    REQ_PTR(q_io && k_in && v_in && q_norm_w && k_norm_w && cos_table && sin_table && pos_ids &&
                k_ptrs && v_ptrs, "oxi_append");
    REQ_BATCH(batch, (h->max_batch > h->max_prefill_rows ? h->max_batch : h->max_prefill_rows), "oxi_append");
    if (!(eps >= 0.0f)) return fail(OXI_ERR_ARG, "oxi_append: eps must be >= 0");
    OXI_CUDA(launch_append((cudaStream_t)stream, q_io, k_in, v_in, q_norm_w, k_norm_w, cos_table,
                           sin_table, pos_ids, k_ptrs, v_ptrs, batch, eps, h->dws.status),
             "append launch");
    return OXI_OK;
}

int32_t oxi_decode_attn(oxi_handle* h, void* stream, void* ctx_out, const void* q,
                        const void* gate, const uint64_t* k_ptrs, const uint64_t* v_ptrs,
                        const uint32_t* seq_lens, uint32_t batch, uint32_t window) {
    REQ_HANDLE("oxi_decode_attn");
    REQ_PTR(ctx_out && q && k_ptrs && v_ptrs && seq_lens, "oxi_decode_attn");
    REQ_BATCH(batch, h->max_batch, "oxi_decode_attn");
    OXI_CUDA(launch_decode_attn((cudaStream_t)stream, take_dws(h), ctx_out, q, gate, k_ptrs, v_ptrs,
                                seq_lens, batch, window),
             "decode_attn launch");
    return OXI_OK;
}

int32_t oxi_append_decode(oxi_handle* h, void* stream, void* ctx_out, void* q_io, const void* k_in,
                          const void* v_in, const void* gate, const void* q_norm_w,
                          const void* k_norm_w, const void* cos_table, const void* sin_table,
                          const uint32_t* pos_ids, const uint32_t* seq_lens,
                          const uint64_t* k_ptrs, const uint64_t* v_ptrs, uint32_t batch,
                          uint32_t window, float eps) {
    REQ_HANDLE("oxi_append_decode");
    REQ_PTR(ctx_out && q_io && k_in && v_in && q_norm_w && k_norm_w && cos_table && sin_table && pos_ids &&
                seq_lens && k_ptrs && v_ptrs, "oxi_append_decode");
    REQ_BATCH(batch, h->max_batch, "oxi_append_decode");
    if (!(eps >= 0.0f)) return fail(OXI_ERR_ARG, "oxi_append_decode: eps must be >= 0");
    OXI_CUDA(launch_append_decode((cudaStream_t)stream, take_dws(h), ctx_out, q_io, k_in, v_in, gate, q_norm_w,
                                  k_norm_w, cos_table, sin_table, seq_lens, k_ptrs, v_ptrs, batch, window, eps),
             "append_decode launch");
    return OXI_OK;
}

int32_t oxi_advance_step(oxi_handle* h, void* stream, uint32_t* pos_ids, uint32_t* seq_lens, uint32_t batch,
                         uint32_t delta) {
    REQ_HANDLE("oxi_advance_step");
    REQ_PTR(pos_ids || seq_lens, "oxi_advance_step");
    if (batch == 0) return fail(OXI_ERR_BATCH, "oxi_advance_step: batch is 0");
    OXI_CUDA(launch_advance_step((cudaStream_t)stream, pos_ids, seq_lens, batch, delta), "advance_step launch");
    return OXI_OK;
}

// Validates a paged layout and converts it to the kernels' form.
static int32_t paged_map(const oxi_paged_layout* l, const char* who, PagedMap* pm) {
    if (!l || !l->k_pool || !l->v_pool || !l->block_tables) return fail(OXI_ERR_NULL, who);
    uint32_t lbs = 0;
    while ((1u << lbs) < l->block_size && lbs < 31) lbs++;
    if (l->block_size < 16 || l->block_size > 256 || (1u << lbs) != l->block_size)
        return fail(OXI_ERR_ARG, "paged layout: block_size must be 16, 32, 64, 128 or 256 tokens");
    if (l->max_blocks == 0 || l->num_blocks == 0) return fail(OXI_ERR_ARG, "paged layout: max_blocks and num_blocks must be positive");
    if ((l->block_stride_bytes & 15ull) != 0ull || l->block_stride_bytes < (uint64_t)l->block_size * KV_ROW_BYTES)
        return fail(OXI_ERR_ARG, "paged layout: block_stride_bytes must be a multiple of 16 and hold block_size rows of 1024 bytes");
    if ((((uintptr_t)l->k_pool | (uintptr_t)l->v_pool) & 15u) != 0) return fail(OXI_ERR_ARG, "paged layout: pools must be 16-byte aligned");
    pm->k_pool = (const unsigned char*)l->k_pool;
    pm->v_pool = (const unsigned char*)l->v_pool;
    pm->block_tables = l->block_tables;
    pm->block_stride = l->block_stride_bytes;
    pm->max_blocks = l->max_blocks;
    pm->lbs = lbs;
    pm->num_blocks = l->num_blocks;
    return OXI_OK;
}

int32_t oxi_append_paged(oxi_handle* h, void* stream, void* q_io, const void* k_in, const void* v_in,
                         const void* q_norm_w, const void* k_norm_w, const void* cos_table,
                         const void* sin_table, const uint32_t* pos_ids, const oxi_paged_layout* layout,
                         uint32_t batch, float eps) {
    REQ_HANDLE("oxi_append_paged");
    REQ_PTR(q_io && k_in && v_in && q_norm_w && k_norm_w && cos_table && sin_table && pos_ids, "oxi_append_paged");
    REQ_BATCH(batch, h->max_batch, "oxi_append_paged");
    if (!(eps >= 0.0f)) return fail(OXI_ERR_ARG, "oxi_append_paged: eps must be >= 0");
    PagedMap pm;
    if (int32_t rc = paged_map(layout, "oxi_append_paged", &pm)) return rc;
    OXI_CUDA(launch_append_paged((cudaStream_t)stream, q_io, k_in, v_in, q_norm_w, k_norm_w, cos_table, sin_table,
                                 pos_ids, pm, batch, eps, h->dws.status),
             "append_paged launch");
    return OXI_OK;
}

int32_t oxi_decode_attn_paged(oxi_handle* h, void* stream, void* ctx_out, const void* q, const void* gate,
                              const oxi_paged_layout* layout, const uint32_t* seq_lens, uint32_t batch,
                              uint32_t window) {
    REQ_HANDLE("oxi_decode_attn_paged");
    REQ_PTR(ctx_out && q && seq_lens, "oxi_decode_attn_paged");
    REQ_BATCH(batch, h->max_batch, "oxi_decode_attn_paged");
    PagedMap pm;
    if (int32_t rc = paged_map(layout, "oxi_decode_attn_paged", &pm)) return rc;
    OXI_CUDA(launch_decode_attn_paged((cudaStream_t)stream, take_dws(h), ctx_out, q, gate, pm, seq_lens, batch, window),
             "decode_attn_paged launch");
    return OXI_OK;
}

int32_t oxi_append_decode_paged(oxi_handle* h, void* stream, void* ctx_out, void* q_io, const void* k_in,
                                const void* v_in, const void* gate, const void* q_norm_w,
                                const void* k_norm_w, const void* cos_table, const void* sin_table,
                                const uint32_t* seq_lens, const oxi_paged_layout* layout, uint32_t batch,
                                uint32_t window, float eps) {
    REQ_HANDLE("oxi_append_decode_paged");
    REQ_PTR(ctx_out && q_io && k_in && v_in && q_norm_w && k_norm_w && cos_table && sin_table && seq_lens,
            "oxi_append_decode_paged");
    REQ_BATCH(batch, h->max_batch, "oxi_append_decode_paged");
    if (!(eps >= 0.0f)) return fail(OXI_ERR_ARG, "oxi_append_decode_paged: eps must be >= 0");
    PagedMap pm;
    if (int32_t rc = paged_map(layout, "oxi_append_decode_paged", &pm)) return rc;
    OXI_CUDA(launch_append_decode_paged((cudaStream_t)stream, take_dws(h), ctx_out, q_io, k_in, v_in, gate, q_norm_w,
                                        k_norm_w, cos_table, sin_table, seq_lens, pm, batch, window, eps),
             "append_decode_paged launch");
    return OXI_OK;
}

uint64_t oxi_prefill_split_slot_bytes(void) { return (uint64_t)prefill_split_slot_bytes(); }

int32_t oxi_prefill_split_configure(oxi_handle* h, uint32_t part_keys, uint32_t slots) {
    REQ_HANDLE("oxi_prefill_split_configure");
    if (part_keys != 0u && part_keys < 256u)
        return fail(OXI_ERR_ARG, "oxi_prefill_split_configure: part_keys must be 0 or at least 256");
    if (slots > 4096u) return fail(OXI_ERR_ARG, "oxi_prefill_split_configure: at most 4096 slots");
    OXI_CUDA(cudaSetDevice(h->device), "cudaSetDevice");
    OXI_CUDA(cudaDeviceSynchronize(), "oxi_prefill_split_configure sync");
    if (h->pf_split.max_slots) h->bytes -= prefill_split_table_bytes() + (size_t)h->pf_split.max_slots * prefill_split_slot_bytes();
    cudaFree(h->pf_split.units);
    cudaFree(h->pf_split.part);
    h->pf_split = PrefillSplitWs{};
    h->pf_part_keys = 0;
    if (part_keys == 0u || slots == 0u) return OXI_OK;
    if (int32_t rc = dev_alloc(h, (void**)&h->pf_split.units, prefill_split_table_bytes())) return rc;
    if (int32_t rc = dev_alloc(h, (void**)&h->pf_split.part, (size_t)slots * prefill_split_slot_bytes())) {
        cudaFree(h->pf_split.units);
        h->bytes -= prefill_split_table_bytes();
        h->pf_split = PrefillSplitWs{};
        return rc;
    }
    h->pf_split.max_slots = slots;
    h->pf_part_keys = part_keys;
    return OXI_OK;
}

int32_t oxi_register_kv_slab(oxi_handle* h, const void* base, uint64_t bytes) {
    REQ_HANDLE("oxi_register_kv_slab");
    h->pf_slab = PrefillSlab{};
    if (!base || bytes == 0) return OXI_OK;  // unregistered
    if (((uintptr_t)base & 15u) != 0u) return fail(OXI_ERR_ARG, "oxi_register_kv_slab: base must be 16-byte aligned");
    const uint64_t rows = bytes / KV_ROW_BYTES;
    if (rows == 0 || rows > 0x7fffffffull) return fail(OXI_ERR_ARG, "oxi_register_kv_slab: 1 .. 2^31-1 rows of 1024 bytes");
    typedef CUresult (*encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    OXI_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres), "cudaGetDriverEntryPoint");
    if (!fn || qres != cudaDriverEntryPointSuccess) return fail(OXI_ERR_NO_DEVICE, "oxi_register_kv_slab: driver has no cuTensorMapEncodeTiled");
    static_assert(sizeof(CUtensorMap) == sizeof(TmaDesc), "tensor map size");
    // rows of [4 KV heads][128] f16; a box is 64 rows x 64 elements (128 bytes, one swizzle span)
    const cuuint64_t dims[2] = {(cuuint64_t)(NKV * HD), (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)KV_ROW_BYTES};
    const cuuint32_t box[2] = {64u, 64u};
    const cuuint32_t estr[2] = {1u, 1u};
    PrefillSlab s{};
    const CUresult r = ((encode_fn)fn)(reinterpret_cast<CUtensorMap*>(&s.map), CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                                       const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                       CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(OXI_ERR_ARG, "oxi_register_kv_slab: cuTensorMapEncodeTiled rejected the slab");
    s.base = (uint64_t)(uintptr_t)base;
    s.rows = (uint32_t)rows;
    h->pf_slab = s;
    return OXI_OK;
}

int32_t oxi_prefill_attn_paged(oxi_handle* h, void* stream, void* ctx_out, const void* q, const void* gate,
                               const oxi_paged_layout* layout, const uint32_t* row_seq, const uint32_t* seq_lens,
                               uint32_t rows, uint32_t window) {
    REQ_HANDLE("oxi_prefill_attn_paged");
    REQ_PTR(ctx_out && q && row_seq && seq_lens, "oxi_prefill_attn_paged");
    REQ_BATCH(rows, h->max_prefill_rows, "oxi_prefill_attn_paged");
    PagedMap pm;
    if (int32_t rc = paged_map(layout, "oxi_prefill_attn_paged", &pm)) return rc;
    const WaitFault flt = take_prefill_fault(h);
    OXI_CUDA(launch_prefill_attn((cudaStream_t)stream, ctx_out, q, gate, nullptr, nullptr, seq_lens, rows, window,
                                 h->dws.status, h->num_sms, h->pf_order, h->dws.status + 48, &pm, row_seq,
                                 &h->pf_split, h->pf_part_keys, nullptr, &flt),
             "prefill_attn_paged launch");
    return OXI_OK;
}

int32_t oxi_prefill_attn(oxi_handle* h, void* stream, void* ctx_out, const void* q,
                         const void* gate, const uint64_t* k_ptrs, const uint64_t* v_ptrs,
                         const uint32_t* seq_lens, uint32_t rows, uint32_t window) {
    REQ_HANDLE("oxi_prefill_attn");
    REQ_PTR(ctx_out && q && k_ptrs && v_ptrs && seq_lens, "oxi_prefill_attn");
    REQ_BATCH(rows, h->max_prefill_rows, "oxi_prefill_attn");
    const WaitFault flt = take_prefill_fault(h);
    OXI_CUDA(launch_prefill_attn((cudaStream_t)stream, ctx_out, q, gate, k_ptrs, v_ptrs, seq_lens,
                                 rows, window, h->dws.status, h->num_sms, h->pf_order, h->dws.status + 48, nullptr,
                                 nullptr, &h->pf_split, h->pf_part_keys, &h->pf_slab, &flt),
             "prefill_attn launch");
    return OXI_OK;
}

int32_t oxi_conv_decode(oxi_handle* h, void* stream, void* y_out, const uint64_t* conv_ptrs,
                        const void* bcx, const void* conv_w, uint32_t batch) {
    REQ_HANDLE("oxi_conv_decode");
    REQ_PTR(y_out && conv_ptrs && bcx && conv_w, "oxi_conv_decode");
    REQ_BATCH(batch, 65535u, "oxi_conv_decode");
    OXI_CUDA(launch_conv_decode((cudaStream_t)stream, y_out, conv_ptrs, bcx, conv_w, batch,
                                h->dws.status),
             "conv_decode launch");
    return OXI_OK;
}

int32_t oxi_conv_prefill(oxi_handle* h, void* stream, void* y_out, const uint64_t* carry_ptrs,
                         const uint32_t* origin, const uint32_t* local_pos, const void* bcx,
                         const void* conv_w, uint32_t rows) {
    REQ_HANDLE("oxi_conv_prefill");
    REQ_PTR(y_out && carry_ptrs && origin && local_pos && bcx && conv_w, "oxi_conv_prefill");
    REQ_BATCH(rows, h->max_prefill_rows, "oxi_conv_prefill");
    if (rows > 65535u) return fail(OXI_ERR_BATCH, "oxi_conv_prefill: at most 65535 rows per wave");
    OXI_CUDA(launch_conv_prefill((cudaStream_t)stream, y_out, carry_ptrs, origin, local_pos, bcx,
                                 conv_w, rows, h->conv_stage, h->dws.status),
             "conv_prefill launch");
    return OXI_OK;
}

int32_t oxi_embed_lookup(oxi_handle* h, void* stream, void* out, const void* table,
                         const uint32_t* token_ids, uint32_t hidden, uint32_t table_rows, uint32_t batch) {
    REQ_HANDLE("oxi_embed_lookup");
    REQ_PTR(out && table && token_ids, "oxi_embed_lookup");
    REQ_BATCH(batch, 65535u, "oxi_embed_lookup");
    if (hidden == 0 || table_rows == 0) return fail(OXI_ERR_ARG, "oxi_embed_lookup: hidden and table_rows must be positive");
    OXI_CUDA(launch_embed_lookup((cudaStream_t)stream, out, table, token_ids, hidden, table_rows, batch, h->dws.status),
             "embed_lookup launch");
    return OXI_OK;
}

int32_t oxi_argmax(oxi_handle* h, void* stream, uint32_t* tokens_out, const void* logits, uint32_t vocab,
                   uint32_t batch) {
    REQ_HANDLE("oxi_argmax");
    REQ_PTR(tokens_out && logits, "oxi_argmax");
    REQ_BATCH(batch, h->max_batch, "oxi_argmax");
    if (vocab == 0 || vocab > 0x7fffff00u) return fail(OXI_ERR_ARG, "oxi_argmax: vocab out of range");
    OXI_CUDA(launch_argmax((cudaStream_t)stream, tokens_out, logits, vocab, batch, h->num_sms, h->am_cand, h->am_count),
             "argmax launch");
    return OXI_OK;
}

int32_t oxi_qk_rmsnorm(oxi_handle* h, void* stream, void* x_io, const void* weight, float eps,
                       uint32_t num_heads, uint32_t batch) {
    REQ_HANDLE("oxi_qk_rmsnorm");
    REQ_PTR(x_io && weight, "oxi_qk_rmsnorm");
    if (batch == 0) return fail(OXI_ERR_BATCH, "oxi_qk_rmsnorm: batch is 0");
    if (num_heads == 0 || num_heads > 1024) return fail(OXI_ERR_ARG, "oxi_qk_rmsnorm: num_heads out of range");
    OXI_CUDA(launch_qk_rmsnorm((cudaStream_t)stream, x_io, weight, eps, num_heads, batch), "qk_rmsnorm launch");
    return OXI_OK;
}

int32_t oxi_rope(oxi_handle* h, void* stream, void* x_io, const void* cos_table,
                 const void* sin_table, const uint32_t* pos_ids, uint32_t num_heads,
                 uint32_t batch) {
    REQ_HANDLE("oxi_rope");
    REQ_PTR(x_io && cos_table && sin_table && pos_ids, "oxi_rope");
    if (batch == 0) return fail(OXI_ERR_BATCH, "oxi_rope: batch is 0");
    if (num_heads == 0 || num_heads > 1024) return fail(OXI_ERR_ARG, "oxi_rope: num_heads out of range");
    OXI_CUDA(launch_rope((cudaStream_t)stream, x_io, cos_table, sin_table, pos_ids, num_heads, batch), "rope launch");
    return OXI_OK;
}

int32_t oxi_kv_copy(oxi_handle* h, void* stream, const uint64_t* dst_ptrs, const void* src,
                    const uint32_t* pos_ids, uint32_t batch) {
    REQ_HANDLE("oxi_kv_copy");
    REQ_PTR(dst_ptrs && src && pos_ids, "oxi_kv_copy");
    if (batch == 0) return fail(OXI_ERR_BATCH, "oxi_kv_copy: batch is 0");
    OXI_CUDA(launch_kv_copy((cudaStream_t)stream, dst_ptrs, src, pos_ids, batch, h->dws.status), "kv_copy launch");
    return OXI_OK;
}

int32_t oxi_sigmoid_gate(oxi_handle* h, void* stream, void* ctx_io, const void* gate,
                         uint32_t batch) {
    REQ_HANDLE("oxi_sigmoid_gate");
    REQ_PTR(ctx_io && gate, "oxi_sigmoid_gate");
    if (batch == 0) return fail(OXI_ERR_BATCH, "oxi_sigmoid_gate: batch is 0");
    OXI_CUDA(launch_sigmoid_gate((cudaStream_t)stream, ctx_io, gate, batch), "sigmoid_gate launch");
    return OXI_OK;
}

// ---- linear layers on either side of the path (tensor maps over the caller's weights; host objects only)
struct oxi_linear_s {
    TmaDesc maps[4];        // boxes of 128 weight rows x 64 k; qkvg: q, k, v, gate; plain: maps[0]
    uint32_t out_features;  // plain: rows of the weight matrix; qkvg: 3088
    bool qkvg;
};

static int32_t linear_map(TmaDesc* m, const void* w, uint64_t rows, uint32_t box_rows, const char* who) {
    if (!w) return fail(OXI_ERR_NULL, who);
    if (((uintptr_t)w & 15u) != 0u) return fail(OXI_ERR_ARG, "weights must be 16-byte aligned");
    const int rc = proj_encode_map(m, w, rows, box_rows);
    if (rc == -1) return fail(OXI_ERR_NO_DEVICE, "driver has no cuTensorMapEncodeTiled");
    if (rc != 0) return fail(OXI_ERR_ARG, "cuTensorMapEncodeTiled rejected the weight matrix");
    return OXI_OK;
}

int32_t oxi_qkvg_create(oxi_linear** out, const void* wq, const void* wk, const void* wv, const void* wg) {
    if (!out) return fail(OXI_ERR_NULL, "oxi_qkvg_create: out is null");
    *out = nullptr;
    oxi_linear_s* l = new (std::nothrow) oxi_linear_s();
    if (!l) return fail(OXI_ERR_WORKSPACE, "oxi_qkvg_create: host allocation failed");
    int32_t rc = OXI_OK;
    if ((rc = linear_map(&l->maps[0], wq, NQ * HD, 128u, "oxi_qkvg_create: q_proj is null")) ||
        (rc = linear_map(&l->maps[1], wk, NKV * HD, 128u, "oxi_qkvg_create: k_proj is null")) ||
        (rc = linear_map(&l->maps[2], wv, NKV * HD, 128u, "oxi_qkvg_create: v_proj is null")) ||
        (rc = linear_map(&l->maps[3], wg, NQ, 128u, "oxi_qkvg_create: gate_proj is null"))) {
        delete l;
        return rc;
    }
    l->out_features = NQ * HD + 2 * NKV * HD + NQ;
    l->qkvg = true;
    *out = reinterpret_cast<oxi_linear*>(l);
    return OXI_OK;
}

int32_t oxi_linear_create(oxi_linear** out, const void* w, uint32_t out_features) {
    if (!out) return fail(OXI_ERR_NULL, "oxi_linear_create: out is null");
    *out = nullptr;
    if (out_features == 0 || out_features > (1u << 20)) return fail(OXI_ERR_ARG, "oxi_linear_create: out_features out of range");
    oxi_linear_s* l = new (std::nothrow) oxi_linear_s();
    if (!l) return fail(OXI_ERR_WORKSPACE, "oxi_linear_create: host allocation failed");
    const int32_t rc = linear_map(&l->maps[0], w, out_features, 128u, "oxi_linear_create: weights are null");
    if (rc != OXI_OK) {
        delete l;
        return rc;
    }
    l->out_features = out_features;
    l->qkvg = false;
    *out = reinterpret_cast<oxi_linear*>(l);
    return OXI_OK;
}

int32_t oxi_linear_destroy(oxi_linear* l) {
    delete reinterpret_cast<oxi_linear_s*>(l);
    return OXI_OK;
}

int32_t oxi_project_append(oxi_handle* h, void* stream, const oxi_linear* qkvg, const void* x, void* q_out, void* gate_out,
                           void* raw_out, const void* q_norm_w, const void* k_norm_w, const void* cos_table,
                           const void* sin_table, const uint32_t* pos_ids, const uint64_t* k_ptrs, const uint64_t* v_ptrs,
                           uint32_t rows, float eps) {
    REQ_HANDLE("oxi_project_append");
    const oxi_linear_s* l = reinterpret_cast<const oxi_linear_s*>(qkvg);
    REQ_PTR(l && x && q_out && gate_out && q_norm_w && k_norm_w && cos_table && sin_table && pos_ids && k_ptrs && v_ptrs,
            "oxi_project_append");
    if (!l->qkvg) return fail(OXI_ERR_ARG, "oxi_project_append: the weights object was not made by oxi_qkvg_create");
    REQ_BATCH(rows, (h->max_batch > h->max_prefill_rows ? h->max_batch : h->max_prefill_rows), "oxi_project_append");
    if (!(eps >= 0.0f)) return fail(OXI_ERR_ARG, "oxi_project_append: eps must be >= 0");
    if ((((uintptr_t)x | (uintptr_t)q_out | (uintptr_t)gate_out | (uintptr_t)raw_out | (uintptr_t)cos_table |
          (uintptr_t)sin_table) & 15u) != 0u)
        return fail(OXI_ERR_ARG, "oxi_project_append: x, q_out, gate_out, raw_out and the rope tables must be 16-byte aligned");
    const WaitFault flt = take_proj_fault(h);
    OXI_CUDA(launch_project_append((cudaStream_t)stream, l->maps, h->num_sms, x, rows, q_out, gate_out, raw_out, q_norm_w, k_norm_w,
                                   cos_table, sin_table, pos_ids, k_ptrs, v_ptrs, eps, h->dws.status, &flt),
             "project_append launch");
    return OXI_OK;
}

int32_t oxi_linear_forward(oxi_handle* h, void* stream, const oxi_linear* w, const void* x, void* y, uint32_t rows) {
    REQ_HANDLE("oxi_linear_forward");
    const oxi_linear_s* l = reinterpret_cast<const oxi_linear_s*>(w);
    REQ_PTR(l && x && y, "oxi_linear_forward");
    if (l->qkvg) return fail(OXI_ERR_ARG, "oxi_linear_forward: the weights object was made by oxi_qkvg_create");
    if (rows == 0 || rows > (1u << 20)) return fail(OXI_ERR_BATCH, "oxi_linear_forward: rows out of range");
    if ((((uintptr_t)x | (uintptr_t)y) & 15u) != 0u) return fail(OXI_ERR_ARG, "oxi_linear_forward: x and y must be 16-byte aligned");
    const WaitFault flt = take_proj_fault(h);
    OXI_CUDA(launch_linear((cudaStream_t)stream, l->maps, h->num_sms, l->out_features, x, rows, y, h->dws.status, &flt), "linear launch");
    return OXI_OK;
}

int32_t oxi_decode_step_host(oxi_handle* h, void* stream, void* ctx_host, const void* q_host,
                             const void* k_host, const void* v_host, const void* gate_host,
                             const void* q_norm_w_dev, const void* k_norm_w_dev,
                             const void* cos_table_dev, const void* sin_table_dev,
                             const uint32_t* pos_ids_host, const uint64_t* k_ptrs_host,
                             const uint64_t* v_ptrs_host, uint32_t batch, uint32_t layers,
                             uint32_t window, float eps) {
    REQ_HANDLE("oxi_decode_step_host");
    REQ_PTR(ctx_host && q_host && k_host && v_host && q_norm_w_dev && k_norm_w_dev &&
                cos_table_dev && sin_table_dev && pos_ids_host && k_ptrs_host && v_ptrs_host,
            "oxi_decode_step_host");
    REQ_BATCH(batch, h->max_batch, "oxi_decode_step_host");
    if (layers == 0 || layers > 4096) return fail(OXI_ERR_ARG, "oxi_decode_step_host: layers out of range");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t qb = (size_t)batch * NQ * HD * 2, kb = (size_t)batch * NKV * HD * 2;
    const size_t gb = (size_t)batch * NQ * 2, tb = (size_t)batch * 8;
    const cudaMemcpyKind H2D = cudaMemcpyHostToDevice;
    // the copy streams start after everything already enqueued on the caller's stream
    OXI_CUDA(cudaEventRecord(h->ev_start, s), "event record");
    OXI_CUDA(cudaStreamWaitEvent(h->h2d, h->ev_start, 0), "stream wait");
    OXI_CUDA(cudaStreamWaitEvent(h->d2h, h->ev_start, 0), "stream wait");
    // step metadata: only the positions cross the bus; the lengths (seq_len counts the appended
    // token) are derived on the device.  Nothing is read from pos_ids_host at enqueue time, so
    // steps may be enqueued back to back without a sync, and a captured graph of this call
    // re-reads pos_ids_host (pinned) at every replay.
    OXI_CUDA(cudaMemcpyAsync(h->stg_pos, pos_ids_host, (size_t)batch * 4, H2D, h->h2d), "pos upload");
    OXI_CUDA(launch_len_from_pos(h->h2d, h->stg_pos, h->stg_len, batch), "len_from_pos launch");
    // Layers are processed in groups of up to stg_sets layers staged side by side.  Inside a group the inputs go
    // up in chunks of 1, 1, 2, 4, 8 layers, each chunk with ONE copy per kind (the caller's arrays are layer-major,
    // the staging is compact for this batch), and the caller's stream waits once per chunk, in front of the chunk's
    // first layer.  A chunk has the compute time of all the layers before it to arrive (as long as a layer's
    // kernels take, a chunk of as many layers needs no more than ~5 GB/s of host-to-device bandwidth at the
    // benchmark shape), the first layer's kernels start after six small copies, and between the layers of a chunk
    // nothing sits in the stream, so they keep their programmatic overlap with the layer before (a wait between two
    // launches takes it away; with a wait in front of every layer the step measured 1.341 ms instead of 1.31).
    // Contexts go back layer by layer on the download stream.
    const uint32_t G = h->stg_sets;
    for (uint32_t g0 = 0; g0 < layers; g0 += G) {
        const uint32_t g1 = (g0 + G < layers) ? g0 + G : layers, gn = g1 - g0;
        if (g0 > 0) {
            // the staging is reused: the previous group's kernels and downloads must be done
            OXI_CUDA(cudaStreamWaitEvent(h->h2d, h->ev_comp[G - 1u], 0), "stream wait");
            OXI_CUDA(cudaStreamWaitEvent(s, h->ev_down_last, 0), "stream wait");
        }
        auto upload = [&](uint32_t slot, uint32_t n) -> cudaError_t {  // n layers from slot `slot` of the group
            const size_t l0 = (size_t)g0 + slot;
            cudaError_t e = cudaMemcpyAsync(h->stg_q + slot * qb, (const char*)q_host + l0 * qb, n * qb, H2D, h->h2d);
            if (e == cudaSuccess) e = cudaMemcpyAsync(h->stg_k + slot * kb, (const char*)k_host + l0 * kb, n * kb, H2D, h->h2d);
            if (e == cudaSuccess) e = cudaMemcpyAsync(h->stg_v + slot * kb, (const char*)v_host + l0 * kb, n * kb, H2D, h->h2d);
            if (e == cudaSuccess && gate_host)
                e = cudaMemcpyAsync(h->stg_gate + slot * gb, (const char*)gate_host + l0 * gb, n * gb, H2D, h->h2d);
            if (e == cudaSuccess) e = cudaMemcpyAsync(h->stg_kp + slot * tb, k_ptrs_host + l0 * batch, n * tb, H2D, h->h2d);
            if (e == cudaSuccess) e = cudaMemcpyAsync(h->stg_vp + slot * tb, v_ptrs_host + l0 * batch, n * tb, H2D, h->h2d);
            return e;
        };
        // chunk c covers slots [start(c), start(c + 1)) with start = 0, 1, 2, 4, 8, 16
        for (uint32_t c0 = 0, c = 0; c0 < gn; c++) {
            const uint32_t c1 = (c0 == 0u) ? 1u : (2u * c0 < gn ? 2u * c0 : gn);
            OXI_CUDA(upload(c0, c1 - c0), "input upload");
            OXI_CUDA(cudaEventRecord(h->ev_up[c], h->h2d), "event record");
            c0 = c1;
        }
        for (uint32_t slot = 0, c = 0; slot < gn; slot++) {
            const uint32_t l = g0 + slot;
            if (slot == 0u || (slot & (slot - 1u)) == 0u) {  // slots 0, 1, 2, 4, 8: a chunk starts here
                OXI_CUDA(cudaStreamWaitEvent(s, h->ev_up[c], 0), "stream wait");
                c++;
            }
            OXI_CUDA(launch_append_decode(s, take_dws(h), h->stg_ctx + slot * qb, h->stg_q + slot * qb, h->stg_k + slot * kb,
                                          h->stg_v + slot * kb, gate_host ? h->stg_gate + slot * gb : nullptr,
                                          (const char*)q_norm_w_dev + (size_t)l * HD * 2,
                                          (const char*)k_norm_w_dev + (size_t)l * HD * 2, cos_table_dev, sin_table_dev,
                                          h->stg_len, (const uint64_t*)(h->stg_kp + slot * tb),
                                          (const uint64_t*)(h->stg_vp + slot * tb), batch, window, eps),
                     "append_decode launch");
            OXI_CUDA(cudaEventRecord(h->ev_comp[slot], s), "event record");
            OXI_CUDA(cudaStreamWaitEvent(h->d2h, h->ev_comp[slot], 0), "stream wait");
            OXI_CUDA(cudaMemcpyAsync((char*)ctx_host + (size_t)l * qb, h->stg_ctx + slot * qb, qb, cudaMemcpyDeviceToHost, h->d2h),
                     "ctx download");
        }
        OXI_CUDA(cudaEventRecord(h->ev_down_last, h->d2h), "event record");
    }
    // the caller's stream completes only after the last download (the download stream is in order)
    OXI_CUDA(cudaStreamWaitEvent(s, h->ev_down_last, 0), "stream wait");
    return OXI_OK;
}

}  // extern "C"
