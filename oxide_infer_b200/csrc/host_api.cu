// C API over the host layer (host/kv_host.hpp): the slab pool with its per-request leases and the
// layer-major step tables, for hosts that cannot include a C++ header (the reference's engine is
// Rust: crates/oxide-infer-server/src/kv_pool.rs and batch_engine.rs:709-740).
// No exception crosses the ABI: every entry returns an OXI_* status or a plain value.
#include <cstdio>
#include <new>

#include "../../include/oxi_kv.h"
#include "host/kv_host.hpp"

using oxi_host::KvLayout;
using oxi_host::KvPool;
using oxi_host::Lease;

struct oxi_kv_pool {
    std::unique_ptr<KvPool> pool;
    uint32_t max_batch;
};

// Step tables: a host image (rows set one by one), a ring of pinned staging blocks so that a new
// upload never overwrites one that has not executed yet, and the device tables the kernels read.
struct oxi_step_tables {
    static constexpr int RING = 4;
    std::shared_ptr<const KvLayout> layout;
    uint32_t max_batch = 0, layers = 0, batch = 0;
    std::vector<uint64_t> k, v, conv;   // [layer][max_batch] host image (row stride max_batch)
    std::vector<uint32_t> pos;
    uint64_t *d_k = nullptr, *d_v = nullptr, *d_conv = nullptr;  // [layer][batch] after an upload
    uint32_t *d_pos = nullptr, *d_len = nullptr;
    unsigned char* stage[RING] = {};
    cudaEvent_t done[RING] = {};
    uint32_t next = 0;
    size_t stage_bytes() const { return (size_t)3 * layers * max_batch * 8 + (size_t)2 * max_batch * 4; }
};

static thread_local char g_host_err[200] = "";
static int32_t hfail(int32_t code, const char* msg) {
    snprintf(g_host_err, sizeof(g_host_err), "%s", msg);
    return code;
}

extern "C" {

const char* oxi_host_last_error_string(void) { return g_host_err; }

int32_t oxi_pool_create(oxi_kv_pool** out, const uint8_t* layer_is_conv, uint32_t num_layers, uint32_t max_batch,
                        uint64_t capacity_tokens) {
    if (!out || !layer_is_conv) return hfail(OXI_ERR_NULL, "oxi_pool_create: null argument");
    *out = nullptr;
    if (num_layers == 0 || max_batch == 0 || capacity_tokens == 0) return hfail(OXI_ERR_ARG, "invalid KV pool geometry");
    try {
        std::vector<bool> kinds(layer_is_conv, layer_is_conv + num_layers);
        std::unique_ptr<oxi_kv_pool> p(new oxi_kv_pool());
        p->pool = KvPool::create(kinds, max_batch, (size_t)capacity_tokens);
        p->max_batch = max_batch;
        *out = p.release();
        return OXI_OK;
    } catch (const std::invalid_argument& e) {
        return hfail(OXI_ERR_ARG, e.what());
    } catch (const std::exception& e) {
        return hfail(OXI_ERR_WORKSPACE, e.what());
    }
}

int32_t oxi_pool_destroy(oxi_kv_pool* p) {
    delete p;
    return OXI_OK;
}

uint64_t oxi_pool_capacity_tokens(const oxi_kv_pool* p) { return p ? p->pool->layout()->capacity_tokens() : 0; }
uint64_t oxi_pool_free_tokens(const oxi_kv_pool* p) { return p ? p->pool->free_tokens() : 0; }
uint32_t oxi_pool_free_slots(const oxi_kv_pool* p) { return p ? (uint32_t)p->pool->free_slots() : 0; }

int32_t oxi_pool_acquire(oxi_kv_pool* p, void* stream, uint64_t tokens, oxi_lease* out) {
    if (!p || !out) return hfail(OXI_ERR_NULL, "oxi_pool_acquire: null argument");
    const auto l = p->pool->acquire((size_t)tokens, stream);
    if (!l) return hfail(OXI_ERR_WORKSPACE, "oxi_pool_acquire: no conv slot or no contiguous range of that many tokens is free");
    out->tok_off = l->tok_off;
    out->tokens = l->tokens;
    out->slot = l->slot;
    return OXI_OK;
}

int32_t oxi_pool_release(oxi_kv_pool* p, const oxi_lease* l) {
    if (!p || !l) return hfail(OXI_ERR_NULL, "oxi_pool_release: null argument");
    if (l->tokens == 0 || l->tok_off + l->tokens > p->pool->layout()->capacity_tokens() || l->slot >= p->max_batch)
        return hfail(OXI_ERR_ARG, "oxi_pool_release: not a lease of this pool");
    p->pool->release(Lease{(size_t)l->tok_off, (size_t)l->tokens, (size_t)l->slot});
    return OXI_OK;
}

// 0 when the layer is not of that kind (or an argument is null)
uint64_t oxi_pool_k_ptr(const oxi_kv_pool* p, uint32_t layer, const oxi_lease* l) {
    if (!p || !l || layer >= p->pool->layout()->num_layers() || p->pool->layout()->is_conv(layer)) return 0;
    return p->pool->layout()->k_cache_ptr(layer, (size_t)l->tok_off);
}
uint64_t oxi_pool_v_ptr(const oxi_kv_pool* p, uint32_t layer, const oxi_lease* l) {
    if (!p || !l || layer >= p->pool->layout()->num_layers() || p->pool->layout()->is_conv(layer)) return 0;
    return p->pool->layout()->v_cache_ptr(layer, (size_t)l->tok_off);
}
uint64_t oxi_pool_conv_ptr(const oxi_kv_pool* p, uint32_t layer, const oxi_lease* l) {
    if (!p || !l || layer >= p->pool->layout()->num_layers() || !p->pool->layout()->is_conv(layer)) return 0;
    return p->pool->layout()->conv_state_ptr(layer, (size_t)l->slot);
}

int32_t oxi_tables_destroy(oxi_step_tables* t) {
    if (!t) return OXI_OK;
    cudaFree(t->d_k);
    cudaFree(t->d_v);
    cudaFree(t->d_conv);
    cudaFree(t->d_pos);
    cudaFree(t->d_len);
    for (int i = 0; i < oxi_step_tables::RING; i++) {
        if (t->stage[i]) cudaFreeHost(t->stage[i]);
        if (t->done[i]) cudaEventDestroy(t->done[i]);
    }
    cudaGetLastError();
    delete t;
    return OXI_OK;
}

int32_t oxi_tables_create(oxi_step_tables** out, const oxi_kv_pool* pool, uint32_t max_batch) {
    if (!out || !pool) return hfail(OXI_ERR_NULL, "oxi_tables_create: null argument");
    *out = nullptr;
    if (max_batch == 0 || max_batch > 1024) return hfail(OXI_ERR_BATCH, "oxi_tables_create: max_batch must be 1..1024");
    oxi_step_tables* t = new (std::nothrow) oxi_step_tables();
    if (!t) return hfail(OXI_ERR_WORKSPACE, "oxi_tables_create: host allocation failed");
    t->layout = pool->pool->layout();
    t->max_batch = max_batch;
    t->layers = (uint32_t)t->layout->num_layers();
    const size_t n = (size_t)t->layers * max_batch;
    t->k.assign(n, 0);
    t->v.assign(n, 0);
    t->conv.assign(n, 0);
    t->pos.assign(max_batch, 0);
    cudaError_t e = cudaMalloc((void**)&t->d_k, n * 8);
    if (e == cudaSuccess) e = cudaMalloc((void**)&t->d_v, n * 8);
    if (e == cudaSuccess) e = cudaMalloc((void**)&t->d_conv, n * 8);
    if (e == cudaSuccess) e = cudaMalloc((void**)&t->d_pos, (size_t)max_batch * 4);
    if (e == cudaSuccess) e = cudaMalloc((void**)&t->d_len, (size_t)max_batch * 4);
    for (int i = 0; i < oxi_step_tables::RING && e == cudaSuccess; i++) {
        e = cudaMallocHost((void**)&t->stage[i], t->stage_bytes());
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&t->done[i], cudaEventDisableTiming);
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        oxi_tables_destroy(t);
        return hfail((int32_t)e, cudaGetErrorString(e));
    }
    *out = t;
    return OXI_OK;
}

int32_t oxi_tables_set_row(oxi_step_tables* t, uint32_t row, const oxi_lease* l, uint32_t position) {
    if (!t || !l) return hfail(OXI_ERR_NULL, "oxi_tables_set_row: null argument");
    if (row >= t->max_batch) return hfail(OXI_ERR_BATCH, "oxi_tables_set_row: row beyond max_batch");
    if ((uint64_t)position >= l->tokens) return hfail(OXI_ERR_ARG, "oxi_tables_set_row: position beyond the lease");
    for (uint32_t layer = 0; layer < t->layers; layer++) {
        const size_t i = (size_t)layer * t->max_batch + row;
        if (t->layout->is_conv(layer)) {
            t->conv[i] = t->layout->conv_state_ptr(layer, (size_t)l->slot);
        } else {
            t->k[i] = t->layout->k_cache_ptr(layer, (size_t)l->tok_off);
            t->v[i] = t->layout->v_cache_ptr(layer, (size_t)l->tok_off);
        }
    }
    t->pos[row] = position;
    return OXI_OK;
}

int32_t oxi_tables_upload(oxi_step_tables* t, void* stream, uint32_t batch) {
    if (!t) return hfail(OXI_ERR_NULL, "oxi_tables_upload: null argument");
    if (batch == 0 || batch > t->max_batch) return hfail(OXI_ERR_BATCH, "oxi_tables_upload: batch is 0 or exceeds max_batch");
    cudaStream_t s = (cudaStream_t)stream;
    const uint32_t slot = t->next++ % oxi_step_tables::RING;
    // the staging block's previous upload (RING uploads ago) must have executed before it is rewritten
    cudaError_t e = cudaEventSynchronize(t->done[slot]);
    if (e != cudaSuccess) return hfail((int32_t)e, cudaGetErrorString(e));
    const size_t n = (size_t)t->layers * batch;
    uint64_t* hk = (uint64_t*)t->stage[slot];
    uint64_t* hv = hk + n;
    uint64_t* hc = hv + n;
    uint32_t* hp = (uint32_t*)(hc + n);
    uint32_t* hl = hp + batch;
    for (uint32_t layer = 0; layer < t->layers; layer++)
        for (uint32_t i = 0; i < batch; i++) {  // compact to row stride `batch`: tbl[layer * batch + i]
            hk[(size_t)layer * batch + i] = t->k[(size_t)layer * t->max_batch + i];
            hv[(size_t)layer * batch + i] = t->v[(size_t)layer * t->max_batch + i];
            hc[(size_t)layer * batch + i] = t->conv[(size_t)layer * t->max_batch + i];
        }
    for (uint32_t i = 0; i < batch; i++) {
        hp[i] = t->pos[i];
        hl[i] = t->pos[i] + 1u;  // the key count includes the token appended in this step
    }
    e = cudaMemcpyAsync(t->d_k, hk, n * 8, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(t->d_v, hv, n * 8, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(t->d_conv, hc, n * 8, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(t->d_pos, hp, (size_t)batch * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(t->d_len, hl, (size_t)batch * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaEventRecord(t->done[slot], s);
    if (e != cudaSuccess) return hfail((int32_t)e, cudaGetErrorString(e));
    t->batch = batch;
    return OXI_OK;
}

int32_t oxi_tables_advance(oxi_handle* h, oxi_step_tables* t, void* stream, uint32_t delta) {
    if (!h || !t) return hfail(OXI_ERR_NULL, "oxi_tables_advance: null argument");
    if (t->batch == 0) return hfail(OXI_ERR_BATCH, "oxi_tables_advance: nothing uploaded yet");
    for (uint32_t i = 0; i < t->batch; i++) t->pos[i] += delta;  // the host image follows the device tables
    return oxi_advance_step(h, stream, t->d_pos, t->d_len, t->batch, delta);
}

uint32_t oxi_tables_batch(const oxi_step_tables* t) { return t ? t->batch : 0; }
const uint64_t* oxi_tables_k_ptrs(const oxi_step_tables* t, uint32_t layer) {
    return (t && layer < t->layers) ? t->d_k + (size_t)layer * t->batch : nullptr;
}
const uint64_t* oxi_tables_v_ptrs(const oxi_step_tables* t, uint32_t layer) {
    return (t && layer < t->layers) ? t->d_v + (size_t)layer * t->batch : nullptr;
}
const uint64_t* oxi_tables_conv_ptrs(const oxi_step_tables* t, uint32_t layer) {
    return (t && layer < t->layers) ? t->d_conv + (size_t)layer * t->batch : nullptr;
}
const uint32_t* oxi_tables_pos_ids(const oxi_step_tables* t) { return t ? t->d_pos : nullptr; }
const uint32_t* oxi_tables_seq_lens(const oxi_step_tables* t) { return t ? t->d_len : nullptr; }

}  // extern "C"
