// C++ host layer above the C ABI (include/oxi_kv.h): the pieces of the reference's Rust
// engine that own the pointer tables of the KV-cache path, re-stated for a C++ host.
//
//   KvLayout / KvPool   slab addressing and the per-request lease
//                       (crates/oxide-infer-server/src/kv_pool.rs:31-251)
//   BatchSequence       what the engine asks of a sequence
//                       (crates/oxide-infer-server/src/batch_engine.rs:78-87)
//   StepTables          layer-major k/v/conv pointer tables + positions, uploaded once per
//                       step (batch_engine.rs:681-751)
//   KvPathEngine        the per-layer launch sites of the hot path
//                       (batch_engine.rs:840-899, 941-1239) on top of liboxi_kv
//
// Header-only; needs the CUDA runtime only for KvPool's owning constructor, StepTables'
// uploads and KvPathEngine.  Define OXI_HOST_NO_CUDA to use the allocator logic alone
// (externally owned slabs), e.g. in host-only unit tests.
#pragma once
#include <cstddef>
#include <cstdint>
#include <map>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

#ifndef OXI_HOST_NO_CUDA
#include <cuda_runtime.h>
#include "../../../include/oxi_kv.h"
#endif

namespace oxi_host {

constexpr size_t KV_DIM = 512;        // 4 KV heads x 128
constexpr size_t HIDDEN = 2048;       // conv channels
constexpr size_t CONV_STATE_ELEMS = 6;  // live conv-state slots per channel (kv_pool.rs:26)
constexpr size_t ELEM = 2;            // fp16

// Immutable addressing of the two slabs.  K and V of attention layer a live in planes 2a and
// 2a+1 of the KV slab, each `capacity_tokens` rows of 1024 B; conv state of (slot, conv layer c)
// is a [2048][6] block.
class KvLayout {
  public:
    KvLayout(uint64_t kv_base, uint64_t conv_base, const std::vector<bool>& is_conv, size_t capacity_tokens)
        : kv_base_(kv_base), conv_base_(conv_base), capacity_(capacity_tokens) {
        for (bool c : is_conv) {
            attn_plane_.push_back(c ? -1 : (int)n_attn_++);
            conv_plane_.push_back(c ? (int)n_conv_++ : -1);
        }
    }
    uint64_t k_cache_ptr(size_t layer, size_t tok_off) const {
        return kv_base_ + ((size_t)plane(attn_plane_, layer) * 2 * capacity_ + tok_off) * KV_DIM * ELEM;
    }
    uint64_t v_cache_ptr(size_t layer, size_t tok_off) const {
        return kv_base_ + (((size_t)plane(attn_plane_, layer) * 2 + 1) * capacity_ + tok_off) * KV_DIM * ELEM;
    }
    uint64_t conv_state_ptr(size_t layer, size_t slot) const {
        return conv_base_ + (slot * n_conv_ + (size_t)plane(conv_plane_, layer)) * conv_plane_bytes();
    }
    size_t capacity_tokens() const { return capacity_; }
    size_t num_layers() const { return attn_plane_.size(); }
    size_t num_attention_layers() const { return n_attn_; }
    size_t num_conv_layers() const { return n_conv_; }
    bool is_conv(size_t layer) const { return conv_plane_.at(layer) >= 0; }
    static constexpr size_t conv_plane_bytes() { return HIDDEN * CONV_STATE_ELEMS * ELEM; }
    size_t kv_slab_bytes() const { return n_attn_ * 2 * capacity_ * KV_DIM * ELEM; }
    uint64_t conv_base() const { return conv_base_; }

  private:
    static int plane(const std::vector<int>& v, size_t layer) {
        const int p = v.at(layer);
        if (p < 0) throw std::invalid_argument("layer has no plane of that kind");
        return p;
    }
    uint64_t kv_base_, conv_base_;
    size_t capacity_, n_attn_ = 0, n_conv_ = 0;
    std::vector<int> attn_plane_, conv_plane_;
};

struct Lease {
    size_t tok_off, tokens, slot;
};

// First-fit contiguous token ranges + a conv slot per request.  The free list is an ordered
// map start -> length, so release coalesces with both neighbours in O(log n).
class KvPool {
  public:
    // Slabs owned by the caller (or none at all: pure bookkeeping).
    KvPool(std::shared_ptr<const KvLayout> layout, size_t max_batch) : layout_(std::move(layout)) {
        if (!layout_ || layout_->capacity_tokens() == 0 || max_batch == 0)
            throw std::invalid_argument("invalid KV pool geometry");
        free_[0] = layout_->capacity_tokens();
        for (size_t s = max_batch; s-- > 0;) free_slots_.push_back(s);
    }
#ifndef OXI_HOST_NO_CUDA
    // Allocates both slabs on the current device; the capacity is halved until the KV slab fits
    // (never below 4096 tokens), as the reference does (kv_pool.rs:103-119).
    static std::unique_ptr<KvPool> create(const std::vector<bool>& is_conv, size_t max_batch, size_t capacity_tokens) {
        size_t n_attn = 0, n_conv = 0;
        for (bool c : is_conv) (c ? n_conv : n_attn)++;
        if (!n_attn || !n_conv || !max_batch || !capacity_tokens) throw std::invalid_argument("invalid KV pool geometry");
        void* kv = nullptr;
        size_t cap = capacity_tokens;
        for (;;) {
            if (cudaMalloc(&kv, n_attn * 2 * cap * KV_DIM * ELEM) == cudaSuccess) break;
            cudaGetLastError();
            if (cap <= 4096) throw std::runtime_error("KV slab allocation failed");
            cap /= 2;
        }
        void* conv = nullptr;
        const size_t conv_bytes = max_batch * n_conv * KvLayout::conv_plane_bytes();
        if (cudaMalloc(&conv, conv_bytes) != cudaSuccess) {
            cudaFree(kv);
            throw std::runtime_error("conv-state slab allocation failed");
        }
        cudaMemset(kv, 0, n_attn * 2 * cap * KV_DIM * ELEM);
        cudaMemset(conv, 0, conv_bytes);
        auto layout = std::make_shared<KvLayout>((uint64_t)kv, (uint64_t)conv, is_conv, cap);
        std::unique_ptr<KvPool> p(new KvPool(layout, max_batch));
        p->owned_kv_ = kv;
        p->owned_conv_ = conv;
        return p;
    }
    ~KvPool() {
        if (owned_kv_) cudaFree(owned_kv_);
        if (owned_conv_) cudaFree(owned_conv_);
    }
#endif
    KvPool(const KvPool&) = delete;
    KvPool& operator=(const KvPool&) = delete;

    std::shared_ptr<const KvLayout> layout() const { return layout_; }
    size_t free_tokens() const {
        size_t n = 0;
        for (auto& r : free_) n += r.second;
        return n;
    }
    size_t free_slots() const { return free_slots_.size(); }
    size_t fragments() const { return free_.size(); }

    // Lease `tokens` contiguous rows and a conv slot; the slot's conv state is zeroed on `stream`
    // (kv_pool.rs:175-218).  nullopt when no slot or no range fits.
    std::optional<Lease> acquire(size_t tokens, void* stream = nullptr) {
        if (tokens == 0 || tokens > layout_->capacity_tokens() || free_slots_.empty()) return std::nullopt;
        auto it = free_.begin();
        while (it != free_.end() && it->second < tokens) ++it;
        if (it == free_.end()) return std::nullopt;
        const size_t start = it->first, len = it->second;
        const size_t slot = free_slots_.back();
#ifndef OXI_HOST_NO_CUDA
        if (layout_->conv_base() && layout_->num_conv_layers()) {
            const size_t bytes = layout_->num_conv_layers() * KvLayout::conv_plane_bytes();
            if (cudaMemsetAsync((void*)(layout_->conv_base() + slot * bytes), 0, bytes, (cudaStream_t)stream) != cudaSuccess) {
                cudaGetLastError();
                return std::nullopt;
            }
        }
#else
        (void)stream;
#endif
        free_slots_.pop_back();
        free_.erase(it);
        if (len > tokens) free_[start + tokens] = len - tokens;
        return Lease{start, tokens, slot};
    }

    void release(const Lease& l) {
        free_slots_.push_back(l.slot);
        size_t start = l.tok_off, len = l.tokens;
        auto next = free_.lower_bound(start);
        if (next != free_.begin()) {
            auto prev = std::prev(next);
            if (prev->first + prev->second == start) {
                start = prev->first;
                len += prev->second;
                free_.erase(prev);
            }
        }
        if (next != free_.end() && start + len == next->first) {
            len += next->second;
            free_.erase(next);
        }
        free_[start] = len;
    }

  private:
    std::shared_ptr<const KvLayout> layout_;
    std::map<size_t, size_t> free_;
    std::vector<size_t> free_slots_;
    void* owned_kv_ = nullptr;
    void* owned_conv_ = nullptr;
};

// What the engine needs from a live sequence (batch_engine.rs:78-87, minus hidden_ptr which
// belongs to the parts of the model outside this path).
struct BatchSequence {
    virtual ~BatchSequence() = default;
    virtual uint64_t k_cache_ptr(size_t layer) const = 0;
    virtual uint64_t v_cache_ptr(size_t layer) const = 0;
    virtual uint64_t conv_state_ptr(size_t layer) const = 0;
};

class LeasedSequence : public BatchSequence {
  public:
    LeasedSequence(std::shared_ptr<const KvLayout> layout, Lease lease) : layout_(std::move(layout)), lease_(lease) {}
    uint64_t k_cache_ptr(size_t layer) const override { return layout_->k_cache_ptr(layer, lease_.tok_off); }
    uint64_t v_cache_ptr(size_t layer) const override { return layout_->v_cache_ptr(layer, lease_.tok_off); }
    uint64_t conv_state_ptr(size_t layer) const override { return layout_->conv_state_ptr(layer, lease_.slot); }
    const Lease& lease() const { return lease_; }

  private:
    std::shared_ptr<const KvLayout> layout_;
    Lease lease_;
};

// Host image of one step's tables, layer-major: tbl[layer * b + i] (batch_engine.rs:709-731).
// seq_lens = pos_ids + 1: the key count includes the token appended in this step.
struct StepTablesHost {
    size_t batch = 0, layers = 0;
    std::vector<uint64_t> k_ptrs, v_ptrs, conv_ptrs;
    std::vector<uint32_t> pos_ids, seq_lens;

    void build(const std::vector<const BatchSequence*>& seqs, const std::vector<uint32_t>& positions, const KvLayout& layout) {
        if (seqs.size() != positions.size()) throw std::invalid_argument("one position per sequence");
        batch = seqs.size();
        layers = layout.num_layers();
        k_ptrs.assign(layers * batch, 0);
        v_ptrs.assign(layers * batch, 0);
        conv_ptrs.assign(layers * batch, 0);
        pos_ids = positions;
        seq_lens.resize(batch);
        for (size_t i = 0; i < batch; i++) seq_lens[i] = positions[i] + 1u;
        for (size_t l = 0; l < layers; l++)
            for (size_t i = 0; i < batch; i++) {
                if (layout.is_conv(l)) {
                    conv_ptrs[l * batch + i] = seqs[i]->conv_state_ptr(l);
                } else {
                    k_ptrs[l * batch + i] = seqs[i]->k_cache_ptr(l);
                    v_ptrs[l * batch + i] = seqs[i]->v_cache_ptr(l);
                }
            }
    }
};

#ifndef OXI_HOST_NO_CUDA
// Device copy of the tables; uploads are asynchronous on the caller's stream from pinned
// memory (batch_engine.rs:732-740), so nothing synchronises on the decode path.
class StepTables {
  public:
    StepTables(size_t max_batch, size_t layers) : max_batch_(max_batch), layers_(layers) {
        const size_t n = max_batch * layers;
        check(cudaMalloc((void**)&d_k_, n * 8), "tables");
        check(cudaMalloc((void**)&d_v_, n * 8), "tables");
        check(cudaMalloc((void**)&d_conv_, n * 8), "tables");
        check(cudaMalloc((void**)&d_pos_, max_batch * 4), "tables");
        check(cudaMalloc((void**)&d_len_, max_batch * 4), "tables");
        check(cudaMallocHost((void**)&h_, (3 * n * 8) + 2 * max_batch * 4), "pinned tables");
    }
    ~StepTables() {
        cudaFree(d_k_); cudaFree(d_v_); cudaFree(d_conv_); cudaFree(d_pos_); cudaFree(d_len_);
        if (h_) cudaFreeHost(h_);
    }
    StepTables(const StepTables&) = delete;
    StepTables& operator=(const StepTables&) = delete;

    void upload(const StepTablesHost& t, cudaStream_t s) {
        if (t.batch > max_batch_ || t.layers != layers_) throw std::invalid_argument("tables exceed the allocated size");
        batch_ = t.batch;
        const size_t n = t.batch * t.layers;
        uint64_t* hk = (uint64_t*)h_;
        uint64_t* hv = hk + max_batch_ * layers_;
        uint64_t* hc = hv + max_batch_ * layers_;
        uint32_t* hp = (uint32_t*)(hc + max_batch_ * layers_);
        uint32_t* hl = hp + max_batch_;
        std::copy(t.k_ptrs.begin(), t.k_ptrs.end(), hk);
        std::copy(t.v_ptrs.begin(), t.v_ptrs.end(), hv);
        std::copy(t.conv_ptrs.begin(), t.conv_ptrs.end(), hc);
        std::copy(t.pos_ids.begin(), t.pos_ids.end(), hp);
        std::copy(t.seq_lens.begin(), t.seq_lens.end(), hl);
        check(cudaMemcpyAsync(d_k_, hk, n * 8, cudaMemcpyHostToDevice, s), "upload");
        check(cudaMemcpyAsync(d_v_, hv, n * 8, cudaMemcpyHostToDevice, s), "upload");
        check(cudaMemcpyAsync(d_conv_, hc, n * 8, cudaMemcpyHostToDevice, s), "upload");
        check(cudaMemcpyAsync(d_pos_, hp, t.batch * 4, cudaMemcpyHostToDevice, s), "upload");
        check(cudaMemcpyAsync(d_len_, hl, t.batch * 4, cudaMemcpyHostToDevice, s), "upload");
    }
    size_t batch() const { return batch_; }
    const uint64_t* k_ptrs(size_t layer) const { return d_k_ + layer * batch_; }
    const uint64_t* v_ptrs(size_t layer) const { return d_v_ + layer * batch_; }
    const uint64_t* conv_ptrs(size_t layer) const { return d_conv_ + layer * batch_; }
    const uint32_t* pos_ids() const { return d_pos_; }
    const uint32_t* seq_lens() const { return d_len_; }
    uint32_t* pos_ids_mut() { return d_pos_; }
    uint32_t* seq_lens_mut() { return d_len_; }

  private:
    static void check(cudaError_t e, const char* what) {
        if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
    }
    size_t max_batch_, layers_, batch_ = 0;
    uint64_t *d_k_ = nullptr, *d_v_ = nullptr, *d_conv_ = nullptr;
    uint32_t *d_pos_ = nullptr, *d_len_ = nullptr;
    void* h_ = nullptr;
};

// The hot-path launch sites of one layer, on the caller's stream.  Throws std::runtime_error
// with the library's message on a non-zero status (the engine's anyhow style).
class KvPathEngine {
  public:
    KvPathEngine(int device, uint32_t max_batch, uint32_t max_seq_len, uint32_t max_prefill_rows) {
        const int32_t rc = oxi_create(&h_, device, max_batch, max_seq_len, max_prefill_rows);
        if (rc != OXI_OK) throw std::runtime_error(std::string("oxi_create: ") + oxi_last_error_string());
    }
    ~KvPathEngine() { oxi_destroy(h_); }
    KvPathEngine(const KvPathEngine&) = delete;
    KvPathEngine& operator=(const KvPathEngine&) = delete;

    // batch_engine.rs:941-1239 for attention layer `layer`: append, then gated decode attention.
    void attention_decode(cudaStream_t s, const StepTables& t, size_t layer, void* ctx, void* q_io, const void* k,
                          const void* v, const void* gate, const void* q_norm_w, const void* k_norm_w,
                          const void* cos_table, const void* sin_table, uint32_t window, float eps = 1e-5f) {
        ok(oxi_append_decode(h_, s, ctx, q_io, k, v, gate, q_norm_w, k_norm_w, cos_table, sin_table, t.pos_ids(),
                             t.seq_lens(), t.k_ptrs(layer), t.v_ptrs(layer), (uint32_t)t.batch(), window, eps),
           "oxi_append_decode");
    }
    // batch_engine.rs:840-899 for conv layer `layer` (decode rows).
    void conv_decode(cudaStream_t s, const StepTables& t, size_t layer, void* y, const void* bcx, const void* conv_w) {
        ok(oxi_conv_decode(h_, s, y, t.conv_ptrs(layer), bcx, conv_w, (uint32_t)t.batch()), "oxi_conv_decode");
    }
    // Moves every row of the tables one token ahead on the device.  While the batch membership is
    // unchanged, a captured graph of (all layers + this call) replays step after step with no upload
    // (the engine re-uploads its tables every step, batch_engine.rs:709-740).
    void advance(cudaStream_t s, StepTables& t, uint32_t delta = 1) {
        ok(oxi_advance_step(h_, s, t.pos_ids_mut(), t.seq_lens_mut(), (uint32_t)t.batch(), delta), "oxi_advance_step");
    }
    uint32_t device_status(cudaStream_t s) {
        uint32_t bits = 0;
        ok(oxi_device_status(h_, s, &bits), "oxi_device_status");
        return bits;
    }
    oxi_handle* handle() { return h_; }

  private:
    static void ok(int32_t rc, const char* what) {
        if (rc != OXI_OK) throw std::runtime_error(std::string(what) + ": " + oxi_last_error_string());
    }
    oxi_handle* h_ = nullptr;
};
#endif  // OXI_HOST_NO_CUDA

}  // namespace oxi_host
