// C++ host layer above the C ABI (include/oxi_kv.h): the pieces of the reference's Rust
// engine that own the pointer tables of the KV-cache path, re-stated for a C++ host.
//
//   KvLayout / KvPool   slab addressing and the per-request lease
//                       (crates/oxide-infer-server/src/kv_pool.rs:31-251)
//   BatchSequence       what the engine asks of a sequence
//                       (crates/oxide-infer-server/src/batch_engine.rs:78-87)
//   StepTables          layer-major k/v/conv pointer tables + positions, uploaded once per
//                       step (batch_engine.rs:681-751)
//   PagedKvPool / PagedBlockManager / PagedStepTables
//                       block pool, per-sequence block lists with shared-prefix reference counts
//                       and the step's block tables (crates/oxide-infer-core/src/paged_pool.rs,
//                       crates/oxide-infer-scheduler/src/block_manager.rs)
//   PrefillPlanner      prompts -> chunks -> waves (bin/server.rs:1076-1112)
//   WaveTables          a wave's per-row tables: positions, chunk origins, carry-state and K/V
//                       pointers (PrefillMeta, batch_engine.rs:156-160; bin/server.rs:1113-1141)
//   KvPathEngine        the per-layer launch sites of the hot path
//                       (batch_engine.rs:840-899, 941-1239) on top of liboxi_kv
//
// Header-only; needs the CUDA runtime only for KvPool's owning constructor, StepTables'
// uploads and KvPathEngine.  Define OXI_HOST_NO_CUDA to use the allocator logic alone
// (externally owned slabs), e.g. in host-only unit tests.
#pragma once
#include <algorithm>
#include <cstddef>
#include <cstdint>
#include <deque>
#include <map>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <unordered_map>
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

// ---- paged K/V (core/src/paged_pool.rs, scheduler/src/block_manager.rs) -----------------------

// Geometry of the paged pool: every block holds K and V rows of all attention layers,
// [layer][K | V][block_size tokens][4 KV heads][128] f16 (paged_pool.rs:11-24 with the path's
// 4 heads x 128 dims).
struct PagedPoolConfig {
    size_t num_blocks = 0, block_size = 0, num_layers = 0;
    size_t rows_per_block() const { return 2 * num_layers * block_size; }
    size_t block_bytes() const { return rows_per_block() * KV_DIM * ELEM; }
};

// Physical blocks and their free list (paged_pool.rs:27-75): blocks are handed out in the order
// 0, 1, 2, ...; a freed block goes to the back of the queue.
class PagedKvPool {
  public:
    // Memory owned by the caller (or none: pure bookkeeping with base 0).
    PagedKvPool(uint64_t base, const PagedPoolConfig& cfg) : base_(base), cfg_(cfg) {
        const size_t bs = cfg.block_size;
        if (!cfg.num_blocks || !cfg.num_layers || bs < 16 || bs > 256 || (bs & (bs - 1)))
            throw std::invalid_argument("paged pool: block_size must be 16, 32, 64, 128 or 256; blocks and layers > 0");
        for (size_t i = 0; i < cfg.num_blocks; i++) free_.push_back(i);
    }
#ifndef OXI_HOST_NO_CUDA
    static std::shared_ptr<PagedKvPool> create(const PagedPoolConfig& cfg) {
        void* p = nullptr;
        if (cudaMalloc(&p, cfg.num_blocks * cfg.block_bytes()) != cudaSuccess) throw std::runtime_error("paged pool allocation failed");
        cudaMemset(p, 0, cfg.num_blocks * cfg.block_bytes());
        std::shared_ptr<PagedKvPool> pool;
        try {
            pool.reset(new PagedKvPool((uint64_t)p, cfg));
        } catch (...) {
            cudaFree(p);
            throw;
        }
        pool->owned_ = p;
        return pool;
    }
    ~PagedKvPool() {
        if (owned_) cudaFree(owned_);
    }
#endif
    PagedKvPool(const PagedKvPool&) = delete;
    PagedKvPool& operator=(const PagedKvPool&) = delete;

    std::optional<size_t> allocate_block() {
        if (free_.empty()) return std::nullopt;
        const size_t b = free_.front();
        free_.pop_front();
        return b;
    }
    void free_block(size_t block) { free_.push_back(block); }
    size_t free_block_count() const { return free_.size(); }
    const PagedPoolConfig& config() const { return cfg_; }
    // First K (V) row of attention layer `layer` inside block 0; block i is block_bytes() further.
    uint64_t k_rows(size_t layer) const { return base_ + (2 * layer) * cfg_.block_size * KV_DIM * ELEM; }
    uint64_t v_rows(size_t layer) const { return base_ + (2 * layer + 1) * cfg_.block_size * KV_DIM * ELEM; }

  private:
    uint64_t base_;
    PagedPoolConfig cfg_;
    std::deque<size_t> free_;
    void* owned_ = nullptr;
};

// Logical-to-physical block lists of the live sequences with reference counts for shared prefix
// blocks (block_manager.rs:17-131).  Not thread-safe: one scheduler thread owns it.
class PagedBlockManager {
  public:
    explicit PagedBlockManager(std::shared_ptr<PagedKvPool> pool) : pool_(std::move(pool)) {
        if (!pool_) throw std::invalid_argument("paged block manager needs a pool");
    }
    size_t block_size() const { return pool_->config().block_size; }

    // Blocks for the first num_tokens tokens of a new sequence: the shared prefix blocks are
    // adopted (one more reference each), the rest come from the pool.  If the pool runs dry the
    // blocks taken so far are given back and std::runtime_error is thrown.
    void allocate_for_seq(uint64_t seq_id, size_t num_tokens, const std::vector<size_t>& shared_blocks = {}) {
        if (tables_.count(seq_id)) throw std::invalid_argument("sequence already has a block table");
        const size_t needed = (num_tokens + block_size() - 1) / block_size();
        std::vector<size_t> blocks;
        for (size_t b : shared_blocks) {
            ++refs_[b];
            blocks.push_back(b);
        }
        while (blocks.size() < needed) {
            const auto b = pool_->allocate_block();
            if (!b) {
                for (size_t x : blocks) drop(x);
                throw std::runtime_error("paged KV pool exhausted");
            }
            refs_[*b] = 1;
            blocks.push_back(*b);
        }
        tables_[seq_id] = std::move(blocks);
    }
    // Called before the token at position current_token_len is appended: a new block is taken
    // only when that position opens a block.  Returns the new block, if any.
    std::optional<size_t> append_token(uint64_t seq_id, size_t current_token_len) {
        auto it = tables_.find(seq_id);
        if (it == tables_.end()) throw std::invalid_argument("unknown sequence");
        if (current_token_len % block_size() != 0) return std::nullopt;
        const auto b = pool_->allocate_block();
        if (!b) throw std::runtime_error("paged KV pool exhausted");
        refs_[*b] = 1;
        it->second.push_back(*b);
        return b;
    }
    const std::vector<size_t>* get_block_table(uint64_t seq_id) const {
        auto it = tables_.find(seq_id);
        return it == tables_.end() ? nullptr : &it->second;
    }
    // Drops the sequence; a block returns to the pool when its last reference goes.
    void free_seq(uint64_t seq_id) {
        auto it = tables_.find(seq_id);
        if (it == tables_.end()) return;
        for (size_t b : it->second) drop(b);
        tables_.erase(it);
    }
    const PagedKvPool& pool() const { return *pool_; }

  private:
    void drop(size_t b) {
        auto r = refs_.find(b);
        if (r == refs_.end()) return;
        if (r->second > 0) --r->second;
        if (r->second == 0) {
            refs_.erase(r);
            pool_->free_block(b);
        }
    }
    std::shared_ptr<PagedKvPool> pool_;
    std::unordered_map<uint64_t, std::vector<size_t>> tables_;
    std::unordered_map<size_t, size_t> refs_;
};

// Host image of one decode step over the paged layout: block_tables[b][i] = block of tokens
// [i * block_size, (i + 1) * block_size) of row b, padded with 0.
struct PagedStepTablesHost {
    size_t batch = 0, max_blocks = 0;
    std::vector<uint32_t> block_tables, pos_ids, seq_lens;

    void build(const PagedBlockManager& mgr, const std::vector<uint64_t>& seq_ids, const std::vector<uint32_t>& positions,
               size_t max_blocks_per_row) {
        if (seq_ids.size() != positions.size()) throw std::invalid_argument("one position per sequence");
        batch = seq_ids.size();
        max_blocks = max_blocks_per_row;
        block_tables.assign(batch * max_blocks, 0u);
        pos_ids = positions;
        seq_lens.resize(batch);
        for (size_t i = 0; i < batch; i++) {
            seq_lens[i] = positions[i] + 1u;
            const std::vector<size_t>* t = mgr.get_block_table(seq_ids[i]);
            if (!t) throw std::invalid_argument("unknown sequence");
            if (t->size() > max_blocks || (size_t)positions[i] / mgr.block_size() >= t->size())
                throw std::invalid_argument("block table does not cover the step's position");
            for (size_t j = 0; j < t->size(); j++) block_tables[i * max_blocks + j] = (uint32_t)(*t)[j];
        }
    }
};

// ---- prefill waves (bin/server.rs:1076-1131) --------------------------------------------------

// Rows [start, start + len) of request `req`'s prompt, consecutive rows of one wave.
struct WaveChunk {
    size_t req, start, len;
    bool operator==(const WaveChunk& o) const { return req == o.req && start == o.start && len == o.len; }
};

// Cuts prompts into chunks of at most max_rows tokens and packs whole chunks into waves of at most
// max_rows rows, as the reference's worker does: requests in order of increasing prompt length
// (stable), a request's chunks in order, a wave takes the next chunks for as long as they fit.
// The chunk rows of a request stay contiguous inside a wave; the request's persistent conv state
// carries the 6-token history across its chunks, which therefore never share a wave.
class PrefillPlanner {
  public:
    PrefillPlanner(const std::vector<size_t>& prompt_lens, size_t max_rows) : max_rows_(max_rows) {
        if (max_rows == 0) throw std::invalid_argument("a wave needs at least one row");
        std::vector<size_t> order(prompt_lens.size());
        for (size_t i = 0; i < order.size(); i++) order[i] = i;
        std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) { return prompt_lens[a] < prompt_lens[b]; });
        for (size_t r : order)
            for (size_t start = 0; start < prompt_lens[r]; start += max_rows)
                chunks_.push_back({r, start, std::min(max_rows, prompt_lens[r] - start)});
    }
    // The next wave, or an empty vector when every chunk has been handed out.
    std::vector<WaveChunk> next() {
        std::vector<WaveChunk> wave;
        size_t used = 0;
        while (next_ < chunks_.size()) {
            const WaveChunk& c = chunks_[next_];
            if (used + c.len > max_rows_) break;
            // two chunks of one request depend on each other through the carried conv state (with the
            // sizes above they never fit one wave anyway: all but a request's last chunk fill a wave)
            if (!wave.empty() && wave.back().req == c.req) break;
            wave.push_back(c);
            used += c.len;
            ++next_;
        }
        return wave;
    }
    size_t chunks_left() const { return chunks_.size() - next_; }

  private:
    size_t max_rows_, next_ = 0;
    std::vector<WaveChunk> chunks_;
};

// Host image of one wave's per-row tables (PrefillMeta, batch_engine.rs:156-160, and the rows of
// bin/server.rs:1113-1131): row r of the wave is token start + j of its request, at cache
// position first_pos[req] + start + j.  Pointer tables are layer-major, tbl[layer * rows + r].
struct WaveTablesHost {
    size_t rows = 0, layers = 0;
    std::vector<uint64_t> k_ptrs, v_ptrs, carry_ptrs;
    std::vector<uint32_t> pos_ids, seq_lens, origins, local_pos, row_req;

    // seqs[req] is the request's sequence; first_pos[req] the cache position of its prompt's first
    // token (0 unless a prefix is already cached).
    void build(const std::vector<WaveChunk>& wave, const std::vector<const BatchSequence*>& seqs,
               const std::vector<uint32_t>& first_pos, const KvLayout& layout) {
        if (seqs.size() != first_pos.size()) throw std::invalid_argument("one first position per request");
        rows = 0;
        for (const WaveChunk& c : wave) {
            if (c.req >= seqs.size() || c.len == 0) throw std::invalid_argument("bad wave chunk");
            rows += c.len;
        }
        layers = layout.num_layers();
        pos_ids.clear(); seq_lens.clear(); origins.clear(); local_pos.clear(); row_req.clear();
        for (const WaveChunk& c : wave) {
            const uint32_t origin = (uint32_t)pos_ids.size();
            for (size_t j = 0; j < c.len; j++) {
                const uint32_t pos = first_pos[c.req] + (uint32_t)(c.start + j);
                pos_ids.push_back(pos);
                seq_lens.push_back(pos + 1u);  // causal: the row sees the keys up to itself
                origins.push_back(origin);
                local_pos.push_back((uint32_t)j);
                row_req.push_back((uint32_t)c.req);
            }
        }
        k_ptrs.assign(layers * rows, 0);
        v_ptrs.assign(layers * rows, 0);
        carry_ptrs.assign(layers * rows, 0);
        for (size_t l = 0; l < layers; l++)
            for (size_t r = 0; r < rows; r++) {
                const BatchSequence* sq = seqs[row_req[r]];
                if (layout.is_conv(l)) {
                    carry_ptrs[l * rows + r] = sq->conv_state_ptr(l);
                } else {
                    k_ptrs[l * rows + r] = sq->k_cache_ptr(l);
                    v_ptrs[l * rows + r] = sq->v_cache_ptr(l);
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
        check(cudaEventCreateWithFlags(&uploaded_, cudaEventDisableTiming), "event");
    }
    ~StepTables() {
        cudaFree(d_k_); cudaFree(d_v_); cudaFree(d_conv_); cudaFree(d_pos_); cudaFree(d_len_);
        if (h_) cudaFreeHost(h_);
        if (uploaded_) cudaEventDestroy(uploaded_);
    }
    StepTables(const StepTables&) = delete;
    StepTables& operator=(const StepTables&) = delete;

    void upload(const StepTablesHost& t, cudaStream_t s) {
        if (t.batch > max_batch_ || t.layers != layers_) throw std::invalid_argument("tables exceed the allocated size");
        batch_ = t.batch;
        const size_t n = t.batch * t.layers;
        // the pinned image is reused: the previous upload must have executed before it is rewritten
        check(cudaEventSynchronize(uploaded_), "upload");
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
        check(cudaEventRecord(uploaded_, s), "upload");
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
    cudaEvent_t uploaded_ = nullptr;
};

// Device copy of a wave's tables (one pinned staging block, asynchronous uploads).
class WaveTables {
  public:
    WaveTables(size_t max_rows, size_t layers) : max_rows_(max_rows), layers_(layers) {
        const size_t n = max_rows * layers;
        check(cudaMalloc((void**)&d_k_, n * 8), "wave tables");
        check(cudaMalloc((void**)&d_v_, n * 8), "wave tables");
        check(cudaMalloc((void**)&d_carry_, n * 8), "wave tables");
        check(cudaMalloc((void**)&d_u32_, 4 * max_rows * 4), "wave tables");
        check(cudaMallocHost((void**)&h_, 3 * n * 8 + 4 * max_rows * 4), "pinned wave tables");
    }
    ~WaveTables() {
        cudaFree(d_k_); cudaFree(d_v_); cudaFree(d_carry_); cudaFree(d_u32_);
        if (h_) cudaFreeHost(h_);
    }
    WaveTables(const WaveTables&) = delete;
    WaveTables& operator=(const WaveTables&) = delete;

    // The staging block is reused: the previous upload must have completed on its stream.
    void upload(const WaveTablesHost& t, cudaStream_t s) {
        if (t.rows == 0 || t.rows > max_rows_ || t.layers != layers_) throw std::invalid_argument("wave exceeds the allocated size");
        rows_ = t.rows;
        const size_t n = t.rows * t.layers;
        uint64_t* hk = (uint64_t*)h_;
        uint64_t* hv = hk + max_rows_ * layers_;
        uint64_t* hc = hv + max_rows_ * layers_;
        uint32_t* hu = (uint32_t*)(hc + max_rows_ * layers_);
        std::copy(t.k_ptrs.begin(), t.k_ptrs.end(), hk);
        std::copy(t.v_ptrs.begin(), t.v_ptrs.end(), hv);
        std::copy(t.carry_ptrs.begin(), t.carry_ptrs.end(), hc);
        std::copy(t.pos_ids.begin(), t.pos_ids.end(), hu);
        std::copy(t.seq_lens.begin(), t.seq_lens.end(), hu + max_rows_);
        std::copy(t.origins.begin(), t.origins.end(), hu + 2 * max_rows_);
        std::copy(t.local_pos.begin(), t.local_pos.end(), hu + 3 * max_rows_);
        check(cudaMemcpyAsync(d_k_, hk, n * 8, cudaMemcpyHostToDevice, s), "upload");
        check(cudaMemcpyAsync(d_v_, hv, n * 8, cudaMemcpyHostToDevice, s), "upload");
        check(cudaMemcpyAsync(d_carry_, hc, n * 8, cudaMemcpyHostToDevice, s), "upload");
        check(cudaMemcpyAsync(d_u32_, hu, 4 * max_rows_ * 4, cudaMemcpyHostToDevice, s), "upload");
    }
    size_t rows() const { return rows_; }
    const uint64_t* k_ptrs(size_t layer) const { return d_k_ + layer * rows_; }
    const uint64_t* v_ptrs(size_t layer) const { return d_v_ + layer * rows_; }
    const uint64_t* carry_ptrs(size_t layer) const { return d_carry_ + layer * rows_; }
    const uint32_t* pos_ids() const { return d_u32_; }
    const uint32_t* seq_lens() const { return d_u32_ + max_rows_; }
    const uint32_t* origins() const { return d_u32_ + 2 * max_rows_; }
    const uint32_t* local_pos() const { return d_u32_ + 3 * max_rows_; }

  private:
    static void check(cudaError_t e, const char* what) {
        if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
    }
    size_t max_rows_, layers_, rows_ = 0;
    uint64_t *d_k_ = nullptr, *d_v_ = nullptr, *d_carry_ = nullptr;
    uint32_t* d_u32_ = nullptr;
    void* h_ = nullptr;
};

// Device copy of a paged decode step's tables.
class PagedStepTables {
  public:
    PagedStepTables(size_t max_batch, size_t max_blocks) : max_batch_(max_batch), max_blocks_(max_blocks) {
        check(cudaMalloc((void**)&d_, words() * 4), "paged tables");
        check(cudaMallocHost((void**)&h_, words() * 4), "pinned paged tables");
    }
    ~PagedStepTables() {
        cudaFree(d_);
        if (h_) cudaFreeHost(h_);
    }
    PagedStepTables(const PagedStepTables&) = delete;
    PagedStepTables& operator=(const PagedStepTables&) = delete;

    // The staging block is reused: the previous upload must have completed on its stream.
    void upload(const PagedStepTablesHost& t, cudaStream_t s) {
        if (t.batch == 0 || t.batch > max_batch_ || t.max_blocks != max_blocks_) throw std::invalid_argument("paged tables exceed the allocated size");
        batch_ = t.batch;
        std::copy(t.block_tables.begin(), t.block_tables.end(), h_);
        std::copy(t.pos_ids.begin(), t.pos_ids.end(), h_ + max_batch_ * max_blocks_);
        std::copy(t.seq_lens.begin(), t.seq_lens.end(), h_ + max_batch_ * max_blocks_ + max_batch_);
        check(cudaMemcpyAsync(d_, h_, words() * 4, cudaMemcpyHostToDevice, s), "upload");
    }
    size_t batch() const { return batch_; }
    const uint32_t* pos_ids() const { return d_ + max_batch_ * max_blocks_; }
    const uint32_t* seq_lens() const { return d_ + max_batch_ * max_blocks_ + max_batch_; }
    // The layout argument of the paged entry points for attention layer `layer` of `pool`.
    oxi_paged_layout layout(const PagedKvPool& pool, size_t layer) const {
        oxi_paged_layout l{};
        l.k_pool = (const void*)pool.k_rows(layer);
        l.v_pool = (const void*)pool.v_rows(layer);
        l.block_tables = d_;
        l.block_stride_bytes = pool.config().block_bytes();
        l.max_blocks = (uint32_t)max_blocks_;
        l.block_size = (uint32_t)pool.config().block_size;
        l.num_blocks = (uint32_t)pool.config().num_blocks;
        return l;
    }

  private:
    size_t words() const { return max_batch_ * max_blocks_ + 2 * max_batch_; }
    static void check(cudaError_t e, const char* what) {
        if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
    }
    size_t max_batch_, max_blocks_, batch_ = 0;
    uint32_t *d_ = nullptr, *h_ = nullptr;
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
    // The same step over the paged layout (the K/V row is written into its block, then attention
    // over the block table); `layer` counts attention layers, as the pool does.
    void attention_decode_paged(cudaStream_t s, const PagedStepTables& t, const PagedKvPool& pool, size_t layer, void* ctx,
                                void* q_io, const void* k, const void* v, const void* gate, const void* q_norm_w,
                                const void* k_norm_w, const void* cos_table, const void* sin_table, uint32_t window,
                                float eps = 1e-5f) {
        const oxi_paged_layout l = t.layout(pool, layer);
        ok(oxi_append_decode_paged(h_, s, ctx, q_io, k, v, gate, q_norm_w, k_norm_w, cos_table, sin_table, t.seq_lens(), &l,
                                   (uint32_t)t.batch(), window, eps),
           "oxi_append_decode_paged");
    }
    // batch_engine.rs:840-899 for conv layer `layer` (decode rows).
    void conv_decode(cudaStream_t s, const StepTables& t, size_t layer, void* y, const void* bcx, const void* conv_w) {
        ok(oxi_conv_decode(h_, s, y, t.conv_ptrs(layer), bcx, conv_w, (uint32_t)t.batch()), "oxi_conv_decode");
    }
    // A prefill wave through attention layer `layer` (batch_engine.rs:941-1014 on the wave's rows, then
    // :1045-1077): every row's K/V is appended at its position, then the rows attend causally.
    void attention_prefill(cudaStream_t s, const WaveTables& t, size_t layer, void* ctx, void* q_io, const void* k,
                           const void* v, const void* gate, const void* q_norm_w, const void* k_norm_w,
                           const void* cos_table, const void* sin_table, uint32_t window, float eps = 1e-5f) {
        ok(oxi_append(h_, s, q_io, k, v, q_norm_w, k_norm_w, cos_table, sin_table, t.pos_ids(), t.k_ptrs(layer),
                      t.v_ptrs(layer), (uint32_t)t.rows(), eps),
           "oxi_append");
        ok(oxi_prefill_attn(h_, s, ctx, q_io, gate, t.k_ptrs(layer), t.v_ptrs(layer), t.seq_lens(), (uint32_t)t.rows(),
                            window),
           "oxi_prefill_attn");
    }
    // A prefill wave through conv layer `layer` (batch_engine.rs:847-899 and the copy-back of
    // bin/server.rs:1192-1224): the requests' persistent states are updated by the call.
    void conv_prefill(cudaStream_t s, const WaveTables& t, size_t layer, void* y, const void* bcx, const void* conv_w) {
        ok(oxi_conv_prefill(h_, s, y, t.carry_ptrs(layer), t.origins(), t.local_pos(), bcx, conv_w, (uint32_t)t.rows()),
           "oxi_conv_prefill");
    }
    // Lets small waves of long prompts use idle SMs (see oxi_prefill_split_configure).
    void configure_prefill_split(uint32_t min_part_keys, uint32_t slots) {
        ok(oxi_prefill_split_configure(h_, min_part_keys, slots), "oxi_prefill_split_configure");
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
