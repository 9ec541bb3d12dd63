// Host-only checks of the C++ host layer: layout addressing (kv_pool.rs:46-61), first-fit
// leases with coalescing release (kv_pool.rs:175-251), layer-major table building
// (batch_engine.rs:709-731).  No CUDA: slabs are plain numbers.
#define OXI_HOST_NO_CUDA
#include "../../oxide_infer_b200/csrc/host/kv_host.hpp"

#include <cstdio>
#include <cstdlib>

using namespace oxi_host;

#define CHECK(c) do { if (!(c)) { std::printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #c); std::exit(1); } } while (0)

int main() {
    // LFM-style mix: conv, conv, attention, conv, attention
    const std::vector<bool> is_conv = {true, true, false, true, false};
    const uint64_t KV = 0x10000000ull, CONV = 0x90000000ull;
    const size_t cap = 1000;
    auto layout = std::make_shared<KvLayout>(KV, CONV, is_conv, cap);
    CHECK(layout->num_attention_layers() == 2 && layout->num_conv_layers() == 3);
    // K of attention plane p is plane 2p of the slab, V plane 2p+1; rows are 1024 bytes
    CHECK(layout->k_cache_ptr(2, 0) == KV);
    CHECK(layout->v_cache_ptr(2, 0) == KV + cap * 1024);
    CHECK(layout->k_cache_ptr(4, 7) == KV + (2 * cap + 7) * 1024);
    CHECK(layout->v_cache_ptr(4, 7) == KV + (3 * cap + 7) * 1024);
    CHECK(layout->conv_state_ptr(3, 5) == CONV + (5 * 3 + 2) * 2048 * 6 * 2);
    bool threw = false;
    try { layout->k_cache_ptr(0, 0); } catch (const std::invalid_argument&) { threw = true; }
    CHECK(threw);

    KvPool pool(layout, 3);
    CHECK(pool.free_tokens() == cap && pool.free_slots() == 3);
    auto a = pool.acquire(300), b = pool.acquire(300), c = pool.acquire(300);
    CHECK(a && b && c);
    CHECK(a->tok_off == 0 && b->tok_off == 300 && c->tok_off == 600);
    CHECK(a->slot != b->slot && b->slot != c->slot && a->slot != c->slot);
    CHECK(!pool.acquire(50));            // no slot left
    pool.release(*b);
    CHECK(!pool.acquire(301));           // slot free, but no range of 301 (300-hole and 100-tail)
    CHECK(pool.free_slots() == 1);       // a failed acquire gives the slot back
    auto d = pool.acquire(100);          // first fit: the hole at 300
    CHECK(d && d->tok_off == 300);
    pool.release(*a);
    pool.release(*d);
    CHECK(pool.fragments() == 2);        // [0,600) after coalescing 0-300 + 300-400 + 400-600, and [900,1000)
    pool.release(*c);
    CHECK(pool.fragments() == 1 && pool.free_tokens() == cap && pool.free_slots() == 3);
    CHECK(!pool.acquire(0) && !pool.acquire(cap + 1));

    // tables: tbl[layer * b + i]; seq_len counts the appended token
    auto l0 = pool.acquire(128), l1 = pool.acquire(64);
    LeasedSequence s0(layout, *l0), s1(layout, *l1);
    StepTablesHost t;
    t.build({&s0, &s1}, {10, 63}, *layout);
    CHECK(t.batch == 2 && t.layers == 5);
    CHECK(t.seq_lens[0] == 11 && t.seq_lens[1] == 64);
    CHECK(t.k_ptrs[2 * 2 + 1] == layout->k_cache_ptr(2, l1->tok_off));
    CHECK(t.v_ptrs[4 * 2 + 0] == layout->v_cache_ptr(4, l0->tok_off));
    CHECK(t.conv_ptrs[1 * 2 + 1] == layout->conv_state_ptr(1, l1->slot));
    CHECK(t.k_ptrs[0] == 0 && t.conv_ptrs[2 * 2] == 0);  // a layer has entries of its own kind only
    std::printf("kv_host cpu checks passed\n");
    return 0;
}
