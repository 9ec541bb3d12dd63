// Host-only checks of the C++ host layer: layout addressing (kv_pool.rs:46-61), first-fit
// leases with coalescing release (kv_pool.rs:175-251), layer-major table building
// (batch_engine.rs:709-731), prefill wave planning and per-row wave tables
// (bin/server.rs:1076-1141).  No CUDA: slabs are plain numbers.
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
    // prefill waves: requests by increasing prompt length, chunks of at most 128 rows, whole chunks
    // packed while they fit (bin/server.rs:1076-1112)
    {
        PrefillPlanner pl({300, 5, 130, 0, 128}, 128);
        const std::vector<std::vector<WaveChunk>> want = {
            {{1, 0, 5}},                  // the 128-row chunk of request 4 does not fit beside it
            {{4, 0, 128}},
            {{2, 0, 128}},
            {{2, 128, 2}},                // 2 + 128 > 128
            {{0, 0, 128}}, {{0, 128, 128}}, {{0, 256, 44}}};
        for (const auto& w : want) CHECK(pl.next() == w);
        CHECK(pl.next().empty() && pl.chunks_left() == 0);
        PrefillPlanner small({3, 4, 200, 6}, 16);  // short prompts share a wave; equal keys keep their order
        CHECK((small.next() == std::vector<WaveChunk>{{0, 0, 3}, {1, 0, 4}, {3, 0, 6}}));
        CHECK((small.next() == std::vector<WaveChunk>{{2, 0, 16}}));
        bool bad = false;
        try { PrefillPlanner none({1}, 0); } catch (const std::invalid_argument&) { bad = true; }
        CHECK(bad);
    }
    {
        // per-row tables of a wave: positions, chunk origins, positions inside the chunk, pointers
        WaveTablesHost w;
        const std::vector<WaveChunk> wave = {{1, 0, 3}, {0, 64, 2}};
        w.build(wave, {&s0, &s1}, {100, 0}, *layout);
        CHECK(w.rows == 5 && w.layers == 5);
        const uint32_t pos[5] = {0, 1, 2, 164, 165}, org[5] = {0, 0, 0, 3, 3}, lp[5] = {0, 1, 2, 0, 1};
        for (int r = 0; r < 5; r++) {
            CHECK(w.pos_ids[r] == pos[r] && w.seq_lens[r] == pos[r] + 1 && w.origins[r] == org[r] && w.local_pos[r] == lp[r]);
            CHECK(w.row_req[r] == (r < 3 ? 1u : 0u));
        }
        CHECK(w.k_ptrs[2 * 5 + 0] == s1.k_cache_ptr(2) && w.k_ptrs[2 * 5 + 4] == s0.k_cache_ptr(2));
        CHECK(w.v_ptrs[4 * 5 + 3] == s0.v_cache_ptr(4));
        CHECK(w.carry_ptrs[3 * 5 + 1] == s1.conv_state_ptr(3) && w.carry_ptrs[0 * 5 + 4] == s0.conv_state_ptr(0));
        CHECK(w.k_ptrs[0] == 0 && w.carry_ptrs[2 * 5] == 0);
        bool bad = false;
        try { w.build({{2, 0, 1}}, {&s0, &s1}, {0, 0}, *layout); } catch (const std::invalid_argument&) { bad = true; }
        CHECK(bad);
    }
    std::printf("kv_host cpu checks passed\n");
    return 0;
}
