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
        // random allocate / grow / free with shared prefix blocks: no block is lost or handed out twice
        PagedPoolConfig cfg;
        cfg.num_blocks = 64; cfg.block_size = 16; cfg.num_layers = 2;
        auto pp = std::make_shared<PagedKvPool>(0, cfg);
        PagedBlockManager mgr(pp);
        uint32_t st = 7u;
        auto rnd = [&](uint32_t n) { st = st * 1664525u + 1013904223u; return (st >> 8) % n; };
        std::map<uint64_t, size_t> live;  // sequence -> tokens
        uint64_t next_id = 1;
        for (int step = 0; step < 3000; step++) {
            const uint32_t op = rnd(4);
            if (op == 0 || live.empty()) {
                const size_t tokens = 1 + rnd(100);
                std::vector<size_t> shared;
                if (!live.empty() && rnd(2)) {  // adopt a prefix of full blocks of a live sequence
                    auto it = live.begin();
                    std::advance(it, rnd((uint32_t)live.size()));
                    const auto* t = mgr.get_block_table(it->first);
                    const size_t full = std::min(it->second, tokens) / 16;
                    for (size_t i = 0; i < full && i < t->size(); i++) shared.push_back((*t)[i]);
                }
                try {
                    mgr.allocate_for_seq(next_id, tokens, shared);
                    live[next_id++] = tokens;
                } catch (const std::runtime_error&) {
                }
            } else if (op == 1) {
                auto it = live.begin();
                std::advance(it, rnd((uint32_t)live.size()));
                try {
                    mgr.append_token(it->first, it->second);
                    it->second += 1;
                } catch (const std::runtime_error&) {
                }
            } else if (op == 2) {
                auto it = live.begin();
                std::advance(it, rnd((uint32_t)live.size()));
                mgr.free_seq(it->first);
                live.erase(it);
            }
            // invariants: tables cover the tokens; distinct blocks in use + free blocks = all blocks
            std::map<size_t, int> used;
            for (auto& kv : live) {
                const auto* t = mgr.get_block_table(kv.first);
                CHECK(t && t->size() >= (kv.second + 15) / 16);
                for (size_t b : *t) {
                    CHECK(b < cfg.num_blocks);
                    used[b]++;
                }
            }
            CHECK(used.size() + pp->free_block_count() == cfg.num_blocks);
        }
        for (auto& kv : live) mgr.free_seq(kv.first);
        CHECK(pp->free_block_count() == cfg.num_blocks);
    }
    {
        // properties on random prompt sets: every token is handed out exactly once and in order, a wave
        // holds at most max_rows rows, chunks of one request never share a wave, short requests go first
        uint32_t st = 99u;
        auto rnd = [&](uint32_t n) { st = st * 1664525u + 1013904223u; return (st >> 8) % n; };
        for (int trial = 0; trial < 200; trial++) {
            const size_t nreq = 1 + rnd(12), max_rows = 1 + rnd(200);
            std::vector<size_t> lens(nreq);
            for (auto& l : lens) l = rnd(4) == 0 ? 0 : rnd(700);
            PrefillPlanner pl(lens, max_rows);
            std::vector<size_t> next_tok(nreq, 0);
            size_t last_len = 0;
            for (auto wave = pl.next(); !wave.empty(); wave = pl.next()) {
                size_t used = 0;
                for (size_t i = 0; i < wave.size(); i++) {
                    const WaveChunk& c = wave[i];
                    CHECK(c.req < nreq && c.len >= 1 && c.len <= max_rows);
                    CHECK(c.start == next_tok[c.req]);  // a request's chunks come in order, without gaps
                    next_tok[c.req] += c.len;
                    CHECK(next_tok[c.req] <= lens[c.req]);
                    CHECK(lens[c.req] >= last_len);     // requests by increasing prompt length
                    last_len = lens[c.req];
                    for (size_t k = 0; k < i; k++) CHECK(wave[k].req != c.req);
                    used += c.len;
                }
                CHECK(used <= max_rows);
            }
            for (size_t r = 0; r < nreq; r++) CHECK(next_tok[r] == lens[r]);
        }
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
    {
        // paged blocks: the scenario of the reference's own unit test (block_manager.rs:139-178): 10 blocks
        // of 16 tokens; 32 tokens take 2 blocks; a second sequence adopts the first block as a shared
        // prefix and takes one new block; a shared block returns to the pool with its last owner
        PagedPoolConfig cfg;
        cfg.num_blocks = 10; cfg.block_size = 16; cfg.num_layers = 1;
        auto pp = std::make_shared<PagedKvPool>(0x40000000ull, cfg);
        PagedBlockManager mgr(pp);
        mgr.allocate_for_seq(1001, 32);
        const auto* b1 = mgr.get_block_table(1001);
        CHECK(b1 && b1->size() == 2 && pp->free_block_count() == 8);
        mgr.allocate_for_seq(1002, 32, {(*b1)[0]});
        const auto* b2 = mgr.get_block_table(1002);
        CHECK(b2 && b2->size() == 2 && (*b2)[0] == (*b1)[0] && pp->free_block_count() == 7);
        mgr.free_seq(1001);
        CHECK(pp->free_block_count() == 8 && !mgr.get_block_table(1001));
        mgr.free_seq(1002);
        CHECK(pp->free_block_count() == 10);
        // growth: a block is taken only when the position opens one
        mgr.allocate_for_seq(7, 16);
        CHECK(mgr.get_block_table(7)->size() == 1);
        CHECK(!mgr.append_token(7, 15));
        CHECK(mgr.append_token(7, 16).has_value() && mgr.get_block_table(7)->size() == 2);
        CHECK(!mgr.append_token(7, 17));
        // exhaustion gives everything back, also the extra reference on an adopted block
        const size_t shared = (*mgr.get_block_table(7))[0], before = pp->free_block_count();
        bool oom = false;
        try { mgr.allocate_for_seq(8, 16 * 11, {shared}); } catch (const std::runtime_error&) { oom = true; }
        CHECK(oom && pp->free_block_count() == before && !mgr.get_block_table(8));
        mgr.free_seq(7);
        CHECK(pp->free_block_count() == 10);
        bool unknown = false;
        try { mgr.append_token(99, 16); } catch (const std::invalid_argument&) { unknown = true; }
        CHECK(unknown && pp->free_block_count() == 10);
        // addressing: [layer][K | V][block_size][512] inside a block
        PagedPoolConfig c3;
        c3.num_blocks = 4; c3.block_size = 32; c3.num_layers = 3;
        PagedKvPool p3(0x1000, c3);
        CHECK(c3.block_bytes() == 2 * 3 * 32 * 1024);
        CHECK(p3.k_rows(0) == 0x1000 && p3.v_rows(0) == 0x1000 + 32 * 1024 && p3.k_rows(2) == 0x1000 + 4 * 32 * 1024);
        bool badbs = false;
        try { PagedPoolConfig c4 = c3; c4.block_size = 24; PagedKvPool p4(0, c4); } catch (const std::invalid_argument&) { badbs = true; }
        CHECK(badbs);
        // the step's block tables
        mgr.allocate_for_seq(1, 40);   // 3 blocks
        mgr.allocate_for_seq(2, 5);    // 1 block
        PagedStepTablesHost pt;
        pt.build(mgr, {2, 1}, {4, 39}, 4);
        CHECK(pt.batch == 2 && pt.seq_lens[0] == 5 && pt.seq_lens[1] == 40);
        CHECK(pt.block_tables[0] == (*mgr.get_block_table(2))[0] && pt.block_tables[1] == 0);
        for (int j = 0; j < 3; j++) CHECK(pt.block_tables[4 + j] == (*mgr.get_block_table(1))[j]);
        bool uncovered = false;
        try { pt.build(mgr, {2}, {16}, 4); } catch (const std::invalid_argument&) { uncovered = true; }  // position 16 needs a 2nd block
        CHECK(uncovered);
    }
    std::printf("kv_host cpu checks passed\n");
    return 0;
}
