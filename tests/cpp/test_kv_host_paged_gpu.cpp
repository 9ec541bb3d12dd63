// Forty decode steps of three sequences through the host layer, once over contiguous leases
// (KvPool -> StepTables -> attention_decode) and once over paged blocks (PagedKvPool ->
// PagedBlockManager -> PagedStepTables -> attention_decode_paged, 16-token blocks handed out
// interleaved between the sequences): the context bytes of every step must be identical, and
// the K/V rows must sit in the right slot of the right block.
#include "../../oxide_infer_b200/csrc/host/kv_host.hpp"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cuda_fp16.h>

using namespace oxi_host;

#define CHECK(c) do { if (!(c)) { std::printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #c); std::exit(1); } } while (0)
#define CU(x) CHECK((x) == cudaSuccess)

static uint32_t rng_state = 4242u;
static float rnd() {
    rng_state = rng_state * 1664525u + 1013904223u;
    return (float)(rng_state >> 8) / 8388608.0f - 1.0f;
}
static std::vector<__half> randh(size_t n, float scale = 1.0f) {
    std::vector<__half> v(n);
    for (auto& x : v) x = __float2half(rnd() * scale);
    return v;
}
template <class T> static T* to_dev(const std::vector<T>& v) {
    T* d;
    CU(cudaMalloc((void**)&d, v.size() * sizeof(T)));
    CU(cudaMemcpy(d, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice));
    return d;
}

int main() {
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) { std::printf("no device\n"); return 77; }
    const size_t B = 3, STEPS = 40, LAYERS = 2, LAYER = 1, BS = 16, MAXB = 4;
    cudaStream_t s;
    CU(cudaStreamCreate(&s));

    // contiguous side: attention layers 0 and 1 of the paged pool are layers 1 and 2 here
    const std::vector<bool> is_conv = {true, false, false};
    auto pool = KvPool::create(is_conv, 4, 4096);
    auto layout = pool->layout();
    std::vector<std::unique_ptr<LeasedSequence>> seqs;
    std::vector<const BatchSequence*> ptrs;
    for (size_t i = 0; i < B; i++) {
        auto l = pool->acquire(STEPS + 8, s);
        CHECK(l);
        seqs.emplace_back(new LeasedSequence(layout, *l));
        ptrs.push_back(seqs.back().get());
    }
    // paged side
    PagedPoolConfig cfg;
    cfg.num_blocks = 12; cfg.block_size = BS; cfg.num_layers = LAYERS;
    auto ppool = PagedKvPool::create(cfg);
    PagedBlockManager mgr(ppool);
    const std::vector<uint64_t> ids = {11, 22, 33};
    for (uint64_t id : ids) mgr.allocate_for_seq(id, 1);  // blocks 0, 1, 2

    std::vector<__half> hw(128), hcos(64 * 128), hsin(64 * 128);
    for (auto& x : hw) x = __float2half(1.0f + 0.05f * rnd());
    for (size_t p = 0; p < 64; p++)
        for (size_t d = 0; d < 128; d++) {
            const size_t i = d % 64;
            const float inv = i < 32 ? 1.0f / std::pow(1e6f, (float)(2 * i) / 128.0f) : 0.0f;
            hcos[p * 128 + d] = __float2half(std::cos((float)p * inv));
            hsin[p * 128 + d] = __float2half(std::sin((float)p * inv));
        }
    __half *dw = to_dev(hw), *dcos = to_dev(hcos), *dsin = to_dev(hsin);
    __half *dq, *dq2, *dk, *dv, *dg, *dctx, *dctx2;
    CU(cudaMalloc((void**)&dq, B * 2048 * 2));
    CU(cudaMalloc((void**)&dq2, B * 2048 * 2));
    CU(cudaMalloc((void**)&dk, B * 512 * 2));
    CU(cudaMalloc((void**)&dv, B * 512 * 2));
    CU(cudaMalloc((void**)&dg, B * 16 * 2));
    CU(cudaMalloc((void**)&dctx, B * 2048 * 2));
    CU(cudaMalloc((void**)&dctx2, B * 2048 * 2));

    KvPathEngine engine(0, 4, 4096, 0);
    StepTables st(4, layout->num_layers());
    PagedStepTables pst(4, MAXB);
    std::vector<std::vector<__half>> vrows(B);
    for (size_t t = 0; t < STEPS; t++) {
        auto hq = randh(B * 2048), hk = randh(B * 512), hv = randh(B * 512), hg = randh(B * 16);
        for (size_t i = 0; i < B; i++) vrows[i].insert(vrows[i].end(), hv.begin() + i * 512, hv.begin() + (i + 1) * 512);
        CU(cudaMemcpy(dq, hq.data(), hq.size() * 2, cudaMemcpyHostToDevice));
        CU(cudaMemcpy(dq2, hq.data(), hq.size() * 2, cudaMemcpyHostToDevice));
        CU(cudaMemcpy(dk, hk.data(), hk.size() * 2, cudaMemcpyHostToDevice));
        CU(cudaMemcpy(dv, hv.data(), hv.size() * 2, cudaMemcpyHostToDevice));
        CU(cudaMemcpy(dg, hg.data(), hg.size() * 2, cudaMemcpyHostToDevice));
        const std::vector<uint32_t> pos(B, (uint32_t)t);
        StepTablesHost th;
        th.build(ptrs, pos, *layout);
        st.upload(th, s);
        engine.attention_decode(s, st, LAYER + 1, dctx, dq, dk, dv, dg, dw, dw, dcos, dsin, 0);
        if (t > 0)
            for (uint64_t id : ids) {
                const auto nb = mgr.append_token(id, t);
                CHECK(nb.has_value() == (t % BS == 0));
            }
        PagedStepTablesHost ph;
        ph.build(mgr, ids, pos, MAXB);
        pst.upload(ph, s);
        engine.attention_decode_paged(s, pst, *ppool, LAYER, dctx2, dq2, dk, dv, dg, dw, dw, dcos, dsin, 0);
        CU(cudaStreamSynchronize(s));
        std::vector<__half> c1(B * 2048), c2(B * 2048);
        CU(cudaMemcpy(c1.data(), dctx, c1.size() * 2, cudaMemcpyDeviceToHost));
        CU(cudaMemcpy(c2.data(), dctx2, c2.size() * 2, cudaMemcpyDeviceToHost));
        CHECK(std::memcmp(c1.data(), c2.data(), c1.size() * 2) == 0);
    }
    CHECK(engine.device_status(s) == 0);
    // blocks were handed out round robin: 0 1 2, then 3 4 5 at step 16, 6 7 8 at step 32
    for (size_t i = 0; i < B; i++) {
        const auto* tbl = mgr.get_block_table(ids[i]);
        CHECK(tbl && tbl->size() == 3 && (*tbl)[0] == i && (*tbl)[1] == 3 + i && (*tbl)[2] == 6 + i);
        // V rows are copied verbatim: token t of sequence i sits in block tbl[t / 16], slot t % 16 of layer LAYER's V rows
        for (size_t t = 0; t < STEPS; t += 7) {
            std::vector<__half> row(512);
            const uint64_t src = ppool->v_rows(LAYER) + (*tbl)[t / BS] * cfg.block_bytes() + (t % BS) * 1024;
            CU(cudaMemcpy(row.data(), (void*)src, 1024, cudaMemcpyDeviceToHost));
            CHECK(std::memcmp(row.data(), &vrows[i][t * 512], 1024) == 0);
        }
    }
    CHECK(ppool->free_block_count() == 3);
    for (uint64_t id : ids) mgr.free_seq(id);
    CHECK(ppool->free_block_count() == 12);
    std::printf("kv_host paged checks passed (%zu steps, contexts identical)\n", STEPS);
    return 0;
}
