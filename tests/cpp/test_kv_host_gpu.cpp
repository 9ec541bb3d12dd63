// One decode step through the C++ host layer (KvPool -> LeasedSequence -> StepTables ->
// KvPathEngine) compared with the same step issued directly through the C ABI on tables
// written by hand: the context bytes and the appended K/V rows must be identical.
#include "../../oxide_infer_b200/csrc/host/kv_host.hpp"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cuda_fp16.h>

using namespace oxi_host;

#define CHECK(c) do { if (!(c)) { std::printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #c); std::exit(1); } } while (0)
#define CU(x) CHECK((x) == cudaSuccess)

static uint32_t rng_state = 12345u;
static float rnd() {  // uniform in [-1, 1)
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
    const std::vector<bool> is_conv = {true, false, true, false};  // attention layers 1 and 3
    const size_t B = 5, cap = 4096;
    const uint32_t lens[B] = {17, 300, 1, 777, 256};  // old lengths; the new token lands at this position
    auto pool = KvPool::create(is_conv, 8, cap);
    auto layout = pool->layout();
    cudaStream_t s;
    CU(cudaStreamCreate(&s));

    std::vector<Lease> leases;
    std::vector<std::unique_ptr<LeasedSequence>> seqs;
    std::vector<const BatchSequence*> ptrs;
    std::vector<uint32_t> pos;
    for (size_t i = 0; i < B; i++) {
        auto l = pool->acquire(lens[i] + 65, s);
        CHECK(l);
        leases.push_back(*l);
        seqs.emplace_back(new LeasedSequence(layout, *l));
        ptrs.push_back(seqs.back().get());
        pos.push_back(lens[i]);
    }
    // fill the old tokens of both attention layers with random K/V
    for (size_t layer : {size_t(1), size_t(3)})
        for (size_t i = 0; i < B; i++) {
            auto k = randh(lens[i] * KV_DIM), v = randh(lens[i] * KV_DIM);
            if (lens[i]) {
                CU(cudaMemcpy((void*)seqs[i]->k_cache_ptr(layer), k.data(), k.size() * 2, cudaMemcpyHostToDevice));
                CU(cudaMemcpy((void*)seqs[i]->v_cache_ptr(layer), v.data(), v.size() * 2, cudaMemcpyHostToDevice));
            }
        }
    // step inputs for layer 3
    auto hq = randh(B * 2048), hk = randh(B * 512), hv = randh(B * 512), hg = randh(B * 16);
    std::vector<__half> hw(128, __float2half(1.0f)), hcos(2048 * 128), hsin(2048 * 128);
    for (size_t p = 0; p < 2048; p++)
        for (size_t d = 0; d < 128; d++) {
            const size_t i = d % 64;
            const float inv = i < 32 ? 1.0f / std::pow(1e6f, (float)(2 * i) / 128.0f) : 0.0f;
            hcos[p * 128 + d] = __float2half(std::cos((float)p * inv));
            hsin[p * 128 + d] = __float2half(std::sin((float)p * inv));
        }
    __half *dq = to_dev(hq), *dq2 = to_dev(hq), *dk = to_dev(hk), *dv = to_dev(hv), *dg = to_dev(hg);
    __half *dw = to_dev(hw), *dcos = to_dev(hcos), *dsin = to_dev(hsin), *dctx, *dctx2;
    CU(cudaMalloc((void**)&dctx, B * 2048 * 2));
    CU(cudaMalloc((void**)&dctx2, B * 2048 * 2));

    // ---- through the host layer
    StepTablesHost th;
    th.build(ptrs, pos, *layout);
    StepTables tables(8, layout->num_layers());
    tables.upload(th, s);
    KvPathEngine engine(0, 8, 4096, 0);
    engine.attention_decode(s, tables, 3, dctx, dq, dk, dv, dg, dw, dw, dcos, dsin, 0);
    CU(cudaStreamSynchronize(s));
    CHECK(engine.device_status(s) == 0);
    std::vector<__half> ctx1(B * 2048), krow1(B * 512), vrow1(B * 512);
    CU(cudaMemcpy(ctx1.data(), dctx, ctx1.size() * 2, cudaMemcpyDeviceToHost));
    for (size_t i = 0; i < B; i++) {
        CU(cudaMemcpy(&krow1[i * 512], (void*)(seqs[i]->k_cache_ptr(3) + (size_t)lens[i] * 1024), 1024, cudaMemcpyDeviceToHost));
        CU(cudaMemcpy(&vrow1[i * 512], (void*)(seqs[i]->v_cache_ptr(3) + (size_t)lens[i] * 1024), 1024, cudaMemcpyDeviceToHost));
    }
    CHECK(std::memcmp(vrow1.data(), hv.data(), B * 1024) == 0);  // V is copied verbatim

    // ---- the same step straight through the C ABI with hand-written tables
    std::vector<uint64_t> kp(B), vp(B);
    std::vector<uint32_t> sl(B);
    for (size_t i = 0; i < B; i++) {
        kp[i] = layout->k_cache_ptr(3, leases[i].tok_off);
        vp[i] = layout->v_cache_ptr(3, leases[i].tok_off);
        sl[i] = lens[i] + 1;
    }
    uint64_t *dkp = to_dev(kp), *dvp = to_dev(vp);
    uint32_t *dpos = to_dev(pos), *dsl = to_dev(sl);
    CHECK(oxi_append(engine.handle(), s, dq2, dk, dv, dw, dw, dcos, dsin, dpos, dkp, dvp, B, 1e-5f) == 0);
    CHECK(oxi_decode_attn(engine.handle(), s, dctx2, dq2, dg, dkp, dvp, dsl, B, 0) == 0);
    CU(cudaStreamSynchronize(s));
    std::vector<__half> ctx2(B * 2048), krow2(B * 512);
    CU(cudaMemcpy(ctx2.data(), dctx2, ctx2.size() * 2, cudaMemcpyDeviceToHost));
    for (size_t i = 0; i < B; i++)
        CU(cudaMemcpy(&krow2[i * 512], (void*)(kp[i] + (size_t)lens[i] * 1024), 1024, cudaMemcpyDeviceToHost));
    CHECK(std::memcmp(ctx1.data(), ctx2.data(), ctx1.size() * 2) == 0);
    CHECK(std::memcmp(krow1.data(), krow2.data(), krow1.size() * 2) == 0);
    double sum = 0;
    for (auto x : ctx1) { CHECK(std::isfinite(__half2float(x))); sum += std::fabs(__half2float(x)); }
    CHECK(sum > 1.0);

    // conv layer 0 through the host layer: state of a fresh lease is zero, so y = C * (B*x * w6)
    auto hbcx = randh(B * 6144), hcw = randh(2048 * 7, 0.1f);
    __half *dbcx = to_dev(hbcx), *dcw = to_dev(hcw), *dy;
    CU(cudaMalloc((void**)&dy, B * 2048 * 2));
    engine.conv_decode(s, tables, 0, dy, dbcx, dcw);
    CU(cudaStreamSynchronize(s));
    std::vector<__half> y(B * 2048);
    CU(cudaMemcpy(y.data(), dy, y.size() * 2, cudaMemcpyDeviceToHost));
    for (size_t i = 0; i < B; i++)
        for (size_t c = 0; c < 2048; c += 97) {
            const float fin = __half2float(hbcx[i * 6144 + c]) * __half2float(hbcx[i * 6144 + 4096 + c]);
            const float acc = std::fma(fin, __half2float(hcw[c * 7 + 6]), 0.0f);
            const __half want = __float2half(acc * __half2float(hbcx[i * 6144 + 2048 + c]));
            CHECK(std::memcmp(&want, &y[i * 2048 + c], 2) == 0);
        }
    for (auto& l : leases) pool->release(l);
    CHECK(pool->free_tokens() == pool->layout()->capacity_tokens());
    std::printf("kv_host gpu checks passed (|ctx| sum %.3f)\n", sum);
    return 0;
}
