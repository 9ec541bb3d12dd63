// Prompts of three requests prefilled in waves through the C++ host layer (PrefillPlanner ->
// WaveTablesHost -> WaveTables -> KvPathEngine::attention_prefill / conv_prefill) against the
// same tokens fed one at a time through the decode path of the same engine:
//   K/V cache rows, conv outputs and the final conv states must be byte-identical,
//   attention outputs within the attention tolerance (2e-3).
#include "../../oxide_infer_b200/csrc/host/kv_host.hpp"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cuda_fp16.h>

using namespace oxi_host;

#define CHECK(c) do { if (!(c)) { std::printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #c); std::exit(1); } } while (0)
#define CU(x) CHECK((x) == cudaSuccess)

static uint32_t rng_state = 777u;
static float rnd() {
    rng_state = rng_state * 1664525u + 1013904223u;
    return (float)(rng_state >> 8) / 8388608.0f - 1.0f;
}
static std::vector<__half> randh(size_t n, float scale = 1.0f) {
    std::vector<__half> v(n);
    for (auto& x : v) x = __float2half(rnd() * scale);
    return v;
}
template <class T> static T* dev_alloc(size_t n) {
    T* d;
    CU(cudaMalloc((void**)&d, n * sizeof(T)));
    CU(cudaMemset(d, 0, n * sizeof(T)));
    return d;
}
template <class T> static T* to_dev(const std::vector<T>& v) {
    T* d = dev_alloc<T>(v.size());
    CU(cudaMemcpy(d, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice));
    return d;
}
template <class T> static std::vector<T> to_host(const void* d, size_t n) {
    std::vector<T> v(n);
    CU(cudaMemcpy(v.data(), d, n * sizeof(T), cudaMemcpyDeviceToHost));
    return v;
}

int main() {
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) { std::printf("no device\n"); return 77; }
    const std::vector<bool> is_conv = {true, false};  // layer 0 conv, layer 1 attention
    const std::vector<size_t> prompt = {5, 150, 40};
    const size_t R = prompt.size(), MAX_ROWS = 64, CAP = 2048;
    const uint32_t WINDOW = 0;
    auto pool = KvPool::create(is_conv, 8, CAP);
    auto layout = pool->layout();
    cudaStream_t s;
    CU(cudaStreamCreate(&s));

    // two leases per request: one filled by waves, one token by token
    std::vector<std::unique_ptr<LeasedSequence>> wave_seq, step_seq;
    std::vector<const BatchSequence*> wave_ptrs;
    for (size_t r = 0; r < R; r++) {
        auto a = pool->acquire(prompt[r] + 8, s), b = pool->acquire(prompt[r] + 8, s);
        CHECK(a && b);
        wave_seq.emplace_back(new LeasedSequence(layout, *a));
        step_seq.emplace_back(new LeasedSequence(layout, *b));
        wave_ptrs.push_back(wave_seq.back().get());
    }
    // per-request inputs of the two layers, one row per prompt token
    std::vector<std::vector<__half>> q(R), k(R), v(R), g(R), bcx(R);
    for (size_t r = 0; r < R; r++) {
        q[r] = randh(prompt[r] * 2048);
        k[r] = randh(prompt[r] * 512);
        v[r] = randh(prompt[r] * 512);
        g[r] = randh(prompt[r] * 16);
        bcx[r] = randh(prompt[r] * 6144);
    }
    std::vector<__half> hw(128), hcos(256 * 128), hsin(256 * 128);
    for (auto& x : hw) x = __float2half(1.0f + 0.05f * rnd());
    for (size_t p = 0; p < 256; p++)
        for (size_t d = 0; d < 128; d++) {
            const size_t i = d % 64;
            const float inv = i < 32 ? 1.0f / std::pow(1e6f, (float)(2 * i) / 128.0f) : 0.0f;
            hcos[p * 128 + d] = __float2half(std::cos((float)p * inv));
            hsin[p * 128 + d] = __float2half(std::sin((float)p * inv));
        }
    auto hcw = randh(2048 * 7, 0.1f);
    __half *dw = to_dev(hw), *dcos = to_dev(hcos), *dsin = to_dev(hsin), *dcw = to_dev(hcw);

    KvPathEngine engine(0, 8, CAP, (uint32_t)MAX_ROWS);

    // ---- waves
    PrefillPlanner planner(prompt, MAX_ROWS);
    const std::vector<std::vector<WaveChunk>> want_waves = {
        {{0, 0, 5}, {2, 0, 40}}, {{1, 0, 64}}, {{1, 64, 64}}, {{1, 128, 22}}};
    WaveTables wt(MAX_ROWS, layout->num_layers());
    __half *dq = dev_alloc<__half>(MAX_ROWS * 2048), *dk = dev_alloc<__half>(MAX_ROWS * 512);
    __half *dv = dev_alloc<__half>(MAX_ROWS * 512), *dg = dev_alloc<__half>(MAX_ROWS * 16);
    __half *dbcx = dev_alloc<__half>(MAX_ROWS * 6144), *dctx = dev_alloc<__half>(MAX_ROWS * 2048);
    __half* dy = dev_alloc<__half>(MAX_ROWS * 2048);
    std::vector<std::vector<__half>> ctx_wave(R), y_wave(R);
    for (size_t r = 0; r < R; r++) {
        ctx_wave[r].resize(prompt[r] * 2048);
        y_wave[r].resize(prompt[r] * 2048);
    }
    const std::vector<uint32_t> first_pos(R, 0u);
    size_t nwaves = 0;
    for (auto wave = planner.next(); !wave.empty(); wave = planner.next(), nwaves++) {
        CHECK(nwaves < want_waves.size() && wave == want_waves[nwaves]);
        WaveTablesHost th;
        th.build(wave, wave_ptrs, first_pos, *layout);
        // gather the wave's input rows
        size_t row = 0;
        for (const WaveChunk& c : wave) {
            CU(cudaMemcpy(dq + row * 2048, &q[c.req][c.start * 2048], c.len * 2048 * 2, cudaMemcpyHostToDevice));
            CU(cudaMemcpy(dk + row * 512, &k[c.req][c.start * 512], c.len * 512 * 2, cudaMemcpyHostToDevice));
            CU(cudaMemcpy(dv + row * 512, &v[c.req][c.start * 512], c.len * 512 * 2, cudaMemcpyHostToDevice));
            CU(cudaMemcpy(dg + row * 16, &g[c.req][c.start * 16], c.len * 16 * 2, cudaMemcpyHostToDevice));
            CU(cudaMemcpy(dbcx + row * 6144, &bcx[c.req][c.start * 6144], c.len * 6144 * 2, cudaMemcpyHostToDevice));
            row += c.len;
        }
        CHECK(row == th.rows);
        wt.upload(th, s);
        engine.conv_prefill(s, wt, 0, dy, dbcx, dcw);
        engine.attention_prefill(s, wt, 1, dctx, dq, dk, dv, dg, dw, dw, dcos, dsin, WINDOW);
        CU(cudaStreamSynchronize(s));
        row = 0;
        for (const WaveChunk& c : wave) {
            CU(cudaMemcpy(&ctx_wave[c.req][c.start * 2048], dctx + row * 2048, c.len * 2048 * 2, cudaMemcpyDeviceToHost));
            CU(cudaMemcpy(&y_wave[c.req][c.start * 2048], dy + row * 2048, c.len * 2048 * 2, cudaMemcpyDeviceToHost));
            row += c.len;
        }
    }
    CHECK(nwaves == want_waves.size() && planner.chunks_left() == 0);
    CHECK(engine.device_status(s) == 0);

    // ---- the same tokens one at a time through the decode path
    StepTables st(8, layout->num_layers());
    double worst = 0.0;
    for (size_t r = 0; r < R; r++) {
        for (size_t t = 0; t < prompt[r]; t++) {
            StepTablesHost th;
            th.build({step_seq[r].get()}, {(uint32_t)t}, *layout);
            st.upload(th, s);
            CU(cudaMemcpyAsync(dq, &q[r][t * 2048], 2048 * 2, cudaMemcpyHostToDevice, s));
            CU(cudaMemcpyAsync(dk, &k[r][t * 512], 512 * 2, cudaMemcpyHostToDevice, s));
            CU(cudaMemcpyAsync(dv, &v[r][t * 512], 512 * 2, cudaMemcpyHostToDevice, s));
            CU(cudaMemcpyAsync(dg, &g[r][t * 16], 16 * 2, cudaMemcpyHostToDevice, s));
            CU(cudaMemcpyAsync(dbcx, &bcx[r][t * 6144], 6144 * 2, cudaMemcpyHostToDevice, s));
            engine.conv_decode(s, st, 0, dy, dbcx, dcw);
            engine.attention_decode(s, st, 1, dctx, dq, dk, dv, dg, dw, dw, dcos, dsin, WINDOW);
            CU(cudaStreamSynchronize(s));  // the pinned staging block of the tables is reused
            auto y1 = to_host<__half>(dy, 2048), c1 = to_host<__half>(dctx, 2048);
            CHECK(std::memcmp(y1.data(), &y_wave[r][t * 2048], 2048 * 2) == 0);
            for (size_t i = 0; i < 2048; i++)
                worst = std::fmax(worst, std::fabs((double)__half2float(c1[i]) - (double)__half2float(ctx_wave[r][t * 2048 + i])));
        }
        // caches and conv state of the two leases
        auto ka = to_host<__half>((void*)wave_seq[r]->k_cache_ptr(1), prompt[r] * 512);
        auto kb = to_host<__half>((void*)step_seq[r]->k_cache_ptr(1), prompt[r] * 512);
        auto va = to_host<__half>((void*)wave_seq[r]->v_cache_ptr(1), prompt[r] * 512);
        auto vb = to_host<__half>((void*)step_seq[r]->v_cache_ptr(1), prompt[r] * 512);
        auto sa = to_host<__half>((void*)wave_seq[r]->conv_state_ptr(0), 2048 * 6);
        auto sb = to_host<__half>((void*)step_seq[r]->conv_state_ptr(0), 2048 * 6);
        CHECK(std::memcmp(ka.data(), kb.data(), ka.size() * 2) == 0);
        CHECK(std::memcmp(va.data(), vb.data(), va.size() * 2) == 0);
        CHECK(std::memcmp(va.data(), v[r].data(), va.size() * 2) == 0);
        CHECK(std::memcmp(sa.data(), sb.data(), sa.size() * 2) == 0);
    }
    CHECK(engine.device_status(s) == 0);
    CHECK(worst <= 2e-3);
    std::printf("kv_host prefill checks passed (4 waves, worst |ctx| difference %.2e)\n", worst);
    return 0;
}
