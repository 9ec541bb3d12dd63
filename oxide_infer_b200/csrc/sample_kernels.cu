// The two table-driven kernels on the sampling side of a decode step:
//
//   embed_lookup_kernel   out[b][:] = table[token_ids[b]][:]
//                         replaces batched_embed_lookup_fp16 (batched_attn.rs:664-714, launched at
//                         batch_engine.rs:765-779)
//   argmax_kernel         tokens_out[b] = argmax over the vocabulary of logits[b][:] (f16)
//                         replaces batched_argmax_direct_f16 (batched_attn.rs:890-1023, launched
//                         with 256 threads per row at batch_engine.rs:1367-1378)
//
// Both are HBM-bound byte/index work.  The reference's argmax resolves ties by its scan order
// and its reduction tree, not by the lowest index: thread t of 256 scans t, t+256, ... keeping
// the first strict maximum (start -1e30 / index 0, NaN never wins), then a shuffle-down tree in
// each warp and over the 8 warps, where a lane takes its partner's pair only if strictly greater.
// argmax_kernel reproduces exactly that result with a different memory schedule: the 256
// "virtual threads" of the reference are kept as 256 (value, index) candidates, but each physical
// thread reads 16-byte vectors (8 consecutive logits = 8 consecutive virtual threads, the same 8
// for every vector the thread reads), rows are split over several CTAs so that small batches
// still fill the GPU, and the CTA that finishes a row last merges the splits and runs the
// reference's tree on the 256 candidates.
#include "common.cuh"
#include "kernels.h"

namespace oxi {

namespace sm {
constexpr int VT = 256;          // virtual threads = the reference's block size
constexpr int THREADS = 256;
constexpr int MAX_SPLITS = 8;    // CTAs per row at most
constexpr int LOADS = 8;         // 16-byte loads in flight per thread
constexpr int CTAS_PER_SM = 2;   // grid size aimed at
constexpr int RESIDENT = 3;      // CTAs that fit an SM (80 registers; 85 are the limit for three)
}  // namespace sm

__global__ void __launch_bounds__(256)
embed_lookup_kernel(uint16_t* __restrict__ out, const uint16_t* __restrict__ table,
                    const uint32_t* __restrict__ token_ids, uint32_t hidden, uint32_t table_rows,
                    uint32_t batch, uint32_t* __restrict__ status) {
    const uint32_t b = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();  // the ids come from the preceding kernel (the argmax of the step before)
    if (b >= batch) return;
    const uint32_t tok = token_ids[b];
    const bool bad = tok >= table_rows;
    if (bad && threadIdx.x == 0) atomicOr(status, DEV_BAD_TOKEN);
    const size_t row_bytes = (size_t)hidden * 2;
    const char* src = reinterpret_cast<const char*>(table) + (size_t)(bad ? 0u : tok) * row_bytes;
    char* dst = reinterpret_cast<char*>(out) + (size_t)b * row_bytes;
    if ((((uintptr_t)src | (uintptr_t)dst | row_bytes) & 15u) == 0) {
        for (size_t i = (size_t)threadIdx.x * 16; i < row_bytes; i += (size_t)blockDim.x * 16) {
            const uint4 v = bad ? make_uint4(0u, 0u, 0u, 0u) : __ldg(reinterpret_cast<const uint4*>(src + i));
            *reinterpret_cast<uint4*>(dst + i) = v;
        }
    } else {
        for (uint32_t i = threadIdx.x; i < hidden; i += blockDim.x)
            reinterpret_cast<uint16_t*>(dst)[i] = bad ? (uint16_t)0 : reinterpret_cast<const uint16_t*>(src)[i];
    }
}

// One step of the reference's reduction tree: take the partner's pair only if strictly greater.
__device__ __forceinline__ void tree_step(float& v, uint32_t& ix, int off) {
    const float pv = __shfl_down_sync(0xffffffffu, v, off);
    const uint32_t pi = __shfl_down_sync(0xffffffffu, ix, off);
    if (pv > v) {
        v = pv;
        ix = pi;
    }
}

// Grid (splits, batch).  Scratch per row: splits x 256 candidates (float value, uint32 index) and
// one arrival counter that the last CTA of the row resets to zero.
__global__ void __launch_bounds__(sm::THREADS)
argmax_kernel(uint32_t* __restrict__ tokens_out, const uint16_t* __restrict__ logits,
              uint32_t vocab, uint32_t batch, uint32_t splits, float2* __restrict__ cand_scratch,
              uint32_t* __restrict__ counters) {
    using namespace sm;
    __shared__ float s_v[8][VT];
    __shared__ uint32_t s_i[8][VT];
    __shared__ uint32_t s_last;
    const uint32_t b = blockIdx.y, split = blockIdx.x;
    const int tid = threadIdx.x;
    pdl_launch_dependents();  // a dependent only sets itself up until this grid has finished
    const uint32_t c = tid & 31, grp = tid >> 5;  // this thread serves virtual threads 8c .. 8c+7
    const uint16_t* row = logits + (size_t)b * vocab;

    // Rows of 256 logits ("k-rows": index 256k + t belongs to virtual thread t) are dealt to the
    // splits in contiguous ranges and, inside a split, to the 8 warps round robin.
    const uint32_t nk = (vocab + VT - 1) / VT;
    const uint32_t per = (nk + splits - 1) / splits;
    const uint32_t k0 = min(nk, split * per), k1 = min(nk, k0 + per);
    float mx[8];
    uint32_t bi[8];
#pragma unroll
    for (int e = 0; e < 8; e++) {
        mx[e] = -1.0e30f;
        bi[e] = 0u;
    }
    const bool vec_ok = ((uintptr_t)row & 15u) == 0;
    auto take = [&](int e, uint16_t h, uint32_t idx) {
        const float f = h2f(h);
        if (f > mx[e]) {  // strict: the first maximum of a virtual thread stays (k-rows are visited in increasing order)
            mx[e] = f;
            bi[e] = idx;
        }
    };
    // LOADS vectors in flight per thread; a k-row that is ragged (the last one) or unaligned takes the scalar
    // loads, in the same position of the visiting order
    pdl_wait();  // the logits come from the preceding kernel
    auto is_vec = [&](uint32_t kk) { return vec_ok && kk < k1 && (size_t)kk * VT + VT <= vocab; };
    auto load = [&](uint4 (&v)[LOADS], uint32_t k) {
#pragma unroll
        for (int u = 0; u < LOADS; u++) {
            const uint32_t kk = k + 8 * u;
            if (is_vec(kk)) v[u] = __ldg(reinterpret_cast<const uint4*>(row + (size_t)kk * VT + 8 * c));
        }
    };
    auto scan = [&](const uint4 (&v)[LOADS], uint32_t k) {
#pragma unroll
        for (int u = 0; u < LOADS; u++) {
            const uint32_t kk = k + 8 * u, base = kk * VT + 8 * c;
            if (is_vec(kk)) {
                const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
                for (int e = 0; e < 8; e++) take(e, (uint16_t)(w[e >> 1] >> ((e & 1) * 16)), base + e);
            } else if (kk < k1) {
#pragma unroll
                for (int e = 0; e < 8; e++)
                    if (base + e < vocab) take(e, row[base + e], base + e);
            }
        }
    };
    // one batch at a time: a second register buffer that holds the next batch's loads while this one is scanned
    // measured the same, and at 128 registers no longer fits the grid into one wave
    uint4 vbuf[LOADS];
    for (uint32_t k = k0 + grp; k < k1; k += 8 * LOADS) {
        load(vbuf, k);
        scan(vbuf, k);
    }
#pragma unroll
    for (int e = 0; e < 8; e++) {
        s_v[grp][8 * c + e] = mx[e];
        s_i[grp][8 * c + e] = bi[e];
    }
    __syncthreads();
    // candidate of virtual thread t = tid over this split: the maximum; among equal values the lowest
    // index, which is the one the reference's thread would have met first
    float v = s_v[0][tid];
    uint32_t ix = s_i[0][tid];
#pragma unroll
    for (int g = 1; g < 8; g++) {
        const float gv = s_v[g][tid];
        const uint32_t gi = s_i[g][tid];
        if (gv > v || (gv == v && gv > -1.0e30f && gi < ix)) {
            v = gv;
            ix = gi;
        }
    }
    if (splits > 1) {
        float2* mine = cand_scratch + ((size_t)b * MAX_SPLITS + split) * VT;
        mine[tid] = make_float2(v, __uint_as_float(ix));
        __threadfence();
        __syncthreads();
        if (tid == 0) s_last = atomicAdd(&counters[b], 1u) == splits - 1 ? 1u : 0u;
        __syncthreads();
        if (!s_last) return;
        __threadfence();
        if (tid == 0) counters[b] = 0u;  // ready for the next launch
        v = -1.0e30f;
        ix = 0u;
        float2 cnd[MAX_SPLITS];
#pragma unroll
        for (int s = 0; s < MAX_SPLITS; s++)  // all loads in flight at once
            if ((uint32_t)s < splits) cnd[s] = __ldcg(cand_scratch + ((size_t)b * MAX_SPLITS + s) * VT + tid);
#pragma unroll
        for (int s = 0; s < MAX_SPLITS; s++)  // splits hold increasing index ranges: strict > keeps the first
            if ((uint32_t)s < splits && cnd[s].x > v) {
                v = cnd[s].x;
                ix = __float_as_uint(cnd[s].y);
            }
    }
    // the reference's tree over the 256 candidates
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) tree_step(v, ix, off);
    __syncthreads();
    if ((tid & 31) == 0) {
        s_v[0][tid >> 5] = v;
        s_i[0][tid >> 5] = ix;
    }
    __syncthreads();
    if (tid < 32) {
        v = tid < 8 ? s_v[0][tid] : -1.0e30f;
        ix = tid < 8 ? s_i[0][tid] : 0u;
        // offsets 4, 2, 1 over lanes 0..7; lanes 8.. only feed lanes that never reach lane 0
#pragma unroll
        for (int off = 4; off >= 1; off >>= 1) {
            const float pv = __shfl_down_sync(0xffffffffu, v, off);
            const uint32_t pi = __shfl_down_sync(0xffffffffu, ix, off);
            if (tid + off < 8 && pv > v) {
                v = pv;
                ix = pi;
            }
        }
        if (tid == 0) tokens_out[b] = ix;
    }
}

uint32_t argmax_max_splits() { return sm::MAX_SPLITS; }

cudaError_t launch_embed_lookup(cudaStream_t stream, void* out, const void* table,
                                const uint32_t* token_ids, uint32_t hidden, uint32_t table_rows,
                                uint32_t batch, uint32_t* status) {
    return launch_pdl(embed_lookup_kernel, dim3(batch), dim3(256), 0, stream, (uint16_t*)out, (const uint16_t*)table, token_ids,
                      hidden, table_rows, batch, status);
}

cudaError_t launch_argmax(cudaStream_t stream, uint32_t* tokens_out, const void* logits, uint32_t vocab,
                          uint32_t batch, int num_sms, void* cand_scratch, uint32_t* counters) {
    // enough CTAs for two per SM, all resident at once (a grid that needs a second wave measured 40 % slower),
    // but no split shorter than 32 k-rows (8192 logits)
    uint32_t splits = (uint32_t)(sm::CTAS_PER_SM * num_sms + (int)batch - 1) / batch;
    const uint32_t nk = (vocab + sm::VT - 1) / sm::VT;
    const uint32_t by_len = nk / 32u;
    if (splits > by_len) splits = by_len;
    if (splits > (uint32_t)sm::MAX_SPLITS) splits = sm::MAX_SPLITS;
    while (splits > 1u && splits * batch > (uint32_t)(sm::RESIDENT * num_sms)) splits--;
    if (splits < 1u) splits = 1u;
    return launch_pdl(argmax_kernel, dim3(splits, batch), dim3(sm::THREADS), 0, stream, tokens_out, (const uint16_t*)logits, vocab,
                      batch, splits, (float2*)cand_scratch, counters);
}

}  // namespace oxi
