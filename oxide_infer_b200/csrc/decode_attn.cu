// Split-KV flash-decode GQA attention with the sigmoid output gate, one launch.
//
// Replaces batched_gqa_attention_split4_fp16 + batched_gqa_attn_combine_fp16 +
// batched_sigmoid_gate_fp16 (batched_attn.rs:2665-3035, 1597-1717, 583-655).
//
// Work decomposition.  A work item is (row b, key range c) where the ranges
// are fixed CHUNK-key slices of the row's own [window start, seq_len) interval,
// so a row's arithmetic never depends on which other rows share the launch.
// The grid is persistent (a fixed number of CTAs per SM); every CTA derives the
// item list from seq_lens on the device (prefix sum of per-row chunk counts in
// shared memory) and takes items blockIdx.x, +gridDim.x, ...  The host needs no
// knowledge of the lengths and the launch shape never changes.
//
// Inside a CTA: one producer warp streams K and V rows (1024 B each: all four
// KV heads of one token are contiguous) into a ring of shared-memory stages
// with 1-D bulk copies (TMA engine) that complete on mbarriers; four consumer
// warps, one per KV head, each serve the 4 query heads of their group from
// that single K/V read: S = Q K^T and O += P V run on tensor cores
// (mma.sync.m16n8k16, f16 in, f32 accumulate; the 4 heads are rows 0..3 of the
// M=16 tile), the online-softmax row reductions are quad shuffles.  Rows are
// stored with a 1040-byte pitch so the 8 row addresses of every ldmatrix phase
// fall in distinct banks.
//
// A row covered by one item is finished in registers.  Otherwise each consumer
// warp writes its (max, sum, acc[128]) partials, bumps an arrival counter for
// (row, kv head), and the warp that arrives last merges all partials of that
// (row, kv head) in key-range order (deterministic), applies 1/sum, rounds to
// f16, applies the gate exactly as the reference's gate kernel does on the f16
// context, and resets the counter.  Nothing spins on another CTA.
#include "common.cuh"
#include "kernels.h"

namespace oxi {

namespace dec {
constexpr int KS = 32;                        // keys per pipeline stage
constexpr int NSTAGE = 3;                     // ring depth
constexpr int PITCH = KV_ROW_BYTES + 16;      // 1040 B per key row in shared memory
constexpr int STAGE_BYTES = 2 * KS * PITCH;   // K rows then V rows
constexpr int CHUNK = 256;                    // keys per work item
constexpr int N_CONSUMER_WARPS = NKV;         // one per KV head
constexpr int THREADS = (N_CONSUMER_WARPS + 1) * 32;
constexpr int MAX_ROWS = 4096;                // rows per launch (prefix array in shared memory)
constexpr int CTAS_PER_SM = 1;
constexpr float QK_SCALE_LOG2 = ATTN_SCALE * LOG2E;
constexpr size_t SMEM_BYTES = (size_t)NSTAGE * STAGE_BYTES + 2 * NSTAGE * 8 + 16 +
                              (MAX_ROWS + 1) * sizeof(uint32_t);
static_assert(SMEM_BYTES <= 227 * 1024, "decode kernel shared memory");
static_assert(CHUNK % KS == 0, "a work item is a whole number of stages");
}  // namespace dec

struct DecodeParams {
    uint16_t* ctx_out;
    const uint16_t* q;
    const uint16_t* gate;  // may be null
    const uint64_t* k_ptrs;
    const uint64_t* v_ptrs;
    const uint32_t* seq_lens;
    float* partial_acc;
    float* partial_stats;
    uint32_t* counters;
    uint32_t* status;
    uint32_t batch;
    uint32_t window;
    uint32_t max_chunks;
    uint32_t max_seq_len;
};

__device__ __forceinline__ uint32_t row_chunks(uint32_t slen, uint32_t window) {
    const uint32_t eff = slen - window_start(slen, window);
    return (eff + dec::CHUNK - 1) / dec::CHUNK;
}

// largest b with prefix[b] <= item  (prefix[0] = 0, prefix[batch] = total)
__device__ __forceinline__ uint32_t find_row(const uint32_t* prefix, uint32_t batch, uint32_t item) {
    uint32_t lo = 0, hi = batch;  // answer in [lo, hi)
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (prefix[mid] <= item) lo = mid; else hi = mid;
    }
    return lo;
}

__global__ void __launch_bounds__(dec::THREADS, dec::CTAS_PER_SM)
decode_attn_kernel(const DecodeParams p) {
    using namespace dec;
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* stages = smem;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)NSTAGE * STAGE_BYTES);
    uint64_t* empty_bar = full_bar + NSTAGE;
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(empty_bar + NSTAGE);
    uint32_t* prefix = const_cast<uint32_t*>(reinterpret_cast<volatile uint32_t*>(abort_flag) + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // ---- prologue: barriers, per-row chunk counts, prefix sum
    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGE; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], N_CONSUMER_WARPS);
        }
        *abort_flag = 0u;
        prefix[0] = 0u;
        mbar_fence_init();
    }
    for (uint32_t b = threadIdx.x; b < p.batch; b += THREADS) {
        const uint32_t slen = p.seq_lens[b];
        uint32_t n = 0;
        if (slen == 0u || slen > p.max_seq_len) {
            if (blockIdx.x == 0) atomicOr(p.status, DEV_BAD_SEQ_LEN);
        } else if (((p.k_ptrs[b] | p.v_ptrs[b]) & 15ull) != 0ull) {
            if (blockIdx.x == 0) atomicOr(p.status, DEV_MISALIGNED_PTR);
        } else {
            n = row_chunks(slen, p.window);
        }
        prefix[b + 1] = n;
    }
    __syncthreads();
    if (warp == 0) {
        uint32_t carry = 0;
        for (uint32_t base = 0; base < p.batch; base += 32) {
            const uint32_t i = base + lane;
            uint32_t v = (i < p.batch) ? prefix[i + 1] : 0u;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const uint32_t t = __shfl_up_sync(0xffffffffu, v, off);
                if (lane >= off) v += t;
            }
            v += carry;
            if (i < p.batch) prefix[i + 1] = v;
            carry = __shfl_sync(0xffffffffu, v, 31);
        }
    }
    __syncthreads();
    const uint32_t total_items = prefix[p.batch];

    if (warp == N_CONSUMER_WARPS) {
        // =========================== producer warp ===========================
        const uint64_t policy = l2_policy_evict_first();
        uint32_t fill = 0;
        bool ok = true;
        for (uint32_t item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
            const uint32_t b = find_row(prefix, p.batch, item);
            const uint32_t c = item - prefix[b];
            const uint32_t slen = p.seq_lens[b];
            const uint32_t t0 = window_start(slen, p.window) + c * CHUNK;
            const uint32_t t1 = min(t0 + (uint32_t)CHUNK, slen);
            const char* kp = reinterpret_cast<const char*>(p.k_ptrs[b]);
            const char* vp = reinterpret_cast<const char*>(p.v_ptrs[b]);
            for (uint32_t t = t0; t < t1; t += KS, ++fill) {
                const uint32_t slot = fill % NSTAGE;
                if (fill >= NSTAGE) {
                    if (!mbar_wait_bounded(&empty_bar[slot], ((fill / NSTAGE) & 1u) ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                }
                const uint32_t nvalid = min((uint32_t)KS, t1 - t);
                if (lane == 0) mbar_arrive_expect_tx(&full_bar[slot], nvalid * 2u * KV_ROW_BYTES);
                __syncwarp();
                const uint32_t sbase = smem_u32(stages + (size_t)slot * STAGE_BYTES);
                for (uint32_t i = lane; i < 2u * nvalid; i += 32) {
                    const bool is_v = i >= nvalid;
                    const uint32_t key = is_v ? i - nvalid : i;
                    const char* src = (is_v ? vp : kp) + (size_t)(t + key) * KV_ROW_BYTES;
                    const uint32_t dst = sbase + (is_v ? KS * PITCH : 0) + key * PITCH;
                    bulk_g2s_hint(dst, src, KV_ROW_BYTES, &full_bar[slot], policy);
                }
            }
        }
        if (!ok) {
            // Pipeline gave up: report, then give the copies already issued a bounded
            // time to land before this CTA's shared memory is released.
            if (lane == 0) atomicOr(p.status, DEV_WAIT_TIMEOUT);
            for (uint32_t k = fill > NSTAGE ? fill - NSTAGE : 0; k < fill; ++k)
                mbar_wait_iters(&full_bar[k % NSTAGE], (k / NSTAGE) & 1u, 1u << 16);
        }
        return;
    }

    // ============================= consumer warps =============================
    const int kvh = warp;            // this warp's KV head
    const int g = lane >> 2;         // fragment row (query head within the group when g < 4)
    const int t4 = lane & 3;         // fragment column pair
    uint32_t take = 0;               // stages consumed so far (mirrors the producer's `fill`)
    bool ok = true;

    for (uint32_t item = blockIdx.x; item < total_items; item += gridDim.x) {
        const uint32_t b = find_row(prefix, p.batch, item);
        const uint32_t c = item - prefix[b];
        const uint32_t nchunks = prefix[b + 1] - prefix[b];
        const uint32_t slen = p.seq_lens[b];
        const uint32_t t0 = window_start(slen, p.window) + c * CHUNK;
        const uint32_t t1 = min(t0 + (uint32_t)CHUNK, slen);

        // Q fragments (A operand, rows 0..3 = the group's heads, rows 4..15 zero)
        uint32_t qa[8][2];
        {
            const uint16_t* qrow = p.q + ((size_t)b * NQ + kvh * 4 + (g & 3)) * HD;
#pragma unroll
            for (int ks = 0; ks < 8; ks++) {
                uint32_t lo = 0, hi = 0;
                if (g < 4) {
                    lo = *reinterpret_cast<const uint32_t*>(qrow + 16 * ks + 2 * t4);
                    hi = *reinterpret_cast<const uint32_t*>(qrow + 16 * ks + 8 + 2 * t4);
                }
                qa[ks][0] = lo;
                qa[ks][1] = hi;
            }
        }
        float o[16][4];
#pragma unroll
        for (int j = 0; j < 16; j++) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f; }
        float m_run = -1.0e30f, l_run = 0.0f;

        for (uint32_t t = t0; t < t1; t += KS, ++take) {
            const uint32_t slot = take % NSTAGE;
            if (ok) ok = mbar_wait_bounded(&full_bar[slot], (take / NSTAGE) & 1u, abort_flag);
            const uint32_t nvalid = min((uint32_t)KS, t1 - t);
            unsigned char* kst = stages + (size_t)slot * STAGE_BYTES + kvh * (HD * 2);
            unsigned char* vst = kst + KS * PITCH;
            if (nvalid < KS) {
                // tail stage: rows past the range keep stale bytes; zero this head's V slice there
                // so that 0 * stale can never produce NaN.
                for (uint32_t i = lane; i < (KS - nvalid) * 16u; i += 32) {
                    const uint32_t row = nvalid + (i >> 4);
                    *reinterpret_cast<uint4*>(vst + row * PITCH + (i & 15u) * 16u) = make_uint4(0, 0, 0, 0);
                }
                __syncwarp();
            }

            // ---- S = Q K^T for 32 keys: 4 n-blocks of 8 keys
            float s[4][4];
#pragma unroll
            for (int nb = 0; nb < 4; nb++) {
                s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.0f;
                const uint32_t kaddr = smem_u32(kst) + (nb * 8 + (lane & 7)) * PITCH + (lane >> 3) * 16;
#pragma unroll
                for (int kk = 0; kk < 4; kk++) {
                    uint32_t r0, r1, r2, r3;
                    ldmatrix_x4(kaddr + kk * 64, r0, r1, r2, r3);
                    mma_16816(s[nb], qa[2 * kk][0], 0u, qa[2 * kk][1], 0u, r0, r1);
                    mma_16816(s[nb], qa[2 * kk + 1][0], 0u, qa[2 * kk + 1][1], 0u, r2, r3);
                }
            }
            // ---- online softmax on row g (keys nb*8 + 2*t4 + {0,1})
            float mx = -1.0e30f;
#pragma unroll
            for (int nb = 0; nb < 4; nb++) {
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const uint32_t key = nb * 8 + 2 * t4 + j;
                    float v = s[nb][j] * QK_SCALE_LOG2;
                    v = (key < nvalid) ? v : -INFINITY;
                    s[nb][j] = v;
                    mx = fmaxf(mx, v);
                }
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run, mx);
            const float corr = ex2_approx_ftz(m_run - m_new);
            m_run = m_new;
            float psum = 0.0f;
            uint32_t pa[4];
#pragma unroll
            for (int nb = 0; nb < 4; nb++) {
                const float p0 = ex2_approx_ftz(s[nb][0] - m_new);
                const float p1 = ex2_approx_ftz(s[nb][1] - m_new);
                psum += p0 + p1;
                pa[nb] = pack_h2(p0, p1);
            }
            l_run = l_run * corr + psum;
#pragma unroll
            for (int j = 0; j < 16; j++) { o[j][0] *= corr; o[j][1] *= corr; }

            // ---- O += P V : 2 k-steps of 16 keys, 16 n-blocks of 8 dims
#pragma unroll
            for (int k2 = 0; k2 < 2; k2++) {
                const uint32_t vaddr = smem_u32(vst) +
                                       (k2 * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * PITCH +
                                       (lane >> 4) * 16;
#pragma unroll
                for (int jn = 0; jn < 8; jn++) {
                    uint32_t r0, r1, r2, r3;
                    ldmatrix_x4_trans(vaddr + jn * 32, r0, r1, r2, r3);
                    mma_16816(o[2 * jn], pa[2 * k2], 0u, pa[2 * k2 + 1], 0u, r0, r1);
                    mma_16816(o[2 * jn + 1], pa[2 * k2], 0u, pa[2 * k2 + 1], 0u, r2, r3);
                }
            }
            // release the stage (generic writes of a tail stage are ordered before later bulk copies)
            if (nvalid < KS) fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[slot]);
        }

        // ---- finish the item: row sums across the quad
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
        const uint32_t head = kvh * 4 + (g & 3);

        if (nchunks == 1) {
            if (g < 4) {
                const float inv = rcp_approx_ftz(l_run);
                const float sig = p.gate ? sigmoid_ref(h2f(p.gate[(size_t)b * NQ + head])) : 1.0f;
                uint16_t* out = p.ctx_out + ((size_t)b * NQ + head) * HD;
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    uint16_t h0 = f2h(__fmul_rn(o[j][0], inv));
                    uint16_t h1 = f2h(__fmul_rn(o[j][1], inv));
                    if (p.gate) {
                        h0 = f2h(__fmul_rn(h2f(h0), sig));
                        h1 = f2h(__fmul_rn(h2f(h1), sig));
                    }
                    *reinterpret_cast<uint32_t*>(out + 8 * j + 2 * t4) = (uint32_t)h0 | ((uint32_t)h1 << 16);
                }
            }
            continue;
        }

        // ---- several items cover this row: publish partials, last arrival merges
        const size_t pbase = ((size_t)b * p.max_chunks + c) * NQ;
        if (g < 4) {
            float* pacc = p.partial_acc + (pbase + head) * HD;
#pragma unroll
            for (int j = 0; j < 16; j++)
                __stcg(reinterpret_cast<float2*>(pacc + 8 * j + 2 * t4), make_float2(o[j][0], o[j][1]));
            if (t4 == 0)
                __stcg(reinterpret_cast<float2*>(p.partial_stats + (pbase + head) * 2),
                       make_float2(m_run, l_run));
        }
        __threadfence();
        __syncwarp();
        uint32_t arrived = 0;
        if (lane == 0) arrived = atomicAdd(&p.counters[b * NKV + kvh], 1u);
        arrived = __shfl_sync(0xffffffffu, arrived, 0);
        if (arrived != nchunks - 1) continue;

        __threadfence();
        // merge in key-range order; lane owns dims 4*lane .. 4*lane+3 of each head
        for (int hh = 0; hh < 4; hh++) {
            const uint32_t hd = kvh * 4 + hh;
            float m = -1.0e30f, l = 0.0f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (uint32_t cc = 0; cc < nchunks; cc++) {
                const size_t pi = ((size_t)b * p.max_chunks + cc) * NQ + hd;
                const float2 st = __ldcg(reinterpret_cast<const float2*>(p.partial_stats + pi * 2));
                const float4 pv = __ldcg(reinterpret_cast<const float4*>(p.partial_acc + pi * HD) + lane);
                const float m_new = fmaxf(m, st.x);
                const float c_old = ex2_approx_ftz(m - m_new);
                const float c_new = ex2_approx_ftz(st.x - m_new);
                l = l * c_old + c_new * st.y;
                acc.x = acc.x * c_old + c_new * pv.x;
                acc.y = acc.y * c_old + c_new * pv.y;
                acc.z = acc.z * c_old + c_new * pv.z;
                acc.w = acc.w * c_old + c_new * pv.w;
                m = m_new;
            }
            const float inv = rcp_approx_ftz(l);
            uint16_t h[4] = {f2h(__fmul_rn(acc.x, inv)), f2h(__fmul_rn(acc.y, inv)),
                             f2h(__fmul_rn(acc.z, inv)), f2h(__fmul_rn(acc.w, inv))};
            if (p.gate) {
                const float sig = sigmoid_ref(h2f(p.gate[(size_t)b * NQ + hd]));
#pragma unroll
                for (int i = 0; i < 4; i++) h[i] = f2h(__fmul_rn(h2f(h[i]), sig));
            }
            uint2 packed = make_uint2((uint32_t)h[0] | ((uint32_t)h[1] << 16),
                                      (uint32_t)h[2] | ((uint32_t)h[3] << 16));
            *reinterpret_cast<uint2*>(p.ctx_out + ((size_t)b * NQ + hd) * HD + 4 * lane) = packed;
        }
        if (lane == 0) p.counters[b * NKV + kvh] = 0u;  // ready for the next launch
    }
    if (!ok && lane == 0) atomicOr(p.status, DEV_WAIT_TIMEOUT);
}

uint32_t decode_chunk_keys() { return dec::CHUNK; }

cudaError_t decode_attn_init() {
    return cudaFuncSetAttribute(decode_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)dec::SMEM_BYTES);
}

cudaError_t launch_decode_attn(cudaStream_t stream, const DecodeWorkspace& ws, void* ctx_out,
                               const void* q, const void* gate, const uint64_t* k_ptrs,
                               const uint64_t* v_ptrs, const uint32_t* seq_lens, uint32_t batch,
                               uint32_t window) {
    DecodeParams p;
    p.ctx_out = (uint16_t*)ctx_out;
    p.q = (const uint16_t*)q;
    p.gate = (const uint16_t*)gate;
    p.k_ptrs = k_ptrs;
    p.v_ptrs = v_ptrs;
    p.seq_lens = seq_lens;
    p.partial_acc = ws.partial_acc;
    p.partial_stats = ws.partial_stats;
    p.counters = ws.counters;
    p.status = ws.status;
    p.batch = batch;
    p.window = window;
    p.max_chunks = ws.max_chunks;
    p.max_seq_len = ws.max_seq_len;
    const int grid = ws.num_sms * dec::CTAS_PER_SM;
    decode_attn_kernel<<<grid, dec::THREADS, dec::SMEM_BYTES, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace oxi
