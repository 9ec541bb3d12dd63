// Chunked-prefill causal GQA attention with the sigmoid gate over per-row
// pointer tables, as one fused flash-attention kernel (scores and weights stay
// on chip).
//
// Replaces BatchEngine::gemm_attention_chunk (batch_engine.rs:439-592: pack_q,
// cuBLASLt QK^T to f32 scores in HBM, softmax_mask to f16 weights in HBM,
// cuBLASLt PV, gate_scatter) and the per-row online-kernel fallback
// (batch_engine.rs:1214-1239).
//
// Row r of the wave attends keys [window start(seq_lens[r]), seq_lens[r]) of
// the cache k_ptrs[r] / v_ptrs[r]; all rows' K/V were appended before the call,
// so causality is the per-row upper bound.  A CTA owns TM consecutive wave rows
// and one KV head; its four warps are the four query heads of that group, so a
// K/V tile is read once for 4*TM (row, head) pairs.  Rows of a tile that point
// at different caches are handled as separate runs of equal pointers, so any
// table contents are legal; rows of one request with consecutive positions
// (what the engine produces) form one run.
#include "common.cuh"
#include "kernels.h"

namespace oxi {

namespace pf {
constexpr int TM = 16;                 // wave rows per CTA
constexpr int TK = 64;                 // keys per tile
constexpr int PITCH = HD * 2 + 16;     // 272 B per key row of one KV head in shared memory
constexpr int TILE_BYTES = TK * PITCH; // one K (or V) tile
constexpr int NBUF = 2;
constexpr int THREADS = 128;
constexpr size_t SMEM_BYTES = (size_t)NBUF * 2 * TILE_BYTES;
constexpr float QK_SCALE_LOG2 = ATTN_SCALE * LOG2E;
}  // namespace pf

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
    const uint32_t n = valid ? 16u : 0u;  // 0 source bytes: destination is zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__global__ void __launch_bounds__(pf::THREADS)
prefill_attn_kernel(uint16_t* __restrict__ ctx_out, const uint16_t* __restrict__ q,
                    const uint16_t* __restrict__ gate, const uint64_t* __restrict__ k_ptrs,
                    const uint64_t* __restrict__ v_ptrs, const uint32_t* __restrict__ seq_lens,
                    uint32_t rows, uint32_t window, uint32_t* __restrict__ status) {
    using namespace pf;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ uint64_t s_kp[TM], s_vp[TM];
    __shared__ uint32_t s_len[TM];

    const uint32_t row0 = blockIdx.x * TM;
    const int kvh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const int head = kvh * 4 + warp;
    const uint32_t nrows = min((uint32_t)TM, rows - row0);

    if (threadIdx.x < TM) {
        const uint32_t r = row0 + threadIdx.x;
        uint64_t kp = 0, vp = 0;
        uint32_t sl = 0;
        if (threadIdx.x < nrows) {
            kp = k_ptrs[r];
            vp = v_ptrs[r];
            sl = seq_lens[r];
            if (((kp | vp) & 15ull) != 0ull) {
                if (kvh == 0) atomicOr(status, DEV_MISALIGNED_PTR);
                sl = 0;
            } else if (sl == 0u) {
                if (kvh == 0) atomicOr(status, DEV_BAD_SEQ_LEN);
            }
        }
        s_kp[threadIdx.x] = kp;
        s_vp[threadIdx.x] = vp;
        s_len[threadIdx.x] = sl;  // 0 marks a row that is skipped
    }
    __syncthreads();

    // Q fragments for rows g and g+8 of this warp's head
    uint32_t qa[8][4];
    {
        const bool v0 = (uint32_t)g < nrows, v1 = (uint32_t)(g + 8) < nrows;
        const uint16_t* q0 = q + ((size_t)(row0 + g) * NQ + head) * HD;
        const uint16_t* q1 = q + ((size_t)(row0 + g + 8) * NQ + head) * HD;
#pragma unroll
        for (int ks = 0; ks < 8; ks++) {
            qa[ks][0] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + 16 * ks + 2 * t4) : 0u;
            qa[ks][1] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + 16 * ks + 2 * t4) : 0u;
            qa[ks][2] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + 16 * ks + 8 + 2 * t4) : 0u;
            qa[ks][3] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + 16 * ks + 8 + 2 * t4) : 0u;
        }
    }
    float o[16][4];
#pragma unroll
    for (int j = 0; j < 16; j++) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f; }
    float m_run[2] = {-1.0e30f, -1.0e30f}, l_run[2] = {0.0f, 0.0f};

    // ---- runs of rows that share one cache
    uint32_t run0 = 0;
    while (run0 < nrows) {
        uint32_t run1 = run0 + 1;
        while (run1 < nrows && s_kp[run1] == s_kp[run0] && s_vp[run1] == s_vp[run0]) run1++;
        uint32_t lo = 0xffffffffu, hi = 0;
        for (uint32_t i = run0; i < run1; i++) {
            const uint32_t sl = s_len[i];
            if (sl == 0) continue;
            lo = min(lo, window_start(sl, window));
            hi = max(hi, sl);
        }
        if (hi > lo) {
            // this thread's two rows: valid key interval inside the run, empty if not in the run
            uint32_t rlo[2], rhi[2];
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const uint32_t rr = g + 8 * i;
                const bool in = rr >= run0 && rr < run1 && s_len[rr] != 0;
                rhi[i] = in ? s_len[rr] : 0u;
                rlo[i] = in ? window_start(s_len[rr], window) : 0u;
            }
            const char* kbase = reinterpret_cast<const char*>(s_kp[run0]) + kvh * (HD * 2);
            const char* vbase = reinterpret_cast<const char*>(s_vp[run0]) + kvh * (HD * 2);
            const uint32_t ntiles = (hi - lo + TK - 1) / TK;

            auto load_tile = [&](uint32_t tile, int buf) {
                const uint32_t kbeg = lo + tile * TK;
                unsigned char* kb = smem + (size_t)buf * 2 * TILE_BYTES;
                const uint32_t ks_addr = smem_u32(kb), vs_addr = smem_u32(kb + TILE_BYTES);
                for (uint32_t i = threadIdx.x; i < TK * 16; i += THREADS) {
                    const uint32_t key = i >> 4, seg = i & 15u;
                    const bool valid = kbeg + key < hi;
                    const size_t goff = (size_t)(valid ? kbeg + key : lo) * KV_ROW_BYTES + seg * 16;
                    cp_async_16(ks_addr + key * PITCH + seg * 16, kbase + goff, valid);
                    cp_async_16(vs_addr + key * PITCH + seg * 16, vbase + goff, valid);
                }
                cp_async_commit();
            };

            __syncthreads();  // previous run's tiles fully consumed
            load_tile(0, 0);
            for (uint32_t tile = 0; tile < ntiles; tile++) {
                const int buf = tile & 1;
                if (tile + 1 < ntiles) {
                    load_tile(tile + 1, buf ^ 1);
                    cp_async_wait<1>();
                } else {
                    cp_async_wait<0>();
                }
                __syncthreads();
                const uint32_t kbeg = lo + tile * TK;
                const uint32_t ks_addr = smem_u32(smem + (size_t)buf * 2 * TILE_BYTES);
                const uint32_t vs_addr = ks_addr + TILE_BYTES;

                // S = Q K^T : 8 n-blocks of 8 keys
                float s[8][4];
#pragma unroll
                for (int nb = 0; nb < 8; nb++) {
                    s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.0f;
                    const uint32_t kaddr = ks_addr + (nb * 8 + (lane & 7)) * PITCH + (lane >> 3) * 16;
#pragma unroll
                    for (int kk = 0; kk < 4; kk++) {
                        uint32_t r0, r1, r2, r3;
                        ldmatrix_x4(kaddr + kk * 64, r0, r1, r2, r3);
                        mma_16816(s[nb], qa[2 * kk][0], qa[2 * kk][1], qa[2 * kk][2], qa[2 * kk][3], r0, r1);
                        mma_16816(s[nb], qa[2 * kk + 1][0], qa[2 * kk + 1][1], qa[2 * kk + 1][2],
                                  qa[2 * kk + 1][3], r2, r3);
                    }
                }
                // masks + online softmax for rows g (regs 0,1) and g+8 (regs 2,3)
                float mx[2] = {-1.0e30f, -1.0e30f};
#pragma unroll
                for (int nb = 0; nb < 8; nb++) {
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const int i = j >> 1;
                        const uint32_t key = kbeg + nb * 8 + 2 * t4 + (j & 1);
                        float v = s[nb][j] * QK_SCALE_LOG2;
                        v = (key >= rlo[i] && key < rhi[i]) ? v : -INFINITY;
                        s[nb][j] = v;
                        mx[i] = fmaxf(mx[i], v);
                    }
                }
                float corr[2];
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
                    const float m_new = fmaxf(m_run[i], mx[i]);
                    corr[i] = ex2_approx_ftz(m_run[i] - m_new);
                    m_run[i] = m_new;
                }
                uint32_t pa[8][2];
                float psum[2] = {0.0f, 0.0f};
#pragma unroll
                for (int nb = 0; nb < 8; nb++) {
                    const float p0 = ex2_approx_ftz(s[nb][0] - m_run[0]);
                    const float p1 = ex2_approx_ftz(s[nb][1] - m_run[0]);
                    const float p2 = ex2_approx_ftz(s[nb][2] - m_run[1]);
                    const float p3 = ex2_approx_ftz(s[nb][3] - m_run[1]);
                    psum[0] += p0 + p1;
                    psum[1] += p2 + p3;
                    pa[nb][0] = pack_h2(p0, p1);
                    pa[nb][1] = pack_h2(p2, p3);
                }
#pragma unroll
                for (int i = 0; i < 2; i++) l_run[i] = l_run[i] * corr[i] + psum[i];
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    o[j][0] *= corr[0]; o[j][1] *= corr[0];
                    o[j][2] *= corr[1]; o[j][3] *= corr[1];
                }
                // O += P V : 4 k-steps of 16 keys
#pragma unroll
                for (int k2 = 0; k2 < 4; k2++) {
                    const uint32_t vaddr = vs_addr + (k2 * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * PITCH +
                                           (lane >> 4) * 16;
#pragma unroll
                    for (int jn = 0; jn < 8; jn++) {
                        uint32_t r0, r1, r2, r3;
                        ldmatrix_x4_trans(vaddr + jn * 32, r0, r1, r2, r3);
                        mma_16816(o[2 * jn], pa[2 * k2][0], pa[2 * k2][1], pa[2 * k2 + 1][0],
                                  pa[2 * k2 + 1][1], r0, r1);
                        mma_16816(o[2 * jn + 1], pa[2 * k2][0], pa[2 * k2][1], pa[2 * k2 + 1][0],
                                  pa[2 * k2 + 1][1], r2, r3);
                    }
                }
                __syncthreads();  // tile consumed before its buffer is refilled
            }
        }
        run0 = run1;
    }

    // ---- epilogue: 1/sum, f16, gate on the f16 value (as online kernel + gate kernel)
#pragma unroll
    for (int i = 0; i < 2; i++) {  // row sums across the quad (every lane takes part)
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    }
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const uint32_t rr = g + 8 * i;
        if (rr >= nrows || s_len[rr] == 0) continue;
        const float inv = rcp_approx_ftz(l_run[i]);
        const size_t rh = (size_t)(row0 + rr) * NQ + head;
        const float sig = gate ? sigmoid_ref(h2f(gate[rh])) : 1.0f;
        uint16_t* out = ctx_out + rh * HD;
#pragma unroll
        for (int j = 0; j < 16; j++) {
            uint16_t h0 = f2h(__fmul_rn(o[j][2 * i], inv));
            uint16_t h1 = f2h(__fmul_rn(o[j][2 * i + 1], inv));
            if (gate) {
                h0 = f2h(__fmul_rn(h2f(h0), sig));
                h1 = f2h(__fmul_rn(h2f(h1), sig));
            }
            *reinterpret_cast<uint32_t*>(out + 8 * j + 2 * t4) = (uint32_t)h0 | ((uint32_t)h1 << 16);
        }
    }
}

cudaError_t prefill_attn_init() {
    return cudaFuncSetAttribute(prefill_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)pf::SMEM_BYTES);
}

cudaError_t launch_prefill_attn(cudaStream_t stream, void* ctx_out, const void* q,
                                const void* gate, const uint64_t* k_ptrs, const uint64_t* v_ptrs,
                                const uint32_t* seq_lens, uint32_t rows, uint32_t window,
                                uint32_t* status, int num_sms) {
    (void)num_sms;
    dim3 grid((rows + pf::TM - 1) / pf::TM, NKV);
    prefill_attn_kernel<<<grid, pf::THREADS, pf::SMEM_BYTES, stream>>>(
        (uint16_t*)ctx_out, (const uint16_t*)q, (const uint16_t*)gate, k_ptrs, v_ptrs, seq_lens,
        rows, window, status);
    return cudaGetLastError();
}

}  // namespace oxi
