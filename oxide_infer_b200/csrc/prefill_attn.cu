// Chunked-prefill causal GQA attention with the sigmoid gate over per-row
// pointer tables, as one fused flash-attention kernel on the 5th-generation
// tensor cores: tcgen05.mma with accumulators in tensor memory (TMEM).  Scores
// and weights stay on chip.
//
// Replaces BatchEngine::gemm_attention_chunk (batch_engine.rs:439-592: pack_q,
// cuBLASLt QK^T to f32 scores in HBM, softmax_mask to f16 weights in HBM,
// cuBLASLt PV, gate_scatter) and the per-row online-kernel fallback
// (batch_engine.rs:1214-1239).
//
// Row r of the wave attends keys [window start(seq_lens[r]), seq_lens[r]) of
// the cache k_ptrs[r] / v_ptrs[r]; all rows' K/V were appended before the call,
// so causality is the per-row upper bound.
//
// A CTA owns 32 consecutive wave rows (tokens) and one KV head: its M = 128
// tile is (4 query heads of the group) x (32 tokens), row = head*32 + token, so
// a K/V tile is read once for 128 (token, head) pairs and warp w / lane l of the
// CTA owns exactly row (head w, token l) of the accumulator, which is TMEM lane
// 32*w + l: the softmax is thread-local, no shuffles.
//
// Per 64-key tile:  S = Q K^T  (tcgen05.mma, A = Q from shared memory, B = K tile
// from shared memory, both K-major with the 128-byte swizzle, D = S in TMEM)
// -> each thread loads its S row (tcgen05.ld), applies scale, causal/window
// mask and the online-softmax update, writes P as f16 back to TMEM
// (tcgen05.st) -> O_tile = P V (tcgen05.mma, A = P from TMEM, B = V tile from
// shared memory, MN-major) -> each thread adds its O_tile row into its f32
// accumulator registers (rescaled by the softmax correction while the MMA runs).
// K/V tiles are double buffered with cp.async (16-byte chunks written straight
// into the swizzled layout, zero-filled past the run's last key).  Two CTAs are
// resident per SM (256 of the 512 TMEM columns each), so one CTA's softmax
// overlaps the other's MMAs.
//
// Rows of a 32-row block that point at different caches are processed as
// separate runs of equal pointers (rows outside the run are masked), so any
// table contents are legal; the engine's waves (consecutive positions of one
// request per chunk) give one run per block except where a chunk boundary falls
// inside a block.
#include "common.cuh"
#include "kernels.h"

namespace oxi {

namespace pf {
constexpr int TOK = 32;                      // wave rows per CTA
constexpr int M = 128;                       // accumulator rows = 4 heads x 32 tokens
constexpr int TK = 64;                       // keys per tile
constexpr int THREADS = 128;
constexpr int ROW_B = 128;                   // bytes per swizzled row (64 f16)
constexpr int Q_SUB = M * ROW_B;             // one 64-dim half of Q: 16 KB
constexpr int Q_BYTES = 2 * Q_SUB;           // 32 KB
constexpr int KV_SUB = TK * ROW_B;           // one 64-dim half of a K (or V) tile: 8 KB
constexpr int KV_TILE = 2 * KV_SUB;          // 16 KB
constexpr int STAGE = 2 * KV_TILE;           // K then V: 32 KB
constexpr int NBUF = 2;
constexpr size_t SMEM_BYTES = 1024 + Q_BYTES + NBUF * STAGE;  // + slack for 1024-byte alignment
constexpr uint32_t TMEM_COLS = 256;          // S [0,64) | O_tile [64,192) | P [192,224)
constexpr uint32_t S_COL = 0, O_COL = 64, P_COL = 192;
constexpr float QK_SCALE_LOG2 = ATTN_SCALE * LOG2E;
// instruction descriptors (kind::f16): D = f32, A = B = f16, M = 128
constexpr uint32_t IDESC_QK = (1u << 4) | ((uint32_t)(TK >> 3) << 17) | ((uint32_t)(M >> 4) << 24);          // N = 64, A and B K-major
constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(M >> 4) << 24);  // N = 128, B MN-major
}  // namespace pf

// shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// this thread's TMEM lane, 32 consecutive 32-bit columns
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
    const uint32_t n = valid ? 16u : 0u;  // 0 source bytes: destination is zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__global__ void __launch_bounds__(pf::THREADS, 2)
prefill_attn_kernel(uint16_t* __restrict__ ctx_out, const uint16_t* __restrict__ q,
                    const uint16_t* __restrict__ gate, const uint64_t* __restrict__ k_ptrs,
                    const uint64_t* __restrict__ v_ptrs, const uint32_t* __restrict__ seq_lens,
                    uint32_t rows, uint32_t window, uint32_t* __restrict__ status) {
    using namespace pf;
    extern __shared__ unsigned char smem_raw[];
    __shared__ uint64_t s_kp[TOK], s_vp[TOK];
    __shared__ uint32_t s_len[TOK];
    __shared__ __align__(8) uint64_t bar_s, bar_o;
    __shared__ uint32_t s_tmem, s_abort;

    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;  // 1024-byte aligned tiles
    const uint32_t q_s = sbase;
    const uint32_t kv_s = sbase + Q_BYTES;

    const uint32_t row0 = blockIdx.x * TOK;
    const int kvh = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int head = kvh * 4 + warp;          // this thread's query head
    const uint32_t nrows = min((uint32_t)TOK, rows - row0);

    // ---- tables of the block's rows, TMEM allocation, barriers
    if (tid < TOK) {
        uint64_t kp = 0, vp = 0;
        uint32_t sl = 0;
        if ((uint32_t)tid < nrows) {
            const uint32_t r = row0 + tid;
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
        s_kp[tid] = kp;
        s_vp[tid] = vp;
        s_len[tid] = sl;  // 0 marks a row that is skipped
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        mbar_init(&bar_s, 1);
        mbar_init(&bar_o, 1);
        s_abort = 0u;
        mbar_fence_init();
    }
    // ---- Q tile: row = head*32 + token, two 64-dim halves, 16-byte chunks swizzled by (row & 7)
    for (uint32_t i = tid; i < (uint32_t)M * 16u; i += THREADS) {
        const uint32_t r = i >> 4, c = i & 15u;
        const uint32_t hh = r >> 5, tok = r & 31u;
        const bool valid = tok < nrows;
        const uint16_t* src = q + ((size_t)(row0 + (valid ? tok : 0u)) * NQ + kvh * 4 + hh) * HD + c * 8;
        cp_async_16(q_s + (c >> 3) * Q_SUB + r * ROW_B + (((c & 7u) ^ (r & 7u)) << 4), src, valid);
    }
    cp_async_commit();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);

    float acc[HD];
#pragma unroll
    for (int d = 0; d < HD; d++) acc[d] = 0.0f;
    float m_run = -1.0e30f, l_run = 0.0f;
    uint32_t par_s = 0, par_o = 0;
    bool ok = true;

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
            // this thread's row (token = lane): valid key interval inside the run, empty if not in the run
            const bool in = (uint32_t)lane >= run0 && (uint32_t)lane < run1 && s_len[lane] != 0;
            const uint32_t rhi = in ? s_len[lane] : 0u;
            const uint32_t rlo = in ? window_start(s_len[lane], window) : 0u;
            const char* kbase = reinterpret_cast<const char*>(s_kp[run0]) + kvh * (HD * 2);
            const char* vbase = reinterpret_cast<const char*>(s_vp[run0]) + kvh * (HD * 2);
            const uint32_t ntiles = (hi - lo + TK - 1) / TK;

            auto load_tile = [&](uint32_t tile, uint32_t buf) {
                const uint32_t kbeg = lo + tile * TK;
                const uint32_t ks = kv_s + buf * STAGE, vs = ks + KV_TILE;
                for (uint32_t i = tid; i < (uint32_t)TK * 16u; i += THREADS) {
                    const uint32_t r = i >> 4, c = i & 15u;
                    const bool valid = kbeg + r < hi;
                    const size_t goff = (size_t)(valid ? kbeg + r : lo) * KV_ROW_BYTES + c * 16;
                    const uint32_t soff = (c >> 3) * KV_SUB + r * ROW_B + (((c & 7u) ^ (r & 7u)) << 4);
                    cp_async_16(ks + soff, kbase + goff, valid);
                    cp_async_16(vs + soff, vbase + goff, valid);
                }
                cp_async_commit();
            };

            load_tile(0, 0);
            for (uint32_t tile = 0; tile < ntiles; tile++) {
                const uint32_t buf = tile & 1u;
                if (tile + 1 < ntiles) {
                    load_tile(tile + 1, buf ^ 1u);
                    cp_async_wait<1>();
                } else {
                    cp_async_wait<0>();
                }
                fence_proxy_async_smem();  // cp.async-written tiles become visible to the tensor core
                tc_fence_before();
                __syncthreads();
                const uint32_t ks = kv_s + buf * STAGE, vs = ks + KV_TILE;
                if (tid == 0) {
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < 8; kk++) {  // 128 dims = 8 k-steps of 16
                        const uint64_t ad = umma_desc(q_s + (kk >> 2) * Q_SUB + (kk & 3) * 32, 16, 1024);
                        const uint64_t bd = umma_desc(ks + (kk >> 2) * KV_SUB + (kk & 3) * 32, 16, 1024);
                        umma_ss(tmem + S_COL, ad, bd, IDESC_QK, kk > 0 ? 1u : 0u);
                    }
                    umma_commit(&bar_s);
                }
                // A wait that gives up (after ~1 s; cannot happen unless the MMA never completes)
                // does not leave the loop: all threads keep the same barrier sequence, later
                // waits return at once, the status word is set and no output is written.
                ok &= mbar_wait_bounded(&bar_s, par_s, &s_abort);
                par_s ^= 1u;
                __syncwarp();
                tc_fence_after();

                // ---- this thread's S row: scale, mask, online softmax, P -> TMEM as f16
                const uint32_t kbeg = lo + tile * TK;
                uint32_t sr[2][32];
                tmem_ld32(lane_base + S_COL, sr[0]);
                tmem_ld32(lane_base + S_COL + 32, sr[1]);
                tmem_wait_ld();
                float mx = -1.0e30f;
#pragma unroll
                for (int c = 0; c < TK; c++) {
                    const uint32_t key = kbeg + c;
                    float v = __uint_as_float(sr[c >> 5][c & 31]) * QK_SCALE_LOG2;
                    v = (key >= rlo && key < rhi) ? v : -INFINITY;
                    sr[c >> 5][c & 31] = __float_as_uint(v);
                    mx = fmaxf(mx, v);
                }
                const float m_new = fmaxf(m_run, mx);
                const float corr = ex2_approx_ftz(m_run - m_new);
                m_run = m_new;
                float psum = 0.0f;
                uint32_t pk[32];
#pragma unroll
                for (int c = 0; c < TK; c += 2) {
                    const float p0 = ex2_approx_ftz(__uint_as_float(sr[c >> 5][c & 31]) - m_new);
                    const float p1 = ex2_approx_ftz(__uint_as_float(sr[(c + 1) >> 5][(c + 1) & 31]) - m_new);
                    psum += p0 + p1;
                    pk[c >> 1] = pack_h2(p0, p1);
                }
                tmem_st32(lane_base + P_COL, pk);
                tmem_wait_st();
                tc_fence_before();
                __syncthreads();
                if (tid == 0) {
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < TK / 16; kk++) {  // 64 keys = 4 k-steps of 16
                        const uint64_t bd = umma_desc(vs + kk * 16 * ROW_B, KV_SUB, 1024);
                        umma_ts(tmem + O_COL, tmem + P_COL + kk * 8, bd, IDESC_PV, kk > 0 ? 1u : 0u);
                    }
                    umma_commit(&bar_o);
                }
                // while the MMA runs: rescale the running accumulator
                l_run = l_run * corr + psum;
#pragma unroll
                for (int d = 0; d < HD; d++) acc[d] *= corr;
                ok &= mbar_wait_bounded(&bar_o, par_o, &s_abort);
                par_o ^= 1u;
                __syncwarp();
                tc_fence_after();
#pragma unroll
                for (int ch = 0; ch < 4; ch++) {
                    uint32_t orow[32];
                    tmem_ld32(lane_base + O_COL + ch * 32, orow);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i++) acc[ch * 32 + i] += __uint_as_float(orow[i]);
                }
                tc_fence_before();
            }
        }
        run0 = run1;
    }
    if (!ok && tid == 0) atomicOr(status, DEV_WAIT_TIMEOUT);

    // ---- epilogue: 1/sum, f16, gate on the f16 value (as online kernel + gate kernel)
    if ((uint32_t)lane < nrows && s_len[lane] != 0 && ok) {
        const float inv = rcp_approx_ftz(l_run);
        const size_t rh = (size_t)(row0 + lane) * NQ + head;
        const float sig = gate ? sigmoid_ref(h2f(gate[rh])) : 1.0f;
        uint4* out = reinterpret_cast<uint4*>(ctx_out + rh * HD);
#pragma unroll
        for (int v8 = 0; v8 < HD / 8; v8++) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                uint16_t h0 = f2h(__fmul_rn(acc[v8 * 8 + 2 * j], inv));
                uint16_t h1 = f2h(__fmul_rn(acc[v8 * 8 + 2 * j + 1], inv));
                if (gate) {
                    h0 = f2h(__fmul_rn(h2f(h0), sig));
                    h1 = f2h(__fmul_rn(h2f(h1), sig));
                }
                w[j] = (uint32_t)h0 | ((uint32_t)h1 << 16);
            }
            out[v8] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
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
    dim3 grid((rows + pf::TOK - 1) / pf::TOK, NKV);
    prefill_attn_kernel<<<grid, pf::THREADS, pf::SMEM_BYTES, stream>>>(
        (uint16_t*)ctx_out, (const uint16_t*)q, (const uint16_t*)gate, k_ptrs, v_ptrs, seq_lens,
        rows, window, status);
    return cudaGetLastError();
}

}  // namespace oxi
