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
// (tcgen05.st) -> O += P V (tcgen05.mma, A = P from TMEM, B = V tile from shared
// memory, MN-major, D = O accumulating in TMEM across all tiles).
// The running maximum used for the exponentials is only raised when a tile's
// maximum exceeds it by more than 2^8 (then the thread rescales its O row in
// TMEM); otherwise the stale maximum is kept, which is exact after the final
// division by the row sum and keeps O untouched between MMAs.
// S is double buffered in TMEM and P(t) is written over the first columns of S(t): QK(t+1)
// is issued before the threads start the softmax of tile t, so the tensor core computes the
// next scores while the CUDA cores work, and PV(t) follows as soon as P(t) is stored;
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
constexpr uint32_t TMEM_COLS = 256;          // S0 [0,64) | S1 [64,128) | O [128,256); P(t) overwrites the head of S(t)
constexpr uint32_t S_COL = 0, O_COL = 128;
constexpr float RESCALE_THRESHOLD = 8.0f;    // log2 units: the stale maximum may lag by a factor 256
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

// true in exactly one lane of a converged warp
__device__ __forceinline__ uint32_t elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred;
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
    const uint32_t n = valid ? 16u : 0u;  // 0 source bytes: destination is zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Orders the 32-row blocks of the wave by decreasing work (key tiles to scan) with a counting
// sort, so that the persistent CTAs of the main kernel claim the longest items first, and
// resets the claim counter.  One CTA.
__global__ void __launch_bounds__(1024)
prefill_plan_kernel(const uint32_t* __restrict__ seq_lens, uint32_t rows, uint32_t window,
                    uint32_t* __restrict__ order, uint32_t* __restrict__ counter) {
    using namespace pf;
    constexpr int NB = 1024;
    __shared__ uint32_t hist[NB];
    __shared__ uint32_t warp_tot[32];
    const uint32_t nblocks = (rows + TOK - 1) / TOK;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    hist[tid] = 0u;
    if (tid == 0) *counter = 0u;
    __syncthreads();
    auto key_of = [&](uint32_t blk) {
        uint32_t lo = 0xffffffffu, hi = 0;
        const uint32_t r1 = min(rows, (blk + 1) * TOK);
#pragma unroll 8
        for (uint32_t r = blk * TOK; r < r1; r++) {
            const uint32_t sl = seq_lens[r];
            if (sl == 0) continue;
            lo = min(lo, window_start(sl, window));
            hi = max(hi, sl);
        }
        const uint32_t tiles = hi > lo ? (hi - lo + TK - 1) / TK : 0u;
        return (uint32_t)(NB - 1) - min(tiles, (uint32_t)(NB - 1));  // bucket 0 = most work
    };
    uint32_t my_key[4];  // keys of this thread's first blocks are kept for the scatter pass
    {
        int j = 0;
        for (uint32_t blk = tid; blk < nblocks; blk += 1024, j++) {
            const uint32_t k = key_of(blk);
            if (j < 4) my_key[j] = k;
            atomicAdd(&hist[k], 1u);
        }
    }
    __syncthreads();
    // exclusive prefix sum of the 1024 buckets
    uint32_t v = hist[tid], incl = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += t;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        uint32_t w = warp_tot[lane], wi = w;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const uint32_t t = __shfl_up_sync(0xffffffffu, wi, off);
            if (lane >= off) wi += t;
        }
        warp_tot[lane] = wi - w;
    }
    __syncthreads();
    hist[tid] = warp_tot[warp] + incl - v;
    __syncthreads();
    {
        int j = 0;
        for (uint32_t blk = tid; blk < nblocks; blk += 1024, j++)
            order[atomicAdd(&hist[j < 4 ? my_key[j] : key_of(blk)], 1u)] = blk;
    }
}

__global__ void __launch_bounds__(pf::THREADS, 2)
prefill_attn_kernel(uint16_t* __restrict__ ctx_out, const uint16_t* __restrict__ q,
                    const uint16_t* __restrict__ gate, const uint64_t* __restrict__ k_ptrs,
                    const uint64_t* __restrict__ v_ptrs, const uint32_t* __restrict__ seq_lens,
                    uint32_t rows, uint32_t window, uint32_t* __restrict__ status,
                    const uint32_t* __restrict__ order, uint32_t* __restrict__ counter) {
    using namespace pf;
    extern __shared__ unsigned char smem_raw[];
    __shared__ uint64_t s_kp[TOK], s_vp[TOK];
    __shared__ uint32_t s_len[TOK];
    __shared__ __align__(8) uint64_t bar_s[2], bar_o;
    __shared__ uint32_t s_tmem, s_abort, s_item;

    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;  // 1024-byte aligned tiles
    const uint32_t q_s = sbase;
    const uint32_t kv_s = sbase + Q_BYTES;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // The MMAs are issued by one elected lane of warp 0 inside warp-uniform control flow, with
    // descriptors derived from values the compiler can prove uniform (a shuffle from lane 0):
    // issued under `if (tid == 0)` the same 12 MMAs per tile took ~1100 clocks instead of ~550.
    const int warp_u = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const uint32_t nitems = ((rows + TOK - 1) / TOK) * NKV;

    // ---- once per CTA: TMEM allocation, barriers
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        mbar_init(&bar_s[0], 1);
        mbar_init(&bar_s[1], 1);
        mbar_init(&bar_o, 1);
        s_abort = 0u;
        mbar_fence_init();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = __shfl_sync(0xffffffffu, s_tmem, 0);
    const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
    uint32_t gt = 0;      // tiles processed by this CTA so far: S buffer gt & 1, its barrier phase (gt >> 1) & 1
    uint32_t par_o = 0;
    bool ok = true;

    // per-thread constants of the tile loaders: this thread copies chunk c of rows r0, r0+8, ...
    const uint32_t ld_r0 = tid >> 4, ld_c = tid & 15u;
    const uint32_t ld_soff = (ld_c >> 3) * KV_SUB + ld_r0 * ROW_B + (((ld_c & 7u) ^ (ld_r0 & 7u)) << 4);

  // ======== persistent loop over (32-row block, KV head) items, longest first ========
  for (;;) {
    tc_fence_before();
    __syncthreads();  // the previous item's tables, Q tile and TMEM contents are no longer in use
    if (tid == 0) s_item = atomicAdd(counter, 1u);
    __syncthreads();
    const uint32_t item = s_item;
    if (item >= nitems) break;
    const uint32_t row0 = order[item >> 2] * TOK;
    const int kvh = item & 3u;
    const int head = kvh * 4 + warp;          // this thread's query head
    const uint32_t nrows = min((uint32_t)TOK, rows - row0);

    // ---- tables of the block's rows
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
    // ---- Q tile: row = head*32 + token, two 64-dim halves, 16-byte chunks swizzled by (row & 7)
    for (uint32_t i = tid; i < (uint32_t)M * 16u; i += THREADS) {
        const uint32_t r = i >> 4, c = i & 15u;
        const uint32_t hh = r >> 5, tok = r & 31u;
        const bool valid = tok < nrows;
        const uint16_t* src = q + ((size_t)(row0 + (valid ? tok : 0u)) * NQ + kvh * 4 + hh) * HD + c * 8;
        cp_async_16(q_s + (c >> 3) * Q_SUB + r * ROW_B + (((c & 7u) ^ (r & 7u)) << 4), src, valid);
    }
    cp_async_commit();
    __syncthreads();

    float m_ref = -1.0e30f, l_run = 0.0f;  // maximum used for the exponentials (may be stale), row sum
    bool o_valid = false;   // O in TMEM holds a sum (false until the CTA's first PV)
    bool pv_pending = false;  // a PV MMA has been committed to bar_o and not yet waited for

    // descriptors of the tiles at the start of each buffer; a sub-tile / k-step / stage is an
    // offset added to the 16-byte-unit start address field (no carry: shared addresses < 256 KB)
    const uint64_t q_desc = umma_desc(q_s, 16, 1024);
    const uint64_t k_desc0 = umma_desc(kv_s, 16, 1024);                // K tiles: K-major
    const uint64_t v_desc0 = umma_desc(kv_s + KV_TILE, KV_SUB, 1024);  // V tiles: MN-major
    auto issue_qk = [&](uint32_t stage, uint32_t sbuf) {  // whole warp 0; S[sbuf] = Q K^T, 128 dims = 8 k-steps of 16
        const uint64_t kd = k_desc0 + (uint64_t)(stage * (STAGE >> 4));
        if (elect_one()) {
#pragma unroll
            for (int kk = 0; kk < 8; kk++) {
                const uint32_t qoff = (uint32_t)(((kk >> 2) * Q_SUB + (kk & 3) * 32) >> 4);
                const uint32_t koff = (uint32_t)(((kk >> 2) * KV_SUB + (kk & 3) * 32) >> 4);
                umma_ss(tmem + S_COL + sbuf * TK, q_desc + qoff, kd + koff, IDESC_QK, kk > 0 ? 1u : 0u);
            }
            umma_commit(&bar_s[sbuf]);
        }
        __syncwarp();
    };

    // ---- runs of rows that share one cache
    uint32_t run0 = 0;
    while (run0 < nrows) {
        uint32_t run1 = run0 + 1;
        while (run1 < nrows && s_kp[run1] == s_kp[run0] && s_vp[run1] == s_vp[run0]) run1++;
        uint32_t lo = 0xffffffffu, hi = 0, lo_max = 0, hi_min = 0xffffffffu;
        bool full_run = (run1 - run0 == (uint32_t)TOK);  // every row of the M tile belongs to the run
        for (uint32_t i = run0; i < run1; i++) {
            const uint32_t sl = s_len[i];
            if (sl == 0) { full_run = false; continue; }
            lo = min(lo, window_start(sl, window));
            hi = max(hi, sl);
            lo_max = max(lo_max, window_start(sl, window));
            hi_min = min(hi_min, sl);
        }
        if (hi > lo) {
            // this thread's row (token = lane): valid key interval inside the run, empty if not in the run
            const bool in = (uint32_t)lane >= run0 && (uint32_t)lane < run1 && s_len[lane] != 0;
            const uint32_t rhi = in ? s_len[lane] : 0u;
            const uint32_t rlo = in ? window_start(s_len[lane], window) : 0u;
            const char* kbase = reinterpret_cast<const char*>(s_kp[run0]) + kvh * (HD * 2);
            const char* vbase = reinterpret_cast<const char*>(s_vp[run0]) + kvh * (HD * 2);
            const uint32_t ntiles = (hi - lo + TK - 1) / TK;

            // K and V tiles have separate double buffers and separate cp.async groups: K(t+2) is
            // requested when QK(t) has completed, V(t+1) when PV(t-1) has completed, so every load
            // has a whole iteration to land.  One group is committed per call (possibly empty) so
            // that wait_group counts stay uniform.
            auto load_half = [&](uint32_t tile, uint32_t dst, const char* base) {
                if (tile < ntiles) {
                    const uint32_t kbeg = lo + tile * TK;
                    const char* src = base + (size_t)(kbeg + ld_r0) * KV_ROW_BYTES + ld_c * 16;
                    const uint32_t d = dst + ld_soff;
                    if (kbeg + TK <= hi) {
#pragma unroll
                        for (int k = 0; k < TK / 8; k++)  // rows r0 + 8k: same swizzle phase, fixed strides
                            cp_async_16(d + k * 8 * ROW_B, src + (size_t)k * 8 * KV_ROW_BYTES, true);
                    } else {
#pragma unroll
                        for (int k = 0; k < TK / 8; k++) {
                            const bool valid = kbeg + ld_r0 + 8 * k < hi;
                            cp_async_16(d + k * 8 * ROW_B, valid ? src + (size_t)k * 8 * KV_ROW_BYTES : base, valid);
                        }
                    }
                }
                cp_async_commit();
            };
            auto k_buf = [&](uint32_t tile) { return kv_s + (tile & 1u) * STAGE; };
            auto v_buf = [&](uint32_t tile) { return kv_s + (tile & 1u) * STAGE + KV_TILE; };

            // The previous run's last PV may still be reading its V tile and P.
            if (pv_pending) {
                ok &= mbar_wait_bounded(&bar_o, par_o, &s_abort);
                par_o ^= 1u;
                pv_pending = false;
                __syncwarp();
                tc_fence_after();
            }
            // prologue of the run: K(0), V(0), K(1) requested; S(0) issued as soon as K(0) landed
            load_half(0, k_buf(0), kbase);
            load_half(0, v_buf(0), vbase);
            load_half(1, k_buf(1), kbase);
            cp_async_wait<0>();
            fence_proxy_async_smem();  // cp.async-written tiles become visible to the tensor core
            tc_fence_before();
            __syncthreads();
            if (warp_u == 0) {
                tc_fence_after();
                issue_qk(0u, gt & 1u);
            }

            for (uint32_t tile = 0; tile < ntiles; tile++) {
                // A wait that gives up (after ~1 s; cannot happen unless an MMA never completes)
                // does not leave the loop: all threads keep the same barrier sequence, later
                // waits return at once, the status word is set and no output is written.
                const uint32_t sbuf = gt & 1u;
                ok &= mbar_wait_bounded(&bar_s[sbuf], (gt >> 1) & 1u, &s_abort);
                __syncwarp();
                tc_fence_after();
                load_half(tile + 2, k_buf(tile), kbase);  // QK(tile) is done with its K buffer
                // K(tile+1) (requested one iteration ago) must have landed: QK(tile+1) is issued now, into
                // the other S buffer, so that it runs while the threads do the softmax of this tile
                cp_async_wait<2>();
                fence_proxy_async_smem();
                tc_fence_before();
                __syncthreads();
                if (warp_u == 0 && tile + 1 < ntiles) {
                    tc_fence_after();
                    issue_qk((tile + 1) & 1u, sbuf ^ 1u);
                }

                // ---- this thread's S row: scale, mask, softmax weights against the reference maximum
                const uint32_t kbeg = lo + tile * TK;
                uint32_t sr[2][32];
                tmem_ld32(lane_base + S_COL + sbuf * TK, sr[0]);
                tmem_ld32(lane_base + S_COL + sbuf * TK + 32, sr[1]);
                tmem_wait_ld();
                // Interior tiles (every key valid for every row of the M tile) skip the masks.
                const bool interior = full_run && kbeg >= lo_max && kbeg + TK <= hi_min;
                // four independent accumulators keep the max / sum dependency chains short (one warp
                // per scheduler per CTA: latency, not issue bandwidth, is what limits this loop)
                float mxa[4] = {-1.0e30f, -1.0e30f, -1.0e30f, -1.0e30f};
                if (interior) {
#pragma unroll
                    for (int c = 0; c < TK; c++) mxa[c & 3] = fmaxf(mxa[c & 3], __uint_as_float(sr[c >> 5][c & 31]));
                } else {
#pragma unroll
                    for (int c = 0; c < TK; c++) {
                        const uint32_t key = kbeg + c;
                        float v = __uint_as_float(sr[c >> 5][c & 31]);
                        v = (key >= rlo && key < rhi) ? v : -INFINITY;
                        sr[c >> 5][c & 31] = __float_as_uint(v);
                        mxa[c & 3] = fmaxf(mxa[c & 3], v);
                    }
                }
                float mx = fmaxf(fmaxf(mxa[0], mxa[1]), fmaxf(mxa[2], mxa[3]));
                mx = mx > -1.0e29f ? mx * QK_SCALE_LOG2 : -1.0e30f;  // stays -1e30 when the whole row is masked
                const bool raise = mx > m_ref + RESCALE_THRESHOLD;
                const float corr = raise ? ex2_approx_ftz(m_ref - mx) : 1.0f;
                if (raise) m_ref = mx;
                float psa[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                uint32_t pk[32];
                const float neg_m = -m_ref;
#pragma unroll
                for (int c = 0; c < TK; c += 2) {  // p = 2^(s*scale*log2e - m): one fma + one ex2 per key
                    const float p0 = ex2_approx_ftz(fmaf(__uint_as_float(sr[c >> 5][c & 31]), QK_SCALE_LOG2, neg_m));
                    const float p1 = ex2_approx_ftz(fmaf(__uint_as_float(sr[(c + 1) >> 5][(c + 1) & 31]), QK_SCALE_LOG2, neg_m));
                    psa[(c >> 1) & 3] += p0 + p1;
                    pk[c >> 1] = pack_h2(p0, p1);
                }
                const float psum = (psa[0] + psa[1]) + (psa[2] + psa[3]);
                l_run = l_run * corr + psum;

                // ---- PV(tile-1) must be complete before P is overwritten and before O is rescaled;
                // its V stage is then free for tile+1 (tile 1 of a run was loaded in the prologue)
                if (pv_pending) {
                    ok &= mbar_wait_bounded(&bar_o, par_o, &s_abort);
                    par_o ^= 1u;
                    pv_pending = false;
                    __syncwarp();
                    tc_fence_after();
                }
                load_half(tile + 1, v_buf(tile + 1), vbase);  // PV(tile-1) is done with that V buffer
                if (o_valid && __any_sync(0xffffffffu, raise)) {
                    // rare: the reference maximum of some row of this warp moved; rescale the warp's O rows
#pragma unroll
                    for (int ch = 0; ch < 4; ch++) {
                        uint32_t orow[32];
                        tmem_ld32(lane_base + O_COL + ch * 32, orow);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; i++) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * corr);
                        tmem_st32(lane_base + O_COL + ch * 32, orow);
                    }
                }
                tmem_st32(lane_base + S_COL + sbuf * TK, pk);  // P(tile) over the head of S(tile)
                tmem_wait_st();
                // V(tile) must have landed before PV(tile); the two groups requested in this
                // iteration may still be in flight
                cp_async_wait<2>();
                fence_proxy_async_smem();
                tc_fence_before();
                __syncthreads();
                if (warp_u == 0) {
                    tc_fence_after();
                    const uint64_t vd = v_desc0 + (uint64_t)((tile & 1u) * (STAGE >> 4));
                    if (elect_one()) {
#pragma unroll
                        for (int kk = 0; kk < TK / 16; kk++)  // 64 keys = 4 k-steps of 16
                            umma_ts(tmem + O_COL, tmem + S_COL + sbuf * TK + kk * 8,
                                    vd + (uint32_t)((kk * 16 * ROW_B) >> 4), IDESC_PV, (kk > 0 || o_valid) ? 1u : 0u);
                        umma_commit(&bar_o);
                    }
                    __syncwarp();
                }
                o_valid = true;
                pv_pending = true;
                ++gt;
            }
        }
        run0 = run1;
    }
    if (pv_pending) {
        ok &= mbar_wait_bounded(&bar_o, par_o, &s_abort);
        par_o ^= 1u;
        pv_pending = false;
        __syncwarp();
        tc_fence_after();
    }

    // ---- epilogue: O row from TMEM, 1/sum, f16, gate on the f16 value (as online kernel + gate kernel)
    {
        const bool write = (uint32_t)lane < nrows && s_len[lane] != 0 && ok && o_valid;
        const float inv = rcp_approx_ftz(l_run);
        const size_t rh = (size_t)(row0 + (write ? lane : 0)) * NQ + head;
        const float sig = (gate && write) ? sigmoid_ref(h2f(gate[rh])) : 1.0f;
        uint4* out = reinterpret_cast<uint4*>(ctx_out + rh * HD);
        if (o_valid) {
#pragma unroll
            for (int ch = 0; ch < 4; ch++) {
                uint32_t orow[32];
                tmem_ld32(lane_base + O_COL + ch * 32, orow);
                tmem_wait_ld();
                if (write) {
#pragma unroll
                    for (int v8 = 0; v8 < 4; v8++) {
                        uint32_t w[4];
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            uint16_t h0 = f2h(__fmul_rn(__uint_as_float(orow[v8 * 8 + 2 * j]), inv));
                            uint16_t h1 = f2h(__fmul_rn(__uint_as_float(orow[v8 * 8 + 2 * j + 1]), inv));
                            if (gate) {
                                h0 = f2h(__fmul_rn(h2f(h0), sig));
                                h1 = f2h(__fmul_rn(h2f(h1), sig));
                            }
                            w[j] = (uint32_t)h0 | ((uint32_t)h1 << 16);
                        }
                        out[ch * 4 + v8] = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    }
  }  // item loop
    if (!ok && tid == 0) atomicOr(status, DEV_WAIT_TIMEOUT);
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
                                uint32_t* status, int num_sms, uint32_t* order, uint32_t* counter) {
    const uint32_t nitems = ((rows + pf::TOK - 1) / pf::TOK) * NKV;
    prefill_plan_kernel<<<1, 1024, 0, stream>>>(seq_lens, rows, window, order, counter);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const uint32_t grid = nitems < (uint32_t)(2 * num_sms) ? nitems : (uint32_t)(2 * num_sms);
    prefill_attn_kernel<<<grid, pf::THREADS, pf::SMEM_BYTES, stream>>>(
        (uint16_t*)ctx_out, (const uint16_t*)q, (const uint16_t*)gate, k_ptrs, v_ptrs, seq_lens,
        rows, window, status, order, counter);
    return cudaGetLastError();
}

}  // namespace oxi
