// Chunked-prefill causal GQA attention with the sigmoid gate over per-row
// pointer tables, as one fused flash-attention kernel on the 5th-generation
// tensor cores: tcgen05.mma with accumulators, weights and the query tile in
// tensor memory (TMEM).  Scores and weights stay on chip.
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
// Work item = 64 consecutive wave rows (tokens) and one KV head, processed by one
// persistent CTA per SM as TWO M = 128 query tiles (tokens 0-31 and 32-63; a tile is
// (4 query heads of the group) x (32 tokens), row = head*32 + token) that share every
// K/V tile brought into shared memory.  Warp roles:
//   warps 0-3   softmax of query tile 0: warp w / lane l owns accumulator row (head w,
//               token l) = TMEM lane 32*w + l, so the softmax is thread-local, no shuffles
//   warps 4-7   softmax of query tile 1 (same TMEM lanes, other columns)
//   warp 8 / 11 issue the tcgen05.mma of query tile 0 / 1 (one elected lane, warp-uniform
//               control flow), alternating strictly by a token so that bursts never interleave
//   warp 9 / 10 K / V tile loaders: cp.async 16-byte chunks written straight into the
//               128-byte-swizzled layout (zero-filled past the run's last key), a ring of
//               4 stages each, 3 tiles in flight
// all connected by mbarriers only (no CTA-wide barrier inside an item).
//
// Per 64-key tile and query tile j:  S_j = Q_j K^T  (B = K tile from shared memory, K-major,
// D = S_j in TMEM; A = Q_0 from TMEM for tile 0, Q_1 from shared memory for tile 1, which does
// not fit into TMEM) -> each softmax thread loads its S row (tcgen05.ld) and at once hands S_j
// back, applies scale, causal/window mask and the online-softmax update, writes P as f16 to
// its own TMEM columns (tcgen05.st) -> O_j += P_j V  (A = P_j from TMEM, B = V tile from shared
// memory, MN-major, D = O_j accumulating in TMEM across all tiles).
// Scores run one tile ahead of the softmax: MMA warp j's step t is the burst PV_j(t-2), QK_j(t),
// and QK_j(t) only needs S_j(t-1) to have been read into registers.  In steady state the softmax
// warps therefore find their next scores ready, and the two query tiles keep the tensor pipe and
// the special-function units busy at the same time.
// The running maximum used for the exponentials is only raised when a tile's
// maximum exceeds it by more than 2^8 (then the thread rescales its O row in
// TMEM); otherwise the stale maximum is kept, which is exact after the final
// division by the row sum and keeps O untouched between MMAs.
//
// TMEM (all 512 columns, one CTA per SM): Q_0 (64: 128 dims as f16 pairs) | S_0 S_1 (64 each) |
// P_0 P_1 (32 each) | O_0 O_1 (128 each).
//
// Rows of a 64-row block that point at different caches are processed as
// separate runs of equal pointers (rows outside the run are masked), so any
// table contents are legal; the engine's waves (consecutive positions of one
// request per chunk) give one run per block except where a chunk boundary falls
// inside a block.
//
// Every wait is bounded (about one second); a wait that gives up sets a CTA-wide flag that
// makes every later wait return at once, the kernel then finishes its control flow without
// writing output and reports OXI_DEV_WAIT_TIMEOUT in the status word.
#include "common.cuh"
#include "kernels.h"
#include "tc5.cuh"

namespace oxi {

namespace pf {
constexpr int TOK = 32;                      // wave rows per query tile
constexpr int BLK = 64;                      // wave rows per work item (two query tiles)
constexpr int M = 128;                       // accumulator rows = 4 heads x 32 tokens
constexpr int TK = 64;                       // keys per tile
constexpr int THREADS = 384;                 // 8 softmax warps, 2 MMA warps, K loader, V loader
constexpr int W_MMA0 = 8, W_KLOAD = 9, W_VLOAD = 10, W_MMA1 = 11;
constexpr int ROW_B = 128;                   // bytes per swizzled row (64 f16)
constexpr int KV_SUB = TK * ROW_B;           // one 64-dim half of a K (or V) tile: 8 KB
constexpr int KV_TILE = 2 * KV_SUB;          // 16 KB
constexpr int NS = 4;                        // ring stages, for K and for V
constexpr int DEPTH = 3;                     // tiles a loader keeps in flight
constexpr int Q_SUB = M * ROW_B;             // one 64-dim half of a query tile in shared memory: 16 KB
constexpr int Q_BYTES = 2 * Q_SUB;           // 32 KB
constexpr size_t SMEM_BYTES = 1024 + Q_BYTES + 2 * NS * KV_TILE;  // + slack for 1024-byte alignment; > half an SM: one CTA per SM
constexpr uint32_t TMEM_COLS = 512;
// Q_0 (64) | S_0 S_1 (64 each) | P_0 P_1 (32 each) | O_0 O_1 (128 each); Q_1 does not fit and stays in shared memory
constexpr uint32_t Q0_COL = 0, S_COL = 64, P_COL = 192, O_COL = 256;  // S + j*64, P + j*32, O + j*128 for query tile j
constexpr float RESCALE_THRESHOLD = 8.0f;    // log2 units: the stale maximum may lag by a factor 256
constexpr float QK_SCALE_LOG2 = ATTN_SCALE * LOG2E;
// instruction descriptors (kind::f16): D = f32, A = B = f16, M = 128
constexpr uint32_t IDESC_QK = (1u << 4) | ((uint32_t)(TK >> 3) << 17) | ((uint32_t)(M >> 4) << 24);          // N = 64, A and B K-major
constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(M >> 4) << 24);  // N = 128, B MN-major
}  // namespace pf

// Key-range split of long blocks (off when part_tiles == 0), for waves with fewer (block, KV head)
// items than the GPU has SMs.  The plan kernel picks the smallest part size P >= part_tiles (in
// 64-key tiles) for which the wave has at most target_items items: a block that scans more than P
// tiles becomes ns = ceil(tiles / P) <= 32 work units, each with its own partial result
// (unnormalised O, reference maximum, row sum per accumulator row) in a slot of the partial
// workspace, merged by prefill_merge_kernel.  One round of near-equal items keeps the partial
// traffic low.  A wave whose split blocks need more slots than the workspace has runs unsplit.
constexpr int PF_MAX_SPLIT = 32;
struct PfSplit {
    uint32_t* units;      // [units] block | part << 16 | ns << 24, longest unit first
    uint32_t* slots;      // [units] partial slot of the unit (blocks with ns > 1 only)
    uint32_t* blkmeta;    // [blocks] ns | first slot << 8
    float* part_o;        // [slot][kv head][query tile][128 rows][128] f32
    float* part_ml;       // [slot][kv head][query tile][128 rows][2] f32
    uint32_t part_tiles;    // smallest part, in tiles; 0: no split
    uint32_t max_slots;     // slots of part_o / part_ml
    uint32_t target_items;  // items the wave should not exceed (the SM count)
};

// Orders the 64-row blocks of the wave by decreasing work (key tiles to scan) with a counting
// sort, so that the persistent CTAs of the main kernel claim the longest items first, and
// resets the claim counter.  One CTA.
__global__ void __launch_bounds__(1024)
prefill_plan_kernel(const uint32_t* __restrict__ seq_lens, uint32_t rows, uint32_t window,
                    uint32_t* __restrict__ order, uint32_t* __restrict__ counter) {
    using namespace pf;
    constexpr int NB = 1024;
    __shared__ uint32_t hist[NB];
    __shared__ uint32_t warp_tot[32];
    const uint32_t nblocks = (rows + BLK - 1) / BLK;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    hist[tid] = 0u;
    if (tid == 0) *counter = 0u;
    __syncthreads();
    auto key_of = [&](uint32_t blk) {
        uint32_t lo = 0xffffffffu, hi = 0;
        const uint32_t r1 = min(rows, (blk + 1) * BLK);
#pragma unroll 8
        for (uint32_t r = blk * BLK; r < r1; r++) {
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

// The same order for waves of at most 1024 blocks (65,536 rows), the usual case, in a few
// microseconds: the rows are read once, coalesced, block extents are formed with shared-memory
// atomics, and every block finds its rank by counting the blocks with more work.  Lets the
// attention kernel, launched as a programmatic dependent, run its prologue meanwhile.
__global__ void __launch_bounds__(1024)
prefill_plan_small_kernel(const uint32_t* __restrict__ seq_lens, uint32_t rows, uint32_t window,
                          uint32_t* __restrict__ order, uint32_t* __restrict__ counter, const PfSplit sp) {
    using namespace pf;
    __shared__ uint32_t s_lo[1024], s_hi[1024], s_key[1024], s_ns[1024];
    __shared__ uint32_t s_slots, s_part;
    const uint32_t nblocks = (rows + BLK - 1) / BLK;
    const uint32_t tid = threadIdx.x;
    pdl_launch_dependents();
    s_lo[tid] = 0xffffffffu;
    s_hi[tid] = 0u;
    if (tid == 0) s_slots = 0u;
    __syncthreads();
    for (uint32_t r = tid; r < rows; r += 1024) {
        const uint32_t sl = seq_lens[r];
        if (sl != 0u) {
            atomicMin(&s_lo[r / BLK], window_start(sl, window));
            atomicMax(&s_hi[r / BLK], sl);
        }
    }
    __syncthreads();
    // key = key tiles one work unit scans (the union of the block's rows, as in the general kernel)
    uint32_t key = 0, ns = 1;
    if (tid < nblocks) {
        const uint32_t lo = s_lo[tid], hi = s_hi[tid];
        key = hi > lo ? (hi - lo + TK - 1) / TK : 0u;
    }
    if (sp.part_tiles != 0u) {
        // Part size: the smallest P >= part_tiles with sum_b ceil(tiles_b / P) * 4 <= target_items and
        // at most 32 parts per block, by bisection in warp 0 (a split wave has at most 64 blocks).
        if (tid < 32) {
            const uint32_t t0 = key;  // tiles of block tid and of block tid + 32
            uint32_t tb = 0u;
            if (tid + 32 < nblocks) {
                const uint32_t lo2 = s_lo[tid + 32], hi2 = s_hi[tid + 32];
                tb = hi2 > lo2 ? (hi2 - lo2 + TK - 1) / TK : 0u;
            }
            uint32_t tmax = max(t0, tb);
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) tmax = max(tmax, __shfl_xor_sync(0xffffffffu, tmax, off));
            auto items_at = [&](uint32_t P) {
                uint32_t n = (t0 + P - 1) / P + (tb + P - 1) / P;
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) n += __shfl_xor_sync(0xffffffffu, n, off);
                return n * NKV;
            };
            uint32_t lo = max(sp.part_tiles, (tmax + PF_MAX_SPLIT - 1) / PF_MAX_SPLIT), hi = max(lo, tmax);
            while (lo < hi) {  // items_at is non-increasing in P; items_at(hi) <= blocks * 4 <= target_items
                const uint32_t mid = (lo + hi) / 2;
                if (items_at(mid) <= sp.target_items) hi = mid; else lo = mid + 1;
            }
            if (tid == 0) s_part = max(lo, 1u);
        }
        __syncthreads();
        if (tid < nblocks && key > s_part) {
            ns = (key + s_part - 1) / s_part;
            atomicAdd(&s_slots, ns);
        }
    }
    __syncthreads();
    if (tid < nblocks) {
        if (s_slots > sp.max_slots) ns = 1;  // not enough partial slots: the wave runs unsplit
        key = (key + ns - 1) / ns;
        s_key[tid] = key;
        s_ns[tid] = ns;
    }
    __syncthreads();
    uint32_t rank = 0, slot = 0, total = 0;
    if (tid < nblocks) {
        for (uint32_t j = 0; j < nblocks; j++) {
            const uint32_t kj = s_key[j], nj = s_ns[j];
            rank += (kj > key || (kj == key && j < tid)) ? nj : 0u;
            slot += (j < tid && nj > 1u) ? nj : 0u;
            total += nj;
        }
    }
    // Launched as a programmatic dependent itself: everything above only read seq_lens (a step input)
    // and overlapped the kernel before (the wave's append, or the previous layer's attention, which may
    // still be claiming items through `order` and `counter`); the outputs are written after it finished.
    pdl_wait();
    if (tid == 0) {
        counter[0] = 0u;
        counter[1] = total;  // work units (x 4 KV heads = items)
    }
    if (tid < nblocks) {
        if (sp.part_tiles == 0u) {
            order[rank] = tid;
        } else {
            for (uint32_t i = 0; i < ns; i++) {
                sp.units[rank + i] = tid | (i << 16) | (ns << 24);
                sp.slots[rank + i] = slot + i;
            }
            sp.blkmeta[tid] = ns | (slot << 8);
        }
    }
}

// A run of consecutive block rows that share one cache, with the union of their key intervals.
struct PfRun {
    uint32_t r0, r1, lo, hi;
};

// Takes the next run of the block's run list (built once per item by warp 0, see the kernel)
// that has keys to scan.  Every warp role walks the same list, so all see the same sequence
// of runs and tiles.
__device__ __forceinline__ bool pf_next_run(uint32_t& next, uint32_t nruns, const uint32_t (*s_runs)[4], PfRun& run) {
    while (next < nruns) {
        const uint4 r = *reinterpret_cast<const uint4*>(s_runs[next++]);
        if (r.w > r.z) {
            run.r0 = r.x;
            run.r1 = r.y;
            run.lo = r.z;
            run.hi = r.w;
            return true;
        }
    }
    return false;
}

// kFault (test support only) compiles in the hooks of oxi_debug_arm_wait_fault: a wait limit taken from the
// launch, a K tile of CTA 0 that is never published, and the propagation of a give-up to the roles whose own
// waits passed (the MMA warps withhold "O is final", the CTA claims nothing more).  The production
// instantiations carry none of it: the loop is sensitive to a few instructions in its waits and hand-overs
// (measured 3-5 % on the 4,096-row wave), and there a wait only runs out after an internal error, which the
// status word reports.
template <bool kPaged, bool kSplit, bool kTma, bool kFault>
__global__ void __launch_bounds__(pf::THREADS, 1)
prefill_attn_kernel(uint16_t* __restrict__ ctx_out, const uint16_t* __restrict__ q,
                    const uint16_t* __restrict__ gate, const uint64_t* __restrict__ k_ptrs,
                    const uint64_t* __restrict__ v_ptrs, const uint32_t* __restrict__ seq_lens,
                    uint32_t rows, uint32_t window, uint32_t* __restrict__ status,
                    const uint32_t* __restrict__ order, uint32_t* __restrict__ counter,
                    const PagedMap pm, const uint32_t* __restrict__ row_seq, const PfSplit sp,
                    const __grid_constant__ TmaDesc tmap, const uint64_t slab_base, const uint32_t slab_rows,
                    const WaitFault fault) {
    using namespace pf;
    const uint32_t wait_us = kFault ? fault.limit_us : WAIT_LIMIT_US;
    // paged K/V: k_ptrs / v_ptrs are unused, wave row r reads row row_seq[r] of pm.block_tables
    constexpr bool paged = kPaged;
    extern __shared__ unsigned char smem_raw[];
    // per-item tables, double buffered: the K loader prepares the next item's while the current one finishes
    __shared__ uint64_t s_kp[2][BLK], s_vp[2][BLK];
    __shared__ uint32_t s_len[2][BLK];
    __shared__ __align__(16) uint32_t s_runs[2][BLK][4];  // runs of equal pointers: first row, end row, first key, end key
    __shared__ uint32_t s_nruns[2];
    __shared__ uint32_t s_tile[2][2][3];  // per query tile: largest window start, smallest length, all 32 rows valid
    // loaders -> MMA warps (32 arrivals) and back (one tcgen05.commit from each MMA warp)
    __shared__ __align__(8) uint64_t bar_kfull[NS], bar_kempty[NS], bar_vfull[NS], bar_vempty[NS];
    // per query tile: S ready (commit), S read into registers (128 arrivals), P stored (128 arrivals),
    // PV of a tile complete (commit), Q stored (128 arrivals), O final (commit)
    __shared__ __align__(8) uint64_t bar_sfull[2], bar_sfree[2], bar_pfull[2], bar_pvdone[2], bar_qfull[2], bar_ofull[2];
    __shared__ __align__(8) uint64_t bar_tok[2];  // issue token of MMA warp j
    __shared__ uint32_t s_tmem, s_abort, s_item[2], s_unit[2];

    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;  // 1024-byte aligned tiles
    const uint32_t q1_s = sbase, k_s = sbase + Q_BYTES, v_s = k_s + NS * KV_TILE;
    const int tid = threadIdx.x, lane = tid & 31;
    // warp index the compiler can prove uniform: role branches and MMA issue stay in uniform control flow
    const int warp_u = __shfl_sync(0xffffffffu, tid >> 5, 0);

    // ---- once per CTA: TMEM allocation (all 512 columns; one CTA per SM), barriers
    if (warp_u == W_MMA0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        for (int s = 0; s < NS; s++) {
            mbar_init(&bar_kfull[s], 32);
            mbar_init(&bar_vfull[s], 32);
            mbar_init(&bar_kempty[s], 2);  // one commit from each MMA warp
            mbar_init(&bar_vempty[s], 2);
        }
        for (int j = 0; j < 2; j++) {
            mbar_init(&bar_sfull[j], 1);
            mbar_init(&bar_sfree[j], M);
            mbar_init(&bar_pfull[j], M);
            mbar_init(&bar_pvdone[j], 1);
            mbar_init(&bar_qfull[j], M);
            mbar_init(&bar_ofull[j], 1);
            mbar_init(&bar_tok[j], 1);
        }
        s_abort = 0u;
        mbar_fence_init();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = __shfl_sync(0xffffffffu, s_tmem, 0);
    pdl_wait();  // the plan kernel's order and counter (and everything before it in the stream) are visible from here on
    const uint32_t nitems = (kSplit ? counter[1] : (rows + BLK - 1) / BLK) * NKV;

    // Every role counts the same sequence of K/V tiles: tile gk uses ring stage gk % NS in its
    // (gk / NS)-th use and phase gk & 1 of the per-tile barriers.
    uint32_t gk = 0;
    uint32_t n_o = 0;  // items of this CTA that had tiles (phase of bar_ofull)
    uint32_t n_burst = 0;  // MMA warps: bursts issued so far (phase of bar_tok)
    bool ok = true;

    // Claims the next item and prepares its tables in buffer `buf`; run by all lanes of the K loader warp
    // while the other roles finish the current item (before the loop for the first item).
    auto prepare_item = [&](uint32_t buf) {
        uint32_t item = 0xffffffffu;  // kFault: a CTA one of whose waits gave up claims nothing more, the others take its share
        if (lane == 0 && (!kFault || *const_cast<volatile uint32_t*>(&s_abort) == 0u)) item = atomicAdd(counter, 1u);
        item = __shfl_sync(0xffffffffu, item, 0);
        if (lane == 0) s_item[buf] = item;
        if (item >= nitems) return;
        const uint32_t ud = kSplit ? sp.units[item >> 2] : order[item >> 2];
        if (lane == 0) s_unit[buf] = ud;
        const uint32_t row0 = (kSplit ? (ud & 0xffffu) : ud) * BLK;
        const int kvh = item & 3u;
        const uint32_t nrows = min((uint32_t)BLK, rows - row0);
    // ---- tables of the block's rows and the list of runs, by one warp (lane l: rows l and l + 32).
    // A run is a maximal range of consecutive rows that share one cache (equal pointers); its key
    // interval is the union of its rows' intervals.
        uint64_t kp[2], vp[2];
        uint32_t sl[2], ws[2];
#pragma unroll
        for (int hf = 0; hf < 2; hf++) {
            const uint32_t rr = (uint32_t)lane + 32u * hf;
            kp[hf] = vp[hf] = 0;
            sl[hf] = 0;
            if (rr < nrows) {
                const uint32_t r = row0 + rr;
                sl[hf] = seq_lens[r];
                bool too_long = false;
                if (paged) {
                    // the run logic below only compares these two words: (table row + 1) * 16 keeps rows of one
                    // sequence equal, non-zero and "aligned"
                    kp[hf] = vp[hf] = ((uint64_t)row_seq[r] + 1ull) << 4;
                    too_long = sl[hf] != 0u && ((sl[hf] - 1u) >> pm.lbs) >= pm.max_blocks;  // more blocks than the table has columns
                } else {
                    kp[hf] = k_ptrs[r];
                    vp[hf] = v_ptrs[r];
                }
                if (((kp[hf] | vp[hf]) & 15ull) != 0ull) {
                    if (kvh == 0) atomicOr(status, DEV_MISALIGNED_PTR);
                    sl[hf] = 0;
                } else if (sl[hf] == 0u || too_long) {
                    if (kvh == 0) atomicOr(status, DEV_BAD_SEQ_LEN);
                    sl[hf] = 0;
                }
            }
            ws[hf] = sl[hf] ? window_start(sl[hf], window) : 0u;
            s_kp[buf][rr] = kp[hf];
            s_vp[buf][rr] = vp[hf];
            s_len[buf][rr] = sl[hf];  // 0 marks a row that is skipped
            s_runs[buf][rr][0] = 0u;
            s_runs[buf][rr][1] = 0u;
            s_runs[buf][rr][2] = 0xffffffffu;
            s_runs[buf][rr][3] = 0u;
        }
        // a row starts a run when its pointers differ from the row before
        uint32_t mask[2];
#pragma unroll
        for (int hf = 0; hf < 2; hf++) {
            uint64_t pk = __shfl_up_sync(0xffffffffu, kp[hf], 1), pv = __shfl_up_sync(0xffffffffu, vp[hf], 1);
            const uint64_t k31 = __shfl_sync(0xffffffffu, kp[0], 31), v31 = __shfl_sync(0xffffffffu, vp[0], 31);
            if (lane == 0) {
                pk = k31;
                pv = v31;
            }
            const uint32_t rr = (uint32_t)lane + 32u * hf;
            const bool start = rr < nrows && (rr == 0u || kp[hf] != pk || vp[hf] != pv);
            mask[hf] = __ballot_sync(0xffffffffu, start);
        }
        __syncwarp();
        const uint64_t starts = (uint64_t)mask[0] | ((uint64_t)mask[1] << 32);
#pragma unroll
        for (int hf = 0; hf < 2; hf++) {
            const uint32_t rr = (uint32_t)lane + 32u * hf;
            if (rr < nrows) {
                const uint32_t id = (uint32_t)__popcll(starts & (~0ull >> (63u - rr))) - 1u;  // runs that start at or before rr
                if (sl[hf] != 0u) {
                    atomicMin(&s_runs[buf][id][2], ws[hf]);
                    atomicMax(&s_runs[buf][id][3], sl[hf]);
                }
                if ((starts >> rr) & 1ull) {
                    const uint64_t later = rr < 63u ? starts >> (rr + 1u) : 0ull;
                    s_runs[buf][id][0] = rr;
                    s_runs[buf][id][1] = later ? rr + (uint32_t)__ffsll((long long)later) : nrows;
                }
            }
            // mask-free tiles of query tile hf need every one of its 32 rows: their common key range
            const bool all = __all_sync(0xffffffffu, sl[hf] != 0u);
            const uint32_t lo_max = __reduce_max_sync(0xffffffffu, ws[hf]);
            const uint32_t hi_min = __reduce_min_sync(0xffffffffu, sl[hf]);
            if (lane == 0) {
                s_tile[buf][hf][0] = lo_max;
                s_tile[buf][hf][1] = hi_min;
                s_tile[buf][hf][2] = all ? 1u : 0u;
            }
        }
        if (lane == 0) s_nruns[buf] = (uint32_t)__popcll(starts);
    };
    if (warp_u == W_KLOAD) prepare_item(0u);

  // ======== persistent loop over (64-row block, KV head) items, longest first ========
  for (uint32_t it = 0;; ++it) {
    // every role is done with the previous item; this item's tables (written by the K loader) are visible
    __syncthreads();
    const uint32_t buf = it & 1u;
    const uint32_t item = s_item[buf];
    if (item >= nitems) break;
    const uint64_t* const c_kp = s_kp[buf];
    const uint64_t* const c_vp = s_vp[buf];
    const uint32_t* const c_len = s_len[buf];
    const uint32_t (*const c_runs)[4] = s_runs[buf];
    const uint32_t (*const c_tile)[3] = s_tile[buf];
    const uint32_t nruns = s_nruns[buf];
    // work unit: a 64-row block, or (with a key-range split) one of its ns parts
    const uint32_t ud = s_unit[buf];
    const uint32_t row0 = (kSplit ? (ud & 0xffffu) : ud) * BLK;
    const uint32_t part = kSplit ? (ud >> 16) & 0xffu : 0u, nparts = kSplit ? ud >> 24 : 1u;
    const int kvh = item & 3u;
    const uint32_t nrows = min((uint32_t)BLK, rows - row0);

    // with a key-range split this unit takes tiles [t_lo, t_hi) of the block's tile sequence
    uint32_t t_lo = 0, t_hi = 0xffffffffu;
    if (kSplit) {
        uint32_t gt = 0, next = 0;
        PfRun run;
        while (pf_next_run(next, nruns, c_runs, run)) gt += (run.hi - run.lo + TK - 1) / TK;
        t_lo = (uint32_t)((uint64_t)gt * part / nparts);
        t_hi = (uint32_t)((uint64_t)gt * (part + 1u) / nparts);
    }

    if (warp_u < 8) {
        // ================= softmax warps: query tile j, accumulator row (head hw, token lane) =================
        const int j = warp_u >> 2, hw = warp_u & 3;
        const uint32_t tok = (uint32_t)(j * TOK + lane);
        const int head = kvh * 4 + hw;
        const uint32_t lane_base = tmem + ((uint32_t)(hw * 32) << 16);
        const uint32_t s_t = lane_base + S_COL + j * 64, p_t = lane_base + P_COL + j * 32;
        const uint32_t o_t = lane_base + O_COL + j * 128;
        // This thread's query row becomes a row of the A operand of the score MMAs: in TMEM for
        // query tile 0 (128 dims = 64 columns of f16 pairs), in shared memory (K-major, 128-byte
        // swizzle) for query tile 1.  The previous item's MMAs on this query tile completed before
        // this warp left that item's epilogue.
        {
            const bool valid = tok < nrows;
            const uint4* src = reinterpret_cast<const uint4*>(q + ((size_t)(row0 + (valid ? tok : 0u)) * NQ + head) * HD);
            if (j == 0) {
#pragma unroll
                for (int hf = 0; hf < 2; hf++) {
                    uint32_t qr[32];
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const uint4 v = valid ? __ldg(src + hf * 8 + i) : make_uint4(0u, 0u, 0u, 0u);
                        qr[4 * i] = v.x;
                        qr[4 * i + 1] = v.y;
                        qr[4 * i + 2] = v.z;
                        qr[4 * i + 3] = v.w;
                    }
                    tmem_st32(lane_base + Q0_COL + hf * 32, qr);
                }
                tmem_wait_st();
                tc_fence_before();
            } else {
                const uint32_t r = (uint32_t)(hw * 32 + lane);
#pragma unroll
                for (uint32_t c = 0; c < 16; c++) {
                    const uint4 v = valid ? __ldg(src + c) : make_uint4(0u, 0u, 0u, 0u);
                    const uint32_t dst = q1_s + (c >> 3) * Q_SUB + r * ROW_B + (((c & 7u) ^ (r & 7u)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
                }
                fence_proxy_async_smem();
            }
            mbar_arrive(&bar_qfull[j]);
        }

        float m_ref = -1.0e30f, l_run = 0.0f;  // maximum used for the exponentials (may be stale), row sum
        bool o_valid = false;                  // O in TMEM holds a sum (false until the item's first PV)
        uint32_t tflat = 0;                    // tiles of the block's runs before this one (key-range split)
        uint32_t next = 0;
        PfRun run;
        while (pf_next_run(next, nruns, c_runs, run)) {
            // this thread's row: valid key interval inside the run, empty if not in the run
            const bool in = tok >= run.r0 && tok < run.r1 && c_len[tok] != 0;
            const uint32_t rhi = in ? c_len[tok] : 0u;
            const uint32_t rlo = in ? window_start(c_len[tok], window) : 0u;
            // key range that is valid for every row of this query tile (mask-free tiles)
            const uint32_t lo_max = c_tile[j][0], hi_min = c_tile[j][1];
            const bool full = run.r0 <= (uint32_t)(j * TOK) && run.r1 >= (uint32_t)(j * TOK + TOK) && c_tile[j][2] != 0u;
            const uint32_t ntiles = (run.hi - run.lo + TK - 1) / TK;
            uint32_t tile0 = 0, tile1 = ntiles;  // this unit's tiles of the run
            if (kSplit) {
                tile0 = min(ntiles, max(t_lo, tflat) - tflat);
                tile1 = min(ntiles, max(t_hi, tflat) - tflat);
                tflat += ntiles;
            }
            for (uint32_t tile = tile0; tile < tile1; tile++) {
                ok &= mbar_wait_bounded(&bar_sfull[j], gk & 1u, &s_abort, wait_us);  // S_j(tile) complete
                __syncwarp();
                tc_fence_after();
                const uint32_t kbeg = run.lo + tile * TK;
                uint32_t sr[2][32];
                tmem_ld32(s_t, sr[0]);
                tmem_ld32(s_t + 32, sr[1]);
                tmem_wait_ld();
                tc_fence_before();
                mbar_arrive(&bar_sfree[j]);  // the next tile's scores may overwrite S_j now
                // PV_j of the tile before has long completed as a rule: polled here, needed before P is stored
                const bool pv_prev_done = mbar_try_wait(&bar_pvdone[j], (gk - 1u) & 1u);
                const bool interior = full && kbeg >= lo_max && kbeg + TK <= hi_min;
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
                l_run = l_run * corr + ((psa[0] + psa[1]) + (psa[2] + psa[3]));
                // P_j and O_j are free once PV_j of the tile before is complete (first tile of the CTA: passes)
                if (!pv_prev_done) ok &= mbar_wait_bounded(&bar_pvdone[j], (gk - 1u) & 1u, &s_abort, wait_us);
                __syncwarp();
                tc_fence_after();
                if (o_valid && __any_sync(0xffffffffu, raise)) {
                    // rare: the reference maximum of some row of this warp moved; rescale the warp's O rows
                    // (no MMA touches O_j between the completion seen above and the arrival below)
#pragma unroll
                    for (int ch = 0; ch < 4; ch++) {
                        uint32_t orow[32];
                        tmem_ld32(o_t + ch * 32, orow);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; i++) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * corr);
                        tmem_st32(o_t + ch * 32, orow);
                    }
                }
                tmem_st32(p_t, pk);
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(&bar_pfull[j]);
                o_valid = true;
                ++gk;
            }
        }

        // ---- a part of a split block leaves its unnormalised O row, reference maximum and row sum for
        // prefill_merge_kernel (a part without tiles leaves an empty sum)
        if (kSplit && nparts > 1u) {
            const uint32_t row = (uint32_t)(hw * 32 + lane);
            const size_t pidx = ((size_t)sp.slots[item >> 2] * NKV + kvh) * 2 + j;
            const bool live = tok < nrows && c_len[tok] != 0;
            // bounds build: the part's slot lies inside the reserved workspace
            const bool slot_ok = OXI_IN_BOUNDS(sp.slots[item >> 2] < sp.max_slots, status);
            if (o_valid && !slot_ok) {
                ok &= mbar_wait_bounded(&bar_ofull[j], n_o & 1u, &s_abort, wait_us);
                ++n_o;
            } else if (o_valid) {
                ok &= mbar_wait_bounded(&bar_ofull[j], n_o & 1u, &s_abort, wait_us);
                ++n_o;
                __syncwarp();
                tc_fence_after();
                uint4* po = reinterpret_cast<uint4*>(sp.part_o + (pidx * M + row) * HD);
#pragma unroll
                for (int ch = 0; ch < 4; ch++) {
                    uint32_t orow[32];
                    tmem_ld32(o_t + ch * 32, orow);
                    tmem_wait_ld();
#pragma unroll
                    for (int v4 = 0; v4 < 8; v4++)
                        po[ch * 8 + v4] = make_uint4(orow[4 * v4], orow[4 * v4 + 1], orow[4 * v4 + 2], orow[4 * v4 + 3]);
                }
            }
            if (slot_ok) *reinterpret_cast<float2*>(sp.part_ml + (pidx * M + row) * 2) =
                make_float2(m_ref, (o_valid && live && ok) ? l_run : 0.0f);
        } else
        // ---- epilogue: O row from TMEM, 1/sum, f16, gate on the f16 value (as online kernel + gate kernel)
        if (o_valid) {
            ok &= mbar_wait_bounded(&bar_ofull[j], n_o & 1u, &s_abort, wait_us);
            ++n_o;
            __syncwarp();
            tc_fence_after();
            // nothing is written once a wait of this thread gave up (kFault: or any wait of the CTA - the MMA warp
            // then withholds bar_ofull, so the wait above has failed too)
            const bool write = OXI_IN_BOUNDS(row0 + tok < rows || tok >= nrows, status) && tok < nrows && c_len[tok] != 0 && ok;
            const float inv = rcp_approx_ftz(l_run);
            const size_t rh = (size_t)(row0 + (write ? tok : 0u)) * NQ + head;
            const float sig = (gate && write) ? sigmoid_ref(h2f(gate[rh])) : 1.0f;
            uint4* out = reinterpret_cast<uint4*>(ctx_out + rh * HD);
#pragma unroll
            for (int ch = 0; ch < 4; ch++) {
                uint32_t orow[32];
                tmem_ld32(o_t + ch * 32, orow);
                tmem_wait_ld();
                if (write) {
#pragma unroll
                    for (int v8 = 0; v8 < 4; v8++) {
                        uint32_t w[4];
#pragma unroll
                        for (int jj = 0; jj < 4; jj++) {
                            uint16_t h0 = f2h(__fmul_rn(__uint_as_float(orow[v8 * 8 + 2 * jj]), inv));
                            uint16_t h1 = f2h(__fmul_rn(__uint_as_float(orow[v8 * 8 + 2 * jj + 1]), inv));
                            if (gate) {
                                h0 = f2h(__fmul_rn(h2f(h0), sig));
                                h1 = f2h(__fmul_rn(h2f(h1), sig));
                            }
                            w[jj] = (uint32_t)h0 | ((uint32_t)h1 << 16);
                        }
                        out[ch * 4 + v8] = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    } else if (warp_u == W_MMA0 || warp_u == W_MMA1) {
        // ================= MMA warps: warp W_MMAj issues the MMAs of query tile j =================
        // One elected lane issues, the whole warp waits.  The tensor pipe accepts an MMA only when
        // the one before has started, so the issuing thread is held for about the MMAs' execution
        // time and every barrier wait between two bursts would leave the pipe idle.  Hence two
        // issuing warps that alternate strictly (a token passed through bar_tok): while one warp
        // issues its burst, the other one waits for the data of its next burst.  Bursts are never
        // interleaved: MMAs that accumulate into the same tile stay back to back on the pipe.
        const uint32_t j = warp_u == W_MMA0 ? 0u : 1u;
        ok &= mbar_wait_bounded(&bar_qfull[j], it & 1u, &s_abort, wait_us);
        __syncwarp();
        tc_fence_after();
        // descriptors of ring stage 0; a stage / sub-tile / k-step is an offset added to the
        // 16-byte-unit start address field (no carry: shared addresses < 256 KB)
        const uint64_t k_desc0 = umma_desc(k_s, 16, 1024);      // K tiles: K-major
        const uint64_t v_desc0 = umma_desc(v_s, KV_SUB, 1024);  // V tiles: MN-major
        const uint64_t q1_desc = umma_desc(q1_s, 16, 1024);     // query tile 1: K-major
        auto qk = [&](uint32_t stage) {  // S_j = Q_j K^T: 128 dims = 8 k-steps of 16
            const uint64_t kd = k_desc0 + (uint64_t)(stage * (KV_TILE >> 4));
#pragma unroll
            for (int kk = 0; kk < 8; kk++) {
                const uint32_t koff = (uint32_t)(((kk >> 2) * KV_SUB + (kk & 3) * 32) >> 4);
                if (j == 0)
                    umma_ts(tmem + S_COL, tmem + Q0_COL + kk * 8, kd + koff, IDESC_QK, kk > 0 ? 1u : 0u);
                else
                    umma_ss(tmem + S_COL + 64, q1_desc + (uint32_t)(((kk >> 2) * Q_SUB + (kk & 3) * 32) >> 4), kd + koff,
                            IDESC_QK, kk > 0 ? 1u : 0u);
            }
            umma_commit(&bar_sfull[j]);
            umma_commit(&bar_kempty[stage]);
        };
        auto pv = [&](uint32_t stage, bool acc) {  // O_j (+)= P_j V: 64 keys = 4 k-steps of 16
            const uint64_t vd = v_desc0 + (uint64_t)(stage * (KV_TILE >> 4));
#pragma unroll
            for (int kk = 0; kk < TK / 16; kk++)
                umma_ts(tmem + O_COL + j * 128, tmem + P_COL + j * 32 + kk * 8,
                        vd + (uint32_t)((kk * 16 * ROW_B) >> 4), IDESC_PV, (kk > 0 || acc) ? 1u : 0u);
            umma_commit(&bar_pvdone[j]);
            umma_commit(&bar_vempty[stage]);
        };
        // Tile t of the item has global index g0 + t.  Step t of this warp is one burst: PV_j(t-2),
        // which needs P_j(t-2) stored, then QK_j(t), which needs S_j(t-1) read into registers by the
        // softmax warps - scores are produced one tile ahead of the softmax, so that the softmax warps
        // do not wait for the tensor pipe in steady state.  Steps G and G+1 drain the last two PVs.
        const uint32_t g0 = gk;
        auto step = [&](uint32_t t, bool has_pv, bool has_qk, bool last) {
            uint32_t sv = 0, sk = 0;
            if (has_pv) {
                const uint32_t g = g0 + t - 2;
                sv = g % NS;
                ok &= mbar_wait_bounded(&bar_vfull[sv], (g / NS) & 1u, &s_abort, wait_us);
                ok &= mbar_wait_bounded(&bar_pfull[j], g & 1u, &s_abort, wait_us);
            }
            if (has_qk) {
                const uint32_t g = g0 + t;
                sk = g % NS;
                ok &= mbar_wait_bounded(&bar_kfull[sk], (g / NS) & 1u, &s_abort, wait_us);
                if (t >= 1) ok &= mbar_wait_bounded(&bar_sfree[j], (g - 1u) & 1u, &s_abort, wait_us);
            }
            // the token: warp 0's n-th burst follows warp 1's (n-1)-th, warp 1's n-th follows warp 0's n-th
            ok &= mbar_wait_bounded(&bar_tok[j], (j == 0 ? n_burst + 1u : n_burst) & 1u, &s_abort, wait_us);
            __syncwarp();
            tc_fence_after();
            if (elect_one()) {
                if (has_pv) {
                    pv(sv, t > 2);
                    // "O is final" is only signalled while no wait of this CTA has given up: after a give-up the
                    // softmax warps' wait for it fails at once (the flag is set) and they write nothing
                    if (last && (!kFault || *const_cast<volatile uint32_t*>(&s_abort) == 0u)) umma_commit(&bar_ofull[j]);
                }
                if (has_qk) qk(sk);
                mbar_arrive(&bar_tok[j ^ 1u]);
            }
            __syncwarp();
            ++n_burst;
        };
        uint32_t nt = 0;  // tiles of this item whose score MMAs have been issued
        if (kSplit) {
            for (uint32_t t = t_lo; t < t_hi; t++) {
                step(nt, nt >= 2, true, false);
                ++nt;
                ++gk;
            }
        } else {
            uint32_t next = 0;
            PfRun run;
            while (pf_next_run(next, nruns, c_runs, run)) {
                const uint32_t ntiles = (run.hi - run.lo + TK - 1) / TK;
                for (uint32_t tile = 0; tile < ntiles; tile++) {
                    step(nt, nt >= 2, true, false);
                    ++nt;
                    ++gk;
                }
            }
        }
        if (nt > 0) {
            step(nt, nt >= 2, false, false);
            step(nt + 1, true, false, true);
            ++n_o;
        }
    } else if (warp_u == W_KLOAD || warp_u == W_VLOAD) {
        // ================= loader warps: one for the K ring, one for the V ring =================
        const bool is_k = warp_u == W_KLOAD;
        uint64_t* full = is_k ? bar_kfull : bar_vfull;
        uint64_t* empty = is_k ? bar_kempty : bar_vempty;
        const uint32_t ring = is_k ? k_s : v_s;
        // lane copies 16-byte chunk c of rows r0, r0+2, ...; chunk c of row r lands in sub-tile c/8 at
        // row r, chunk position (c%8) ^ (r%8)
        const uint32_t c = lane & 15u, r0 = lane >> 4;
        uint32_t pending = 0;  // tiles requested whose full barrier has not been signalled yet
        // publishes K (or V) tile number g to the tensor core; test support: CTA 0's K loader withholds one
        // tile (its copies have landed, the arrival never comes), so the MMA warps' wait for it runs out
        auto publish = [&](uint32_t g) {
            if (kFault && is_k && blockIdx.x == 0 && g + 1u == fault.skip_plus1) return;
            mbar_arrive(&full[g % NS]);
        };
        uint32_t tflat = 0;    // tiles of the block's runs before this one (key-range split)
        uint32_t next = 0;
        PfRun run;
        while (pf_next_run(next, nruns, c_runs, run)) {
            const char* base = paged ? reinterpret_cast<const char*>(is_k ? pm.k_pool : pm.v_pool) + kvh * (HD * 2)
                                     : reinterpret_cast<const char*>(is_k ? c_kp[run.r0] : c_vp[run.r0]) + kvh * (HD * 2);
            const uint32_t ntiles = (run.hi - run.lo + TK - 1) / TK;
            // paged: lane l holds the block of page (tile's first page + l); a 64-key tile spans at most 5
            // blocks of >= 16 tokens; the next tile's entries are fetched while this tile is copied
            const uint32_t* trow = paged ? pm.block_tables + (size_t)((c_kp[run.r0] >> 4) - 1ull) * pm.max_blocks : nullptr;
            const uint32_t last_page = paged ? (run.hi - 1u) >> pm.lbs : 0u;
            auto fetch_pages = [&](uint32_t kb) -> uint32_t {
                const uint32_t pg = (kb >> pm.lbs) + (uint32_t)lane;
                uint32_t id = 0;
                if (lane < 8 && pg <= last_page) {
                    id = __ldg(trow + pg);
                    if (id >= pm.num_blocks) {
                        atomicOr(status, DEV_BAD_BLOCK);
                        id = 0;
                    }
                }
                return id;
            };
            uint32_t tile0 = 0, tile1 = ntiles;  // this unit's tiles of the run
            if (kSplit) {
                tile0 = min(ntiles, max(t_lo, tflat) - tflat);
                tile1 = min(ntiles, max(t_hi, tflat) - tflat);
                tflat += ntiles;
            }
            uint32_t pg_next = (paged && tile0 < tile1) ? fetch_pages(run.lo + tile0 * TK) : 0u;
            // Rows of a registered slab (at a whole number of 1024-byte rows from its base) come through the
            // TMA unit: two boxes per full tile, written in the same swizzled layout, completion counted on
            // the stage's barrier.  The run's ragged last tile keeps the zero-filling copies below.
            bool tma_run = false;
            uint32_t tma_y0 = 0;
            if (kTma) {
                const uint64_t ptr = is_k ? c_kp[run.r0] : c_vp[run.r0];
                const uint64_t off = ptr - slab_base;
                tma_run = ptr >= slab_base && (off & 1023ull) == 0ull && (off >> 10) + run.hi <= (uint64_t)slab_rows;
                tma_y0 = (uint32_t)(off >> 10);
                if (tma_run && pending) {  // tiles of an earlier run still in flight as plain copies
                    cp_async_wait<0>();
                    fence_proxy_async_smem();
                    for (; pending > 0; --pending) publish(gk - pending);
                }
            }
            for (uint32_t tile = tile0; tile < tile1; tile++) {
                const uint32_t st = gk % NS;
                // the MMAs that read this stage's previous tile have completed (first use: passes at once)
                ok &= mbar_wait_bounded(&empty[st], ((gk / NS) & 1u) ^ 1u, &s_abort, wait_us);
                const uint32_t kbeg = run.lo + tile * TK;
                if (kTma && tma_run && kbeg + TK <= run.hi) {
                    if (lane == 0 && ok) {  // after a wait gave up nothing more is copied
                        mbar_arrive_expect_tx(&full[st], (uint32_t)KV_TILE);
                        tma_load_box(ring + st * KV_TILE, &tmap, (uint32_t)kvh * HD, tma_y0 + kbeg, &full[st]);
                        tma_load_box(ring + st * KV_TILE + KV_SUB, &tmap, (uint32_t)kvh * HD + 64u, tma_y0 + kbeg, &full[st]);
                    } else {
                        mbar_arrive(&full[st]);
                    }
                    ++gk;
                    continue;
                }
                const uint32_t dst = ring + st * KV_TILE + (c >> 3) * KV_SUB;
                const char* src = base + (size_t)(kbeg + r0) * KV_ROW_BYTES + c * 16;
                if (paged) {
                    const uint32_t pg_cur = pg_next;
                    if (tile + 1 < tile1) pg_next = fetch_pages(kbeg + TK);
                    const uint32_t p0 = kbeg >> pm.lbs, mask = (1u << pm.lbs) - 1u;
#pragma unroll 8
                    for (int k = 0; k < TK / 2; k++) {
                        const uint32_t row = r0 + 2 * k, tkn = kbeg + row;
                        const uint32_t pid = __shfl_sync(0xffffffffu, pg_cur, ((tkn >> pm.lbs) - p0) & 31u);
                        const bool valid = tkn < run.hi;  // rows past the run's last key are zero-filled
                        cp_async_16(dst + row * ROW_B + (((c & 7u) ^ (row & 7u)) << 4),
                                    valid ? base + (size_t)pid * pm.block_stride + (size_t)(tkn & mask) * KV_ROW_BYTES + c * 16 : base,
                                    valid);
                    }
                } else if (kbeg + TK <= run.hi) {
#pragma unroll
                    for (int k = 0; k < TK / 2; k++) {
                        const uint32_t row = r0 + 2 * k;
                        cp_async_16(dst + row * ROW_B + (((c & 7u) ^ (row & 7u)) << 4), src + (size_t)k * 2 * KV_ROW_BYTES, true);
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < TK / 2; k++) {
                        const uint32_t row = r0 + 2 * k;
                        const bool valid = kbeg + row < run.hi;  // rows past the run's last key are zero-filled
                        cp_async_16(dst + row * ROW_B + (((c & 7u) ^ (row & 7u)) << 4),
                                    valid ? src + (size_t)k * 2 * KV_ROW_BYTES : base, valid);
                    }
                }
                cp_async_commit();
                ++pending;
                ++gk;
                if (kTma && tma_run) {  // the one ragged tile of a run loaded by TMA: publish it at once
                    cp_async_wait<0>();
                    fence_proxy_async_smem();
                    publish(gk - 1u);
                    --pending;
                } else if (pending == DEPTH) {  // the oldest tile in flight has landed: publish it to the tensor core
                    cp_async_wait<DEPTH - 1>();
                    fence_proxy_async_smem();
                    publish(gk - DEPTH);
                    --pending;
                }
            }
        }
        cp_async_wait<0>();
        fence_proxy_async_smem();
        for (; pending > 0; --pending) publish(gk - pending);
        // all tiles of this item are on their way to the tensor core: claim the next item and prepare its
        // tables while the other roles work through the last tiles
        if (is_k) prepare_item(buf ^ 1u);
    }
  }  // item loop

    if (!ok) atomicOr(status, DEV_WAIT_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    if (warp_u == W_MMA0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// Combines the partial results of split blocks: one warp per accumulator row (grid = blocks x
// 4 KV heads x 2 query tiles x 32 groups of 4 rows), a lane holds 4 of the 128 dimensions.  Part s
// of a row holds O_s = sum_k 2^(x_k - m_s) v_k and l_s = sum_k 2^(x_k - m_s); the row's result is
// sum_s 2^(m_s - m) O_s / sum_s 2^(m_s - m) l_s with m = max_s m_s, rounded to f16 and gated like
// the unsplit epilogue.
__global__ void __launch_bounds__(128)
prefill_merge_kernel(uint16_t* __restrict__ ctx_out, const uint16_t* __restrict__ gate,
                     uint32_t rows, const PfSplit sp) {
    using namespace pf;
    const uint32_t tile = blockIdx.x >> 5;  // (block, KV head, query tile)
    const uint32_t blk = tile >> 3, kvh = (tile >> 1) & 3u, j = tile & 1u;
    const uint32_t meta = sp.blkmeta[blk];
    const uint32_t ns = meta & 0xffu, slot0 = meta >> 8;
    if (ns <= 1u) return;  // written by the attention kernel
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t row = (blockIdx.x & 31u) * 4 + (threadIdx.x >> 5);
    const uint32_t row0 = blk * BLK, nrows = min((uint32_t)BLK, rows - row0);
    const uint32_t tok = j * TOK + (row & 31u), head = kvh * 4 + (row >> 5);
    if (tok >= nrows) return;
    // lane s holds (m, l) of part s; a part without keys for this row has l = 0
    float m_s = -1.0e30f, l_s = 0.0f;
    if (lane < ns) {
        const size_t pidx = ((size_t)(slot0 + lane) * NKV + kvh) * 2 + j;
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(sp.part_ml + (pidx * M + row) * 2));
        if (ml.y > 0.0f) {
            m_s = ml.x;
            l_s = ml.y;
        }
    }
    float m = m_s;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    const float w_s = l_s > 0.0f ? ex2_approx_ftz(m_s - m) : 0.0f;
    float lsum = w_s * l_s;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, off);
    if (!(lsum > 0.0f)) return;  // row without keys: not written, as in the unsplit kernel
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (uint32_t s0 = 0; s0 < ns; s0 += 8) {  // eight loads in flight
        float4 o[8];
        float w[8];
#pragma unroll
        for (uint32_t u = 0; u < 8; u++) {
            const uint32_t s = s0 + u;
            w[u] = __shfl_sync(0xffffffffu, w_s, s & 31u);
            if (s >= ns) w[u] = 0.0f;
            const size_t pidx = ((size_t)(slot0 + s) * NKV + kvh) * 2 + j;
            // a part with weight 0 may never have been written
            o[u] = w[u] != 0.0f ? __ldcg(reinterpret_cast<const float4*>(sp.part_o + (pidx * M + row) * HD) + lane)
                                : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
#pragma unroll
        for (uint32_t u = 0; u < 8; u++) {
            acc.x = fmaf(w[u], o[u].x, acc.x);
            acc.y = fmaf(w[u], o[u].y, acc.y);
            acc.z = fmaf(w[u], o[u].z, acc.z);
            acc.w = fmaf(w[u], o[u].w, acc.w);
        }
    }
    const float inv = rcp_approx_ftz(lsum);
    const size_t rh = (size_t)(row0 + tok) * NQ + head;
    uint16_t h[4] = {f2h(__fmul_rn(acc.x, inv)), f2h(__fmul_rn(acc.y, inv)), f2h(__fmul_rn(acc.z, inv)),
                     f2h(__fmul_rn(acc.w, inv))};
    if (gate) {
        const float sig = sigmoid_ref(h2f(gate[rh]));
#pragma unroll
        for (int e = 0; e < 4; e++) h[e] = f2h(__fmul_rn(h2f(h[e]), sig));
    }
    reinterpret_cast<uint2*>(ctx_out + rh * HD)[lane] =
        make_uint2((uint32_t)h[0] | ((uint32_t)h[1] << 16), (uint32_t)h[2] | ((uint32_t)h[3] << 16));
}

size_t prefill_split_table_bytes() { return (size_t)3 * 1024 * PF_MAX_SPLIT * sizeof(uint32_t); }
size_t prefill_split_slot_bytes() { return (size_t)NKV * 2 * pf::M * (HD + 2) * sizeof(float); }

template <bool kPaged, bool kSplit, bool kTma, bool kFault = false>
static cudaError_t pf_set_smem() {
    return cudaFuncSetAttribute(prefill_attn_kernel<kPaged, kSplit, kTma, kFault>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)pf::SMEM_BYTES);
}

cudaError_t prefill_attn_init() {
    cudaError_t e = cudaSuccess;
    if ((e = pf_set_smem<false, false, false>())) return e;
    if ((e = pf_set_smem<true, false, false>())) return e;
    if ((e = pf_set_smem<false, true, false>())) return e;
    if ((e = pf_set_smem<true, true, false>())) return e;
    if ((e = pf_set_smem<false, false, true>())) return e;
    if ((e = pf_set_smem<false, false, false, true>())) return e;
    return pf_set_smem<false, true, true>();
}

template <bool kPaged, bool kSplit, bool kTma, bool kFault = false>
static cudaError_t launch_pf(cudaStream_t stream, uint32_t grid, void* ctx_out, const void* q, const void* gate,
                             const uint64_t* k_ptrs, const uint64_t* v_ptrs, const uint32_t* seq_lens, uint32_t rows,
                             uint32_t window, uint32_t* status, uint32_t* order, uint32_t* counter, const PagedMap& pm,
                             const uint32_t* row_seq, const PfSplit& sp, const PrefillSlab& slab, const WaitFault& fault) {
    // programmatic dependent of the plan kernel: TMEM allocation and barrier set-up overlap it
    return launch_pdl(prefill_attn_kernel<kPaged, kSplit, kTma, kFault>, dim3(grid), dim3(pf::THREADS), pf::SMEM_BYTES, stream,
                      (uint16_t*)ctx_out, (const uint16_t*)q, (const uint16_t*)gate, k_ptrs, v_ptrs, seq_lens, rows,
                      window, status, (const uint32_t*)order, counter, pm, row_seq, sp, slab.map, slab.base, slab.rows, fault);
}

cudaError_t launch_prefill_attn(cudaStream_t stream, void* ctx_out, const void* q,
                                const void* gate, const uint64_t* k_ptrs, const uint64_t* v_ptrs,
                                const uint32_t* seq_lens, uint32_t rows, uint32_t window,
                                uint32_t* status, int num_sms, uint32_t* order, uint32_t* counter,
                                const PagedMap* pm, const uint32_t* row_seq, const PrefillSplitWs* ws,
                                uint32_t part_keys, const PrefillSlab* slab, const WaitFault* fault) {
    const WaitFault flt = fault ? *fault : WaitFault{};
    const uint32_t nblocks = (rows + pf::BLK - 1) / pf::BLK;
    // the split is for waves that leave SMs idle; larger waves balance by claiming longest first
    // an armed test fault runs the plain instantiation: pointer tables, unsplit, per-thread copies
    const bool armed = flt.skip_plus1 != 0u && !pm;
    const bool split = !armed && ws && ws->max_slots != 0u && part_keys != 0u && nblocks * NKV < (uint32_t)num_sms;
    PfSplit sp{};
    if (split) {
        sp.units = ws->units;
        sp.slots = ws->units + 1024 * PF_MAX_SPLIT;
        sp.blkmeta = ws->units + 2 * 1024 * PF_MAX_SPLIT;
        sp.part_o = ws->part;
        sp.part_ml = ws->part + (size_t)ws->max_slots * NKV * 2 * pf::M * HD;
        sp.part_tiles = (part_keys + pf::TK - 1) / pf::TK;
        sp.max_slots = ws->max_slots;
        sp.target_items = (uint32_t)num_sms;
    }
    if (nblocks <= 1024u)
        (void)launch_pdl(prefill_plan_small_kernel, dim3(1), dim3(1024), 0, stream, seq_lens, rows, window, order, counter, sp);
    else
        prefill_plan_kernel<<<1, 1024, 0, stream>>>(seq_lens, rows, window, order, counter);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const PagedMap map = pm ? *pm : PagedMap{};
    const PrefillSlab none{};
    const bool tma = !armed && !pm && slab && slab->rows != 0u;
    const PrefillSlab& sl = tma ? *slab : none;
#define OXI_PF_ARGS ctx_out, q, gate, k_ptrs, v_ptrs, seq_lens, rows, window, status, order, counter, map, row_seq, sp, sl, flt
    if (!split) {
        const uint32_t nitems = nblocks * NKV;
        const uint32_t grid = nitems < (uint32_t)num_sms ? nitems : (uint32_t)num_sms;
        if (pm) return launch_pf<true, false, false>(stream, grid, OXI_PF_ARGS);
        if (armed) return launch_pf<false, false, false, true>(stream, grid, OXI_PF_ARGS);
        return tma ? launch_pf<false, false, true>(stream, grid, OXI_PF_ARGS)
                   : launch_pf<false, false, false>(stream, grid, OXI_PF_ARGS);
    }
    // the unit count is only known on the device: one CTA per SM, those without a unit leave at once
    const uint32_t grid = (uint32_t)num_sms;
    if (pm) e = launch_pf<true, true, false>(stream, grid, OXI_PF_ARGS);
    else e = tma ? launch_pf<false, true, true>(stream, grid, OXI_PF_ARGS) : launch_pf<false, true, false>(stream, grid, OXI_PF_ARGS);
#undef OXI_PF_ARGS
    if (e != cudaSuccess) return e;
    // a plain launch: as a programmatic dependent it measured no faster
    prefill_merge_kernel<<<nblocks * 8 * 32, 128, 0, stream>>>((uint16_t*)ctx_out, (const uint16_t*)gate, rows, sp);
    return cudaGetLastError();
}

}  // namespace oxi
