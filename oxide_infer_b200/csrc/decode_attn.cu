// Split-KV flash-decode GQA attention with the sigmoid output gate.
//
// Replaces batched_gqa_attention_split4_fp16 + batched_gqa_attn_combine_fp16 +
// batched_sigmoid_gate_fp16 (batched_attn.rs:2665-3035, 1597-1717, 583-655).
//
// Work decomposition.  A work item is (row b, key range c) where the ranges
// are fixed CHUNK-key slices of the row's own [window start, seq_len) interval,
// so a row's arithmetic never depends on which other rows share the launch.
// The grid is persistent (one CTA per SM); every CTA derives the item list from
// seq_lens on the device (prefix sum of per-row range counts in shared memory),
// takes item blockIdx.x first and then claims further items from a global work
// counter (claimed two items ahead, so the claim's latency is off the critical
// path).  The host needs no knowledge of the lengths, the launch shape never
// changes, and SMs that receive less memory bandwidth simply claim fewer items.
//
// Inside a CTA: one producer warp streams K and V rows (1024 B each: all four
// KV heads of one token are contiguous) into a ring of shared-memory stages
// with 1-D bulk copies (TMA engine) that complete on mbarriers; four consumer
// warps, one per KV head, each serve the 4 query heads of their group from
// that single K/V read: S = Q K^T and O += P V run on tensor cores
// (mma.sync.m16n8k16, f16 in, f32 accumulate; the 4 heads are rows 0..3 of the
// M=16 tile), the online-softmax row reductions are quad shuffles.  K/V rows
// are copied in groups of 4 consecutive tokens (4 KB per bulk copy: large
// copies keep the TMA issue rate off the critical path) and each group is
// padded by 16 bytes in shared memory; an 8x8 ldmatrix tile takes its 8 rows
// from 8 different groups (keys j, j+4, ..., j+28), so the 8 row addresses of
// every ldmatrix phase fall in distinct banks.  The key order inside a stage is
// therefore a permutation, applied consistently to the P columns and V rows.
//
// Every stage carries a 16-byte descriptor written by the producer (row, range,
// valid keys, first/last-of-item flags), and the first stage of an item also
// carries the row's q (4 KB, one more bulk copy); seq_lens are staged in shared
// memory.  A consumer warp therefore issues no global load of its own while
// streaming: under a saturated memory pipe every dependent global access costs
// microseconds of queueing behind the stream.
//
// Fused variant (kFused, behind oxi_append_decode): the per-head Q/K RMSNorm + RoPE + KV append
// of batched_attn.rs:13-287 runs inside this kernel, so q never makes a round trip through
// HBM before it is used and the append launch disappears.  The producer delivers the RAW q
// row plus the position's cos/sin rows with an item's first stage; each consumer warp
// normalises and rotates its 4 query heads in shared memory with the append kernel's exact
// arithmetic.  The item holding a row's LAST key range is the row's "owner": the key at
// position seq_len-1 does not exist in the cache yet, so the producer copies one key less
// and delivers the raw k/v rows instead; each consumer warp normalises/rotates its K head,
// drops K and V into the stage at that key's place, and writes the cache row to global
// memory.  No other item reads that cache row, so nothing waits on another CTA.  The caller's
// q buffer is not modified.  Context and cache bytes are identical to append followed by the
// unfused kernel.
//
// A row covered by one item is finished in registers (1/sum, f16, gate).
// Otherwise each consumer warp stores its (max, sum, acc[128]) partials and
// moves on; a second, tiny kernel merges the partials of every multi-item row
// in key-range order (deterministic), applies 1/sum, rounds to f16 and applies
// the gate exactly as the reference's gate kernel does on the f16 context, and
// resets the work counter.  Nothing spins on another CTA; the only waits are on
// this CTA's own mbarriers and they are time-bounded.
#include <mutex>

#include "../../include/oxi_kv.h"
#include "common.cuh"
#include "kernels.h"
#include "norm_rope.cuh"

#ifndef OXI_DEC_NSTAGE
#define OXI_DEC_NSTAGE 3
#endif
#ifndef OXI_DEC_CHUNK
#define OXI_DEC_CHUNK 256
#endif
#ifndef OXI_DEC_MAXROWS
#define OXI_DEC_MAXROWS 1024
#endif

namespace oxi {

namespace dec {
constexpr int KS = 32;                          // keys per pipeline stage
constexpr int NSTAGE = OXI_DEC_NSTAGE;          // ring depth
constexpr int GK = 4;                           // keys per bulk copy (one group)
constexpr int GROUP_BYTES = GK * KV_ROW_BYTES;  // 4096 B copied at once
constexpr int GPITCH = GROUP_BYTES + 16;        // group pitch in shared memory
constexpr int NGROUP = KS / GK;                 // 8 groups per stage = the 8 rows of an ldmatrix tile
constexpr int HALF_BYTES = NGROUP * GPITCH;     // K part (then V part) of a stage
constexpr int Q_BYTES = NQ * HD * 2;            // the row's q (all heads), carried by an item's first stage
// extra inputs of the fused variant: cos row, sin row (256 B each), raw k row, raw v row (1 KB each)
constexpr int X_COS = 0, X_SIN = 256, X_K = 512, X_V = 512 + KV_ROW_BYTES;
constexpr int X_BYTES = 512 + 2 * KV_ROW_BYTES;
constexpr int DESC_BYTES = 32;
constexpr int Q_OFF = 2 * HALF_BYTES, X_OFF = Q_OFF + Q_BYTES, DESC_OFF = X_OFF + X_BYTES;
constexpr int STAGE_BYTES = DESC_OFF + DESC_BYTES;
constexpr int CHUNK = OXI_DEC_CHUNK;            // keys per work item
constexpr int N_CONSUMER_WARPS = NKV;           // one per KV head
constexpr int THREADS = (N_CONSUMER_WARPS + 1) * 32;
constexpr int MAX_ROWS = OXI_DEC_MAXROWS;       // rows per launch (prefix + length arrays in shared memory)
constexpr float QK_SCALE_LOG2 = ATTN_SCALE * LOG2E;
constexpr int W_BYTES = 2 * HD * 2;  // q and k norm weights (fused variant)
constexpr size_t SMEM_BYTES = (size_t)NSTAGE * STAGE_BYTES + 2 * NSTAGE * 8 + 16 + W_BYTES +
                              (2 * MAX_ROWS + 1) * sizeof(uint32_t);
static_assert(SMEM_BYTES <= 227 * 1024, "decode kernel shared memory");
static_assert(CHUNK % KS == 0, "a work item is a whole number of stages");
static_assert(NGROUP == 8, "ldmatrix tiles take one row from each of 8 groups");
static_assert(STAGE_BYTES % 16 == 0, "stage alignment");

// stage descriptor flags (word z)
constexpr uint32_t F_FIRST = 0x100u, F_LAST = 0x200u, F_END = 0x400u;
constexpr uint32_t F_LASTRANGE = 0x800u;  // the item is its row's last key range (fused: the row's owner)
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
    uint32_t* work_counter;
    uint32_t* status;
    float* merge_acc;      // [batch][16][ceil(max_chunks / 16)][132]: slice sums of rows with more than 16 key ranges
    uint32_t* merge_count; // [batch][4] arrival counters of those rows, zero between launches
    uint32_t batch;
    uint32_t window;
    uint32_t max_chunks;
    uint32_t max_seq_len;
    // paged variant only: K/V rows live in fixed-size blocks of a pool, block_tables[b][i] is the
    // block that holds tokens [i*bs, (i+1)*bs) of row b (k_ptrs / v_ptrs are then unused)
    PagedMap paged;
    // fused variant only (q is then the raw projected q)
    const uint16_t* k_in;
    const uint16_t* v_in;
    const uint16_t* q_norm_w;
    const uint16_t* k_norm_w;
    const uint16_t* cos_t;
    const uint16_t* sin_t;
    float eps;
    WaitFault fault;  // test support; zero on every normal launch
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

template <bool kFused, bool kPaged>
__global__ void __launch_bounds__(dec::THREADS, 1)
decode_attn_kernel(const DecodeParams p) {
    using namespace dec;
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* stages = smem;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)NSTAGE * STAGE_BYTES);
    uint64_t* empty_bar = full_bar + NSTAGE;
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(empty_bar + NSTAGE);
    uint16_t* s_w = const_cast<uint16_t*>(reinterpret_cast<volatile uint16_t*>(abort_flag) + 8);  // [q_norm_w | k_norm_w]
    uint32_t* prefix = reinterpret_cast<uint32_t*>(s_w + 2 * HD);
    uint32_t* s_len = prefix + MAX_ROWS + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t wait_us = p.fault.skip_plus1 ? p.fault.limit_us : WAIT_LIMIT_US;
    pdl_launch_dependents();  // the merge kernel may be scheduled now; it waits for this grid to finish

    // ---- prologue: barriers, per-row range counts, prefix sum, lengths into shared memory
    // (reads only the step's tables, which no kernel writes)
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
        } else if (kPaged && ((slen - 1u) >> p.paged.lbs) >= p.paged.max_blocks) {
            if (blockIdx.x == 0) atomicOr(p.status, DEV_BAD_SEQ_LEN);  // more blocks than the table has columns
        } else if (!kPaged && ((p.k_ptrs[b] | p.v_ptrs[b]) & 15ull) != 0ull) {
            if (blockIdx.x == 0) atomicOr(p.status, DEV_MISALIGNED_PTR);
        } else {
            n = row_chunks(slen, p.window);
        }
        prefix[b + 1] = n;
        s_len[b] = slen;
    }
    if (kFused) {
        for (uint32_t i = threadIdx.x; i < 2u * HD; i += THREADS)
            s_w[i] = i < (uint32_t)HD ? p.q_norm_w[i] : p.k_norm_w[i - HD];
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
    pdl_wait();  // K/V rows and q written by the preceding kernel are visible from here on

    if (warp == N_CONSUMER_WARPS) {
        // =========================== producer warp ===========================
        const uint64_t policy = l2_policy_evict_first();
        uint32_t fill = 0;
        bool ok = true;
        // Item pipeline: `cur` is streamed now; `nxt` is known and its pointers are being
        // fetched; the claim for the item after `nxt` is in flight (lane 0's `claim`).
        uint32_t cur = blockIdx.x;
        uint32_t cb = 0, cc = 0, cslen = 0;
        uint64_t ckp = 0, cvp = 0;
        // paged: lane l holds the block of the item's l-th page (an item spans at most CHUNK / 16 + 1 = 17
        // pages), fetched one item ahead like the row pointers
        uint32_t cpg = 0, cfp = 0;
        auto fetch_pages = [&](uint32_t b, uint32_t c, uint32_t slen, uint32_t& first_page) -> uint32_t {
            const uint32_t t0 = window_start(slen, p.window) + c * CHUNK;
            const uint32_t t1 = min(t0 + (uint32_t)CHUNK, slen);
            first_page = t0 >> p.paged.lbs;
            const uint32_t pg = first_page + (uint32_t)lane;
            uint32_t id = 0;
            if (pg <= ((t1 - 1u) >> p.paged.lbs)) {
                id = __ldg(p.paged.block_tables + (size_t)b * p.paged.max_blocks + pg);
                if (id >= p.paged.num_blocks) {
                    atomicOr(p.status, DEV_BAD_BLOCK);
                    id = 0;
                }
            }
            return id;
        };
        if (cur < total_items) {
            cb = find_row(prefix, p.batch, cur);
            cc = cur - prefix[cb];
            cslen = s_len[cb];
            if (kPaged) {
                cpg = fetch_pages(cb, cc, cslen, cfp);
            } else {
                ckp = p.k_ptrs[cb];
                cvp = p.v_ptrs[cb];
            }
        }
        uint32_t claim = 0;
        if (lane == 0 && cur < total_items) claim = atomicAdd(p.work_counter, 1u);

        while (cur < total_items && ok) {
            uint32_t nxt = __shfl_sync(0xffffffffu, claim, 0);
            nxt = (nxt >= total_items) ? total_items : min(nxt + gridDim.x, total_items);
            uint32_t nb = 0, nc = 0, nslen = 0, npg = 0, nfp = 0;
            uint64_t nkp = 0, nvp = 0;
            claim = 0xffffffffu;  // "no more items" unless a new claim is made
            if (nxt < total_items) {
                if (lane == 0) claim = atomicAdd(p.work_counter, 1u);
                nb = find_row(prefix, p.batch, nxt);
                nc = nxt - prefix[nb];
                nslen = s_len[nb];
                if (kPaged) {
                    npg = fetch_pages(nb, nc, nslen, nfp);
                } else {
                    nkp = p.k_ptrs[nb];
                    nvp = p.v_ptrs[nb];
                }
            }
            const uint32_t nchunks = prefix[cb + 1] - prefix[cb];
            const bool last_range = (cc + 1 == nchunks);
            const uint32_t pos = cslen - 1u;  // position of the token appended in this step
            const char* qp = reinterpret_cast<const char*>(p.q) + (size_t)cb * Q_BYTES;
            const char* kp = reinterpret_cast<const char*>(ckp);
            const char* vp = reinterpret_cast<const char*>(cvp);
            const uint32_t t0 = window_start(cslen, p.window) + cc * CHUNK;
            const uint32_t t1 = min(t0 + (uint32_t)CHUNK, cslen);
            const uint32_t bs_mask = kPaged ? (1u << p.paged.lbs) - 1u : 0u;
            if (kPaged && kFused) {
                // the consumers write the appended row at base + pos * row bytes: give them the base that
                // makes this the row's place in its block (only meaningful in the row's last range)
                const uint32_t pid = __shfl_sync(0xffffffffu, cpg, ((pos >> p.paged.lbs) - cfp) & 31u);
                const uint64_t off = (uint64_t)pid * p.paged.block_stride + (uint64_t)(pos & bs_mask) * KV_ROW_BYTES -
                                     (uint64_t)pos * KV_ROW_BYTES;
                ckp = (uint64_t)(uintptr_t)p.paged.k_pool + off;
                cvp = (uint64_t)(uintptr_t)p.paged.v_pool + off;
            }
            for (uint32_t t = t0; t < t1; t += KS, ++fill) {
                const uint32_t slot = fill % NSTAGE;
                if (fill >= NSTAGE &&
                    !mbar_wait_bounded(&empty_bar[slot], ((fill / NSTAGE) & 1u) ^ 1u, abort_flag, wait_us)) {
                    ok = false;
                    break;
                }
                // test support: this CTA's stage goes missing (no descriptor, no arrival, no copy), so the
                // consumers' wait for it runs out
                if (p.fault.skip_plus1 && blockIdx.x == 0 && fill + 1u == p.fault.skip_plus1) continue;
                const uint32_t nvalid = min((uint32_t)KS, t1 - t);
                const bool first = (t == t0), last = (t + KS >= t1);
                // fused: the owner's last stage ends with the key being appended; it is not in the
                // cache yet, so one key less is copied and the raw k/v rows are delivered instead
                const bool owner = kFused && last && last_range;
                const uint32_t ncopy = owner ? nvalid - 1u : nvalid;
                unsigned char* sb = stages + (size_t)slot * STAGE_BYTES;
                if (lane == 0) {
                    *reinterpret_cast<uint4*>(sb + DESC_OFF) =
                        make_uint4(cb, cc | (nchunks << 16),
                                   nvalid | (first ? F_FIRST : 0u) | (last ? F_LAST : 0u) |
                                       (last_range ? F_LASTRANGE : 0u), pos);
                    *reinterpret_cast<uint4*>(sb + DESC_OFF + 16) =
                        make_uint4((uint32_t)ckp, (uint32_t)(ckp >> 32), (uint32_t)cvp, (uint32_t)(cvp >> 32));
                    uint32_t bytes = ncopy * 2u * KV_ROW_BYTES + (first ? Q_BYTES : 0);
                    if (kFused) bytes += ((first || owner) ? 512u : 0u) + (owner ? 2u * KV_ROW_BYTES : 0u);
                    mbar_arrive_expect_tx(&full_bar[slot], bytes);
                }
                __syncwarp();
                const uint32_t sbase = smem_u32(sb);
                // lanes 0..7 copy the K groups, lanes 8..15 the V groups (up to 4 KB each), lane 16 the q
                // row; fused: lanes 17/18 the cos/sin rows, lanes 19/20 the raw k/v rows of the owner
                // paged: a group of 4 tokens lies in one block or straddles two (blocks hold >= 16 tokens)
                uint32_t pid0 = 0, pid1 = 0;
                if (kPaged) {
                    const uint32_t pi = ((t + (lane & (NGROUP - 1)) * GK) >> p.paged.lbs) - cfp;
                    pid0 = __shfl_sync(0xffffffffu, cpg, pi & 31u);
                    pid1 = __shfl_sync(0xffffffffu, cpg, (pi + 1u) & 31u);
                }
                if (lane < 2 * NGROUP) {
                    const uint32_t grp = lane & (NGROUP - 1);
                    const bool is_v = lane >= NGROUP;
                    if (grp * GK < ncopy) {
                        const uint32_t nk = min((uint32_t)GK, ncopy - grp * GK);
                        const uint32_t dst = sbase + (is_v ? HALF_BYTES : 0) + grp * GPITCH;
                        // bounds build: the copied rows lie inside the row's keys and inside the stage
                        if (!OXI_IN_BOUNDS(cb < p.batch && t + grp * GK + nk <= cslen &&
                                               grp * GPITCH + nk * KV_ROW_BYTES <= (uint32_t)HALF_BYTES, p.status)) {
                            // nothing is copied; the stage's expected byte count must still be met
                            asm volatile("mbarrier.complete_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&full_bar[slot])),
                                         "r"(nk * KV_ROW_BYTES) : "memory");
                        } else if (kPaged) {
                            const unsigned char* pool = is_v ? p.paged.v_pool : p.paged.k_pool;
                            const uint32_t off = (t + grp * GK) & bs_mask;
                            const uint32_t n1 = min(nk, bs_mask + 1u - off);
                            bulk_g2s_hint(dst, pool + (size_t)pid0 * p.paged.block_stride + (size_t)off * KV_ROW_BYTES,
                                          n1 * KV_ROW_BYTES, &full_bar[slot], policy);
                            if (n1 < nk)
                                bulk_g2s_hint(dst + n1 * KV_ROW_BYTES, pool + (size_t)pid1 * p.paged.block_stride,
                                              (nk - n1) * KV_ROW_BYTES, &full_bar[slot], policy);
                        } else {
                            const char* src = (is_v ? vp : kp) + (size_t)(t + grp * GK) * KV_ROW_BYTES;
                            bulk_g2s_hint(dst, src, nk * KV_ROW_BYTES, &full_bar[slot], policy);
                        }
                    }
                } else if (first && lane == 2 * NGROUP) {
                    bulk_g2s(sbase + Q_OFF, qp, Q_BYTES, &full_bar[slot]);
                } else if (kFused && (first || owner) && (lane == 17 || lane == 18)) {
                    const uint16_t* tbl = (lane == 17) ? p.cos_t : p.sin_t;
                    bulk_g2s(sbase + X_OFF + (lane == 17 ? X_COS : X_SIN), tbl + (size_t)pos * HD, 256, &full_bar[slot]);
                } else if (kFused && owner && (lane == 19 || lane == 20)) {
                    const uint16_t* src = (lane == 19 ? p.k_in : p.v_in) + (size_t)cb * (NKV * HD);
                    bulk_g2s(sbase + X_OFF + (lane == 19 ? X_K : X_V), src, KV_ROW_BYTES, &full_bar[slot]);
                }
            }
            cur = nxt; cb = nb; cc = nc; cslen = nslen; ckp = nkp; cvp = nvp; cpg = npg; cfp = nfp;
        }
        if (ok) {
            // end-of-work descriptor so the consumers leave their loop
            const uint32_t slot = fill % NSTAGE;
            if (fill < NSTAGE || mbar_wait_bounded(&empty_bar[slot], ((fill / NSTAGE) & 1u) ^ 1u, abort_flag, wait_us)) {
                if (lane == 0) {
                    *reinterpret_cast<uint4*>(stages + (size_t)slot * STAGE_BYTES + DESC_OFF) =
                        make_uint4(0u, 0u, F_END, 0u);
                    mbar_arrive(&full_bar[slot]);
                }
                ++fill;
            } else {
                ok = false;
            }
        }
        if (!ok) {
            // Pipeline gave up: report, then give the copies already issued a bounded
            // time to land before this CTA's shared memory is released.
            if (lane == 0) atomicOr(p.status, DEV_WAIT_TIMEOUT);
            for (uint32_t k = fill > NSTAGE ? fill - NSTAGE : 0; k < fill; ++k)
                mbar_wait_drain(&full_bar[k % NSTAGE], (k / NSTAGE) & 1u, wait_us);
        }
        return;
    }

    // ============================= consumer warps =============================
    const int kvh = warp;            // this warp's KV head
    const int g = lane >> 2;         // fragment row (query head within the group when g < 4)
    const int t4 = lane & 3;         // fragment column pair
    const uint32_t head = kvh * 4 + (g & 3);
    const uint64_t keep_policy = l2_policy_evict_last();

    uint32_t qa[8][2];  // Q fragments (A operand, rows 0..3 = the group's heads, rows 4..15 zero)
    float o[16][4];
    float m_run = -1.0e30f, l_run = 0.0f;
#pragma unroll
    for (int ks = 0; ks < 8; ks++) { qa[ks][0] = qa[ks][1] = 0u; }
#pragma unroll
    for (int j = 0; j < 16; j++) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f; }

    for (uint32_t take = 0;; ++take) {
        const uint32_t slot = take % NSTAGE;
        if (!mbar_wait_bounded(&full_bar[slot], (take / NSTAGE) & 1u, abort_flag, wait_us)) {
            if (lane == 0) atomicOr(p.status, DEV_WAIT_TIMEOUT);
            break;
        }
        unsigned char* sb = stages + (size_t)slot * STAGE_BYTES;
        const uint4 desc = *reinterpret_cast<const uint4*>(sb + DESC_OFF);
        if (desc.z & F_END) break;
        const uint32_t nvalid = desc.z & 0xffu;
        unsigned char* kst = sb + kvh * (HD * 2);
        unsigned char* vst = kst + HALF_BYTES;

        if (desc.z & F_FIRST) {  // new item: reset the running state, take the row's q from the stage
            if (kFused) {
                // raw q arrived: RMSNorm + RoPE of this group's 4 heads in place in the stage (same
                // arithmetic and lane/dim mapping as the append kernel).  The q buffer in global memory
                // is left untouched: other items of the row still read the raw row.
                float cv[4], sv[4], wv[4];
                load4(reinterpret_cast<const uint16_t*>(sb + X_OFF + X_COS), lane, cv);
                load4(reinterpret_cast<const uint16_t*>(sb + X_OFF + X_SIN), lane, sv);
                load4(s_w, lane, wv);
#pragma unroll
                for (int hh = 0; hh < 4; hh++) {
                    uint16_t* qh = reinterpret_cast<uint16_t*>(sb + Q_OFF) + (kvh * 4 + hh) * HD;
                    uint16_t out[4];
                    head_norm_rope<true, true>(qh, wv, p.eps, cv, sv, lane, out);
#pragma unroll
                    for (int i = 0; i < 4; i++) qh[lane + 32 * i] = out[i];
                }
                __syncwarp();
            }
            const unsigned char* qrow = sb + Q_OFF + head * (HD * 2);
#pragma unroll
            for (int ks = 0; ks < 8; ks++) {
                uint32_t lo = 0, hi = 0;
                if (g < 4) {
                    lo = *reinterpret_cast<const uint32_t*>(qrow + (16 * ks + 2 * t4) * 2);
                    hi = *reinterpret_cast<const uint32_t*>(qrow + (16 * ks + 8 + 2 * t4) * 2);
                }
                qa[ks][0] = lo;
                qa[ks][1] = hi;
            }
#pragma unroll
            for (int j = 0; j < 16; j++) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f; }
            m_run = -1.0e30f;
            l_run = 0.0f;
        }
        const bool owner = kFused && (desc.z & F_LAST) && (desc.z & F_LASTRANGE);
        if (owner) {
            // the key being appended is the stage's last valid key: build its K (norm + rope) and V
            // for this KV head in the stage, and write the cache row
            const uint32_t kidx = nvalid - 1u;
            float cv[4], sv[4], wv[4];
            load4(reinterpret_cast<const uint16_t*>(sb + X_OFF + X_COS), lane, cv);
            load4(reinterpret_cast<const uint16_t*>(sb + X_OFF + X_SIN), lane, sv);
            load4(s_w + HD, lane, wv);
            uint16_t out[4];
            head_norm_rope<true, true>(reinterpret_cast<const uint16_t*>(sb + X_OFF + X_K) + kvh * HD, wv, p.eps, cv, sv,
                                       lane, out);
            const uint32_t roff = (kidx >> 2) * GPITCH + (kidx & 3u) * KV_ROW_BYTES;
            uint16_t* krow_s = reinterpret_cast<uint16_t*>(kst + roff);
            const uint64_t kp64 = *reinterpret_cast<const uint64_t*>(sb + DESC_OFF + 16);
            const uint64_t vp64 = *reinterpret_cast<const uint64_t*>(sb + DESC_OFF + 24);
            uint16_t* krow_g = reinterpret_cast<uint16_t*>(kp64 + (size_t)desc.w * KV_ROW_BYTES) + kvh * HD;
            // bounds build: the appended row is the row's last key and lies inside the stage
            const bool row_ok = OXI_IN_BOUNDS(desc.w < p.max_seq_len && kidx < (uint32_t)KS, p.status);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                krow_s[lane + 32 * i] = out[i];
                if (row_ok) krow_g[lane + 32 * i] = out[i];
            }
            const uint2 vv = *reinterpret_cast<const uint2*>(sb + X_OFF + X_V + kvh * (HD * 2) + lane * 8);
            *reinterpret_cast<uint2*>(vst + roff + lane * 8) = vv;
            if (row_ok) *reinterpret_cast<uint2*>(vp64 + (size_t)desc.w * KV_ROW_BYTES + kvh * (HD * 2) + lane * 8) = vv;
            __syncwarp();
        }
        if (nvalid < KS) {
            // tail stage: rows past the range keep stale bytes; zero this head's V slice there
            // so that 0 * stale can never produce NaN.
            for (uint32_t i = lane; i < (KS - nvalid) * 16u; i += 32) {
                const uint32_t row = nvalid + (i >> 4);
                *reinterpret_cast<uint4*>(vst + (row >> 2) * GPITCH + (row & 3u) * KV_ROW_BYTES +
                                          (i & 15u) * 16u) = make_uint4(0, 0, 0, 0);
            }
            __syncwarp();
        }

        // ---- S = Q K^T for 32 keys: n-block nb holds keys nb + 4*n (n = 0..7, one per group)
        float s[4][4];
#pragma unroll
        for (int nb = 0; nb < 4; nb++) {
            s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.0f;
            const uint32_t kaddr = smem_u32(kst) + (lane & 7) * GPITCH + nb * KV_ROW_BYTES + (lane >> 3) * 16;
#pragma unroll
            for (int kk = 0; kk < 4; kk++) {
                uint32_t r0, r1, r2, r3;
                ldmatrix_x4(kaddr + kk * 64, r0, r1, r2, r3);
                mma_16816(s[nb], qa[2 * kk][0], 0u, qa[2 * kk][1], 0u, r0, r1);
                mma_16816(s[nb], qa[2 * kk + 1][0], 0u, qa[2 * kk + 1][1], 0u, r2, r3);
            }
        }
        // ---- online softmax on row g (this thread: keys nb + 4*(2*t4 + {0,1}))
        float mx = -1.0e30f;
#pragma unroll
        for (int nb = 0; nb < 4; nb++) {
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const uint32_t key = nb + 4 * (2 * t4 + j);
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

        // ---- O += P V : 2 k-steps of 16 keys (the keys of n-blocks 2*k2 and 2*k2+1, same
        // permutation as P's columns), 16 n-blocks of 8 dims
#pragma unroll
        for (int k2 = 0; k2 < 2; k2++) {
            const uint32_t vaddr = smem_u32(vst) + (lane & 7) * GPITCH +
                                   (2 * k2 + ((lane >> 3) & 1)) * KV_ROW_BYTES + (lane >> 4) * 16;
#pragma unroll
            for (int jn = 0; jn < 8; jn++) {
                uint32_t r0, r1, r2, r3;
                ldmatrix_x4_trans(vaddr + jn * 32, r0, r1, r2, r3);
                mma_16816(o[2 * jn], pa[2 * k2], 0u, pa[2 * k2 + 1], 0u, r0, r1);
                mma_16816(o[2 * jn + 1], pa[2 * k2], 0u, pa[2 * k2 + 1], 0u, r2, r3);
            }
        }
        // release the stage (generic writes of a tail stage are ordered before later bulk copies)
        if (nvalid < KS || owner || (kFused && (desc.z & F_FIRST))) fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[slot]);

        if (!(desc.z & F_LAST)) continue;

        // ---- the item is complete: row sums across the quad, then output or partials
        const uint32_t b = desc.x, c = desc.y & 0xffffu, nchunks = desc.y >> 16;
        float l_tot = l_run;
        l_tot += __shfl_xor_sync(0xffffffffu, l_tot, 1);
        l_tot += __shfl_xor_sync(0xffffffffu, l_tot, 2);
        if (g >= 4) continue;
        if (nchunks == 1) {
            const float inv = rcp_approx_ftz(l_tot);
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
        } else if (OXI_IN_BOUNDS(b < p.batch && c < p.max_chunks && nchunks <= p.max_chunks, p.status)) {
            const size_t pslot = ((size_t)b * p.max_chunks + c) * NQ + head;
            float* pacc = p.partial_acc + pslot * HD;
#pragma unroll
            // partials are read back by the merge kernel a few microseconds later: ask L2 to keep
            // them while the K/V stream (evict_first) passes through
            for (int j = 0; j < 16; j++) st_global_f2_hint(pacc + 8 * j + 2 * t4, o[j][0], o[j][1], keep_policy);
            if (t4 == 0) st_global_f2_hint(p.partial_stats + pslot * 2, m_run, l_tot, keep_policy);
        }
    }
}

// Merges the partials of every row that was covered by more than one item, and
// resets the work counter for the next launch.
// grid = (B*4, E) CTAs of 4 warps: warp = one query head of one row; lane owns dims
// 4*lane .. 4*lane+3.  Loads are issued in blocks of 16 key ranges, all
// independent of the arithmetic, which runs in key-range order, so the result
// does not depend on scheduling.  A row of up to 16 key ranges (4096 keys) is one
// such block: two memory round trips, done by the CTA with blockIdx.y = 0.
// A longer row is cut into slices of 16 key ranges; slice s is summed (weights
// relative to the row's maximum) by CTA y = s mod E into a scratch slot, and the
// CTA of the row that arrives last adds the slices in slice order.  The slices
// and the order of every sum depend on the row's own length only, never on E or
// on the other rows of the batch; E only spreads a long row's loads over more
// CTAs (a 32,768-key row: 4 round trips instead of 9).
constexpr int MERGE_BLK = 16;            // key ranges per block of loads = per slice
constexpr int MERGE_SLOT = HD + 4;       // floats per slice slot: 128 sums, the weight sum, padding to 16 bytes
constexpr int MERGE_MAX_Y = 8;

template <bool kSliced>  // false: the workspace holds rows of at most 16 key ranges (no slice scratch)
__global__ void __launch_bounds__(128)
decode_merge_kernel(const DecodeParams p) {
    pdl_launch_dependents();
    const uint32_t b = blockIdx.x >> 2;
    const int lane = threadIdx.x & 31;
    const uint32_t hd = (blockIdx.x & 3u) * 4 + (threadIdx.x >> 5);
    // step inputs (not written by any kernel): fetched while the streaming kernel drains
    const uint32_t slen = p.seq_lens[b];
    const uint64_t kvp = p.paged.block_tables ? 0ull : (p.k_ptrs[b] | p.v_ptrs[b]);
    const float gate_f = p.gate ? h2f(p.gate[(size_t)b * NQ + hd]) : 0.0f;
    pdl_wait();
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *p.work_counter = 0u;
    if (slen == 0u || slen > p.max_seq_len || (kvp & 15ull) != 0ull) return;
    if (p.paged.block_tables && ((slen - 1u) >> p.paged.lbs) >= p.paged.max_blocks) return;
    const uint32_t nchunks = row_chunks(slen, p.window);
    if (nchunks <= 1) return;
    const uint32_t nslices = kSliced ? (nchunks + MERGE_BLK - 1) / MERGE_BLK : 1u;
    // CTAs that work on this row and head group: several only where that saves memory round trips
    // (one CTA: 1 + nslices, several: 3 + nslices / ny); the sums are the same either way
    const uint32_t ny = (kSliced && nslices >= 4u) ? min(gridDim.y, nslices) : 1u;
    if (blockIdx.y >= ny) return;
    const float* stats = p.partial_stats + (((size_t)b * p.max_chunks) * NQ + hd) * 2;
    const float* accs = p.partial_acc + (((size_t)b * p.max_chunks) * NQ + hd) * HD;
    float m = -1.0e30f;
    for (uint32_t cc = lane; cc < nchunks; cc += 32) m = fmaxf(m, __ldcg(stats + (size_t)cc * NQ * 2));
    constexpr int BLK = MERGE_BLK;
    float l = 0.0f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    bool have_max = false;
    const uint32_t slots_per_head = (p.max_chunks + MERGE_BLK - 1) / MERGE_BLK;
    float* slot0 = kSliced ? p.merge_acc + ((size_t)b * NQ + hd) * slots_per_head * MERGE_SLOT : nullptr;
    float l_tot = 0.0f;  // ny == 1: the slice sums are added here, in slice order, as the last CTA would
    float4 acc_tot = make_float4(0.f, 0.f, 0.f, 0.f);
    // without slices: one pass over all key ranges, block after block, sums carried across the blocks
    const uint32_t nloop = kSliced ? nslices : (nchunks + BLK - 1) / BLK;
    for (uint32_t sl = blockIdx.y; sl < nloop; sl += ny) {
        const uint32_t c0 = sl * BLK;
        float2 st[BLK];
        float4 pv[BLK];
#pragma unroll
        for (int i = 0; i < BLK; i++) {
            const uint32_t cc = min(c0 + i, nchunks - 1);  // clamped loads; weights of clamped slots are dropped
            st[i] = __ldcg(reinterpret_cast<const float2*>(stats + (size_t)cc * NQ * 2));
            pv[i] = __ldcg(reinterpret_cast<const float4*>(accs + (size_t)cc * NQ * HD) + lane);
        }
        if (!have_max) {
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
            have_max = true;
        }
        if (kSliced) {
            l = 0.0f;
            acc = make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < BLK; i++) {
            const float wgt = (c0 + i < nchunks) ? ex2_approx_ftz(st[i].x - m) : 0.0f;
            l = fmaf(wgt, st[i].y, l);
            acc.x = fmaf(wgt, pv[i].x, acc.x);
            acc.y = fmaf(wgt, pv[i].y, acc.y);
            acc.z = fmaf(wgt, pv[i].z, acc.z);
            acc.w = fmaf(wgt, pv[i].w, acc.w);
        }
        if (ny > 1u) {
            float* slot = slot0 + (size_t)sl * MERGE_SLOT;
            __stcg(reinterpret_cast<float4*>(slot) + lane, acc);
            if (lane == 0) __stcg(slot + HD, l);
        } else if (nslices > 1u) {
            l_tot += l;
            acc_tot.x += acc.x;
            acc_tot.y += acc.y;
            acc_tot.z += acc.z;
            acc_tot.w += acc.w;
        }
    }
    if (ny == 1u && nslices > 1u) {
        l = l_tot;
        acc = acc_tot;
    }
    if (ny > 1u) {
        // the CTA of this (row, head group) that arrives last adds the slices in slice order
        __shared__ uint32_t s_last;
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            uint32_t* cnt = p.merge_count + blockIdx.x;
            const bool last = atomicAdd(cnt, 1u) == ny - 1u;
            if (last) *cnt = 0u;  // ready for the next launch
            s_last = last ? 1u : 0u;
        }
        __syncthreads();
        if (!s_last) return;
        __threadfence();
        l = 0.0f;
        acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t s0 = 0; s0 < nslices; s0 += 8) {
            float4 sv[8];
            float sw[8];
#pragma unroll
            for (uint32_t u = 0; u < 8; u++) {
                const float* slot = slot0 + (size_t)min(s0 + u, nslices - 1u) * MERGE_SLOT;
                sv[u] = __ldcg(reinterpret_cast<const float4*>(slot) + lane);
                sw[u] = __ldcg(slot + HD);
            }
#pragma unroll
            for (uint32_t u = 0; u < 8; u++) {
                if (s0 + u < nslices) {
                    l += sw[u];
                    acc.x += sv[u].x;
                    acc.y += sv[u].y;
                    acc.z += sv[u].z;
                    acc.w += sv[u].w;
                }
            }
        }
    }
    const float inv = rcp_approx_ftz(l);
    uint16_t h[4] = {f2h(__fmul_rn(acc.x, inv)), f2h(__fmul_rn(acc.y, inv)),
                     f2h(__fmul_rn(acc.z, inv)), f2h(__fmul_rn(acc.w, inv))};
    if (p.gate) {
        const float sig = sigmoid_ref(gate_f);
#pragma unroll
        for (int i = 0; i < 4; i++) h[i] = f2h(__fmul_rn(h2f(h[i]), sig));
    }
    uint2 packed = make_uint2((uint32_t)h[0] | ((uint32_t)h[1] << 16),
                              (uint32_t)h[2] | ((uint32_t)h[3] << 16));
    *reinterpret_cast<uint2*>(p.ctx_out + ((size_t)b * NQ + hd) * HD + 4 * lane) = packed;
}

// CTAs per (row, head group) of the merge: enough to spread the slices of long rows, few enough
// that the CTAs without work (short rows) do not cost a second wave.
static dim3 merge_grid(const DecodeWorkspace& ws, uint32_t batch) {
    const uint32_t slices = (ws.max_chunks + MERGE_BLK - 1) / MERGE_BLK;
    uint32_t y = slices >= 4u ? slices : 1u;  // rows of fewer than 4 slices stay with one CTA
#ifndef OXI_MERGE_CTAS_PER_SM
#define OXI_MERGE_CTAS_PER_SM 16
#endif
    const uint32_t cap = (uint32_t)(OXI_MERGE_CTAS_PER_SM * ws.num_sms) / (batch * NKV);  // about one resident wave of 128-thread CTAs
    if (y > cap) y = cap;
    if (y > (uint32_t)MERGE_MAX_Y) y = MERGE_MAX_Y;
    if (y < 1u) y = 1u;
    return dim3(batch * NKV, y);
}

static cudaError_t launch_merge(cudaStream_t stream, const DecodeWorkspace& ws, uint32_t batch, const DecodeParams& p) {
    if (ws.merge_acc) return launch_pdl(decode_merge_kernel<true>, merge_grid(ws, batch), dim3(128), 0, stream, p);
    return launch_pdl(decode_merge_kernel<false>, dim3(batch * NKV), dim3(128), 0, stream, p);
}

size_t decode_merge_scratch_bytes(uint32_t max_batch, uint32_t max_chunks) {
    const size_t slices = (max_chunks + MERGE_BLK - 1) / MERGE_BLK;
    return slices > 1 ? (size_t)max_batch * NQ * slices * MERGE_SLOT * sizeof(float) : 0;
}

uint32_t decode_chunk_keys() { return dec::CHUNK; }
uint32_t decode_max_rows() { return dec::MAX_ROWS; }

cudaError_t decode_attn_init() {
    cudaError_t e = cudaFuncSetAttribute(decode_attn_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)dec::SMEM_BYTES);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(decode_attn_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dec::SMEM_BYTES);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(decode_attn_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dec::SMEM_BYTES);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(decode_attn_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dec::SMEM_BYTES);
    return e;
}

static DecodeParams make_params(const DecodeWorkspace& ws, void* ctx_out, const void* q, const void* gate,
                                const uint64_t* k_ptrs, const uint64_t* v_ptrs, const uint32_t* seq_lens,
                                uint32_t batch, uint32_t window) {
    DecodeParams p = {};
    p.ctx_out = (uint16_t*)ctx_out;
    p.q = (const uint16_t*)q;
    p.gate = (const uint16_t*)gate;
    p.k_ptrs = k_ptrs;
    p.v_ptrs = v_ptrs;
    p.seq_lens = seq_lens;
    p.partial_acc = ws.partial_acc;
    p.partial_stats = ws.partial_stats;
    p.work_counter = ws.work_counter;
    p.status = ws.status;
    p.merge_acc = ws.merge_acc;
    p.merge_count = ws.merge_count;
    p.batch = batch;
    p.window = window;
    p.max_chunks = ws.max_chunks;
    p.max_seq_len = ws.max_seq_len;
    p.fault = ws.fault;
    return p;
}

cudaError_t launch_decode_attn(cudaStream_t stream, const DecodeWorkspace& ws, void* ctx_out,
                               const void* q, const void* gate, const uint64_t* k_ptrs,
                               const uint64_t* v_ptrs, const uint32_t* seq_lens, uint32_t batch,
                               uint32_t window) {
    const DecodeParams p = make_params(ws, ctx_out, q, gate, k_ptrs, v_ptrs, seq_lens, batch, window);
    cudaError_t e = launch_pdl(decode_attn_kernel<false, false>, dim3(ws.num_sms), dim3(dec::THREADS), dec::SMEM_BYTES,
                               stream, p);
    if (e != cudaSuccess) return e;
    return launch_merge(stream, ws, batch, p);
}

cudaError_t launch_append_decode(cudaStream_t stream, const DecodeWorkspace& ws, void* ctx_out, const void* q_io,
                                 const void* k_in, const void* v_in, const void* gate, const void* q_norm_w,
                                 const void* k_norm_w, const void* cos_t, const void* sin_t,
                                 const uint32_t* seq_lens, const uint64_t* k_ptrs, const uint64_t* v_ptrs,
                                 uint32_t batch, uint32_t window, float eps) {
    DecodeParams p = make_params(ws, ctx_out, q_io, gate, k_ptrs, v_ptrs, seq_lens, batch, window);
    p.k_in = (const uint16_t*)k_in;
    p.v_in = (const uint16_t*)v_in;
    p.q_norm_w = (const uint16_t*)q_norm_w;
    p.k_norm_w = (const uint16_t*)k_norm_w;
    p.cos_t = (const uint16_t*)cos_t;
    p.sin_t = (const uint16_t*)sin_t;
    p.eps = eps;
    cudaError_t e = launch_pdl(decode_attn_kernel<true, false>, dim3(ws.num_sms), dim3(dec::THREADS), dec::SMEM_BYTES,
                               stream, p);
    if (e != cudaSuccess) return e;
    return launch_merge(stream, ws, batch, p);
}

cudaError_t launch_decode_attn_paged(cudaStream_t stream, const DecodeWorkspace& ws, void* ctx_out, const void* q,
                                     const void* gate, const PagedMap& pm, const uint32_t* seq_lens, uint32_t batch,
                                     uint32_t window) {
    DecodeParams p = make_params(ws, ctx_out, q, gate, nullptr, nullptr, seq_lens, batch, window);
    p.paged = pm;
    cudaError_t e = launch_pdl(decode_attn_kernel<false, true>, dim3(ws.num_sms), dim3(dec::THREADS), dec::SMEM_BYTES,
                               stream, p);
    if (e != cudaSuccess) return e;
    return launch_merge(stream, ws, batch, p);
}

cudaError_t launch_append_decode_paged(cudaStream_t stream, const DecodeWorkspace& ws, void* ctx_out, const void* q_io,
                                       const void* k_in, const void* v_in, const void* gate, const void* q_norm_w,
                                       const void* k_norm_w, const void* cos_t, const void* sin_t,
                                       const uint32_t* seq_lens, const PagedMap& pm, uint32_t batch, uint32_t window,
                                       float eps) {
    DecodeParams p = make_params(ws, ctx_out, q_io, gate, nullptr, nullptr, seq_lens, batch, window);
    p.paged = pm;
    p.k_in = (const uint16_t*)k_in;
    p.v_in = (const uint16_t*)v_in;
    p.q_norm_w = (const uint16_t*)q_norm_w;
    p.k_norm_w = (const uint16_t*)k_norm_w;
    p.cos_t = (const uint16_t*)cos_t;
    p.sin_t = (const uint16_t*)sin_t;
    p.eps = eps;
    cudaError_t e = launch_pdl(decode_attn_kernel<true, true>, dim3(ws.num_sms), dim3(dec::THREADS), dec::SMEM_BYTES,
                               stream, p);
    if (e != cudaSuccess) return e;
    return launch_merge(stream, ws, batch, p);
}

}  // namespace oxi

// ---------------------------------------------------------------------------
// Decode attention for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc at the point where they
// need attention: a plugin running inside someone else's memory budget, a
// callback that executes while the application's allocator is locked, a
// process that handed all device memory to its own pool at start-up.  They
// also cannot create an oxi_handle, because oxi_create allocates.  For them the
// split-KV partials, the work counter and the status word live in the array
// below, which is part of the library image: every GPU that loads liboxi_kv
// holds these ~2.1 MB from module load until the process exits.
namespace oxi {
namespace nalloc {
constexpr uint32_t MAX_ROWS = OXI_STATIC_MAX_BATCH;
constexpr uint32_t MAX_CHUNKS = (OXI_STATIC_MAX_SEQ_LEN + dec::CHUNK - 1) / dec::CHUNK;
constexpr size_t CTRL_BYTES = 256;  // status word at +0, work counter at +128
constexpr size_t ACC_BYTES = (size_t)MAX_ROWS * MAX_CHUNKS * NQ * HD * sizeof(float);
constexpr size_t STATS_BYTES = (size_t)MAX_ROWS * MAX_CHUNKS * NQ * 2 * sizeof(float);
constexpr size_t TOTAL_BYTES = CTRL_BYTES + ACC_BYTES + STATS_BYTES;
constexpr int MAX_DEVICES = 64;

struct PerDevice {
    bool ready = false;
    unsigned char* base = nullptr;  // DEVICE address of g_scratch on that device
    int num_sms = 0;
};
}  // namespace nalloc
}  // namespace oxi

// In host code this name is only a stand-in for the symbol; the device address is obtained
// with cudaGetSymbolAddress below, once per device, and that address is what kernels receive.
static __device__ __align__(256) unsigned char g_scratch[oxi::nalloc::TOTAL_BYTES];

static oxi::nalloc::PerDevice g_nalloc_dev[oxi::nalloc::MAX_DEVICES];
static std::mutex g_nalloc_mutex;

extern "C" int32_t oxi_decode_attn_static(void* stream, void* ctx_out, const void* q, const void* gate,
                                          const uint64_t* k_ptrs, const uint64_t* v_ptrs,
                                          const uint32_t* seq_lens, uint32_t batch,
                                          uint32_t max_seq_len, uint32_t window) {
    using namespace oxi;
    if (!ctx_out || !q || !k_ptrs || !v_ptrs || !seq_lens) return OXI_ERR_NULL;
    if (batch == 0 || batch > nalloc::MAX_ROWS) return OXI_ERR_BATCH;
    if (max_seq_len == 0 || max_seq_len > OXI_STATIC_MAX_SEQ_LEN) return OXI_ERR_ARG;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int32_t)e;
    if (dev < 0 || dev >= nalloc::MAX_DEVICES) return OXI_ERR_NO_DEVICE;
    nalloc::PerDevice& pd = g_nalloc_dev[dev];
    {
        // First call on this device: resolve the scratch array's device address and size the
        // kernel's shared memory.  Neither call allocates; both must happen outside stream capture.
        std::lock_guard<std::mutex> lock(g_nalloc_mutex);
        if (!pd.ready) {
            void* ptr = nullptr;
            e = cudaGetSymbolAddress(&ptr, g_scratch);
            if (e != cudaSuccess) return (int32_t)e;
            int sms = 0, major = 0;
            e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            if (e == cudaSuccess) e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
            if (e != cudaSuccess) return (int32_t)e;
            if (major != 10) return OXI_ERR_NO_DEVICE;
            e = decode_attn_init();
            if (e != cudaSuccess) return (int32_t)e;
            pd.base = static_cast<unsigned char*>(ptr);
            pd.num_sms = sms;
            pd.ready = true;
        }
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // The array keeps whatever the previous call left.  The work counter must start at zero; the
    // status word is left alone, so bits raised by earlier calls stay until
    // oxi_static_device_status reads and clears them.
    e = cudaMemsetAsync(pd.base + 128, 0, 128, s);
    if (e != cudaSuccess) return (int32_t)e;
    DecodeWorkspace ws{};  // no slice scratch: rows are at most 16 key ranges long here
    ws.status = reinterpret_cast<uint32_t*>(pd.base);
    ws.work_counter = reinterpret_cast<uint32_t*>(pd.base + 128);
    ws.partial_acc = reinterpret_cast<float*>(pd.base + nalloc::CTRL_BYTES);
    ws.partial_stats = reinterpret_cast<float*>(pd.base + nalloc::CTRL_BYTES + nalloc::ACC_BYTES);
    ws.max_chunks = nalloc::MAX_CHUNKS;
    ws.max_seq_len = max_seq_len;
    ws.num_sms = pd.num_sms;
    e = launch_decode_attn(s, ws, ctx_out, q, gate, k_ptrs, v_ptrs, seq_lens, batch, window);
    return (int32_t)e;
}

// Reads and clears the status word of the allocation-free path on the current device
// (synchronises `stream`; allocates nothing).  Before the first oxi_decode_attn_static call on a
// device nothing can have been raised: the word reads as zero.
extern "C" int32_t oxi_static_device_status(void* stream, uint32_t* bits_out) {
    using namespace oxi;
    if (!bits_out) return OXI_ERR_NULL;
    *bits_out = 0u;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int32_t)e;
    if (dev < 0 || dev >= nalloc::MAX_DEVICES) return OXI_ERR_NO_DEVICE;
    unsigned char* base = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_nalloc_mutex);
        if (!g_nalloc_dev[dev].ready) return OXI_OK;
        base = g_nalloc_dev[dev].base;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    uint32_t bits = 0;
    e = cudaMemcpyAsync(&bits, base, 4, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaMemsetAsync(base, 0, 4, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return (int32_t)e;
    *bits_out = bits;
    return OXI_OK;
}
