// The GEMM on either side of the pointer-table path, with the path's first operator as its epilogue.
//
// Replaces the four projection GEMMs in front of the path - q_proj, k_proj, v_proj, gate_proj, each
// lt.gemm(out_features, 2048, rows, W, x, y) = cuBLASLt f16 x f16 -> f32 -> f16
// (batch_engine.rs:914-926) - together with the six launches that consume them (Q/K RMSNorm, RoPE,
// KV copy: batched_attn.rs:13-287, launched at batch_engine.rs:941-1014): one kernel computes
// [rows][2048] x [2048][2048 + 512 + 512 + 16] on the tensor cores and its epilogue normalises and rotates
// the q and k heads, writes K and V straight into the cache rows named by the pointer tables
// (k_ptrs[b] + pos * 1024) and q / gate for the decode kernel.  The projected q, k, v never make a
// round trip through HBM.  The plain mode (no epilogue arithmetic) is the same GEMM for o_proj on the
// far side of the path (batch_engine.rs:1241-1245).
//
// Tile = 128 rows (tokens) x 128 output features = exactly one head of all 128 rows: tcgen05.mma
// M = 128, N = 128, K = 16 per instruction (kind::f16, f32 accumulate), the accumulator [128][128] f32
// in 128 columns of tensor memory, operands A = x tile and B = W tile (both K-major, 64 k-elements =
// one 128-byte swizzle span per row) brought in by TMA tile copies (no multicast) through a ring of
// shared-memory stages that complete on mbarriers.  Warp 0 issues the copies, warp 1 the MMAs (one
// elected lane), the other warps run the epilogue.  Two kernels:
//   * proj_gemm_splitk_kernel (rows <= 256, the decode shape): a cluster of four CTAs per tile, each
//     a quarter of k, partial accumulators exchanged through distributed shared memory; four threads
//     finish a row's head.  8.9 us at 128 rows, where one CTA per tile needed 15.1 us (it has to pull
//     1 MB through one SM's port while 123 SMs idle) and a split of k that met in an L2 workspace
//     16-18 us.
//   * proj_gemm_pair_kernel (larger waves): persistent CTA pairs on 256 x 256 tiles (tcgen05.mma.cta_group::2),
//     two accumulators per CTA, eight epilogue warps (two threads per row; a thread serves both heads of the tile).
//
// Bit parity.  The projections are rounded to f16 exactly as the reference's GEMM output is, and
// the epilogue applies the append kernel's arithmetic to those f16 values: the RMSNorm sum is formed
// in the reference's order (32 partial sums over dims l, l+32, l+64, l+96 with fma, then the
// shfl.down tree 16, 8, 4, 2, 1 - here as the same additions on 32 registers of a thread),
// div.approx / rsqrt.approx, two separate multiplies, f16 round trip, then mul + fma for RoPE.  Given
// the same f16 projections, q and the cache rows are the bytes oxi_append writes.
#include <cuda.h>  // CUtensorMap and its enums only

#include "../../include/oxi_kv.h"
#include "common.cuh"
#include "kernels.h"
#include "tc5.cuh"

namespace oxi {

namespace pg {
constexpr int BM = 128, BN = 128, BK = 64;      // tile rows (tokens), tile columns (features), k-block
constexpr int KDIM = HIDDEN;                    // 2048 input features
constexpr int NKB = KDIM / BK;                  // 32 k-blocks
constexpr int NS = 3;                           // ring stages: 3 x 32 KB, two CTAs per SM
constexpr int TILE_BYTES = BM * BK * 2;         // 16 KB per operand tile
constexpr int STAGE_BYTES = 2 * TILE_BYTES;
constexpr int THREADS = 192;                    // TMA warp, MMA warp, 4 epilogue warps
constexpr size_t SMEM_BYTES = 1024 + (size_t)NS * STAGE_BYTES;
constexpr uint32_t TMEM_COLS = 128;
constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);  // f32 += f16 x f16, K-major A and B
constexpr int N_QKVG = 2048 + 512 + 512 + 16;   // q | k | v | gate output features
constexpr int TILES_QKVG = 16 + 4 + 4 + 1;
}  // namespace pg

struct ProjMaps {
    TmaDesc x;      // [rows][2048] f16, box {64, 128}, 128-byte swizzle
    TmaDesc w[4];   // qkvg mode: q [2048][2048], k [512][2048], v [512][2048], gate [16][2048]; plain mode: w[0]
};

struct ProjParams {
    uint32_t rows;
    uint32_t out_features;     // plain mode
    uint16_t* y;               // plain mode: [rows][out_features]
    uint16_t* q_out;           // [rows][16][128] normalised + rotated q
    uint16_t* gate_out;        // [rows][16]
    uint16_t* raw_out;         // nullable: [rows][3088] the f16 projections before the epilogue arithmetic
    const uint16_t* q_norm_w;
    const uint16_t* k_norm_w;
    const uint16_t* cos_t;
    const uint16_t* sin_t;
    const uint32_t* pos_ids;
    const uint64_t* k_ptrs;
    const uint64_t* v_ptrs;
    uint32_t* status;
    float eps;
    uint32_t wait_us;          // limit of every pipeline wait of this launch (a second unless a test armed a fault)
    uint32_t skip_plus1;       // test support: CTA 0 issues no copies for its (skip_plus1 - 1)-th k-block; 0 = off
};

// this thread's TMEM lane, 16 consecutive 32-bit columns
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// 16 accumulator columns -> the f16 the GEMM outputs (bit patterns) and their f32 values
__device__ __forceinline__ void round16(const uint32_t (&acc)[16], uint16_t (&h)[16], float (&f)[16]) {
#pragma unroll
    for (int i = 0; i < 16; i++) {
        h[i] = f2h(__uint_as_float(acc[i]));
        f[i] = h2f(h[i]);
    }
}
// 32 bytes per thread in one 256-bit access where the address allows it (half the instructions and half the L1
// wavefronts of two 16-byte accesses: a thread of the epilogue works on its own row, so every lane touches another line)
__device__ __forceinline__ void st_pairs(uint16_t* dst, const uint32_t (&w)[8]) {  // 16 f16 = 32 bytes, 16-byte aligned
    if ((reinterpret_cast<uintptr_t>(dst) & 31u) == 0u) {
        asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]),
                     "r"(w[5]), "r"(w[6]), "r"(w[7])
                     : "memory");
    } else {
        reinterpret_cast<uint4*>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
        reinterpret_cast<uint4*>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
    }
}
__device__ __forceinline__ void store16(uint16_t* dst, const uint16_t (&h)[16]) {  // 32 bytes, 16-byte aligned
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; i++) w[i] = h[2 * i] | ((uint32_t)h[2 * i + 1] << 16);
    st_pairs(dst, w);
}
__device__ __forceinline__ void ld_pairs(const uint16_t* src, uint32_t (&w)[8]) {  // read-only data; 16 f16 = 32 bytes, 16-byte aligned
    if ((reinterpret_cast<uintptr_t>(src) & 31u) == 0u) {
        asm volatile("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
                     : "l"(src));
    } else {
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(src)), b = __ldg(reinterpret_cast<const uint4*>(src) + 1);
        w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
        w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
    }
}

// ---------------------------------------------------------------------------------------------------
// The decode shape (rows <= 256: one or two row tiles).  One CTA per (row tile, head) has to pull 1 MB of
// operands through one SM's port (~7 us for 25 CTAs while 123 SMs idle), so the k dimension is cut into
// four parts computed by the four CTAs of a thread-block cluster, which meet in shared memory:
//   1. CTA c runs the main loop over k-blocks [8c, 8c + 8) into its own accumulator; meanwhile its epilogue
//      threads fetch the table entries and rotary values of the rows they will finish;
//   2. cluster barrier: every main loop of the cluster is over, so every ring is free to receive;
//   3. the four epilogue warps push the f32 accumulator: the 32 rows of TMEM lane quarter q go to CTA q, slot c
//      of its receive area (the ring's bytes), with 16-byte remote stores laid out so that a warp's stores and
//      the later loads are conflict-free (remote stores need no round trip; fetching from the peers instead
//      measured 0.5 us slower, a cluster of eight 3 us slower);
//   4. cluster barrier; CTA c finishes rows [32c, 32c + 32) of the tile from its own shared memory: thread
//      (warp j, lane t) adds the four parts of 32 of row t's 128 columns in k order - the dims l, l + 32, l + 64,
//      l + 96 for l in [8j, 8j + 8), i.e. what lanes 8j .. 8j + 7 of the reference's warp own, so the row's
//      four threads form the RMSNorm partial sums with the reference's fma chains, exchange the 32 partials
//      through shared memory, and each runs the reference's shfl.down tree on them; both members of every RoPE
//      pair (d, d + 64) sit in the same thread.  After the second barrier a CTA touches only its own shared
//      memory, so it may leave without waiting for its peers.
// The barriers are hardware cluster barriers reached by every thread on every path (all other waits in the
// kernel are bounded and fall through), so they cannot be left waiting; a CTA that gave up a wait says so
// in a flag pushed to its peers, and nobody writes results.
// Where the time goes at 128 rows (globaltimer stamps in one CTA, ns): set-up 350, main loop 2500, barrier 300,
// push + barrier 1650, adding the parts 350, RMSNorm + RoPE + stores 1050 (q head; gate 250).
namespace pgs {
using pg::BM; using pg::BN; using pg::BK; using pg::NKB; using pg::NS; using pg::TILE_BYTES; using pg::STAGE_BYTES;
using pg::THREADS; using pg::SMEM_BYTES; using pg::TMEM_COLS; using pg::IDESC;
constexpr int KS = 4;                       // CTAs per cluster = parts of k = TMEM lane quarters of the tile
constexpr int KB_PER = NKB / KS;            // 8 k-blocks per CTA
static_assert(KS == 4 && BM == 128, "CTA c of the cluster finishes the 32 rows of lane quarter c");
static_assert((size_t)BM * BN * 4 <= (size_t)NS * STAGE_BYTES, "the exported accumulator reuses the ring");
}  // namespace pgs

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {  // every thread of every CTA of the cluster
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t dsmem_addr(uint32_t local_smem_addr, uint32_t cta) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(cta));
    return r;
}
// 8 f16 bit patterns -> one 16-byte store
__device__ __forceinline__ void store8(uint16_t* dst, const uint16_t* h) {
    *reinterpret_cast<uint4*>(dst) = make_uint4(h[0] | ((uint32_t)h[1] << 16), h[2] | ((uint32_t)h[3] << 16),
                                                 h[4] | ((uint32_t)h[5] << 16), h[6] | ((uint32_t)h[7] << 16));
}

// Finishes 32 columns of one row of a head: v[g][i] = accumulator of dim 32g + 8j + i, i.e. the dims owned by lanes
// 8j .. 8j + 7 of the reference's warp.  Called by all 128 epilogue threads of the CTA (the q/k branch meets in a named
// barrier); t = lane = row inside the CTA's 32 rows; s_part = [32 reference lanes][32 rows] f32 in shared memory.
// What the finishing thread of a row needs from global memory besides the accumulators: fetched while the cluster
// exchanges the partial sums (the table entry, then the rotary values it leads to, are two dependent round trips).
struct RowTables {
    uint32_t pos;
    uint64_t kvp;
    uint4 cs[4], sn[4];  // [2 * pair + 0 / 1]: cos / sin of dims [dl, dl + 8) and 64 + [dl, dl + 8), dl = 32 * pair + 8j
    bool live;
};
template <bool kQkvg>
__device__ __forceinline__ RowTables proj_fetch_row_tables(uint32_t j, uint32_t n_tile, uint32_t row, bool live, const ProjParams& p) {
    RowTables rt;
    rt.pos = 0;
    rt.kvp = 0;
    if (!OXI_IN_BOUNDS(!live || (row < p.rows && (kQkvg ? n_tile <= 24u : n_tile * 128u < p.out_features)), p.status)) live = false;
    rt.live = live;
    if (kQkvg && live && n_tile < 24u) {
        rt.pos = p.pos_ids[row];
        if (n_tile >= 16u && n_tile < 20u) rt.kvp = p.k_ptrs[row];
        if (n_tile >= 20u) rt.kvp = p.v_ptrs[row];
        if (n_tile < 20u) {
            const uint16_t* cs = p.cos_t + (size_t)rt.pos * HD;
            const uint16_t* sn = p.sin_t + (size_t)rt.pos * HD;
#pragma unroll
            for (int pr = 0; pr < 2; pr++) {
                const uint32_t dl = 32u * pr + 8u * j, dh = dl + 64u;
                rt.cs[2 * pr] = __ldg(reinterpret_cast<const uint4*>(cs + dl));
                rt.cs[2 * pr + 1] = __ldg(reinterpret_cast<const uint4*>(cs + dh));
                rt.sn[2 * pr] = __ldg(reinterpret_cast<const uint4*>(sn + dl));
                rt.sn[2 * pr + 1] = __ldg(reinterpret_cast<const uint4*>(sn + dh));
            }
        }
    }
    return rt;
}

template <bool kQkvg>
__device__ __forceinline__ void proj_finish_row(const float (&v)[4][8], uint32_t j, uint32_t t, uint32_t n_tile, uint32_t row,
                                                const RowTables& rt, const ProjParams& p, const uint16_t* s_w, float* s_part) {
    constexpr uint32_t N_QKVG = pg::N_QKVG;
    const bool live = rt.live;
    uint16_t h[4][8];
    float f[4][8];
#pragma unroll
    for (int g = 0; g < 4; g++)
#pragma unroll
        for (int i = 0; i < 8; i++) {
            h[g][i] = f2h(v[g][i]);
            f[g][i] = h2f(h[g][i]);
        }
    if (!kQkvg) {
        // ---- plain linear layer
        if (!live) return;
#pragma unroll
        for (int g = 0; g < 4; g++) {
            const uint32_t n0 = n_tile * 128u + 32u * g + 8u * j;
            if (n0 >= p.out_features) continue;
            uint16_t* dst = p.y + (size_t)row * p.out_features + n0;
            if (n0 + 8u <= p.out_features && (p.out_features & 7u) == 0u) {
                store8(dst, h[g]);
            } else {
                for (uint32_t i = 0; i < 8u && n0 + i < p.out_features; i++) dst[i] = h[g][i];
            }
        }
        return;
    }
    if (n_tile == 24u) {
        // ---- gate: 16 features, dims 8j .. 8j + 7 of threads j = 0, 1
        if (live && j < 2u) {
            store8(p.gate_out + (size_t)row * NQ + 8u * j, h[0]);
            if (p.raw_out) store8(p.raw_out + (size_t)row * N_QKVG + 3072u + 8u * j, h[0]);
        }
        return;
    }
    const uint32_t pos = rt.pos;
    const uint64_t kvp = rt.kvp;
    if (n_tile >= 20u) {
        // ---- v head: the f16 projection is the cache row
        const uint32_t kvh = n_tile - 20u;
        const bool aligned = (kvp & 15ull) == 0ull;
        if (live && !aligned && kvh == 0u && j == 0u) atomicOr(p.status, DEV_MISALIGNED_PTR);
        if (!live) return;
        uint16_t* dst = reinterpret_cast<uint16_t*>(kvp + (size_t)pos * KV_ROW_BYTES) + kvh * HD;
#pragma unroll
        for (int g = 0; g < 4; g++) {
            const uint32_t d0 = 32u * g + 8u * j;
            if (aligned) store8(dst + d0, h[g]);
            if (p.raw_out) store8(p.raw_out + (size_t)row * N_QKVG + 2560u + kvh * HD + d0, h[g]);
        }
        return;
    }
    // ---- q or k head: RMSNorm + RoPE on the f16 projections, the append kernel's arithmetic
    const bool is_k = n_tile >= 16u;
    const uint32_t head = is_k ? n_tile - 16u : n_tile;
    const uint16_t* wn = s_w + (is_k ? HD : 0);
    const bool aligned = !is_k || (kvp & 15ull) == 0ull;
    if (live && !aligned && head == 0u && j == 0u) atomicOr(p.status, DEV_MISALIGNED_PTR);
    if (live && p.raw_out) {
#pragma unroll
        for (int g = 0; g < 4; g++)
            store8(p.raw_out + (size_t)row * N_QKVG + (is_k ? 2048u : 0u) + head * HD + 32u * g + 8u * j, h[g]);
    }
    // the partial sums of reference lanes l = 8j + i: dims l, l + 32, l + 64, l + 96 in that order, fma
#pragma unroll
    for (int i = 0; i < 8; i++) {
        float pp = __fmaf_rn(f[0][i], f[0][i], 0.0f);
        pp = __fmaf_rn(f[1][i], f[1][i], pp);
        pp = __fmaf_rn(f[2][i], f[2][i], pp);
        pp = __fmaf_rn(f[3][i], f[3][i], pp);
        s_part[(8u * j + i) * 32u + t] = pp;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps
    float partial[32];
#pragma unroll
    for (int l = 0; l < 32; l++) partial[l] = s_part[l * 32 + t];
    // the shfl.down tree of the reference on one thread's registers: lane 0's value
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1)
#pragma unroll
        for (int l = 0; l < off; l++) partial[l] = __fadd_rn(partial[l], partial[l + off]);
    float mean = div_approx_ftz(partial[0], 128.0f);
    mean = __fadd_rn(mean, p.eps);
    const float r = rsqrt_approx_ftz(mean);
    if (!live) return;
    uint16_t* dst = is_k ? reinterpret_cast<uint16_t*>(kvp + (size_t)pos * KV_ROW_BYTES) + head * HD
                         : p.q_out + ((size_t)row * NQ + head) * HD;
#pragma unroll
    for (int pr = 0; pr < 2; pr++) {  // dims [dl, dl + 8) pair with dims 64 + [dl, dl + 8)
        const uint32_t dl = 32u * pr + 8u * j, dh = dl + 64u;
        const uint4 clo = rt.cs[2 * pr], chi = rt.cs[2 * pr + 1];
        const uint4 slo = rt.sn[2 * pr], shi = rt.sn[2 * pr + 1];
        const uint32_t cl[4] = {clo.x, clo.y, clo.z, clo.w}, ch[4] = {chi.x, chi.y, chi.z, chi.w};
        const uint32_t sl[4] = {slo.x, slo.y, slo.z, slo.w}, sh4[4] = {shi.x, shi.y, shi.z, shi.w};
        uint16_t olo[8], ohi[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float xlo = f[pr][i], xhi = f[pr + 2][i];
            // y = f16((x * r) * w): two separate multiplies, then the f16 round trip
            const float ylo = h2f(f2h(__fmul_rn(__fmul_rn(xlo, r), h2f(wn[dl + i]))));
            const float yhi = h2f(f2h(__fmul_rn(__fmul_rn(xhi, r), h2f(wn[dh + i]))));
            const int wd = i >> 1, sh = (i & 1) * 16;
            const float c_lo = h2f((uint16_t)(cl[wd] >> sh)), c_hi = h2f((uint16_t)(ch[wd] >> sh));
            const float s_lo = h2f((uint16_t)(sl[wd] >> sh)), s_hi = h2f((uint16_t)(sh4[wd] >> sh));
            // rotate-half: out[d] = fma(-y[d+64], sin[d], y[d]*cos[d]);  out[d+64] = fma(y[d], sin[d+64], y[d+64]*cos[d+64])
            olo[i] = f2h(__fmaf_rn(-yhi, s_lo, __fmul_rn(ylo, c_lo)));
            ohi[i] = f2h(__fmaf_rn(ylo, s_hi, __fmul_rn(yhi, c_hi)));
        }
        if (aligned) {
            store8(dst + dl, olo);
            store8(dst + dh, ohi);
        }
    }
}

template <bool kQkvg>
__global__ void __cluster_dims__(pgs::KS, 1, 1) __launch_bounds__(pgs::THREADS, 2)
proj_gemm_splitk_kernel(const __grid_constant__ ProjMaps maps, const ProjParams p) {
    using namespace pgs;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[NS], bar_empty[NS], bar_acc;
    __shared__ uint32_t s_tmem, s_abort;
    __shared__ __align__(16) uint16_t s_w[2 * HD];  // q and k norm weights
    __shared__ float s_part[32 * 32];       // RMSNorm partials: [reference lane][row of this CTA]
    __shared__ uint32_t s_peer_abort[pgs::KS];  // written by the peers: did CTA cc give up a wait

    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;  // 1024-byte aligned tiles (128-byte swizzle)
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp_u = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const uint32_t crank = cluster_ctarank();                      // which part of k, and which 32 rows to finish
    const uint32_t n_tile = blockIdx.x / KS, m_tile = blockIdx.y;

    pdl_launch_dependents();
    if (warp_u == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        for (int s = 0; s < NS; s++) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 1);
        }
        mbar_init(&bar_acc, 1);
        s_abort = 0u;
        mbar_fence_init();
    }
    if (kQkvg && tid >= 64) {
        const int i = tid - 64;  // 128 threads: both weight vectors (not written by any kernel)
        s_w[i] = p.q_norm_w[i];
        s_w[HD + i] = p.k_norm_w[i];
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;

    uint32_t wsel = 0, wrow = n_tile * BN;
    if (kQkvg) {
        if (n_tile >= 24) { wsel = 3; wrow = 0; }
        else if (n_tile >= 20) { wsel = 2; wrow = (n_tile - 20) * BN; }
        else if (n_tile >= 16) { wsel = 1; wrow = (n_tile - 16) * BN; }
    }
    const uint32_t kb0 = crank * KB_PER;
    bool acc_ok = true;  // epilogue warps: this CTA's accumulator completed
    RowTables rt;
    rt.live = false;

    if (warp_u == 0) {
        // ===================== TMA producer: this CTA's k-blocks =====================
        pdl_wait();  // x is written by the kernel before this one
        bool ok = true;
        uint32_t issued = 0;
        for (uint32_t kb = 0; kb < (uint32_t)KB_PER && ok; kb++, issued++) {
            const uint32_t s = kb % NS;
            if (kb >= (uint32_t)NS && !mbar_wait_bounded(&bar_empty[s], ((kb / NS) & 1u) ^ 1u, &s_abort, p.wait_us)) {
                ok = false;
                break;
            }
            const bool withheld = p.skip_plus1 == kb + 1u && blockIdx.x == 0u && blockIdx.y == 0u;  // test support
            if (lane == 0 && !withheld) {
                mbar_arrive_expect_tx(&bar_full[s], (uint32_t)STAGE_BYTES);
                tma_load_box(sbase + s * STAGE_BYTES, &maps.x, (kb0 + kb) * BK, m_tile * BM, &bar_full[s]);
                tma_load_box(sbase + s * STAGE_BYTES + TILE_BYTES, &maps.w[wsel], (kb0 + kb) * BK, wrow, &bar_full[s]);
            }
            __syncwarp();
        }
        if (!ok) {
            if (lane == 0) atomicOr(p.status, DEV_WAIT_TIMEOUT);
            for (uint32_t k = issued > (uint32_t)NS ? issued - NS : 0; k < issued; ++k)
                mbar_wait_drain(&bar_full[k % NS], (k / NS) & 1u, p.wait_us);
        }
    } else if (warp_u == 1) {
        // ===================== MMA issuer =====================
        bool ok = true;
        for (uint32_t kb = 0; kb < (uint32_t)KB_PER; kb++) {
            const uint32_t s = kb % NS;
            ok = __all_sync(0xffffffffu, ok && mbar_wait_bounded(&bar_full[s], (kb / NS) & 1u, &s_abort, p.wait_us));
            if (!ok) break;  // gave up: nothing more is issued or committed, so the producer stops at its next "empty" wait
            tc_fence_after();
            if (elect_one()) {
                const uint64_t ad = umma_desc(sbase + s * STAGE_BYTES, 16, 1024);
                const uint64_t bd = umma_desc(sbase + s * STAGE_BYTES + TILE_BYTES, 16, 1024);
#pragma unroll
                for (int kk = 0; kk < BK / 16; kk++)
                    umma_ss(tmem, ad + (uint64_t)(kk * 2), bd + (uint64_t)(kk * 2), IDESC, (kb | (uint32_t)kk) != 0u ? 1u : 0u);
                umma_commit(&bar_empty[s]);
                if (kb + 1 == (uint32_t)KB_PER && ok) umma_commit(&bar_acc);  // this CTA's partial accumulator is complete
            }
            __syncwarp();
        }
        if (!ok && lane == 0) atomicOr(p.status, DEV_WAIT_TIMEOUT);
    } else {
        // ===================== while the main loop runs: the tables of the row this thread will finish
        // (thread (warp j, lane t): row 32 crank + t of the tile), final once the kernel before has finished
        pdl_wait();
        const uint32_t frow = m_tile * BM + crank * 32u + (uint32_t)lane;
        rt = proj_fetch_row_tables<kQkvg>((uint32_t)warp_u - 2u, n_tile, frow, frow < p.rows, p);
        // ===================== this CTA's partial accumulator is complete =====================
        acc_ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bar_acc, 0u, &s_abort, p.wait_us));
        tc_fence_after();
        if (!acc_ok && lane == 0) atomicOr(p.status, DEV_WAIT_TIMEOUT);
    }

    // every thread of every CTA: all main loops of the cluster are over, so every CTA's ring is free to receive
    tc_fence_before();
    __syncwarp();
    cluster_sync_all();

    if (warp_u >= 2) {
        // ===================== push: thread = one row of the tile; its 128 columns go to the CTA that finishes
        // the row's quarter, into slot `crank` of that CTA's receive area: [slot][column group of 4][row of the
        // quarter] x 16 bytes (a warp's 32 stores are 512 consecutive bytes).  Remote stores need no round trip.
        const uint32_t quarter = (uint32_t)warp_u & 3u;  // TMEM lanes this warp may read = destination CTA
        tc_fence_after();
        if (acc_ok) {
            const uint32_t t_row = tmem + ((quarter * 32u) << 16);
            const uint32_t dst = dsmem_addr(sbase + (crank * 32u * 32u + (uint32_t)lane) * 16u, quarter);
#pragma unroll 2
            for (int c = 0; c < BN / 16; c++) {
                uint32_t acc[16];
                tmem_ld16(t_row + c * 16, acc);
                tmem_wait_ld();
#pragma unroll
                for (int q4 = 0; q4 < 4; q4++)
                    asm volatile("st.shared::cluster.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(dst + (uint32_t)(c * 4 + q4) * 512u),
                                 "r"(acc[4 * q4]), "r"(acc[4 * q4 + 1]), "r"(acc[4 * q4 + 2]), "r"(acc[4 * q4 + 3])
                                 : "memory");
            }
        }
        if (warp_u == 2 && lane < KS)  // tell every CTA of the cluster whether this one gave up
            asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(dsmem_addr(smem_u32(&s_peer_abort[crank]), (uint32_t)lane)),
                         "r"(acc_ok ? 0u : 1u)
                         : "memory");
    }

    // every thread of every CTA: the partial accumulators and the flags have arrived.  After this barrier a CTA
    // touches only its own shared memory, so it may leave without waiting for its peers.
    tc_fence_before();
    __syncwarp();
    cluster_sync_all();

    if (warp_u >= 2) {
        // ===================== add the four parts + epilogue of rows [32 crank, 32 crank + 32) =====================
        const uint32_t j = (uint32_t)warp_u - 2u, t = (uint32_t)lane;
        bool any_abort = false;
#pragma unroll
        for (int cc = 0; cc < KS; cc++) any_abort |= s_peer_abort[cc] != 0u;
        if (!any_abort) {
            const uint32_t row = m_tile * BM + crank * 32u + t;
            // dims 32g + 8j + i  ->  column groups 8g + 2j and 8g + 2j + 1, row t, of every slot
            const float4* recv = reinterpret_cast<const float4*>(smem_raw + (sbase - smem_u32(smem_raw)));
            float v[4][8];
#pragma unroll
            for (int cc = 0; cc < KS; cc++) {  // k order: part 0 + part 1 + ...
#pragma unroll
                for (int g = 0; g < 4; g++)
#pragma unroll
                    for (int hh = 0; hh < 2; hh++) {
                        const float4 a = recv[((uint32_t)cc * 32u + (uint32_t)(8 * g + 2 * j + hh)) * 32u + t];
                        if (cc == 0) {
                            v[g][4 * hh] = a.x; v[g][4 * hh + 1] = a.y; v[g][4 * hh + 2] = a.z; v[g][4 * hh + 3] = a.w;
                        } else {
                            v[g][4 * hh] = __fadd_rn(v[g][4 * hh], a.x);
                            v[g][4 * hh + 1] = __fadd_rn(v[g][4 * hh + 1], a.y);
                            v[g][4 * hh + 2] = __fadd_rn(v[g][4 * hh + 2], a.z);
                            v[g][4 * hh + 3] = __fadd_rn(v[g][4 * hh + 3], a.w);
                        }
                    }
            }
            proj_finish_row<kQkvg>(v, j, t, n_tile, row, rt, p, s_w, s_part);
        }
    }

    // the tensor-memory loads of the epilogue warps finished before the second cluster barrier
    if (warp_u == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// Epilogue of one head (128 accumulator columns) of one row by TWO threads in two warps of the same TMEM lane quarter
// (a thread serves both heads of a tile, one after the other, with one set of rotary values).
// What the epilogue costs is the number of its memory accesses rather than its arithmetic: a thread works on its own row,
// so each lane of a load or store touches another line and every access is one wavefront of the L1 data pipe that the TMA
// fills and the tensor core's operand reads keep busy; hence 32 bytes per global access and packed reads of the weights.
// Thread j (0 / 1) owns what lanes 16j .. 16j + 15 of the reference's warp own: dims l, l + 32, l + 64, l + 96
// = accumulator columns [32g + 16j, 32g + 16j + 16) for g = 0 .. 3, so the RMSNorm partial sums are the reference's fma
// chains, both members of every RoPE pair (d, d + 64) sit in one thread, and the two threads exchange their 16 partial sums
// through shared memory (named barrier `bar_id` of their two warps) and each run the reference's shfl.down tree on all 32.
// t_row = the thread's TMEM lane base + the head's first column; s_part = [32 reference lanes][32 rows] f32 of this pair of
// warps.  Every lane of both warps must call it.
// The rotary values of a thread's 64 dims: [pair of column groups][cos low, cos high, sin low, sin high][8 packed pairs].
// They depend on the row only, so the caller fetches them once per tile for both heads.
struct RotRegs {
    uint32_t v[2][4][8];
};
template <bool kQkvg>
__device__ __forceinline__ void proj_epilogue_half(uint32_t t_row, uint32_t j, uint32_t n_tile, uint32_t row, bool live, const ProjParams& p,
                                                   const uint16_t* s_w, float* s_part, uint32_t bar_id, uint32_t pos, const RotRegs& rot) {
    constexpr uint32_t N_QKVG = pg::N_QKVG;
    const uint32_t lane = threadIdx.x & 31u;
    if (!OXI_IN_BOUNDS(!live || (row < p.rows && (kQkvg ? n_tile <= 24u : n_tile * 128u < p.out_features)), p.status)) live = false;
    if (!kQkvg) {
        // ---- plain linear layer: y[row][n] = f16(acc)
#pragma unroll 1
        for (int g = 0; g < 4; g++) {
            uint32_t acc[16];
            tmem_ld16(t_row + 32u * g + 16u * j, acc);
            tmem_wait_ld();
            const uint32_t n0 = n_tile * 128u + 32u * g + 16u * j;
            if (live && n0 < p.out_features) {
                uint16_t h[16];
                float f[16];
                round16(acc, h, f);
                uint16_t* dst = p.y + (size_t)row * p.out_features + n0;
                if (n0 + 16 <= p.out_features && (p.out_features & 7u) == 0u) {
                    store16(dst, h);
                } else {
                    for (uint32_t i = 0; i < 16 && n0 + i < p.out_features; i++) dst[i] = h[i];
                }
            }
        }
        return;
    }
    if (n_tile == 24u) {
        // ---- gate: 16 features, all in thread 0's first group
        if (j == 0u) {
            uint32_t acc[16];
            tmem_ld16(t_row, acc);
            tmem_wait_ld();
            if (live) {
                uint16_t h[16];
                float f[16];
                round16(acc, h, f);
                store16(p.gate_out + (size_t)row * NQ, h);
                if (p.raw_out) store16(p.raw_out + (size_t)row * N_QKVG + 3072, h);
            }
        }
        return;
    }
    uint64_t kvp = 0;
    if (live) {
        if (n_tile >= 16u && n_tile < 20u) kvp = p.k_ptrs[row];
        if (n_tile >= 20u) kvp = p.v_ptrs[row];
    }
    if (n_tile >= 20u) {
        // ---- v head: the f16 projection is the cache row
        const uint32_t kvh = n_tile - 20u;
        const bool aligned = (kvp & 15ull) == 0ull;
        if (live && !aligned && kvh == 0u && j == 0u) atomicOr(p.status, DEV_MISALIGNED_PTR);
        uint16_t* dst = reinterpret_cast<uint16_t*>(kvp + (size_t)pos * KV_ROW_BYTES) + kvh * HD;
#pragma unroll 1
        for (int g = 0; g < 4; g++) {
            uint32_t acc[16];
            tmem_ld16(t_row + 32u * g + 16u * j, acc);
            tmem_wait_ld();
            if (live) {
                uint16_t h[16];
                float f[16];
                round16(acc, h, f);
                const uint32_t d0 = 32u * g + 16u * j;
                if (aligned) store16(dst + d0, h);
                if (p.raw_out) store16(p.raw_out + (size_t)row * N_QKVG + 2560 + kvh * HD + d0, h);
            }
        }
        return;
    }
    // ---- q or k head: RMSNorm + RoPE on the f16 projections, the append kernel's arithmetic
    const bool is_k = n_tile >= 16u;
    const uint32_t head = is_k ? n_tile - 16u : n_tile;
    const uint16_t* wn = s_w + (is_k ? HD : 0);
    const bool aligned = !is_k || (kvp & 15ull) == 0ull;
    if (live && !aligned && head == 0u && j == 0u) atomicOr(p.status, DEV_MISALIGNED_PTR);
    // pass 1: partial[i] = sum over dims l, l+32, l+64, l+96 (in that order, fma) for l = 16j + i
    float partial[32];
#pragma unroll
    for (int i = 0; i < 16; i++) partial[i] = 0.0f;
#pragma unroll
    for (int g = 0; g < 4; g++) {
        uint32_t acc[16];
        tmem_ld16(t_row + 32u * g + 16u * j, acc);
        tmem_wait_ld();
        uint16_t h[16];
        float f[16];
        round16(acc, h, f);
#pragma unroll
        for (int i = 0; i < 16; i++) partial[i] = __fmaf_rn(f[i], f[i], partial[i]);
        if (live && p.raw_out)
            store16(p.raw_out + (size_t)row * N_QKVG + (is_k ? 2048 : 0) + head * HD + 32u * g + 16u * j, h);
    }
#pragma unroll
    for (int i = 0; i < 16; i++) s_part[(16u * j + i) * 32u + lane] = partial[i];
    asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory");  // the two warps of this row quarter and head
#pragma unroll
    for (int l = 0; l < 32; l++) partial[l] = s_part[l * 32 + lane];
    asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory");  // both have read: the next tile may overwrite the partials
    // the shfl.down tree of the reference on one thread's registers: lane 0's value
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1)
#pragma unroll
        for (int l = 0; l < off; l++) partial[l] = __fadd_rn(partial[l], partial[l + off]);
    float mean = div_approx_ftz(partial[0], 128.0f);
    mean = __fadd_rn(mean, p.eps);
    const float r = rsqrt_approx_ftz(mean);
    uint16_t* dst = is_k ? reinterpret_cast<uint16_t*>(kvp + (size_t)pos * KV_ROW_BYTES) + head * HD
                         : p.q_out + ((size_t)row * NQ + head) * HD;
    // pass 2: dims [dl, dl + 16) pair with dims 64 + [dl, dl + 16), dl = 32 pr + 16 j
#pragma unroll
    for (int pr = 0; pr < 2; pr++) {
        const uint32_t dl = 32u * pr + 16u * j, dh = dl + 64u;
        uint32_t alo[16], ahi[16];
        tmem_ld16(t_row + dl, alo);
        tmem_ld16(t_row + dh, ahi);
        tmem_wait_ld();
        uint32_t olo[8], ohi[8];
        // the norm weights of the 16 + 16 dims as packed pairs: four 16-byte reads instead of 32 two-byte ones
        const uint4 wl0 = *reinterpret_cast<const uint4*>(wn + dl), wl1 = *reinterpret_cast<const uint4*>(wn + dl + 8);
        const uint4 wh0 = *reinterpret_cast<const uint4*>(wn + dh), wh1 = *reinterpret_cast<const uint4*>(wn + dh + 8);
        const uint32_t wlo[8] = {wl0.x, wl0.y, wl0.z, wl0.w, wl1.x, wl1.y, wl1.z, wl1.w};
        const uint32_t whi[8] = {wh0.x, wh0.y, wh0.z, wh0.w, wh1.x, wh1.y, wh1.z, wh1.w};
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const int wd = i >> 1, sh = (i & 1) * 16;
            const float xlo = h2f(f2h(__uint_as_float(alo[i]))), xhi = h2f(f2h(__uint_as_float(ahi[i])));
            // y = f16((x * r) * w): two separate multiplies, then the f16 round trip
            const float ylo = h2f(f2h(__fmul_rn(__fmul_rn(xlo, r), h2f((uint16_t)(wlo[wd] >> sh)))));
            const float yhi = h2f(f2h(__fmul_rn(__fmul_rn(xhi, r), h2f((uint16_t)(whi[wd] >> sh)))));
            const float c_lo = h2f((uint16_t)(rot.v[pr][0][wd] >> sh)), c_hi = h2f((uint16_t)(rot.v[pr][1][wd] >> sh));
            const float s_lo = h2f((uint16_t)(rot.v[pr][2][wd] >> sh)), s_hi = h2f((uint16_t)(rot.v[pr][3][wd] >> sh));
            // rotate-half: out[d] = fma(-y[d+64], sin[d], y[d]*cos[d]);  out[d+64] = fma(y[d], sin[d+64], y[d+64]*cos[d+64])
            const uint32_t o_lo = f2h(__fmaf_rn(-yhi, s_lo, __fmul_rn(ylo, c_lo)));
            const uint32_t o_hi = f2h(__fmaf_rn(ylo, s_hi, __fmul_rn(yhi, c_hi)));
            if (i & 1) {
                olo[wd] |= o_lo << 16;
                ohi[wd] |= o_hi << 16;
            } else {
                olo[wd] = o_lo;
                ohi[wd] = o_hi;
            }
        }
        if (live && aligned) {
            st_pairs(dst + dl, olo);
            st_pairs(dst + dh, ohi);
        }
    }
}

// ---------------------------------------------------------------------------------------------------
// Waves of rows on CTA PAIRS: two CTAs of a cluster (two SMs) work on one 256-row x 256-feature tile with
// tcgen05.mma.cta_group::2.  Each CTA keeps ITS 128 rows of x and ITS 128 of the tile's 256 weight rows in
// shared memory (32 KB per 64-wide k-block, where one CTA on a 128 x 256 tile needs 48 KB for the same
// tensor-core time: 477 instead of 682 MB from L2 into the SMs on the 4,096-row wave) and the accumulator rows
// of its own 128 tokens in its own tensor memory.
//   * CTA 0 of the pair (the leader) issues every MMA; the instruction reads both CTAs' shared memory at the
//     same offsets.
//   * Both CTAs' copies complete on the LEADER's "full" barrier of the stage (armed by the leader with the
//     bytes of both); the leader's commit after a stage's MMAs arrives on the "empty" barrier of BOTH CTAs
//     (two commits, the second with the peer's mapped address - no multicast anywhere), likewise "accumulator
//     full"; the epilogue warps of both CTAs arrive on the leader's "accumulator empty" barrier.
//   * Tensor memory is allocated and freed by the MMA warp of BOTH CTAs (cta_group::2 forms), the free after a
//     cluster barrier that every thread reaches on every path (all other waits are bounded).
namespace pgp {
constexpr int BM = 128, BN_CTA = 128, BK = 64;            // per CTA: 128 rows of x, 128 weight rows; the pair: 256 x 256
// ring stages: measured on the 4,096-row wave 2: 63.3 us, 3: 46.7, 4: 45.2, 5: 46.0, 6: 47.9 (with the rotary values fetched once per
// tile for both heads: 4: 44.3, 5: 44.5, 6: 45.3) - four stages cover the latency, more shared memory only shrinks the L1 cache
constexpr int NS = 4;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN_CTA * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;  // 16 + 16 KB
constexpr int EPI_WARPS = 8;   // two per TMEM lane quarter: two threads per row, each serving both heads of the tile
constexpr int THREADS = 64 + 32 * EPI_WARPS;  // TMA warp, MMA warp, epilogue warps
constexpr int PART_BYTES = 4 * 32 * 32 * 4;   // RMSNorm partial sums: [quarter][32 reference lanes][32 rows] f32
constexpr size_t SMEM_BYTES = 1024 + (size_t)NS * STAGE_BYTES + PART_BYTES;
constexpr uint32_t TMEM_COLS = 512;   // two accumulators of 256 columns
constexpr uint32_t IDESC_N256 = (1u << 4) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);  // M = 256 over the pair
constexpr uint32_t IDESC_N16 = (1u << 4) | ((uint32_t)(16 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);    // the gate tile
constexpr int TILES_QKVG = 8 + 2 + 2 + 1;
}  // namespace pgp

__device__ __forceinline__ void umma_ss_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on the barrier at shared::cluster address `bar` (own or the peer's) once all MMAs issued so far have completed
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// one box into this CTA's shared memory; completion counted on the barrier at shared::cluster address `bar`.  No multicast.
__device__ __forceinline__ void tma_load_box_pair(uint32_t dst, const TmaDesc* map, uint32_t x, uint32_t y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}

template <bool kQkvg>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(pgp::THREADS, 1)
proj_gemm_pair_kernel(const __grid_constant__ ProjMaps maps, const ProjParams p, const uint32_t tiles_n, const uint32_t tiles_m2) {
    using namespace pgp;
    constexpr int NKB = pg::NKB;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[NS], bar_empty[NS], bar_acc_full[2], bar_acc_empty[2];
    __shared__ uint32_t s_tmem, s_abort;
    __shared__ volatile uint32_t s_fail[4];   // per TMEM lane quarter: one of its two epilogue warps gave up a wait
    __shared__ __align__(16) uint16_t s_w[2 * HD];

    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp_u = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const uint32_t crank = cluster_ctarank();     // 0: leader (issues the MMAs), 1: its peer
    const uint32_t pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

    pdl_launch_dependents();
    if (tid == 0) {
        for (int s = 0; s < NS; s++) {
            mbar_init(&bar_full[s], 1);    // used in the leader: its own arrive.expect_tx; both CTAs' copies complete on it
            mbar_init(&bar_empty[s], 1);   // in both CTAs: one commit of the leader
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&bar_acc_full[b], 1);     // in both CTAs: one commit of the leader
            mbar_init(&bar_acc_empty[b], 2 * EPI_WARPS);   // used in the leader: one arrival per epilogue warp of both CTAs
        }
        s_abort = 0u;
        s_fail[0] = s_fail[1] = s_fail[2] = s_fail[3] = 0u;
        mbar_fence_init();
    }
    if (kQkvg && tid >= 64 && tid < 64 + HD) {
        const int i = tid - 64;
        s_w[i] = p.q_norm_w[i];
        s_w[HD + i] = p.k_norm_w[i];
    }
    // the peer's barriers are initialised before anything of this CTA arrives on them
    __syncwarp();
    cluster_sync_all();
    if (warp_u == 1) {  // the MMA warp of BOTH CTAs: the pair's tensor memory is allocated together
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    const uint32_t total = tiles_n * tiles_m2;

    // pair tile t: feature tile nt = t % tiles_n (256 features; fastest), row tile t / tiles_n (256 rows)
    auto tile_weights = [&](uint32_t nt, uint32_t& wsel, uint32_t& wrow) {   // this CTA's 128 weight rows (8 of the gate's 16)
        wsel = 0;
        wrow = nt * 256u + crank * 128u;
        if (kQkvg) {
            if (nt >= 12) { wsel = 3; wrow = crank * 8u; }
            else if (nt >= 10) { wsel = 2; wrow = (nt - 10) * 256u + crank * 128u; }
            else if (nt >= 8) { wsel = 1; wrow = (nt - 8) * 256u + crank * 128u; }
        }
    };

    if (warp_u == 0) {
        // ===================== TMA producer (both CTAs) =====================
        pdl_wait();  // x is written by the kernel before this one
        bool ok = true;
        uint32_t g = 0;
        for (uint32_t t = pair; t < total && ok; t += npairs) {
            uint32_t wsel, wrow;
            tile_weights(t % tiles_n, wsel, wrow);
            const uint32_t mrow = (t / tiles_n) * 256u + crank * 128u;
            for (uint32_t kb = 0; kb < (uint32_t)NKB; kb++, g++) {
                const uint32_t s = g % NS;
                if (g >= (uint32_t)NS && !mbar_wait_bounded(&bar_empty[s], ((g / NS) & 1u) ^ 1u, &s_abort, p.wait_us)) {
                    ok = false;
                    break;
                }
                const bool withheld = p.skip_plus1 == g + 1u && blockIdx.x == 0u;  // test support: the first pair's leader
                if (lane == 0 && !withheld) {
                    const uint32_t full = dsmem_addr(smem_u32(&bar_full[s]), 0u);   // the leader's barrier
                    if (crank == 0u) mbar_arrive_expect_tx(&bar_full[s], 2u * (uint32_t)STAGE_BYTES);
                    tma_load_box_pair(sbase + s * STAGE_BYTES, &maps.x, kb * BK, mrow, full);
                    tma_load_box_pair(sbase + s * STAGE_BYTES + A_BYTES, &maps.w[wsel], kb * BK, wrow, full);
                }
                __syncwarp();
            }
        }
        if (!ok) {
            if (lane == 0) atomicOr(p.status, DEV_WAIT_TIMEOUT);
            // copies already issued complete on the leader's barriers, which the peer cannot poll: give them time to
            // land before the shared memory is released (they take microseconds)
            const uint64_t t0 = global_timer_ns();
            while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
        }
    } else if (warp_u == 1) {
        // ===================== MMA issuer (the leader only) =====================
        if (crank == 0u) {
            bool ok = true;
            uint32_t g = 0, i = 0;
            for (uint32_t t = pair; t < total; t += npairs, i++) {
                const uint32_t buf = i & 1u;
                const uint32_t idesc = (kQkvg && t % tiles_n == 12u) ? IDESC_N16 : IDESC_N256;
                if (i >= 2u) ok = __all_sync(0xffffffffu, ok && mbar_wait_bounded(&bar_acc_empty[buf], ((i >> 1) & 1u) ^ 1u, &s_abort, p.wait_us));
                for (uint32_t kb = 0; kb < (uint32_t)NKB; kb++, g++) {
                    const uint32_t s = g % NS;
                    ok = __all_sync(0xffffffffu, ok && mbar_wait_bounded(&bar_full[s], (g / NS) & 1u, &s_abort, p.wait_us));
                    if (!ok) break;  // gave up: nothing more is issued or committed, so both producers stop at their next "empty" wait
                    tc_fence_after();
                    if (elect_one()) {
                        const uint64_t ad = umma_desc(sbase + s * STAGE_BYTES, 16, 1024);
                        const uint64_t bd = umma_desc(sbase + s * STAGE_BYTES + A_BYTES, 16, 1024);
#pragma unroll
                        for (int kk = 0; kk < BK / 16; kk++)
                            umma_ss_pair(tmem + buf * 256u, ad + (uint64_t)(kk * 2), bd + (uint64_t)(kk * 2), idesc,
                                         (kb | (uint32_t)kk) != 0u ? 1u : 0u);
                        umma_commit_pair(smem_u32(&bar_empty[s]));
                        umma_commit_pair(dsmem_addr(smem_u32(&bar_empty[s]), 1u));
                        if (kb + 1 == (uint32_t)NKB && ok) {
                            umma_commit_pair(smem_u32(&bar_acc_full[buf]));
                            umma_commit_pair(dsmem_addr(smem_u32(&bar_acc_full[buf]), 1u));
                        }
                    }
                    __syncwarp();
                }
                if (!ok) break;
            }
            if (!ok && lane == 0) atomicOr(p.status, DEV_WAIT_TIMEOUT);
        }
    } else {
        // ===================== epilogue warps (both CTAs): two warps per TMEM lane quarter = the two halves of a head's reference
        // lanes; thread = one row of this CTA's 128, serving both heads of the tile with one set of rotary values
        const uint32_t quarter = (uint32_t)warp_u & 3u, half = ((uint32_t)warp_u - 2u) >> 2;
        float* s_part = reinterpret_cast<float*>(smem_raw + (sbase - smem_u32(smem_raw)) + (size_t)NS * STAGE_BYTES) + quarter * 1024u;
        const uint32_t bar_id = 1u + quarter;
        const uint32_t acc_empty0 = dsmem_addr(smem_u32(&bar_acc_empty[0]), 0u), acc_empty1 = dsmem_addr(smem_u32(&bar_acc_empty[1]), 0u);
        bool ok = true;
        uint32_t i = 0;
        for (uint32_t t = pair; t < total && ok; t += npairs, i++) {
            const uint32_t buf = i & 1u, nt = t % tiles_n;
            const uint32_t row = (t / tiles_n) * 256u + crank * 128u + quarter * 32 + (uint32_t)lane;
            ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bar_acc_full[buf], (i >> 1) & 1u, &s_abort, p.wait_us));
            tc_fence_after();
            // The two warps of a lane quarter meet in named barriers inside the epilogue, so they must take the same decision
            // here: a warp that gave up says so before they meet, and both look afterwards (nobody else writes the word).
            if (!ok && lane == 0) s_fail[quarter] = 1u;
            asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory");
            ok = s_fail[quarter] == 0u;
            if (!ok) {
                if (lane == 0) atomicOr(p.status, DEV_WAIT_TIMEOUT);
                break;
            }
            const uint32_t t_row = tmem + ((quarter * 32) << 16) + buf * 256u;
            uint32_t ct0 = 2u * nt;
            bool two = true;
            if (kQkvg) {
                if (nt >= 12u) { ct0 = 24u; two = false; }
                else if (nt >= 10u) ct0 = 20u + 2u * (nt - 10u);
                else if (nt >= 8u) ct0 = 16u + 2u * (nt - 8u);
            } else {
                two = (ct0 + 1u) * 128u < p.out_features;
            }
            const bool live = row < p.rows;
            uint32_t pos = 0;
            RotRegs rot;
            if (kQkvg && ct0 < 24u) {
                if (live) pos = p.pos_ids[row];
                if (ct0 < 20u) {  // q and k heads rotate: dims [32 pr + 16 half, +16) pair with the dims 64 further on
                    const uint16_t* cs = p.cos_t + (size_t)pos * HD + 16u * half;
                    const uint16_t* sn = p.sin_t + (size_t)pos * HD + 16u * half;
#pragma unroll
                    for (int pr = 0; pr < 2; pr++) {
                        ld_pairs(cs + 32 * pr, rot.v[pr][0]);
                        ld_pairs(cs + 32 * pr + 64, rot.v[pr][1]);
                        ld_pairs(sn + 32 * pr, rot.v[pr][2]);
                        ld_pairs(sn + 32 * pr + 64, rot.v[pr][3]);
                    }
                }
            }
            proj_epilogue_half<kQkvg>(t_row, half, ct0, row, live, p, s_w, s_part, bar_id, pos, rot);
            if (two) proj_epilogue_half<kQkvg>(t_row + 128u, half, ct0 + 1u, row, live, p, s_w, s_part, bar_id, pos, rot);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(buf ? acc_empty1 : acc_empty0);
        }
    }

    // every thread of both CTAs: nothing of the pair is in flight any more (or a wait ran out and was recorded)
    tc_fence_before();
    __syncwarp();
    cluster_sync_all();
    if (warp_u == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

cudaError_t proj_gemm_init() {
    cudaError_t e = cudaFuncSetAttribute(proj_gemm_splitk_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pgs::SMEM_BYTES);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(proj_gemm_splitk_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pgs::SMEM_BYTES);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(proj_gemm_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pgp::SMEM_BYTES);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(proj_gemm_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pgp::SMEM_BYTES);
    return e;
}

// Encodes a tiled map over a row-major [rows][2048] f16 matrix: box = 64 elements x box_rows rows, 128-byte swizzle,
// rows beyond the matrix read as zeros.  Pure host work, no allocation.
int proj_encode_map(TmaDesc* out, const void* base, uint64_t rows, uint32_t box_rows) {
    typedef CUresult (*encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static encode_fn fn = nullptr;
    if (!fn) {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || !f ||
            q != cudaDriverEntryPointSuccess)
            return -1;
        fn = (encode_fn)f;
    }
    static_assert(sizeof(CUtensorMap) == sizeof(TmaDesc), "tensor map size");
    const cuuint64_t dims[2] = {(cuuint64_t)pg::KDIM, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)pg::KDIM * 2};
    const cuuint32_t box[2] = {(cuuint32_t)pg::BK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1u, 1u};
    const CUresult r = fn(reinterpret_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims,
                          strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -2;
}

// rows up to this many run the cluster kernel (four CTAs per 128 x 128 tile), larger waves the persistent one.  Measured (us,
// projection+append / plain 2048-feature layer): 384 rows 16.7 / 10.3 against 22.8 / 15.4, 512 rows 20.6 / 10.8 against 23.1 / 15.4,
// 768 rows 27.6 / 18.1 against 23.5 / 15.4.
constexpr uint32_t PROJ_SMALL_ROWS = 512;

cudaError_t launch_project_append(cudaStream_t stream, const TmaDesc* w_maps /* q, k, v, gate */, int num_sms, const void* x, uint32_t rows,
                                  void* q_out, void* gate_out, void* raw_out, const void* q_norm_w, const void* k_norm_w,
                                  const void* cos_t, const void* sin_t, const uint32_t* pos_ids, const uint64_t* k_ptrs,
                                  const uint64_t* v_ptrs, float eps, uint32_t* status, const WaitFault* fault) {
    ProjMaps maps;
    if (proj_encode_map(&maps.x, x, rows, pg::BM) != 0) return cudaErrorInvalidValue;
    for (int i = 0; i < 4; i++) maps.w[i] = w_maps[i];
    ProjParams p = {};
    p.rows = rows;
    p.q_out = (uint16_t*)q_out;
    p.gate_out = (uint16_t*)gate_out;
    p.raw_out = (uint16_t*)raw_out;
    p.q_norm_w = (const uint16_t*)q_norm_w;
    p.k_norm_w = (const uint16_t*)k_norm_w;
    p.cos_t = (const uint16_t*)cos_t;
    p.sin_t = (const uint16_t*)sin_t;
    p.pos_ids = pos_ids;
    p.k_ptrs = k_ptrs;
    p.v_ptrs = v_ptrs;
    p.status = status;
    p.eps = eps;
    p.wait_us = fault && fault->skip_plus1 ? fault->limit_us : WAIT_LIMIT_US;
    p.skip_plus1 = fault ? fault->skip_plus1 : 0u;
    if (rows > PROJ_SMALL_ROWS) {
        const uint32_t tiles_m2 = (rows + 255u) / 256u, total = (uint32_t)pgp::TILES_QKVG * tiles_m2;
        const uint32_t pairs = total < (uint32_t)num_sms / 2u ? total : (uint32_t)num_sms / 2u;
        return launch_pdl(proj_gemm_pair_kernel<true>, dim3(2u * pairs), dim3(pgp::THREADS), pgp::SMEM_BYTES, stream, maps, p,
                          (uint32_t)pgp::TILES_QKVG, tiles_m2);
    }
    const uint32_t tiles_m = (rows + pg::BM - 1) / pg::BM;
    return launch_pdl(proj_gemm_splitk_kernel<true>, dim3(pg::TILES_QKVG * pgs::KS, tiles_m), dim3(pgs::THREADS), pgs::SMEM_BYTES, stream,
                      maps, p);
}

cudaError_t launch_linear(cudaStream_t stream, const TmaDesc* w_map, int num_sms, uint32_t out_features, const void* x, uint32_t rows,
                          void* y, uint32_t* status, const WaitFault* fault) {
    ProjMaps maps;
    if (proj_encode_map(&maps.x, x, rows, pg::BM) != 0) return cudaErrorInvalidValue;
    maps.w[0] = maps.w[1] = maps.w[2] = maps.w[3] = *w_map;
    ProjParams p = {};
    p.rows = rows;
    p.out_features = out_features;
    p.y = (uint16_t*)y;
    p.status = status;
    p.wait_us = fault && fault->skip_plus1 ? fault->limit_us : WAIT_LIMIT_US;
    p.skip_plus1 = fault ? fault->skip_plus1 : 0u;
    if (rows > PROJ_SMALL_ROWS) {
        const uint32_t tiles_n = (out_features + 255u) / 256u, tiles_m2 = (rows + 255u) / 256u, total = tiles_n * tiles_m2;
        const uint32_t pairs = total < (uint32_t)num_sms / 2u ? total : (uint32_t)num_sms / 2u;
        return launch_pdl(proj_gemm_pair_kernel<false>, dim3(2u * pairs), dim3(pgp::THREADS), pgp::SMEM_BYTES, stream, maps, p, tiles_n,
                          tiles_m2);
    }
    const uint32_t tiles_m = (rows + pg::BM - 1) / pg::BM;
    return launch_pdl(proj_gemm_splitk_kernel<false>, dim3((out_features + pg::BN - 1) / pg::BN * pgs::KS, tiles_m), dim3(pgs::THREADS),
                      pgs::SMEM_BYTES, stream, maps, p);
}

}  // namespace oxi
