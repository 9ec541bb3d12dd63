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
// elected lane), warps 2-5 run the epilogue: thread = one row of the tile (its TMEM lane), so a
// thread holds a whole head of its token and the per-head arithmetic needs no shuffles.
// At the decode shape (128 rows: 25 CTAs) a launch takes ~15 us, of which the tile's 128 MMAs are ~5,
// the epilogue ~4 and launch, set-up and the first copies' latency the rest; cutting K into four parts
// that meet in an L2 workspace (100 CTAs) measured 16-18 us (the exchange costs what the shorter main
// loop saves) and a ring twice as deep changed nothing, so neither is here.
//
// Bit parity.  The projections are rounded to f16 exactly as the reference's GEMM output is, and
// the epilogue applies the append kernel's arithmetic to those f16 values: the RMSNorm sum is formed
// in the reference's order (32 partial sums over dims l, l+32, l+64, l+96 with fma, then the
// shfl.down tree 16, 8, 4, 2, 1 - here as the same additions on 32 registers of one thread),
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
__device__ __forceinline__ void store16(uint16_t* dst, const uint16_t (&h)[16]) {  // 32 bytes, 16-byte aligned
    uint4 a, b;
    a.x = h[0] | ((uint32_t)h[1] << 16);   a.y = h[2] | ((uint32_t)h[3] << 16);
    a.z = h[4] | ((uint32_t)h[5] << 16);   a.w = h[6] | ((uint32_t)h[7] << 16);
    b.x = h[8] | ((uint32_t)h[9] << 16);   b.y = h[10] | ((uint32_t)h[11] << 16);
    b.z = h[12] | ((uint32_t)h[13] << 16); b.w = h[14] | ((uint32_t)h[15] << 16);
    reinterpret_cast<uint4*>(dst)[0] = a;
    reinterpret_cast<uint4*>(dst)[1] = b;
}
__device__ __forceinline__ void ld_pairs(const uint16_t* src, uint32_t (&w)[8]) {  // 16 f16 = 32 bytes, 16-byte aligned
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(src)), b = __ldg(reinterpret_cast<const uint4*>(src) + 1);
    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
    w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
}
__device__ __forceinline__ void st_pairs(uint16_t* dst, const uint32_t (&w)[8]) {
    reinterpret_cast<uint4*>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
    reinterpret_cast<uint4*>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
}

// Epilogue of one 128-column group of an accumulator tile for one row (thread = row = TMEM lane):
// t_row = the thread's TMEM lane base + the group's first column; ct = index of the group among the
// output features in units of 128 (qkvg: 0-15 q heads, 16-19 k heads, 20-23 v heads, 24 gate).
// Every lane of the warp must call it (the tensor-memory loads are warp-wide); `live` says whether the
// row exists.
template <bool kQkvg>
__device__ __forceinline__ void proj_epilogue_cols(uint32_t t_row, uint32_t n_tile, uint32_t row, bool live, const ProjParams& p,
                                                   const uint16_t* s_w) {
    constexpr int BN = 128;
    constexpr int N_QKVG = pg::N_QKVG;
    // bounds build: a live thread's row exists and its feature group is one of the 25 (qkvg) / lies inside y (plain)
    if (!OXI_IN_BOUNDS(!live || (row < p.rows && (kQkvg ? n_tile <= 24u : n_tile * 128u < p.out_features)), p.status)) live = false;
    // the row's table entries (not written by any kernel)
    uint32_t pos = 0;
    uint64_t kvp = 0;
    if (kQkvg && live) {
        pos = p.pos_ids[row];
        if (n_tile >= 16 && n_tile < 20) kvp = p.k_ptrs[row];
        if (n_tile >= 20 && n_tile < 24) kvp = p.v_ptrs[row];
    }
    if (!kQkvg) {
        // ---- plain linear layer: y[row][n] = f16(acc)
#pragma unroll 1
        for (int c = 0; c < BN / 16; c++) {
            uint32_t acc[16];
            tmem_ld16(t_row + c * 16, acc);
            tmem_wait_ld();
            const uint32_t n0 = n_tile * BN + c * 16;
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
    } else if (n_tile == 24) {
        // ---- gate: 16 features
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
    } else if (n_tile >= 20) {
        // ---- v head: the f16 projection is the cache row (batched_kv_copy_fp16 is a pure copy)
        const uint32_t kvh = n_tile - 20;
        const bool aligned = (kvp & 15ull) == 0ull;
        if (live && !aligned && kvh == 0) atomicOr(p.status, DEV_MISALIGNED_PTR);
        uint16_t* dst = reinterpret_cast<uint16_t*>(kvp + (size_t)pos * KV_ROW_BYTES) + kvh * HD;
#pragma unroll 1
        for (int c = 0; c < BN / 16; c++) {
            uint32_t acc[16];
            tmem_ld16(t_row + c * 16, acc);
            tmem_wait_ld();
            if (live) {
                uint16_t h[16];
                float f[16];
                round16(acc, h, f);
                if (aligned) store16(dst + c * 16, h);
                if (p.raw_out) store16(p.raw_out + (size_t)row * N_QKVG + 2560 + kvh * HD + c * 16, h);
            }
        }
    } else {
        // ---- q or k head: RMSNorm + RoPE on the f16 projections, the append kernel's arithmetic
        const bool is_k = n_tile >= 16;
        const uint32_t head = is_k ? n_tile - 16 : n_tile;
        const uint16_t* wn = s_w + (is_k ? HD : 0);
        const bool aligned = !is_k || (kvp & 15ull) == 0ull;
        if (live && !aligned && head == 0) atomicOr(p.status, DEV_MISALIGNED_PTR);
        // pass 1: partial[l] = sum over dims l, l+32, l+64, l+96 (in that order, fma), as lane l of the
        // reference's warp forms it
        float partial[32];
#pragma unroll
        for (int l = 0; l < 32; l++) partial[l] = 0.0f;
#pragma unroll
        for (int c = 0; c < BN / 16; c++) {
            uint32_t acc[16];
            tmem_ld16(t_row + c * 16, acc);
            tmem_wait_ld();
            uint16_t h[16];
            float f[16];
            round16(acc, h, f);
#pragma unroll
            for (int i = 0; i < 16; i++) partial[16 * (c & 1) + i] = __fmaf_rn(f[i], f[i], partial[16 * (c & 1) + i]);
            if (live && p.raw_out)
                store16(p.raw_out + (size_t)row * N_QKVG + (is_k ? 2048 : 0) + head * HD + c * 16, h);
        }
        // the shfl.down tree of the reference on one thread's registers: lane 0's value
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1)
#pragma unroll
            for (int l = 0; l < off; l++) partial[l] = __fadd_rn(partial[l], partial[l + off]);
        float mean = div_approx_ftz(partial[0], 128.0f);
        mean = __fadd_rn(mean, p.eps);
        const float r = rsqrt_approx_ftz(mean);
        // pass 2: dims [16j, 16j+16) pair with dims 64 + [16j, 16j+16)
        const uint16_t* cs = p.cos_t + (size_t)pos * HD;
        const uint16_t* sn = p.sin_t + (size_t)pos * HD;
        uint16_t* dst = is_k ? reinterpret_cast<uint16_t*>(kvp + (size_t)pos * KV_ROW_BYTES) + head * HD
                             : p.q_out + ((size_t)row * NQ + head) * HD;
#pragma unroll 1
        for (int j = 0; j < 4; j++) {
            uint32_t alo[16], ahi[16];
            tmem_ld16(t_row + j * 16, alo);
            tmem_ld16(t_row + 64 + j * 16, ahi);
            tmem_wait_ld();
            if (!live) continue;
            // cos / sin of the 16 + 16 dims as packed f16 pairs (two 16-byte loads each)
            uint32_t clo[8], chi[8], slo[8], shi[8], olo[8], ohi[8];
            ld_pairs(cs + j * 16, clo);
            ld_pairs(cs + 64 + j * 16, chi);
            ld_pairs(sn + j * 16, slo);
            ld_pairs(sn + 64 + j * 16, shi);
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const float xlo = h2f(f2h(__uint_as_float(alo[i]))), xhi = h2f(f2h(__uint_as_float(ahi[i])));
                // y = f16((x * r) * w): two separate multiplies, then the f16 round trip
                const float ylo = h2f(f2h(__fmul_rn(__fmul_rn(xlo, r), h2f(wn[j * 16 + i]))));
                const float yhi = h2f(f2h(__fmul_rn(__fmul_rn(xhi, r), h2f(wn[64 + j * 16 + i]))));
                const int wd = i >> 1, sh = (i & 1) * 16;
                const float c_lo = h2f((uint16_t)(clo[wd] >> sh)), c_hi = h2f((uint16_t)(chi[wd] >> sh));
                const float s_lo = h2f((uint16_t)(slo[wd] >> sh)), s_hi = h2f((uint16_t)(shi[wd] >> sh));
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
            if (aligned) {
                st_pairs(dst + j * 16, olo);
                st_pairs(dst + 64 + j * 16, ohi);
            }
        }
    }
}

template <bool kQkvg>
__global__ void __launch_bounds__(pg::THREADS, 2)
proj_gemm_kernel(const __grid_constant__ ProjMaps maps, const ProjParams p) {
    using namespace pg;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[NS], bar_empty[NS], bar_acc;
    __shared__ uint32_t s_tmem, s_abort;
    __shared__ uint16_t s_w[2 * HD];  // q and k norm weights

    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;  // 1024-byte aligned tiles (128-byte swizzle)
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp_u = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const uint32_t n_tile = blockIdx.x, m_tile = blockIdx.y;

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

    // which weight matrix and which of its rows this tile covers
    uint32_t wsel = 0, wrow = n_tile * BN;
    if (kQkvg) {
        if (n_tile >= 24) { wsel = 3; wrow = 0; }
        else if (n_tile >= 20) { wsel = 2; wrow = (n_tile - 20) * BN; }
        else if (n_tile >= 16) { wsel = 1; wrow = (n_tile - 16) * BN; }
    }

    if (warp_u == 0) {
        // ===================== TMA producer =====================
        pdl_wait();  // x is written by the kernel before this one
        bool ok = true;
        uint32_t issued = 0;
        for (uint32_t kb = 0; kb < (uint32_t)NKB && ok; kb++, issued++) {
            const uint32_t s = kb % NS;
            if (kb >= (uint32_t)NS && !mbar_wait_bounded(&bar_empty[s], ((kb / NS) & 1u) ^ 1u, &s_abort)) {
                ok = false;
                break;
            }
            if (lane == 0) {
                mbar_arrive_expect_tx(&bar_full[s], (uint32_t)STAGE_BYTES);
                tma_load_box(sbase + s * STAGE_BYTES, &maps.x, kb * BK, m_tile * BM, &bar_full[s]);
                tma_load_box(sbase + s * STAGE_BYTES + TILE_BYTES, &maps.w[wsel], kb * BK, wrow, &bar_full[s]);
            }
            __syncwarp();
        }
        if (!ok) {
            if (lane == 0) atomicOr(p.status, DEV_WAIT_TIMEOUT);
            // copies already issued land before the shared memory is released
            for (uint32_t k = issued > (uint32_t)NS ? issued - NS : 0; k < issued; ++k)
                mbar_wait_drain(&bar_full[k % NS], (k / NS) & 1u, WAIT_LIMIT_US);
        }
    } else if (warp_u == 1) {
        // ===================== MMA issuer =====================
        bool ok = true;
        for (uint32_t kb = 0; kb < (uint32_t)NKB; kb++) {
            const uint32_t s = kb % NS;
            ok = __all_sync(0xffffffffu, ok && mbar_wait_bounded(&bar_full[s], (kb / NS) & 1u, &s_abort));
            tc_fence_after();
            if (elect_one()) {
                const uint64_t ad = umma_desc(sbase + s * STAGE_BYTES, 16, 1024);
                const uint64_t bd = umma_desc(sbase + s * STAGE_BYTES + TILE_BYTES, 16, 1024);
#pragma unroll
                for (int kk = 0; kk < BK / 16; kk++)
                    umma_ss(tmem, ad + (uint64_t)(kk * 2), bd + (uint64_t)(kk * 2), IDESC, (kb | (uint32_t)kk) != 0u ? 1u : 0u);
                umma_commit(&bar_empty[s]);                       // the stage is free once these MMAs have read it
                if (kb + 1 == (uint32_t)NKB && ok) umma_commit(&bar_acc);  // accumulator complete
            }
            __syncwarp();
        }
        if (!ok && lane == 0) atomicOr(p.status, DEV_WAIT_TIMEOUT);
    } else {
        // ===================== epilogue: thread = one row (token) of the tile =====================
        const uint32_t quarter = (uint32_t)warp_u & 3u;            // TMEM lanes this warp may read
        const uint32_t row = m_tile * BM + quarter * 32 + (uint32_t)lane;
        // warp-uniform: the tensor-memory loads below are warp-wide instructions
        const bool ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bar_acc, 0u, &s_abort));
        tc_fence_after();
        if (!ok) {
            if (lane == 0) atomicOr(p.status, DEV_WAIT_TIMEOUT);
        } else {
            proj_epilogue_cols<kQkvg>(tmem + ((quarter * 32) << 16), n_tile, row, row < p.rows, p, s_w);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp_u == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------
// The same GEMM for waves of rows (prefill): persistent, one CTA per SM, tiles of 128 rows x 256 features
// (two heads), a ring of four 48 KB stages, and TWO accumulators in tensor memory (2 x 256 of the 512
// columns) so that the epilogue of a tile runs while the tensor core works on the next one.
// Why the larger tile: with 128 x 128 tiles every k-block of 4 MMAs needs 32 KB from L2 (64 flop per
// byte); on the 4,096-row wave that kernel moved 11.7 TB/s from L2 into shared memory with the tensor
// pipe 39 % busy.  128 x 256 tiles need a third less per flop and a stage feeds twice the MMA time, so the
// same bytes in flight cover the L2 latency.
namespace pgw {
constexpr int BM = 128, BN = 256, BK = 64, NS = 4;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;  // 16 + 32 KB
constexpr int THREADS = 320;  // TMA warp, MMA warp, 8 epilogue warps: two per TMEM lane quarter, one per head of the tile
constexpr size_t SMEM_BYTES = 1024 + (size_t)NS * STAGE_BYTES;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t IDESC_N256 = (1u << 4) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
constexpr uint32_t IDESC_N16 = (1u << 4) | ((uint32_t)(16 >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);  // the gate tile
constexpr int TILES_QKVG = 8 + 2 + 2 + 1;
}  // namespace pgw

template <bool kQkvg>
__global__ void __launch_bounds__(pgw::THREADS, 1)
proj_gemm_wave_kernel(const __grid_constant__ ProjMaps maps, const ProjParams p, const uint32_t tiles_n, const uint32_t tiles_m) {
    using namespace pgw;
    constexpr int NKB = pg::NKB;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[NS], bar_empty[NS], bar_acc_full[2], bar_acc_empty[2];
    __shared__ uint32_t s_tmem, s_abort;
    __shared__ uint16_t s_w[2 * HD];

    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp_u = __shfl_sync(0xffffffffu, tid >> 5, 0);

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
        for (int b = 0; b < 2; b++) {
            mbar_init(&bar_acc_full[b], 1);
            mbar_init(&bar_acc_empty[b], 8);  // one arrival per epilogue warp
        }
        s_abort = 0u;
        mbar_fence_init();
    }
    if (kQkvg && tid >= 64 && tid < 64 + HD) {
        const int i = tid - 64;
        s_w[i] = p.q_norm_w[i];
        s_w[HD + i] = p.k_norm_w[i];
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    const uint32_t total = tiles_n * tiles_m;

    // tile t: feature tile nt = t % tiles_n (fastest, so CTAs that run together share the rows' x tiles), row tile t / tiles_n
    auto tile_weights = [&](uint32_t nt, uint32_t& wsel, uint32_t& wrow) {
        wsel = 0;
        wrow = nt * BN;
        if (kQkvg) {
            if (nt >= 12) { wsel = 3; wrow = 0; }
            else if (nt >= 10) { wsel = 2; wrow = (nt - 10) * BN; }
            else if (nt >= 8) { wsel = 1; wrow = (nt - 8) * BN; }
        }
    };

    if (warp_u == 0) {
        // ===================== TMA producer =====================
        pdl_wait();  // x is written by the kernel before this one
        bool ok = true;
        uint32_t g = 0;  // k-blocks issued by this CTA so far (ring position)
        for (uint32_t t = blockIdx.x; t < total && ok; t += gridDim.x) {
            uint32_t wsel, wrow;
            tile_weights(t % tiles_n, wsel, wrow);
            const uint32_t mrow = (t / tiles_n) * BM;
            for (uint32_t kb = 0; kb < (uint32_t)NKB; kb++, g++) {
                const uint32_t s = g % NS;
                if (g >= (uint32_t)NS && !mbar_wait_bounded(&bar_empty[s], ((g / NS) & 1u) ^ 1u, &s_abort)) {
                    ok = false;
                    break;
                }
                if (lane == 0) {
                    mbar_arrive_expect_tx(&bar_full[s], (uint32_t)STAGE_BYTES);
                    tma_load_box(sbase + s * STAGE_BYTES, &maps.x, kb * BK, mrow, &bar_full[s]);
                    tma_load_box(sbase + s * STAGE_BYTES + A_BYTES, &maps.w[wsel], kb * BK, wrow, &bar_full[s]);
                }
                __syncwarp();
            }
        }
        if (!ok) {
            if (lane == 0) atomicOr(p.status, DEV_WAIT_TIMEOUT);
            for (uint32_t k = g > (uint32_t)NS ? g - NS : 0; k < g; ++k)
                mbar_wait_drain(&bar_full[k % NS], (k / NS) & 1u, WAIT_LIMIT_US);
        }
    } else if (warp_u == 1) {
        // ===================== MMA issuer =====================
        bool ok = true;
        uint32_t g = 0, i = 0;
        for (uint32_t t = blockIdx.x; t < total; t += gridDim.x, i++) {
            const uint32_t buf = i & 1u;
            const uint32_t idesc = (kQkvg && t % tiles_n == 12u) ? IDESC_N16 : IDESC_N256;
            // the epilogue has drained this accumulator's previous tile
            if (i >= 2u) ok = __all_sync(0xffffffffu, ok && mbar_wait_bounded(&bar_acc_empty[buf], ((i >> 1) & 1u) ^ 1u, &s_abort));
            for (uint32_t kb = 0; kb < (uint32_t)NKB; kb++, g++) {
                const uint32_t s = g % NS;
                ok = __all_sync(0xffffffffu, ok && mbar_wait_bounded(&bar_full[s], (g / NS) & 1u, &s_abort));
                tc_fence_after();
                if (elect_one()) {
                    const uint64_t ad = umma_desc(sbase + s * STAGE_BYTES, 16, 1024);
                    const uint64_t bd = umma_desc(sbase + s * STAGE_BYTES + A_BYTES, 16, 1024);
#pragma unroll
                    for (int kk = 0; kk < BK / 16; kk++)
                        umma_ss(tmem + buf * 256u, ad + (uint64_t)(kk * 2), bd + (uint64_t)(kk * 2), idesc,
                                (kb | (uint32_t)kk) != 0u ? 1u : 0u);
                    umma_commit(&bar_empty[s]);
                    if (kb + 1 == (uint32_t)NKB && ok) umma_commit(&bar_acc_full[buf]);
                }
                __syncwarp();
            }
        }
        if (!ok && lane == 0) atomicOr(p.status, DEV_WAIT_TIMEOUT);
    } else {
        // ===================== epilogue warps: thread = one row of the tile, warp pair = the tile's two heads =====================
        const uint32_t quarter = (uint32_t)warp_u & 3u;          // TMEM lanes this warp may read
        const uint32_t group = ((uint32_t)warp_u - 2u) >> 2;     // which 128 features of the tile
        bool ok = true;
        uint32_t i = 0;
        for (uint32_t t = blockIdx.x; t < total && ok; t += gridDim.x, i++) {
            const uint32_t buf = i & 1u, nt = t % tiles_n;
            const uint32_t row = (t / tiles_n) * BM + quarter * 32 + (uint32_t)lane;
            ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bar_acc_full[buf], (i >> 1) & 1u, &s_abort));
            tc_fence_after();
            if (!ok) {
                if (lane == 0) atomicOr(p.status, DEV_WAIT_TIMEOUT);
                break;
            }
            const uint32_t t_row = tmem + ((quarter * 32) << 16) + buf * 256u;
            // the tile's two groups of 128 features (qkvg: two heads; the gate tile has one group)
            uint32_t ct0 = 2u * nt;
            bool two = true;
            if (kQkvg) {
                if (nt >= 12u) { ct0 = 24u; two = false; }
                else if (nt >= 10u) ct0 = 20u + 2u * (nt - 10u);
                else if (nt >= 8u) ct0 = 16u + 2u * (nt - 8u);
            } else {
                two = (ct0 + 1u) * 128u < p.out_features;
            }
            if (group == 0u || two) proj_epilogue_cols<kQkvg>(t_row + group * 128u, ct0 + group, row, row < p.rows, p, s_w);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_acc_empty[buf]);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp_u == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

cudaError_t proj_gemm_init() {
    cudaError_t e = cudaFuncSetAttribute(proj_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pg::SMEM_BYTES);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(proj_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pg::SMEM_BYTES);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(proj_gemm_wave_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pgw::SMEM_BYTES);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(proj_gemm_wave_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pgw::SMEM_BYTES);
    return e;
}

// Encodes a tiled map over a row-major [rows][2048] f16 matrix: box = 64 elements x box_rows (128 or 256) rows, 128-byte swizzle,
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

// rows up to this many run the one-tile-per-CTA kernel (more CTAs for a single row tile), larger waves the persistent one
constexpr uint32_t PROJ_SMALL_ROWS = 256;

cudaError_t launch_project_append(cudaStream_t stream, const TmaDesc* w_maps /* q, k, v, gate; box 128 then box 256 */, int num_sms, const void* x, uint32_t rows,
                                  void* q_out, void* gate_out, void* raw_out, const void* q_norm_w, const void* k_norm_w,
                                  const void* cos_t, const void* sin_t, const uint32_t* pos_ids, const uint64_t* k_ptrs,
                                  const uint64_t* v_ptrs, float eps, uint32_t* status) {
    ProjMaps maps;
    if (proj_encode_map(&maps.x, x, rows, pg::BM) != 0) return cudaErrorInvalidValue;
    const bool wave = rows > PROJ_SMALL_ROWS;
    for (int i = 0; i < 4; i++) maps.w[i] = w_maps[wave ? 4 + i : i];
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
    const uint32_t tiles_m = (rows + pg::BM - 1) / pg::BM;
    if (wave) {
        const uint32_t total = (uint32_t)pgw::TILES_QKVG * tiles_m;
        return launch_pdl(proj_gemm_wave_kernel<true>, dim3(total < (uint32_t)num_sms ? total : (uint32_t)num_sms),
                          dim3(pgw::THREADS), pgw::SMEM_BYTES, stream, maps, p, (uint32_t)pgw::TILES_QKVG, tiles_m);
    }
    return launch_pdl(proj_gemm_kernel<true>, dim3(pg::TILES_QKVG, tiles_m), dim3(pg::THREADS), pg::SMEM_BYTES, stream, maps, p);
}

cudaError_t launch_linear(cudaStream_t stream, const TmaDesc* w_maps /* box 128, box 256 */, int num_sms, uint32_t out_features,
                          const void* x, uint32_t rows, void* y, uint32_t* status) {
    ProjMaps maps;
    if (proj_encode_map(&maps.x, x, rows, pg::BM) != 0) return cudaErrorInvalidValue;
    const bool wave = rows > PROJ_SMALL_ROWS;
    maps.w[0] = maps.w[1] = maps.w[2] = maps.w[3] = w_maps[wave ? 1 : 0];
    ProjParams p = {};
    p.rows = rows;
    p.out_features = out_features;
    p.y = (uint16_t*)y;
    p.status = status;
    const uint32_t tiles_m = (rows + pg::BM - 1) / pg::BM;
    if (wave) {
        const uint32_t tiles_n = (out_features + pgw::BN - 1) / pgw::BN, total = tiles_n * tiles_m;
        return launch_pdl(proj_gemm_wave_kernel<false>, dim3(total < (uint32_t)num_sms ? total : (uint32_t)num_sms),
                          dim3(pgw::THREADS), pgw::SMEM_BYTES, stream, maps, p, tiles_n, tiles_m);
    }
    return launch_pdl(proj_gemm_kernel<false>, dim3((out_features + pg::BN - 1) / pg::BN, tiles_m), dim3(pg::THREADS),
                      pg::SMEM_BYTES, stream, maps, p);
}

}  // namespace oxi
