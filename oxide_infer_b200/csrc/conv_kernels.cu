// Causal depthwise conv1d (7 taps) with the 6-slot carry state and B/C gating.
//
// Decode: replaces batched_fused_causal_conv1d_gating_ptr_fp16
// (batched_attn.rs:727-881).  Prefill: replaces conv_state_prefill_fp16
// (batched_attn.rs:1049-1176) + the conv kernel on pool rows + the per-chunk
// state copy-back (server.rs:1192-1224) without materialising per-row states.
//
// Arithmetic kept from the reference so y and the state are bit-exact: the
// newest tap is the UNROUNDED f32 product B*x, history taps are the f16-rounded
// products, taps accumulate oldest first with fma from 0, y = f16(acc * C).
#include "common.cuh"
#include "kernels.h"

namespace oxi {

// 4 channels per thread: state 48 B (3 x 16-byte vectors), weights 56 B
// (7 x 8-byte vectors), B/C/x/y 8-byte vectors.  grid = (4, B), block = 128.
__global__ void __launch_bounds__(128)
conv_decode_kernel(uint16_t* __restrict__ y_out, const uint64_t* __restrict__ conv_ptrs,
                   const uint16_t* __restrict__ bcx, const uint16_t* __restrict__ conv_w,
                   uint32_t* __restrict__ status) {
    const uint32_t b = blockIdx.y;
    const uint32_t c0 = (blockIdx.x * 128 + threadIdx.x) * 4;
    const uint64_t sp = conv_ptrs[b];
    if (sp & 15ull) {
        if (threadIdx.x == 0 && blockIdx.x == 0) atomicOr(status, DEV_MISALIGNED_PTR);
        return;
    }
    if (!OXI_IN_BOUNDS(c0 + 4u <= (uint32_t)HIDDEN, status)) return;  // bounds build: the thread's channels exist
    uint16_t* state = reinterpret_cast<uint16_t*>(sp) + (size_t)c0 * CONV_S;
    const uint16_t* row = bcx + (size_t)b * 3 * HIDDEN;

    union { uint4 v[3]; uint16_t h[24]; } st;
    union { uint2 v[7]; uint16_t h[28]; } w;
    union { uint2 v; uint16_t h[4]; } vb, vc, vx, vy;
#pragma unroll
    for (int i = 0; i < 3; i++) st.v[i] = reinterpret_cast<const uint4*>(state)[i];
#pragma unroll
    for (int i = 0; i < 7; i++) w.v[i] = __ldg(reinterpret_cast<const uint2*>(conv_w + (size_t)c0 * CONV_K) + i);
    vb.v = *reinterpret_cast<const uint2*>(row + c0);
    vc.v = *reinterpret_cast<const uint2*>(row + HIDDEN + c0);
    vx.v = *reinterpret_cast<const uint2*>(row + 2 * HIDDEN + c0);

#pragma unroll
    for (int ch = 0; ch < 4; ch++) {
        const float fin = __fmul_rn(h2f(vb.h[ch]), h2f(vx.h[ch]));
        float acc = 0.0f;
#pragma unroll
        for (int k = 0; k < CONV_S; k++)
            acc = __fmaf_rn(h2f(st.h[ch * CONV_S + k]), h2f(w.h[ch * CONV_K + k]), acc);
        acc = __fmaf_rn(fin, h2f(w.h[ch * CONV_K + CONV_S]), acc);
#pragma unroll
        for (int k = 0; k < CONV_S - 1; k++) st.h[ch * CONV_S + k] = st.h[ch * CONV_S + k + 1];
        st.h[ch * CONV_S + CONV_S - 1] = f2h(fin);
        vy.h[ch] = f2h(__fmul_rn(acc, h2f(vc.h[ch])));
    }
#pragma unroll
    for (int i = 0; i < 3; i++) reinterpret_cast<uint4*>(state)[i] = st.v[i];
    *reinterpret_cast<uint2*>(y_out + (size_t)b * HIDDEN + c0) = vy.v;
}

// Prefill, pass 1.  A row's six history taps are f16(B*x) of the wave rows origin+j
// (j = local_pos-6+k >= 0) or carry[c][6+j] (j < 0).  The chunk's last row also writes the state
// the request must carry forward into `stage[row]` (committed by pass 2, because other rows of the
// chunk may still be reading the carry state).
// A CTA takes CT_ROWS wave rows x CT_CH channels.  All its global loads are
// issued at once (B and x of the tile's rows and of the 6 rows before it, C and the tables of its own
// rows), the f32 products B*x go to shared memory, and after one barrier every thread forms the
// outputs of its rows from shared memory: history taps are the f16-rounded products of the six rows
// before (or carried state for the first six rows of a chunk), the newest tap the unrounded product.
// One memory round trip per CTA instead of one per row (a thread that walked 8 consecutive rows with the
// window in registers: 26.6 us for a 4096-row wave, this kernel 25.6 us; tiles of 32 rows or 128 channels
// measured 1-2 us slower); every row of bcx is fetched (CT_ROWS + 6) / CT_ROWS times, from L2.
#ifndef OXI_CT_ROWS
#define OXI_CT_ROWS 16
#endif
#ifndef OXI_CT_CH
#define OXI_CT_CH 256
#endif
#ifndef OXI_CT_PASS
#define OXI_CT_PASS 4
#endif
#ifndef OXI_CT_MINB
#define OXI_CT_MINB 4
#endif
constexpr int CT_ROWS = OXI_CT_ROWS, CT_CH = OXI_CT_CH, CT_PASS = OXI_CT_PASS;  // rows covered by the CTA at once
constexpr int CT_THREADS = CT_PASS * (CT_CH / 4), CT_HALO = CONV_S;
constexpr int CT_LOADS = (CT_ROWS + CT_HALO + CT_PASS - 1) / CT_PASS;  // row slots per thread in the load phase: 10
constexpr int CT_OUT = CT_ROWS / CT_PASS;                           // output rows per thread: 8

__global__ void __launch_bounds__(CT_THREADS, OXI_CT_MINB)
conv_prefill_kernel(uint16_t* __restrict__ y_out, const uint64_t* __restrict__ carry_ptrs,
                         const uint32_t* __restrict__ origin, const uint32_t* __restrict__ local_pos,
                         const uint16_t* __restrict__ bcx, const uint16_t* __restrict__ conv_w,
                         uint32_t rows, uint16_t* __restrict__ stage, uint32_t* __restrict__ status) {
    __shared__ __align__(16) float prod[CT_ROWS + CT_HALO][CT_CH];  // B*x, row i = wave row r_tile - 6 + i
    __shared__ uint64_t s_cp[CT_ROWS];
    __shared__ int32_t s_lpos[CT_ROWS];
    __shared__ uint32_t s_last[CT_ROWS];
    pdl_launch_dependents();
    const uint32_t r_tile = blockIdx.y * CT_ROWS;
    const uint32_t tx = threadIdx.x % (CT_CH / 4), ty = threadIdx.x / (CT_CH / 4);
    const uint32_t c0 = blockIdx.x * CT_CH + tx * 4;
    // launched as a programmatic dependent: bcx comes from the kernel before, and the carried states may
    // still be written by it (the previous layer's or wave's commit)
    pdl_wait();

    // ---- all loads
    union U2 { uint2 v; uint16_t h[4]; };
    U2 vb[CT_LOADS], vx[CT_LOADS], vc[CT_OUT];
#pragma unroll
    for (int it = 0; it < CT_LOADS; it++) {
        const int32_t i = (int32_t)ty + CT_PASS * it;
        const int64_t g = (int64_t)r_tile + i - CT_HALO;
        const bool valid = i < CT_ROWS + CT_HALO && g >= 0 && g < (int64_t)rows;
        const uint16_t* row = bcx + (size_t)(valid ? g : 0) * 3 * HIDDEN;
        vb[it].v = valid ? *reinterpret_cast<const uint2*>(row + c0) : make_uint2(0u, 0u);
        vx[it].v = valid ? *reinterpret_cast<const uint2*>(row + 2 * HIDDEN + c0) : make_uint2(0u, 0u);
    }
#pragma unroll
    for (int m = 0; m < CT_OUT; m++) {
        const uint32_t r = r_tile + ty + CT_PASS * m;
        vc[m].v = r < rows ? *reinterpret_cast<const uint2*>(bcx + (size_t)r * 3 * HIDDEN + HIDDEN + c0) : make_uint2(0u, 0u);
    }
    union { uint2 v[7]; uint16_t h[28]; } w;
#pragma unroll
    for (int i = 0; i < 7; i++) w.v[i] = __ldg(reinterpret_cast<const uint2*>(conv_w + (size_t)c0 * CONV_K) + i);
    if (threadIdx.x < CT_ROWS) {
        const uint32_t r = r_tile + threadIdx.x;
        if (r < rows) {
            s_cp[threadIdx.x] = carry_ptrs[r];
            s_lpos[threadIdx.x] = (int32_t)local_pos[r];
            s_last[threadIdx.x] = (r + 1 == rows) || (origin[r + 1] != origin[r]);
        }
    }
    // ---- products to shared memory
#pragma unroll
    for (int it = 0; it < CT_LOADS; it++) {
        const int32_t i = (int32_t)ty + CT_PASS * it;
        if (i < CT_ROWS + CT_HALO) {
            float4 f;
            f.x = __fmul_rn(h2f(vb[it].h[0]), h2f(vx[it].h[0]));
            f.y = __fmul_rn(h2f(vb[it].h[1]), h2f(vx[it].h[1]));
            f.z = __fmul_rn(h2f(vb[it].h[2]), h2f(vx[it].h[2]));
            f.w = __fmul_rn(h2f(vb[it].h[3]), h2f(vx[it].h[3]));
            *reinterpret_cast<float4*>(&prod[i][tx * 4]) = f;
        }
    }
    __syncthreads();

    // ---- outputs
#pragma unroll
    for (int m = 0; m < CT_OUT; m++) {
        const uint32_t lr = ty + CT_PASS * m, r = r_tile + lr;
        if (r >= rows) continue;
        const uint64_t cp = s_cp[lr];
        if (cp & 15ull) {
            if (tx == 0 && blockIdx.x == 0) atomicOr(status, DEV_MISALIGNED_PTR);
            continue;
        }
        const int32_t lpos = s_lpos[lr];
        // bounds build: a chunk position cannot lie before the wave's first row, and the staged state has a row per wave row
        if (!OXI_IN_BOUNDS(lpos >= 0 && (uint32_t)lpos <= r && c0 + 4u <= (uint32_t)HIDDEN, status)) continue;
        // slot k of the row's window: the product of chunk position lpos + k - 6, or carried state
        uint16_t win[CONV_S + 1][4];  // [k][channel]; k = 6 is the row's own product (its f16 form, for the state)
        if (lpos < CONV_S) {
            union { uint4 v[3]; uint16_t h[24]; } cs;
            const uint16_t* carry = reinterpret_cast<const uint16_t*>(cp) + (size_t)c0 * CONV_S;
#pragma unroll
            for (int i = 0; i < 3; i++) cs.v[i] = reinterpret_cast<const uint4*>(carry)[i];
#pragma unroll
            for (int k = 0; k < CONV_S; k++) {
                const int32_t j = lpos + k - CONV_S;
                if (j < 0) {
#pragma unroll
                    for (int ch = 0; ch < 4; ch++) win[k][ch] = cs.h[ch * CONV_S + (j + CONV_S)];
                }
            }
        }
#pragma unroll
        for (int k = 0; k <= CONV_S; k++) {
            if (k == CONV_S || lpos + k - CONV_S >= 0) {
                const float4 f = *reinterpret_cast<const float4*>(&prod[lr + k][tx * 4]);  // wave row r - 6 + k
                win[k][0] = f2h(f.x);
                win[k][1] = f2h(f.y);
                win[k][2] = f2h(f.z);
                win[k][3] = f2h(f.w);
            }
        }
        const float4 own = *reinterpret_cast<const float4*>(&prod[lr + CONV_S][tx * 4]);
        const float fin[4] = {own.x, own.y, own.z, own.w};
        U2 vy;
#pragma unroll
        for (int ch = 0; ch < 4; ch++) {
            float acc = 0.0f;
#pragma unroll
            for (int k = 0; k < CONV_S; k++) acc = __fmaf_rn(h2f(win[k][ch]), h2f(w.h[ch * CONV_K + k]), acc);
            acc = __fmaf_rn(fin[ch], h2f(w.h[ch * CONV_K + CONV_S]), acc);
            vy.h[ch] = f2h(__fmul_rn(acc, h2f(vc[m].h[ch])));
        }
        *reinterpret_cast<uint2*>(y_out + (size_t)r * HIDDEN + c0) = vy.v;
        if (s_last[lr]) {  // the chunk's new state: window slots 1 .. 6; layout [channel][slot]
            uint4* dst = reinterpret_cast<uint4*>(stage + ((size_t)r * HIDDEN + c0) * CONV_S);
            uint32_t pw[12];
#pragma unroll
            for (int i = 0; i < 12; i++)
                pw[i] = (uint32_t)win[(2 * i) % CONV_S + 1][(2 * i) / CONV_S] |
                        ((uint32_t)win[(2 * i + 1) % CONV_S + 1][(2 * i + 1) / CONV_S] << 16);
#pragma unroll
            for (int i = 0; i < 3; i++) dst[i] = make_uint4(pw[4 * i], pw[4 * i + 1], pw[4 * i + 2], pw[4 * i + 3]);
        }
    }
}

// Prefill, pass 2: the staged final state of every chunk replaces the
// request's persistent state.  A CTA looks at COMMIT_ROWS wave rows (one per thread) for chunk ends,
// then all its threads copy the state of each end it found (usually one), 4 channels per thread.
constexpr int COMMIT_ROWS = 128;
__global__ void __launch_bounds__(128)
conv_commit_kernel(const uint64_t* __restrict__ carry_ptrs, const uint32_t* __restrict__ origin,
                   uint32_t rows, const uint16_t* __restrict__ stage) {
    __shared__ uint32_t s_cnt[4];
    __shared__ uint32_t s_rows[COMMIT_ROWS];
    const uint32_t c0 = (blockIdx.x * 128 + threadIdx.x) * 4;
    const uint32_t r = blockIdx.y * COMMIT_ROWS + threadIdx.x;
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    // step inputs, not written by pass 1: read while it is still running
    const bool last = r < rows && ((r + 1 == rows) || (origin[r + 1] != origin[r]));
    const uint32_t mask = __ballot_sync(0xffffffffu, last);
    if (lane == 0) s_cnt[warp] = (uint32_t)__popc(mask);
    __syncthreads();
    uint32_t before = 0, n = 0;  // chunk ends are listed in row order
    for (uint32_t wv = 0; wv < 4; wv++) {
        before += wv < warp ? s_cnt[wv] : 0u;
        n += s_cnt[wv];
    }
    if (last) s_rows[before + (uint32_t)__popc(mask & ((1u << lane) - 1u))] = r;
    __syncthreads();
    pdl_wait();  // launched as a programmatic dependent of pass 1: resident early, reads `stage` only after it finished
    for (uint32_t i = 0; i < n; i++) {
        const uint32_t lr = s_rows[i];
        const uint64_t cp = carry_ptrs[lr];
        if (cp & 15ull) continue;
        const uint4* src = reinterpret_cast<const uint4*>(stage + ((size_t)lr * HIDDEN + c0) * CONV_S);
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(cp) + (size_t)c0 * CONV_S);
#pragma unroll
        for (int k = 0; k < 3; k++) dst[k] = src[k];
    }
}

cudaError_t launch_conv_decode(cudaStream_t stream, void* y_out, const uint64_t* conv_ptrs,
                               const void* bcx, const void* conv_w, uint32_t batch,
                               uint32_t* status) {
    dim3 grid(HIDDEN / 512, batch);
    conv_decode_kernel<<<grid, 128, 0, stream>>>((uint16_t*)y_out, conv_ptrs, (const uint16_t*)bcx,
                                                 (const uint16_t*)conv_w, status);
    return cudaGetLastError();
}

cudaError_t launch_conv_prefill(cudaStream_t stream, void* y_out, const uint64_t* carry_ptrs,
                                const uint32_t* origin, const uint32_t* local_pos,
                                const void* bcx, const void* conv_w, uint32_t rows, void* stage,
                                uint32_t* status) {
    dim3 grid_t(HIDDEN / CT_CH, (rows + CT_ROWS - 1) / CT_ROWS);
    cudaError_t e = launch_pdl(conv_prefill_kernel, grid_t, dim3(CT_THREADS), 0, stream, (uint16_t*)y_out, carry_ptrs, origin,
                               local_pos, (const uint16_t*)bcx, (const uint16_t*)conv_w, rows, (uint16_t*)stage, status);
    if (e != cudaSuccess) return e;
    dim3 grid_c(HIDDEN / 512, (rows + COMMIT_ROWS - 1) / COMMIT_ROWS);
    return launch_pdl(conv_commit_kernel, grid_c, dim3(128), 0, stream, carry_ptrs, origin, rows, (const uint16_t*)stage);
}

}  // namespace oxi
