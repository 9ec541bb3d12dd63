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
// A thread walks PF_ROWS consecutive wave rows for its 4 channels and keeps the 6 history products
// in registers: while the next row continues the same chunk the window just slides (one f16 product
// in, one out), otherwise it is rebuilt from the chunk's earlier rows of `bcx` and / or the carried
// state.  Every row of bcx is thus read (PF_ROWS + 6) / PF_ROWS times instead of 7; PF_ROWS is kept small
// because a wave has few rows (4096 x 512 thread columns) and rows of a thread are sequential.
#ifndef OXI_PF_ROWS
#define OXI_PF_ROWS 8
#endif
constexpr int PF_ROWS = OXI_PF_ROWS;  // consecutive wave rows per thread

__global__ void __launch_bounds__(128)
conv_prefill_kernel(uint16_t* __restrict__ y_out, const uint64_t* __restrict__ carry_ptrs,
                    const uint32_t* __restrict__ origin, const uint32_t* __restrict__ local_pos,
                    const uint16_t* __restrict__ bcx, const uint16_t* __restrict__ conv_w,
                    uint32_t rows, uint16_t* __restrict__ stage, uint32_t* __restrict__ status) {
    const uint32_t r_begin = blockIdx.y * PF_ROWS;
    const uint32_t r_end = min(rows, r_begin + (uint32_t)PF_ROWS);
    const uint32_t c0 = (blockIdx.x * 128 + threadIdx.x) * 4;

    union { uint2 v[7]; uint16_t h[28]; } w;
#pragma unroll
    for (int i = 0; i < 7; i++) w.v[i] = __ldg(reinterpret_cast<const uint2*>(conv_w + (size_t)c0 * CONV_K) + i);

    // taps[k][ch]: history products as f16 bit patterns, k = 0 oldest
    uint16_t taps[CONV_S][4];
    int32_t prev_org = -1, prev_lpos = -2;  // the row whose new state `taps` holds
    for (uint32_t r = r_begin; r < r_end; r++) {
        const uint16_t* row = bcx + (size_t)r * 3 * HIDDEN;
        union { uint2 v; uint16_t h[4]; } vb, vc, vx, vy;
        vb.v = *reinterpret_cast<const uint2*>(row + c0);
        vc.v = *reinterpret_cast<const uint2*>(row + HIDDEN + c0);
        vx.v = *reinterpret_cast<const uint2*>(row + 2 * HIDDEN + c0);
        const uint64_t cp = carry_ptrs[r];
        if (cp & 15ull) {
            if (threadIdx.x == 0 && blockIdx.x == 0) atomicOr(status, DEV_MISALIGNED_PTR);
            prev_org = -1;
            continue;
        }
        const int32_t org = (int32_t)origin[r];
        const int32_t lpos = (int32_t)local_pos[r];
        const bool last = (r + 1 == rows) || (origin[r + 1] != origin[r]);
        if (!(org == prev_org && lpos == prev_lpos + 1)) {
            // not the continuation of the row before: build the window from scratch
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
                        for (int ch = 0; ch < 4; ch++) taps[k][ch] = cs.h[ch * CONV_S + (j + CONV_S)];
                    }
                }
            }
#pragma unroll
            for (int k = 0; k < CONV_S; k++) {
                const int32_t j = lpos + k - CONV_S;
                if (j >= 0) {
                    const uint16_t* src = bcx + (size_t)(org + j) * 3 * HIDDEN;
                    union { uint2 v; uint16_t h[4]; } pb, px;
                    pb.v = *reinterpret_cast<const uint2*>(src + c0);
                    px.v = *reinterpret_cast<const uint2*>(src + 2 * HIDDEN + c0);
#pragma unroll
                    for (int ch = 0; ch < 4; ch++) taps[k][ch] = f2h(__fmul_rn(h2f(pb.h[ch]), h2f(px.h[ch])));
                }
            }
        }
#pragma unroll
        for (int ch = 0; ch < 4; ch++) {
            const float fin = __fmul_rn(h2f(vb.h[ch]), h2f(vx.h[ch]));
            float acc = 0.0f;
#pragma unroll
            for (int k = 0; k < CONV_S; k++)
                acc = __fmaf_rn(h2f(taps[k][ch]), h2f(w.h[ch * CONV_K + k]), acc);
            acc = __fmaf_rn(fin, h2f(w.h[ch * CONV_K + CONV_S]), acc);
            vy.h[ch] = f2h(__fmul_rn(acc, h2f(vc.h[ch])));
            // the row's new state, which is the next row's window if that row continues the chunk
#pragma unroll
            for (int k = 0; k < CONV_S - 1; k++) taps[k][ch] = taps[k + 1][ch];
            taps[CONV_S - 1][ch] = f2h(fin);
        }
        *reinterpret_cast<uint2*>(y_out + (size_t)r * HIDDEN + c0) = vy.v;
        if (last) {  // state layout [channel][slot]: half i of the 24 is channel i / 6, slot i % 6
            uint4* dst = reinterpret_cast<uint4*>(stage + ((size_t)r * HIDDEN + c0) * CONV_S);
            uint32_t pw[12];
#pragma unroll
            for (int i = 0; i < 12; i++)
                pw[i] = (uint32_t)taps[(2 * i) % CONV_S][(2 * i) / CONV_S] |
                        ((uint32_t)taps[(2 * i + 1) % CONV_S][(2 * i + 1) / CONV_S] << 16);
#pragma unroll
            for (int i = 0; i < 3; i++) dst[i] = make_uint4(pw[4 * i], pw[4 * i + 1], pw[4 * i + 2], pw[4 * i + 3]);
        }
        prev_org = org;
        prev_lpos = lpos;
    }
}

// Prefill, pass 2: the staged final state of every chunk replaces the
// request's persistent state.
constexpr int COMMIT_ROWS = PF_ROWS;  // wave rows scanned per CTA (64 measured slower: the scan is serial)
__global__ void __launch_bounds__(128)
conv_commit_kernel(const uint64_t* __restrict__ carry_ptrs, const uint32_t* __restrict__ origin,
                   uint32_t rows, const uint16_t* __restrict__ stage) {
    const uint32_t c0 = (blockIdx.x * 128 + threadIdx.x) * 4;
    const uint32_t r_end = min(rows, (blockIdx.y + 1) * (uint32_t)COMMIT_ROWS);
    for (uint32_t r = blockIdx.y * COMMIT_ROWS; r < r_end; r++) {  // chunk ends are rare: most rows only read origin
        const bool last = (r + 1 == rows) || (origin[r + 1] != origin[r]);
        if (!last) continue;
        const uint64_t cp = carry_ptrs[r];
        if (cp & 15ull) continue;
        const uint4* src = reinterpret_cast<const uint4*>(stage + ((size_t)r * HIDDEN + c0) * CONV_S);
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(cp) + (size_t)c0 * CONV_S);
#pragma unroll
        for (int i = 0; i < 3; i++) dst[i] = src[i];
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
    dim3 grid_pf(HIDDEN / 512, (rows + PF_ROWS - 1) / PF_ROWS);
    conv_prefill_kernel<<<grid_pf, 128, 0, stream>>>((uint16_t*)y_out, carry_ptrs, origin, local_pos,
                                                  (const uint16_t*)bcx, (const uint16_t*)conv_w,
                                                  rows, (uint16_t*)stage, status);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    dim3 grid_c(HIDDEN / 512, (rows + COMMIT_ROWS - 1) / COMMIT_ROWS);
    conv_commit_kernel<<<grid_c, 128, 0, stream>>>(carry_ptrs, origin, rows, (const uint16_t*)stage);
    return cudaGetLastError();
}

}  // namespace oxi
