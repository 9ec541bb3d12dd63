// Fused per-head Q/K RMSNorm + RoPE + KV append, and the unfused operators
// with the reference's semantics (batched_attn.rs:13-118, 128-219, 233-287,
// 583-655).  Arithmetic order follows the reference instruction for
// instruction so q, K and V bytes match its kernels exactly on the same GPU:
// lane l sums dims l, l+32, l+64, l+96 with fma, the warp reduces with a
// shfl.down tree, mean = div.approx(sum, 128), r = rsqrt.approx(mean + eps),
// y = f16((x*r)*w); then on the f16-rounded y: f16(fma(+-y[d^64], sin, y*cos)).
#include "common.cuh"
#include "kernels.h"
#include "norm_rope.cuh"

namespace oxi {

// A CTA takes APPEND_ROWS rows; five warps per row: warps 0..3 of a row own four query heads each,
// the fifth the four K heads, so that the row's cos / sin vectors are fetched once per warp and the
// loads of four heads are in flight together (a prefill wave appends thousands of rows).  The
// first 64 threads of a row's warps also copy the 1 KB V row with 16-byte vectors.
// Two rows per CTA measured best on a 4,096-row wave (one: the same; four: 9 us slower; six: 7 us slower).
#ifndef OXI_APPEND_ROWS
#define OXI_APPEND_ROWS 2
#endif
constexpr int APPEND_ROWS = OXI_APPEND_ROWS;
__global__ void __launch_bounds__(APPEND_ROWS * 160)
append_kernel(uint16_t* __restrict__ q_io, const uint16_t* __restrict__ k_in,
              const uint16_t* __restrict__ v_in, const uint16_t* __restrict__ q_norm_w,
              const uint16_t* __restrict__ k_norm_w, const uint16_t* __restrict__ cos_t,
              const uint16_t* __restrict__ sin_t, const uint32_t* __restrict__ pos_ids,
              const uint64_t* __restrict__ k_ptrs, const uint64_t* __restrict__ v_ptrs, float eps,
              uint32_t* __restrict__ status, const PagedMap pm, uint32_t batch) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t b = blockIdx.x * APPEND_ROWS + (uint32_t)(warp / 5);
    const int wq = warp % 5;  // 0..3: query heads 4*wq .. 4*wq+3; 4: the K heads
    const int tid_row = threadIdx.x - (warp / 5) * 160;
    pdl_launch_dependents();
    if (b >= batch) {
        pdl_wait();
        return;
    }
    // the step's tables, norm weights and RoPE rows are not written by any kernel: fetch them
    // while the preceding kernel is still draining
    const uint32_t pos = pos_ids[b];
    uint64_t kp, vp;
    bool page_ok = true;
    if (pm.block_tables) {
        // paged: the base that puts row `pos` at its slot of its block (base + pos * row bytes, as below)
        const uint32_t pg = pos >> pm.lbs;
        uint32_t id = 0;
        if (pg >= pm.max_blocks) {
            page_ok = false;
            if (tid_row == 0) atomicOr(status, DEV_BAD_SEQ_LEN);
        } else {
            id = pm.block_tables[(size_t)b * pm.max_blocks + pg];
            if (id >= pm.num_blocks) {
                page_ok = false;
                if (tid_row == 0) atomicOr(status, DEV_BAD_BLOCK);
            }
        }
        const uint64_t off = (uint64_t)id * pm.block_stride + (uint64_t)(pos & ((1u << pm.lbs) - 1u)) * KV_ROW_BYTES -
                             (uint64_t)pos * KV_ROW_BYTES;
        kp = (uint64_t)(uintptr_t)pm.k_pool + off;
        vp = (uint64_t)(uintptr_t)pm.v_pool + off;
    } else {
        kp = k_ptrs[b];
        vp = v_ptrs[b];
    }
    float wv[4], cv[4], sv[4];
    load4(wq < 4 ? q_norm_w : k_norm_w, lane, wv);
    load4(cos_t + (size_t)pos * HD, lane, cv);
    load4(sin_t + (size_t)pos * HD, lane, sv);
    pdl_wait();  // q/k/v come from the preceding kernel; the caches may still be read by it
    const bool aligned = page_ok && ((kp | vp) & 15ull) == 0ull;
    if (!aligned && page_ok && tid_row == 0) atomicOr(status, DEV_MISALIGNED_PTR);
    // four heads: all loads first (q is normalised in place, so later loads must not wait for earlier stores)
    const uint16_t* xin = wq < 4 ? q_io + ((size_t)b * NQ + wq * 4) * HD : k_in + (size_t)b * NKV * HD;
    float x[4][4];
    uint16_t x16[4][4];
#pragma unroll
    for (int hh = 0; hh < 4; hh++)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            x16[hh][i] = xin[hh * HD + lane + 32 * i];
            x[hh][i] = h2f(x16[hh][i]);
        }
    uint16_t* xout = wq < 4 ? q_io + ((size_t)b * NQ + wq * 4) * HD
                            : reinterpret_cast<uint16_t*>(kp) + (size_t)pos * (NKV * HD);
    const bool store = wq < 4 || aligned;
#pragma unroll
    for (int hh = 0; hh < 4; hh++) {
        uint16_t out[4];
        head_norm_rope_vals<true, true>(x[hh], x16[hh], wv, eps, cv, sv, out);
        if (store) {
#pragma unroll
            for (int i = 0; i < 4; i++) xout[hh * HD + lane + 32 * i] = out[i];
        }
    }
    if (tid_row < 64 && aligned) {
        const uint4* src = reinterpret_cast<const uint4*>(v_in + (size_t)b * (NKV * HD));
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(vp) + (size_t)pos * KV_ROW_BYTES);
        dst[tid_row] = src[tid_row];
    }
}

__global__ void __launch_bounds__(128)
qk_rmsnorm_kernel(uint16_t* __restrict__ x_io, const uint16_t* __restrict__ w, float eps,
                  uint32_t total_heads) {
    const uint32_t head = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (head >= total_heads) return;
    uint16_t out[4];
    uint16_t* xh = x_io + (size_t)head * HD;
    const int lane = threadIdx.x & 31;
    float wv[4];
    const float none[4] = {0.f, 0.f, 0.f, 0.f};
    load4(w, lane, wv);
    head_norm_rope<true, false>(xh, wv, eps, none, none, lane, out);
#pragma unroll
    for (int i = 0; i < 4; i++) xh[lane + 32 * i] = out[i];
}

__global__ void __launch_bounds__(128)
rope_kernel(uint16_t* __restrict__ x_io, const uint16_t* __restrict__ cos_t,
            const uint16_t* __restrict__ sin_t, const uint32_t* __restrict__ pos_ids,
            uint32_t heads, uint32_t total_heads) {
    const uint32_t head = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (head >= total_heads) return;
    const uint32_t pos = pos_ids[head / heads];
    uint16_t out[4];
    uint16_t* xh = x_io + (size_t)head * HD;
    const int lane = threadIdx.x & 31;
    float cv[4], sv[4];
    const float none[4] = {0.f, 0.f, 0.f, 0.f};
    load4(cos_t + (size_t)pos * HD, lane, cv);
    load4(sin_t + (size_t)pos * HD, lane, sv);
    head_norm_rope<false, true>(xh, none, 0.0f, cv, sv, lane, out);
#pragma unroll
    for (int i = 0; i < 4; i++) xh[lane + 32 * i] = out[i];
}

__global__ void __launch_bounds__(64)
kv_copy_kernel(const uint64_t* __restrict__ dst_ptrs, const uint16_t* __restrict__ src,
               const uint32_t* __restrict__ pos_ids, uint32_t* __restrict__ status) {
    const uint32_t b = blockIdx.x;
    const uint64_t dp = dst_ptrs[b];
    if (dp & 15ull) {
        if (threadIdx.x == 0) atomicOr(status, DEV_MISALIGNED_PTR);
        return;
    }
    const uint4* s = reinterpret_cast<const uint4*>(src + (size_t)b * (NKV * HD));
    uint4* d = reinterpret_cast<uint4*>(reinterpret_cast<char*>(dp) + (size_t)pos_ids[b] * KV_ROW_BYTES);
    d[threadIdx.x] = s[threadIdx.x];
}

__global__ void __launch_bounds__(128)
sigmoid_gate_kernel(uint16_t* __restrict__ ctx_io, const uint16_t* __restrict__ gate) {
    const uint32_t bh = blockIdx.x;  // b*16 + head
    const float sig = sigmoid_ref(h2f(gate[bh]));
    uint16_t* p = ctx_io + (size_t)bh * HD + threadIdx.x;
    *p = f2h(__fmul_rn(h2f(*p), sig));
}

// pos_ids[b] += delta, seq_lens[b] += delta: the step tables advance on the device, so a captured
// graph of a decode step can be replayed for consecutive tokens without any upload.
// Kernels of this library read the step tables in their prologue, BEFORE their own
// griddepcontrol.wait (the tables are normally complete before the preceding kernel starts).  A
// kernel that WRITES the tables must therefore release its dependents only after its writes are
// visible device-wide: wait for the predecessors (they still read the old tables), write, fence,
// and only then trigger.  A dependent launched behind this kernel cannot start before every CTA
// has passed the fence, so its prologue sees the advanced tables.
__global__ void __launch_bounds__(256)
advance_step_kernel(uint32_t* __restrict__ pos_ids, uint32_t* __restrict__ seq_lens, uint32_t batch, uint32_t delta) {
    const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_wait();  // the preceding step's kernels still read the tables
    if (b < batch) {
        if (pos_ids) pos_ids[b] += delta;
        if (seq_lens) seq_lens[b] += delta;
    }
    __threadfence();
    __syncthreads();
    pdl_launch_dependents();
}

// seq_lens[b] = pos_ids[b] + 1 (batch_engine.rs:689-691): the host-buffer entry uploads positions
// only and derives the lengths here, so nothing is computed on the CPU at enqueue time.  Launched
// as a plain kernel on the upload stream; consumers are ordered behind it by an event.
__global__ void __launch_bounds__(256)
len_from_pos_kernel(const uint32_t* __restrict__ pos_ids, uint32_t* __restrict__ seq_lens, uint32_t batch) {
    const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < batch) seq_lens[b] = pos_ids[b] + 1u;
}

cudaError_t launch_advance_step(cudaStream_t stream, uint32_t* pos_ids, uint32_t* seq_lens, uint32_t batch,
                                uint32_t delta) {
    return launch_pdl(advance_step_kernel, dim3((batch + 255) / 256), dim3(256), 0, stream, pos_ids, seq_lens, batch,
                      delta);
}

cudaError_t launch_len_from_pos(cudaStream_t stream, const uint32_t* pos_ids, uint32_t* seq_lens, uint32_t batch) {
    len_from_pos_kernel<<<(batch + 255) / 256, 256, 0, stream>>>(pos_ids, seq_lens, batch);
    return cudaGetLastError();
}

cudaError_t launch_append(cudaStream_t stream, void* q_io, const void* k_in, const void* v_in,
                          const void* q_norm_w, const void* k_norm_w, const void* cos_t,
                          const void* sin_t, const uint32_t* pos_ids, const uint64_t* k_ptrs,
                          const uint64_t* v_ptrs, uint32_t batch, float eps, uint32_t* status) {
    return launch_pdl(append_kernel, dim3((batch + APPEND_ROWS - 1) / APPEND_ROWS), dim3(APPEND_ROWS * 160), 0, stream,
                      (uint16_t*)q_io, (const uint16_t*)k_in, (const uint16_t*)v_in, (const uint16_t*)q_norm_w,
                      (const uint16_t*)k_norm_w, (const uint16_t*)cos_t, (const uint16_t*)sin_t, pos_ids,
                      k_ptrs, v_ptrs, eps, status, PagedMap{}, batch);
}

cudaError_t launch_append_paged(cudaStream_t stream, void* q_io, const void* k_in, const void* v_in,
                                const void* q_norm_w, const void* k_norm_w, const void* cos_t,
                                const void* sin_t, const uint32_t* pos_ids, const PagedMap& pm,
                                uint32_t batch, float eps, uint32_t* status) {
    return launch_pdl(append_kernel, dim3((batch + APPEND_ROWS - 1) / APPEND_ROWS), dim3(APPEND_ROWS * 160), 0, stream,
                      (uint16_t*)q_io, (const uint16_t*)k_in, (const uint16_t*)v_in, (const uint16_t*)q_norm_w,
                      (const uint16_t*)k_norm_w, (const uint16_t*)cos_t, (const uint16_t*)sin_t, pos_ids,
                      (const uint64_t*)nullptr, (const uint64_t*)nullptr, eps, status, pm, batch);
}

cudaError_t launch_qk_rmsnorm(cudaStream_t stream, void* x_io, const void* w, float eps,
                              uint32_t heads, uint32_t batch) {
    const uint32_t total = heads * batch;
    qk_rmsnorm_kernel<<<(total + 3) / 4, 128, 0, stream>>>((uint16_t*)x_io, (const uint16_t*)w,
                                                           eps, total);
    return cudaGetLastError();
}

cudaError_t launch_rope(cudaStream_t stream, void* x_io, const void* cos_t, const void* sin_t,
                        const uint32_t* pos_ids, uint32_t heads, uint32_t batch) {
    const uint32_t total = heads * batch;
    rope_kernel<<<(total + 3) / 4, 128, 0, stream>>>((uint16_t*)x_io, (const uint16_t*)cos_t,
                                                     (const uint16_t*)sin_t, pos_ids, heads,
                                                     total);
    return cudaGetLastError();
}

cudaError_t launch_kv_copy(cudaStream_t stream, const uint64_t* dst_ptrs, const void* src,
                           const uint32_t* pos_ids, uint32_t batch, uint32_t* status) {
    kv_copy_kernel<<<batch, 64, 0, stream>>>(dst_ptrs, (const uint16_t*)src, pos_ids, status);
    return cudaGetLastError();
}

cudaError_t launch_sigmoid_gate(cudaStream_t stream, void* ctx_io, const void* gate,
                                uint32_t batch) {
    sigmoid_gate_kernel<<<batch * NQ, 128, 0, stream>>>((uint16_t*)ctx_io, (const uint16_t*)gate);
    return cudaGetLastError();
}

}  // namespace oxi
