// Device helpers shared by the sm_100a kernels: fp16 bit-exact primitives,
// mbarrier + bulk-copy (TMA) wrappers, ldmatrix / mma.sync wrappers.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace oxi {

constexpr int NQ = 16;        // query heads
constexpr int NKV = 4;        // KV heads
constexpr int HD = 128;       // head dim
constexpr int KV_ROW_BYTES = NKV * HD * 2;  // one token of K (or V): 1024 B
constexpr int HIDDEN = 2048;  // conv channels
constexpr int CONV_K = 7;     // taps
constexpr int CONV_S = 6;     // live state slots
constexpr float ATTN_SCALE = 0.0883883476f;  // 1/sqrt(128), the reference's literal
constexpr float LOG2E = 1.44269504f;

constexpr uint32_t DEV_MISALIGNED_PTR = 1u;
constexpr uint32_t DEV_BAD_SEQ_LEN = 2u;
constexpr uint32_t DEV_WAIT_TIMEOUT = 4u;
constexpr uint32_t DEV_BAD_TOKEN = 8u;
constexpr uint32_t DEV_BAD_BLOCK = 16u;
constexpr uint32_t DEV_OUT_OF_BOUNDS = 32u;  // only raised by builds with -DOXI_BOUNDS

// Builds with -DOXI_BOUNDS check the indices of every table-driven access (cache rows, partial
// slots, shared-memory stages, wave rows) and, instead of performing an access that is out of
// range, record DEV_OUT_OF_BOUNDS in the status word.  In normal builds the checks compile away.
#ifdef OXI_BOUNDS
#define OXI_IN_BOUNDS(cond, status_ptr) ((cond) ? true : (atomicOr((status_ptr), ::oxi::DEV_OUT_OF_BOUNDS), false))
#else
#define OXI_IN_BOUNDS(cond, status_ptr) true
#endif

// Test support: makes one pipeline stage of one CTA go missing so that the bounded waits run out.
// skip_plus1 == 0 (every normal launch): nothing is skipped and waits last WAIT_LIMIT_US.
struct WaitFault {
    uint32_t skip_plus1;  // CTA 0 withholds its (skip_plus1 - 1)-th stage / tile
    uint32_t limit_us;    // wait limit of this launch when armed
};

// Paged K/V layout of one layer: token t of row b lives in block block_tables[b][t >> lbs] at slot
// t & (2^lbs - 1); block i's K rows start at k_pool + i * block_stride (V: v_pool), one row =
// 4 KV heads x 128 f16 = 1024 bytes.  block_tables == nullptr means "not paged".
struct PagedMap {
    const unsigned char* k_pool;
    const unsigned char* v_pool;
    const uint32_t* block_tables;  // [batch][max_blocks]
    uint64_t block_stride;         // bytes between consecutive blocks of one pool (multiple of 16)
    uint32_t max_blocks;           // columns of block_tables
    uint32_t lbs;                  // log2(block size in tokens), 4 ... 8
    uint32_t num_blocks;           // blocks in the pool: larger ids are rejected
};

// ---- approximate instructions the reference uses (kept as PTX so results match bit for bit)
__device__ __forceinline__ float ex2_approx_ftz(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float rcp_approx_ftz(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float rsqrt_approx_ftz(float x) {
    float r;
    asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float div_approx_ftz(float a, float b) {
    float r;
    asm("div.approx.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}
// sigmoid exactly as batched_sigmoid_gate_fp16 computes it
__device__ __forceinline__ float sigmoid_ref(float g) {
    float e = ex2_approx_ftz(__fmul_rn(-g, LOG2E));
    return rcp_approx_ftz(__fadd_rn(e, 1.0f));
}

__device__ __forceinline__ float h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }
__device__ __forceinline__ uint16_t f2h(float f) { return __half_as_ushort(__float2half_rn(f)); }

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// ---- shared-memory addressing
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
constexpr uint32_t WAIT_LIMIT_US = 1000000u;  // in-kernel pipeline waits give up after about one second

// Bounded wait: gives up after limit_us microseconds, or at once when another wait of this CTA
// already gave up (*abort_flag != 0).  Returns false on give-up.  The limit is a kernel
// parameter only so that a test can make a wait run out in a millisecond.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity,
                                                  volatile uint32_t* abort_flag,
                                                  uint32_t limit_us = WAIT_LIMIT_US) {
    if (mbar_try_wait(bar, parity)) return true;
    uint64_t t0 = 0;
    // the flag and the clock are looked at every 256 polls only: the waiting warps share issue slots
    // with the warps that do the arithmetic
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 255u) == 0u) {
            if (*abort_flag) return false;
            uint64_t now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > (uint64_t)limit_us * 1000ull) {
                *abort_flag = 1u;
                return false;
            }
        }
    }
}

// Time-limited wait without the abort flag (used on the give-up path to let copies that were
// already issued land before the CTA's shared memory is released).
__device__ __forceinline__ bool mbar_wait_drain(uint64_t* bar, uint32_t parity, uint32_t limit_us) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t limit_ns = (uint64_t)limit_us * 1000ull;
    const uint64_t t0 = global_timer_ns();
    for (;;) {
        if (mbar_try_wait(bar, parity)) return true;
        if (global_timer_ns() - t0 > limit_ns) return false;
    }
}

// ---- 1-D bulk copy global -> shared (TMA engine), completion on an mbarrier.
// Both addresses 16-byte aligned, size a multiple of 16.  No multicast.
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void* src, uint32_t bytes,
                                         uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void bulk_g2s_hint(uint32_t dst_smem, const void* src, uint32_t bytes,
                                              uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1], %2, [%3], %4;"
        ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void st_global_f2_hint(float* addr, float a, float b, uint64_t policy) {
    asm volatile("st.global.L2::cache_hint.v2.f32 [%0], {%1, %2}, %3;" ::"l"(addr), "f"(a), "f"(b), "l"(policy) : "memory");
}
// Orders this thread's generic-proxy shared-memory writes before later
// async-proxy (bulk copy) accesses to the same locations.
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- tensor-core fragments (warp-level mma.sync, f16 in / f32 accumulate)
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                            uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                                  uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- programmatic dependent launch (PDL).  A kernel launched with launch_pdl() may begin
// while its predecessor in the stream is still running; it must execute pdl_wait() before
// it touches anything the predecessor (or, transitively, any earlier kernel) writes, and
// every such kernel executes pdl_wait() before it exits so the chain stays ordered.
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ uint32_t window_start(uint32_t slen, uint32_t window) {
    return (window != 0u && slen > window) ? slen - window : 0u;
}

// Host side: launch `kernel` so that it may overlap the tail of the previous kernel in `stream`.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace oxi
