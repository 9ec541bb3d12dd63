// Read-only HBM streaming probe: the decode kernel's memory pipeline with the arithmetic taken
// out.  One persistent CTA per SM; a producer warp issues 1-D bulk copies (TMA engine, no
// multicast, L2 evict_first) into a ring of shared-memory stages that complete on mbarriers; four
// consumer warps only wait for a stage, touch one word of it and hand it back; work items of
// 512 KB are claimed from a global counter like the decode kernel's.  What this
// sustains is the ceiling of any kernel that reads a stream once through that pipeline - the
// yardstick for the decode kernel beside the read+write copy bandwidth.  No counterpart in the
// reference; used by bench.py and the tests only.
#include "common.cuh"
#include "kernels.h"

namespace oxi {

namespace probe {
constexpr int NSTAGE = 3;
constexpr uint32_t STAGE_BYTES = 65536;  // the decode kernel stages 32 keys x 2 KB = 64 KB
constexpr int THREADS = 160;             // 4 consumer warps + the producer warp
constexpr uint32_t UNIT = 8;             // stages per claimed work item
constexpr size_t SMEM_BYTES = (size_t)NSTAGE * STAGE_BYTES + 2 * NSTAGE * 8 + 32;
}  // namespace probe

__global__ void __launch_bounds__(probe::THREADS, 1)
stream_read_kernel(const unsigned char* __restrict__ src, uint64_t total_bytes, uint32_t copy_bytes,
                   uint32_t* __restrict__ sink, uint32_t* __restrict__ counter, uint32_t* __restrict__ status) {
    using namespace probe;
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)NSTAGE * STAGE_BYTES);
    uint64_t* empty = full + NSTAGE;
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(empty + NSTAGE);
    volatile uint32_t* s_end = abort_flag + 1;  // [NSTAGE]: the stage is the end-of-work marker
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();  // the next launch may set up its barriers while this one streams
    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGE; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], THREADS / 32 - 1);
        }
        *abort_flag = 0u;
        mbar_fence_init();
    }
    __syncthreads();
    pdl_wait();  // the launch before this one resets the claim counter when its last CTA leaves
    // work items of UNIT stages (512 KB, the size of a decode work item), claimed from a global counter
    // two items ahead like the decode kernel: SMs that get less memory bandwidth take fewer items
    const uint64_t nstages = total_bytes / STAGE_BYTES;
    const uint32_t nitems = (uint32_t)((nstages + UNIT - 1) / UNIT);
    if (warp == THREADS / 32 - 1) {
        const uint64_t policy = l2_policy_evict_first();
        const uint32_t ncopies = STAGE_BYTES / copy_bytes;
        uint32_t fill = 0;
        bool ok = true;
        uint32_t cur = blockIdx.x, claim = 0;
        if (lane == 0 && cur < nitems) claim = atomicAdd(counter, 1u);
        while (cur < nitems && ok) {
            uint32_t nxt = __shfl_sync(0xffffffffu, claim, 0);
            nxt = nxt >= nitems ? nitems : min(nxt + gridDim.x, nitems);
            claim = 0xffffffffu;
            if (nxt < nitems && lane == 0) claim = atomicAdd(counter, 1u);
            const uint64_t st1 = min((uint64_t)(cur + 1u) * UNIT, nstages);
            for (uint64_t st = (uint64_t)cur * UNIT; st < st1; ++st, ++fill) {
                const uint32_t slot = fill % NSTAGE;
                if (fill >= NSTAGE && !mbar_wait_bounded(&empty[slot], ((fill / NSTAGE) & 1u) ^ 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                if (lane == 0) {
                    s_end[slot] = 0u;
                    mbar_arrive_expect_tx(&full[slot], STAGE_BYTES);
                }
                __syncwarp();
                for (uint32_t i = lane; i < ncopies; i += 32)
                    bulk_g2s_hint(smem_u32(smem + (size_t)slot * STAGE_BYTES + (size_t)i * copy_bytes),
                                  src + st * STAGE_BYTES + (size_t)i * copy_bytes, copy_bytes, &full[slot], policy);
            }
            cur = nxt;
        }
        if (ok) {
            const uint32_t slot = fill % NSTAGE;
            if (fill < NSTAGE || mbar_wait_bounded(&empty[slot], ((fill / NSTAGE) & 1u) ^ 1u, abort_flag)) {
                if (lane == 0) {
                    s_end[slot] = 1u;
                    mbar_arrive(&full[slot]);
                }
                ++fill;
            } else {
                ok = false;
            }
        }
        if (!ok) {
            if (lane == 0) atomicOr(status, DEV_WAIT_TIMEOUT);
            for (uint32_t k = fill > NSTAGE ? fill - NSTAGE : 0; k < fill; ++k)
                mbar_wait_drain(&full[k % NSTAGE], (k / NSTAGE) & 1u, WAIT_LIMIT_US);
        }
        // this CTA claims nothing more; the last CTA to get here leaves both counters at zero for the next launch
        if (lane == 0 && atomicAdd(counter + 1, 1u) == gridDim.x - 1u) {
            counter[0] = 0u;
            counter[1] = 0u;
        }
        return;
    }
    uint32_t acc = 0;
    for (uint32_t take = 0;; ++take) {
        const uint32_t slot = take % NSTAGE;
        if (!mbar_wait_bounded(&full[slot], (take / NSTAGE) & 1u, abort_flag)) {
            if (lane == 0) atomicOr(status, DEV_WAIT_TIMEOUT);
            break;
        }
        if (s_end[slot]) break;
        acc += *reinterpret_cast<const uint32_t*>(smem + (size_t)slot * STAGE_BYTES + threadIdx.x * 4);
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[slot]);
    }
    if (acc == 0x9e3779b9u) *sink = acc;  // keeps the loads alive
}

cudaError_t stream_probe_init() {
    return cudaFuncSetAttribute(stream_read_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)probe::SMEM_BYTES);
}

cudaError_t launch_stream_read(cudaStream_t stream, const void* src, uint64_t bytes, uint32_t copy_bytes, int num_sms,
                               uint32_t* sink, uint32_t* status) {
    uint32_t* counter = sink + 1;  // claim counter and exit counter: zero between launches (the kernel resets them)
    return launch_pdl(stream_read_kernel, dim3(num_sms), dim3(probe::THREADS), probe::SMEM_BYTES, stream,
                      (const unsigned char*)src, (uint64_t)bytes, copy_bytes, sink, counter, status);
}

uint32_t stream_probe_stage_bytes() { return probe::STAGE_BYTES; }

}  // namespace oxi
