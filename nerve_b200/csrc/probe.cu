// Peak-rate probe of the tensor-core instruction the expert kernels issue
// (tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale, 128 x N x 32 per instruction, E2M1 x E4M3).
//
// The roofline of a tensor-bound workload needs a measured denominator for the instruction kind that
// actually ran.  Every CTA (one per SM) issues a long run of MMAs on operands that already sit in
// shared memory, alternating between two accumulators exactly as the gate/up kernel alternates
// between its gate and up tiles, with the three scale copies in front of every four K steps.  Nothing
// is loaded from global memory, so the time is the tensor pipe's own: FLOP / time over all SMs is
// the rate no grouped-expert kernel of this shape can exceed.  No reference counterpart.
#include "common.cuh"
#include "tcgen05.cuh"

namespace nvmoe {
namespace {

using namespace tc;

struct ProbeBars {
    uint64_t done;
    uint32_t tmem_base;
    uint32_t abort;
};

constexpr uint32_t kProbeSmem = 16384u * 2u + 16384u + 2048u + 1024u + 256u;

__global__ void __launch_bounds__(160, 1) mma_rate_kernel(uint32_t n, uint32_t groups, long long* cycles, uint32_t* status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~uintptr_t(1023u));
    unsigned char *a_tile = smem, *a2_tile = smem + 16384, *b_tile = smem + 32768, *sf = smem + 32768 + 16384;
    ProbeBars* bars = reinterpret_cast<ProbeBars*>(sf + 2048);
    const uint32_t warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        mbar_init(&bars->done, 1);
        bars->abort = 0;
        fence_mbar_init();
    }
    // operands: every code 0x22 (E2M1 1.0 in the low nibble of a byte slot), every scale 127 (1.0)
    for (uint32_t i = threadIdx.x; i < (32768u + 16384u) / 4u; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0x22222222u;
    for (uint32_t i = threadIdx.x; i < 2048u / 4u; i += blockDim.x) reinterpret_cast<uint32_t*>(sf)[i] = 0x7f7f7f7fu;
    fence_proxy_async();
    __syncthreads();
    if (warp == 4u) {
        tmem_alloc(&bars->tmem_base, 512);
        tmem_relinquish();
        tc_fence_before();
    }
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;
    if (warp == 4u) {
        if (elect_one()) {
            const uint32_t idesc = idesc_mxf8f6f4(kFmtE2M1, kFmtE4M3, 128, n);
            const uint64_t ad = desc_k_major_sw128(smem_u32(a_tile)), ad2 = desc_k_major_sw128(smem_u32(a2_tile)),
                           bd = desc_k_major_sw128(smem_u32(b_tile));
            const long long t0 = clock64();
            for (uint32_t g = 0; g < groups; g++) {
                tc_copy_scales(tmem + 256, desc_scale_block(smem_u32(sf)));
                tc_copy_scales(tmem + 260, desc_scale_block(smem_u32(sf + 512)));
                tc_copy_scales(tmem + 264, desc_scale_block(smem_u32(sf + 1024)));
#pragma unroll
                for (uint32_t j = 0; j < 4; j++) {
                    const uint32_t id = idesc_with_scale_ids(idesc, j, j);
                    tc_mma_block_scaled(tmem, ad + 2 * j, bd + 2 * j, id, tmem + 256, tmem + 264, (g | j) ? 1u : 0u);
                    tc_mma_block_scaled(tmem + 128, ad2 + 2 * j, bd + 2 * j, id, tmem + 260, tmem + 264, (g | j) ? 1u : 0u);
                }
            }
            tc_commit(&bars->done);
            mbar_wait(&bars->done, 0, &bars->abort, kDefaultWaitCycles);
            cycles[blockIdx.x] = clock64() - t0;
        }
        __syncwarp();
    }
    __syncthreads();
    if (bars->abort && threadIdx.x == 0) raise_status(status, NVMOE_STATUS_WAIT_EXPIRED);
    if (warp == 4u) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

}  // namespace

cudaError_t launch_mma_rate_probe(uint32_t n_tile, uint32_t groups, uint32_t ctas, long long* cycles, uint32_t* status,
                                  cudaStream_t stream) {
    cudaError_t err = cudaFuncSetAttribute(mma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kProbeSmem);
    if (err != cudaSuccess) return err;
    mma_rate_kernel<<<ctas, 160, kProbeSmem, stream>>>(n_tile, groups, cycles, status);
    return cudaGetLastError();
}

}  // namespace nvmoe
