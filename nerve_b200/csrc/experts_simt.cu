// Expert projections on the CUDA cores: the dequantising GEMV form of the two expert shaders.
//
//   gate/up  runtime-rs/shaders/independent_sparse_moe_gate_up_batch1_mxfp4.comp.template:643-802
//   down     runtime-rs/shaders/independent_sparse_moe_down_batch1_mxfp4.comp.template:507-610
//
// Same arithmetic as the shaders: E4M3 activations with one scale per activation block, E2M1
// weights with one E8M0 scale per 32 columns, exact products, f32 accumulation, bf16 rounding of
// gate and up before the clamp and of the activated value after it; the down result is scaled by
// the route weight before its single bf16 rounding.  Unlike the shaders, which re-read a weight
// row for every (token, route), work is grouped by expert: a block owns 64 weight rows of one
// expert and streams them once per group of four routed tokens, whose dequantised activations
// sit in shared memory.  This is the general path; the tensor-core path replaces it whenever the
// shape allows.
#include "common.cuh"

namespace nvmoe {
namespace {

constexpr uint32_t kRowsPerBlock = 64u;
constexpr uint32_t kTokensPerPass = 4u;
constexpr uint32_t kThreads = 256u;

struct alignas(8) Pair {
    float lo, hi;
};

__device__ __forceinline__ float e4m3_to_f32_fast(uint32_t b) { return nvmoe_e4m3_to_f32(b); }

// Dot products of one weight row with up to kTokensPerPass activation rows held in shared memory.
// A lane takes 16-byte chunks (32 codes = one scale block); the lane sums are folded by the warp.
template <uint32_t NT>
__device__ __forceinline__ void row_dots(const uint8_t* __restrict__ wrow, const uint8_t* __restrict__ srow,
                                         uint32_t k_dim, const float* act, const Pair* lut, uint32_t lane,
                                         float (&acc)[NT]) {
#pragma unroll
    for (uint32_t t = 0; t < NT; t++) acc[t] = 0.0f;
    const uint4* w16 = reinterpret_cast<const uint4*>(wrow);
    for (uint32_t chunk = lane; chunk < k_dim / 32u; chunk += 32u) {
        const uint4 v = __ldg(w16 + chunk);
        const float ws = nvmoe_e8m0_to_f32(__ldg(srow + chunk));
        const uint32_t words[4] = {v.x, v.y, v.z, v.w};
        float part[NT];
#pragma unroll
        for (uint32_t t = 0; t < NT; t++) part[t] = 0.0f;
#pragma unroll
        for (uint32_t j = 0; j < 4u; j++) {
#pragma unroll
            for (uint32_t b = 0; b < 4u; b++) {
                const Pair p = lut[(words[j] >> (8u * b)) & 0xffu];
                const uint32_t col = chunk * 32u + j * 8u + b * 2u;
#pragma unroll
                for (uint32_t t = 0; t < NT; t++) {
                    const float2 a = *reinterpret_cast<const float2*>(act + (size_t)t * k_dim + col);
                    part[t] = fmaf(p.lo, a.x, part[t]);
                    part[t] = fmaf(p.hi, a.y, part[t]);
                }
            }
        }
#pragma unroll
        for (uint32_t t = 0; t < NT; t++) acc[t] = fmaf(part[t], ws, acc[t]);
    }
#pragma unroll
    for (uint32_t t = 0; t < NT; t++) acc[t] = warp_butterfly_sum(acc[t]);
}

// The same for a matrix held as one E4M3 byte per element (pre-expanded or native FP8): a lane takes the 32
// bytes of one 32-column group; the group's scale is its E8M0 byte of the packaged scale row, or, for native
// FP8, the byte of the 128 x 128 block the group lies in
// (independent_sparse_moe_gate_up_batch1_mxfp4.comp.template:250-262,299-355).
template <uint32_t NT>
__device__ __forceinline__ void row_dots_fp8(const uint8_t* __restrict__ wrow, const uint8_t* __restrict__ scales, bool native,
                                             uint32_t k_dim, const float* act, uint32_t lane, float (&acc)[NT]) {
#pragma unroll
    for (uint32_t t = 0; t < NT; t++) acc[t] = 0.0f;
    const uint4* w16 = reinterpret_cast<const uint4*>(wrow);
    for (uint32_t chunk = lane; chunk < k_dim / 32u; chunk += 32u) {
        const uint4 lo = __ldg(w16 + 2u * chunk), hi = __ldg(w16 + 2u * chunk + 1u);
        // native FP8 scales are plain exponent bytes (byte << 23), without the 2^-127 reading of a zero byte
        const float ws = native ? __uint_as_float((uint32_t)__ldg(scales + chunk / 4u) << 23) : nvmoe_e8m0_to_f32(__ldg(scales + chunk));
        const uint32_t words[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        float part[NT];
#pragma unroll
        for (uint32_t t = 0; t < NT; t++) part[t] = 0.0f;
#pragma unroll
        for (uint32_t j = 0; j < 8u; j++) {
#pragma unroll
            for (uint32_t b = 0; b < 4u; b++) {
                const float w = nvmoe_e4m3_to_f32((words[j] >> (8u * b)) & 0xffu);
                const uint32_t col = chunk * 32u + j * 4u + b;
#pragma unroll
                for (uint32_t t = 0; t < NT; t++) part[t] = fmaf(w, act[(size_t)t * k_dim + col], part[t]);
            }
        }
#pragma unroll
        for (uint32_t t = 0; t < NT; t++) acc[t] = fmaf(part[t], ws, acc[t]);
    }
#pragma unroll
    for (uint32_t t = 0; t < NT; t++) acc[t] = warp_butterfly_sum(acc[t]);
}

__device__ __forceinline__ void fill_lut(Pair* lut) {
    for (uint32_t b = threadIdx.x; b < 256u; b += blockDim.x) {
        lut[b].lo = nvmoe_e2m1_to_f32(b & 0xfu);
        lut[b].hi = nvmoe_e2m1_to_f32(b >> 4);
    }
}

// Loads the dequantised activations (code value times its block scale) of `count` rows.
__device__ __forceinline__ void stage_activations(const ExpertLaunch& p, const uint32_t* rows, uint32_t count,
                                                  uint32_t k_dim, float* act) {
    const uint32_t block = p.g.act_block;
    for (uint32_t t = 0; t < kTokensPerPass; t++) {
        for (uint32_t c = threadIdx.x; c < k_dim; c += blockDim.x) {
            float v = 0.0f;
            if (t < count) {
                const size_t row = rows[t];
                v = e4m3_to_f32_fast(p.act_q[row * k_dim + c]) * p.act_scales[row * (k_dim / block) + c / block];
            }
            act[(size_t)t * k_dim + c] = v;
        }
    }
}

template <bool GATE_UP>
__global__ void __launch_bounds__(kThreads) experts_simt_kernel(ExpertLaunch p, uint32_t row_tiles) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const uint32_t H = p.g.hidden_size, I = p.g.intermediate_size;
    const uint32_t K = p.g.routed_k + p.g.always_count;
    const uint32_t k_dim = GATE_UP ? H : I;
    const uint32_t out_rows = GATE_UP ? I : H;
    Pair* lut = reinterpret_cast<Pair*>(smem_raw);
    float* act = reinterpret_cast<float*>(smem_raw + 256u * sizeof(Pair));
    __shared__ uint32_t pass_rows[kTokensPerPass];   // activation row of each token in the pass
    __shared__ uint32_t pass_routes[kTokensPerPass]; // route index t*K + r

    const uint32_t expert = blockIdx.x / row_tiles;
    const uint32_t tile = blockIdx.x % row_tiles;
    if (expert >= p.work.num_experts) return;
    const uint32_t begin = p.work.expert_offsets[expert], end = p.work.expert_offsets[expert + 1u];
    if (begin == end) return;
    const ExpertPtrs ptrs = p.work.experts[expert];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t frame_words = K * (I / 2u) + K;
    fill_lut(lut);

    for (uint32_t first = begin; first < end; first += kTokensPerPass) {
        const uint32_t count = min(kTokensPerPass, end - first);
        __syncthreads();
        if (threadIdx.x < kTokensPerPass) {
            uint32_t ri = threadIdx.x < count ? p.work.grouped_routes[first + threadIdx.x] : 0u;
            pass_routes[threadIdx.x] = ri;
            pass_rows[threadIdx.x] = GATE_UP ? ri / K : ri;  // gate/up reads the token's hidden row
        }
        __syncthreads();
        stage_activations(p, pass_rows, count, k_dim, act);
        __syncthreads();
        for (uint32_t local = warp; local < kRowsPerBlock; local += kThreads / 32u) {
            const uint32_t row = tile * kRowsPerBlock + local;
            if (row >= out_rows) break;
            float a0[kTokensPerPass], a1[kTokensPerPass];
            if (ptrs.format == kFormatCompact) {
                row_dots<kTokensPerPass>(ptrs.w[0] + (size_t)row * (k_dim / 2u), ptrs.s[0] + (size_t)row * (k_dim / 32u),
                                         k_dim, act, lut, lane, a0);
                if (GATE_UP)
                    row_dots<kTokensPerPass>(ptrs.w[1] + (size_t)row * (k_dim / 2u),
                                             ptrs.s[1] + (size_t)row * (k_dim / 32u), k_dim, act, lut, lane, a1);
            } else {
                const bool native = ptrs.format == kFormatNativeFp8;
                // scale bytes of this row: its own 32-column groups, or the blocks of its 128-row band
                const size_t scale_row = native ? (size_t)(row / 128u) * ((k_dim + 127u) / 128u) : (size_t)row * (k_dim / 32u);
                row_dots_fp8<kTokensPerPass>(ptrs.w[0] + (size_t)row * k_dim, ptrs.s[0] + scale_row, native, k_dim, act, lane, a0);
                if (GATE_UP)
                    row_dots_fp8<kTokensPerPass>(ptrs.w[1] + (size_t)row * k_dim, ptrs.s[1] + scale_row, native, k_dim, act, lane, a1);
            }
            if (lane < count) {
                // lane t finishes token t of the pass (all lanes hold every sum after the butterfly)
                float g = 0.0f, u = 0.0f;
#pragma unroll
                for (uint32_t t = 0; t < kTokensPerPass; t++) {
                    if (t == lane) {
                        g = a0[t];
                        if (GATE_UP) u = a1[t];
                    }
                }
                const uint32_t ri = pass_routes[lane];
                if (GATE_UP) {
                    const float a = nvmoe_swiglu(g, u, p.g.swiglu_limit, p.g.swiglu_alpha, p.g.swiglu_up_offset);
                    uint16_t* out = reinterpret_cast<uint16_t*>(p.intermediates + (size_t)(ri / K) * frame_words) +
                                    (size_t)(ri % K) * I;
                    out[row] = (uint16_t)nvmoe_f32_to_bf16(a);
                } else {
                    if (p.partial_outputs) {  // tensor-parallel form: the raw sum over this participant's columns
                        p.partial_outputs[(size_t)ri * H + row] = g;
                    } else {
                        const float weight = nvmoe_bf16_to_f32(p.routes[ri] >> 16);
                        p.outputs[(size_t)ri * H + row] = (uint16_t)nvmoe_f32_to_bf16(__fmul_rn(g, weight));
                    }
                }
            }
        }
    }
}

template <bool GATE_UP>
void launch(const ExpertLaunch& p, cudaStream_t stream) {
    const uint32_t k_dim = GATE_UP ? p.g.hidden_size : p.g.intermediate_size;
    const uint32_t out_rows = GATE_UP ? p.g.intermediate_size : p.g.hidden_size;
    const uint32_t row_tiles = (out_rows + kRowsPerBlock - 1u) / kRowsPerBlock;
    const size_t smem = 256u * sizeof(Pair) + (size_t)kTokensPerPass * k_dim * sizeof(float);
    experts_simt_kernel<GATE_UP><<<p.work.num_experts * row_tiles, kThreads, smem, stream>>>(p, row_tiles);
}

}  // namespace

void configure_simt_kernels() {
    // per device: called by plan creation with that device current
    cudaFuncSetAttribute(experts_simt_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    cudaFuncSetAttribute(experts_simt_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
}
void launch_gate_up_simt(const ExpertLaunch& p, cudaStream_t stream) { launch<true>(p, stream); }
void launch_down_simt(const ExpertLaunch& p, cudaStream_t stream) { launch<false>(p, stream); }

}  // namespace nvmoe
