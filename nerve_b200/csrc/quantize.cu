// Activation quantisation bf16 -> FP8 E4M3 with one power-of-two scale per block of columns.
//
//   quantize_batch_fp8_e4m3.comp.template:47-71 (shared pre-quantisation, power-of-two scale)
//   independent_sparse_moe_gate_up_batch1_mxfp4.comp.template:357-383 (quantize_hidden)
//   independent_sparse_moe_down_batch1_mxfp4.comp.template:307-353 (quantize_intermediate)
//
// scale = 2^ceil(log2(max(|x|, 1e-4) / 448)), q = E4M3(x / scale) with round-to-nearest-even.
// The reference block is 128 columns; any multiple of 32 that divides the row works here.  Besides
// the f32 scales of the reference contract the kernel can emit the same scales as E8M0 bytes, one
// per 32 columns, four to a word — the form a block-scaled MMA reads.
#include <cuda_fp8.h>

#include "common.cuh"

namespace nvmoe {
namespace {

__device__ __forceinline__ uint32_t to_e4m3x4(float a, float b, float c, float d) {
    // cvt.rn.satfinite.e4m3x2.f32: round-to-nearest-even, saturating (|x/scale| <= 448 by construction)
    uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
}

// A lane owns 4 columns at a time, so a block of `block` columns keeps block/4 lanes busy: a warp takes
// one block of 128 or more columns, or 32*4/block smaller ones side by side (four blocks of 32).
// row_of(r) gives the bf16 row pointer, so the same body serves plain matrices and MoE frames.
template <class RowFn>
__device__ void quantize_body(RowFn row_of, uint32_t rows, uint32_t cols, uint32_t block, uint8_t* q,
                              float* scales_f32, uint32_t* scales_e8m0) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warps_per_grid = (gridDim.x * blockDim.x) >> 5;
    const uint32_t blocks_per_row = cols / block;
    const uint32_t words128 = (cols + 127u) / 128u;
    const uint64_t total = (uint64_t)rows * blocks_per_row;
    // lanes per block: a power of two that divides 32 (blocks of 32, 64 or 128+ columns), else the whole warp
    const uint32_t quarter = block / 4u;
    const uint32_t lanes = (quarter == 8u || quarter == 16u) ? quarter : 32u;
    const uint32_t side_by_side = 32u / lanes;
    const uint32_t group = lane / lanes, gl = lane % lanes;
    for (uint64_t first = (uint64_t)((blockIdx.x * blockDim.x + threadIdx.x) >> 5) * side_by_side; first < total;
         first += (uint64_t)warps_per_grid * side_by_side) {
        const uint64_t item = first + group;
        const bool active = item < total;
        const uint32_t r = active ? (uint32_t)(item / blocks_per_row) : 0u, b = active ? (uint32_t)(item % blocks_per_row) : 0u;
        // rows of a frame are only 4-byte aligned when the route count is odd: 4-byte loads
        const uint32_t* in = reinterpret_cast<const uint32_t*>(row_of(r) + (size_t)b * block);
        float m = 0.0f;
        if (active) {
            for (uint32_t c4 = gl; c4 < quarter; c4 += lanes) {
                uint2 v = make_uint2(in[2u * c4], in[2u * c4 + 1u]);
                m = fmaxf(m, fmaxf(fmaxf(fabsf(nvmoe_bf16_to_f32(v.x)), fabsf(nvmoe_bf16_to_f32(v.x >> 16))),
                                   fmaxf(fabsf(nvmoe_bf16_to_f32(v.y)), fabsf(nvmoe_bf16_to_f32(v.y >> 16)))));
            }
        }
        for (uint32_t o = lanes >> 1; o > 0u; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (!active) continue;
        const float scale = nvmoe_rounded_fp8_scale(m);
        const float inv = __fdiv_rn(1.0f, scale);  // exact: the scale is a power of two
        uint32_t* out = reinterpret_cast<uint32_t*>(q + (size_t)r * cols + (size_t)b * block);
        for (uint32_t c4 = gl; c4 < quarter; c4 += lanes) {
            uint2 v = make_uint2(in[2u * c4], in[2u * c4 + 1u]);
            out[c4] = to_e4m3x4(nvmoe_bf16_to_f32(v.x) * inv, nvmoe_bf16_to_f32(v.x >> 16) * inv,
                                nvmoe_bf16_to_f32(v.y) * inv, nvmoe_bf16_to_f32(v.y >> 16) * inv);
        }
        if (scales_f32 && gl == 0u) scales_f32[(size_t)r * blocks_per_row + b] = scale;
        if (scales_e8m0) {
            // one byte per 32 columns; this block covers block/32 of them
            uint8_t* bytes = reinterpret_cast<uint8_t*>(scales_e8m0 + (size_t)r * words128);
            const uint32_t e8 = nvmoe_f32_bits(scale) >> 23;
            for (uint32_t j = gl; j < block / 32u; j += lanes) bytes[b * (block / 32u) + j] = (uint8_t)e8;
        }
    }
}

__global__ void __launch_bounds__(256) quantize_kernel(const uint16_t* input, uint32_t rows, uint32_t cols,
                                                      uint32_t block, size_t row_stride, uint8_t* q,
                                                      float* scales_f32, uint32_t* scales_e8m0) {
    grid_dependency_sync();
    quantize_body([&](uint32_t r) { return input + (size_t)r * row_stride; }, rows, cols, block, q, scales_f32,
                  scales_e8m0);
}

__global__ void __launch_bounds__(256) quantize_frames_kernel(const uint32_t* intermediates, uint32_t tokens,
                                                             uint32_t K, uint32_t I, uint32_t block, uint8_t* q,
                                                             float* scales_f32, uint32_t* scales_e8m0) {
    grid_dependency_sync();
    const uint32_t frame_words = K * (I / 2u) + K;
    quantize_body(
        [&](uint32_t r) {
            return reinterpret_cast<const uint16_t*>(intermediates + (size_t)(r / K) * frame_words) + (size_t)(r % K) * I;
        },
        tokens * K, I, block, q, scales_f32, scales_e8m0);
}

__global__ void __launch_bounds__(256) quantize_grouped_kernel(const void* input, bool frames, const uint32_t* grouped,
                                                              const uint32_t* expert_offsets, uint32_t num_experts,
                                                              uint32_t max_routes, uint32_t K, uint32_t cols, uint32_t I,
                                                              uint32_t block, uint8_t* q, uint32_t* scales_e8m0) {
    grid_dependency_sync();
    const uint32_t total = min(expert_offsets[num_experts], max_routes);
    const uint32_t frame_words = K * (I / 2u) + K;
    quantize_body(
        [&](uint32_t pos) {
            const uint32_t ri = grouped[pos];
            return frames ? reinterpret_cast<const uint16_t*>(static_cast<const uint32_t*>(input) + (size_t)(ri / K) * frame_words) +
                                (size_t)(ri % K) * I
                          : static_cast<const uint16_t*>(input) + (size_t)(ri / K) * cols;
        },
        total, cols, block, q, nullptr, scales_e8m0);
}

// The common cases of the tensor path's gate/up operands (32- or 128-column blocks, hidden rows 16-byte
// aligned): LANES = block / 8 lanes per block, eight values a lane, one 16-byte load and one 8-byte store
// each; a warp takes 32 / LANES blocks side by side. Same values and scales as quantize_body.
template <uint32_t LANES>
__global__ void __launch_bounds__(256) quantize_grouped_rows_kernel(const uint16_t* __restrict__ input,
                                                                   const uint32_t* __restrict__ grouped,
                                                                   const uint32_t* __restrict__ expert_offsets,
                                                                   uint32_t num_experts, uint32_t max_routes, uint32_t K,
                                                                   uint32_t cols, uint8_t* __restrict__ q,
                                                                   uint32_t* __restrict__ scales_e8m0) {
    grid_dependency_sync();
    constexpr uint32_t kBlock = LANES * 8u, kSide = 32u / LANES;
    const uint32_t total_rows = min(expert_offsets[num_experts], max_routes);
    const uint32_t blocks_per_row = cols / kBlock, words128 = (cols + 127u) / 128u;
    const uint64_t total = (uint64_t)total_rows * blocks_per_row;
    const uint32_t lane = threadIdx.x & 31u, sub = lane / LANES, part = lane % LANES;
    const uint64_t warps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
    for (uint64_t first = (((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5) * kSide; first < total; first += warps * kSide) {
        const uint64_t item = first + sub;
        const bool active = item < total;
        const uint32_t pos = active ? (uint32_t)(item / blocks_per_row) : 0u, b = active ? (uint32_t)(item % blocks_per_row) : 0u;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (active) {
            const uint32_t token = __ldg(grouped + pos) / K;
            v = __ldg(reinterpret_cast<const uint4*>(input + (size_t)token * cols + (size_t)b * kBlock) + part);
        }
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        float m = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; i++)
            m = fmaxf(m, fmaxf(fabsf(nvmoe_bf16_to_f32(w[i])), fabsf(nvmoe_bf16_to_f32(w[i] >> 16))));
#pragma unroll
        for (uint32_t o = 1u; o < LANES; o <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (!active) continue;
        const float scale = nvmoe_rounded_fp8_scale(m);
        const float inv = __uint_as_float(0x7f000000u - __float_as_uint(scale));  // 1 / scale, exact (a power of two)
        uint2 out;
        out.x = to_e4m3x4(nvmoe_bf16_to_f32(w[0]) * inv, nvmoe_bf16_to_f32(w[0] >> 16) * inv, nvmoe_bf16_to_f32(w[1]) * inv,
                          nvmoe_bf16_to_f32(w[1] >> 16) * inv);
        out.y = to_e4m3x4(nvmoe_bf16_to_f32(w[2]) * inv, nvmoe_bf16_to_f32(w[2] >> 16) * inv, nvmoe_bf16_to_f32(w[3]) * inv,
                          nvmoe_bf16_to_f32(w[3] >> 16) * inv);
        reinterpret_cast<uint2*>(q + (size_t)pos * cols + (size_t)b * kBlock)[part] = out;
        // one scale byte per 32 columns: a block of 128 fills four
        if (part < kBlock / 32u)
            reinterpret_cast<uint8_t*>(scales_e8m0 + (size_t)pos * words128)[b * (kBlock / 32u) + part] =
                (uint8_t)(nvmoe_f32_bits(scale) >> 23);
    }
}

__global__ void __launch_bounds__(256) scales_to_e8m0_kernel(const float* scales, uint32_t rows, uint32_t cols,
                                                            uint32_t block, uint32_t* scales_e8m0, uint32_t* status) {
    const uint32_t blocks_per_row = cols / block;
    const uint32_t words128 = (cols + 127u) / 128u;
    const uint64_t total = (uint64_t)rows * blocks_per_row;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t r = (uint32_t)(i / blocks_per_row), b = (uint32_t)(i % blocks_per_row);
        const uint32_t bits = nvmoe_f32_bits(scales[i]);
        // a block-scaled MMA can only take power-of-two scales with a biased exponent in 1..254
        if ((bits & 0x807fffffu) != 0u || (bits >> 23) == 0u || (bits >> 23) == 255u) raise_status(status, 1u);
        uint8_t* bytes = reinterpret_cast<uint8_t*>(scales_e8m0 + (size_t)r * words128);
        for (uint32_t j = 0; j < block / 32u; j++) bytes[b * (block / 32u) + j] = (uint8_t)(bits >> 23);
    }
}

// blocks for `warps` warp-sized work items (callers pass one item per scale block; a warp may take several)
uint32_t grid_for(uint64_t warps) {
    // an item is a short dependent chain (load, block maximum, convert, store): the latency is hidden by
    // many resident warps with an item or two each rather than by few warps looping
    uint64_t blocks = (warps / 4u + 7u) / 8u;
    return (uint32_t)(blocks < 1u ? 1u : (blocks > 148u * 256u ? 148u * 256u : blocks));
}

}  // namespace

void launch_quantize(const uint16_t* input, uint32_t rows, uint32_t cols, uint32_t block, size_t input_row_stride,
                     uint8_t* q, float* scales_f32, uint32_t* scales_e8m0, cudaStream_t stream) {
    if (rows == 0u) return;
    launch_chained(quantize_kernel, dim3(grid_for((uint64_t)rows * (cols / block))), dim3(256), 0, stream, input, rows, cols,
                   block, input_row_stride, q, scales_f32, scales_e8m0);
}

void launch_quantize_frames(const uint32_t* intermediates, uint32_t tokens, uint32_t K, uint32_t intermediate_size,
                            uint32_t block, uint8_t* q, float* scales_f32, uint32_t* scales_e8m0,
                            cudaStream_t stream) {
    if (tokens == 0u) return;
    launch_chained(quantize_frames_kernel, dim3(grid_for((uint64_t)tokens * K * (intermediate_size / block))), dim3(256), 0,
                   stream, intermediates, tokens, K, intermediate_size, block, q, scales_f32, scales_e8m0);
}

void launch_quantize_grouped(const void* input, bool frames, const uint32_t* grouped_routes,
                             const uint32_t* expert_offsets, uint32_t num_experts, uint32_t max_routes, uint32_t K,
                             uint32_t cols, uint32_t intermediate_size, uint32_t block, uint8_t* q,
                             uint32_t* scales_e8m0, cudaStream_t stream) {
    if (max_routes == 0u) return;
    if (!frames && (block == 32u || block == 128u) && cols % 8u == 0u && (reinterpret_cast<uintptr_t>(input) & 15u) == 0u) {
        const uint32_t side = block == 32u ? 8u : 2u;  // blocks a warp takes at once
        const uint64_t warps = ((uint64_t)max_routes * (cols / block) + side - 1u) / side;
        uint64_t blocks = (warps + 7u) / 8u;
        if (blocks > 148u * 64u) blocks = 148u * 64u;
        const auto kernel = block == 32u ? quantize_grouped_rows_kernel<4u> : quantize_grouped_rows_kernel<16u>;
        launch_chained(kernel, dim3((uint32_t)blocks), dim3(256), 0, stream, static_cast<const uint16_t*>(input), grouped_routes,
                       expert_offsets, num_experts, max_routes, K, cols, q, scales_e8m0);
        return;
    }
    launch_chained(quantize_grouped_kernel, dim3(grid_for((uint64_t)max_routes * (cols / block))), dim3(256), 0, stream, input,
                   frames, grouped_routes, expert_offsets, num_experts, max_routes, K, cols, intermediate_size, block, q,
                   scales_e8m0);
}

void launch_scales_to_e8m0(const float* scales, uint32_t rows, uint32_t cols, uint32_t block,
                           uint32_t* scales_e8m0, uint32_t* status, cudaStream_t stream) {
    if (rows == 0u) return;
    uint64_t total = (uint64_t)rows * (cols / block);
    uint32_t blocks = (uint32_t)((total + 255u) / 256u);
    scales_to_e8m0_kernel<<<blocks > 2368u ? 2368u : blocks, 256, 0, stream>>>(scales, rows, cols, block,
                                                                               scales_e8m0, status);
}

}  // namespace nvmoe
