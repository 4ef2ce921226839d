// Weighted combine of the per-route expert outputs.
//
//   runtime-rs/shaders/moe_reduce_batch1_bf16.comp.template:29-55
//
// The route weight is already inside each per-route row (the down stage applied it), so the
// combine is a sum over the K routes of a token in route order — ascending expert id — with a
// bf16 rounding after every add, then one multiply by ROUTED_SCALE and a final rounding.  That
// order and those roundings are the reference's and are reproduced exactly.
#include "common.cuh"

namespace nvmoe {
namespace {

__global__ void __launch_bounds__(256) reduce_kernel(const uint32_t* __restrict__ expert_outputs,
                                                    uint32_t* __restrict__ output, uint32_t tokens, uint32_t K,
                                                    uint32_t hidden_words, float routed_scale,
                                                    const uint32_t* __restrict__ computed) {
    grid_dependency_sync();
    const uint64_t total = (uint64_t)tokens * hidden_words;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t t = (uint32_t)(i / hidden_words), word = (uint32_t)(i % hidden_words);
        const uint32_t* in = expert_outputs + (size_t)t * K * hidden_words + word;
        float lo = 0.0f, hi = 0.0f;
        for (uint32_t r = 0; r < K; r++) {
            // a route the down stage skipped (computed[route] says "nowhere") counts as a row of zeros
            const uint32_t c = (computed && computed[(size_t)t * K + r] == kUnboundSlot) ? 0u : in[(size_t)r * hidden_words];
            lo = nvmoe_round_bf16(__fadd_rn(lo, nvmoe_bf16_to_f32(c)));
            hi = nvmoe_round_bf16(__fadd_rn(hi, nvmoe_bf16_to_f32(c >> 16)));
        }
        output[i] = pack_bf16x2(__fmul_rn(lo, routed_scale), __fmul_rn(hi, routed_scale));
    }
}

// The same sum over 16-byte pieces (eight columns a thread) for rows that allow it: the order of the adds
// of a column and every rounding are unchanged.
__global__ void __launch_bounds__(256) reduce_vec_kernel(const uint4* __restrict__ expert_outputs, uint4* __restrict__ output,
                                                        uint32_t tokens, uint32_t K, uint32_t hidden_vecs, float routed_scale,
                                                        const uint32_t* __restrict__ computed) {
    grid_dependency_sync();
    const uint64_t total = (uint64_t)tokens * hidden_vecs;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t t = (uint32_t)(i / hidden_vecs), vec = (uint32_t)(i % hidden_vecs);
        const uint4* in = expert_outputs + (size_t)t * K * hidden_vecs + vec;
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; j++) acc[j] = 0.0f;
        // four routes at a time: their marks and rows are fetched together (one memory round trip instead of one
        // per route), the adds keep the route order
        for (uint32_t r0 = 0; r0 < K; r0 += 4u) {
            bool skipped[4];
            uint4 c[4];
#pragma unroll
            for (uint32_t u = 0; u < 4u; u++)
                // a route the down stage skipped (computed[route] says "nowhere") counts as a row of zeros
                skipped[u] = r0 + u >= K || (computed && __ldg(computed + (size_t)t * K + r0 + u) == kUnboundSlot);
#pragma unroll
            for (uint32_t u = 0; u < 4u; u++) c[u] = skipped[u] ? make_uint4(0u, 0u, 0u, 0u) : in[(size_t)(r0 + u) * hidden_vecs];
#pragma unroll
            for (uint32_t u = 0; u < 4u; u++) {
                if (r0 + u >= K) break;
                const uint32_t w[4] = {c[u].x, c[u].y, c[u].z, c[u].w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    acc[2 * j] = nvmoe_round_bf16(__fadd_rn(acc[2 * j], nvmoe_bf16_to_f32(w[j])));
                    acc[2 * j + 1] = nvmoe_round_bf16(__fadd_rn(acc[2 * j + 1], nvmoe_bf16_to_f32(w[j] >> 16)));
                }
            }
        }
        uint4 out;
        out.x = pack_bf16x2(__fmul_rn(acc[0], routed_scale), __fmul_rn(acc[1], routed_scale));
        out.y = pack_bf16x2(__fmul_rn(acc[2], routed_scale), __fmul_rn(acc[3], routed_scale));
        out.z = pack_bf16x2(__fmul_rn(acc[4], routed_scale), __fmul_rn(acc[5], routed_scale));
        out.w = pack_bf16x2(__fmul_rn(acc[6], routed_scale), __fmul_rn(acc[7], routed_scale));
        output[i] = out;
    }
}

// The combine of an expert-parallel step read straight from the rows that came back from the owners:
// route (t, r) lies at row gather[t * K + r] of `rows` (all-ones: the route was left out and counts as a row
// of zeros). The same adds in the same order with the same roundings as reduce_vec_kernel; only where a row is
// read from differs, which saves the pass that would put the rows back into [T][K][H] order first.
__global__ void __launch_bounds__(256) reduce_gather_kernel(const uint4* __restrict__ rows, const uint32_t* __restrict__ gather,
                                                           uint4* __restrict__ output, uint32_t tokens, uint32_t K,
                                                           uint32_t hidden_vecs, float routed_scale) {
    grid_dependency_sync();
    const uint64_t total = (uint64_t)tokens * hidden_vecs;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t t = (uint32_t)(i / hidden_vecs), vec = (uint32_t)(i % hidden_vecs);
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; j++) acc[j] = 0.0f;
        // four routes at a time, as in reduce_vec_kernel: the row numbers together, then the rows together
        for (uint32_t r0 = 0; r0 < K; r0 += 4u) {
            uint32_t row[4];
            uint4 c[4];
#pragma unroll
            for (uint32_t u = 0; u < 4u; u++) row[u] = r0 + u < K ? __ldg(gather + (size_t)t * K + r0 + u) : kUnboundSlot;
#pragma unroll
            for (uint32_t u = 0; u < 4u; u++)
                c[u] = row[u] == kUnboundSlot ? make_uint4(0u, 0u, 0u, 0u) : rows[(size_t)row[u] * hidden_vecs + vec];
#pragma unroll
            for (uint32_t u = 0; u < 4u; u++) {
                if (r0 + u >= K) break;
                const uint32_t w[4] = {c[u].x, c[u].y, c[u].z, c[u].w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    acc[2 * j] = nvmoe_round_bf16(__fadd_rn(acc[2 * j], nvmoe_bf16_to_f32(w[j])));
                    acc[2 * j + 1] = nvmoe_round_bf16(__fadd_rn(acc[2 * j + 1], nvmoe_bf16_to_f32(w[j] >> 16)));
                }
            }
        }
        uint4 out;
        out.x = pack_bf16x2(__fmul_rn(acc[0], routed_scale), __fmul_rn(acc[1], routed_scale));
        out.y = pack_bf16x2(__fmul_rn(acc[2], routed_scale), __fmul_rn(acc[3], routed_scale));
        out.z = pack_bf16x2(__fmul_rn(acc[4], routed_scale), __fmul_rn(acc[5], routed_scale));
        out.w = pack_bf16x2(__fmul_rn(acc[6], routed_scale), __fmul_rn(acc[7], routed_scale));
        output[i] = out;
    }
}

// The finaliser of a tensor-parallel expert stage
// (runtime-rs/shaders/distributed_sum_f32_scale_packed_bf16_to_bf16.comp:44-66): the participants' f32
// partial planes are added in participant order, the sum is scaled by a bf16 taken from a packed word
// (the route weight in the upper half of a route word) and rounded to bf16 once.
__global__ void __launch_bounds__(256) sum_f32_scale_packed_bf16_kernel(const float* __restrict__ partials,
                                                                       const uint32_t* __restrict__ scales,
                                                                       uint32_t* __restrict__ output, uint32_t element_count,
                                                                       uint32_t participant_count, uint32_t lane_count,
                                                                       uint32_t elements_per_scale, uint32_t scale_bit_offset) {
    grid_dependency_sync();
    const uint32_t words = element_count / 2u, scales_per_lane = element_count / elements_per_scale;
    const uint64_t total = (uint64_t)lane_count * words;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t lane = (uint32_t)(i / words), element = (uint32_t)(i % words) * 2u;
        float lo = 0.0f, hi = 0.0f;
        for (uint32_t part = 0; part < participant_count; part++) {
            const float2 v = *reinterpret_cast<const float2*>(partials + ((size_t)part * lane_count + lane) * element_count + element);
            lo = __fadd_rn(lo, v.x);
            hi = __fadd_rn(hi, v.y);
        }
        const float slo = nvmoe_bf16_to_f32(scales[(size_t)lane * scales_per_lane + element / elements_per_scale] >> scale_bit_offset);
        const float shi = nvmoe_bf16_to_f32(scales[(size_t)lane * scales_per_lane + (element + 1u) / elements_per_scale] >> scale_bit_offset);
        output[i] = pack_bf16x2(__fmul_rn(lo, slo), __fmul_rn(hi, shi));
    }
}

}  // namespace

void launch_sum_f32_scale_packed_bf16(const float* partials, const uint32_t* scales, uint32_t* output, uint32_t element_count,
                                      uint32_t participant_count, uint32_t lane_count, uint32_t elements_per_scale,
                                      uint32_t scale_bit_offset, cudaStream_t stream) {
    const uint64_t total = (uint64_t)lane_count * (element_count / 2u);
    uint64_t blocks = (total + 255u) / 256u;
    if (blocks > 148u * 16u) blocks = 148u * 16u;
    if (blocks == 0u) return;
    launch_chained(sum_f32_scale_packed_bf16_kernel, dim3((uint32_t)blocks), dim3(256), 0, stream, partials, scales, output,
                   element_count, participant_count, lane_count, elements_per_scale, scale_bit_offset);
}

bool launch_reduce_gather(const uint16_t* rows, const uint32_t* gather, uint16_t* output, uint32_t tokens, uint32_t K,
                          uint32_t hidden, float routed_scale, cudaStream_t stream) {
    if (hidden % 8u != 0u || ((reinterpret_cast<uintptr_t>(rows) | reinterpret_cast<uintptr_t>(output)) & 15u) != 0u) return false;
    const uint64_t vecs = (uint64_t)tokens * (hidden / 8u);
    uint64_t blocks = (vecs + 255u) / 256u;
    if (blocks > 148u * 16u) blocks = 148u * 16u;
    if (blocks == 0u) return true;
    launch_chained(reduce_gather_kernel, dim3((uint32_t)blocks), dim3(256), 0, stream, reinterpret_cast<const uint4*>(rows), gather,
                   reinterpret_cast<uint4*>(output), tokens, K, hidden / 8u, routed_scale);
    return true;
}

void launch_reduce(const uint16_t* expert_outputs, uint16_t* output, uint32_t tokens, uint32_t K, uint32_t hidden,
                   float routed_scale, const uint32_t* computed, cudaStream_t stream) {
    if (tokens == 0u) return;
    if (hidden % 8u == 0u && ((reinterpret_cast<uintptr_t>(expert_outputs) | reinterpret_cast<uintptr_t>(output)) & 15u) == 0u) {
        const uint64_t vecs = (uint64_t)tokens * (hidden / 8u);
        uint64_t vec_blocks = (vecs + 255u) / 256u;
        if (vec_blocks > 148u * 16u) vec_blocks = 148u * 16u;
        launch_chained(reduce_vec_kernel, dim3((uint32_t)vec_blocks), dim3(256), 0, stream,
                       reinterpret_cast<const uint4*>(expert_outputs), reinterpret_cast<uint4*>(output), tokens, K, hidden / 8u,
                       routed_scale, computed);
        return;
    }
    const uint64_t total = (uint64_t)tokens * (hidden / 2u);
    uint64_t blocks = (total + 255u) / 256u;
    if (blocks > 148u * 8u) blocks = 148u * 8u;
    launch_chained(reduce_kernel, dim3((uint32_t)blocks), dim3(256), 0, stream,
                   reinterpret_cast<const uint32_t*>(expert_outputs), reinterpret_cast<uint32_t*>(output), tokens, K,
                   hidden / 2u, routed_scale, computed);
}

}  // namespace nvmoe
