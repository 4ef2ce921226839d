// The nodes either side of the MoE chain in the compiler's feed-forward block, and the token-id
// table routing in front of it.
//
//   rms_norm_kernel               runtime-rs/shaders/rms_norm_batch_bf16.comp.template:55-108 (op rms_norm: ffn_norm)
//   silu_multiply_kernel          runtime-rs/shaders/bounded_silu_multiply_batch_bf16.comp.template:26-53 and
//                                 runtime-rs/shaders/silu_multiply_batch_bf16.comp.template:24-52
//   add_kernel                    runtime-rs/shaders/add_batch_bf16.comp.template:36-50 (op residual_add)
//   preselect_table_kernel        runtime-rs/shaders/resource_preselect_table_batch1.comp.template:35-97
//   route_preselected_kernel      runtime-rs/shaders/moe_router_preselected_batch1_bf16.comp.template:56-91
//
// All of them are bound by memory or by latency, not by arithmetic: one pass over the rows with
// 128-byte warp accesses, the transcendental functions out of nvmoe_math.h so that results are the
// CPU checker's bit for bit.
#include "common.cuh"

namespace nvmoe {
namespace {

// One warp per row. The shader's 64 lanes stride over the row's elements; here thread u plays lanes 2u
// and 2u + 1 (one packed word per step), which keeps every lane's sum in ascending element order and makes
// a warp's access one 128-byte line per step. The lane sums are folded with the pinned butterfly
// (32, 16, 8, 4, 2 across threads, 1 inside the thread).
__global__ void __launch_bounds__(256) rms_norm_kernel(const uint32_t* __restrict__ input, const uint32_t* __restrict__ weight,
                                                       uint32_t* __restrict__ output, uint32_t rows, uint32_t hidden,
                                                       float eps, float weight_offset) {
    grid_dependency_sync();
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const uint32_t words = hidden / 2u;
    const uint32_t* x = input + (size_t)row * words;
    float lo = 0.0f, hi = 0.0f;
    constexpr int kDepth = 8;  // loads of eight steps are issued together
    for (uint32_t w0 = lane; w0 < words; w0 += 32u * kDepth) {
        uint32_t v[kDepth];
#pragma unroll
        for (int u = 0; u < kDepth; u++) v[u] = (w0 + 32u * u < words) ? __ldg(x + w0 + 32u * u) : 0u;
#pragma unroll
        for (int u = 0; u < kDepth; u++) {
            if (w0 + 32u * u >= words) break;
            const float a = nvmoe_bf16_to_f32(v[u]), b = nvmoe_bf16_to_f32(v[u] >> 16);
            lo = __fmaf_rn(a, a, lo);
            hi = __fmaf_rn(b, b, hi);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        lo = __fadd_rn(lo, __shfl_xor_sync(0xffffffffu, lo, o));
        hi = __fadd_rn(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    const float total = __fadd_rn(lo, hi);
    const float inv_rms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)hidden), eps)));
    uint32_t* y = output + (size_t)row * words;
    for (uint32_t w = lane; w < words; w += 32u) {
        const uint32_t xv = x[w], wv = __ldg(weight + w);
        const float a = __fmul_rn(__fmul_rn(nvmoe_bf16_to_f32(xv), inv_rms), __fadd_rn(nvmoe_bf16_to_f32(wv), weight_offset));
        const float b = __fmul_rn(__fmul_rn(nvmoe_bf16_to_f32(xv >> 16), inv_rms), __fadd_rn(nvmoe_bf16_to_f32(wv >> 16), weight_offset));
        y[w] = pack_bf16x2(a, b);
    }
}

__device__ __forceinline__ float silu_times(float g, float u, float limit) {
    if (limit > 0.0f) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, nvmoe_expf(-g))), u);
    }
    // the unbounded node rounds the activated gate to bf16 before the product
    return __fmul_rn(nvmoe_round_bf16(__fdiv_rn(g, __fadd_rn(1.0f, nvmoe_expf(-g)))), u);
}

__device__ __forceinline__ uint32_t silu_word(uint32_t g, uint32_t u, float limit) {
    return pack_bf16x2(silu_times(nvmoe_bf16_to_f32(g), nvmoe_bf16_to_f32(u), limit),
                       silu_times(nvmoe_bf16_to_f32(g >> 16), nvmoe_bf16_to_f32(u >> 16), limit));
}

__device__ __forceinline__ uint32_t add_word(uint32_t a, uint32_t b) {
    return pack_bf16x2(__fadd_rn(nvmoe_bf16_to_f32(a), nvmoe_bf16_to_f32(b)),
                       __fadd_rn(nvmoe_bf16_to_f32(a >> 16), nvmoe_bf16_to_f32(b >> 16)));
}

// out[i] = f(a[i], b[i]) over packed bf16 words, 16 bytes per thread where the buffers allow it
template <bool SILU>
__global__ void __launch_bounds__(256) pairwise_kernel(const uint32_t* __restrict__ a, const uint32_t* __restrict__ b,
                                                       uint32_t* __restrict__ out, size_t words, float limit, bool vector) {
    grid_dependency_sync();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (vector) {
        const size_t quads = words / 4u;
        for (; i < quads; i += stride) {
            const uint4 x = __ldg(reinterpret_cast<const uint4*>(a) + i), y = __ldg(reinterpret_cast<const uint4*>(b) + i);
            uint4 r;
            r.x = SILU ? silu_word(x.x, y.x, limit) : add_word(x.x, y.x);
            r.y = SILU ? silu_word(x.y, y.y, limit) : add_word(x.y, y.y);
            r.z = SILU ? silu_word(x.z, y.z, limit) : add_word(x.z, y.z);
            r.w = SILU ? silu_word(x.w, y.w, limit) : add_word(x.w, y.w);
            reinterpret_cast<uint4*>(out)[i] = r;
        }
        i = quads * 4u + ((size_t)blockIdx.x * blockDim.x + threadIdx.x);
    }
    for (; i < words; i += stride) out[i] = SILU ? silu_word(a[i], b[i], limit) : add_word(a[i], b[i]);
}

// One warp per token: the first k lanes look the token's routed resources up, lane 0 sorts and counts.
__global__ void __launch_bounds__(128) preselect_table_kernel(const uint32_t* __restrict__ token_ids,
                                                              const uint32_t* __restrict__ table, uint32_t word_stride,
                                                              uint32_t vocab, uint32_t routed, uint32_t k, uint32_t always,
                                                              uint32_t tokens, uint32_t* __restrict__ selections,
                                                              uint32_t* telemetry, uint32_t* status) {
    __shared__ uint32_t ids[4][kMaxTopK];
    grid_dependency_sync();
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t t = blockIdx.x * 4u + warp;
    if (t >= tokens) return;
    const uint32_t total_k = k + always, total_resources = routed + always;
    const uint32_t token_id = token_ids[t];
    bool invalid = token_id >= vocab;
    if (!invalid) {
        for (uint32_t r = lane; r < k; r += 32u) {
            const size_t element = (size_t)token_id * k + r;
            const uint32_t index = table[element * word_stride];
            const uint32_t high = word_stride == 2u ? table[element * word_stride + 1u] : 0u;
            if (index >= routed || high != 0u) invalid = true;
            for (uint32_t previous = 0; previous < r; previous++)
                if (index == table[((size_t)token_id * k + previous) * word_stride]) invalid = true;
            ids[warp][r] = min(index, routed - 1u);
        }
        for (uint32_t a = lane; a < always; a += 32u) ids[warp][k + a] = routed + a;
    }
    invalid = __any_sync(0xffffffffu, invalid);
    __syncwarp();
    if (lane != 0u) return;
    uint32_t* out = selections + (size_t)t * total_k;
    if (invalid) {
        for (uint32_t r = 0; r < total_k; r++) out[r] = kUnboundSlot;
        raise_status(status, NVMOE_STATUS_ROUTE_OUT_OF_RANGE);
        return;
    }
    uint32_t* mine = ids[warp];
    for (uint32_t r = 1; r < total_k; r++) {
        const uint32_t index = mine[r];
        uint32_t ins = r;
        while (ins > 0u && mine[ins - 1u] > index) {
            mine[ins] = mine[ins - 1u];
            ins--;
        }
        mine[ins] = index;
    }
    for (uint32_t r = 0; r < total_k; r++) {
        out[r] = mine[r];
        if (telemetry) atomicAdd(telemetry + mine[r], 1u);
    }
    if (telemetry) {
        for (uint32_t l = 0; l < total_k; l++)
            for (uint32_t rr = l + 1u; rr < total_k; rr++) {
                const uint32_t left = mine[l], right = mine[rr];
                const uint32_t preceding = left * (2u * total_resources - left - 1u) / 2u;
                atomicAdd(telemetry + total_resources + preceding + right - left - 1u, 1u);
            }
    }
}

// One warp per token: lanes evaluate the activation of the selected logits side by side, lane 0 sums
// them in their stored order and packs the route words.
__global__ void __launch_bounds__(128) route_preselected_kernel(const uint32_t* __restrict__ logits,
                                                                const uint32_t* __restrict__ selections, uint32_t tokens,
                                                                uint32_t* __restrict__ routes, uint32_t* status, nvmoe_geometry g) {
    __shared__ float values[4][kMaxTopK];
    grid_dependency_sync();
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t t = blockIdx.x * 4u + warp;
    if (t >= tokens) return;
    const uint32_t E = g.routed_experts, k = g.routed_k, total_k = k + g.always_count;
    const uint32_t* sel = selections + (size_t)t * total_k;
    const uint32_t* row = logits + (size_t)t * ((E + 1u) / 2u);
    bool bad = false;
    for (uint32_t r = lane; r < k; r += 32u) {
        const uint32_t index = sel[r] & 0xffffu;
        if (index >= E) {
            bad = true;
            continue;
        }
        const uint32_t packed = row[index >> 1];
        const float v = nvmoe_bf16_to_f32((index & 1u) ? packed >> 16 : packed);
        values[warp][r] = g.activation == NVMOE_ACT_SIGMOID ? nvmoe_sigmoidf(v) : __fsqrt_rn(nvmoe_softplusf(v));
    }
    bad = __any_sync(0xffffffffu, bad);
    __syncwarp();
    if (lane != 0u) return;
    uint32_t* out = routes + (size_t)t * total_k;
    if (bad) {  // an invalid token of the preselection: weight 0 and an id no expert kernel accepts
        for (uint32_t r = 0; r < total_k; r++) out[r] = 0x0000ffffu;
        raise_status(status, NVMOE_STATUS_ROUTE_OUT_OF_RANGE);
        return;
    }
    float den = 0.0f;
    if (g.normalize_selected)
        for (uint32_t r = 0; r < k; r++) den = __fadd_rn(den, values[warp][r]);
    for (uint32_t r = 0; r < total_k; r++) {
        float w = g.always_weight;
        if (r < k)
            w = g.normalize_selected ? __fmul_rn(__fdiv_rn(values[warp][r], den), g.routed_scale)
                                     : __fmul_rn(values[warp][r], g.routed_scale);
        out[r] = (nvmoe_f32_to_bf16(w) << 16) | (sel[r] & 0xffffu);
    }
}

// Identity schedule of a dense linear run as one always-selected resource: every row is a route of
// expert 0 in row order, the (expert, token tile) list covers the rows.
__global__ void dense_schedule_kernel(uint32_t rows, uint32_t n_tile, uint32_t* grouped, uint32_t* offsets, uint32_t* position,
                                      uint32_t* tiles, uint32_t* tile_count) {
    grid_dependency_sync();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < rows) {
        grouped[i] = i;
        position[i] = i;
    }
    const uint32_t tile_total = (rows + n_tile - 1u) / n_tile;
    if (tiles && i < tile_total) tiles[i] = i;  // (expert 0 << 16) | token tile
    if (i == 0u) {
        offsets[0] = 0u;
        offsets[1] = rows;
        if (tile_count) *tile_count = tile_total;
    }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0u; }

}  // namespace

void launch_rms_norm(const uint16_t* input, const uint16_t* weight, uint16_t* output, uint32_t rows, uint32_t hidden, float eps,
                     float weight_offset, cudaStream_t stream) {
    launch_chained(rms_norm_kernel, dim3((rows + 7u) / 8u), dim3(256), 0, stream, reinterpret_cast<const uint32_t*>(input),
                   reinterpret_cast<const uint32_t*>(weight), reinterpret_cast<uint32_t*>(output), rows, hidden, eps, weight_offset);
}

static uint32_t pairwise_blocks(size_t words) {
    const size_t want = (words / 4u + 255u) / 256u;
    return (uint32_t)(want < 1u ? 1u : want > 148u * 16u ? 148u * 16u : want);
}

void launch_silu_multiply(const uint16_t* gate, const uint16_t* up, uint16_t* out, size_t elements, float limit, cudaStream_t stream) {
    const size_t words = elements / 2u;
    const bool vector = aligned16(gate) && aligned16(up) && aligned16(out);
    launch_chained(pairwise_kernel<true>, dim3(pairwise_blocks(words)), dim3(256), 0, stream, reinterpret_cast<const uint32_t*>(gate),
                   reinterpret_cast<const uint32_t*>(up), reinterpret_cast<uint32_t*>(out), words, limit, vector);
}

void launch_add_bf16(const uint16_t* a, const uint16_t* b, uint16_t* out, size_t elements, cudaStream_t stream) {
    const size_t words = elements / 2u;
    const bool vector = aligned16(a) && aligned16(b) && aligned16(out);
    launch_chained(pairwise_kernel<false>, dim3(pairwise_blocks(words)), dim3(256), 0, stream, reinterpret_cast<const uint32_t*>(a),
                   reinterpret_cast<const uint32_t*>(b), reinterpret_cast<uint32_t*>(out), words, 0.0f, vector);
}

void launch_preselect_table(const uint32_t* token_ids, const uint32_t* table, uint32_t word_stride, uint32_t vocab, uint32_t routed,
                            uint32_t k, uint32_t always, uint32_t tokens, uint32_t* selections, uint32_t* telemetry, uint32_t* status,
                            cudaStream_t stream) {
    launch_chained(preselect_table_kernel, dim3((tokens + 3u) / 4u), dim3(128), 0, stream, token_ids, table, word_stride, vocab, routed,
                   k, always, tokens, selections, telemetry, status);
}

void launch_route_preselected(const uint32_t* logits, const uint32_t* selections, uint32_t tokens, uint32_t* routes, uint32_t* status,
                              const nvmoe_geometry& g, cudaStream_t stream) {
    launch_chained(route_preselected_kernel, dim3((tokens + 3u) / 4u), dim3(128), 0, stream, logits, selections, tokens, routes, status, g);
}

void launch_dense_schedule(uint32_t rows, uint32_t n_tile, uint32_t* grouped, uint32_t* offsets, uint32_t* position, uint32_t* tiles,
                           uint32_t* tile_count, cudaStream_t stream) {
    launch_chained(dense_schedule_kernel, dim3((rows + 255u) / 256u), dim3(256), 0, stream, rows, n_tile, grouped, offsets, position,
                   tiles, tile_count);
}

}  // namespace nvmoe
