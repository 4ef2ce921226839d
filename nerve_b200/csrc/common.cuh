// Shared declarations of the CUDA MoE backend: launch parameter blocks, the resolved expert
// pointer table, fail-closed status bits and small device helpers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/nerve_cuda_moe.h"
#include "../../include/nvmoe_math.h"

namespace nvmoe {

constexpr uint32_t kUnboundSlot = 0xffffffffu;
constexpr uint32_t kRecordWords = 8u;
constexpr uint32_t kMaxTopK = 64u;       // routed_k + always_count
constexpr uint32_t kMaxExperts = 4096u;  // ids travel in the low 16 bits of a route word
// Programmatic dependent launch: a kernel launched with launch_chained may start (and run whatever
// precedes its grid_dependency_sync) while the kernel before it in the stream is still running;
// grid_dependency_sync returns once that kernel has completed and its writes are visible, and lets
// the next kernel in the stream start in the same way. Every thread of a chained kernel calls it
// before touching global memory and before any return, so completion still implies that all earlier
// kernels have completed. Launched the ordinary way, the same kernels run unchanged.
#ifdef __CUDACC__
__device__ __forceinline__ void grid_dependency_sync() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <class... Params, class... Args>
inline cudaError_t launch_chained(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                  Args&&... args) {
    cudaLaunchConfig_t config{};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}
#endif

constexpr uint32_t kSortChunk = 256u;    // routes per block in the multi-block counting sort

// Weight pointers of one expert after the address/slot tables were validated
// (address_record_is_resident + dynamic_expert_is_valid of
// runtime-rs/shaders/independent_sparse_moe_gate_up_batch1_mxfp4.comp.template:120-228).
// A null w pointer means "not resident": every route to that expert is skipped.
enum : uint32_t {
    kFormatCompact = 0u,   // packaged MXFP4: E2M1 codes two per byte, E8M0 scale per 32 columns
    kFormatExpanded = 1u,  // the same matrix pre-expanded to one E4M3 byte per element, same scales
    kFormatNativeFp8 = 2u  // E4M3 bytes with one E8M0 scale per 128 x 128 block
};
struct ExpertPtrs {
    const uint8_t* w[2];   // gate/up: w1, w3;  down: w2, unused
    const uint8_t* s[2];   // matching E8M0 scales as packaged: [rows][cols/32], or [rows/128][cols/128] (native FP8)
    const uint8_t* ts[2];  // derived copy of the scales, tiled for tcgen05.cp: [row tile][K block][512 bytes]
    uint64_t gen[2];       // generation word of the scale records (what the derived copy is keyed on)
    uint32_t format;       // kFormat* of the expert's matrices
    uint32_t reserved;
};

// Everything a grouped expert kernel needs to find its work, produced by group_slots().
struct GroupedWork {
    const uint32_t* grouped_routes;   // route indices (t*K + r) sorted by expert, stable
    const uint32_t* expert_offsets;   // [num_experts + 1] into grouped_routes
    const ExpertPtrs* experts;        // [num_experts]
    uint32_t num_experts;
};

__device__ __forceinline__ void raise_status(uint32_t* status, uint32_t bit) {
    if (status) atomicOr(status, bit);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    return nvmoe_f32_to_bf16(lo) | (nvmoe_f32_to_bf16(hi) << 16);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// xor-butterfly sum: every lane ends with the same bits; the order is part of the numeric contract
__device__ __forceinline__ float warp_butterfly_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ---- kernels launched by capi.cu (defined in the .cu file named in the comment) ------------

struct RouterLaunch {  // router.cu
    const uint32_t* logits;
    const void* bias;
    uint32_t* routes;
    uint32_t* telemetry;
    uint32_t* status;
    uint32_t tokens;
    nvmoe_geometry g;
};
void launch_router(const RouterLaunch& p, cudaStream_t stream);
void launch_router_linear(const uint16_t* x, const uint16_t* w, const uint16_t* bias, uint32_t* logits,
                          uint32_t tokens, uint32_t hidden, uint32_t outputs, cudaStream_t stream);

struct SortScratch {  // schedule.cu: scratch of the counting sort, sized for max_tokens
    uint32_t* block_hist;      // [blocks][buckets]
    uint32_t* bucket_base;     // [buckets + 1]
    uint32_t blocks_capacity;
    uint32_t buckets_capacity;
};
// moe_route_compact_batch1 / moe_route_count_batch1
void launch_route_compact(const uint32_t* routes, uint32_t* intermediates, const uint32_t* slots,
                          uint32_t slot_words, uint32_t params_per_resource, uint32_t* control,
                          uint32_t max_tokens, uint32_t K, uint32_t intermediate_size,
                          uint32_t tiles_per_route, uint32_t num_experts, const SortScratch& scratch,
                          cudaStream_t stream);
void launch_route_count(const uint32_t* routes, const uint32_t* slots, uint32_t slot_words,
                        uint32_t params_per_resource, uint32_t* control, uint32_t max_tokens, uint32_t K,
                        uint32_t tiles_per_route, cudaStream_t stream);
// (expert, token tile) list of the tensor-core expert kernels from the expert offsets
void launch_build_tiles(const uint32_t* expert_offsets, uint32_t num_experts, uint32_t n_tile, uint32_t* tiles,
                        uint32_t* count, cudaStream_t stream);
// One-launch schedule of a whole layer call for small T*K (layer_schedule_is_small): control words,
// compact list, owned count, and per expert stage [gate/up, down] the grouped routes, expert offsets
// and (when tiles[stage] is set) the tile list. experts[stage] must already be resolved.
struct LayerSchedule {
    const uint32_t* routes;
    uint32_t* intermediates;
    const uint32_t* slots[2];
    uint32_t slot_words[2];
    uint32_t* control[2];
    const ExpertPtrs* experts[2];
    uint32_t* grouped[2];
    uint32_t* offsets[2];
    uint32_t* position[2];  // optional inverse of grouped: position[stage][route] (0xffffffff if dropped)
    uint32_t* tiles[2];
    uint32_t* tile_count[2];
    uint32_t* status;
    uint32_t tokens, expert_start, expert_count, K, I, tiles_per_route[2], num_experts, n_tile[2];
};
bool layer_schedule_is_small(uint32_t tokens, uint32_t K, uint32_t num_experts);
void launch_layer_schedule_small(const LayerSchedule& s, cudaStream_t stream);
// validates the address/slot tables of every expert once per call
// (rows, cols: logical shape of one matrix; experts from native_start on hold native FP8; with
// whole_blocks_only an FP8-form matrix whose columns are not whole 128-blocks is treated as not resident:
// the tensor path stages such a tail for the compact form only)
void launch_resolve_experts(const uint32_t* addresses, uint32_t address_words, const uint32_t* slots,
                            uint32_t slot_words, uint32_t params_per_resource, uint32_t num_experts,
                            uint32_t rows, uint32_t cols, uint32_t native_start, bool whole_blocks_only,
                            uint8_t* derived_scales, size_t derived_matrix_bytes, ExpertPtrs* out, cudaStream_t stream);
// groups the compact slots the expert shaders would visit by expert (stable), skipping what the
// shaders skip; writes grouped_routes and expert_offsets and, if `position` is given, the inverse
// position[route] = place in grouped_routes (0xffffffff for routes that were skipped)
void launch_group_slots(const uint32_t* routes, const uint32_t* intermediates, const uint32_t* control,
                        const ExpertPtrs* experts, uint32_t num_experts, uint32_t max_tokens, uint32_t K,
                        uint32_t intermediate_size, uint32_t* grouped_routes, uint32_t* expert_offsets,
                        uint32_t* position, uint32_t* status, const SortScratch& scratch, cudaStream_t stream);

// expert-parallel dispatch (schedule.cu): routes grouped by the rank owning their expert, stable
// in source order; send_index[i] = position of source route i (kUnboundSlot if dropped),
// send_source[pos] = source route; hidden rows are gathered into send_rows in that order
void launch_ep_pack(const uint16_t* hidden, const uint32_t* routes, const uint32_t* owner, uint32_t tokens,
                    uint32_t K, uint32_t hidden_size, uint32_t num_experts, uint32_t world, uint32_t self,
                    uint16_t* send_rows, uint32_t* send_routes, uint32_t* send_index, uint32_t* send_source,
                    uint32_t* dest_counts, uint32_t* total, uint32_t segment_rows, uint32_t* contiguous_routes,
                    uint32_t* status, const SortScratch& scratch, cudaStream_t stream);
void launch_ep_unpack(const uint16_t* returned_rows, const uint32_t* send_index, uint32_t tokens, uint32_t K,
                      uint32_t hidden_size, uint16_t* expert_outputs, cudaStream_t stream);

// quantize.cu: bf16 rows -> E4M3 bytes + per-block power-of-two scales.
// scales_f32 ([rows][cols/block]) and scales_e8m0 ([rows][ceil(cols/128)] words, four E8M0 bytes of
// consecutive 32-column blocks per word) are both optional.
void launch_quantize(const uint16_t* input, uint32_t rows, uint32_t cols, uint32_t block,
                     size_t input_row_stride, uint8_t* q, float* scales_f32, uint32_t* scales_e8m0,
                     cudaStream_t stream);
// The tensor path's operand form: row `pos` of the output is the quantised source row of route
// grouped_routes[pos] (the token's hidden row when frames is false: source row = route / K of
// `input` with `cols` columns; the route's own row of the intermediates frames otherwise), for pos below
// expert_offsets[num_experts]. Scales as E8M0 words only. Expert-grouped rows are what a tiled TMA
// load can fetch as one box per (expert, token tile).
void launch_quantize_grouped(const void* input, bool frames, const uint32_t* grouped_routes,
                             const uint32_t* expert_offsets, uint32_t num_experts, uint32_t max_routes, uint32_t K,
                             uint32_t cols, uint32_t intermediate_size, uint32_t block, uint8_t* q,
                             uint32_t* scales_e8m0, cudaStream_t stream);
// the same for the K rows of every intermediates frame (skips the schedule words)
void launch_quantize_frames(const uint32_t* intermediates, uint32_t tokens, uint32_t K,
                            uint32_t intermediate_size, uint32_t block, uint8_t* q, float* scales_f32,
                            uint32_t* scales_e8m0, cudaStream_t stream);
// f32 scales -> packed E8M0 words, for prequantised inputs; sets *not_pow2 if a scale is not a power of two
void launch_scales_to_e8m0(const float* scales, uint32_t rows, uint32_t cols, uint32_t block,
                           uint32_t* scales_e8m0, uint32_t* status, cudaStream_t stream);

struct ExpertLaunch {  // experts_simt.cu and experts_tc.cu
    GroupedWork work;
    const uint8_t* act_q;        // [rows][K_dim] E4M3; row = token (gate/up) or route index (down)
    const float* act_scales;     // [rows][K_dim/act_block] f32
    const uint32_t* act_e8m0;    // [rows][ceil(K_dim/128)] packed E8M0 (tensor path)
    const uint32_t* routes;      // route words (down: weights)
    uint32_t* intermediates;     // gate/up output frames
    uint16_t* outputs;           // down output [T][K][H]
    float* partial_outputs;      // down, tensor-parallel form: raw f32 sums [T][K][H] instead of `outputs` (no route weight, no rounding)
    uint32_t* status;
    const uint8_t* tmaps;        // tensor path: 128-byte tensor maps [expert][matrix], null = move weights with cp.async
    // tensor path: act_q / act_e8m0 hold expert-grouped rows (row = position in grouped_routes);
    // act_tmap is the tensor map of act_q with a box of [token tile][128 bytes] (null: fetch rows with cp.async)
    const uint8_t* act_tmap;
    // tensor path, gate/up only: where the down stage's grouping puts each route (its operand row)
    const uint32_t* down_position;
    // tensor path, gate/up only, optional: the down stage's activation quantisation done in the epilogue
    // (E4M3 bytes [down_position][I], E8M0 bytes [down_position][ceil(I/128)] words); needs act_block 32
    uint8_t* q_out;
    uint32_t* q_e8m0;
    uint64_t* cta_trace;         // tensor path diagnostics: [2][grid][4] words per CTA, or null
    uint64_t* scale_stamps;      // tensor path: {scale pointer, generation} the derived tiles were built from
    uint32_t* tile_list;         // tensor path scratch: routes / 16 + experts + 1 words
    uint32_t* tile_count;        // tensor path scratch: one word
    uint32_t tokens;             // upper bound (max over what control may hold)
    long long wait_cycles;       // tensor path: clock cycles after which a bounded in-kernel wait gives up
    uint32_t debug_flags;        // tensor path: bit 0 = CTA 0 leaves out its first stage arrival (exercises the give-up path)
    nvmoe_geometry g;
};
void configure_simt_kernels();
void launch_gate_up_simt(const ExpertLaunch& p, cudaStream_t stream);
void launch_down_simt(const ExpertLaunch& p, cudaStream_t stream);

// ffn_tail.cu: the nodes either side of the MoE chain and the token-id table routing
void launch_rms_norm(const uint16_t* input, const uint16_t* weight, uint16_t* output, uint32_t rows, uint32_t hidden, float eps,
                     float weight_offset, cudaStream_t stream);
void launch_silu_multiply(const uint16_t* gate, const uint16_t* up, uint16_t* out, size_t elements, float limit, cudaStream_t stream);
void launch_add_bf16(const uint16_t* a, const uint16_t* b, uint16_t* out, size_t elements, cudaStream_t stream);
void launch_preselect_table(const uint32_t* token_ids, const uint32_t* table, uint32_t word_stride, uint32_t vocab, uint32_t routed,
                            uint32_t k, uint32_t always, uint32_t tokens, uint32_t* selections, uint32_t* telemetry, uint32_t* status,
                            cudaStream_t stream);
void launch_route_preselected(const uint32_t* logits, const uint32_t* selections, uint32_t tokens, uint32_t* routes, uint32_t* status,
                              const nvmoe_geometry& g, cudaStream_t stream);
// every row a route of expert 0 in row order: grouped list, offsets [0, rows], inverse, (expert, token tile) list
void launch_dense_schedule(uint32_t rows, uint32_t n_tile, uint32_t* grouped, uint32_t* offsets, uint32_t* position, uint32_t* tiles,
                           uint32_t* tile_count, cudaStream_t stream);

// reduce.cu: the same combine with route (t, r) read from row gather[t * K + r] of `rows` (all-ones = a row of
// zeros); false when the shape needs the plain form (hidden not a multiple of 8, unaligned buffers)
bool launch_reduce_gather(const uint16_t* rows, const uint32_t* gather, uint16_t* output, uint32_t tokens, uint32_t K,
                          uint32_t hidden, float routed_scale, cudaStream_t stream);
// reduce.cu: distributed_sum_f32_scale_packed_bf16_to_bf16: out[lane][e] = bf16(sum over participants of
// partials[participant][lane][e] * bf16(scales[lane * (elements / elements_per_scale) + e / elements_per_scale] >> bit_offset))
void launch_sum_f32_scale_packed_bf16(const float* partials, const uint32_t* scales, uint32_t* output, uint32_t element_count,
                                      uint32_t participant_count, uint32_t lane_count, uint32_t elements_per_scale,
                                      uint32_t scale_bit_offset, cudaStream_t stream);

// probe.cu: a run of `groups` x 8 block-scaled MMAs (128 x n_tile x 32, two alternating accumulators)
// on every one of `ctas` CTAs; cycles[cta] = clock cycles from first issue to completion
cudaError_t launch_mma_rate_probe(uint32_t n_tile, uint32_t groups, uint32_t ctas, long long* cycles, uint32_t* status,
                                  cudaStream_t stream);

// reduce.cu: moe_reduce_batch1_bf16. `computed` (optional, [tokens * K]) marks with 0xffffffff the routes
// whose rows were never written: they count as zeros, so the rows need no clearing beforehand.
void launch_reduce(const uint16_t* expert_outputs, uint16_t* output, uint32_t tokens, uint32_t K,
                   uint32_t hidden, float routed_scale, const uint32_t* computed, cudaStream_t stream);

}  // namespace nvmoe
