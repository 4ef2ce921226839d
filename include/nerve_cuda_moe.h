/*
 * nerve_cuda_moe.h — C ABI of the CUDA (sm_100a) backend for NERVE's route-native sparse-expert
 * (MoE) layer with packaged MXFP4 expert weights.
 *
 * The reference runtime has no FFI for this path: its seam is Rust-internal, between the
 * component runner that walks the kernel steps of a mounted component
 *   runtime-rs/src/vulkan_stream_circuit/component_batch_slice_runner.rs:1867-2009 (run_segment)
 * and the Vulkan device object that owns buffers and dispatches
 *   runtime-rs/src/vulkan_compute/compute_device_dispatch.rs:2-273
 *   runtime-rs/src/vulkan_compute/resident_buffers.rs:39-232.
 * This header is what a `cuda-backend` crate would bind at that seam.  It mirrors the device
 * object model (device, resident buffer, create-once/run-many plan), the binding order of each MoE
 * operator (runtime-rs/src/vulkan_stream_circuit/circuit_binding_builder.rs:1-96) and the buffer
 * contracts of the shaders, so that the runtime's slot planner and package layout stay untouched.
 *
 * Conventions
 *   - every call returns 0 on success or a negative nvmoe_status; the text of the last failure is
 *     kept per device (the reference returns Result<_, VulkanError(String)>,
 *     runtime-rs/src/vulkan_compute/features.rs:276-285);
 *   - argument validation is eager and happens before any launch
 *     (compute_device_dispatch.rs:94-130); kernels never fault on bad dynamic metadata, they
 *     leave the output untouched (fail closed) and raise a bit in the plan's status word;
 *   - a device object is single-threaded, like the reference's (device_types.rs:13);
 *   - "word" is a little-endian u32; bf16 values are packed two per word, even element low.
 *
 * Buffer contracts (T = batch_width tokens, K = experts_per_token = routed_k + always_count)
 *   hidden          [T][H] bf16
 *   router weights  [E][H] bf16 row-major
 *   logits          [T][ceil(E/2)] words
 *   routes          [T][K] words, (bf16 weight << 16) | expert id, ascending expert id per token
 *   intermediates   [T][K*I/2 data words | K schedule words]   (frame = K*I/2 + K words)
 *   expert outputs  [T][K][H] bf16
 *   output          [T][H] bf16
 *   control         7 words {batch_width, expert_start, expert_count, owned_route_count,
 *                   dispatch_x, dispatch_y, dispatch_z}
 *   address table   32-byte records {device_address u64, byte_count u64, generation u64,
 *                   resident u32, representation u32}
 *                   (runtime-rs/src/vulkan_compute/stable_resource_address_space.rs:1297-1317)
 *   slot table      expert*P + parameter -> record index or 0xffffffff; P = 4 for gate/up
 *                   (w1, w1 scales, w3, w3 scales), P = 2 for down (w2, w2 scales)
 *   expert weight   I8 [rows][cols/2], low nibble = even column; scales F8_E8M0 [rows][cols/32]
 *                   (nerve/model_package_independent_experts.py:182-257). A record whose representation
 *                   word is 1 holds the same matrix pre-expanded to one E4M3 byte per element
 *                   [rows][cols] (same scales); both matrices of a gate/up pair share one form. A native
 *                   FP8 resource (geometry.native_fp8_resources) holds E4M3 [rows][cols] with E8M0 scales
 *                   [ceil(rows/128)][ceil(cols/128)]
 *                   (independent_sparse_moe_gate_up_batch1_mxfp4.comp.template:166-228,250-355)
 *   telemetry       [R_total counts | R_total(R_total-1)/2 pair counts] u32
 */
#ifndef NERVE_CUDA_MOE_H
#define NERVE_CUDA_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct nvmoe_device nvmoe_device;
typedef struct nvmoe_buffer nvmoe_buffer;
typedef struct nvmoe_plan nvmoe_plan;

typedef enum nvmoe_status {
    NVMOE_OK = 0,
    NVMOE_ERR_INVALID_ARGUMENT = -1, /* geometry, sizes, null handles, range overflow */
    NVMOE_ERR_CUDA = -2,             /* a CUDA runtime call failed; text holds its message */
    NVMOE_ERR_TIMEOUT = -3,          /* nvmoe_sync ran out of time */
    NVMOE_ERR_OUT_OF_MEMORY = -4,
    NVMOE_ERR_UNSUPPORTED = -5,      /* valid in the reference but not built here */
    NVMOE_ERR_COLLECTIVE = -6,       /* expert-parallel exchange failed */
    NVMOE_ERR_DEVICE_STATUS = -7     /* a kernel raised a fail-closed status bit */
} nvmoe_status;

/* Which reference router shader the plan's route call follows. */
typedef enum nvmoe_router_kind {
    NVMOE_ROUTER_SCORE_TOPK = 0,   /* moe_router_score_topk_batch1_bf16.comp.template */
    NVMOE_ROUTER_TOPK_SOFTMAX = 1, /* moe_topk_bf16.comp.template (softmax over the k selected) */
    NVMOE_ROUTER_TOPK_ROUTED = 2,  /* moe_topk_routed_batch1_bf16.comp.template */
    NVMOE_ROUTER_PRESELECTED = 3   /* moe_router_preselected_batch1_bf16.comp.template (nvmoe_route_preselected) */
} nvmoe_router_kind;

typedef enum nvmoe_router_activation {
    NVMOE_ACT_SIGMOID = 0,
    NVMOE_ACT_SOFTMAX = 1,
    NVMOE_ACT_SQRT_SOFTPLUS = 2
} nvmoe_router_activation;

typedef enum nvmoe_bias_dtype { NVMOE_BIAS_NONE = 0, NVMOE_BIAS_F32 = 1, NVMOE_BIAS_BF16 = 2 } nvmoe_bias_dtype;

/* Bits of the device status word (nvmoe_plan_status). */
enum {
    NVMOE_STATUS_ROUTE_NONFINITE = 1u << 0,   /* a token had no selectable finite score */
    NVMOE_STATUS_ROUTE_OUT_OF_RANGE = 1u << 1,/* compact slot or expert id out of range: skipped */
    NVMOE_STATUS_EXPERT_NOT_RESIDENT = 1u << 2,/* address record failed validation: skipped */
    NVMOE_STATUS_WAIT_EXPIRED = 1u << 3,      /* a bounded in-kernel wait gave up */
    NVMOE_STATUS_EXCHANGE_OVERFLOW = 1u << 4, /* more rows were bound for one rank than its segment holds: the
                                                 excess routes were left out (their rows count as zeros) */
    NVMOE_STATUS_INTERNAL = 1u << 5           /* a kernel found a precondition of its own broken (shared-memory
                                                 alignment) and did nothing */
};

/*
 * Everything the reference bakes into shader file names and template constants
 * (nerve/model_package_moe_routing.py:51-82,160-213; nerve/circuit_lowering_sparse_experts.py:80-211).
 * Fields marked "extension" have no counterpart in the reference; their zero/one defaults give
 * the reference behaviour.
 */
typedef struct nvmoe_geometry {
    uint32_t hidden_size;        /* H, multiple of 32 (the reference insists on 128) */
    uint32_t intermediate_size;  /* I, multiple of 32 */
    uint32_t routed_experts;     /* E = routed_resource_count, 0 < k <= E, E + always <= 4096 */
    uint32_t routed_k;           /* routed_selection_count */
    uint32_t always_count;       /* always-selected resources appended with ids E.. */
    float always_weight;         /* their common route weight */
    uint32_t router_kind;        /* nvmoe_router_kind */
    uint32_t activation;         /* nvmoe_router_activation (SCORE_TOPK; ROUTED uses sigmoid flag) */
    uint32_t normalize_selected; /* NORMALIZE_SELECTED */
    uint32_t bias_dtype;         /* nvmoe_bias_dtype of the selection bias */
    float routed_scale;          /* ROUTED_SCALE applied by the router */
    float logit_softcap;         /* TOPK_ROUTED only; 0 = off */
    uint32_t n_group;            /* extension: group-limited routing, 0 = off */
    uint32_t topk_group;         /* extension: groups kept */
    float swiglu_limit;          /* SWIGLU_LIMIT, 0 = off */
    float swiglu_alpha;          /* extension: sigmoid slope, 1 = reference */
    float swiglu_up_offset;      /* extension: added to the up value, 0 = reference */
    uint32_t act_block;          /* activation quantisation block: 128 = reference; 32 for shapes
                                    that 128 does not divide (extension) */
    uint32_t gate_tile_rows;     /* TILE_ROWS of the gate/up shader (32): only shapes control.dispatch_x */
    uint32_t down_tile_rows;     /* TILE_ROWS of the down shader (64) */
    float reduce_scale;          /* ROUTED_SCALE of moe_reduce (1.0 when the router already scaled) */
    uint32_t max_tokens;         /* largest batch_width any call will pass */
    uint32_t native_fp8_resources; /* how many resources at the end of the id range hold native FP8 weights
                                    (E4M3 [rows][cols] with one E8M0 scale per 128 x 128 block): the reference's
                                    NATIVE_FP8_RESOURCE_START = total resources - this count. 0 = none. */
} nvmoe_geometry;

/* Fills a geometry with the reference defaults for the given sizes. */
void nvmoe_geometry_default(nvmoe_geometry* g, uint32_t hidden, uint32_t intermediate,
                            uint32_t experts, uint32_t k);

/* ---- device and resident buffers --------------------------------------------------------- */

/* VulkanComputeDevice::new_for_device_uuid (vulkan_compute/mxfp4_tests.rs:56). */
int nvmoe_device_open(int cuda_ordinal, nvmoe_device** out);
void nvmoe_device_close(nvmoe_device* device);
/* Text of the last error on this device; valid until the next failing call. With a null device
 * it returns the text of the last failed nvmoe_device_open of this thread. */
const char* nvmoe_last_error(const nvmoe_device* device);
/* The CUDA stream every launch of this device uses (a cudaStream_t). */
void* nvmoe_device_stream(const nvmoe_device* device);
/* Launch on a stream the caller owns instead (null restores the device's own stream), so that
 * the operators order with the caller's collectives without events. */
int nvmoe_device_set_stream(nvmoe_device* device, void* cuda_stream);

/* create_resident_buffer / write_bytes[_at] / read_bytes[_at] / device_address
 * (vulkan_compute/resident_buffers.rs:39-232). Buffers are zero-filled at creation. */
int nvmoe_buffer_create(nvmoe_device* device, size_t bytes, nvmoe_buffer** out);
void nvmoe_buffer_destroy(nvmoe_buffer* buffer);
int nvmoe_buffer_write(nvmoe_buffer* buffer, size_t offset, const void* src, size_t bytes);
int nvmoe_buffer_read(nvmoe_buffer* buffer, size_t offset, void* dst, size_t bytes);
int nvmoe_buffer_fill(nvmoe_buffer* buffer, size_t offset, int byte_value, size_t bytes);
/* A handle over device memory the caller allocated (for example a tensor of the host framework);
 * destroying it frees the handle only. The reference's buffers are always device-owned
 * (resident_buffers.rs:39-60); this exists so that collectives and kernels can share memory. */
int nvmoe_buffer_wrap(nvmoe_device* device, void* device_ptr, size_t bytes, nvmoe_buffer** out);
/* The address is for the caller's own kernels and copies. What a plan resolved from an address or slot
 * table (validated pointers, re-tiled scales, tensor maps) is kept until the table is written through
 * nvmoe_buffer_write or nvmoe_buffer_fill; a caller that changes a table through this address instead says
 * so with nvmoe_buffer_mark_dirty before the next call that uses the table, or the old resolution is used.
 * (Tables in wrapped buffers are resolved afresh on every call and need no mark.) */
uint64_t nvmoe_buffer_device_address(const nvmoe_buffer* buffer);
int nvmoe_buffer_mark_dirty(nvmoe_buffer* buffer);
size_t nvmoe_buffer_byte_capacity(const nvmoe_buffer* buffer);

/* Bounded wait for everything queued on the device (run_resident_kernel_sequence's
 * wait-with-timeout, vulkan_compute/compute_device_sequence.rs:746). */
int nvmoe_sync(nvmoe_device* device, uint64_t timeout_ns);

/* ---- plan: one MoE layer geometry, created once and run many times ------------------------ */

int nvmoe_plan_create(nvmoe_device* device, const nvmoe_geometry* geometry, nvmoe_plan** out);
void nvmoe_plan_destroy(nvmoe_plan* plan);
/* Reads and clears the device status word (synchronises the stream). */
int nvmoe_plan_status(nvmoe_plan* plan, uint32_t* status_bits);
/* Chooses the expert kernels: 0 = automatic, 1 = CUDA-core dequant-GEMV, 2 = tcgen05 grouped MMA. */
int nvmoe_plan_set_expert_path(nvmoe_plan* plan, int path);
/* Every wait inside the tensor-core expert kernels (on a pipeline stage, an accumulator) gives up after
 * this many SM clock cycles, raises NVMOE_STATUS_WAIT_EXPIRED and winds the kernel down; the context
 * stays usable and the next call starts clean. Default (and 0): 4e9 cycles, about two seconds. The
 * counterpart of the reference's queue-progress watchdog
 * (runtime-rs/src/vulkan_compute/queue_progress_watchdog.rs:18-60), inside the kernel. */
int nvmoe_plan_set_wait_limit(nvmoe_plan* plan, uint64_t clock_cycles);
/* With profiling on, nvmoe_layer brackets every stage with CUDA events (nvmoe_work_report.stage_ms),
 * the counterpart of the per-step GPU timestamps of
 * runtime-rs/src/vulkan_compute/compute_device_sequence.rs:27-190. Off by default. */
int nvmoe_plan_set_profiling(nvmoe_plan* plan, int enabled);

/* Router projection, op `linear` (runtime-rs/shaders/linear_bf16.comp.template:39-95) or, with a
 * non-null bias, `linear_bias` (runtime-rs/shaders/linear_bias_bf16.comp.template:31-84).
 * bindings: 0 hidden, 1 logits, 2 router weights, 3 bias [E] bf16. */
int nvmoe_router_linear(nvmoe_plan* plan, uint32_t batch_width, const nvmoe_buffer* hidden,
                        nvmoe_buffer* logits, const nvmoe_buffer* router_weights,
                        const nvmoe_buffer* router_bias);

/* op `moe_route` (moe_router_score_topk_batch1_bf16.comp.template:109-220, moe_topk_bf16.comp.template:44-145,
 * moe_topk_routed_batch1_bf16.comp.template:71-182). bindings: 0 logits, 1 routes, 2 bias, 3 telemetry
 * (tests/test_model_package_moe_components.py:490-492). bias may be null when bias_dtype is NONE;
 * telemetry may be null. */
int nvmoe_route(nvmoe_plan* plan, uint32_t batch_width, const nvmoe_buffer* logits,
                nvmoe_buffer* routes, const nvmoe_buffer* bias, nvmoe_buffer* telemetry);

/* op `parameter_table_resource_preselection`
 * (runtime-rs/shaders/resource_preselect_table_batch1.comp.template:35-97): every token's routed
 * resources looked up in a [vocab_size][routed_k] table of 32-bit (table_word_stride 1) or 64-bit
 * (2) integers, always-selected ids appended, ascending. bindings: 0 token ids [T] u32, 1 resource
 * routes [T][K] u32, 2 table, 3 telemetry (optional). A token id beyond the table, an index beyond the
 * routed resources or a repeated index invalidates the token: its words become 0xffffffff, nothing is
 * counted, NVMOE_STATUS_ROUTE_OUT_OF_RANGE is raised. */
int nvmoe_resource_preselect_table(nvmoe_plan* plan, uint32_t batch_width, const nvmoe_buffer* token_ids,
                                   nvmoe_buffer* resource_routes, const nvmoe_buffer* table, uint32_t vocab_size,
                                   uint32_t table_word_stride, nvmoe_buffer* telemetry);

/* op `moe_route` with selection "preselected_resource_indices"
 * (runtime-rs/shaders/moe_router_preselected_batch1_bf16.comp.template:56-91): route words for resources
 * chosen elsewhere, weight = activation(logit) normalised over the routed selections in their stored
 * order. bindings: 0 logits, 1 resource routes, 2 routes. The plan's router_kind must be
 * NVMOE_ROUTER_PRESELECTED. An invalid token of the preselection gives route words 0x0000ffff (weight 0,
 * an id every expert kernel skips) where the shader would read past its logits row. */
int nvmoe_route_preselected(nvmoe_plan* plan, uint32_t batch_width, const nvmoe_buffer* logits,
                            const nvmoe_buffer* resource_routes, nvmoe_buffer* routes);

/* Route scheduler in front of gate/up (runtime-rs/shaders/moe_route_compact_batch1.comp.template:26-105).
 * bindings: 1 routes, 2 intermediates, 3 slots (optional), 31 control. The caller writes
 * {batch_width, expert_start, expert_count, 0,0,0,0} into control first; expert_count == 0 selects
 * the stable expert-major ranking, otherwise the owned-route filter in source order.
 * batch_width is the host's copy of control[0]: it sizes the launch, as the reference host sizes its
 * dispatch (component_batch_slice_runner.rs:909-918); kernels use min(control[0], batch_width). */
int nvmoe_route_compact(nvmoe_plan* plan, uint32_t batch_width, const nvmoe_buffer* routes,
                        nvmoe_buffer* intermediates, const nvmoe_buffer* gate_up_slots,
                        nvmoe_buffer* control);

/* nvmoe_route_compact for callers that must not reach the device allocator (no counterpart in the
 * reference, whose scheduler shader needs no scratch). Same arguments, outputs and errors as
 * nvmoe_route_compact; the scratch of the multi-block counting sort is a fixed array in the library's
 * own device memory instead of the plan's allocation, so the call allocates and frees nothing on the
 * device. Use it where free device memory has been handed to something else (a key/value cache that
 * takes all of it), where the caller holds the allocator's lock, or where an allocation would
 * synchronise the device.
 * Limits: ceil(batch_width * top_k / 256) * (num_experts + 1) <= 65536 and num_experts <= 1022;
 * larger calls return NVMOE_ERR_INVALID_ARGUMENT with the sizes in nvmoe_last_error.
 * The first call on a device looks up the array's address (no allocation, but a runtime call that is
 * not a stream operation); later calls on that device only launch kernels.
 * Every plan and every call on a device shares the one array. Nothing in it has to start at zero
 * (each call writes every word it later reads), so calls that follow one another on one stream need
 * no clearing; calls that overlap on different streams of one device race on it and must be
 * serialised by the caller. */
int nvmoe_route_compact_static(nvmoe_plan* plan, uint32_t batch_width, const nvmoe_buffer* routes,
                               nvmoe_buffer* intermediates, const nvmoe_buffer* gate_up_slots,
                               nvmoe_buffer* control);

/* Route counter in front of down (runtime-rs/shaders/moe_route_count_batch1.comp.template:21-58).
 * bindings: 1 routes, 3 slots (optional), 31 control. */
int nvmoe_route_count(nvmoe_plan* plan, uint32_t batch_width, const nvmoe_buffer* routes,
                      const nvmoe_buffer* down_slots, nvmoe_buffer* control);

/* Shared activation pre-quantisation (runtime-rs/shaders/quantize_batch_fp8_e4m3.comp.template:47-71).
 * bindings: 0 input [rows][columns] bf16, 1 quantised [rows][columns] E4M3 bytes, 2 scales
 * [rows][columns/block] f32. block is geometry.act_block. */
int nvmoe_quantize_fp8(nvmoe_plan* plan, uint32_t rows, uint32_t columns, const nvmoe_buffer* input,
                       nvmoe_buffer* quantized, nvmoe_buffer* scales);

/* op `independent_sparse_moe_gate_up`
 * (runtime-rs/shaders/independent_sparse_moe_gate_up_batch1_mxfp4.comp.template:643-802).
 * bindings: 0 hidden, 1 routes, 2 intermediates, 3 addresses, 4 slots, 31 control. Reads the
 * compact list from the schedule words of `intermediates` exactly as the shader does. */
int nvmoe_gate_up(nvmoe_plan* plan, uint32_t batch_width, const nvmoe_buffer* hidden,
                  const nvmoe_buffer* routes, nvmoe_buffer* intermediates,
                  const nvmoe_buffer* addresses, const nvmoe_buffer* slots,
                  const nvmoe_buffer* control);

/* The `_prequant` variant: bindings 0 q_hidden, 1 scales, 2 routes, 3 intermediates, 4 addresses,
 * 5 slots, 31 control (same template, PREQUANTIZED_INPUT = 1). The f32 scales may be any positive
 * value (both pre-quantisation contracts of nerve/physical_representations.py:9-12). */
int nvmoe_gate_up_prequant(nvmoe_plan* plan, uint32_t batch_width, const nvmoe_buffer* quantized_hidden,
                           const nvmoe_buffer* hidden_scales, const nvmoe_buffer* routes,
                           nvmoe_buffer* intermediates, const nvmoe_buffer* addresses,
                           const nvmoe_buffer* slots, const nvmoe_buffer* control);

/* op `independent_sparse_moe_down`
 * (runtime-rs/shaders/independent_sparse_moe_down_batch1_mxfp4.comp.template:507-610).
 * bindings: 0 intermediates, 1 routes, 2 outputs, 3 addresses, 4 slots, 31 control. */
int nvmoe_down(nvmoe_plan* plan, uint32_t batch_width, const nvmoe_buffer* intermediates,
               const nvmoe_buffer* routes, nvmoe_buffer* outputs, const nvmoe_buffer* addresses,
               const nvmoe_buffer* slots, const nvmoe_buffer* control);

/* Intra-expert tensor parallelism, the reference's `tensor_parallel_expert` strategy
 * (nerve/model_package_physical_experts.py:98-327): the intermediate dimension is cut into ranges aligned to
 * 128, one per participant. A participant is a plan whose intermediate_size is its range: nvmoe_gate_up on
 * the row range of w1/w3 gives its slice of the intermediates (replicated input, partitioned output), and
 * nvmoe_down_partial on the column range of w2 (resident as a [hidden][range/2] matrix with its
 * [hidden][range/32] scales) gives the raw f32 sums over that range
 * (independent_sparse_moe_down_batch1_mxfp4.comp.template:421-505): no route weight, no rounding.
 * bindings as nvmoe_down with `partial_outputs` [T][K][hidden] f32 in place of the outputs; rows of routes
 * the participant skips are zero. */
int nvmoe_down_partial(nvmoe_plan* plan, uint32_t batch_width, const nvmoe_buffer* intermediates,
                       const nvmoe_buffer* routes, nvmoe_buffer* partial_outputs, const nvmoe_buffer* addresses,
                       const nvmoe_buffer* slots, const nvmoe_buffer* control);

/* The finalisation of a reduced output (runtime-rs/shaders/distributed_sum_f32_scale_packed_bf16_to_bf16.comp:44-66):
 * partials [participants][lanes][element_count] f32 are added in participant order, scaled by the bf16 in
 * bits [scale_bit_offset, +16) of scales[lane][element / elements_per_scale] and rounded to bf16 once. For the
 * expert outputs: element_count = K * hidden, elements_per_scale = hidden, scales = the route words, offset 16.
 * bindings: 0 partials, 1 scales, 2 output [lanes][element_count] bf16. */
int nvmoe_sum_f32_scale_packed_bf16(nvmoe_plan* plan, const nvmoe_buffer* partials, const nvmoe_buffer* scales,
                                    nvmoe_buffer* output, uint32_t element_count, uint32_t participant_count,
                                    uint32_t lane_count, uint32_t elements_per_scale, uint32_t scale_bit_offset);

/* op `moe_reduce` (runtime-rs/shaders/moe_reduce_batch1_bf16.comp.template:29-55).
 * bindings: 0 expert outputs, 1 output. */
int nvmoe_reduce(nvmoe_plan* plan, uint32_t batch_width, const nvmoe_buffer* expert_outputs,
                 nvmoe_buffer* output);

/* ---- the nodes either side of the MoE chain (nerve/circuit_lowering_sparse_experts.py:173-209,
 * nerve/circuit_lowering_nodes.py:541-599) ----------------------------------------------------------- */

/* op `rms_norm`, the block's ffn_norm (runtime-rs/shaders/rms_norm_batch_bf16.comp.template:55-108).
 * bindings: 0 input [rows][element_count] bf16, 1 output, 2 weight [element_count] bf16.
 * y = bf16(x * rsqrt(mean(x^2) + eps) * (w + weight_offset)). */
int nvmoe_rms_norm(nvmoe_plan* plan, uint32_t rows, uint32_t element_count, const nvmoe_buffer* input,
                   nvmoe_buffer* output, const nvmoe_buffer* weight, float eps, float weight_offset);

/* ops `bounded_silu_multiply` (limit > 0: runtime-rs/shaders/bounded_silu_multiply_batch_bf16.comp.template:26-53)
 * and `silu_multiply` (limit == 0: runtime-rs/shaders/silu_multiply_batch_bf16.comp.template:24-52, which
 * rounds the activated gate to bf16 before the product). bindings: 0 gate, 1 up, 2 output. */
int nvmoe_silu_multiply(nvmoe_plan* plan, uint32_t rows, uint32_t element_count, const nvmoe_buffer* gate,
                        const nvmoe_buffer* up, nvmoe_buffer* output, float limit);

/* op `residual_add` (runtime-rs/shaders/add_batch_bf16.comp.template:36-50). bindings: 0 a, 1 b, 2 output. */
int nvmoe_residual_add(nvmoe_plan* plan, uint32_t rows, uint32_t element_count, const nvmoe_buffer* a,
                       const nvmoe_buffer* b, nvmoe_buffer* output);

/* op `linear` of the dense shared expert over a packaged MXFP4 matrix (weights I8 [rows][cols/2], scales
 * F8_E8M0 [rows][cols/32], the experts' own tensor contract). bindings: 0 input [T][cols] bf16, 1 output
 * [T][rows] bf16, 2 weights, 3 scales. The reference has no dense MXFP4 linear shader (its dense linears are
 * bf16 or block-scaled FP8); this one computes what the MoE node computes for a resource every token selects
 * with weight one (independent_sparse_moe_down_batch1_mxfp4.comp.template:507-610): activations quantised
 * to E4M3 per geometry.act_block, f32 accumulation, one bf16 rounding, on the same kernels. */
int nvmoe_dense_linear(nvmoe_plan* plan, uint32_t batch_width, const nvmoe_buffer* input, nvmoe_buffer* output,
                       const nvmoe_buffer* weights, const nvmoe_buffer* scales, uint32_t rows, uint32_t cols);

/*
 * The whole chain of nerve/circuit_lowering_sparse_experts.py:80-172 in one call:
 * linear -> moe_route -> (compact -> gate_up) -> (count -> down) -> moe_reduce, with the
 * intermediate frames held in plan-owned memory. router_weights may be null when `logits` is
 * supplied instead (then the projection is skipped). routes_out, telemetry and logits are optional.
 * expert_start/expert_count describe the experts this device owns (0,0 = all).
 * routes_in (optional) hands in routes that were selected elsewhere, [batch_width][top_k] words in the
 * router's output format: projection and router are skipped (the reference's preselected-route
 * form, which an expert-parallel owner runs on the rows it received). expert_outputs (optional)
 * receives the weighted per-route rows [batch_width][top_k][hidden] and the combine is skipped;
 * `output` may then be null.
 */
typedef struct nvmoe_layer_args {
    uint32_t batch_width;
    uint32_t expert_start;
    uint32_t expert_count;
    const nvmoe_buffer* hidden;
    const nvmoe_buffer* router_weights;
    const nvmoe_buffer* router_bias; /* optional bf16 bias of the router projection */
    nvmoe_buffer* logits;
    const nvmoe_buffer* bias;        /* selection bias of the router, per geometry.bias_dtype */
    const nvmoe_buffer* gate_up_addresses;
    const nvmoe_buffer* gate_up_slots;
    const nvmoe_buffer* down_addresses;
    const nvmoe_buffer* down_slots;
    nvmoe_buffer* output;
    nvmoe_buffer* routes_out;
    nvmoe_buffer* telemetry;
    const nvmoe_buffer* routes_in;
    nvmoe_buffer* expert_outputs;
} nvmoe_layer_args;

int nvmoe_layer(nvmoe_plan* plan, const nvmoe_layer_args* args);

/* Host-buffer form of nvmoe_layer: copies `hidden` in from host memory and `output` back inside
 * the call (pinned staging owned by the plan) — the call a runtime makes per decode step. The wait for
 * the result is bounded (60 s, NVMOE_ERR_TIMEOUT after that). */
int nvmoe_layer_host(nvmoe_plan* plan, const nvmoe_layer_args* args, const void* hidden_host,
                     void* output_host);

/* Device time of the last nvmoe_layer call in milliseconds (CUDA events on the device stream);
 * the per-stage report mirrors RuntimeSparseMoeWorkReport
 * (runtime-rs/src/vulkan_stream_circuit/sparse_moe_execution.rs:176-208). */
enum { NVMOE_STAGE_LINEAR, NVMOE_STAGE_ROUTE, NVMOE_STAGE_SCHEDULE, NVMOE_STAGE_QUANTIZE_HIDDEN,
       NVMOE_STAGE_GATE_UP, NVMOE_STAGE_QUANTIZE_INTERMEDIATE, NVMOE_STAGE_DOWN, NVMOE_STAGE_REDUCE,
       NVMOE_STAGE_COUNT };
typedef struct nvmoe_work_report {
    float total_ms;
    float stage_ms[NVMOE_STAGE_COUNT]; /* zeros unless profiling is on */
    float gate_up_kernel_ms;           /* the gate/up expert kernel alone (profiling on) */
    float down_kernel_ms;              /* the down expert kernel alone (profiling on) */
    uint32_t tensor_path;              /* 1 when the expert kernels ran on tcgen05 */
    uint32_t batch_width;
    uint32_t routes;
    uint32_t distinct_experts;
    uint32_t kernel_launches;
    uint64_t weight_bytes_touched;
} nvmoe_work_report;
int nvmoe_plan_last_report(nvmoe_plan* plan, nvmoe_work_report* report);
/* ---- diagnostics (unstable: not part of the drop-in surface, may change between builds) --------------
 * The expert kernels that run by default are compiled without any of these; arming the per-CTA trace
 * switches the plan to instantiations that carry them.
 *
 * Diagnostics of the last tensor-core expert kernels (valid once the trace is armed): counters of CTA 0, twelve words for
 * gate/up then twelve for down: cycles {producer wait, producer total, MMA wait-operands, MMA
 * wait-accumulator, MMA total}, stages, cycles {epilogue wait, epilogue total}, then global-timer
 * nanoseconds {kernel entry, MMA loop begin, MMA loop end, latest exit of any CTA}. Synchronises
 * the stream. No reference counterpart. */
int nvmoe_plan_debug_counters(nvmoe_plan* plan, uint64_t* out24);
/* Per-CTA diagnostics of the tensor-core expert kernels. The first call arms the trace (and writes
 * the CTA count); later calls copy [2 stages][ctas][4] words {loop begin ns, loop end ns, stages
 * consumed, SM id} of the most recent kernels into `out` (room for max_ctas CTAs per stage).
 * Synchronises the stream. No reference counterpart. */
int nvmoe_plan_debug_cta_trace(nvmoe_plan* plan, uint64_t* out, uint32_t max_ctas, uint32_t* ctas);
/* Makes CTA 0 of the gate/up tensor-core kernel leave out its first pipeline-stage arrival, so that its
 * consumer's bounded wait runs out: the way the give-up path (nvmoe_plan_set_wait_limit) is tested
 * without faulting or hanging anything. The call's output is incomplete and NVMOE_STATUS_WAIT_EXPIRED is
 * raised; switch it off again for the next call. */
int nvmoe_plan_debug_withhold_arrival(nvmoe_plan* plan, int enabled);
/* Kernels launched through this plan since it was created. */
uint64_t nvmoe_plan_launch_count(const nvmoe_plan* plan);

/* Measured peak of the tensor-core instruction the expert kernels issue (tcgen05.mma kind::mxf8f6f4,
 * block-scaled, 128 x n_tile x 32 per instruction, E2M1 weights x E4M3 activations): one CTA per SM
 * issues k_groups x 8 instructions on operands resident in shared memory, alternating two accumulators
 * as the gate/up kernel does. tflops is the rate over all SMs (CUDA events, best of two runs): the
 * denominator of the tensor-bound roofline for the instruction kind that runs. No reference counterpart. */
typedef struct nvmoe_mma_probe {
    uint32_t n_tile;
    uint32_t ctas;
    uint64_t mmas_per_cta;
    float elapsed_ms;
    double cycles_per_mma;        /* slowest CTA's cycles / instructions issued */
    double tflops;
    double sm_clock_mhz_nominal;  /* the device's advertised SM clock, for reading cycles_per_mma */
} nvmoe_mma_probe;
int nvmoe_probe_mma_rate(nvmoe_device* device, uint32_t n_tile, uint32_t k_groups, nvmoe_mma_probe* out);

/*
 * Expert-parallel exchange, the all-to-all form of the reference's expert-range ownership
 * (nerve/physical_execution_contracts.py:690-757; ownership "every resource owned exactly once",
 * runtime-rs/src/vulkan_distributed/selected_resource_placement.rs:289-351).
 *
 * nvmoe_ep_pack groups the T*K routes of this rank's tokens by the rank that owns their expert
 * (owner_table[expert] = rank, 0xffffffff = replicated on every rank, i.e. kept local), stably in
 * source order, and gathers the hidden row of each route into send_rows in that order.
 *   send_routes[pos]  the route word travelling with row pos
 *   send_index[i]     position of source route i = t*K + r (0xffffffff if it was dropped)
 *   dest_counts[rank] rows bound for each rank (the split sizes of the all-to-all)
 * nvmoe_ep_unpack puts the rows that came back (same positions) into expert_outputs [T][K][H] so
 * that moe_reduce runs unchanged.
 * segment_rows = 0 packs the rows back to back (split sizes = dest_counts, which the host must read
 * before the exchange). segment_rows > 0 (at least T*K) gives every destination rank its own segment
 * of that many slots in send_rows / send_routes (world_size * segment_rows slots in all): unused
 * slots carry the route word 0xffffffff, which no scheduler keeps, so the exchange can use equal
 * splits and nothing has to reach the host; send_index then holds slots of that layout. Segments of
 * T*K rows can never overflow. Smaller segments (a capacity bound, say twice the mean T*K/world) move
 * and schedule proportionally less; if more rows are bound for a rank than its segment holds, the excess
 * routes are left out, their rows count as zeros in the combine, and NVMOE_STATUS_EXCHANGE_OVERFLOW is
 * raised in the plan's status word: the caller repeats the step with full segments.
 */
int nvmoe_ep_pack(nvmoe_plan* plan, uint32_t batch_width, const nvmoe_buffer* hidden,
                  const nvmoe_buffer* routes, const nvmoe_buffer* owner_table, uint32_t world_size,
                  uint32_t rank, nvmoe_buffer* send_rows, nvmoe_buffer* send_routes,
                  nvmoe_buffer* send_index, nvmoe_buffer* dest_counts, uint32_t segment_rows);
int nvmoe_ep_unpack(nvmoe_plan* plan, uint32_t batch_width, const nvmoe_buffer* returned_rows,
                    const nvmoe_buffer* send_index, nvmoe_buffer* expert_outputs);

/*
 * The expert-parallel layer with the collectives inside the call: one process per GPU, each opening
 * its device, creating its plans and joining the same communicator. NCCL is bound at run time: the
 * libnccl.so.2 already in the process, else the file NVMOE_NCCL_LIBRARY names, else the system's. A
 * process shares one libnccl.so.2: a framework that ships its own must be loaded before the first call
 * here (or its copy named in NVMOE_NCCL_LIBRARY).
 *
 *   rank 0:      nvmoe_ep_unique_id(id)        then hands the 128 bytes to every rank (any transport)
 *   every rank:  nvmoe_ep_create(device, id, rank, world, &ep)     collective: all ranks must call it
 *   per step:    nvmoe_ep_layer(ep, home, work, &args)             collective
 *
 * `home` is the plan of this rank's tokens (the layer's geometry, max_tokens the same on every
 * rank); `work` the owner-side plan: top_k 1 over the same experts and sizes, max_tokens at least
 * world_size * the segment size (args.capacity_rows, or home.max_tokens * home.top_k when that is 0). The slot tables name the experts this rank holds
 * (0xffffffff for the others); owner_table[expert] is the rank holding each expert (0xffffffff =
 * replicated, kept local). One step is: projection and router on the rank's tokens, rows placed in
 * fixed segments per owner (nvmoe_ep_pack with segment_rows), one grouped send/receive of rows and
 * route words, the preselected-route form of nvmoe_layer on the received rows, one grouped
 * send/receive back, nvmoe_ep_unpack and the combine. Nothing is read on the host; everything is
 * ordered on the device's stream. The result equals the single-device layer bit for bit.
 * The reference shards this layer by expert range with the hidden frame replicated
 * (runtime-rs/src/vulkan_distributed/execution_plans.rs:1201-1205); it has no counterpart of the
 * exchange.
 */
typedef struct nvmoe_ep nvmoe_ep;
typedef struct nvmoe_ep_layer_args {
    uint32_t batch_width;               /* tokens of this rank in this step */
    const nvmoe_buffer* hidden;         /* [batch_width][hidden] bf16 */
    const nvmoe_buffer* router_weights;
    const nvmoe_buffer* router_bias;    /* optional */
    const nvmoe_buffer* bias;           /* selection bias, optional */
    const nvmoe_buffer* owner_table;    /* [experts] u32 */
    const nvmoe_buffer* gate_up_addresses;
    const nvmoe_buffer* gate_up_slots;
    const nvmoe_buffer* down_addresses;
    const nvmoe_buffer* down_slots;
    nvmoe_buffer* output;               /* [batch_width][hidden] bf16 */
    nvmoe_buffer* telemetry;            /* optional */
    uint32_t capacity_rows;             /* rows of the segment each rank keeps for each peer, the same on every rank;
                                           0 = home.max_tokens * top_k (cannot overflow). See nvmoe_ep_pack. */
} nvmoe_ep_layer_args;
int nvmoe_ep_unique_id(void* id128);
int nvmoe_ep_create(nvmoe_device* device, const void* id128, uint32_t rank, uint32_t world_size, nvmoe_ep** out);
void nvmoe_ep_destroy(nvmoe_ep* ep);
int nvmoe_ep_layer(nvmoe_ep* ep, nvmoe_plan* home, nvmoe_plan* work, const nvmoe_ep_layer_args* args);
/* Failure behaviour of nvmoe_ep_layer. Whatever can fail on one rank alone (allocation, the resolution of the
 * expert tables) happens before the first exchange; once a rank has posted the first exchange it always posts
 * the second, and reports the first error afterwards, so that no peer is left waiting for a half-finished
 * step. A peer that does not take part at all (it crashed, or returned before the exchange) is detected by
 * time: nvmoe_ep_sync waits for the stream for at most timeout_ns, polling the communicator for asynchronous
 * errors meanwhile, and on an error or on timeout aborts the communicator, which ends the kernels waiting on
 * the peer; it returns NVMOE_ERR_COLLECTIVE or NVMOE_ERR_TIMEOUT and the communicator refuses further calls.
 * The counterpart of the reference's queue-progress watchdog
 * (runtime-rs/src/vulkan_compute/queue_progress_watchdog.rs:18-60) for a step that spans devices. */
int nvmoe_ep_sync(nvmoe_ep* ep, uint64_t timeout_ns);

#ifdef __cplusplus
}
#endif

#endif /* NERVE_CUDA_MOE_H */
