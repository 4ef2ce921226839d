/*
 * moe_oracle.h — CPU restatement of the reference MoE shaders.  TEST INFRASTRUCTURE ONLY.
 *
 * This library is the checker the CUDA path is compared with.  It is linked or loaded only by
 * the tests, by the smoke check and by the CPU-baseline leg of the benchmark; nothing in the
 * product may call it, and the product has no CPU fallback.
 *
 * Parity status.  Integer results (expert ids, route order, compact lists, control words,
 * telemetry) are pinned by the shader source, which defines them exactly.  The E2M1/E4M3/E8M0
 * tables are pinned against the reference's own Python tables and known-answer tests.  Route
 * WEIGHTS and expert outputs of the reference depend on GLSL transcendental precision, subgroup
 * reduction order and the driver's FP8 dot-product, none of which the reference pins with a test
 * on non-trivial values: at that level this oracle is "parity unpinned" against the reference GPU
 * and pinned only against the constant-fill known answers of
 * runtime-rs/src/vulkan_compute/mxfp4_tests.rs:89-215.
 *
 * Address tables passed to the expert functions hold HOST pointers in the device_address field.
 */
#ifndef MOE_ORACLE_H
#define MOE_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct oracle_router {
    uint32_t routed_experts;
    uint32_t routed_k;
    uint32_t always_count;
    float always_weight;
    uint32_t kind;       /* 0 score_topk, 1 topk_softmax, 2 topk_routed, 3 preselected (oracle_route_preselected) */
    uint32_t activation; /* 0 sigmoid, 1 softmax, 2 sqrt(softplus) */
    uint32_t normalize_selected;
    uint32_t bias_dtype; /* 0 none, 1 f32, 2 bf16 */
    float routed_scale;
    float logit_softcap;
    uint32_t n_group;
    uint32_t topk_group;
} oracle_router;

typedef struct oracle_expert {
    uint32_t hidden_size;
    uint32_t intermediate_size;
    uint32_t num_experts; /* routed + always */
    uint32_t experts_per_token;
    uint32_t tile_rows;
    float swiglu_limit;
    float swiglu_alpha;
    float swiglu_up_offset;
    uint32_t act_block;
    uint32_t tier; /* 0 faithful f32 order, 1 same operands with f64 accumulation, 2 ideal (bf16 activations, f64) */
    uint32_t native_fp8_start; /* NATIVE_FP8_RESOURCE_START: resources from here on hold E4M3 weights with one E8M0
                                  scale per 128 x 128 block; num_experts = none (a zero is read as none too) */
} oracle_expert;

/* linear_bf16.comp.template:39-95; with a non-null bias, linear_bias_bf16.comp.template:31-84 */
void oracle_linear_bf16(const uint16_t* x, const uint16_t* w, const uint16_t* bias,
                        uint32_t tokens, uint32_t hidden, uint32_t outputs, uint32_t* out_words);

/* moe_router_score_topk_batch1_bf16 / moe_topk_bf16 / moe_topk_routed_batch1_bf16.
 * returns the number of tokens that had no selectable score (0 for finite inputs). */
int oracle_route(const oracle_router* p, const uint32_t* logit_words, const void* bias,
                 uint32_t tokens, uint32_t* routes, uint32_t* telemetry);

/* moe_route_compact_batch1.comp.template:26-105 */
void oracle_route_compact(const uint32_t* routes, uint32_t* intermediates, const uint32_t* slots,
                          uint32_t slot_words, uint32_t params_per_resource, uint32_t* control,
                          uint32_t intermediate_size, uint32_t experts_per_token,
                          uint32_t tiles_per_route);

/* The same list by the quadratic ranking the shader literally performs (small inputs only). */
void oracle_route_compact_quadratic(const uint32_t* routes, uint32_t* intermediates,
                                    uint32_t* control, uint32_t intermediate_size,
                                    uint32_t experts_per_token, uint32_t tiles_per_route);

/* moe_route_count_batch1.comp.template:21-58 */
void oracle_route_count(const uint32_t* routes, const uint32_t* slots, uint32_t slot_words,
                        uint32_t params_per_resource, uint32_t* control,
                        uint32_t experts_per_token, uint32_t tiles_per_route);

/* quantize_batch_fp8_e4m3.comp.template:47-71 with the dynamic power-of-two scale */
void oracle_quantize_fp8(const uint16_t* input, uint32_t rows, uint32_t columns, uint32_t block,
                         uint8_t* quantized, float* scales);

/* independent_sparse_moe_gate_up_batch1_mxfp4.comp.template:643-802 */
void oracle_gate_up(const oracle_expert* p, const uint16_t* hidden, const uint32_t* routes,
                    uint32_t* intermediates, const uint32_t* addresses, uint32_t address_words,
                    const uint32_t* slots, uint32_t slot_words, const uint32_t* control);

/* the PREQUANTIZED_INPUT = 1 rendering of the same template */
void oracle_gate_up_prequant(const oracle_expert* p, const uint8_t* q_hidden,
                             const float* hidden_scales, const uint32_t* routes,
                             uint32_t* intermediates, const uint32_t* addresses,
                             uint32_t address_words, const uint32_t* slots, uint32_t slot_words,
                             const uint32_t* control);

/* independent_sparse_moe_down_batch1_mxfp4.comp.template:507-610 */
void oracle_down(const oracle_expert* p, const uint32_t* intermediates, const uint32_t* routes,
                 uint16_t* outputs, const uint32_t* addresses, uint32_t address_words,
                 const uint32_t* slots, uint32_t slot_words, const uint32_t* control);

/* moe_reduce_batch1_bf16.comp.template:29-55 */
void oracle_reduce(const uint16_t* expert_outputs, uint16_t* output, uint32_t tokens,
                   uint32_t experts_per_token, uint32_t hidden, float routed_scale);

/* distributed_sum_f32_scale_packed_bf16_to_bf16.comp:44-66 */
void oracle_sum_f32_scale_packed_bf16(const float* partials, const uint32_t* scales,
                                      uint32_t* out_words, uint32_t element_count,
                                      uint32_t participant_count, uint32_t lane_count,
                                      uint32_t elements_per_scale, uint32_t scale_bit_offset);

/* resource_preselect_table_batch1.comp.template:35-97; returns the number of invalid tokens */
int oracle_resource_preselect_table(const uint32_t* token_ids, const uint32_t* table_words,
                                    uint32_t word_stride, uint32_t vocab, uint32_t routed,
                                    uint32_t k, uint32_t always, uint32_t tokens,
                                    uint32_t* selections, uint32_t* telemetry);

/* moe_router_preselected_batch1_bf16.comp.template:56-91 */
void oracle_route_preselected(const oracle_router* p, const uint32_t* logit_words,
                              const uint32_t* selections, uint32_t tokens, uint32_t* routes);

/* rms_norm_batch_bf16.comp.template:55-108 */
void oracle_rms_norm(const uint16_t* input, const uint16_t* weight, uint16_t* output, uint32_t rows,
                     uint32_t hidden, float eps, float weight_offset);

/* bounded_silu_multiply_batch_bf16.comp.template:26-53 (limit > 0) or
 * silu_multiply_batch_bf16.comp.template:24-52 (limit == 0) */
void oracle_silu_multiply(const uint16_t* gate, const uint16_t* up, uint16_t* out, uint64_t count, float limit);

/* add_batch_bf16.comp.template:36-50 */
void oracle_add_bf16(const uint16_t* a, const uint16_t* b, uint16_t* out, uint64_t count);

/* scalar helpers exported for table tests */
uint32_t oracle_e2m1_to_e4m3(uint32_t nibble);
float oracle_e2m1_value(uint32_t nibble);
float oracle_e4m3_value(uint32_t byte);
uint32_t oracle_f32_to_e4m3(float v);
float oracle_e8m0_value(uint32_t byte);
float oracle_rounded_fp8_scale(float block_max);
uint32_t oracle_f32_to_bf16(float v);
float oracle_expf(float v);
float oracle_logf(float v);
float oracle_tanhf(float v);
void oracle_dequant_mxfp4(const uint8_t* packed, const uint8_t* scales, uint32_t rows,
                          uint32_t columns, float* out);
int oracle_max_threads(void);
int oracle_set_threads(int threads);

#ifdef __cplusplus
}
#endif
#endif
