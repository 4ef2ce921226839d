/*
 * moe_oracle.c — CPU restatement of the reference MoE shaders.  TEST INFRASTRUCTURE ONLY:
 * loaded by the tests, the smoke check and the benchmark's CPU-baseline leg, never by the
 * product.  See moe_oracle.h for the parity status of each part.
 *
 * Every function names the reference shader lines it follows (paths relative to the reference
 * project root).  Scalar arithmetic that the shaders leave to the GLSL implementation
 * (exp/log/tanh precision, subgroup reduction order) uses the pinned definitions of
 * include/nvmoe_math.h and the reduction orders stated in the comments below.
 */
#include "moe_oracle.h"

#include <stdlib.h>
#include <string.h>

#include "../include/nvmoe_math.h"

#ifdef _OPENMP
#include <omp.h>
#endif

#define NEG_INF (-nvmoe_bits_f32(0x7f800000u))
#define UNBOUND_SLOT 0xffffffffu
#define RECORD_WORDS 8u

/* ------------------------------------------------------------------------------------------ */
/* small exported helpers                                                                     */

uint32_t oracle_e2m1_to_e4m3(uint32_t nibble) { return nvmoe_e2m1_to_e4m3_bits(nibble); }
float oracle_e2m1_value(uint32_t nibble) { return nvmoe_e2m1_to_f32(nibble); }
float oracle_e4m3_value(uint32_t byte) { return nvmoe_e4m3_to_f32(byte); }
uint32_t oracle_f32_to_e4m3(float v) { return nvmoe_f32_to_e4m3(v); }
float oracle_e8m0_value(uint32_t byte) { return nvmoe_e8m0_to_f32(byte); }
float oracle_rounded_fp8_scale(float block_max) { return nvmoe_rounded_fp8_scale(block_max); }
uint32_t oracle_f32_to_bf16(float v) { return nvmoe_f32_to_bf16(v); }
float oracle_expf(float v) { return nvmoe_expf(v); }
float oracle_logf(float v) { return nvmoe_logf(v); }
float oracle_tanhf(float v) { return nvmoe_tanhf(v); }

int oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* threads the next calls use (a benchmark's single-core figure); returns the previous setting */
int oracle_set_threads(int threads) {
#ifdef _OPENMP
    int before = omp_get_max_threads();
    if (threads > 0) omp_set_num_threads(threads);
    return before;
#else
    (void)threads;
    return 1;
#endif
}

static inline float unpack_bf16(const uint32_t* words, uint32_t index) {
    uint32_t packed = words[index >> 1];
    return nvmoe_bf16_to_f32((index & 1u) == 0u ? packed : packed >> 16);
}

/* Pinned stand-in for subgroupAdd over 64 lanes: xor butterfly 32,16,8,4,2,1. */
static float butterfly_sum64(float* lanes) {
    for (uint32_t step = 32u; step >= 1u; step >>= 1) {
        float next[64];
        for (uint32_t lane = 0; lane < 64u; lane++) next[lane] = lanes[lane] + lanes[lane ^ step];
        memcpy(lanes, next, sizeof(next));
    }
    return lanes[0];
}

void oracle_dequant_mxfp4(const uint8_t* packed, const uint8_t* scales, uint32_t rows,
                          uint32_t columns, float* out) {
    for (uint32_t r = 0; r < rows; r++) {
        for (uint32_t c = 0; c < columns; c++) {
            uint8_t byte = packed[(size_t)r * (columns / 2u) + c / 2u];
            uint32_t nibble = (c & 1u) ? (byte >> 4) : (byte & 0xfu);
            out[(size_t)r * columns + c] =
                nvmoe_e2m1_to_f32(nibble) * nvmoe_e8m0_to_f32(scales[(size_t)r * (columns / 32u) + c / 32u]);
        }
    }
}

/* ------------------------------------------------------------------------------------------ */
/* router projection: linear_bf16.comp.template:39-95, linear_bias_bf16.comp.template:31-84    */
/* 64 lanes stride over the packed input words with two f32 fma per word (:52-66); the         */
/* subgroupAdd of :69-70 is taken as the pinned butterfly.                                     */

void oracle_linear_bf16(const uint16_t* x, const uint16_t* w, const uint16_t* bias,
                        uint32_t tokens, uint32_t hidden, uint32_t outputs, uint32_t* out_words) {
    uint32_t input_words = hidden / 2u;
    uint32_t out_word_count = (outputs + 1u) / 2u;
#pragma omp parallel for schedule(static)
    for (int64_t tt = 0; tt < (int64_t)tokens; tt++) {
        uint32_t t = (uint32_t)tt;
        const uint16_t* xr = x + (size_t)t * hidden;
        for (uint32_t ow = 0; ow < out_word_count; ow++) {
            uint32_t packed = 0;
            for (uint32_t half = 0; half < 2u; half++) {
                uint32_t row = ow * 2u + half;
                if (row >= outputs) continue;
                const uint16_t* wr = w + (size_t)row * hidden;
                float lanes[64];
                for (uint32_t lane = 0; lane < 64u; lane++) {
                    float sum = 0.0f;
                    for (uint32_t cw = lane; cw < input_words; cw += 64u) {
                        sum = fmaf(nvmoe_bf16_to_f32(xr[2u * cw]), nvmoe_bf16_to_f32(wr[2u * cw]), sum);
                        sum = fmaf(nvmoe_bf16_to_f32(xr[2u * cw + 1u]), nvmoe_bf16_to_f32(wr[2u * cw + 1u]), sum);
                    }
                    lanes[lane] = sum;
                }
                float total = butterfly_sum64(lanes);
                /* linear_bias_bf16.comp.template:31-35 adds the bias before the one bf16 rounding */
                if (bias) total = total + nvmoe_bf16_to_f32(bias[row]);
                packed |= nvmoe_f32_to_bf16(total) << (16u * half);
            }
            out_words[(size_t)t * out_word_count + ow] = packed;
        }
    }
}

/* ------------------------------------------------------------------------------------------ */
/* routers                                                                                     */

static float read_bias(const oracle_router* p, const void* bias, uint32_t expert) {
    if (p->bias_dtype == 1u) return ((const float*)bias)[expert];
    if (p->bias_dtype == 2u) return nvmoe_bf16_to_f32(((const uint16_t*)bias)[expert]);
    return 0.0f;
}

/* Extension: keep the topk_group groups with the largest (best + second best) selection score;
 * ties go to the lower group index. allowed[e] = 1 when expert e may be selected. */
static void group_mask(const oracle_router* p, const float* score, uint8_t* allowed) {
    uint32_t E = p->routed_experts;
    if (p->n_group == 0u) {
        memset(allowed, 1, E);
        return;
    }
    uint32_t per = E / p->n_group;
    float* gscore = (float*)malloc(sizeof(float) * p->n_group);
    uint8_t* kept = (uint8_t*)calloc(p->n_group, 1);
    for (uint32_t g = 0; g < p->n_group; g++) {
        float first = NEG_INF, second = NEG_INF;
        for (uint32_t j = 0; j < per; j++) {
            float s = score[g * per + j];
            if (s > first) {
                second = first;
                first = s;
            } else if (s > second) {
                second = s;
            }
        }
        gscore[g] = per >= 2u ? first + second : first;
    }
    for (uint32_t round = 0; round < p->topk_group; round++) {
        float best = NEG_INF;
        uint32_t best_g = UNBOUND_SLOT;
        for (uint32_t g = 0; g < p->n_group; g++) {
            if (kept[g]) continue;
            if (gscore[g] > best || (gscore[g] == best && g < best_g)) {
                best = gscore[g];
                best_g = g;
            }
        }
        if (best_g != UNBOUND_SLOT) kept[best_g] = 1;
    }
    for (uint32_t e = 0; e < E; e++) allowed[e] = kept[e / per];
    free(gscore);
    free(kept);
}

static void write_routes_and_telemetry(uint32_t* routes_row, uint32_t* telemetry,
                                       const uint32_t* ids, const float* weights, uint32_t count,
                                       uint32_t total_resources) {
    for (uint32_t r = 0; r < count; r++) {
        routes_row[r] = (nvmoe_f32_to_bf16(weights[r]) << 16) | ids[r];
        if (telemetry) {
#pragma omp atomic
            telemetry[ids[r]]++;
        }
    }
    if (!telemetry) return;
    for (uint32_t l = 0; l < count; l++) {
        uint32_t left = ids[l];
        for (uint32_t rr = l + 1u; rr < count; rr++) {
            uint32_t right = ids[rr];
            if (left < right) {
                uint32_t preceding = left * (2u * total_resources - left - 1u) / 2u;
                uint32_t pair_index = preceding + right - left - 1u;
#pragma omp atomic
                telemetry[total_resources + pair_index]++;
            }
        }
    }
}

static void insertion_sort_routes(uint32_t* ids, float* weights, uint32_t count) {
    for (uint32_t route = 1; route < count; route++) {
        uint32_t expert = ids[route];
        float weight = weights[route];
        uint32_t insertion = route;
        while (insertion > 0u && ids[insertion - 1u] > expert) {
            ids[insertion] = ids[insertion - 1u];
            weights[insertion] = weights[insertion - 1u];
            insertion--;
        }
        ids[insertion] = expert;
        weights[insertion] = weight;
    }
}

/* k rounds of argmax with the shader's comparator; returns how many rounds found no candidate */
static uint32_t select_topk(const float* score, const uint8_t* allowed, uint32_t E, uint32_t k,
                            uint32_t* top, uint8_t* selected) {
    uint32_t missing = 0;
    memset(selected, 0, E);
    for (uint32_t route = 0; route < k; route++) {
        float best = NEG_INF;
        uint32_t best_e = UNBOUND_SLOT;
        for (uint32_t e = 0; e < E; e++) {
            if (selected[e] || (allowed && !allowed[e])) continue;
            float s = score[e];
            if (s > best || (s == best && e < best_e)) {
                best = s;
                best_e = e;
            }
        }
        if (best_e == UNBOUND_SLOT) {
            missing++;
            top[route] = UNBOUND_SLOT;
        } else {
            top[route] = best_e;
            selected[best_e] = 1;
        }
    }
    return missing;
}

/* moe_router_score_topk_batch1_bf16.comp.template:109-220 */
static int route_score_topk(const oracle_router* p, const uint32_t* logit_words, const void* bias,
                            uint32_t t, uint32_t* routes, uint32_t* telemetry, float* raw,
                            float* values, float* score, uint8_t* allowed, uint8_t* selected) {
    uint32_t E = p->routed_experts, k = p->routed_k;
    uint32_t total_k = k + p->always_count;
    uint32_t router_words = (E + 1u) / 2u;
    const uint32_t* row = logit_words + (size_t)t * router_words;
    for (uint32_t e = 0; e < E; e++) raw[e] = unpack_bf16(row, e);
    float softmax_max = NEG_INF, softmax_den = 0.0f;
    if (p->activation == 1u) {
        /* :77-107; the lane-strided partial sums are from the shader, the cross-lane sum is pinned */
        for (uint32_t e = 0; e < E; e++) softmax_max = fmaxf(softmax_max, raw[e]);
        float lanes[64];
        for (uint32_t lane = 0; lane < 64u; lane++) {
            float s = 0.0f;
            for (uint32_t e = lane; e < E; e += 64u) s += nvmoe_expf(raw[e] - softmax_max);
            lanes[lane] = s;
        }
        softmax_den = butterfly_sum64(lanes);
    }
    for (uint32_t e = 0; e < E; e++) {
        float v = raw[e];
        if (p->activation == 0u) {
            values[e] = nvmoe_sigmoidf(v);
        } else if (p->activation == 1u) {
            values[e] = nvmoe_expf(v - softmax_max) / softmax_den;
        } else {
            values[e] = sqrtf(nvmoe_softplusf(v));
        }
        score[e] = values[e] + read_bias(p, bias, e);
    }
    group_mask(p, score, allowed);
    uint32_t top[64];
    float weights[64];
    uint32_t missing = select_topk(score, allowed, E, k, top, selected);
    if (missing) {
        /* fail closed: the reference would index out of bounds here (:152-161) */
        for (uint32_t r = 0; r < total_k; r++) routes[(size_t)t * total_k + r] = 0u;
        return 1;
    }
    float denominator = 0.0f;
    if (p->normalize_selected) {
        for (uint32_t r = 0; r < k; r++) denominator += values[top[r]];
    }
    for (uint32_t r = 0; r < k; r++) {
        float weight = values[top[r]];
        if (p->normalize_selected) {
            weight = weight / denominator * p->routed_scale;
        } else {
            weight *= p->routed_scale;
        }
        weights[r] = weight;
    }
    for (uint32_t offset = 0; offset < p->always_count; offset++) {
        top[k + offset] = E + offset;
        weights[k + offset] = p->always_weight;
    }
    insertion_sort_routes(top, weights, total_k);
    write_routes_and_telemetry(routes + (size_t)t * total_k, telemetry, top, weights, total_k,
                               E + p->always_count);
    return 0;
}

/* moe_topk_bf16.comp.template:44-145 (softmax over the k selected, max = first selected) */
static int route_topk_softmax(const oracle_router* p, const uint32_t* logit_words, uint32_t t,
                              uint32_t* routes, uint32_t* telemetry, float* raw, uint8_t* allowed,
                              uint8_t* selected) {
    uint32_t E = p->routed_experts, k = p->routed_k;
    uint32_t router_words = (E + 1u) / 2u;
    const uint32_t* row = logit_words + (size_t)t * router_words;
    for (uint32_t e = 0; e < E; e++) raw[e] = unpack_bf16(row, e);
    group_mask(p, raw, allowed);
    uint32_t top[64];
    float scores[64], weights[64];
    if (select_topk(raw, allowed, E, k, top, selected)) {
        for (uint32_t r = 0; r < k; r++) routes[(size_t)t * k + r] = 0u;
        return 1;
    }
    for (uint32_t r = 0; r < k; r++) scores[r] = raw[top[r]];
    float maximum = scores[0];
    float denominator = 0.0f;
    for (uint32_t r = 0; r < k; r++) denominator += nvmoe_expf(scores[r] - maximum);
    insertion_sort_routes(top, scores, k);
    for (uint32_t r = 0; r < k; r++) weights[r] = nvmoe_expf(scores[r] - maximum) / denominator;
    write_routes_and_telemetry(routes + (size_t)t * k, telemetry, top, weights, k, E);
    return 0;
}

/* moe_topk_routed_batch1_bf16.comp.template:71-182 */
static int route_topk_routed(const oracle_router* p, const uint32_t* logit_words, const void* bias,
                             uint32_t t, uint32_t* routes, uint32_t* telemetry, float* values,
                             float* score, uint8_t* allowed, uint8_t* selected) {
    uint32_t E = p->routed_experts, k = p->routed_k;
    uint32_t router_words = (E + 1u) / 2u;
    const uint32_t* row = logit_words + (size_t)t * router_words;
    int sigmoid = p->activation == 0u;
    for (uint32_t e = 0; e < E; e++) {
        float v = unpack_bf16(row, e);
        if (p->logit_softcap > 0.0f) v = nvmoe_tanhf(v / p->logit_softcap) * p->logit_softcap;
        values[e] = v;
        score[e] = (sigmoid ? nvmoe_sigmoidf(v) : v) + read_bias(p, bias, e);
    }
    group_mask(p, score, allowed);
    uint32_t top[64];
    float weights[64];
    if (select_topk(score, allowed, E, k, top, selected)) {
        for (uint32_t r = 0; r < k; r++) routes[(size_t)t * k + r] = 0u;
        return 1;
    }
    float maximum = values[top[0]];
    float denominator = 0.0f;
    if (p->normalize_selected) {
        for (uint32_t r = 0; r < k; r++) {
            float logit = values[top[r]];
            denominator += sigmoid ? nvmoe_sigmoidf(logit) : nvmoe_expf(logit - maximum);
        }
    } else if (!sigmoid) {
        maximum = NEG_INF;
        for (uint32_t e = 0; e < E; e++) maximum = fmaxf(maximum, values[e]);
        for (uint32_t e = 0; e < E; e++) denominator += nvmoe_expf(values[e] - maximum);
    }
    for (uint32_t r = 0; r < k; r++) weights[r] = 0.0f;
    insertion_sort_routes(top, weights, k);
    for (uint32_t r = 0; r < k; r++) {
        float logit = values[top[r]];
        float weight = sigmoid ? nvmoe_sigmoidf(logit) : nvmoe_expf(logit - maximum);
        if (p->normalize_selected || !sigmoid) weight /= denominator;
        weights[r] = weight;
    }
    write_routes_and_telemetry(routes + (size_t)t * k, telemetry, top, weights, k, E);
    return 0;
}

int oracle_route(const oracle_router* p, const uint32_t* logit_words, const void* bias,
                 uint32_t tokens, uint32_t* routes, uint32_t* telemetry) {
    int bad = 0;
    uint32_t E = p->routed_experts;
#pragma omp parallel reduction(+ : bad)
    {
        float* raw = (float*)malloc(sizeof(float) * E);
        float* values = (float*)malloc(sizeof(float) * E);
        float* score = (float*)malloc(sizeof(float) * E);
        uint8_t* allowed = (uint8_t*)malloc(E);
        uint8_t* selected = (uint8_t*)malloc(E);
#pragma omp for schedule(static)
        for (int64_t tt = 0; tt < (int64_t)tokens; tt++) {
            uint32_t t = (uint32_t)tt;
            if (p->kind == 0u) {
                bad += route_score_topk(p, logit_words, bias, t, routes, telemetry, raw, values,
                                        score, allowed, selected);
            } else if (p->kind == 1u) {
                bad += route_topk_softmax(p, logit_words, t, routes, telemetry, raw, allowed,
                                          selected);
            } else {
                bad += route_topk_routed(p, logit_words, bias, t, routes, telemetry, values, score,
                                         allowed, selected);
            }
        }
        free(raw);
        free(values);
        free(score);
        free(allowed);
        free(selected);
    }
    return bad;
}

/* ------------------------------------------------------------------------------------------ */
/* route scheduler: moe_route_compact_batch1.comp.template / moe_route_count_batch1            */

static int resource_is_local(const uint32_t* slots, uint32_t slot_words, uint32_t params,
                             uint32_t expert) {
    if (!slots) return 1;
    uint64_t index = (uint64_t)expert * params;
    if (index >= slot_words) return 0;
    return slots[index] != UNBOUND_SLOT;
}

static inline uint32_t* schedule_word(uint32_t* intermediates, uint32_t rank, uint32_t K,
                                      uint32_t frame_words, uint32_t data_words) {
    return intermediates + (size_t)(rank / K) * frame_words + data_words + rank % K;
}

void oracle_route_compact(const uint32_t* routes, uint32_t* intermediates, const uint32_t* slots,
                          uint32_t slot_words, uint32_t params_per_resource, uint32_t* control,
                          uint32_t intermediate_size, uint32_t K, uint32_t tiles_per_route) {
    uint32_t data_words = K * (intermediate_size / 2u);
    uint32_t frame_words = data_words + K;
    uint32_t T = control[0];
    uint32_t source_count = T * K;
    if (control[2] != 0u) {
        /* :27-60 owned-route filter in source order */
        uint32_t start = control[1], end = control[1] + control[2];
        uint32_t owned = 0;
        for (uint32_t s = 0; s < source_count; s++) {
            uint32_t expert = routes[s] & 0xffffu;
            if (expert < start || expert >= end ||
                !resource_is_local(slots, slot_words, params_per_resource, expert))
                continue;
            *schedule_word(intermediates, owned, K, frame_words, data_words) = s;
            owned++;
        }
        control[3] = owned;
        control[4] = owned * tiles_per_route;
        control[5] = 1u;
        control[6] = 1u;
        return;
    }
    /* :66-105 rank(s) = #{c : expert(c) < expert(s) or (equal and c < s)} — a stable counting sort */
    control[3] = source_count;
    control[4] = K * tiles_per_route;
    control[5] = T;
    control[6] = 1u;
    uint32_t* offsets = (uint32_t*)calloc(65537u, sizeof(uint32_t));
    for (uint32_t s = 0; s < source_count; s++) offsets[(routes[s] & 0xffffu) + 1u]++;
    for (uint32_t e = 0; e < 65536u; e++) offsets[e + 1u] += offsets[e];
    for (uint32_t s = 0; s < source_count; s++) {
        uint32_t rank = offsets[routes[s] & 0xffffu]++;
        *schedule_word(intermediates, rank, K, frame_words, data_words) = s;
    }
    free(offsets);
}

void oracle_route_compact_quadratic(const uint32_t* routes, uint32_t* intermediates,
                                    uint32_t* control, uint32_t intermediate_size, uint32_t K,
                                    uint32_t tiles_per_route) {
    uint32_t data_words = K * (intermediate_size / 2u);
    uint32_t frame_words = data_words + K;
    uint32_t T = control[0];
    uint32_t route_count = T * K;
    control[3] = route_count;
    control[4] = K * tiles_per_route;
    control[5] = T;
    control[6] = 1u;
    for (uint32_t s = 0; s < route_count; s++) {
        uint32_t source_expert = routes[s] & 0xffffu;
        uint32_t rank = 0;
        for (uint32_t c = 0; c < route_count; c++) {
            uint32_t ce = routes[c] & 0xffffu;
            if (ce < source_expert || (ce == source_expert && c < s)) rank++;
        }
        *schedule_word(intermediates, rank, K, frame_words, data_words) = s;
    }
}

void oracle_route_count(const uint32_t* routes, const uint32_t* slots, uint32_t slot_words,
                        uint32_t params_per_resource, uint32_t* control, uint32_t K,
                        uint32_t tiles_per_route) {
    uint32_t T = control[0];
    if (control[2] == 0u) {
        control[3] = T * K;
        control[4] = K * tiles_per_route;
        control[5] = T;
        control[6] = 1u;
        return;
    }
    uint32_t start = control[1], end = control[1] + control[2];
    uint32_t owned = 0;
    for (uint32_t s = 0; s < T * K; s++) {
        uint32_t expert = routes[s] & 0xffffu;
        if (expert >= start && expert < end &&
            resource_is_local(slots, slot_words, params_per_resource, expert))
            owned++;
    }
    control[3] = owned;
    control[4] = owned * tiles_per_route;
    control[5] = 1u;
    control[6] = 1u;
}

/* ------------------------------------------------------------------------------------------ */
/* activation quantisation                                                                     */

static void quantize_row(const uint16_t* in, uint32_t columns, uint32_t block, uint8_t* q,
                         float* scales) {
    for (uint32_t b = 0; b < columns / block; b++) {
        float block_max = 0.0f;
        for (uint32_t c = 0; c < block; c++)
            block_max = fmaxf(block_max, fabsf(nvmoe_bf16_to_f32(in[b * block + c])));
        float scale = nvmoe_rounded_fp8_scale(block_max);
        scales[b] = scale;
        for (uint32_t c = 0; c < block; c++)
            q[b * block + c] = (uint8_t)nvmoe_f32_to_e4m3(nvmoe_bf16_to_f32(in[b * block + c]) / scale);
    }
}

void oracle_quantize_fp8(const uint16_t* input, uint32_t rows, uint32_t columns, uint32_t block,
                         uint8_t* quantized, float* scales) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)rows; r++) {
        quantize_row(input + (size_t)r * columns, columns, block, quantized + (size_t)r * columns,
                     scales + (size_t)r * (columns / block));
    }
}

/* ------------------------------------------------------------------------------------------ */
/* expert projections                                                                          */

typedef struct record_view {
    const uint8_t* ptr;
    uint64_t bytes;
    uint32_t representation;
} record_view;

/* how an expert's matrices are held (independent_sparse_moe_gate_up_batch1_mxfp4.comp.template:166-228,250-355) */
enum { FORM_COMPACT = 0, FORM_EXPANDED = 1, FORM_NATIVE_FP8 = 2 };

/* address_record_is_resident + dynamic_parameter_record_is_valid
 * (independent_sparse_moe_gate_up_batch1_mxfp4.comp.template:120-165) */
static int resolve_parameter(const uint32_t* addresses, uint32_t address_words,
                             const uint32_t* slots, uint32_t slot_words, uint32_t params,
                             uint32_t expert, uint32_t parameter, uint64_t required,
                             record_view* out) {
    uint64_t index = (uint64_t)expert * params + parameter;
    if (index >= slot_words) return 0;
    uint32_t slot = slots[index];
    if (slot == UNBOUND_SLOT || slot >= address_words / RECORD_WORDS) return 0;
    const uint32_t* rec = addresses + (size_t)slot * RECORD_WORDS;
    uint64_t address = (uint64_t)rec[0] | ((uint64_t)rec[1] << 32);
    uint64_t bytes = (uint64_t)rec[2] | ((uint64_t)rec[3] << 32);
    uint32_t generation_nonzero = rec[4] | rec[5];
    if (address == 0u || (address & 3u) != 0u || bytes < required || generation_nonzero == 0u ||
        rec[6] != 1u)
        return 0;
    out->ptr = (const uint8_t*)(uintptr_t)address;
    out->bytes = bytes;
    out->representation = rec[7];
    return 1;
}

/* representation word of a parameter's record, 0 when the slot names no record (dynamic_parameter_representation, :150-157) */
static uint32_t parameter_representation(const uint32_t* addresses, uint32_t address_words, const uint32_t* slots,
                                         uint32_t slot_words, uint32_t params, uint32_t expert, uint32_t parameter) {
    uint64_t index = (uint64_t)expert * params + parameter;
    if (index >= slot_words) return 0u;
    uint32_t slot = slots[index];
    if (slot == UNBOUND_SLOT || slot >= address_words / RECORD_WORDS) return 0u;
    return addresses[(size_t)slot * RECORD_WORDS + 7u];
}

/* The form of an expert's matrices and the bytes its weight and scale records must hold (:184-228).
 * Returns 0 when the records' representation words rule the expert out. */
static int expert_form(const oracle_expert* p, const uint32_t* addresses, uint32_t address_words, const uint32_t* slots,
                       uint32_t slot_words, uint32_t params, uint32_t expert, uint32_t rows, uint32_t cols,
                       uint32_t* form, uint64_t* weight_bytes, uint64_t* scale_bytes) {
    uint32_t native_start = p->native_fp8_start ? p->native_fp8_start : p->num_experts;
    int native = expert >= native_start;
    uint32_t rep0 = parameter_representation(addresses, address_words, slots, slot_words, params, expert, 0u);
    uint32_t rep1 = params == 4u ? parameter_representation(addresses, address_words, slots, slot_words, params, expert, 2u) : rep0;
    if (native) {
        if (rep0 != 0u || rep1 != 0u) return 0;
        *form = FORM_NATIVE_FP8;
    } else {
        if (rep0 > 1u || rep1 > 1u || rep0 != rep1) return 0;
        *form = rep0 == 1u ? FORM_EXPANDED : FORM_COMPACT;
    }
    *weight_bytes = *form == FORM_COMPACT ? (uint64_t)rows * (cols / 2u) : (uint64_t)rows * cols;
    *scale_bytes = *form == FORM_NATIVE_FP8 ? (uint64_t)((rows + 127u) / 128u) * ((cols + 127u) / 128u)
                                            : (uint64_t)rows * (cols / 32u);
    return 1;
}

/* Byte -> the two E2M1 values it packs (low nibble first), built once. */
static float g_pair_lut[256][2];
static float g_e4m3_lut[256];
static int g_lut_ready = 0;

static void build_luts(void) {
    if (g_lut_ready) return;
#pragma omp critical(oracle_luts)
    {
        if (!g_lut_ready) {
            for (uint32_t b = 0; b < 256u; b++) {
                g_pair_lut[b][0] = nvmoe_e2m1_to_f32(b & 0xfu);
                g_pair_lut[b][1] = nvmoe_e2m1_to_f32(b >> 4);
                /* the shader multiplies E4M3 codes: decode the weight through its E4M3 byte */
                if (nvmoe_e4m3_to_f32(nvmoe_e2m1_to_e4m3_bits(b & 0xfu)) != g_pair_lut[b][0]) abort();
                g_e4m3_lut[b] = nvmoe_e4m3_to_f32(b);
            }
            g_lut_ready = 1;
        }
    }
}

/* One row dot product in the chosen tier.
 *  af:     activations as f32 — decoded E4M3 codes without their scale (tiers 0 and 1) or the
 *          bf16 activations themselves (tier 2, where `scales` is null)
 *  scales: one f32 activation scale per `block` columns
 * Weight values are exact in every tier (E2M1 code times a power of two). */
static float row_dot(const uint8_t* wrow, const uint8_t* srow, uint32_t columns, uint32_t block,
                     const float* af, const float* scales, uint32_t tier) {
    if (tier == 0u) {
        /* the shader's order (:730-767): a 64-wide subgroup strides over 4-column words, each
         * word is fma(dot4, act_scale * weight_scale, acc); lanes are then summed (pinned butterfly). */
        float lanes[64];
        uint32_t words = columns / 4u;
        for (uint32_t lane = 0; lane < 64u; lane++) {
            float acc = 0.0f;
            for (uint32_t word = lane; word < words; word += 64u) {
                uint32_t column = word * 4u;
                const float* w0 = g_pair_lut[wrow[column / 2u]];
                const float* w1 = g_pair_lut[wrow[column / 2u + 1u]];
                double dot = (double)af[column] * w0[0] + (double)af[column + 1u] * w0[1] +
                             (double)af[column + 2u] * w1[0] + (double)af[column + 3u] * w1[1];
                float scale = scales[column / block] * nvmoe_e8m0_to_f32(srow[column / 32u]);
                acc = fmaf((float)dot, scale, acc);
            }
            lanes[lane] = acc;
        }
        return butterfly_sum64(lanes);
    }
    double total = 0.0;
    for (uint32_t b32 = 0; b32 < columns / 32u; b32++) {
        double dot = 0.0;
        const uint8_t* wb = wrow + b32 * 16u;
        const float* ab = af + b32 * 32u;
        for (uint32_t j = 0; j < 16u; j++) {
            const float* w = g_pair_lut[wb[j]];
            dot += (double)ab[2u * j] * w[0] + (double)ab[2u * j + 1u] * w[1];
        }
        double sa = scales ? (double)scales[(b32 * 32u) / block] : 1.0;
        total += dot * sa * (double)nvmoe_e8m0_to_f32(srow[b32]);
    }
    return (float)total;
}

/* A row of a matrix in any of the three forms: for the two one-byte-per-element forms the weight value
 * is its E4M3 byte decoded (:250-262) and the scale of a 32-column group its E8M0 byte of the packaged
 * scale row, or, for native FP8, the exponent byte of the 128 x 128 block the group lies in (:299-355:
 * byte << 23, where a zero byte gives 0). */
static float matrix_row_dot(const record_view* w, const record_view* s, uint32_t form, uint32_t row, uint32_t columns,
                            uint32_t block, const float* af, const float* scales, uint32_t tier) {
    if (form == FORM_COMPACT)
        return row_dot(w->ptr + (size_t)row * (columns / 2u), s->ptr + (size_t)row * (columns / 32u), columns, block, af, scales, tier);
    const uint8_t* wrow = w->ptr + (size_t)row * columns;
    uint32_t native_columns = (columns + 127u) / 128u;
    if (tier == 0u) {
        float lanes[64];
        uint32_t words = columns / 4u;
        for (uint32_t lane = 0; lane < 64u; lane++) {
            float acc = 0.0f;
            for (uint32_t word = lane; word < words; word += 64u) {
                uint32_t column = word * 4u;
                double dot = 0.0;
                for (uint32_t j = 0; j < 4u; j++) dot += (double)af[column + j] * g_e4m3_lut[wrow[column + j]];
                float ws = form == FORM_NATIVE_FP8
                               ? nvmoe_bits_f32((uint32_t)s->ptr[(size_t)(row / 128u) * native_columns + column / 128u] << 23)
                               : nvmoe_e8m0_to_f32(s->ptr[(size_t)row * (columns / 32u) + column / 32u]);
                acc = fmaf((float)dot, scales[column / block] * ws, acc);
            }
            lanes[lane] = acc;
        }
        return butterfly_sum64(lanes);
    }
    double total = 0.0;
    for (uint32_t b32 = 0; b32 < columns / 32u; b32++) {
        double dot = 0.0;
        for (uint32_t j = 0; j < 32u; j++) dot += (double)af[b32 * 32u + j] * g_e4m3_lut[wrow[b32 * 32u + j]];
        double sa = scales ? (double)scales[(b32 * 32u) / block] : 1.0;
        double ws = form == FORM_NATIVE_FP8
                        ? (double)nvmoe_bits_f32((uint32_t)s->ptr[(size_t)(row / 128u) * native_columns + b32 / 4u] << 23)
                        : (double)nvmoe_e8m0_to_f32(s->ptr[(size_t)row * (columns / 32u) + b32]);
        total += dot * sa * ws;
    }
    return (float)total;
}

/* Decode of one compact slot exactly as both expert shaders do (:643-669). Returns 0 to skip. */
static int decode_slot(const oracle_expert* p, const uint32_t* intermediates,
                       const uint32_t* routes, const uint32_t* control, uint32_t linear_route,
                       int route_native, uint32_t compact_batch_y, uint32_t* batch_index,
                       uint32_t* route, uint32_t* packed_route) {
    uint32_t K = p->experts_per_token;
    uint32_t data_words = K * (p->intermediate_size / 2u);
    uint32_t frame_words = data_words + K;
    uint32_t compact_batch = route_native ? linear_route / K : compact_batch_y;
    uint32_t compact_route = route_native ? linear_route % K : linear_route;
    if ((route_native && linear_route >= control[3]) || (!route_native && compact_batch >= control[0]) ||
        (!route_native && compact_route >= K))
        return 0;
    uint32_t route_index = intermediates[(size_t)compact_batch * frame_words + data_words + compact_route];
    uint32_t capacity = control[0] * K;
    if (route_index >= capacity) return 0;
    *batch_index = route_index / K;
    *route = route_index % K;
    *packed_route = routes[(size_t)(*batch_index) * K + *route];
    return 1;
}

static void gate_up_impl(const oracle_expert* p, const uint16_t* hidden, const uint8_t* q_hidden,
                         const float* hidden_scales, const uint32_t* routes,
                         uint32_t* intermediates, const uint32_t* addresses,
                         uint32_t address_words, const uint32_t* slots, uint32_t slot_words,
                         const uint32_t* control) {
    uint32_t H = p->hidden_size, I = p->intermediate_size, K = p->experts_per_token;
    uint32_t data_words = K * (I / 2u);
    uint32_t frame_words = data_words + K;
    uint32_t block = p->act_block;
    int route_native = control[2] != 0u;
    uint32_t T = control[0];
    int64_t slot_total = route_native ? (int64_t)control[3] : (int64_t)T * K;
    build_luts();
    /* The compact list lives in the same frames the results are written to; results never touch
     * the schedule words, so snapshotting is unnecessary. */
#pragma omp parallel
    {
        uint8_t* q = (uint8_t*)malloc(H);
        float* scales = (float*)malloc(sizeof(float) * (H / block));
        float* af = (float*)malloc(sizeof(float) * H);
#pragma omp for schedule(dynamic, 1)
        for (int64_t s = 0; s < slot_total; s++) {
            uint32_t linear_route = route_native ? (uint32_t)s : (uint32_t)(s % K);
            uint32_t batch_y = route_native ? 0u : (uint32_t)(s / K);
            uint32_t batch_index, route, packed;
            if (!decode_slot(p, intermediates, routes, control, linear_route, route_native, batch_y,
                             &batch_index, &route, &packed))
                continue;
            uint32_t expert = packed & 0xffffu;
            if (expert >= p->num_experts) continue;
            record_view w1, s1, w3, s3;
            uint64_t weight_bytes, scale_bytes;
            uint32_t form;
            if (!expert_form(p, addresses, address_words, slots, slot_words, 4u, expert, I, H, &form, &weight_bytes, &scale_bytes))
                continue;
            if (!resolve_parameter(addresses, address_words, slots, slot_words, 4u, expert, 0u, weight_bytes, &w1) ||
                !resolve_parameter(addresses, address_words, slots, slot_words, 4u, expert, 1u, scale_bytes, &s1) ||
                !resolve_parameter(addresses, address_words, slots, slot_words, 4u, expert, 2u, weight_bytes, &w3) ||
                !resolve_parameter(addresses, address_words, slots, slot_words, 4u, expert, 3u, scale_bytes, &s3))
                continue;
            const uint8_t* qa;
            const float* sa;
            if (q_hidden) {
                qa = q_hidden + (size_t)batch_index * H;
                sa = hidden_scales + (size_t)batch_index * (H / block);
            } else {
                quantize_row(hidden + (size_t)batch_index * H, H, block, q, scales);
                qa = q;
                sa = scales;
            }
            if (p->tier == 2u && !q_hidden) {
                for (uint32_t c = 0; c < H; c++) af[c] = nvmoe_bf16_to_f32(hidden[(size_t)batch_index * H + c]);
                sa = NULL;
            } else {
                for (uint32_t c = 0; c < H; c++) af[c] = g_e4m3_lut[qa[c]];
            }
            uint16_t* out = (uint16_t*)(intermediates + (size_t)batch_index * frame_words + (size_t)route * (I / 2u));
            for (uint32_t row = 0; row < I; row++) {
                uint32_t tier = sa ? (p->tier == 2u ? 1u : p->tier) : 2u;
                float gate = matrix_row_dot(&w1, &s1, form, row, H, block, af, sa, tier);
                float up = matrix_row_dot(&w3, &s3, form, row, H, block, af, sa, tier);
                out[row] = (uint16_t)nvmoe_f32_to_bf16(
                    nvmoe_swiglu(gate, up, p->swiglu_limit, p->swiglu_alpha, p->swiglu_up_offset));
            }
        }
        free(q);
        free(scales);
        free(af);
    }
}

void oracle_gate_up(const oracle_expert* p, const uint16_t* hidden, const uint32_t* routes,
                    uint32_t* intermediates, const uint32_t* addresses, uint32_t address_words,
                    const uint32_t* slots, uint32_t slot_words, const uint32_t* control) {
    gate_up_impl(p, hidden, NULL, NULL, routes, intermediates, addresses, address_words, slots,
                 slot_words, control);
}

void oracle_gate_up_prequant(const oracle_expert* p, const uint8_t* q_hidden,
                             const float* hidden_scales, const uint32_t* routes,
                             uint32_t* intermediates, const uint32_t* addresses,
                             uint32_t address_words, const uint32_t* slots, uint32_t slot_words,
                             const uint32_t* control) {
    gate_up_impl(p, NULL, q_hidden, hidden_scales, routes, intermediates, addresses, address_words,
                 slots, slot_words, control);
}

void oracle_down(const oracle_expert* p, const uint32_t* intermediates, const uint32_t* routes,
                 uint16_t* outputs, const uint32_t* addresses, uint32_t address_words,
                 const uint32_t* slots, uint32_t slot_words, const uint32_t* control) {
    uint32_t H = p->hidden_size, I = p->intermediate_size, K = p->experts_per_token;
    uint32_t data_words = K * (I / 2u);
    uint32_t frame_words = data_words + K;
    uint32_t block = p->act_block;
    int route_native = control[2] != 0u;
    uint32_t T = control[0];
    int64_t slot_total = route_native ? (int64_t)control[3] : (int64_t)T * K;
    build_luts();
#pragma omp parallel
    {
        uint8_t* q = (uint8_t*)malloc(I);
        float* scales = (float*)malloc(sizeof(float) * (I / block));
        float* af = (float*)malloc(sizeof(float) * I);
#pragma omp for schedule(dynamic, 1)
        for (int64_t s = 0; s < slot_total; s++) {
            uint32_t linear_route = route_native ? (uint32_t)s : (uint32_t)(s % K);
            uint32_t batch_y = route_native ? 0u : (uint32_t)(s / K);
            uint32_t batch_index, route, packed;
            if (!decode_slot(p, intermediates, routes, control, linear_route, route_native, batch_y,
                             &batch_index, &route, &packed))
                continue;
            uint32_t expert = packed & 0xffffu;
            if (expert >= p->num_experts) continue;
            record_view w2, s2;
            uint64_t weight_bytes, scale_bytes;
            uint32_t form;
            if (!expert_form(p, addresses, address_words, slots, slot_words, 2u, expert, H, I, &form, &weight_bytes, &scale_bytes))
                continue;
            if (!resolve_parameter(addresses, address_words, slots, slot_words, 2u, expert, 0u, weight_bytes, &w2) ||
                !resolve_parameter(addresses, address_words, slots, slot_words, 2u, expert, 1u, scale_bytes, &s2))
                continue;
            float route_weight = nvmoe_bf16_to_f32(packed >> 16);
            const uint16_t* in = (const uint16_t*)(intermediates + (size_t)batch_index * frame_words + (size_t)route * (I / 2u));
            const float* sa = scales;
            if (p->tier == 2u) {
                for (uint32_t c = 0; c < I; c++) af[c] = nvmoe_bf16_to_f32(in[c]);
                sa = NULL;
            } else {
                quantize_row(in, I, block, q, scales);
                for (uint32_t c = 0; c < I; c++) af[c] = g_e4m3_lut[q[c]];
            }
            uint16_t* out = outputs + ((size_t)batch_index * K + route) * H;
            for (uint32_t row = 0; row < H; row++) {
                float value = matrix_row_dot(&w2, &s2, form, row, I, block, af, sa, p->tier);
                out[row] = (uint16_t)nvmoe_f32_to_bf16(value * route_weight);
            }
        }
        free(q);
        free(scales);
        free(af);
    }
}

void oracle_reduce(const uint16_t* expert_outputs, uint16_t* output, uint32_t tokens, uint32_t K,
                   uint32_t hidden, float routed_scale) {
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < (int64_t)tokens; t++) {
        for (uint32_t h = 0; h < hidden; h++) {
            float acc = 0.0f;
            for (uint32_t r = 0; r < K; r++)
                acc = nvmoe_round_bf16(acc + nvmoe_bf16_to_f32(expert_outputs[((size_t)t * K + r) * hidden + h]));
            output[(size_t)t * hidden + h] = (uint16_t)nvmoe_f32_to_bf16(acc * routed_scale);
        }
    }
}

void oracle_sum_f32_scale_packed_bf16(const float* partials, const uint32_t* scales,
                                      uint32_t* out_words, uint32_t element_count,
                                      uint32_t participant_count, uint32_t lane_count,
                                      uint32_t elements_per_scale, uint32_t scale_bit_offset) {
    uint32_t scales_per_lane = element_count / elements_per_scale;
    for (uint32_t lane = 0; lane < lane_count; lane++) {
        for (uint32_t word = 0; word < element_count / 2u; word++) {
            uint32_t element = word * 2u;
            float lo = 0.0f, hi = 0.0f;
            for (uint32_t part = 0; part < participant_count; part++) {
                size_t base = ((size_t)part * lane_count + lane) * element_count;
                lo += partials[base + element];
                hi += partials[base + element + 1u];
            }
            float slo = nvmoe_bf16_to_f32(scales[lane * scales_per_lane + element / elements_per_scale] >> scale_bit_offset);
            float shi = nvmoe_bf16_to_f32(scales[lane * scales_per_lane + (element + 1u) / elements_per_scale] >> scale_bit_offset);
            out_words[(size_t)lane * (element_count / 2u) + word] =
                (nvmoe_f32_to_bf16(hi * shi) << 16) | nvmoe_f32_to_bf16(lo * slo);
        }
    }
}

/* ------------------------------------------------------------------------------------------ */
/* token-id table routing: resource_preselect_table_batch1.comp.template:35-97 and             */
/* moe_router_preselected_batch1_bf16.comp.template:56-91                                      */

/* Looks every token's routed resources up in a [vocab][k] table of 32- or 64-bit integers
 * (word_stride 1 or 2), appends the always-selected ids, sorts ascending (:74-82) and counts the
 * selection telemetry (:83-96).  A token id beyond the table, an index beyond the routed
 * resources, a non-zero high word or a repeated index makes the whole token invalid: its
 * selections become 0xffffffff (:67-73) and nothing is counted.  Returns the invalid tokens. */
int oracle_resource_preselect_table(const uint32_t* token_ids, const uint32_t* table_words,
                                    uint32_t word_stride, uint32_t vocab, uint32_t routed,
                                    uint32_t k, uint32_t always, uint32_t tokens,
                                    uint32_t* selections, uint32_t* telemetry) {
    uint32_t total_k = k + always, total_resources = routed + always;
    int invalid_tokens = 0;
    for (uint32_t t = 0; t < tokens; t++) {
        uint32_t ids[64];
        uint32_t token_id = token_ids[t];
        int invalid = token_id >= vocab;
        for (uint32_t lane = 0; lane < k && !invalid; lane++) {
            size_t element = (size_t)token_id * k + lane;
            uint32_t index = table_words[element * word_stride];
            uint32_t high = word_stride == 2u ? table_words[element * word_stride + 1u] : 0u;
            if (index >= routed || high != 0u) invalid = 1;
            for (uint32_t previous = 0; previous < lane; previous++)
                if (index == table_words[((size_t)token_id * k + previous) * word_stride]) invalid = 1;
            ids[lane] = index < routed ? index : routed - 1u;
        }
        uint32_t* out = selections + (size_t)t * total_k;
        if (invalid) {
            for (uint32_t r = 0; r < total_k; r++) out[r] = 0xffffffffu;
            invalid_tokens++;
            continue;
        }
        for (uint32_t a = 0; a < always; a++) ids[k + a] = routed + a;
        for (uint32_t r = 1; r < total_k; r++) {
            uint32_t index = ids[r], ins = r;
            while (ins > 0u && ids[ins - 1u] > index) {
                ids[ins] = ids[ins - 1u];
                ins--;
            }
            ids[ins] = index;
        }
        for (uint32_t r = 0; r < total_k; r++) {
            out[r] = ids[r];
            if (telemetry) telemetry[ids[r]]++;
        }
        if (telemetry)
            for (uint32_t l = 0; l < total_k; l++)
                for (uint32_t rr = l + 1u; rr < total_k; rr++) {
                    uint32_t left = ids[l], right = ids[rr];
                    uint32_t preceding = left * (2u * total_resources - left - 1u) / 2u;
                    telemetry[total_resources + preceding + right - left - 1u]++;
                }
    }
    return invalid_tokens;
}

/* Route words of preselected resources: weight = activation(logit) of each routed selection
 * (sigmoid, or sqrt(softplus)), normalised over the routed selections in their stored order and
 * scaled, always-selected resources at their constant weight (:72-90).  A selection whose index is
 * not a routed resource where one is expected (the 0xffffffff of an invalid token) gives the route
 * word 0x0000ffff (weight 0, an id no expert kernel accepts) instead of the shader's read past
 * the logits row. */
void oracle_route_preselected(const oracle_router* p, const uint32_t* logit_words,
                              const uint32_t* selections, uint32_t tokens, uint32_t* routes) {
    uint32_t E = p->routed_experts, k = p->routed_k, total_k = k + p->always_count;
    uint32_t words = (E + 1u) / 2u;
    for (uint32_t t = 0; t < tokens; t++) {
        const uint32_t* sel = selections + (size_t)t * total_k;
        uint32_t* out = routes + (size_t)t * total_k;
        float values[64];
        int bad = 0;
        for (uint32_t r = 0; r < k; r++)
            if ((sel[r] & 0xffffu) >= E) bad = 1;
        if (bad) {
            for (uint32_t r = 0; r < total_k; r++) out[r] = 0x0000ffffu;
            continue;
        }
        for (uint32_t r = 0; r < k; r++) {
            float v = unpack_bf16(logit_words + (size_t)t * words, sel[r] & 0xffffu);
            values[r] = p->activation == 0u ? nvmoe_sigmoidf(v) : sqrtf(nvmoe_softplusf(v));
        }
        float den = 0.0f;
        if (p->normalize_selected)
            for (uint32_t r = 0; r < k; r++) den = den + values[r];
        for (uint32_t r = 0; r < total_k; r++) {
            float w = p->always_weight;
            if (r < k) w = p->normalize_selected ? values[r] / den * p->routed_scale : values[r] * p->routed_scale;
            out[r] = (nvmoe_f32_to_bf16(w) << 16) | (sel[r] & 0xffffu);
        }
    }
}

/* ------------------------------------------------------------------------------------------ */
/* the steps either side of the MoE node chain                                                 */

/* rms_norm_batch_bf16.comp.template:55-108: 64 lanes stride over the row with fma(x, x, sum)
 * (:63-75), the lane sums are added (subgroupAdd then a sum over subgroups, :76-90: taken as the
 * pinned butterfly over 64 lanes), inv_rms = 1 / sqrt(total / H + eps) out of an IEEE division and
 * square root, and y = bf16(x * inv_rms * (w + offset)) (:92-107). */
void oracle_rms_norm(const uint16_t* input, const uint16_t* weight, uint16_t* output, uint32_t rows,
                     uint32_t hidden, float eps, float weight_offset) {
#pragma omp parallel for schedule(static)
    for (int64_t rr = 0; rr < (int64_t)rows; rr++) {
        const uint16_t* x = input + (size_t)rr * hidden;
        float lanes[64];
        for (uint32_t lane = 0; lane < 64u; lane++) {
            float sum = 0.0f;
            for (uint32_t i = lane; i < hidden; i += 64u) {
                float v = nvmoe_bf16_to_f32(x[i]);
                sum = fmaf(v, v, sum);
            }
            lanes[lane] = sum;
        }
        float total = butterfly_sum64(lanes);
        float inv_rms = 1.0f / sqrtf(total / (float)hidden + eps);
        for (uint32_t i = 0; i < hidden; i++) {
            float w = nvmoe_bf16_to_f32(weight[i]) + weight_offset;
            output[(size_t)rr * hidden + i] = (uint16_t)nvmoe_f32_to_bf16(nvmoe_bf16_to_f32(x[i]) * inv_rms * w);
        }
    }
}

/* limit > 0: bounded_silu_multiply_batch_bf16.comp.template:26-30 (gate = min(gate, L), up clamped to
 * +-L, one rounding at the end); limit == 0: silu_multiply_batch_bf16.comp.template:24-27,45-51,
 * where the activated gate is rounded to bf16 before it meets the up value. */
void oracle_silu_multiply(const uint16_t* gate, const uint16_t* up, uint16_t* out, uint64_t count, float limit) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)count; i++) {
        float g = nvmoe_bf16_to_f32(gate[i]), u = nvmoe_bf16_to_f32(up[i]);
        float value;
        if (limit > 0.0f) {
            g = fminf(g, limit);
            u = fminf(fmaxf(u, -limit), limit);
            value = g / (1.0f + nvmoe_expf(-g)) * u;
        } else {
            value = nvmoe_round_bf16(g / (1.0f + nvmoe_expf(-g))) * u;
        }
        out[i] = (uint16_t)nvmoe_f32_to_bf16(value);
    }
}

/* add_batch_bf16.comp.template:36-50 (op residual_add) */
void oracle_add_bf16(const uint16_t* a, const uint16_t* b, uint16_t* out, uint64_t count) {
    for (uint64_t i = 0; i < count; i++)
        out[i] = (uint16_t)nvmoe_f32_to_bf16(nvmoe_bf16_to_f32(a[i]) + nvmoe_bf16_to_f32(b[i]));
}
