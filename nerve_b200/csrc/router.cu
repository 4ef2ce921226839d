// Router projection and the three route-native router forms.
//
//   router_linear_kernel   runtime-rs/shaders/linear_bf16.comp.template:39-95 and
//                          linear_bias_bf16.comp.template:31-84
//   router_kernel          runtime-rs/shaders/moe_router_score_topk_batch1_bf16.comp.template:109-220
//                          runtime-rs/shaders/moe_topk_bf16.comp.template:44-145
//                          runtime-rs/shaders/moe_topk_routed_batch1_bf16.comp.template:71-182
//
// One warp routes one token.  Selection is k rounds of a (score, index) arg-max whose comparator
// is the shaders' own: higher score wins, equal scores go to the lower expert index, a NaN score
// is never chosen.  Route weights use the pinned transcendentals of nvmoe_math.h and the summation
// orders the shaders fix (selection order for the selected-only denominators, index order for
// the softmax-over-all of the routed form); the one order the shaders leave to the hardware, the
// subgroup sum of the score_topk softmax, is pinned to 64 lane-strided partials folded by an xor
// butterfly (32,16,8,4,2,1) — the same definition the CPU checker uses.
#include "common.cuh"

namespace nvmoe {
namespace {

constexpr float kNegInf = -__builtin_huge_valf();

__device__ __forceinline__ float unpack_logit(const uint32_t* row, uint32_t e) {
    uint32_t packed = row[e >> 1];
    return nvmoe_bf16_to_f32((e & 1u) ? (packed >> 16) : packed);
}

__device__ __forceinline__ bool better(float s, uint32_t e, float best, uint32_t best_e) {
    return s > best || (s == best && e < best_e);
}

// warp-wide arg-max of (score, expert) pairs under `better`; all lanes return the winner
__device__ __forceinline__ void warp_argmax(float& s, uint32_t& e) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float os = __shfl_xor_sync(0xffffffffu, s, o);
        uint32_t oe = __shfl_xor_sync(0xffffffffu, e, o);
        // an empty candidate carries e == kUnboundSlot and can only win over another empty one
        bool take = (oe != kUnboundSlot) && (e == kUnboundSlot || better(os, oe, s, e));
        if (take) {
            s = os;
            e = oe;
        }
    }
}

struct WarpSmem {
    float* values;      // activated value (score_topk) or soft-capped logit (routed) or raw logit
    float* score;       // selection score
    uint32_t* flags;    // bit0 selected, bit1 allowed
    uint32_t* top;      // [kMaxTopK]
    float* top_w;       // [kMaxTopK]
    float* group_score; // [32]
};

__device__ __forceinline__ float read_bias(const void* bias, uint32_t dtype, uint32_t e) {
    if (dtype == NVMOE_BIAS_F32) return reinterpret_cast<const float*>(bias)[e];
    if (dtype == NVMOE_BIAS_BF16) return nvmoe_bf16_to_f32(reinterpret_cast<const uint16_t*>(bias)[e]);
    return 0.0f;
}

__global__ void __launch_bounds__(128) router_kernel(RouterLaunch p, uint32_t warps_per_block) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    grid_dependency_sync();
    const uint32_t E = p.g.routed_experts;
    const uint32_t k = p.g.routed_k;
    const uint32_t kind = p.g.router_kind;
    const uint32_t always = kind == NVMOE_ROUTER_SCORE_TOPK ? p.g.always_count : 0u;
    const uint32_t total_k = k + always;
    const uint32_t total_resources = E + always;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t token = blockIdx.x * warps_per_block + warp;
    if (warp >= warps_per_block || token >= p.tokens) return;

    const size_t per_warp = (size_t)E * 12u + kMaxTopK * 8u + 32u * 4u;
    unsigned char* base = smem_raw + per_warp * warp;
    WarpSmem s;
    s.values = reinterpret_cast<float*>(base);
    s.score = s.values + E;
    s.flags = reinterpret_cast<uint32_t*>(s.score + E);
    s.top = s.flags + E;
    s.top_w = reinterpret_cast<float*>(s.top + kMaxTopK);
    s.group_score = s.top_w + kMaxTopK;

    const uint32_t* row = p.logits + (size_t)token * ((E + 1u) / 2u);

    // ---- activation and selection score ---------------------------------------------------
    if (kind == NVMOE_ROUTER_SCORE_TOPK) {
        float smax = kNegInf, sden = 0.0f;
        if (p.g.activation == NVMOE_ACT_SOFTMAX) {
            for (uint32_t e = lane; e < E; e += 32u) smax = fmaxf(smax, unpack_logit(row, e));
            smax = warp_max(smax);
            float lo = 0.0f, hi = 0.0f;  // virtual lanes `lane` and `lane + 32` of a 64-wide group
            for (uint32_t e = lane; e < E; e += 64u) lo = __fadd_rn(lo, nvmoe_expf(__fsub_rn(unpack_logit(row, e), smax)));
            for (uint32_t e = lane + 32u; e < E; e += 64u) hi = __fadd_rn(hi, nvmoe_expf(__fsub_rn(unpack_logit(row, e), smax)));
            sden = warp_butterfly_sum(__fadd_rn(lo, hi));
        }
        for (uint32_t e = lane; e < E; e += 32u) {
            float v = unpack_logit(row, e);
            float a;
            if (p.g.activation == NVMOE_ACT_SIGMOID) {
                a = nvmoe_sigmoidf(v);
            } else if (p.g.activation == NVMOE_ACT_SOFTMAX) {
                a = __fdiv_rn(nvmoe_expf(__fsub_rn(v, smax)), sden);
            } else {
                a = __fsqrt_rn(nvmoe_softplusf(v));
            }
            s.values[e] = a;
            s.score[e] = __fadd_rn(a, read_bias(p.bias, p.g.bias_dtype, e));
        }
    } else if (kind == NVMOE_ROUTER_TOPK_SOFTMAX) {
        for (uint32_t e = lane; e < E; e += 32u) {
            float v = unpack_logit(row, e);
            s.values[e] = v;
            s.score[e] = v;
        }
    } else {
        const bool sigmoid = p.g.activation == NVMOE_ACT_SIGMOID;
        for (uint32_t e = lane; e < E; e += 32u) {
            float v = unpack_logit(row, e);
            if (p.g.logit_softcap > 0.0f)
                v = __fmul_rn(nvmoe_tanhf(__fdiv_rn(v, p.g.logit_softcap)), p.g.logit_softcap);
            s.values[e] = v;
            s.score[e] = __fadd_rn(sigmoid ? nvmoe_sigmoidf(v) : v, read_bias(p.bias, p.g.bias_dtype, e));
        }
    }
    __syncwarp();

    // ---- group-limited mask (extension; n_group == 0 keeps every expert) -------------------
    if (p.g.n_group == 0u) {
        for (uint32_t e = lane; e < E; e += 32u) s.flags[e] = 2u;
    } else {
        const uint32_t per = E / p.g.n_group;
        if (lane < p.g.n_group) {
            float first = kNegInf, second = kNegInf;
            for (uint32_t j = 0; j < per; j++) {
                float v = s.score[lane * per + j];
                if (v > first) {
                    second = first;
                    first = v;
                } else if (v > second) {
                    second = v;
                }
            }
            s.group_score[lane] = per >= 2u ? __fadd_rn(first, second) : first;
        }
        __syncwarp();
        uint32_t kept = 0u;  // computed redundantly by every lane: n_group <= 32
        for (uint32_t round = 0; round < p.g.topk_group; round++) {
            float best = kNegInf;
            uint32_t best_g = kUnboundSlot;
            for (uint32_t g = 0; g < p.g.n_group; g++) {
                if (kept & (1u << g)) continue;
                float v = s.group_score[g];
                if (better(v, g, best, best_g)) {
                    best = v;
                    best_g = g;
                }
            }
            if (best_g != kUnboundSlot) kept |= 1u << best_g;
        }
        for (uint32_t e = lane; e < E; e += 32u) s.flags[e] = (kept >> (e / per)) & 1u ? 2u : 0u;
    }
    __syncwarp();

    // ---- k rounds of arg-max -------------------------------------------------------------
    bool missing = false;
    for (uint32_t r = 0; r < k; r++) {
        float best = kNegInf;
        uint32_t best_e = kUnboundSlot;
        for (uint32_t e = lane; e < E; e += 32u) {
            if (s.flags[e] != 2u) continue;  // not allowed, or already selected (bit0)
            float v = s.score[e];
            if (better(v, e, best, best_e)) {
                best = v;
                best_e = e;
            }
        }
        warp_argmax(best, best_e);
        if (best_e == kUnboundSlot) {
            missing = true;
            break;
        }
        if (lane == 0) {
            s.top[r] = best_e;
            s.flags[best_e] = 3u;
        }
        __syncwarp();
    }

    if (lane != 0) return;
    uint32_t* out = p.routes + (size_t)token * total_k;
    if (missing) {
        // no selectable score (NaN logits): fail closed instead of indexing out of bounds
        for (uint32_t r = 0; r < total_k; r++) out[r] = 0u;
        raise_status(p.status, NVMOE_STATUS_ROUTE_NONFINITE);
        return;
    }

    // ---- weights, in the summation orders the shaders fix ----------------------------------
    if (kind == NVMOE_ROUTER_SCORE_TOPK) {
        float den = 0.0f;
        if (p.g.normalize_selected)
            for (uint32_t r = 0; r < k; r++) den = __fadd_rn(den, s.values[s.top[r]]);
        for (uint32_t r = 0; r < k; r++) {
            float w = s.values[s.top[r]];
            w = p.g.normalize_selected ? __fmul_rn(__fdiv_rn(w, den), p.g.routed_scale) : __fmul_rn(w, p.g.routed_scale);
            s.top_w[r] = w;
        }
        for (uint32_t o = 0; o < always; o++) {
            s.top[k + o] = E + o;
            s.top_w[k + o] = p.g.always_weight;
        }
    } else if (kind == NVMOE_ROUTER_TOPK_SOFTMAX) {
        float maximum = s.values[s.top[0]];
        float den = 0.0f;
        for (uint32_t r = 0; r < k; r++) den = __fadd_rn(den, nvmoe_expf(__fsub_rn(s.values[s.top[r]], maximum)));
        for (uint32_t r = 0; r < k; r++)
            s.top_w[r] = __fdiv_rn(nvmoe_expf(__fsub_rn(s.values[s.top[r]], maximum)), den);
    } else {
        const bool sigmoid = p.g.activation == NVMOE_ACT_SIGMOID;
        float maximum = s.values[s.top[0]];
        float den = 0.0f;
        if (p.g.normalize_selected) {
            for (uint32_t r = 0; r < k; r++) {
                float v = s.values[s.top[r]];
                den = __fadd_rn(den, sigmoid ? nvmoe_sigmoidf(v) : nvmoe_expf(__fsub_rn(v, maximum)));
            }
        } else if (!sigmoid) {
            maximum = kNegInf;
            for (uint32_t e = 0; e < E; e++) maximum = fmaxf(maximum, s.values[e]);
            for (uint32_t e = 0; e < E; e++) den = __fadd_rn(den, nvmoe_expf(__fsub_rn(s.values[e], maximum)));
        }
        for (uint32_t r = 0; r < k; r++) {
            float v = s.values[s.top[r]];
            float w = sigmoid ? nvmoe_sigmoidf(v) : nvmoe_expf(__fsub_rn(v, maximum));
            if (p.g.normalize_selected || !sigmoid) w = __fdiv_rn(w, den);
            s.top_w[r] = w;
        }
    }

    // ---- ascending expert id (insertion sort of the shaders), pack, telemetry ---------------
    for (uint32_t r = 1; r < total_k; r++) {
        uint32_t e = s.top[r];
        float w = s.top_w[r];
        uint32_t ins = r;
        while (ins > 0u && s.top[ins - 1u] > e) {
            s.top[ins] = s.top[ins - 1u];
            s.top_w[ins] = s.top_w[ins - 1u];
            ins--;
        }
        s.top[ins] = e;
        s.top_w[ins] = w;
    }
    for (uint32_t r = 0; r < total_k; r++) {
        out[r] = (nvmoe_f32_to_bf16(s.top_w[r]) << 16) | s.top[r];
        if (p.telemetry) atomicAdd(p.telemetry + s.top[r], 1u);
    }
    if (p.telemetry) {
        for (uint32_t l = 0; l < total_k; l++) {
            uint32_t left = s.top[l];
            for (uint32_t rr = l + 1u; rr < total_k; rr++) {
                uint32_t right = s.top[rr];
                if (left < right) {
                    uint32_t preceding = left * (2u * total_resources - left - 1u) / 2u;
                    atomicAdd(p.telemetry + total_resources + preceding + right - left - 1u, 1u);
                }
            }
        }
    }
}

// ---- the same router with a token's experts in registers ------------------------------------------
// For up to 32 * EPL experts and at most 32 selections a token, without group-limited masking: lane l keeps the
// experts l, l + 32, .. in registers, lane r keeps selection r once it is made, and everything the kernel above
// does through shared memory by one lane (the weights, the ascending order, packing, telemetry) is done by the
// lanes side by side. Every sum that has an order keeps it (values travel by shuffle and are added in the same
// sequence); the results are bit for bit those of router_kernel, which remains for the other cases.
template <int EPL>
__global__ void __launch_bounds__(128) router_reg_kernel(RouterLaunch p) {
    grid_dependency_sync();
    constexpr uint32_t kFull = 0xffffffffu;
    const uint32_t E = p.g.routed_experts;
    const uint32_t k = p.g.routed_k;
    const uint32_t kind = p.g.router_kind;
    const uint32_t always = kind == NVMOE_ROUTER_SCORE_TOPK ? p.g.always_count : 0u;
    const uint32_t total_k = k + always;
    const uint32_t total_resources = E + always;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t token = blockIdx.x * 4u + warp;
    if (token >= p.tokens) return;
    const uint32_t* row = p.logits + (size_t)token * ((E + 1u) / 2u);

    float val[EPL], score[EPL];
#pragma unroll
    for (int j = 0; j < EPL; j++) {
        const uint32_t e = lane + 32u * j;
        val[j] = e < E ? unpack_logit(row, e) : 0.0f;
        score[j] = 0.0f;
    }
    // ---- activation and selection score ---------------------------------------------------
    if (kind == NVMOE_ROUTER_SCORE_TOPK) {
        if (p.g.activation == NVMOE_ACT_SOFTMAX) {
            float smax = kNegInf;
#pragma unroll
            for (int j = 0; j < EPL; j++)
                if (lane + 32u * j < E) smax = fmaxf(smax, val[j]);
            smax = warp_max(smax);
            float lo = 0.0f, hi = 0.0f;  // virtual lanes `lane` and `lane + 32` of a 64-wide group
#pragma unroll
            for (int j = 0; j < EPL; j++) {
                if (lane + 32u * j < E) {
                    val[j] = nvmoe_expf(__fsub_rn(val[j], smax));
                    if (j & 1) hi = __fadd_rn(hi, val[j]); else lo = __fadd_rn(lo, val[j]);
                }
            }
            const float sden = warp_butterfly_sum(__fadd_rn(lo, hi));
#pragma unroll
            for (int j = 0; j < EPL; j++) val[j] = __fdiv_rn(val[j], sden);
        } else {
#pragma unroll
            for (int j = 0; j < EPL; j++)
                val[j] = p.g.activation == NVMOE_ACT_SIGMOID ? nvmoe_sigmoidf(val[j]) : __fsqrt_rn(nvmoe_softplusf(val[j]));
        }
#pragma unroll
        for (int j = 0; j < EPL; j++) {
            const uint32_t e = lane + 32u * j;
            score[j] = e < E ? __fadd_rn(val[j], read_bias(p.bias, p.g.bias_dtype, e)) : 0.0f;
        }
    } else if (kind == NVMOE_ROUTER_TOPK_SOFTMAX) {
#pragma unroll
        for (int j = 0; j < EPL; j++) score[j] = val[j];
    } else {
        const bool sigmoid = p.g.activation == NVMOE_ACT_SIGMOID;
#pragma unroll
        for (int j = 0; j < EPL; j++) {
            const uint32_t e = lane + 32u * j;
            float v = val[j];
            if (p.g.logit_softcap > 0.0f) v = __fmul_rn(nvmoe_tanhf(__fdiv_rn(v, p.g.logit_softcap)), p.g.logit_softcap);
            val[j] = v;
            score[j] = e < E ? __fadd_rn(sigmoid ? nvmoe_sigmoidf(v) : v, read_bias(p.bias, p.g.bias_dtype, e)) : 0.0f;
        }
    }

    // ---- k rounds of arg-max: lane r keeps selection r ---------------------------------------
    uint32_t taken = 0u, my_e = kUnboundSlot;
    float my_v = 0.0f;
    bool missing = false;
    for (uint32_t r = 0; r < k; r++) {
        float best = kNegInf, best_v = 0.0f;
        uint32_t best_e = kUnboundSlot;
#pragma unroll
        for (int j = 0; j < EPL; j++) {
            const uint32_t e = lane + 32u * j;
            if (e < E && ((taken >> j) & 1u) == 0u && better(score[j], e, best, best_e)) {
                best = score[j];
                best_e = e;
                best_v = val[j];
            }
        }
        float s = best;
        uint32_t winner = best_e;
        warp_argmax(s, winner);
        if (winner == kUnboundSlot) {
            missing = true;
            break;
        }
        // the winner is the best candidate of the lane that owns it
        const float winner_v = __shfl_sync(kFull, best_v, winner & 31u);
        if (lane == (winner & 31u)) taken |= 1u << (winner >> 5);
        if (lane == r) {
            my_e = winner;
            my_v = winner_v;
        }
    }
    uint32_t* out = p.routes + (size_t)token * total_k;
    if (missing) {
        // no selectable score (NaN logits): fail closed instead of indexing out of bounds
        if (lane == 0u) {
            for (uint32_t r = 0; r < total_k; r++) out[r] = 0u;
            raise_status(p.status, NVMOE_STATUS_ROUTE_NONFINITE);
        }
        return;
    }

    // ---- weights, in the summation orders the shaders fix ----------------------------------
    float w = 0.0f;
    if (kind == NVMOE_ROUTER_SCORE_TOPK) {
        float den = 0.0f;
        if (p.g.normalize_selected)
            for (uint32_t r = 0; r < k; r++) den = __fadd_rn(den, __shfl_sync(kFull, my_v, r));
        w = p.g.normalize_selected ? __fmul_rn(__fdiv_rn(my_v, den), p.g.routed_scale) : __fmul_rn(my_v, p.g.routed_scale);
        if (lane >= k && lane < total_k) {
            my_e = E + (lane - k);
            w = p.g.always_weight;
        }
    } else {
        const bool sigmoid = kind == NVMOE_ROUTER_TOPK_ROUTED && p.g.activation == NVMOE_ACT_SIGMOID;
        const bool divide = kind == NVMOE_ROUTER_TOPK_SOFTMAX || p.g.normalize_selected || !sigmoid;
        const float maximum = __shfl_sync(kFull, my_v, 0);
        const float t = sigmoid ? nvmoe_sigmoidf(my_v) : nvmoe_expf(__fsub_rn(my_v, maximum));
        float den = 0.0f;
        for (uint32_t r = 0; r < k; r++) den = __fadd_rn(den, __shfl_sync(kFull, t, r));
        w = divide ? __fdiv_rn(t, den) : t;
    }

    // ---- ascending expert id, pack, telemetry ----------------------------------------------------
    uint32_t rank = 0u;
    for (uint32_t q = 0; q < total_k; q++) {
        const uint32_t other = __shfl_sync(kFull, my_e, q);
        if (other < my_e) rank++;
    }
    if (lane < total_k) {
        out[rank] = (nvmoe_f32_to_bf16(w) << 16) | my_e;
        if (p.telemetry) atomicAdd(p.telemetry + my_e, 1u);
    }
    if (p.telemetry) {
        for (uint32_t q = 0; q < total_k; q++) {
            const uint32_t right = __shfl_sync(kFull, my_e, q);
            if (lane < total_k && my_e < right) {
                const uint32_t preceding = my_e * (2u * total_resources - my_e - 1u) / 2u;
                atomicAdd(p.telemetry + total_resources + preceding + right - my_e - 1u, 1u);
            }
        }
    }
}

// ---- router projection ----------------------------------------------------------------------
// The shader gives every output row 64 lanes that stride over the packed input words with two
// f32 fma per word and then sums the lanes.  Here a block of 64 threads owns a TT x ET tile of
// (token, output) pairs: thread v plays lane v of every pair in the tile, so each x and w word is
// loaded once per thread and reused across the tile, and the 64 lane sums of a pair are folded
// with the pinned butterfly (step 32 through shared memory, 16..1 by shuffles).
template <int TT, int ET>
__global__ void __launch_bounds__(64) router_linear_kernel(const uint16_t* __restrict__ x,
                                                           const uint16_t* __restrict__ w,
                                                           const uint16_t* __restrict__ bias,
                                                           uint32_t* __restrict__ logits, uint32_t tokens,
                                                           uint32_t hidden, uint32_t outputs) {
    __shared__ float fold[TT * ET][32];
    __shared__ float result[TT * ET];
    grid_dependency_sync();
    const uint32_t v = threadIdx.x;
    const uint32_t t0 = blockIdx.y * TT, e0 = blockIdx.x * ET;
    const uint32_t words = hidden / 2u;
    const uint32_t* xw = reinterpret_cast<const uint32_t*>(x);
    const uint32_t* ww = reinterpret_cast<const uint32_t*>(w);
    float acc[TT][ET];
#pragma unroll
    for (int a = 0; a < TT; a++)
#pragma unroll
        for (int b = 0; b < ET; b++) acc[a][b] = 0.0f;

    // The sum order of a lane is fixed (its words in ascending order), the load order is not: the
    // loads of kDepth steps are issued together so that their latencies overlap.
    constexpr int kDepth = TT * ET <= 16 ? 8 : 2;
    for (uint32_t cw0 = v; cw0 < words; cw0 += 64u * kDepth) {
        uint32_t xr[kDepth][TT], wr[kDepth][ET];
#pragma unroll
        for (int u = 0; u < kDepth; u++) {
            const uint32_t cw = cw0 + 64u * u;
            const bool in = cw < words;
#pragma unroll
            for (int a = 0; a < TT; a++) xr[u][a] = (in && t0 + a < tokens) ? __ldg(xw + (size_t)(t0 + a) * words + cw) : 0u;
#pragma unroll
            for (int b = 0; b < ET; b++) wr[u][b] = (in && e0 + b < outputs) ? __ldg(ww + (size_t)(e0 + b) * words + cw) : 0u;
        }
#pragma unroll
        for (int u = 0; u < kDepth; u++) {
            if (cw0 + 64u * u >= words) break;  // a step past the end must not even add zeros (-0 + 0 = +0)
#pragma unroll
            for (int a = 0; a < TT; a++) {
                float xl = nvmoe_bf16_to_f32(xr[u][a]), xh = nvmoe_bf16_to_f32(xr[u][a] >> 16);
#pragma unroll
                for (int b = 0; b < ET; b++) {
                    acc[a][b] = __fmaf_rn(xl, nvmoe_bf16_to_f32(wr[u][b]), acc[a][b]);
                    acc[a][b] = __fmaf_rn(xh, nvmoe_bf16_to_f32(wr[u][b] >> 16), acc[a][b]);
                }
            }
        }
    }
    // butterfly step 32: lanes v and v^32 live in different warps
    if (v >= 32u) {
#pragma unroll
        for (int a = 0; a < TT; a++)
#pragma unroll
            for (int b = 0; b < ET; b++) fold[a * ET + b][v - 32u] = acc[a][b];
    }
    __syncthreads();
    if (v < 32u) {
#pragma unroll
        for (int a = 0; a < TT; a++)
#pragma unroll
            for (int b = 0; b < ET; b++) {
                float sum = warp_butterfly_sum(__fadd_rn(acc[a][b], fold[a * ET + b][v]));
                if (v == 0u) result[a * ET + b] = sum;
            }
    }
    __syncthreads();
    // pack pairs of outputs into words; ET is even so a word never straddles two blocks
    const uint32_t out_words = (outputs + 1u) / 2u;
    for (uint32_t i = v; i < TT * (ET / 2); i += 64u) {
        uint32_t a = i / (ET / 2), bw = i % (ET / 2);
        uint32_t t = t0 + a, e = e0 + 2u * bw;
        if (t >= tokens || e >= outputs) continue;
        float lo = result[a * ET + 2u * bw];
        float hi = result[a * ET + 2u * bw + 1u];
        if (bias) {
            lo = __fadd_rn(lo, nvmoe_bf16_to_f32(bias[e]));
            if (e + 1u < outputs) hi = __fadd_rn(hi, nvmoe_bf16_to_f32(bias[e + 1u]));
        }
        uint32_t word = nvmoe_f32_to_bf16(lo);
        if (e + 1u < outputs) word |= nvmoe_f32_to_bf16(hi) << 16;
        logits[(size_t)t * out_words + e / 2u] = word;
    }
}

// The same projection for large batches. What bounds the kernel above there is not the arithmetic but the
// operands: a block of 4 x 16 pairs reads its 20 rows from L2 for 128 multiply-adds a step, and every weight row is
// fetched again by every block of four tokens. Here a block of 256 threads owns 32 tokens x 16 outputs: the rows of
// a 128-column chunk are staged in shared memory by 16-byte asynchronous copies (two buffers, the next chunk lands
// while this one is used) and shared by the block's eight warps, each of which owns 8 tokens x 8 outputs. A thread
// plays two of the shader's 64 lanes, l and l + 32, for every pair of its warp's tile: the first butterfly step
// (lane v with lane v ^ 32) is then an add inside the thread and the other five are the usual shuffles. Sums, their
// order and the roundings are those of router_linear_kernel, bit for bit.
constexpr int kTileTokens = 32, kTileOutputs = 16, kSubTokens = 8, kSubOutputs = 8;
__global__ void __launch_bounds__(256, 1) router_linear_tiled_kernel(const uint16_t* __restrict__ x,
                                                                    const uint16_t* __restrict__ w,
                                                                    const uint16_t* __restrict__ bias,
                                                                    uint32_t* __restrict__ logits, uint32_t tokens,
                                                                    uint32_t hidden, uint32_t outputs) {
    constexpr int kRows = kTileTokens + kTileOutputs;
    __shared__ __align__(16) uint32_t stage[2][kRows][64];   // [buffer][token rows, then output rows][word of the chunk]
    __shared__ float result[kTileTokens][kTileOutputs];
    grid_dependency_sync();
    const uint32_t warp = threadIdx.x >> 5, l = threadIdx.x & 31u;
    const uint32_t t0 = blockIdx.y * kTileTokens, e0 = blockIdx.x * kTileOutputs;
    const uint32_t ta = (warp >> 1) * kSubTokens, eb = (warp & 1u) * kSubOutputs;  // this warp's corner of the block's tile
    const uint32_t words = hidden / 2u;
    const uint32_t chunks = (words + 63u) / 64u;
    const uint32_t* xw = reinterpret_cast<const uint32_t*>(x);
    const uint32_t* ww = reinterpret_cast<const uint32_t*>(w);
    // the 16-byte pieces of a chunk this thread copies: row = piece / 16, four words from word 4 (piece % 16)
    auto fetch = [&](uint32_t chunk, uint32_t buffer) {
#pragma unroll
        for (uint32_t i = 0; i < (kRows * 16u) / 256u; i++) {
            const uint32_t piece = threadIdx.x + 256u * i;
            const uint32_t row = piece >> 4, col = (piece & 15u) * 4u;
            const uint32_t cw = chunk * 64u + col;
            const bool token_row = row < (uint32_t)kTileTokens;
            const uint32_t index = token_row ? t0 + row : e0 + row - kTileTokens;
            const bool ok = cw < words && index < (token_row ? tokens : outputs);
            const uint32_t* src = ok ? (token_row ? xw : ww) + (size_t)index * words + cw : xw;
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(&stage[buffer][row][col]);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(ok ? 16u : 0u) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float acc[2][kSubTokens][kSubOutputs];
#pragma unroll
    for (int h = 0; h < 2; h++)
#pragma unroll
        for (int a = 0; a < kSubTokens; a++)
#pragma unroll
            for (int b = 0; b < kSubOutputs; b++) acc[h][a][b] = 0.0f;
    fetch(0u, 0u);
    for (uint32_t chunk = 0; chunk < chunks; chunk++) {
        const uint32_t buffer = chunk & 1u;
        if (chunk + 1u < chunks) {
            fetch(chunk + 1u, buffer ^ 1u);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
#pragma unroll
        for (int h = 0; h < 2; h++) {
            // lane l + 32 h of the shader; a lane whose word lies past the row adds nothing (not even zeros: -0 + 0 = +0)
            if (chunk * 64u + l + 32u * h < words) {
                uint32_t xr[kSubTokens], wr[kSubOutputs];
#pragma unroll
                for (int a = 0; a < kSubTokens; a++) xr[a] = stage[buffer][ta + a][l + 32u * h];
#pragma unroll
                for (int b = 0; b < kSubOutputs; b++) wr[b] = stage[buffer][kTileTokens + eb + b][l + 32u * h];
#pragma unroll
                for (int a = 0; a < kSubTokens; a++) {
                    const float xl = nvmoe_bf16_to_f32(xr[a]), xh = nvmoe_bf16_to_f32(xr[a] >> 16);
#pragma unroll
                    for (int b = 0; b < kSubOutputs; b++) {
                        acc[h][a][b] = __fmaf_rn(xl, nvmoe_bf16_to_f32(wr[b]), acc[h][a][b]);
                        acc[h][a][b] = __fmaf_rn(xh, nvmoe_bf16_to_f32(wr[b] >> 16), acc[h][a][b]);
                    }
                }
            }
        }
        __syncthreads();  // the buffer is refilled by the fetch of the next round
    }
#pragma unroll
    for (int a = 0; a < kSubTokens; a++)
#pragma unroll
        for (int b = 0; b < kSubOutputs; b++) {
            // butterfly step 32 (lane l with lane l + 32) inside the thread, then 16 .. 1 across the warp
            const float sum = warp_butterfly_sum(__fadd_rn(acc[0][a][b], acc[1][a][b]));
            if (l == 0u) result[ta + a][eb + b] = sum;
        }
    __syncthreads();
    const uint32_t out_words = (outputs + 1u) / 2u;
    for (uint32_t i = threadIdx.x; i < kTileTokens * (kTileOutputs / 2); i += 256u) {
        const uint32_t a = i / (kTileOutputs / 2), bw = i % (kTileOutputs / 2);
        const uint32_t t = t0 + a, e = e0 + 2u * bw;
        if (t >= tokens || e >= outputs) continue;
        float lo = result[a][2u * bw], hi = result[a][2u * bw + 1u];
        if (bias) {
            lo = __fadd_rn(lo, nvmoe_bf16_to_f32(bias[e]));
            if (e + 1u < outputs) hi = __fadd_rn(hi, nvmoe_bf16_to_f32(bias[e + 1u]));
        }
        uint32_t word = nvmoe_f32_to_bf16(lo);
        if (e + 1u < outputs) word |= nvmoe_f32_to_bf16(hi) << 16;
        logits[(size_t)t * out_words + e / 2u] = word;
    }
}

}  // namespace

void launch_router(const RouterLaunch& p, cudaStream_t stream) {
    const uint32_t E = p.g.routed_experts;
    const uint32_t total_k = p.g.routed_k + (p.g.router_kind == NVMOE_ROUTER_SCORE_TOPK ? p.g.always_count : 0u);
    // the routed form's softmax over all experts (neither normalised over the selection nor sigmoid) sums in expert order
    const bool sums_all = p.g.router_kind == NVMOE_ROUTER_TOPK_ROUTED && !p.g.normalize_selected && p.g.activation != NVMOE_ACT_SIGMOID;
    if (E <= 256u && total_k <= 32u && p.g.n_group == 0u && !sums_all && p.g.router_kind <= NVMOE_ROUTER_TOPK_ROUTED) {
        const dim3 grid((p.tokens + 3u) / 4u), block(128);
        if (E <= 32u) {
            launch_chained(router_reg_kernel<1>, grid, block, 0, stream, p);
        } else if (E <= 128u) {
            launch_chained(router_reg_kernel<4>, grid, block, 0, stream, p);
        } else {
            launch_chained(router_reg_kernel<8>, grid, block, 0, stream, p);
        }
        return;
    }
    const size_t per_warp = (size_t)E * 12u + kMaxTopK * 8u + 32u * 4u;
    uint32_t warps = E <= 1024u ? 4u : 1u;
    size_t smem = per_warp * warps;
    if (smem > 48u * 1024u)
        cudaFuncSetAttribute(router_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    uint32_t blocks = (p.tokens + warps - 1u) / warps;
    launch_chained(router_kernel, dim3(blocks), dim3(warps * 32u), smem, stream, p, warps);
}

void launch_router_linear(const uint16_t* x, const uint16_t* w, const uint16_t* bias, uint32_t* logits,
                          uint32_t tokens, uint32_t hidden, uint32_t outputs, cudaStream_t stream) {
    if (tokens <= 256u) {
        dim3 grid((outputs + 3u) / 4u, (tokens + 1u) / 2u);
        launch_chained(router_linear_kernel<2, 4>, grid, dim3(64), 0, stream, x, w, bias, logits, tokens, hidden, outputs);
    } else if (hidden % 8u == 0u && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15u) == 0u) {
        dim3 grid((outputs + kTileOutputs - 1u) / kTileOutputs, (tokens + kTileTokens - 1u) / kTileTokens);
        launch_chained(router_linear_tiled_kernel, grid, dim3(256), 0, stream, x, w, bias, logits, tokens, hidden, outputs);
    } else {
        dim3 grid((outputs + 15u) / 16u, (tokens + 3u) / 4u);
        launch_chained(router_linear_kernel<4, 16>, grid, dim3(64), 0, stream, x, w, bias, logits, tokens, hidden, outputs);
    }
}

}  // namespace nvmoe
