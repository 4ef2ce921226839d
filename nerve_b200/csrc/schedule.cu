// Route scheduling: the reference's compact/count stages and the expert grouping the grouped
// expert kernels consume.
//
//   route_compact   runtime-rs/shaders/moe_route_compact_batch1.comp.template:26-105
//   route_count     runtime-rs/shaders/moe_route_count_batch1.comp.template:21-58
//
// The reference ranks every (token, route) against every other one — quadratic in T*K.  The
// rank it computes, #{c : expert(c) < expert(s) or (expert(c) == expert(s) and c < s)}, is the
// position of s in a STABLE sort by expert id, so the same list comes out of a counting sort:
// per-block histograms, an exclusive scan over (expert, block), and a scatter in which equal
// experts keep source order (warp match + popcount of lower lanes, warps taken in order).
// Route ids at or above the expert count cannot be produced by the routers here; they are placed
// after every valid id in source order (the reference would order them by id).
#include "common.cuh"

namespace nvmoe {
namespace {

// ---- generic stable counting sort over `count` keys ------------------------------------------
// KeyFn(i) -> bucket in [0, buckets) or kUnboundSlot to drop item i.  EmitFn(rank, i) stores it.

template <class KeyFn>
__device__ void block_histogram(uint32_t begin, uint32_t end, uint32_t buckets, uint32_t* hist, KeyFn key) {
    for (uint32_t b = threadIdx.x; b < buckets; b += blockDim.x) hist[b] = 0u;
    __syncthreads();
    for (uint32_t i = begin + threadIdx.x; i < end; i += blockDim.x) {
        uint32_t kb = key(i);
        if (kb != kUnboundSlot) atomicAdd(hist + kb, 1u);
    }
    __syncthreads();
}

// Stable scatter of items [begin, end) given running[b] = rank of the next item of bucket b.
// blockDim.x must be a multiple of 32; warps take turns so that source order is kept.
template <class KeyFn, class EmitFn>
__device__ void block_stable_scatter(uint32_t begin, uint32_t end, uint32_t* running, KeyFn key, EmitFn emit) {
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (uint32_t base = begin; base < end; base += blockDim.x) {
        uint32_t i = base + threadIdx.x;
        uint32_t kb = i < end ? key(i) : kUnboundSlot;
        for (uint32_t w = 0; w < warps; w++) {
            if (w == warp) {
                uint32_t peers = __match_any_sync(0xffffffffu, kb);
                if (kb != kUnboundSlot) {
                    uint32_t before = __popc(peers & ((1u << lane) - 1u));
                    uint32_t leader = __ffs(peers) - 1u;
                    uint32_t start = 0u;
                    if (lane == leader) {
                        start = running[kb];
                        running[kb] = start + __popc(peers);
                    }
                    start = __shfl_sync(peers, start, leader);
                    emit(start + before, i);
                }
            }
            __syncthreads();
        }
    }
}

// One block does the whole sort (small inputs: one launch instead of three).
template <class KeyFn, class EmitFn, class DoneFn>
__device__ void sort_single_block(uint32_t count, uint32_t buckets, uint32_t* smem_hist, KeyFn key,
                                  EmitFn emit, DoneFn done) {
    block_histogram(0u, count, buckets, smem_hist, key);
    // exclusive scan over buckets by one warp (buckets <= 4097)
    if (threadIdx.x < 32u) {
        uint32_t carry = 0u;
        for (uint32_t b0 = 0; b0 < buckets; b0 += 32u) {
            uint32_t b = b0 + threadIdx.x;
            uint32_t v = b < buckets ? smem_hist[b] : 0u;
            uint32_t incl = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                uint32_t n = __shfl_up_sync(0xffffffffu, incl, o);
                if ((int)threadIdx.x >= o) incl += n;
            }
            if (b < buckets) smem_hist[b] = carry + incl - v;
            carry += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (threadIdx.x == 0u) smem_hist[buckets] = carry;
    }
    __syncthreads();
    done(smem_hist);  // bucket bases (exclusive) with the total at [buckets]
    __syncthreads();
    block_stable_scatter(0u, count, smem_hist, key, emit);
}

// ---- keys ----------------------------------------------------------------------------------

struct RouteKey {  // compact: rank all T*K routes by expert id
    const uint32_t* routes;
    uint32_t num_experts;
    __device__ uint32_t operator()(uint32_t i) const {
        uint32_t e = routes[i] & 0xffffu;
        return e < num_experts ? e : num_experts;
    }
};

__device__ __forceinline__ bool resource_is_local(const uint32_t* slots, uint32_t slot_words,
                                                  uint32_t params, uint32_t expert) {
    if (!slots) return true;
    uint64_t index = (uint64_t)expert * params;
    if (index >= slot_words) return false;
    return slots[index] != kUnboundSlot;
}

struct OwnedKey {  // partitioned compact: keep owned routes, in source order (one bucket)
    const uint32_t* routes;
    const uint32_t* slots;
    uint32_t slot_words, params, start, end;
    __device__ uint32_t operator()(uint32_t i) const {
        uint32_t e = routes[i] & 0xffffu;
        if (e < start || e >= end || !resource_is_local(slots, slot_words, params, e)) return kUnboundSlot;
        return 0u;
    }
};

struct ScheduleEmit {  // writes the compact list into the schedule words of the frames
    uint32_t* intermediates;
    uint32_t K, frame_words, data_words;
    uint32_t* copy = nullptr;  // optional second, flat copy of the list
    __device__ void operator()(uint32_t rank, uint32_t i) const {
        intermediates[(size_t)(rank / K) * frame_words + data_words + rank % K] = i;
        if (copy) copy[rank] = i;
    }
};

// the slot the expert shaders read for compact position c, or kUnboundSlot when they return early
struct SlotKey {
    const uint32_t* routes;
    const uint32_t* intermediates;
    const ExpertPtrs* experts;
    uint32_t* status;
    uint32_t num_experts, K, frame_words, data_words, capacity;
    const uint8_t* resident = nullptr;  // optional per-expert copy of "experts[e].w[0] != nullptr" (a faster place)
    __device__ uint32_t route_index(uint32_t c) const {
        return intermediates[(size_t)(c / K) * frame_words + data_words + c % K];
    }
    __device__ uint32_t operator()(uint32_t c) const {
        uint32_t ri = route_index(c);
        if (ri >= capacity) {
            raise_status(status, NVMOE_STATUS_ROUTE_OUT_OF_RANGE);
            return kUnboundSlot;
        }
        uint32_t e = routes[ri] & 0xffffu;
        if (e >= num_experts) {
            raise_status(status, NVMOE_STATUS_ROUTE_OUT_OF_RANGE);
            return kUnboundSlot;
        }
        if (resident ? resident[e] == 0u : experts[e].w[0] == nullptr) {
            raise_status(status, NVMOE_STATUS_EXPERT_NOT_RESIDENT);
            return kUnboundSlot;
        }
        return e;
    }
};

struct GroupEmit {
    const SlotKey key;
    uint32_t* grouped;
    uint32_t* position;  // optional inverse: position[route] = its place in `grouped`
    __device__ void operator()(uint32_t rank, uint32_t c) const {
        const uint32_t ri = key.route_index(c);
        grouped[rank] = ri;
        if (position) position[ri] = rank;
    }
};

// ---- kernels ---------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t min_u32(uint32_t a, uint32_t b) { return a < b ? a : b; }

// Single-block compact (T*K small).  `control` is read for batch_width / expert range and the
// owned count and indirect-dispatch words are written back exactly as the shader does.
__device__ void compact_small_body(const uint32_t* routes, uint32_t* intermediates, const uint32_t* slots,
                                   uint32_t slot_words, uint32_t params, uint32_t* control, uint32_t max_tokens,
                                   uint32_t K, uint32_t I, uint32_t tiles_per_route, uint32_t num_experts,
                                   uint32_t* hist, uint32_t* list_copy = nullptr) {
    const uint32_t T = min_u32(control[0], max_tokens);
    const uint32_t count = T * K;
    const uint32_t data_words = K * (I / 2u);
    ScheduleEmit emit{intermediates, K, data_words + K, data_words, list_copy};
    if (control[2] != 0u) {
        OwnedKey key{routes, slots, slot_words, params, control[1], control[1] + control[2]};
        sort_single_block(count, 1u, hist, key, emit, [&](const uint32_t* base) {
            if (threadIdx.x == 0u) {
                control[3] = base[1];
                control[4] = base[1] * tiles_per_route;
                control[5] = 1u;
                control[6] = 1u;
            }
        });
    } else {
        RouteKey key{routes, num_experts};
        sort_single_block(count, num_experts + 1u, hist, key, emit, [&](const uint32_t*) {
            if (threadIdx.x == 0u) {
                control[3] = count;
                control[4] = K * tiles_per_route;
                control[5] = T;
                control[6] = 1u;
            }
        });
    }
}

__global__ void __launch_bounds__(1024) compact_small_kernel(const uint32_t* routes, uint32_t* intermediates,
                                                            const uint32_t* slots, uint32_t slot_words,
                                                            uint32_t params, uint32_t* control,
                                                            uint32_t max_tokens, uint32_t K, uint32_t I,
                                                            uint32_t tiles_per_route, uint32_t num_experts) {
    extern __shared__ uint32_t hist[];
    compact_small_body(routes, intermediates, slots, slot_words, params, control, max_tokens, K, I, tiles_per_route,
                       num_experts, hist);
}

// Multi-block sort, phase 1: per-block histograms.
template <class KeyFn>
__device__ void phase_hist(uint32_t count, uint32_t buckets, uint32_t* block_hist, KeyFn key) {
    extern __shared__ uint32_t hist[];
    uint32_t begin = blockIdx.x * kSortChunk;
    if (begin >= count) {
        for (uint32_t b = threadIdx.x; b < buckets; b += blockDim.x) block_hist[(size_t)blockIdx.x * buckets + b] = 0u;
        return;
    }
    uint32_t end = min_u32(begin + kSortChunk, count);
    block_histogram(begin, end, buckets, hist, key);
    for (uint32_t b = threadIdx.x; b < buckets; b += blockDim.x) block_hist[(size_t)blockIdx.x * buckets + b] = hist[b];
}

// phase 2 (one block): block_hist[blk][b] <- rank of the first item of bucket b in block blk;
// bucket_base[b] <- exclusive scan of bucket totals, total at [buckets].
__global__ void __launch_bounds__(1024) phase_scan_kernel(uint32_t* block_hist, uint32_t* bucket_base,
                                                         uint32_t blocks, uint32_t buckets) {
    extern __shared__ uint32_t totals[];
    // a warp per bucket: thirty-two blocks' counts are scanned at a time with shuffles
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (uint32_t b = warp; b < buckets; b += warps) {
        uint32_t run = 0u;
        for (uint32_t blk0 = 0; blk0 < blocks; blk0 += 32u) {
            const uint32_t blk = blk0 + lane;
            const uint32_t v = blk < blocks ? block_hist[(size_t)blk * buckets + b] : 0u;
            uint32_t incl = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t n = __shfl_up_sync(0xffffffffu, incl, o);
                if ((int)lane >= o) incl += n;
            }
            if (blk < blocks) block_hist[(size_t)blk * buckets + b] = run + incl - v;
            run += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0u) totals[b] = run;
    }
    __syncthreads();
    if (threadIdx.x < 32u) {
        uint32_t carry = 0u;
        for (uint32_t b0 = 0; b0 < buckets; b0 += 32u) {
            uint32_t b = b0 + threadIdx.x;
            uint32_t v = b < buckets ? totals[b] : 0u;
            uint32_t incl = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                uint32_t n = __shfl_up_sync(0xffffffffu, incl, o);
                if ((int)threadIdx.x >= o) incl += n;
            }
            if (b < buckets) bucket_base[b] = carry + incl - v;
            carry += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (threadIdx.x == 0u) bucket_base[buckets] = carry;
    }
}

template <class KeyFn, class EmitFn>
__device__ void phase_scatter(uint32_t count, uint32_t buckets, const uint32_t* block_hist,
                              const uint32_t* bucket_base, KeyFn key, EmitFn emit) {
    extern __shared__ uint32_t running[];
    uint32_t begin = blockIdx.x * kSortChunk;
    if (begin >= count) return;
    uint32_t end = min_u32(begin + kSortChunk, count);
    for (uint32_t b = threadIdx.x; b < buckets; b += blockDim.x)
        running[b] = bucket_base[b] + block_hist[(size_t)blockIdx.x * buckets + b];
    __syncthreads();
    block_stable_scatter(begin, end, running, key, emit);
}

__global__ void __launch_bounds__(256) compact_hist_kernel(const uint32_t* routes, const uint32_t* slots,
                                                          uint32_t slot_words, uint32_t params,
                                                          const uint32_t* control, uint32_t max_tokens,
                                                          uint32_t K, uint32_t num_experts, uint32_t* block_hist) {
    const uint32_t count = min_u32(control[0], max_tokens) * K;
    if (control[2] != 0u) {
        OwnedKey key{routes, slots, slot_words, params, control[1], control[1] + control[2]};
        phase_hist(count, num_experts + 1u, block_hist, key);  // one bucket used, same stride
    } else {
        RouteKey key{routes, num_experts};
        phase_hist(count, num_experts + 1u, block_hist, key);
    }
}

__global__ void __launch_bounds__(256) compact_scatter_kernel(const uint32_t* routes, uint32_t* intermediates,
                                                             const uint32_t* slots, uint32_t slot_words,
                                                             uint32_t params, uint32_t* control,
                                                             uint32_t max_tokens, uint32_t K, uint32_t I,
                                                             uint32_t tiles_per_route, uint32_t num_experts,
                                                             const uint32_t* block_hist, const uint32_t* bucket_base) {
    const uint32_t T = min_u32(control[0], max_tokens);
    const uint32_t count = T * K;
    const uint32_t data_words = K * (I / 2u);
    ScheduleEmit emit{intermediates, K, data_words + K, data_words};
    const bool partitioned = control[2] != 0u;
    // every block has read what it needs from control[0..2]; block 0 publishes the command words
    if (partitioned) {
        OwnedKey key{routes, slots, slot_words, params, control[1], control[1] + control[2]};
        phase_scatter(count, num_experts + 1u, block_hist, bucket_base, key, emit);
        if (blockIdx.x == 0u && threadIdx.x == 0u) {
            uint32_t owned = bucket_base[1];
            control[3] = owned;
            control[4] = owned * tiles_per_route;
            control[5] = 1u;
            control[6] = 1u;
        }
    } else {
        RouteKey key{routes, num_experts};
        phase_scatter(count, num_experts + 1u, block_hist, bucket_base, key, emit);
        if (blockIdx.x == 0u && threadIdx.x == 0u) {
            control[3] = count;
            control[4] = K * tiles_per_route;
            control[5] = T;
            control[6] = 1u;
        }
    }
}

// moe_route_count: the owned count only (one block; a grid-stride count is plenty here)
// (every thread of the block calls it; the branch is uniform)
__device__ void route_count_body(const uint32_t* routes, const uint32_t* slots, uint32_t slot_words, uint32_t params,
                                 uint32_t* control, uint32_t max_tokens, uint32_t K, uint32_t tiles_per_route) {
    __shared__ uint32_t owned;
    const uint32_t T = min_u32(control[0], max_tokens);
    const uint32_t start = control[1], owned_experts = control[2];
    __syncthreads();  // every thread has read the control words before one of them rewrites the tail
    if (owned_experts == 0u) {
        if (threadIdx.x == 0u) {
            control[3] = T * K;
            control[4] = K * tiles_per_route;
            control[5] = T;
            control[6] = 1u;
        }
        return;
    }
    if (threadIdx.x == 0u) owned = 0u;
    __syncthreads();
    const uint32_t end = start + owned_experts;
    uint32_t mine = 0u;
    for (uint32_t i = threadIdx.x; i < T * K; i += blockDim.x) {
        uint32_t e = routes[i] & 0xffffu;
        if (e >= start && e < end && resource_is_local(slots, slot_words, params, e)) mine++;
    }
    atomicAdd(&owned, mine);
    __syncthreads();
    if (threadIdx.x == 0u) {
        control[3] = owned;
        control[4] = owned * tiles_per_route;
        control[5] = 1u;
        control[6] = 1u;
    }
}

__global__ void __launch_bounds__(1024) route_count_kernel(const uint32_t* routes, const uint32_t* slots,
                                                          uint32_t slot_words, uint32_t params, uint32_t* control,
                                                          uint32_t max_tokens, uint32_t K, uint32_t tiles_per_route) {
    route_count_body(routes, slots, slot_words, params, control, max_tokens, K, tiles_per_route);
}

// address_record_is_resident + dynamic_parameter_record_is_valid for every expert, once per call
// (dynamic_expert_is_valid of independent_sparse_moe_gate_up_batch1_mxfp4.comp.template:166-228: a weight record's
// representation word is 0 (compact) or 1 (pre-expanded FP8), the same for both matrices of a pair; resources
// from native_start on are native FP8 and must say 0)
__global__ void resolve_experts_kernel(const uint32_t* addresses, uint32_t address_words, const uint32_t* slots,
                                       uint32_t slot_words, uint32_t params, uint32_t num_experts,
                                       uint32_t rows, uint32_t cols, uint32_t native_start, bool whole_blocks_only,
                                       uint8_t* derived_scales, size_t derived_matrix_bytes, ExpertPtrs* out) {
    uint32_t e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= num_experts) return;
    ExpertPtrs r{{nullptr, nullptr}, {nullptr, nullptr}, {nullptr, nullptr}, {0u, 0u}, kFormatCompact, 0u};
    bool ok = true;
    const uint8_t* ptrs[4] = {nullptr, nullptr, nullptr, nullptr};
    uint64_t gens[4] = {0u, 0u, 0u, 0u};
    const bool native = e >= native_start;
    // the form of the expert's matrices: the representation word of its first weight record
    uint32_t format = native ? kFormatNativeFp8 : kFormatCompact;
    if (!native && (uint64_t)e * params < slot_words) {
        const uint32_t slot = slots[(uint64_t)e * params];
        if (slot != kUnboundSlot && slot < address_words / kRecordWords && addresses[(size_t)slot * kRecordWords + 7u] == 1u)
            format = kFormatExpanded;
    }
    if (format != kFormatCompact && whole_blocks_only && cols % 128u != 0u) ok = false;
    const uint64_t weight_bytes = format == kFormatCompact ? (uint64_t)rows * (cols / 2u) : (uint64_t)rows * cols;
    const uint64_t scale_bytes = format == kFormatNativeFp8 ? (uint64_t)((rows + 127u) / 128u) * ((cols + 127u) / 128u)
                                                            : (uint64_t)rows * (cols / 32u);
    for (uint32_t j = 0; j < params && ok; j++) {
        uint64_t index = (uint64_t)e * params + j;
        if (index >= slot_words) {
            ok = false;
            break;
        }
        uint32_t slot = slots[index];
        if (slot == kUnboundSlot || slot >= address_words / kRecordWords) {
            ok = false;
            break;
        }
        const uint32_t* rec = addresses + (size_t)slot * kRecordWords;
        uint64_t address = (uint64_t)rec[0] | ((uint64_t)rec[1] << 32);
        uint64_t bytes = (uint64_t)rec[2] | ((uint64_t)rec[3] << 32);
        uint64_t required = (j & 1u) ? scale_bytes : weight_bytes;
        // what the record must say about its form: weights of a compact or native resource 0, of a pre-expanded one 1
        // (a pair that disagrees fails closed); scale records are not looked at, as in the shader
        const uint32_t expected = format == kFormatExpanded ? 1u : 0u;
        // the kernels read rows with 16-byte loads and TMA boxes, so the shader's 4-byte address rule becomes 32
        // (native FP8 scale blocks are read byte by byte: 4 as in the shader)
        const uint64_t align_mask = ((j & 1u) && format == kFormatNativeFp8) ? 3u : 31u;
        if (address == 0u || (address & align_mask) != 0u || bytes < required || (rec[4] | rec[5]) == 0u ||
            rec[6] != 1u || (!(j & 1u) && rec[7] != expected)) {
            ok = false;
            break;
        }
        ptrs[j] = reinterpret_cast<const uint8_t*>(address);
        gens[j] = (uint64_t)rec[4] | ((uint64_t)rec[5] << 32);
    }
    if (ok) {
        const uint32_t matrices = params / 2u;
        r.w[0] = ptrs[0];
        r.s[0] = ptrs[1];
        r.gen[0] = gens[1];
        r.w[1] = params == 4u ? ptrs[2] : nullptr;
        r.s[1] = params == 4u ? ptrs[3] : nullptr;
        r.gen[1] = params == 4u ? gens[3] : 0u;
        r.format = format;
        if (derived_scales) {
            r.ts[0] = derived_scales + ((size_t)e * matrices) * derived_matrix_bytes;
            // gate and up blocks of the same (row tile, K block) lie side by side, 512 bytes each: one copy brings both
            r.ts[1] = params == 4u ? r.ts[0] + 512u : nullptr;
        }
    }
    out[e] = r;
}

__device__ __forceinline__ uint32_t slot_count(const uint32_t* control, uint32_t max_tokens, uint32_t K) {
    const uint32_t T = min_u32(control[0], max_tokens);
    // route-native calls visit owned_route_count slots, the others every (batch, route) position
    return control[2] != 0u ? min_u32(control[3], T * K) : T * K;
}

__device__ void group_small_body(SlotKey key, const uint32_t* control, uint32_t max_tokens, uint32_t* grouped,
                                 uint32_t* expert_offsets, uint32_t* position, uint32_t* hist) {
    const uint32_t T = min_u32(control[0], max_tokens);
    key.capacity = T * key.K;
    const uint32_t count = slot_count(control, max_tokens, key.K);
    if (position) {  // routes the grouping drops keep "nowhere"
        for (uint32_t i = threadIdx.x; i < key.capacity; i += blockDim.x) position[i] = kUnboundSlot;
        __syncthreads();
    }
    GroupEmit emit{key, grouped, position};
    const uint32_t buckets = key.num_experts;
    sort_single_block(count, buckets, hist, key, emit, [&](const uint32_t* base) {
        for (uint32_t b = threadIdx.x; b <= buckets; b += blockDim.x) expert_offsets[b] = base[b];
    });
}

__global__ void __launch_bounds__(1024) group_small_kernel(SlotKey key, const uint32_t* control,
                                                          uint32_t max_tokens, uint32_t* grouped,
                                                          uint32_t* expert_offsets, uint32_t* position) {
    extern __shared__ uint32_t hist[];
    group_small_body(key, control, max_tokens, grouped, expert_offsets, position, hist);
}

// (expert, token tile) pairs in expert order for the tensor-core expert kernels: entry =
// (expert << 16) | token tile within the expert; every thread of one block calls it
__device__ void build_tiles_body(const uint32_t* expert_offsets, uint32_t num_experts, uint32_t n_tile,
                                 uint32_t* tiles, uint32_t* count) {
    __shared__ uint32_t warp_sums[32];
    __shared__ uint32_t carry;
    if (threadIdx.x == 0u) carry = 0u;
    __syncthreads();
    for (uint32_t base = 0; base < num_experts; base += blockDim.x) {
        const uint32_t e = base + threadIdx.x;
        uint32_t mine = 0u;
        if (e < num_experts) mine = (expert_offsets[e + 1u] - expert_offsets[e] + n_tile - 1u) / n_tile;
        // block-wide exclusive scan
        uint32_t incl = mine;
        const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            uint32_t n = __shfl_up_sync(0xffffffffu, incl, o);
            if ((int)lane >= o) incl += n;
        }
        if (lane == 31u) warp_sums[warp] = incl;
        __syncthreads();
        if (warp == 0u) {
            uint32_t v = lane < (blockDim.x >> 5) ? warp_sums[lane] : 0u;
            uint32_t sum = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                uint32_t n = __shfl_up_sync(0xffffffffu, sum, o);
                if ((int)lane >= o) sum += n;
            }
            warp_sums[lane] = sum - v;
        }
        __syncthreads();
        const uint32_t start = carry + warp_sums[warp] + incl - mine;
        for (uint32_t j = 0; j < mine; j++) tiles[start + j] = (e << 16) | j;
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1u) carry = start + mine;
        __syncthreads();
    }
    if (threadIdx.x == 0u) *count = carry;
}

__global__ void __launch_bounds__(1024) build_tiles_kernel(const uint32_t* expert_offsets, uint32_t num_experts,
                                                          uint32_t n_tile, uint32_t* tiles, uint32_t* count) {
    build_tiles_body(expert_offsets, num_experts, n_tile, tiles, count);
}

// The whole schedule of one layer call in one block (T*K small): the control words the host of the
// reference writes, the compact list in front of gate/up, the owned count in front of down, and for
// each of the two expert stages the expert-grouped route list and the tensor-path tile list.
// Shared memory of the fused schedule: sort histogram, then copies of what the five passes would otherwise
// fetch from global memory through chains of dependent loads: the route words, the compact list, and
// per stage whether each expert is resident.
__host__ __device__ inline size_t layer_schedule_smem_bytes(uint32_t count, uint32_t num_experts) {
    return ((size_t)num_experts + 2u + 2u * count) * sizeof(uint32_t) + 2u * (size_t)num_experts;
}

__global__ void __launch_bounds__(1024) layer_schedule_small_kernel(LayerSchedule s) {
    extern __shared__ uint32_t hist[];
    const uint32_t count = s.tokens * s.K;
    uint32_t* route_words = hist + s.num_experts + 2u;
    uint32_t* compact_list = route_words + count;
    uint8_t* resident = reinterpret_cast<uint8_t*>(compact_list + count);
    grid_dependency_sync();
    if (threadIdx.x < 14u) {
        const uint32_t j = threadIdx.x % 7u;
        s.control[threadIdx.x / 7u][j] = j == 0u ? s.tokens : j == 1u ? s.expert_start : j == 2u ? s.expert_count : 0u;
    }
    for (uint32_t i = threadIdx.x; i < count; i += blockDim.x) {
        route_words[i] = s.routes[i];
        compact_list[i] = kUnboundSlot;  // positions past the owned count stay out of range
    }
    for (uint32_t e = threadIdx.x; e < 2u * s.num_experts; e += blockDim.x)
        resident[e] = s.experts[e / s.num_experts][e % s.num_experts].w[0] != nullptr ? 1u : 0u;
    __syncthreads();
    compact_small_body(route_words, s.intermediates, s.slots[0], s.slot_words[0], 4u, s.control[0], s.tokens, s.K, s.I,
                       s.tiles_per_route[0], s.num_experts, hist, compact_list);
    __syncthreads();
    route_count_body(route_words, s.slots[1], s.slot_words[1], 2u, s.control[1], s.tokens, s.K, s.tiles_per_route[1]);
    __syncthreads();
    for (uint32_t stage = 0; stage < 2u; stage++) {
        // the flat copy of the compact list stands in for the schedule words of the frames: frame = K words, no data
        SlotKey key{route_words, compact_list, s.experts[stage], s.status, s.num_experts, s.K, s.K, 0u, 0u,
                    resident + stage * s.num_experts};
        group_small_body(key, s.control[stage], s.tokens, s.grouped[stage], s.offsets[stage], s.position[stage], hist);
        __syncthreads();
        if (s.tiles[stage]) build_tiles_body(s.offsets[stage], s.num_experts, s.n_tile[stage], s.tiles[stage], s.tile_count[stage]);
        __syncthreads();
    }
}

// The same schedule from one pass over the routes.  The compact list and both expert groupings are one
// stable sort of the routes by expert id seen through different filters: the rank r of a route among the
// listed routes of its expert is found once, and every list position is a per-list bucket base plus r.
// Rank: a warp ranks its 32 routes with match_any and leaves its per-bucket counts in a table
// [warp][bucket]; a column-wise running sum turns the counts into the ranks where each warp's routes start.
// The partitioned call (expert_count != 0) lists only owned routes, in source order (one more table column
// counts them per warp), and its down stage visits the first owned-by-the-down-table-count of them.
// One round trip to global memory, five block barriers.
constexpr uint32_t kRankChunks = 16u;  // routes per thread at most (count <= 16 * blockDim); the kernel is built for 1, 4 and 16
constexpr uint32_t kNotListed = 0xffffu;  // bucket field of a route that is in no list

__host__ __device__ inline uint32_t layer_schedule_rank_threads(uint32_t count) { return count <= 256u ? 256u : 1024u; }

__host__ __device__ inline size_t layer_schedule_rank_smem_bytes(uint32_t count, uint32_t num_experts) {
    const size_t columns = (size_t)num_experts + 2u;  // experts, out-of-range ids, owned routes
    const size_t warps = ((size_t)count + 31u) / 32u;
    // table (u16, rounded to words); hist, hist_down, base_all, gbase[2], tile_base[2] (columns + 1 words each);
    // two totals; kept[2] (a byte per column)
    return ((warps * columns + 1u) / 2u + 7u * (columns + 1u) + 2u) * sizeof(uint32_t) + 2u * columns;
}

template <uint32_t CHUNKS>
__global__ void __launch_bounds__(1024) layer_schedule_rank_kernel(LayerSchedule s) {
    extern __shared__ uint32_t smem_words[];
    const uint32_t count = s.tokens * s.K;
    const uint32_t E = s.num_experts;
    const uint32_t B = E + 1u;   // bucket E collects out-of-range expert ids
    const uint32_t C = E + 2u;   // column B counts the owned routes of a warp (partitioned calls)
    const uint32_t V = (count + 31u) / 32u;
    const uint32_t table_words = (V * C + 1u) / 2u;
    uint16_t* table = reinterpret_cast<uint16_t*>(smem_words);
    uint32_t* hist = smem_words + table_words;  // listed routes per bucket
    uint32_t* hist_down = hist + (C + 1u);      // of which the down stage visits
    uint32_t* base_all = hist + 2u * (C + 1u);
    uint32_t* gbase[2] = {hist + 3u * (C + 1u), hist + 4u * (C + 1u)};
    uint32_t* tile_base[2] = {hist + 5u * (C + 1u), hist + 6u * (C + 1u)};
    uint32_t* totals = hist + 7u * (C + 1u);  // owned routes under the gate/up and the down slot table
    uint8_t* kept = reinterpret_cast<uint8_t*>(totals + 2u);  // [2][C]: the stage keeps routes of this bucket
    const uint32_t lane = threadIdx.x & 31u;
    const bool partitioned = s.expert_count != 0u;
    const uint32_t owned_end = s.expert_start + s.expert_count;

    for (uint32_t w = threadIdx.x; w < table_words; w += blockDim.x) smem_words[w] = 0u;
    if (threadIdx.x < 2u) totals[threadIdx.x] = 0u;
    grid_dependency_sync();
    // residency of every expert for both stages (bucket E is never kept)
    for (uint32_t i = threadIdx.x; i < 2u * C; i += blockDim.x) {
        const uint32_t stage = i / C, b = i % C;
        kept[i] = (b < E && s.experts[stage][b].w[0] != nullptr) ? 1u : 0u;
    }
    // per route: bucket (16 bits) | routes of the same bucket before it in its warp (8) | owned routes before it (8)
    uint32_t state[CHUNKS];
    __syncthreads();
#pragma unroll
    for (uint32_t c = 0; c < CHUNKS; c++) {
        const uint32_t i = c * blockDim.x + threadIdx.x;
        state[c] = kNotListed;
        if (c * blockDim.x < count) {  // uniform over the block: whole warps take part in the votes
            bool listed = i < count, owned_down = false;
            uint32_t e = 0u;
            if (listed) e = s.routes[i] & 0xffffu;
            if (partitioned) {
                const bool in_range = listed && e >= s.expert_start && e < owned_end;
                listed = in_range && resource_is_local(s.slots[0], s.slot_words[0], 4u, e);
                owned_down = in_range && resource_is_local(s.slots[1], s.slot_words[1], 2u, e);
                const uint32_t owners = __ballot_sync(0xffffffffu, listed);
                const uint32_t owners_down = __ballot_sync(0xffffffffu, owned_down);
                state[c] |= (uint32_t)__popc(owners & ((1u << lane) - 1u)) << 24;
                if (lane == 0u) {
                    if (owners) {  // a warp past the end of the routes has no row in the table
                        table[(size_t)(i >> 5) * C + B] = (uint16_t)__popc(owners);
                        atomicAdd(totals + 0, (uint32_t)__popc(owners));
                    }
                    if (owners_down) atomicAdd(totals + 1, (uint32_t)__popc(owners_down));
                }
            }
            const uint32_t bucket = listed ? min_u32(e, E) : kNotListed;
            const uint32_t peers = __match_any_sync(0xffffffffu, bucket);
            state[c] = (state[c] & 0xff000000u) | ((uint32_t)__popc(peers & ((1u << lane) - 1u)) << 16) | bucket;
            if (listed && lane == (uint32_t)__ffs(peers) - 1u) table[(size_t)(i >> 5) * C + bucket] = (uint16_t)__popc(peers);
        }
    }
    __syncthreads();
    // the down stage of a partitioned call visits the first totals[1] entries of the compact list
    const uint32_t listed_total = partitioned ? totals[0] : count;
    const uint32_t down_total = partitioned ? totals[1] : count;
    const bool cut = down_total < listed_total;
    for (uint32_t b = threadIdx.x; b < C; b += blockDim.x) {
        uint32_t running = 0u;
        for (uint32_t v = 0; v < V; v++) {
            const uint32_t here = table[(size_t)v * C + b];
            table[(size_t)v * C + b] = (uint16_t)running;
            running += here;
        }
        hist[b] = running;
        hist_down[b] = cut ? 0u : running;
    }
    __syncthreads();
    if (cut) {
        // the entries cut off are the last in source order, so the ranks of the others stand; only the counts change
#pragma unroll
        for (uint32_t c = 0; c < CHUNKS; c++) {
            const uint32_t i = c * blockDim.x + threadIdx.x;
            const uint32_t bucket = state[c] & 0xffffu;
            if (i < count && bucket != kNotListed && table[(size_t)(i >> 5) * C + B] + (state[c] >> 24) < down_total)
                atomicAdd(hist_down + bucket, 1u);
        }
        __syncthreads();
    }
    // five exclusive scans over the buckets, a warp each: the compact list of an unpartitioned call, and per
    // stage the grouped list and the tile list
    const uint32_t warp = threadIdx.x >> 5;
    if (warp < 5u) {
        const uint32_t stage = warp == 0u ? 0u : (warp - 1u) & 1u;
        const bool tiles = warp >= 3u;
        uint32_t* out = warp == 0u ? base_all : tiles ? tile_base[stage] : gbase[stage];
        const uint32_t* counts = stage == 1u ? hist_down : hist;
        uint32_t carry = 0u;
        for (uint32_t b0 = 0; b0 < B; b0 += 32u) {
            const uint32_t b = b0 + lane;
            uint32_t v = b < B ? counts[b] : 0u;
            if (warp != 0u && b < B) {
                v = kept[stage * C + b] ? v : 0u;
                if (tiles) v = (v + s.n_tile[stage] - 1u) / s.n_tile[stage];
            }
            uint32_t incl = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t n = __shfl_up_sync(0xffffffffu, incl, o);
                if ((int)lane >= o) incl += n;
            }
            if (b < B) out[b] = carry + incl - v;
            carry += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0u) out[B] = carry;
    }
    __syncthreads();
    if (threadIdx.x < 14u) {
        const uint32_t stage = threadIdx.x / 7u, j = threadIdx.x % 7u;
        const uint32_t visited = stage == 0u ? listed_total : down_total;
        uint32_t value = 1u;  // word 6; word 5 of a partitioned call
        if (j == 0u) value = s.tokens;
        if (j == 1u) value = s.expert_start;
        if (j == 2u) value = s.expert_count;
        if (j == 3u) value = visited;
        if (j == 4u) value = (partitioned ? visited : s.K) * s.tiles_per_route[stage];
        if (j == 5u && !partitioned) value = s.tokens;
        s.control[stage][j] = value;
    }
    // a down count beyond the compact list makes the down stage read entries that were never written
    if (threadIdx.x == 0u && down_total > listed_total) raise_status(s.status, NVMOE_STATUS_ROUTE_OUT_OF_RANGE);
    const uint32_t data_words = s.K * (s.I / 2u), frame_words = data_words + s.K;
#pragma unroll
    for (uint32_t c = 0; c < CHUNKS; c++) {
        const uint32_t i = c * blockDim.x + threadIdx.x;
        if (i >= count) continue;
        const uint32_t b = state[c] & 0xffffu;
        const bool listed = b != kNotListed;
        uint32_t rank = 0u, at = 0u;
        if (listed) {
            rank = table[(size_t)(i >> 5) * C + b] + ((state[c] >> 16) & 0xffu);
            at = partitioned ? table[(size_t)(i >> 5) * C + B] + (state[c] >> 24) : base_all[b] + rank;
            s.intermediates[(size_t)(at / s.K) * frame_words + data_words + at % s.K] = i;
        }
        for (uint32_t stage = 0; stage < 2u; stage++) {
            uint32_t place = kUnboundSlot;
            if (listed && (stage == 0u || at < down_total)) {
                if (kept[stage * C + b]) {
                    place = gbase[stage][b] + rank;
                    s.grouped[stage][place] = i;
                } else {
                    raise_status(s.status, b == E ? NVMOE_STATUS_ROUTE_OUT_OF_RANGE : NVMOE_STATUS_EXPERT_NOT_RESIDENT);
                }
            }
            if (s.position[stage]) s.position[stage][i] = place;
        }
    }
    for (uint32_t i = threadIdx.x; i < 2u * B; i += blockDim.x) {
        const uint32_t stage = i / B, b = i % B;
        // bucket E is never kept, so gbase[stage][E] is already the total the offsets end with
        s.offsets[stage][b] = gbase[stage][b];
        if (s.tiles[stage] && b < E) {
            const uint32_t first = tile_base[stage][b], n = tile_base[stage][b + 1u] - first;
            for (uint32_t j = 0; j < n; j++) s.tiles[stage][first + j] = (b << 16) | j;
        }
        if (s.tiles[stage] && b == E) *s.tile_count[stage] = tile_base[stage][E];
    }
}

__global__ void __launch_bounds__(256) group_hist_kernel(SlotKey key, const uint32_t* control,
                                                        uint32_t max_tokens, uint32_t* block_hist, uint32_t* position) {
    key.capacity = min_u32(control[0], max_tokens) * key.K;
    key.status = nullptr;  // raised once, by the scatter pass
    if (position)  // routes the grouping drops keep "nowhere"; the scatter pass (a later launch) fills the rest
        for (uint32_t i = blockIdx.x * kSortChunk + threadIdx.x; i < min_u32(key.capacity, (blockIdx.x + 1u) * kSortChunk); i += blockDim.x)
            position[i] = kUnboundSlot;
    phase_hist(slot_count(control, max_tokens, key.K), key.num_experts, block_hist, key);
}

__global__ void __launch_bounds__(256) group_scatter_kernel(SlotKey key, const uint32_t* control,
                                                           uint32_t max_tokens, uint32_t* grouped,
                                                           uint32_t* expert_offsets, const uint32_t* block_hist,
                                                           const uint32_t* bucket_base, uint32_t* position) {
    key.capacity = min_u32(control[0], max_tokens) * key.K;
    GroupEmit emit{key, grouped, position};
    phase_scatter(slot_count(control, max_tokens, key.K), key.num_experts, block_hist, bucket_base, key, emit);
    if (blockIdx.x == 0u)
        for (uint32_t b = threadIdx.x; b <= key.num_experts; b += blockDim.x) expert_offsets[b] = bucket_base[b];
}

// ---- expert-parallel dispatch: group routes by the rank that owns their expert ------------------

struct DestKey {  // bucket = destination rank; kUnboundSlot in the owner table means "this rank"
    const uint32_t* routes;
    const uint32_t* owner;
    uint32_t num_experts, world, self;
    __device__ uint32_t operator()(uint32_t i) const {
        uint32_t e = routes[i] & 0xffffu;
        if (e >= num_experts) return kUnboundSlot;
        uint32_t r = owner[e];
        if (r == kUnboundSlot) r = self;
        return r < world ? r : kUnboundSlot;
    }
};

struct PackEmit {  // one warp-wide row copy per route would be faster; rows are copied by a second kernel
    const uint32_t* routes;
    uint32_t* send_routes;
    uint32_t* send_index;
    uint32_t* send_source;
    __device__ void operator()(uint32_t rank, uint32_t i) const {
        send_routes[rank] = routes[i];
        send_index[i] = rank;
        send_source[rank] = i;
    }
};

__global__ void __launch_bounds__(1024) ep_pack_small_kernel(DestKey key, PackEmit emit, uint32_t count,
                                                            uint32_t* dest_counts) {
    extern __shared__ uint32_t hist[];
    grid_dependency_sync();
    for (uint32_t i = threadIdx.x; i < count; i += blockDim.x) emit.send_index[i] = kUnboundSlot;
    __syncthreads();
    sort_single_block(count, key.world, hist, key, emit, [&](const uint32_t* base) {
        for (uint32_t b = threadIdx.x; b < key.world; b += blockDim.x) dest_counts[b] = base[b + 1u] - base[b];
    });
}

__global__ void __launch_bounds__(256) ep_pack_hist_kernel(DestKey key, uint32_t count, uint32_t* block_hist,
                                                          uint32_t* send_index) {
    for (uint32_t i = blockIdx.x * kSortChunk + threadIdx.x; i < min_u32(count, (blockIdx.x + 1u) * kSortChunk); i += blockDim.x)
        send_index[i] = kUnboundSlot;
    phase_hist(count, key.world, block_hist, key);
}

__global__ void __launch_bounds__(256) ep_pack_scatter_kernel(DestKey key, PackEmit emit, uint32_t count,
                                                             const uint32_t* block_hist, const uint32_t* bucket_base,
                                                             uint32_t* dest_counts) {
    phase_scatter(count, key.world, block_hist, bucket_base, key, emit);
    if (blockIdx.x == 0u)
        for (uint32_t b = threadIdx.x; b < key.world; b += blockDim.x) dest_counts[b] = bucket_base[b + 1u] - bucket_base[b];
}

// send_rows[p] = hidden[token of route send_source[p]]; one warp per row, 16-byte pieces
__global__ void __launch_bounds__(256) ep_gather_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                            const uint32_t* __restrict__ index, const uint32_t* total,
                                                            uint32_t max_rows, uint32_t divide, uint32_t row_vec) {
    grid_dependency_sync();
    const uint32_t rows = total ? min_u32(*total, max_rows) : max_rows;
    const uint32_t warps = (gridDim.x * blockDim.x) >> 5, lane = threadIdx.x & 31u;
    for (uint32_t r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
        const uint32_t s = index[r];
        if (s == kUnboundSlot) {
            for (uint32_t c = lane; c < row_vec; c += 32u) dst[(size_t)r * row_vec + c] = make_uint4(0u, 0u, 0u, 0u);
            continue;
        }
        const uint4* from = src + (size_t)(s / divide) * row_vec;
        uint4* to = dst + (size_t)r * row_vec;
        // eight loads in flight a lane (see ep_pad_kernel)
        for (uint32_t c0 = lane; c0 < row_vec; c0 += 256u) {
            uint4 piece[8];
#pragma unroll
            for (uint32_t u = 0; u < 8u; u++)
                if (c0 + 32u * u < row_vec) piece[u] = __ldg(from + c0 + 32u * u);
#pragma unroll
            for (uint32_t u = 0; u < 8u; u++)
                if (c0 + 32u * u < row_vec) to[c0 + 32u * u] = piece[u];
        }
    }
}

// Padded dispatch layout: destination rank d owns slots [d*cap, (d+1)*cap) of the send buffers, the
// first dest_counts[d] of them filled in source order, the others marked with an all-ones route word
// (expert id 0xffff: no scheduler keeps it). Every slot is written, so the buffers can be exchanged
// with equal splits and no count has to reach the host. One warp per slot.
__global__ void __launch_bounds__(256) ep_pad_kernel(const uint4* __restrict__ hidden, const uint32_t* __restrict__ routes,
                                                    const uint32_t* __restrict__ dest_counts,
                                                    const uint32_t* __restrict__ send_source, uint32_t world, uint32_t cap,
                                                    uint32_t K, uint32_t row_vec, uint4* __restrict__ rows_out,
                                                    uint32_t* __restrict__ routes_out, uint32_t* __restrict__ send_index,
                                                    uint32_t* status) {
    grid_dependency_sync();
    const uint32_t warps = (gridDim.x * blockDim.x) >> 5, lane = threadIdx.x & 31u;
    const uint32_t slots = world * cap;
    // a segment that cannot hold what is bound for its rank: the excess routes stay "nowhere" (send_index keeps
    // its all-ones mark, the combine counts their rows as zeros) and the caller is told
    if (blockIdx.x == 0u && threadIdx.x < world && dest_counts[threadIdx.x] > cap) raise_status(status, NVMOE_STATUS_EXCHANGE_OVERFLOW);
    for (uint32_t slot = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; slot < slots; slot += warps) {
        const uint32_t d = slot / cap, j = slot % cap;
        if (j >= min_u32(dest_counts[d], cap)) {
            if (lane == 0u) routes_out[slot] = kUnboundSlot;
            continue;
        }
        uint32_t offset = 0u;
        for (uint32_t x = lane; x < d; x += 32u) offset += dest_counts[x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) offset += __shfl_xor_sync(0xffffffffu, offset, o);
        const uint32_t i = send_source[offset + j];
        if (lane == 0u) {
            routes_out[slot] = routes[i];
            send_index[i] = slot;
        }
        const uint4* from = hidden + (size_t)(i / K) * row_vec;
        uint4* to = rows_out + (size_t)slot * row_vec;
        // eight loads in flight a lane: a row copied piece by piece costs one memory round trip per piece
        for (uint32_t c0 = lane; c0 < row_vec; c0 += 256u) {
            uint4 piece[8];
#pragma unroll
            for (uint32_t u = 0; u < 8u; u++)
                if (c0 + 32u * u < row_vec) piece[u] = __ldg(from + c0 + 32u * u);
#pragma unroll
            for (uint32_t u = 0; u < 8u; u++)
                if (c0 + 32u * u < row_vec) to[c0 + 32u * u] = piece[u];
        }
    }
}

__global__ void sum_counts_kernel(const uint32_t* counts, uint32_t n, uint32_t* total) {
    if (threadIdx.x == 0u && blockIdx.x == 0u) {
        uint32_t s = 0u;
        for (uint32_t i = 0; i < n; i++) s += counts[i];
        *total = s;
    }
}

constexpr uint32_t kSmallSortLimit = 4096u;

}  // namespace

void launch_ep_pack(const uint16_t* hidden, const uint32_t* routes, const uint32_t* owner, uint32_t tokens,
                    uint32_t K, uint32_t hidden_size, uint32_t num_experts, uint32_t world, uint32_t self,
                    uint16_t* send_rows, uint32_t* send_routes, uint32_t* send_index, uint32_t* send_source,
                    uint32_t* dest_counts, uint32_t* total, uint32_t segment_rows, uint32_t* contiguous_routes,
                    uint32_t* status, const SortScratch& scratch, cudaStream_t stream) {
    const uint32_t count = tokens * K;
    DestKey key{routes, owner, num_experts, world, self};
    // the padded form packs positions only; its route words and rows are placed by ep_pad_kernel
    PackEmit emit{routes, segment_rows ? contiguous_routes : send_routes, send_index, send_source};
    if (count <= kSmallSortLimit) {
        launch_chained(ep_pack_small_kernel, dim3(1), dim3(count <= 256u ? 256u : 1024u), (world + 1u) * sizeof(uint32_t),
                       stream, key, emit, count, dest_counts);
    } else {
        const uint32_t blocks = (count + kSortChunk - 1u) / kSortChunk;
        ep_pack_hist_kernel<<<blocks, 256, world * sizeof(uint32_t), stream>>>(key, count, scratch.block_hist, send_index);
        phase_scan_kernel<<<1, 1024, world * sizeof(uint32_t), stream>>>(scratch.block_hist, scratch.bucket_base, blocks, world);
        ep_pack_scatter_kernel<<<blocks, 256, world * sizeof(uint32_t), stream>>>(key, emit, count, scratch.block_hist,
                                                                                 scratch.bucket_base, dest_counts);
    }
    const uint32_t row_vec = hidden_size / 8u;  // uint4 per bf16 row
    if (segment_rows) {
        uint32_t pad_blocks = (world * segment_rows + 7u) / 8u;
        if (pad_blocks > 148u * 8u) pad_blocks = 148u * 8u;
        launch_chained(ep_pad_kernel, dim3(pad_blocks), dim3(256), 0, stream, reinterpret_cast<const uint4*>(hidden), routes,
                       dest_counts, send_source, world, segment_rows, K, row_vec, reinterpret_cast<uint4*>(send_rows),
                       send_routes, send_index, status);
        return;
    }
    sum_counts_kernel<<<1, 32, 0, stream>>>(dest_counts, world, total);
    uint32_t blocks = (count + 7u) / 8u;
    if (blocks > 148u * 8u) blocks = 148u * 8u;
    ep_gather_rows_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const uint4*>(hidden), reinterpret_cast<uint4*>(send_rows),
                                                      send_source, total, count, K, row_vec);
}

void launch_ep_unpack(const uint16_t* returned_rows, const uint32_t* send_index, uint32_t tokens, uint32_t K,
                      uint32_t hidden_size, uint16_t* expert_outputs, cudaStream_t stream) {
    const uint32_t count = tokens * K;
    uint32_t blocks = (count + 7u) / 8u;
    if (blocks > 148u * 8u) blocks = 148u * 8u;
    // expert_outputs[t][r] = returned_rows[send_index[t*K + r]]; routes that were dropped give zeros
    launch_chained(ep_gather_rows_kernel, dim3(blocks), dim3(256), 0, stream, reinterpret_cast<const uint4*>(returned_rows),
                   reinterpret_cast<uint4*>(expert_outputs), send_index, (const uint32_t*)nullptr, count, 1u, hidden_size / 8u);
}

void launch_route_compact(const uint32_t* routes, uint32_t* intermediates, const uint32_t* slots,
                          uint32_t slot_words, uint32_t params_per_resource, uint32_t* control,
                          uint32_t max_tokens, uint32_t K, uint32_t intermediate_size,
                          uint32_t tiles_per_route, uint32_t num_experts, const SortScratch& scratch,
                          cudaStream_t stream) {
    const uint32_t count = max_tokens * K;
    const uint32_t buckets = num_experts + 1u;
    if (count <= kSmallSortLimit) {
        uint32_t threads = count <= 256u ? 256u : 1024u;
        compact_small_kernel<<<1, threads, (buckets + 1u) * sizeof(uint32_t), stream>>>(
            routes, intermediates, slots, slot_words, params_per_resource, control, max_tokens, K,
            intermediate_size, tiles_per_route, num_experts);
        return;
    }
    const uint32_t blocks = (count + kSortChunk - 1u) / kSortChunk;
    compact_hist_kernel<<<blocks, 256, buckets * sizeof(uint32_t), stream>>>(
        routes, slots, slot_words, params_per_resource, control, max_tokens, K, num_experts, scratch.block_hist);
    // the partitioned form uses one bucket; scanning all of them costs nothing and needs no host read
    phase_scan_kernel<<<1, 1024, buckets * sizeof(uint32_t), stream>>>(scratch.block_hist, scratch.bucket_base,
                                                                        blocks, buckets);
    compact_scatter_kernel<<<blocks, 256, buckets * sizeof(uint32_t), stream>>>(
        routes, intermediates, slots, slot_words, params_per_resource, control, max_tokens, K,
        intermediate_size, tiles_per_route, num_experts, scratch.block_hist, scratch.bucket_base);
}

static bool rank_schedule_fits(uint64_t count, uint32_t num_experts) {
    return count <= (uint64_t)kRankChunks * layer_schedule_rank_threads((uint32_t)count) && num_experts < kNotListed - 1u &&
           layer_schedule_rank_smem_bytes((uint32_t)count, num_experts) <= 48u * 1024u;
}

static bool three_sort_schedule_fits(uint64_t count, uint32_t num_experts) {
    return count <= kSmallSortLimit && layer_schedule_smem_bytes((uint32_t)count, num_experts) <= 48u * 1024u;
}

bool layer_schedule_is_small(uint32_t tokens, uint32_t K, uint32_t num_experts) {
    const uint64_t count = (uint64_t)tokens * K;
    return rank_schedule_fits(count, num_experts) || three_sort_schedule_fits(count, num_experts);
}

void launch_layer_schedule_small(const LayerSchedule& s, cudaStream_t stream) {
    const uint32_t count = s.tokens * s.K;
    if (rank_schedule_fits(count, s.num_experts)) {
        const uint32_t threads = layer_schedule_rank_threads(count);
        const uint32_t chunks = (count + threads - 1u) / threads;
        auto kernel = chunks <= 1u ? layer_schedule_rank_kernel<1> : chunks <= 4u ? layer_schedule_rank_kernel<4>
                                                                                  : layer_schedule_rank_kernel<kRankChunks>;
        launch_chained(kernel, dim3(1), dim3(threads),
                       layer_schedule_rank_smem_bytes(count, s.num_experts), stream, s);
        return;
    }
    launch_chained(layer_schedule_small_kernel, dim3(1), dim3(count <= 256u ? 256u : 1024u),
                   layer_schedule_smem_bytes(count, s.num_experts), stream, s);
}

void launch_build_tiles(const uint32_t* expert_offsets, uint32_t num_experts, uint32_t n_tile, uint32_t* tiles,
                        uint32_t* count, cudaStream_t stream) {
    // tiles holds routes / 16 + experts + 1 entries: enough for any token tile size
    build_tiles_kernel<<<1, 1024, 0, stream>>>(expert_offsets, num_experts, n_tile, tiles, count);
}

void launch_route_count(const uint32_t* routes, const uint32_t* slots, uint32_t slot_words,
                        uint32_t params_per_resource, uint32_t* control, uint32_t max_tokens, uint32_t K,
                        uint32_t tiles_per_route, cudaStream_t stream) {
    route_count_kernel<<<1, 1024, 0, stream>>>(routes, slots, slot_words, params_per_resource, control,
                                               max_tokens, K, tiles_per_route);
}

void launch_resolve_experts(const uint32_t* addresses, uint32_t address_words, const uint32_t* slots,
                            uint32_t slot_words, uint32_t params_per_resource, uint32_t num_experts,
                            uint32_t rows, uint32_t cols, uint32_t native_start, bool whole_blocks_only,
                            uint8_t* derived_scales, size_t derived_matrix_bytes, ExpertPtrs* out, cudaStream_t stream) {
    resolve_experts_kernel<<<(num_experts + 127u) / 128u, 128, 0, stream>>>(
        addresses, address_words, slots, slot_words, params_per_resource, num_experts, rows, cols, native_start,
        whole_blocks_only, derived_scales, derived_matrix_bytes, out);
}

void launch_group_slots(const uint32_t* routes, const uint32_t* intermediates, const uint32_t* control,
                        const ExpertPtrs* experts, uint32_t num_experts, uint32_t max_tokens, uint32_t K,
                        uint32_t intermediate_size, uint32_t* grouped_routes, uint32_t* expert_offsets,
                        uint32_t* position, uint32_t* status, const SortScratch& scratch, cudaStream_t stream) {
    const uint32_t data_words = K * (intermediate_size / 2u);
    SlotKey key{routes, intermediates, experts, status, num_experts, K, data_words + K, data_words, 0u};
    const uint32_t count = max_tokens * K;
    if (count <= kSmallSortLimit) {
        uint32_t threads = count <= 256u ? 256u : 1024u;
        group_small_kernel<<<1, threads, (num_experts + 1u) * sizeof(uint32_t), stream>>>(
            key, control, max_tokens, grouped_routes, expert_offsets, position);
        return;
    }
    const uint32_t blocks = (count + kSortChunk - 1u) / kSortChunk;
    group_hist_kernel<<<blocks, 256, num_experts * sizeof(uint32_t), stream>>>(key, control, max_tokens,
                                                                               scratch.block_hist, position);
    phase_scan_kernel<<<1, 1024, num_experts * sizeof(uint32_t), stream>>>(scratch.block_hist, scratch.bucket_base,
                                                                            blocks, num_experts);
    group_scatter_kernel<<<blocks, 256, num_experts * sizeof(uint32_t), stream>>>(
        key, control, max_tokens, grouped_routes, expert_offsets, scratch.block_hist, scratch.bucket_base, position);
}

}  // namespace nvmoe
