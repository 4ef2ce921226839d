// Grouped expert projections on the Blackwell tensor cores (tcgen05, sm_100a).
//
//   gate/up  runtime-rs/shaders/independent_sparse_moe_gate_up_batch1_mxfp4.comp.template:643-802
//   down     runtime-rs/shaders/independent_sparse_moe_down_batch1_mxfp4.comp.template:507-610
//
// Arithmetic.  The shaders multiply E4M3 activation codes by E2M1 weight codes, scale each group
// of products by (activation scale x E8M0 weight scale) and accumulate in f32.  That is exactly a
// block-scaled MMA of kind::mxf8f6f4: A = packaged E2M1 weight codes with their E8M0 scale per 32
// columns, B = E4M3 activation codes with a UE8M0 scale per 32 columns (the reference's
// power-of-two activation scale, repeated over the 32-column groups of its block), f32
// accumulators in tensor memory.  Products are exact; only the accumulation order differs.
//
// Shape.  The weights are the M side ("swap-AB"): D[128 weight rows x N tokens] = W . X^T, so the
// packaged row-major weight tensor is the K-major A operand as it lies in HBM, a decode batch with
// a handful of tokens per expert still fills an MMA (N = 16), and every weight byte is read once.
// One CTA per SM walks a list of (expert, token tile) x weight-row tiles.
//
// Roles (288 threads): warps 0-3 epilogue (TMEM lane quadrant = warp), warp 4 allocates TMEM and
// one of its lanes issues the scale copies and MMAs, warps 5-8 stage operands into shared memory
// with cp.async whose completion arrives on the stage's mbarrier without stalling the issuer.
// E2M1 codes travel as 8-byte pieces into the low half of 16-byte slots (the padded 4-bit format
// the f8f6f4 kinds read), rows are gathered through the expert-grouped route list, and E8M0 scales
// come as ready 32x16-byte blocks (the layout tcgen05.cp expands into TMEM) from a derived copy of
// the packaged scale tensors that is rebuilt whenever a scale record's address or generation
// changes.  Stages are handed over with mbarriers; every wait is bounded (tcgen05.cuh).
#include "experts_tc.cuh"
#include "tcgen05.cuh"

namespace nvmoe {
namespace {

using namespace tc;

constexpr uint32_t kBlockM = 128u;   // weight rows per tile
constexpr uint32_t kBlockK = 128u;   // K elements per pipeline stage = 4 MMAs of K = 32
constexpr uint32_t kProducerThreads = 128u;
constexpr uint32_t kEpilogueThreads = 128u;
constexpr uint32_t kThreads = 288u;
constexpr uint32_t kATileBytes = kBlockM * 128u;   // one byte slot per element
constexpr uint32_t kScaleBlockBytes = 512u;        // 128 rows x 4 scale bytes
constexpr uint32_t kSmemBudget = 215u * 1024u;
constexpr uint32_t kMaxStages = 8u;

struct TileList {
    const uint32_t* tiles;   // (expert << 16) | token tile within the expert
    const uint32_t* count;   // number of entries
};

template <bool GATE_UP, uint32_t N_TILE>
struct Config {
    static constexpr uint32_t kMatrices = GATE_UP ? 2u : 1u;
    static constexpr uint32_t kBTileBytes = N_TILE * 128u;
    // every stage starts on a 1024-byte boundary: the 128-byte swizzle is a function of the address
    static constexpr uint32_t kStageBytes =
        (kMatrices * kATileBytes + kBTileBytes + (kMatrices + 1u) * kScaleBlockBytes + 1023u) / 1024u * 1024u;
    static constexpr uint32_t kStagesRaw = kSmemBudget / kStageBytes;
    static constexpr uint32_t kStages = kStagesRaw > kMaxStages ? kMaxStages : kStagesRaw;
    static constexpr uint32_t kAccColumns = kMatrices * N_TILE;
    static constexpr uint32_t kAccStages = (2u * kAccColumns + 16u <= 512u) ? 2u : 1u;
    static constexpr uint32_t kScaleColumns = 4u * (kMatrices + 1u);
    static constexpr uint32_t kColumnsUsed = kAccStages * kAccColumns + kScaleColumns;
    static constexpr uint32_t kTmemColumns = kColumnsUsed <= 32u ? 32u : kColumnsUsed <= 64u ? 64u : kColumnsUsed <= 128u ? 128u : kColumnsUsed <= 256u ? 256u : 512u;
    static constexpr uint32_t kSmemBytes = kStages * kStageBytes + 1024u /* alignment slack */ + 256u /* barriers */;
    static_assert(N_TILE % 16u == 0u && N_TILE >= 16u && N_TILE <= 128u, "token tile");
    static_assert(kStages >= 3u, "pipeline too shallow");
};

struct Barriers {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint64_t drain;
    uint32_t tmem_base;
    uint32_t abort;
};

template <bool GATE_UP, uint32_t N_TILE>
__global__ void __launch_bounds__(kThreads, 1) experts_tc_kernel(ExpertLaunch p, TileList list) {
    using C = Config<GATE_UP, N_TILE>;
    extern __shared__ unsigned char smem_raw[];
    // operand tiles need 1024-byte alignment for the 128-byte swizzle
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~uintptr_t(1023u));
    Barriers* bars = reinterpret_cast<Barriers*>(smem + C::kStages * C::kStageBytes);
    volatile uint32_t* abort_flag = &bars->abort;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t H = p.g.hidden_size, I = p.g.intermediate_size;
    const uint32_t K = p.g.routed_k + p.g.always_count;
    const uint32_t k_dim = GATE_UP ? H : I;
    const uint32_t out_rows = GATE_UP ? I : H;
    const uint32_t k_blocks = (k_dim + kBlockK - 1u) / kBlockK;
    const uint32_t m_tiles = (out_rows + kBlockM - 1u) / kBlockM;
    const uint32_t pair_count = *list.count;
    const uint32_t tile_count = pair_count * m_tiles;

    // ---- one-time setup ---------------------------------------------------------------------
    if (threadIdx.x == 0u) {
        for (uint32_t s = 0; s < C::kStages; s++) {
            mbar_init(&bars->full[s], kProducerThreads);
            mbar_init(&bars->empty[s], 1u);
        }
        for (uint32_t a = 0; a < 2u; a++) {
            mbar_init(&bars->acc_full[a], 1u);
            mbar_init(&bars->acc_empty[a], kEpilogueThreads);
        }
        mbar_init(&bars->drain, 1u);
        bars->abort = 0u;
        fence_mbar_init();
    }
    // the padding halves of the 4-bit slots are never written by the copies: clear them once
    for (uint32_t i = threadIdx.x; i < C::kStages * C::kStageBytes / 16u; i += kThreads)
        reinterpret_cast<uint4*>(smem)[i] = make_uint4(0u, 0u, 0u, 0u);
    fence_proxy_async();
    __syncthreads();
    if (warp == 4u) {
        tmem_alloc(&bars->tmem_base, C::kTmemColumns);
        tmem_relinquish();
        tc_fence_before();
    }
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_base;
    const uint32_t tmem_scales = tmem_base + C::kAccStages * C::kAccColumns;

    if (warp >= 5u && warp <= 8u) {
        // ===== operand producers: cp.async into the swizzled tiles, completion arrives on `full` =====
        const uint32_t pt = threadIdx.x - 160u;  // 0..127
        uint32_t it = 0u;
        bool alive = true;
        for (uint32_t tile = blockIdx.x; tile < tile_count && alive; tile += gridDim.x) {
            const uint32_t pair = list.tiles[tile / m_tiles];
            const uint32_t m_tile = tile % m_tiles;
            const uint32_t expert = pair >> 16, n_tile = pair & 0xffffu;
            const uint32_t e_begin = p.work.expert_offsets[expert], e_end = p.work.expert_offsets[expert + 1u];
            const uint32_t first = e_begin + n_tile * N_TILE;
            const uint32_t valid = min(N_TILE, e_end - first);
            const ExpertPtrs ptrs = p.work.experts[expert];
            // activation rows this thread gathers: token (pt / 8) + 16 i of the tile
            // (gate/up reads the token's hidden row, down the route's own row)
            uint32_t code_rows[N_TILE / 16u];
#pragma unroll
            for (uint32_t i = 0; i < N_TILE / 16u; i++) {
                const uint32_t n = (pt >> 3) + 16u * i;
                const uint32_t ri = n < valid ? __ldg(p.work.grouped_routes + first + n) : 0u;
                code_rows[i] = GATE_UP ? ri / K : ri;
            }
            uint32_t scale_row = 0u;  // activation row whose scale word this thread gathers
            if (pt < valid) {
                const uint32_t ri = __ldg(p.work.grouped_routes + first + pt);
                scale_row = GATE_UP ? ri / K : ri;
            }
            const uint32_t row0 = m_tile * kBlockM;
            for (uint32_t kb = 0; kb < k_blocks; kb++, it++) {
                const uint32_t slot = it % C::kStages;
                if (!mbar_wait(&bars->empty[slot], ((it / C::kStages) & 1u) ^ 1u, abort_flag)) {
                    alive = false;
                    break;
                }
                unsigned char* stage = smem + slot * C::kStageBytes;
                const uint32_t k_left = k_dim - kb * kBlockK;  // elements of K from this block on
                // weights: 8-byte pieces of 16 codes into the low half of 16-byte slots
#pragma unroll
                for (uint32_t mx = 0; mx < C::kMatrices; mx++) {
                    const uint32_t a_base = smem_u32(stage + mx * kATileBytes);
                    const uint8_t* wbase = ptrs.w[mx];
#pragma unroll
                    for (uint32_t i = 0; i < 8u; i++) {
                        const uint32_t r = (pt >> 3) + 16u * i, c = pt & 7u;
                        const bool ok = (row0 + r < out_rows) && (c * 16u < k_left);
                        const uint8_t* src = ok ? wbase + (size_t)(row0 + r) * (k_dim / 2u) + kb * 64u + c * 8u : wbase;
                        cp_async_8(a_base + swizzle128_offset(r, c), src, ok ? 8u : 0u);
                    }
                }
                // activations: 16-byte pieces of 16 E4M3 codes, rows gathered through the route list
                const uint32_t b_base = smem_u32(stage + C::kMatrices * kATileBytes);
#pragma unroll
                for (uint32_t i = 0; i < N_TILE / 16u; i++) {
                    const uint32_t n = (pt >> 3) + 16u * i, c = pt & 7u;
                    const bool ok = (n < valid) && (c * 16u < k_left);
                    const uint8_t* src = ok ? p.act_q + (size_t)code_rows[i] * k_dim + kb * kBlockK + c * 16u : p.act_q;
                    cp_async_16(b_base + swizzle128_offset(n, c), src, ok ? 16u : 0u);
                }
                // scales: the derived copy already has the 32x16-byte layout tcgen05.cp reads, one 512-byte
                // block per (row tile, K block); token scales are gathered four bytes (one K block) a row
                unsigned char* sf = stage + C::kMatrices * kATileBytes + C::kBTileBytes;
                if (pt < 32u * C::kMatrices) {
                    const uint32_t mx = pt >> 5, l = pt & 31u;
                    const uint8_t* src = ptrs.ts[mx] + ((size_t)m_tile * k_blocks + kb) * kScaleBlockBytes + l * 16u;
                    cp_async_16(smem_u32(sf + mx * kScaleBlockBytes + l * 16u), src, 16u);
                }
                if (pt < N_TILE) {
                    const bool ok = pt < valid;
                    const uint32_t* src = ok ? p.act_e8m0 + (size_t)scale_row * k_blocks + kb : p.act_e8m0;
                    cp_async_4(smem_u32(sf + C::kMatrices * kScaleBlockBytes + (pt & 31u) * 16u + (pt >> 5) * 4u), src,
                               ok ? 4u : 0u);
                }
                // the arrival fires when this thread's copies have landed; the thread moves on at once
                cp_async_arrive_noinc(&bars->full[slot]);
            }
        }
        cp_async_wait_all();  // nothing of this thread may still be landing when the CTA retires
    } else if (warp == 4u) {
        // ===== MMA issue (one elected lane) ======================================================
        if (elect_one()) {
            const uint32_t idesc = idesc_mxf8f6f4(kFmtE2M1, kFmtE4M3, kBlockM, N_TILE);
            uint32_t it = 0u, acc_it = 0u;
            bool alive = true;
            for (uint32_t tile = blockIdx.x; tile < tile_count && alive; tile += gridDim.x, acc_it++) {
                const uint32_t acc = acc_it % C::kAccStages;
                if (!mbar_wait(&bars->acc_empty[acc], ((acc_it / C::kAccStages) & 1u) ^ 1u, abort_flag)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * C::kAccColumns;
                for (uint32_t kb = 0; kb < k_blocks; kb++, it++) {
                    const uint32_t slot = it % C::kStages;
                    if (!mbar_wait(&bars->full[slot], (it / C::kStages) & 1u, abort_flag)) {
                        alive = false;
                        break;
                    }
                    tc_fence_after();
                    fence_proxy_async();  // the stage was written through the generic proxy
                    const uint32_t stage = smem_u32(smem + slot * C::kStageBytes);
                    const uint32_t sf = stage + C::kMatrices * kATileBytes + C::kBTileBytes;
#pragma unroll
                    for (uint32_t mx = 0; mx <= C::kMatrices; mx++)
                        tc_copy_scales(tmem_scales + 4u * mx, desc_scale_block(sf + mx * kScaleBlockBytes));
                    const uint64_t b_desc = desc_k_major_sw128(stage + C::kMatrices * kATileBytes);
                    const uint32_t groups = min(4u, (k_dim - kb * kBlockK) / 32u);
                    for (uint32_t j = 0; j < groups; j++) {
                        const uint32_t id = idesc_with_scale_ids(idesc, j, j);
#pragma unroll
                        for (uint32_t mx = 0; mx < C::kMatrices; mx++) {
                            const uint64_t a_desc = desc_k_major_sw128(stage + mx * kATileBytes);
                            // a K step of 32 elements is 32 bytes: two 16-byte units of the start address
                            tc_mma_block_scaled(d_tmem + mx * N_TILE, a_desc + 2u * j, b_desc + 2u * j, id,
                                                tmem_scales + 4u * mx, tmem_scales + 4u * C::kMatrices,
                                                (kb | j) != 0u ? 1u : 0u);
                        }
                    }
                    tc_commit(&bars->empty[slot]);  // the stage may be refilled once these MMAs retire
                }
                if (alive) tc_commit(&bars->acc_full[acc]);
            }
            // nothing of this CTA may still be using tensor memory when it is released
            tc_commit(&bars->drain);
            mbar_wait(&bars->drain, 0u, abort_flag);
        }
        __syncwarp();
    } else {
        // ===== epilogue: TMEM -> registers -> global =============================================
        const uint32_t frame_words = K * (I / 2u) + K;
        uint32_t acc_it = 0u;
        for (uint32_t tile = blockIdx.x; tile < tile_count; tile += gridDim.x, acc_it++) {
            const uint32_t pair = list.tiles[tile / m_tiles];
            const uint32_t m_tile = tile % m_tiles;
            const uint32_t expert = pair >> 16, n_tile = pair & 0xffffu;
            const uint32_t e_begin = p.work.expert_offsets[expert], e_end = p.work.expert_offsets[expert + 1u];
            const uint32_t first = e_begin + n_tile * N_TILE;
            const uint32_t valid = min(N_TILE, e_end - first);
            const uint32_t acc = acc_it % C::kAccStages;
            if (!mbar_wait(&bars->acc_full[acc], (acc_it / C::kAccStages) & 1u, abort_flag)) break;
            tc_fence_after();
            const uint32_t row = m_tile * kBlockM + warp * 32u + lane;
            const bool row_ok = row < out_rows;
            const uint32_t lane_addr = tmem_base + ((warp * 32u) << 16) + acc * C::kAccColumns;
            for (uint32_t c0 = 0; c0 < N_TILE; c0 += 16u) {
                if (c0 >= valid) break;  // uniform: no token of this tile lives in the remaining columns
                uint32_t d0[16], d1[16];
                tmem_ld16(lane_addr + c0, d0);
                if (GATE_UP) tmem_ld16(lane_addr + N_TILE + c0, d1);
                tmem_ld_wait();
#pragma unroll
                for (uint32_t j = 0; j < 16u; j++) {
                    const uint32_t n = c0 + j;
                    if (n >= valid || !row_ok) continue;
                    const uint32_t ri = __ldg(p.work.grouped_routes + first + n);
                    if (GATE_UP) {
                        const float a = nvmoe_swiglu(__uint_as_float(d0[j]), __uint_as_float(d1[j]), p.g.swiglu_limit,
                                                     p.g.swiglu_alpha, p.g.swiglu_up_offset);
                        uint16_t* out = reinterpret_cast<uint16_t*>(p.intermediates + (size_t)(ri / K) * frame_words) +
                                        (size_t)(ri % K) * I;
                        out[row] = (uint16_t)nvmoe_f32_to_bf16(a);
                    } else {
                        const float weight = nvmoe_bf16_to_f32(__ldg(p.routes + ri) >> 16);
                        p.outputs[(size_t)ri * H + row] = (uint16_t)nvmoe_f32_to_bf16(__fmul_rn(__uint_as_float(d0[j]), weight));
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(&bars->acc_empty[acc]);
        }
    }

    // ---- teardown -------------------------------------------------------------------------------
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0u) raise_status(p.status, NVMOE_STATUS_WAIT_EXPIRED);
    if (warp == 4u) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::kTmemColumns);
    }
}

// (expert, token tile) pairs in expert order; one block, experts <= 4096
__global__ void __launch_bounds__(1024) build_tiles_kernel(const uint32_t* expert_offsets, uint32_t num_experts,
                                                          uint32_t n_tile, uint32_t* tiles, uint32_t* count) {
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
            uint32_t s = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                uint32_t n = __shfl_up_sync(0xffffffffu, s, o);
                if ((int)lane >= o) s += n;
            }
            warp_sums[lane] = s - v;
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

// Re-tiles the packaged [rows][cols/32] scale bytes of one expert matrix into 512-byte blocks, one
// per (128-row tile, 128-column block): row r of the tile sits at (r % 32) * 16 + (r / 32) * 4 and
// holds the four scales of the block; positions past the matrix edge hold 127 (1.0) and are never
// multiplied with anything but zeros.  A block re-tiles only when the stamp differs.
__global__ void __launch_bounds__(128) derive_scales_kernel(const ExpertPtrs* experts, const uint64_t* stamps,
                                                           uint32_t matrices, uint32_t rows, uint32_t cols) {
    const uint32_t m_tiles = (rows + kBlockM - 1u) / kBlockM, k_blocks = (cols + kBlockK - 1u) / kBlockK;
    const uint32_t e = blockIdx.x / (matrices * m_tiles);
    const uint32_t mx = (blockIdx.x / m_tiles) % matrices, m_tile = blockIdx.x % m_tiles;
    const ExpertPtrs ptrs = experts[e];
    if (ptrs.w[0] == nullptr || ptrs.ts[mx] == nullptr) return;
    const uint64_t* stamp = stamps + ((size_t)e * matrices + mx) * 2u;
    if (stamp[0] == (uint64_t)(uintptr_t)ptrs.s[mx] && stamp[1] == ptrs.gen[mx]) return;
    const uint32_t r = threadIdx.x, row = m_tile * kBlockM + r, row_bytes = cols / 32u;
    uint8_t* out = const_cast<uint8_t*>(ptrs.ts[mx]) + (size_t)m_tile * k_blocks * kScaleBlockBytes + (r & 31u) * 16u + (r >> 5) * 4u;
    for (uint32_t kb = 0; kb < k_blocks; kb++) {
        uint32_t word = 0x7f7f7f7fu;
        if (row < rows) {
            word = 0u;
            for (uint32_t j = 0; j < 4u; j++) {
                const uint32_t c = kb * 4u + j;
                word |= (uint32_t)(c < row_bytes ? ptrs.s[mx][(size_t)row * row_bytes + c] : 127u) << (8u * j);
            }
        }
        *reinterpret_cast<uint32_t*>(out + (size_t)kb * kScaleBlockBytes) = word;
    }
}

__global__ void commit_stamps_kernel(const ExpertPtrs* experts, uint64_t* stamps, uint32_t matrices, uint32_t count) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const ExpertPtrs ptrs = experts[i / matrices];
    const uint32_t mx = i % matrices;
    if (ptrs.w[0] == nullptr) return;
    stamps[(size_t)i * 2u] = (uint64_t)(uintptr_t)ptrs.s[mx];
    stamps[(size_t)i * 2u + 1u] = ptrs.gen[mx];
}

int g_sm_count[16] = {0};

template <bool GATE_UP, uint32_t N_TILE>
void launch_n(const ExpertLaunch& p, cudaStream_t stream) {
    using C = Config<GATE_UP, N_TILE>;
    int dev = 0;
    cudaGetDevice(&dev);
    if (g_sm_count[dev & 15] == 0) cudaDeviceGetAttribute(&g_sm_count[dev & 15], cudaDevAttrMultiProcessorCount, dev);
    experts_tc_kernel<GATE_UP, N_TILE><<<g_sm_count[dev & 15], kThreads, C::kSmemBytes, stream>>>(
        p, TileList{p.tile_list, p.tile_count});
}

template <bool GATE_UP>
void launch(const ExpertLaunch& p, cudaStream_t stream) {
    switch (tc_token_tile(p)) {
        case 16u: launch_n<GATE_UP, 16u>(p, stream); break;
        case 32u: launch_n<GATE_UP, 32u>(p, stream); break;
        case 64u: launch_n<GATE_UP, 64u>(p, stream); break;
        default: launch_n<GATE_UP, 128u>(p, stream); break;
    }
}

template <bool GATE_UP, uint32_t N_TILE>
void configure_one() {
    cudaFuncSetAttribute(experts_tc_kernel<GATE_UP, N_TILE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)Config<GATE_UP, N_TILE>::kSmemBytes);
}

}  // namespace

bool tc_shape_supported(const nvmoe_geometry& g) {
    return g.hidden_size % 32u == 0u && g.intermediate_size % 32u == 0u && g.act_block % 32u == 0u;
}

bool tc_enabled_by_default() { return false; }

uint32_t tc_token_tile(const ExpertLaunch& p) {
    // tokens per expert if routing were uniform; skew only adds token tiles
    const uint32_t routes = p.tokens * (p.g.routed_k + p.g.always_count);
    const uint32_t per_expert = (routes + p.work.num_experts - 1u) / p.work.num_experts;
    return per_expert <= 12u ? 16u : per_expert <= 24u ? 32u : per_expert <= 48u ? 64u : 128u;
}

size_t tc_derived_scale_bytes(uint32_t rows, uint32_t cols) {
    return (size_t)((rows + kBlockM - 1u) / kBlockM) * ((cols + kBlockK - 1u) / kBlockK) * kScaleBlockBytes;
}

void launch_derive_scales_tc(const ExpertLaunch& p, bool gate_up, cudaStream_t stream) {
    const uint32_t matrices = gate_up ? 2u : 1u;
    const uint32_t rows = gate_up ? p.g.intermediate_size : p.g.hidden_size;
    const uint32_t cols = gate_up ? p.g.hidden_size : p.g.intermediate_size;
    const uint32_t m_tiles = (rows + kBlockM - 1u) / kBlockM;
    derive_scales_kernel<<<p.work.num_experts * matrices * m_tiles, 128, 0, stream>>>(p.work.experts, p.scale_stamps,
                                                                                      matrices, rows, cols);
    const uint32_t count = p.work.num_experts * matrices;
    commit_stamps_kernel<<<(count + 127u) / 128u, 128, 0, stream>>>(p.work.experts, p.scale_stamps, matrices, count);
}

void launch_build_tiles_tc(const ExpertLaunch& p, cudaStream_t stream) {
    // tile_list holds routes / 16 + experts + 1 entries: enough for any token tile size
    build_tiles_kernel<<<1, 1024, 0, stream>>>(p.work.expert_offsets, p.work.num_experts, tc_token_tile(p),
                                               p.tile_list, p.tile_count);
}

void tc_configure_kernels() {
    configure_one<true, 16u>();
    configure_one<true, 32u>();
    configure_one<true, 64u>();
    configure_one<true, 128u>();
    configure_one<false, 16u>();
    configure_one<false, 32u>();
    configure_one<false, 64u>();
    configure_one<false, 128u>();
}

void launch_gate_up_tc(const ExpertLaunch& p, cudaStream_t stream) { launch<true>(p, stream); }
void launch_down_tc(const ExpertLaunch& p, cudaStream_t stream) { launch<false>(p, stream); }

}  // namespace nvmoe
