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
// Roles: warps 0-3 epilogue (TMEM lane quadrant = warp); warp 4 allocates TMEM and one of its lanes
// issues the scale copies and MMAs; one lane of warp 5 issues TMA loads of whole 128 x 128 boxes of
// weight codes through a per-expert tensor map (the template map with the expert's address patched in
// on the device; the padded 4-bit tensor-map type spreads the codes into the 16-byte slots the f8f6f4
// kinds read and applies the 128-byte swizzle); warps 6.. stage the token rows, the scales and any
// trailing partial K block with cp.async whose completion arrives on the stage's mbarrier without
// stalling the issuer.  Shapes the tensor map cannot describe (K % 64 != 0) move the weights with
// cp.async too: 8-byte pieces into the low half of the 16-byte slots.  Token rows are gathered
// through the expert-grouped route list (the permutation costs no pass of its own), and E8M0 scales
// come as ready 32x16-byte blocks (the layout tcgen05.cp expands into TMEM) from a derived copy of
// the packaged scale tensors that is rebuilt whenever a scale record's address or generation
// changes.  Stages are handed over with mbarriers; every wait is bounded (tcgen05.cuh).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include <cstring>

#include "experts_tc.cuh"
#include "tcgen05.cuh"

namespace nvmoe {
namespace {

using namespace tc;

constexpr uint32_t kBlockM = 128u;   // weight rows per tile
constexpr uint32_t kBlockK = 128u;   // K elements per pipeline stage = 4 MMAs of K = 32
constexpr uint32_t kFirstProducerThread = 192u;    // warps 0-3 epilogue, 4 MMA, 5 TMA, 6.. cp.async, then more epilogue warps
constexpr uint32_t kTmaBoxBytes = kBlockM * 64u;   // global bytes of one 128 x 128 box of 4-bit codes
constexpr uint32_t kATileBytes = kBlockM * 128u;   // one byte slot per element
constexpr uint32_t kScaleBlockBytes = 512u;        // 128 rows x 4 scale bytes
constexpr uint32_t kMaxStages = 8u;
constexpr uint32_t kWatchWarp = 2u;     // the epilogue warp that polls for a finished accumulator (not on the MMA or TMA warp's scheduler)

struct TileList {
    const uint32_t* tiles;   // (expert << 16) | token tile within the expert
    const uint32_t* count;   // number of entries
};

// ROW_PAIR (down only): a tile covers two 128-row tiles of the one weight matrix, handled as the two
// "matrices" of a stage exactly as gate and up are: two accumulators alternate (one MMA cannot follow
// another into the same accumulator at full rate) and the token tile is fetched once for 256 rows. Used
// for the wide token tiles of large batches; small batches keep 128-row tiles, which spread better
// over the SMs.
template <bool GATE_UP, uint32_t N_TILE, bool USE_TMA, bool ROW_PAIR>
struct Config {
    static_assert(!(GATE_UP && ROW_PAIR), "gate/up already holds two matrices a stage");
    static constexpr uint32_t kMatrices = (GATE_UP || ROW_PAIR) ? 2u : 1u;
    static constexpr uint32_t kSources = GATE_UP ? 2u : 1u;        // weight tensors (and tensor maps) per expert
    static constexpr uint32_t kTileRows = kMatrices / kSources * kBlockM;  // weight rows a tile covers
    // matrix mx of a stage = weight tensor source_of(mx), rows shifted by row_shift(mx)
    static constexpr uint32_t source_of(uint32_t mx) { return GATE_UP ? mx : 0u; }
    static constexpr uint32_t row_shift(uint32_t mx) { return ROW_PAIR ? mx * kBlockM : 0u; }
    // cp.async producers: one warp sustains only about one copy instruction every 60-130 cycles, so the
    // copies of a stage are spread over eight warps (with TMA for the weights: token rows on the first
    // four, scales on the other four)
    // With TMA two cp.async warps are left with the token scales and a trailing partial K block, and the
    // warps they free become epilogue warps: the epilogue (activation, rounding, re-quantisation: a
    // couple of hundred instructions per value) is what large token tiles wait for, and a warp only
    // issues one instruction at a time. Epilogue warps come in groups of four, one per quadrant of
    // tensor-memory lanes (a warp reads the quadrant warp_id % 4); the groups share out a tile's columns.
    static constexpr uint32_t kProducerWarps = USE_TMA ? 2u : 8u;
    static constexpr uint32_t kProducerThreads = 32u * kProducerWarps;
    static constexpr uint32_t kRowsPerPass = kProducerThreads / 8u;  // eight threads cover the 128 bytes of one row
    static constexpr uint32_t kEpilogueGroups = USE_TMA ? 3u : 1u;
    static constexpr uint32_t kEpilogueThreads = 128u * kEpilogueGroups;
    static constexpr uint32_t kFirstExtraEpilogueWarp = 6u + kProducerWarps;  // a multiple of four
    static constexpr uint32_t kThreads = kFirstProducerThread + kProducerThreads + 128u * (kEpilogueGroups - 1u);
    static_assert(kFirstExtraEpilogueWarp % 4u == 0u || kEpilogueGroups == 1u, "extra epilogue warps keep warp % 4 = quadrant");
    static constexpr uint32_t kBTileBytes = N_TILE * 128u;
    // A stage holds kSub K blocks, each with its own operand tiles and scale blocks. Down moves one
    // matrix, so a stage of one block would carry half the bytes of a gate/up stage for the same
    // barrier traffic and issue overhead: it takes two blocks a stage.
    static constexpr uint32_t kSub = kMatrices == 2u ? 1u : 2u;
    // Shared memory is three regions, each an array over (slot, K block of the stage): the weight tiles, the token
    // tiles (both need 1024-byte alignment: the 128-byte swizzle is a function of the address) and the scale blocks.
    // Kept apart, nothing has to be padded to a 1024-byte boundary per K block, and the throughput of the pipeline is
    // the bytes its slots hold in flight: for the narrow down tiles the padding was the difference between five
    // slots and six.
    static constexpr uint32_t kScaleStride = kSources * kScaleBlockBytes;      // between K blocks of the derived weight scales
    static constexpr uint32_t kABytes = kMatrices * kATileBytes;               // weight tiles of one K block
    // weight scale blocks, then the token scale block: 32 entries of 16 bytes, entry n % 32 holding token n's scales.
    // A tile of 16 tokens fills half of it; the copy into tensor memory still reads 512 bytes, the second half
    // being whatever follows in shared memory (the next block's scales, or the barriers): scales of token columns
    // that do not exist.
    static constexpr uint32_t kSfBytes = kMatrices * kScaleBlockBytes + (N_TILE <= 16u ? kScaleBlockBytes / 2u : kScaleBlockBytes);
    static constexpr uint32_t kStageBytes = kSub * (kABytes + kBTileBytes + kSfBytes);
    static constexpr uint32_t kBarrierBytes = 256u;
    // The arrays start at the first 1024-byte boundary of the dynamic shared memory. Room for that round-up is set
    // aside unless leaving it out buys another slot; the kernel then insists on a base that is aligned already
    // (it is when the kernel has no static shared memory) and does nothing, with NVMOE_STATUS_INTERNAL, otherwise.
    static constexpr uint32_t kSmemMax = 227u * 1024u;
    static constexpr uint32_t stages_for(uint32_t slack) {
        const uint32_t n = (kSmemMax - kBarrierBytes - slack) / kStageBytes;
        return n > kMaxStages ? kMaxStages : n;
    }
    static constexpr bool kNeedsAlignedBase = stages_for(0u) > stages_for(1024u);
    static constexpr uint32_t kStages = stages_for(kNeedsAlignedBase ? 0u : 1024u);
    static constexpr uint32_t kBlocks = kStages * kSub;                        // K blocks resident at once
    static constexpr uint32_t kBRegion = kBlocks * kABytes;                    // offset of the token tiles
    static constexpr uint32_t kSfRegion = kBRegion + kBlocks * kBTileBytes;    // offset of the scale blocks
    static constexpr uint32_t kAccColumns = kMatrices * N_TILE;
    static constexpr uint32_t kAccStages = (2u * kAccColumns + 16u <= 512u) ? 2u : 1u;
    static constexpr uint32_t kScaleColumns = 4u * (kMatrices + 1u);
    static constexpr uint32_t kColumnsUsed = kAccStages * kAccColumns + kScaleColumns;
    static constexpr uint32_t kTmemColumns = kColumnsUsed <= 32u ? 32u : kColumnsUsed <= 64u ? 64u : kColumnsUsed <= 128u ? 128u : kColumnsUsed <= 256u ? 256u : 512u;
    static constexpr uint32_t kSmemBytes = kStages * kStageBytes + (kNeedsAlignedBase ? 0u : 1024u) + kBarrierBytes;
    static_assert(N_TILE % 16u == 0u && N_TILE >= 16u && N_TILE <= 128u, "token tile");
    static_assert(kBTileBytes % 1024u == 0u && kABytes % 1024u == 0u, "operand tiles keep their 1024-byte alignment");
    static_assert(kStages >= 3u, "pipeline too shallow");
};

// SwiGLU of the tensor path: the same expression and roundings as nvmoe_swiglu (accumulators rounded
// to bf16, clamp, g / (1 + exp(-alpha g)) * (u + offset), result rounded to bf16) with the hardware's
// approximate exponential and reciprocal (a few units in the last place of f32, far below the bf16
// rounding that follows) instead of the pinned software forms: a wide token tile spends more issue
// slots on its epilogue than on its MMAs, and the pinned forms cost several times as many.
// Returns the bf16 bits. The CUDA-core path keeps the pinned forms.
__device__ __forceinline__ uint32_t swiglu_bf16_bits(float gate_acc, float up_acc, float limit, float alpha, float up_offset) {
    float g = __bfloat162float(__float2bfloat16_rn(gate_acc));
    float u = __bfloat162float(__float2bfloat16_rn(up_acc));
    if (limit > 0.0f) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
    }
    const float act = __fdividef(g, 1.0f + __expf(-alpha * g)) * (u + up_offset);
    return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(act));
}

struct Barriers {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint64_t drain;
    uint32_t tmem_base;
    uint32_t abort;
    uint32_t format[kMaxStages];  // kFormat* of the weights staged in each slot (written before the slot's arrival)
    uint32_t acc_ready[2];        // the verdict of the epilogue warp that watches acc_full, for the others
};

// TRACE compiles the diagnostics in (cycle counters of CTA 0, per-CTA global-timer stamps): the
// instantiation that runs unless a plan's trace was armed has none of them in its loops.
template <bool GATE_UP, uint32_t N_TILE, bool USE_TMA, bool ROW_PAIR, bool TRACE>
__global__ void __launch_bounds__((Config<GATE_UP, N_TILE, USE_TMA, ROW_PAIR>::kThreads), 1)
    experts_tc_kernel(ExpertLaunch p, TileList list) {
    using C = Config<GATE_UP, N_TILE, USE_TMA, ROW_PAIR>;
    const long long wait_limit = p.wait_cycles;
    constexpr uint32_t kProducerThreads = C::kProducerThreads, kRowsPerPass = C::kRowsPerPass;
    extern __shared__ unsigned char smem_raw[];
    // operand tiles need 1024-byte alignment for the 128-byte swizzle
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~uintptr_t(1023u));
    Barriers* bars = reinterpret_cast<Barriers*>(smem + C::kStages * C::kStageBytes);
    static_assert(sizeof(Barriers) <= C::kBarrierBytes, "barrier block");
    volatile uint32_t* abort_flag = &bars->abort;
    if (C::kNeedsAlignedBase && smem != smem_raw) {  // (uniform) no room was set aside for the round-up
        grid_dependency_sync();
        if (threadIdx.x == 0u) raise_status(p.status, NVMOE_STATUS_INTERNAL);
        return;
    }

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t H = p.g.hidden_size, I = p.g.intermediate_size;
    const uint32_t K = p.g.routed_k + p.g.always_count;
    const uint32_t k_dim = GATE_UP ? H : I;
    const uint32_t out_rows = GATE_UP ? I : H;
    const uint32_t k_blocks = (k_dim + kBlockK - 1u) / kBlockK;
    const uint32_t k_stages = (k_blocks + C::kSub - 1u) / C::kSub;
    const uint32_t m_tiles = (out_rows + C::kTileRows - 1u) / C::kTileRows;   // tiles along the weight rows
    const uint32_t row_tiles = (out_rows + kBlockM - 1u) / kBlockM;           // 128-row tiles (scale blocks are kept per these)
    // the derived scale blocks of matrix mx of tile m_tile (a second half past the last rows borrows the first's:
    // its weights arrive as zeros)
    auto scale_tile = [&](uint32_t m_tile, uint32_t mx) {
        const uint32_t t = ROW_PAIR ? 2u * m_tile + mx : m_tile;
        return t < row_tiles ? t : t - 1u;
    };
    // cycle counters of CTA 0, one writer per role (diagnostics; words 16.. of the tile-count block)
    uint64_t* trace = reinterpret_cast<uint64_t*>(const_cast<uint32_t*>(list.count) + 16) + (GATE_UP ? 0 : 12);
    if (TRACE && blockIdx.x == 0u && threadIdx.x == 0u) trace[8] = global_timer_ns();  // kernel entry of CTA 0

    // ---- one-time setup ---------------------------------------------------------------------
    if (threadIdx.x == 0u) {
        for (uint32_t s = 0; s < C::kStages; s++) {
            mbar_init(&bars->full[s], kProducerThreads + (USE_TMA ? 1u : 0u));
            mbar_init(&bars->empty[s], 1u);
        }
        for (uint32_t a = 0; a < 2u; a++) {
            mbar_init(&bars->acc_full[a], 1u);
            mbar_init(&bars->acc_empty[a], C::kEpilogueThreads);
        }
        mbar_init(&bars->drain, 1u);
        bars->abort = 0u;
        fence_mbar_init();
    }
    // (The padding halves of the 4-bit slots, the scale rows past the token tile and whatever else the
    // copies never write stay as they were found: the MMA does not read them. Checked by filling the
    // stages with 0xff first; rows and columns that are read but hold no data are written as zeros by the
    // copies themselves.)
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
    // everything above touched only this CTA's shared and tensor memory; what follows reads what the
    // kernels before this one wrote
    grid_dependency_sync();
    const uint32_t pair_count = *list.count;
    const uint32_t tile_count = pair_count * m_tiles;
    if (USE_TMA) {
        // The per-expert tensor maps were written to global memory by an earlier kernel. A thread block must
        // acquire such a map once before any of its threads hands it to the TMA unit; further uses by the
        // block need no fence. All threads share the maps out, so that the block pays one fence latency here
        // instead of one per map in the lane that issues the loads.
        for (uint32_t m = threadIdx.x; m < p.work.num_experts * C::kSources; m += blockDim.x) tensormap_acquire(p.tmaps + (size_t)m * 128u);
        if (threadIdx.x == 0u) tensormap_acquire(p.act_tmap);
        __syncthreads();
    }

    if (warp == 5u) {
        // ===== TMA issue (one lane): whole 128 x 128 boxes of weight codes, padded and swizzled by the unit =====
        if (USE_TMA && lane == 0u) {
            uint32_t slot = 0u, empty_parity = 1u;
            bool alive = true;
            // What the lane needs to know about a tile. The list entry of a tile is fetched two tiles ahead and
            // what hangs on it (the expert's offset, scale and tensor-map addresses) one tile ahead, so that the
            // chain of dependent loads is over by the time the tile starts: a lane that stalled on it at every
            // tile boundary would leave the memory pipe without new requests for about a microsecond per tile.
            // (The prefetch only loads: whatever is computed from a loaded value is computed when the tile
            // starts, because a thread stalls at the first instruction that needs a load's result.)
            struct Meta {
                uint32_t pair, m_tile, expert_begin, format;
                const uint8_t* ts[C::kSources];
            };
            auto entry_of = [&](uint32_t tile) {
                uint32_t pair = 0u;
                if (tile < tile_count) pair = __ldg(list.tiles + tile / m_tiles);
                return pair;
            };
            auto meta_of = [&](uint32_t tile, uint32_t pair, Meta& m) {
                m.pair = pair;
                m.m_tile = tile % m_tiles;
                const uint32_t expert = pair >> 16;
                m.expert_begin = __ldg(p.work.expert_offsets + expert);
                m.format = p.work.experts[expert].format;
#pragma unroll
                for (uint32_t src = 0; src < C::kSources; src++) m.ts[src] = p.work.experts[expert].ts[src];
            };
            Meta cur{}, nxt{};
            uint32_t pair_nxt = entry_of(blockIdx.x + gridDim.x);
            if (blockIdx.x < tile_count) meta_of(blockIdx.x, entry_of(blockIdx.x), cur);
            // (debug) leave out the very first arrival of CTA 0: its consumer's bounded wait must then give up
            bool withhold = (p.debug_flags & 1u) != 0u && blockIdx.x == 0u;
            uint32_t stage_it = 0u;  // stages this lane has gone through (stage n used slot n % kStages, phase n / kStages)
            for (uint32_t tile = blockIdx.x; tile < tile_count && alive; tile += gridDim.x) {
                const uint32_t pair_nxt2 = entry_of(tile + 2u * gridDim.x);
                if (tile + gridDim.x < tile_count) meta_of(tile + gridDim.x, pair_nxt, nxt);
                const uint32_t m_tile = cur.m_tile;
                const int row0 = (int)(m_tile * C::kTileRows);
                const uint8_t* maps = p.tmaps + (size_t)(cur.pair >> 16) * C::kSources * 128u;
                // first operand row of this token tile in the expert-grouped activation matrix
                const int token0 = (int)(cur.expert_begin + (cur.pair & 0xffffu) * N_TILE);
                const uint8_t* scale_blocks[C::kMatrices];
#pragma unroll
                for (uint32_t mx = 0; mx < C::kMatrices; mx++)
                    scale_blocks[mx] = cur.ts[C::source_of(mx)] + (size_t)scale_tile(m_tile, mx) * k_blocks * C::kScaleStride;
                for (uint32_t ks = 0; ks < k_stages; ks++) {
                    if (!mbar_wait(&bars->empty[slot], empty_parity, abort_flag, wait_limit)) {
                        alive = false;
                        break;
                    }
                    // whole K blocks of this stage come by TMA; a trailing partial one is staged by the cp.async warps
                    uint32_t whole = 0u, present = 0u;
#pragma unroll
                    for (uint32_t sub = 0; sub < C::kSub; sub++) {
                        whole += ((ks * C::kSub + sub + 1u) * kBlockK <= k_dim) ? 1u : 0u;
                        present += (ks * C::kSub + sub < k_blocks) ? 1u : 0u;
                    }
                    if (withhold) {
                        withhold = false;
                    } else {
                    // token rows (zeros past the edge of K) and weight scale blocks of every K block present
                    const uint32_t smem_base = smem_u32(smem);
                    // a box of one-byte elements brings twice the bytes of a box of packed 4-bit codes
                    const uint32_t box_bytes = cur.format == kFormatCompact ? kTmaBoxBytes : 2u * kTmaBoxBytes;
                    *reinterpret_cast<volatile uint32_t*>(&bars->format[slot]) = cur.format;
                    mbar_arrive_expect_tx(&bars->full[slot], whole * C::kMatrices * box_bytes +
                                                                 present * (C::kBTileBytes + C::kMatrices * kScaleBlockBytes));
                    for (uint32_t sub = 0; sub < present; sub++) {
                        const uint32_t kb = ks * C::kSub + sub;
                        const uint32_t block = slot * C::kSub + sub;  // index into the three shared-memory arrays
                        if (sub < whole) {
#pragma unroll
                            for (uint32_t mx = 0; mx < C::kMatrices; mx++)
                                tma_load_3d(smem_base + block * C::kABytes + mx * kATileBytes, maps + C::source_of(mx) * 128u, 0, (int)kb,
                                            row0 + (int)C::row_shift(mx), &bars->full[slot]);  // rows past the matrix: zeros
                        }
                        tma_load_2d(smem_base + C::kBRegion + block * C::kBTileBytes, p.act_tmap, (int)(kb * kBlockK), token0,
                                    &bars->full[slot]);
                        if (C::kSources == 2u) {
                            // the gate and the up block of this (row tile, K block) are neighbours in the derived copy
                            bulk_copy_g2s(smem_base + C::kSfRegion + block * C::kSfBytes, scale_blocks[0] + (size_t)kb * C::kScaleStride,
                                          2u * kScaleBlockBytes, &bars->full[slot]);
                        } else {
#pragma unroll
                            for (uint32_t mx = 0; mx < C::kMatrices; mx++)
                                bulk_copy_g2s(smem_base + C::kSfRegion + block * C::kSfBytes + mx * kScaleBlockBytes,
                                              scale_blocks[mx] + (size_t)kb * C::kScaleStride, kScaleBlockBytes, &bars->full[slot]);
                        }
                    }
                    }
                    stage_it++;
                    if (++slot == C::kStages) {
                        slot = 0u;
                        empty_parity ^= 1u;
                    }
                }
                cur = nxt;
                pair_nxt = pair_nxt2;
            }
            if (!alive) {
                // The pipeline was aborted with copies of this lane possibly still on their way into shared
                // memory: the CTA must not retire under them. Wait, bounded, on the stage barriers of the last
                // round this lane armed; a barrier that also lacks an aborted role's arrivals never completes,
                // and the time spent on it is the grace period instead.
                const uint32_t rounds = stage_it < C::kStages ? stage_it : C::kStages;
                for (uint32_t back = 1u; back <= rounds; back++) {
                    const uint32_t nth = stage_it - back;
                    mbar_wait_winddown(&bars->full[nth % C::kStages], (nth / C::kStages) & 1u, kWinddownCycles / C::kStages);
                }
            }
        }
    } else if (warp >= 6u && warp < 6u + C::kProducerWarps) {
        // ===== operand producers: cp.async into the swizzled tiles, completion arrives on `full` =====
        const uint32_t pt = threadIdx.x - kFirstProducerThread;  // 0..kProducerThreads-1
        const uint32_t my_r = pt >> 3, my_c = pt & 7u;  // this thread's row (plus kRowsPerPass i) and 16-element chunk
        constexpr uint32_t kTokenPasses = (N_TILE + kRowsPerPass - 1u) / kRowsPerPass;
        const uint32_t row_bytes = k_dim / 2u;
        // What a thread needs to know about a tile; the next tile's copy is fetched while the current
        // tile streams, so that the dependent loads (tile list -> offsets -> routes) never stall the pipe.
        struct Meta {
            const uint8_t* w[C::kMatrices];
            const uint8_t* ts[C::kMatrices];
            uint32_t code_rows[kTokenPasses];  // activation row of token my_r + kRowsPerPass i
            uint32_t scale_row;                // activation row of token pt
            uint32_t valid, m_tile, first, format;
        };
        auto load_meta = [&](uint32_t tile, Meta& m) {
            const uint32_t pair = __ldg(list.tiles + tile / m_tiles);
            m.m_tile = tile % m_tiles;
            const uint32_t expert = pair >> 16, n_tile = pair & 0xffffu;
            const uint32_t e_begin = __ldg(p.work.expert_offsets + expert), e_end = __ldg(p.work.expert_offsets + expert + 1u);
            const uint32_t first = e_begin + n_tile * N_TILE;
            m.valid = min(N_TILE, e_end - first);
            m.first = first;
            const ExpertPtrs* ptrs = p.work.experts + expert;
            m.format = ptrs->format;
#pragma unroll
            for (uint32_t mx = 0; mx < C::kMatrices; mx++) {
                m.w[mx] = ptrs->w[C::source_of(mx)];
                m.ts[mx] = ptrs->ts[C::source_of(mx)];
            }
            // the operand matrices are expert-grouped: token n of the tile is row first + n
#pragma unroll
            for (uint32_t i = 0; i < kTokenPasses; i++) m.code_rows[i] = first + my_r + kRowsPerPass * i;
            // (the thread that copies token n's scales is kProducerThreads - 65 - n: see the copy below)
            m.scale_row = first + (kProducerThreads - 65u - pt);
        };
        uint32_t it = 0u, slot = 0u, empty_parity = 1u;  // a fresh barrier passes a wait on parity 1
        long long trace_wait = 0;
        const long long trace_begin = TRACE ? clock64() : 0;
        const uint32_t my_dst = swizzle128_offset(my_r, my_c);
        bool alive = true;
        Meta cur, nxt;
        if (blockIdx.x < tile_count) load_meta(blockIdx.x, cur);
        for (uint32_t tile = blockIdx.x; tile < tile_count && alive; tile += gridDim.x) {
            if (tile + gridDim.x < tile_count) load_meta(tile + gridDim.x, nxt);
            // this thread's first weight row of each matrix of the tile; its other rows are kRowsPerPass apart
            const uint8_t* wcol[C::kMatrices];
            uint32_t rows_here[C::kMatrices];
            // a matrix of one-byte elements (pre-expanded or native FP8) has rows, and pieces of 16 elements, twice as long
            const bool bytes_form = cur.format != kFormatCompact;
            const uint32_t form_row_bytes = bytes_form ? 2u * row_bytes : row_bytes;
#pragma unroll
            for (uint32_t mx = 0; mx < C::kMatrices; mx++) {
                const uint32_t row0 = cur.m_tile * C::kTileRows + C::row_shift(mx);
                rows_here[mx] = row0 < out_rows ? min(kBlockM, out_rows - row0) : 0u;
                wcol[mx] = cur.w[mx] + (size_t)(row0 + my_r) * form_row_bytes + my_c * (bytes_form ? 16u : 8u);
            }
            const size_t row_step = (size_t)kRowsPerPass * form_row_bytes;
            for (uint32_t ks = 0; ks < k_stages; ks++, it++) {
                const long long w0 = TRACE ? clock64() : 0;
                if (!mbar_wait_warp(&bars->empty[slot], empty_parity, abort_flag, wait_limit)) {
                    alive = false;
                    break;
                }
                if (TRACE) trace_wait += clock64() - w0;
#pragma unroll
                for (uint32_t sub = 0; sub < C::kSub; sub++) {
                const uint32_t kb = ks * C::kSub + sub;
                if (kb >= k_blocks) break;  // the last stage of an odd count holds one block
                const uint32_t block = slot * C::kSub + sub;  // index into the three shared-memory arrays
                unsigned char* a_tiles = smem + block * C::kABytes;
                const uint32_t k_left = k_dim - kb * kBlockK;  // elements of K from this block on
                const bool chunk_ok = my_c * 16u < k_left;
                // weights: 8-byte pieces of 16 codes into the low half of 16-byte slots
                // (with TMA only the trailing partial K block comes this way)
                if (!USE_TMA || k_left < kBlockK) {
#pragma unroll
                for (uint32_t mx = 0; mx < C::kMatrices; mx++) {
                    const uint32_t a_dst = smem_u32(a_tiles + mx * kATileBytes) + my_dst;
                    const uint8_t* src = wcol[mx] + kb * (bytes_form ? 128u : 64u);
#pragma unroll
                    for (uint32_t i = 0; i < kBlockM / kRowsPerPass; i++) {
                        // rows my_r + kRowsPerPass i share (row & 7), so the swizzled offset only moves by whole rows
                        const bool ok = chunk_ok && (my_r + kRowsPerPass * i < rows_here[mx]);
                        if (bytes_form) {
                            cp_async_16(a_dst + i * (kRowsPerPass * 128u), ok ? src + i * row_step : cur.w[mx], ok ? 16u : 0u);
                        } else {
                            cp_async_8(a_dst + i * (kRowsPerPass * 128u), ok ? src + i * row_step : cur.w[mx], ok ? 8u : 0u);
                        }
                    }
                }
                }
                // activations: 16-byte pieces of 16 E4M3 codes (with TMA the whole tile is one box)
                const uint32_t b_dst = smem_u32(smem + C::kBRegion + block * C::kBTileBytes) + my_dst;
                if (!USE_TMA) {
#pragma unroll
                for (uint32_t i = 0; i < kTokenPasses; i++) {
                    const uint32_t n = my_r + kRowsPerPass * i;
                    if (n < N_TILE) {
                        const bool ok = chunk_ok && (n < cur.valid);
                        const uint8_t* src = ok ? p.act_q + (size_t)cur.code_rows[i] * k_dim + kb * kBlockK + my_c * 16u : p.act_q;
                        cp_async_16(b_dst + i * (kRowsPerPass * 128u), src, ok ? 16u : 0u);
                    }
                }
                }
                // scales: the derived copy already has the 32x16-byte layout tcgen05.cp reads, one 512-byte
                // block per (row tile, K block); token scales are gathered four bytes (one K block) a row
                unsigned char* sf = smem + C::kSfRegion + block * C::kSfBytes;
                // (threads from the far end of the producer group, so that with few tokens a tile these are not
                // the threads that carry the token rows)
                const uint32_t st = kProducerThreads - 1u - pt;
                if (!USE_TMA && st < 32u * C::kMatrices) {
                    const uint32_t mx = st >> 5, l = st & 31u;
                    const uint8_t* src = cur.ts[mx] + ((size_t)scale_tile(cur.m_tile, mx) * k_blocks + kb) * C::kScaleStride + l * 16u;
                    cp_async_16(smem_u32(sf + mx * kScaleBlockBytes + l * 16u), src, 16u);
                }
                if (USE_TMA) {
                    for (uint32_t n = pt; n < N_TILE; n += kProducerThreads) {
                        const bool ok = n < cur.valid;
                        const uint32_t* src = ok ? p.act_e8m0 + (size_t)(cur.first + n) * k_blocks + kb : p.act_e8m0;
                        cp_async_4(smem_u32(sf + C::kMatrices * kScaleBlockBytes + (n & 31u) * 16u + (n >> 5) * 4u), src,
                                   ok ? 4u : 0u);
                    }
                } else if (st >= 64u && st < 64u + N_TILE) {
                    const uint32_t n = st - 64u;
                    const bool ok = n < cur.valid;
                    const uint32_t* src = ok ? p.act_e8m0 + (size_t)cur.scale_row * k_blocks + kb : p.act_e8m0;
                    cp_async_4(smem_u32(sf + C::kMatrices * kScaleBlockBytes + (n & 31u) * 16u + (n >> 5) * 4u), src,
                               ok ? 4u : 0u);
                }
                }
                if (!USE_TMA && pt == 0u) *reinterpret_cast<volatile uint32_t*>(&bars->format[slot]) = cur.format;
                // the arrival fires when this thread's copies have landed; the thread moves on at once
                cp_async_arrive_noinc(&bars->full[slot]);
                if (++slot == C::kStages) {
                    slot = 0u;
                    empty_parity ^= 1u;
                }
            }
            cur = nxt;
        }
        cp_async_wait_all();  // nothing of this thread may still be landing when the CTA retires
        if (TRACE && blockIdx.x == 0u && pt == 0u) {
            trace[0] = (uint64_t)trace_wait;                    // producer: cycles waiting for a free stage
            trace[1] = (uint64_t)(clock64() - trace_begin);     // producer: cycles in its loop
        }
    } else if (warp == 4u) {
        // ===== MMA issue (one elected lane) ======================================================
        if (elect_one()) {
            // One thread feeds the tensor pipe, and a lone thread retires an instruction every few
            // cycles at best: everything that does not depend on the stage is computed once, the four
            // K steps of a stage are unrolled with compile-time descriptors offsets and scale ids.
            constexpr uint32_t kIdescCompact = idesc_mxf8f6f4(kFmtE2M1, kFmtE4M3, kBlockM, N_TILE);
            constexpr uint32_t kIdescBytes = idesc_mxf8f6f4(kFmtE4M3, kFmtE4M3, kBlockM, N_TILE);  // weights as E4M3 bytes
            // descriptor start addresses count 16 bytes
            const uint32_t base = smem_u32(smem);
            const uint64_t a_desc0 = desc_k_major_sw128(base);
            const uint64_t b_desc0 = desc_k_major_sw128(base + C::kBRegion);
            const uint64_t sf_desc0 = desc_scale_block(base + C::kSfRegion);
            const uint32_t tail_groups = (k_dim % kBlockK) / 32u;  // K steps of a trailing partial block, 0 = none
            const uint32_t sfb_tmem = tmem_scales + 4u * C::kMatrices;
            uint32_t it = 0u, acc_it = 0u, slot = 0u, full_parity = 0u;
            bool alive = true;
            long long trace_full = 0, trace_acc = 0;
            const long long trace_begin = TRACE ? clock64() : 0;
            if (TRACE && blockIdx.x == 0u) trace[9] = global_timer_ns();  // MMA loop begins
            const uint64_t cta_begin = (TRACE && p.cta_trace) ? global_timer_ns() : 0u;
            for (uint32_t tile = blockIdx.x; tile < tile_count && alive; tile += gridDim.x, acc_it++) {
                const uint32_t acc = acc_it % C::kAccStages;
                const long long a0 = TRACE ? clock64() : 0;
                if (!mbar_wait(&bars->acc_empty[acc], ((acc_it / C::kAccStages) & 1u) ^ 1u, abort_flag, wait_limit)) break;
                if (TRACE) trace_acc += clock64() - a0;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * C::kAccColumns;
                for (uint32_t ks = 0; ks < k_stages; ks++, it++) {
                    const long long f0 = TRACE ? clock64() : 0;
                    if (!mbar_wait(&bars->full[slot], full_parity, abort_flag, wait_limit)) {
                        alive = false;
                        break;
                    }
                    if (TRACE) trace_full += clock64() - f0;
                    tc_fence_after();
                    const uint32_t kIdesc = *reinterpret_cast<volatile uint32_t*>(&bars->format[slot]) == kFormatCompact ? kIdescCompact
                                                                                                                 : kIdescBytes;
#pragma unroll
                    for (uint32_t sub = 0; sub < C::kSub; sub++) {
                    const uint32_t kb = ks * C::kSub + sub;
                    if (kb >= k_blocks) break;
                    const uint32_t block = slot * C::kSub + sub;  // index into the three shared-memory arrays
                    const uint64_t a_desc = a_desc0 + (uint64_t)(block * (C::kABytes >> 4));
                    const uint64_t b_desc = b_desc0 + (uint64_t)(block * (C::kBTileBytes >> 4));
                    const uint64_t sf_desc = sf_desc0 + (uint64_t)(block * (C::kSfBytes >> 4));
#pragma unroll
                    for (uint32_t mx = 0; mx <= C::kMatrices; mx++)
                        tc_copy_scales(tmem_scales + 4u * mx, sf_desc + mx * (kScaleBlockBytes >> 4));
                    const uint32_t groups = (kb + 1u == k_blocks && tail_groups != 0u) ? tail_groups : 4u;
#pragma unroll
                    for (uint32_t j = 0; j < 4u; j++) {
                        if (j < groups) {
#pragma unroll
                            for (uint32_t mx = 0; mx < C::kMatrices; mx++) {
                                // a K step of 32 elements is 32 bytes: two 16-byte units of the start address
                                tc_mma_block_scaled(d_tmem + mx * N_TILE, a_desc + (mx * (kATileBytes >> 4) + 2u * j),
                                                    b_desc + 2u * j, kIdesc | (j << 4) | (j << 29), tmem_scales + 4u * mx,
                                                    sfb_tmem, j == 0u ? (kb != 0u ? 1u : 0u) : 1u);
                            }
                        }
                    }
                    }
                    tc_commit(&bars->empty[slot]);  // the stage may be refilled once these MMAs retire
                    if (++slot == C::kStages) {
                        slot = 0u;
                        full_parity ^= 1u;
                    }
                }
                if (alive) tc_commit(&bars->acc_full[acc]);
            }
            // Nothing of this CTA may still be reading shared memory or using tensor memory when they are
            // released: the commit arrives once every MMA and scale copy issued above has retired. This wait has
            // its own limit and does not look at the abort flag, which is already set on the give-up path.
            tc_commit(&bars->drain);
            mbar_wait_winddown(&bars->drain, 0u, kWinddownCycles);
            if (TRACE && p.cta_trace) {  // per-CTA diagnostics: loop begin, loop end, stages, SM id
                uint32_t smid;
                asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
                uint64_t* mine = p.cta_trace + (size_t)((GATE_UP ? 0u : gridDim.x) + blockIdx.x) * 4u;
                mine[0] = cta_begin;
                mine[1] = global_timer_ns();
                mine[2] = it;
                mine[3] = smid;
            }
            if (TRACE && blockIdx.x == 0u) {
                trace[2] = (uint64_t)trace_full;                 // MMA thread: cycles waiting for operands
                trace[3] = (uint64_t)trace_acc;                  // MMA thread: cycles waiting for a free accumulator
                trace[4] = (uint64_t)(clock64() - trace_begin);  // MMA thread: cycles in its loop
                trace[5] = it;                                   // stages consumed
                trace[10] = global_timer_ns();                   // MMA loop ends
            }
        }
        __syncwarp();
    } else {
        // ===== epilogue: TMEM -> registers -> global =============================================
        const uint32_t quad = warp & 3u;  // the quadrant of tensor-memory lanes this warp may read
        const uint32_t epilogue_group = warp < 4u ? 0u : (warp - C::kFirstExtraEpilogueWarp) / 4u + 1u;
        const uint32_t frame_words = K * (I / 2u) + K;
        uint32_t acc_it = 0u;
        long long trace_epi_wait = 0;
        const long long trace_begin = TRACE ? clock64() : 0;
        for (uint32_t tile = blockIdx.x; tile < tile_count; tile += gridDim.x, acc_it++) {
            const uint32_t pair = list.tiles[tile / m_tiles];
            const uint32_t m_tile = tile % m_tiles;
            const uint32_t expert = pair >> 16, n_tile = pair & 0xffffu;
            const uint32_t e_begin = p.work.expert_offsets[expert], e_end = p.work.expert_offsets[expert + 1u];
            const uint32_t first = e_begin + n_tile * N_TILE;
            const uint32_t valid = min(N_TILE, e_end - first);
            const uint32_t acc = acc_it % C::kAccStages;
            const long long e0 = TRACE ? clock64() : 0;
            // One warp watches the accumulator's barrier; the others sleep on a hardware barrier until it has a
            // verdict. A warp that polls takes issue slots from whatever shares its scheduler, and the epilogue warps
            // (three to a scheduler) wait through most of a tile beside the one thread that feeds the tensor pipe
            // and the one that issues the copies. Every epilogue warp reaches the hardware barrier in every round,
            // whatever the verdict, so none is left waiting there.
            if (warp == kWatchWarp) {
                const bool ready = mbar_wait_warp(&bars->acc_full[acc], (acc_it / C::kAccStages) & 1u, abort_flag, wait_limit);
                if (lane == 0u) *reinterpret_cast<volatile uint32_t*>(&bars->acc_ready[acc_it & 1u]) = ready ? 1u : 0u;
                __threadfence_block();
            }
            named_barrier(1u, C::kEpilogueThreads);
            if (*reinterpret_cast<volatile uint32_t*>(&bars->acc_ready[acc_it & 1u]) == 0u) break;
            if (TRACE) trace_epi_wait += clock64() - e0;
            tc_fence_after();
            const uint32_t row = m_tile * C::kTileRows + quad * 32u + lane;  // (with row pairs: of the first half)
            const bool row_ok = row < out_rows;
            const uint32_t lane_addr = tmem_base + ((quad * 32u) << 16) + acc * C::kAccColumns;
            // The epilogue groups share out a wide tile by 16-column chunks. A narrow tile (one or two chunks)
            // is shared out by sets of four tokens instead, every group reading the chunk: a tile of eight
            // tokens is then two groups' work side by side, not one group's in turn.
            constexpr bool kShareByFours = N_TILE <= 32u && C::kEpilogueGroups > 1u;
            for (uint32_t c0 = kShareByFours ? 0u : 16u * epilogue_group; c0 < N_TILE;
                 c0 += kShareByFours ? 16u : 16u * C::kEpilogueGroups) {
                if (c0 >= valid) break;  // uniform: no token of this tile lives in the remaining columns
                if (kShareByFours) {
                    // does any of this chunk's sets of four fall to this group? (uniform)
                    bool mine = false;
#pragma unroll
                    for (uint32_t g0 = 0; g0 < 16u; g0 += 4u)
                        mine = mine || (c0 + g0 < valid && ((c0 + g0) / 4u) % C::kEpilogueGroups == epilogue_group);
                    if (!mine) continue;
                }
                uint32_t d0[16], d1[16];
                tmem_ld16(lane_addr + c0, d0);
                if (C::kMatrices == 2u) tmem_ld16(lane_addr + N_TILE + c0, d1);  // up, or the second 128 rows
                // lane j < 16 works out where token c0 + j of the tile goes (and its route weight)
                // while the accumulators arrive; the sixteen results are then handed round by shuffles
                uint64_t my_row = 0u;
                float my_weight = 0.0f;
                uint32_t my_route = kUnboundSlot;
                if (lane < 16u && c0 + lane < valid) {
                    const uint32_t ri = __ldg(p.work.grouped_routes + first + c0 + lane);
                    // the row of the down stage's operand matrix that this route's activations go to
                    my_route = (GATE_UP && p.q_out != nullptr) ? __ldg(p.down_position + ri) : kUnboundSlot;
                    if (GATE_UP) {
                        my_row = reinterpret_cast<uint64_t>(reinterpret_cast<uint16_t*>(p.intermediates + (size_t)(ri / K) * frame_words) +
                                                            (size_t)(ri % K) * I);
                    } else if (p.partial_outputs != nullptr) {
                        my_row = reinterpret_cast<uint64_t>(p.partial_outputs + (size_t)ri * H);
                    } else {
                        my_row = reinterpret_cast<uint64_t>(p.outputs + (size_t)ri * H);
                        my_weight = nvmoe_bf16_to_f32(__ldg(p.routes + ri) >> 16);
                    }
                }
                tmem_ld_wait();
                const bool quantise = GATE_UP && p.q_out != nullptr;  // host: only with 32-row scale blocks
                // Four tokens at a time go through each step together, with no branch between them, so that
                // their instruction latencies overlap (the activation math is one long dependent chain per
                // value); columns past `valid` hold zeros and are only not stored.
#pragma unroll
                for (uint32_t g0 = 0; g0 < 16u; g0 += 4u) {
                    if (c0 + g0 >= valid) break;  // uniform
                    if (kShareByFours && ((c0 + g0) / 4u) % C::kEpilogueGroups != epilogue_group) continue;  // another group's
                    uint32_t bits[4];
#pragma unroll
                    for (uint32_t t = 0; t < 4u; t++) {
                        const uint32_t j = g0 + t;
                        if (GATE_UP) {
                            bits[t] = swiglu_bf16_bits(__uint_as_float(d0[j]), __uint_as_float(d1[j]), p.g.swiglu_limit,
                                                       p.g.swiglu_alpha, p.g.swiglu_up_offset);
                        } else {
                            const float weight = __shfl_sync(0xffffffffu, my_weight, j);
                            bits[t] = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(__fmul_rn(__uint_as_float(d0[j]), weight)));
                        }
                    }
                    if (!GATE_UP && p.partial_outputs != nullptr) {
                        // tensor-parallel form: the raw f32 sums over this participant's columns, weighted and rounded
                        // only after the participants' planes have been added
#pragma unroll
                        for (uint32_t t = 0; t < 4u; t++) {
                            float* out = reinterpret_cast<float*>(__shfl_sync(0xffffffffu, my_row, g0 + t));
                            if (c0 + g0 + t < valid && row_ok) out[row] = __uint_as_float(d0[g0 + t]);
                            if (ROW_PAIR && c0 + g0 + t < valid && row + kBlockM < out_rows) out[row + kBlockM] = __uint_as_float(d1[g0 + t]);
                        }
                        continue;
                    }
#pragma unroll
                    for (uint32_t t = 0; t < 4u; t++) {
                        uint16_t* out = reinterpret_cast<uint16_t*>(__shfl_sync(0xffffffffu, my_row, g0 + t));
                        if (c0 + g0 + t < valid && row_ok) out[row] = (uint16_t)bits[t];
                        if (ROW_PAIR) {  // the second accumulator holds the next 128 output rows of the same tokens
                            const float weight = __shfl_sync(0xffffffffu, my_weight, g0 + t);
                            const uint32_t second = (uint32_t)__bfloat16_as_ushort(
                                __float2bfloat16_rn(__fmul_rn(__uint_as_float(d1[g0 + t]), weight)));
                            if (c0 + g0 + t < valid && row + kBlockM < out_rows) out[row + kBlockM] = (uint16_t)second;
                        }
                    }
                    if (quantise) {
                        // the activation quantisation of the down stage, on the values just rounded to bf16: one
                        // power-of-two scale per 32 rows, which is exactly this warp's share of the tile
                        float m[4];
#pragma unroll
                        for (uint32_t t = 0; t < 4u; t++) m[t] = row_ok ? fabsf(nvmoe_bf16_to_f32(bits[t])) : 0.0f;
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
                            for (uint32_t t = 0; t < 4u; t++) m[t] = fmaxf(m[t], __shfl_xor_sync(0xffffffffu, m[t], o));
                        }
                        const uint32_t first_row = m_tile * C::kTileRows + quad * 32u;
                        const bool writes_scale = lane == 0u && first_row < out_rows;
#pragma unroll
                        for (uint32_t t = 0; t < 4u; t++) {
                            const uint32_t dp = __shfl_sync(0xffffffffu, my_route, g0 + t);
                            const float scale = nvmoe_rounded_fp8_scale(m[t]);
                            // 1 / scale, exact: the scale is a power of two with a biased exponent in [107, 247]
                            const float inv = __uint_as_float(0x7f000000u - __float_as_uint(scale));
                            const uint8_t q =
                                (uint8_t)__nv_cvt_float_to_fp8(nvmoe_bf16_to_f32(bits[t]) * inv, __NV_SATFINITE, __NV_E4M3);
                            if (dp != kUnboundSlot) {  // (lanes past `valid` and routes the down stage skips)
                                if (row_ok) p.q_out[(size_t)dp * I + row] = q;
                                if (writes_scale)
                                    reinterpret_cast<uint8_t*>(p.q_e8m0 + (size_t)dp * ((I + 127u) / 128u))[first_row / 32u] =
                                        (uint8_t)(nvmoe_f32_bits(scale) >> 23);
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(&bars->acc_empty[acc]);
        }
        if (TRACE && blockIdx.x == 0u && threadIdx.x == 0u) {
            trace[6] = (uint64_t)trace_epi_wait;                 // epilogue: cycles waiting for an accumulator
            trace[7] = (uint64_t)(clock64() - trace_begin);      // epilogue: cycles in its loop
        }
    }

    // ---- teardown -------------------------------------------------------------------------------
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0u) raise_status(p.status, NVMOE_STATUS_WAIT_EXPIRED);
    if (warp == 4u) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::kTmemColumns);
    }
    // latest exit over all CTAs (the timer only grows, so the last launch wins)
    if (TRACE && threadIdx.x == 0u) atomicMax(reinterpret_cast<unsigned long long*>(trace + 11), (unsigned long long)global_timer_ns());
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
    // (the blocks of an expert's `matrices` tensors are interleaved: block (m_tile, kb) of tensor mx lies at
    // ((m_tile * k_blocks + kb) * matrices + mx) * 512, and ts[mx] already points at mx * 512)
    const size_t stride = (size_t)matrices * kScaleBlockBytes;
    uint8_t* out = const_cast<uint8_t*>(ptrs.ts[mx]) + (size_t)m_tile * k_blocks * stride + (r & 31u) * 16u + (r >> 5) * 4u;
    for (uint32_t kb = 0; kb < k_blocks; kb++) {
        uint32_t word = 0x7f7f7f7fu;
        if (row < rows && ptrs.format == kFormatNativeFp8) {
            // one exponent byte per 128 x 128 block, repeated over the block's four 32-column groups
            word = 0x01010101u * (uint32_t)ptrs.s[mx][(size_t)(row / 128u) * k_blocks + kb];
        } else if (row < rows) {
            word = 0u;
            for (uint32_t j = 0; j < 4u; j++) {
                const uint32_t c = kb * 4u + j;
                word |= (uint32_t)(c < row_bytes ? ptrs.s[mx][(size_t)row * row_bytes + c] : 127u) << (8u * j);
            }
        }
        *reinterpret_cast<uint32_t*>(out + (size_t)kb * stride) = word;
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

// One warp per (expert, matrix): the template map with the expert's weight address patched in.
__global__ void __launch_bounds__(32) build_tensormaps_kernel(const ExpertPtrs* experts, const uint8_t* templ,
                                                             uint8_t* maps, uint32_t matrices) {
    __shared__ __align__(128) unsigned char sm[128];
    const uint32_t e = blockIdx.x / matrices, mx = blockIdx.x % matrices;
    const uint8_t* w = experts[e].w[mx];
    if (experts[e].w[0] == nullptr || w == nullptr) return;
    // `templ` holds the map of the compact form followed by the map of the one-byte-per-element forms
    const uint8_t* mine = templ + (experts[e].format == kFormatCompact ? 0u : 128u);
    reinterpret_cast<uint32_t*>(sm)[threadIdx.x] = reinterpret_cast<const uint32_t*>(mine)[threadIdx.x];
    __syncwarp();
    if (threadIdx.x == 0u) tensormap_replace_address(sm, w);
    __syncwarp();
    tensormap_publish(maps + (size_t)blockIdx.x * 128u, sm);
}

int g_sm_count[16] = {0};

// wide token tiles of the down stage take two row tiles at a time
template <bool GATE_UP, uint32_t N_TILE>
constexpr bool row_pair() { return !GATE_UP && N_TILE >= 64u; }

template <bool GATE_UP, uint32_t N_TILE, bool USE_TMA>
void launch_n(const ExpertLaunch& p, cudaStream_t stream) {
    using C = Config<GATE_UP, N_TILE, USE_TMA, row_pair<GATE_UP, N_TILE>()>;
    int dev = 0;
    cudaGetDevice(&dev);
    if (g_sm_count[dev & 15] == 0) cudaDeviceGetAttribute(&g_sm_count[dev & 15], cudaDevAttrMultiProcessorCount, dev);
    // the traced instantiation only when a plan's trace was armed (and only for the TMA form)
    if (USE_TMA && p.cta_trace != nullptr) {
        launch_chained(experts_tc_kernel<GATE_UP, N_TILE, USE_TMA, row_pair<GATE_UP, N_TILE>(), USE_TMA>, dim3(g_sm_count[dev & 15]),
                       dim3(C::kThreads), C::kSmemBytes, stream, p, TileList{p.tile_list, p.tile_count});
    } else {
        launch_chained(experts_tc_kernel<GATE_UP, N_TILE, USE_TMA, row_pair<GATE_UP, N_TILE>(), false>, dim3(g_sm_count[dev & 15]),
                       dim3(C::kThreads), C::kSmemBytes, stream, p, TileList{p.tile_list, p.tile_count});
    }
}

template <bool GATE_UP>
void launch(const ExpertLaunch& p, cudaStream_t stream) {
    constexpr uint32_t kWide = 96u;
    const uint32_t n = tc_token_tile_for(p.tokens, p.g.routed_k + p.g.always_count, p.work.num_experts, GATE_UP);
    if (p.tmaps != nullptr) {
        switch (n) {
            case 16u: launch_n<GATE_UP, 16u, true>(p, stream); break;
            case 32u: launch_n<GATE_UP, 32u, true>(p, stream); break;
            case 64u: launch_n<GATE_UP, 64u, true>(p, stream); break;
            default: launch_n<GATE_UP, kWide, true>(p, stream); break;
        }
    } else {
        switch (n) {
            case 16u: launch_n<GATE_UP, 16u, false>(p, stream); break;
            case 32u: launch_n<GATE_UP, 32u, false>(p, stream); break;
            case 64u: launch_n<GATE_UP, 64u, false>(p, stream); break;
            default: launch_n<GATE_UP, kWide, false>(p, stream); break;
        }
    }
}

template <bool GATE_UP, uint32_t N_TILE>
void configure_one() {
    constexpr bool kPair = row_pair<GATE_UP, N_TILE>();
    cudaFuncSetAttribute(experts_tc_kernel<GATE_UP, N_TILE, true, kPair, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)Config<GATE_UP, N_TILE, true, kPair>::kSmemBytes);
    cudaFuncSetAttribute(experts_tc_kernel<GATE_UP, N_TILE, true, kPair, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)Config<GATE_UP, N_TILE, true, kPair>::kSmemBytes);
    cudaFuncSetAttribute(experts_tc_kernel<GATE_UP, N_TILE, false, kPair, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)Config<GATE_UP, N_TILE, false, kPair>::kSmemBytes);
}

}  // namespace

bool tc_shape_supported(const nvmoe_geometry& g) {
    return g.hidden_size % 32u == 0u && g.intermediate_size % 32u == 0u && g.act_block % 32u == 0u;
}

bool tc_enabled_by_default() { return true; }

uint32_t tc_token_tile_for(uint32_t tokens, uint32_t routes_per_token, uint32_t num_experts, bool gate_up) {
    // tokens per expert if routing were uniform; skew only adds token tiles
    const uint32_t routes = tokens * routes_per_token;
    const uint32_t per_expert = (routes + num_experts - 1u) / num_experts;
    // wide tiles hold two accumulators per token column (gate and up, or two row tiles of down): 96 columns
    // is the widest tile that still leaves tensor memory for a second pair, so that the epilogue of one
    // tile overlaps the MMAs of the next
    (void)gate_up;
    return per_expert <= 12u ? 16u : per_expert <= 24u ? 32u : per_expert <= 48u ? 64u : 96u;
}

uint32_t tc_token_tile_index(uint32_t n_tile) { return n_tile == 16u ? 0u : n_tile == 32u ? 1u : n_tile == 64u ? 2u : 3u; }

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

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// the driver's encoder, looked up through the runtime (no link-time dependency on libcuda)
static EncodeFn tensor_map_encoder() {
    static EncodeFn encode = nullptr;
    if (!encode) {
        cudaDriverEntryPointQueryResult q;
        void* fn = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess || !fn)
            return nullptr;
        encode = reinterpret_cast<EncodeFn>(fn);
    }
    return encode;
}

bool tc_encode_weight_map(void* map128, void* any_device_address, uint32_t rows, uint32_t cols) {
    // The packaged [rows][cols/2] bytes seen as a 3-D tensor of 4-bit elements
    // {128 elements, cols/128 K blocks, rows}: a box {128, 1, 128} is one operand tile. The padded 4-bit
    // type wants 32-byte strides (cols % 64 == 0); a trailing partial K block is not part of the map.
    if (cols < kBlockK || cols % 64u != 0u) return false;
    EncodeFn encode = tensor_map_encoder();
    if (!encode) return false;
    const cuuint64_t dims[3] = {kBlockK, cols / kBlockK, rows};
    const cuuint64_t strides[2] = {kBlockK / 2u, cols / 2u};
    const cuuint32_t box[3] = {kBlockK, 1u, kBlockM};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    CUtensorMap map;
    if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 3, any_device_address, dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    std::memcpy(map128, &map, 128);
    return true;
}

bool tc_encode_weight_map_bytes(void* map128, void* any_device_address, uint32_t rows, uint32_t cols) {
    // One E4M3 byte per element, seen like the compact form as {128 elements, cols/128 K blocks, rows}: the
    // same box coordinates fetch the same operand tile, now without padding.
    if (cols < kBlockK || cols % kBlockK != 0u) return false;
    EncodeFn encode = tensor_map_encoder();
    if (!encode) return false;
    const cuuint64_t dims[3] = {kBlockK, cols / kBlockK, rows};
    const cuuint64_t strides[2] = {kBlockK, cols};
    const cuuint32_t box[3] = {kBlockK, 1u, kBlockM};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    CUtensorMap map;
    if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, any_device_address, dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    std::memcpy(map128, &map, 128);
    return true;
}

bool tc_encode_activation_map(void* map128, void* base, uint32_t rows, uint32_t cols, uint32_t n_tile) {
    if (cols % 16u != 0u || rows == 0u) return false;
    EncodeFn encode = tensor_map_encoder();
    if (!encode) return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols};
    const cuuint32_t box[2] = {kBlockK, n_tile};
    const cuuint32_t estr[2] = {1u, 1u};
    CUtensorMap map;
    if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    std::memcpy(map128, &map, 128);
    return true;
}

void launch_build_tensormaps_tc(const ExpertLaunch& p, bool gate_up, const uint8_t* templ, cudaStream_t stream) {
    const uint32_t matrices = gate_up ? 2u : 1u;
    build_tensormaps_kernel<<<p.work.num_experts * matrices, 32, 0, stream>>>(p.work.experts, templ,
                                                                              const_cast<uint8_t*>(p.tmaps), matrices);
}



void tc_configure_kernels() {
    configure_one<true, 16u>();
    configure_one<true, 32u>();
    configure_one<true, 64u>();
    configure_one<true, 96u>();
    configure_one<false, 16u>();
    configure_one<false, 32u>();
    configure_one<false, 64u>();
    configure_one<false, 96u>();
}

void launch_gate_up_tc(const ExpertLaunch& p, cudaStream_t stream) { launch<true>(p, stream); }
void launch_down_tc(const ExpertLaunch& p, cudaStream_t stream) { launch<false>(p, stream); }

}  // namespace nvmoe
