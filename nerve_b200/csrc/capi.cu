// C ABI of the CUDA MoE backend (declared in include/nerve_cuda_moe.h): device, resident buffers,
// plans, the node-granular operators and the fused layer call.  Host code only; the kernels live
// in the other .cu files of this folder.
#include <atomic>
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <memory>
#include <new>
#include <string>
#include <thread>
#include <type_traits>
#include <vector>

#include <dlfcn.h>
#include <nccl.h>

#include "common.cuh"
#include "experts_tc.cuh"

using namespace nvmoe;

struct nvmoe_device {
    int ordinal = 0;
    cudaStream_t stream = nullptr;      // where launches go: own_stream unless the caller lent one
    cudaStream_t own_stream = nullptr;
    cudaEvent_t sync_event = nullptr;
    std::string error;
};

struct nvmoe_buffer {
    nvmoe_device* device = nullptr;
    void* ptr = nullptr;
    size_t bytes = 0;
    bool owned = true;  // false for handles over memory the caller allocated
    // identity and content version: what a plan resolved from an address or slot table stays valid
    // while both are unchanged. Every write through this interface bumps the version; memory the
    // caller owns can change behind the handle, so tables in wrapped buffers are resolved on every call.
    uint64_t uid = 0;
    uint64_t version = 0;
};

namespace {

thread_local std::string g_open_error;
std::atomic<uint64_t> g_next_buffer_uid{1};

int fail(nvmoe_device* d, int code, const char* fmt, ...) {
    char text[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(text, sizeof(text), fmt, ap);
    va_end(ap);
    if (d) {
        d->error = text;
    } else {
        g_open_error = text;
    }
    return code;
}

#define NVMOE_CUDA(d, call)                                                                      \
    do {                                                                                         \
        cudaError_t err__ = (call);                                                              \
        if (err__ != cudaSuccess)                                                                \
            return fail((d), err__ == cudaErrorMemoryAllocation ? NVMOE_ERR_OUT_OF_MEMORY : NVMOE_ERR_CUDA, \
                        "%s failed: %s", #call, cudaGetErrorString(err__));                      \
    } while (0)

struct DeviceArray {  // plan-owned scratch
    void* ptr = nullptr;
    size_t bytes = 0;
    cudaError_t ensure(size_t want) {
        if (want <= bytes) return cudaSuccess;
        if (ptr) cudaFree(ptr);
        ptr = nullptr;
        bytes = 0;
        cudaError_t err = cudaMalloc(&ptr, want);
        if (err == cudaSuccess) bytes = want;
        return err;
    }
    void release() {
        if (ptr) cudaFree(ptr);
        ptr = nullptr;
        bytes = 0;
    }
    template <class T>
    T* as() const {
        return reinterpret_cast<T*>(ptr);
    }
};

// What one (address table, slot table) pair resolves to for one expert stage: validated weight and
// scale pointers per expert and, for the tensor path, the re-tiled scale copies and the per-expert
// tensor maps. Kept per pair so that a model's layers (one table pair each) resolve once, not per call.
struct ExpertSet {
    uint64_t key[4] = {0, 0, 0, 0};  // address table uid, version, slot table uid, version
    bool cacheable = false;
    bool resolved = false;
    bool resolved_for_tensor = false;  // the path the cached resolution was made for (its limits differ)
    bool tensor_ready = false;
    uint64_t last_use = 0;
    DeviceArray ptrs, derived, stamps, tmaps;
    void release() {
        ptrs.release();
        derived.release();
        stamps.release();
        tmaps.release();
    }
};
constexpr size_t kMaxExpertSets = 64;
constexpr int kHostWaitSeconds = 60;  // how long the host-buffer layer call waits for its result

enum Stage { kStageLinear, kStageRoute, kStageSchedule, kStageQuantX, kStageGateUp, kStageQuantI, kStageDown, kStageReduce, kStageCount };

}  // namespace

struct nvmoe_plan {
    nvmoe_device* device = nullptr;
    nvmoe_geometry g{};
    uint32_t K = 0;            // routes per token
    uint32_t experts = 0;      // routed + always
    uint32_t frame_words = 0;
    int expert_path = 0;
    // scratch every expert call needs
    DeviceArray status, grouped[2], offsets[2], block_hist, bucket_base;
    std::vector<std::unique_ptr<ExpertSet>> sets[2];  // [gate/up, down], least recently used replaced
    uint64_t use_clock = 0;
    DeviceArray xq, x_scales, x_e8m0, iq, i_scales, i_e8m0, tile_list, ep_source;
    // tensor path: expert-grouped quantised activations of the two stages (row = position in grouped[stage]),
    // where each route landed, and the tensor maps of the two matrices for the four token tile sizes
    DeviceArray grouped_q[2], grouped_e8m0[2], position[2], act_maps;
    DeviceArray cta_trace;       // per-CTA diagnostics of the tensor-path kernels, allocated on first request
    DeviceArray tmap_templates;  // tensor maps of the two weight matrix shapes; each expert's map is one with its address patched in
    bool tma[2] = {false, false};
    // scratch of the fused layer call
    DeviceArray logits, routes, frames, expert_outputs, controls, hidden_dev, output_dev;
    void* pinned_in = nullptr;
    void* pinned_out = nullptr;
    size_t pinned_bytes = 0;
    cudaEvent_t ev[kStageCount + 1] = {};
    cudaEvent_t kernel_ev[2][2] = {};  // [gate_up, down][begin, end] around the expert kernel alone
    bool events_valid = false;
    bool profile_stages = false;
    nvmoe_work_report report{};
    uint32_t launches = 0;
    long long wait_cycles = 4000000000ll;  // limit of the bounded in-kernel waits of the tensor path (about 2 s)
    uint32_t debug_flags = 0;
    // dense linears run as one always-selected resource of a plan of their own shape (nvmoe_dense_linear)
    struct DenseLinear {
        uint32_t rows = 0, cols = 0;
        nvmoe_plan* plan = nullptr;
        nvmoe_buffer* addresses = nullptr;
        nvmoe_buffer* slots = nullptr;
        DeviceArray unit_routes;
        const void* weights = nullptr;
        const void* scales = nullptr;
        uint64_t weights_version = 0, scales_version = 0;
    };
    std::vector<DenseLinear> dense;
};

namespace {

// One region per expert stage: 64 header words (entry count, diagnostics) and the (expert, token tile) list.
size_t tile_region_words(const nvmoe_plan* p) {
    const size_t list = (size_t)p->g.max_tokens * p->K / 16u + p->experts + 1u;
    return (64u + list + 63u) / 64u * 64u;
}

size_t scratch_blocks(const nvmoe_plan* p) { return ((size_t)p->g.max_tokens * p->K + kSortChunk - 1u) / kSortChunk; }

SortScratch sort_scratch(const nvmoe_plan* p) {
    return SortScratch{p->block_hist.as<uint32_t>(), p->bucket_base.as<uint32_t>(), (uint32_t)scratch_blocks(p),
                       p->experts + 1u};
}

int check_buffer(nvmoe_plan* p, const nvmoe_buffer* b, size_t need, const char* what) {
    if (!b) return fail(p->device, NVMOE_ERR_INVALID_ARGUMENT, "%s buffer is null", what);
    if (b->device != p->device)
        return fail(p->device, NVMOE_ERR_INVALID_ARGUMENT, "%s buffer belongs to another device", what);
    if (b->bytes < need)
        return fail(p->device, NVMOE_ERR_INVALID_ARGUMENT, "%s buffer holds %zu bytes, the call needs %zu", what,
                    b->bytes, need);
    return NVMOE_OK;
}

int check_tokens(nvmoe_plan* p, uint32_t T) {
    if (T == 0u) return fail(p->device, NVMOE_ERR_INVALID_ARGUMENT, "batch_width is zero");
    if (T > p->g.max_tokens)
        return fail(p->device, NVMOE_ERR_INVALID_ARGUMENT, "batch_width %u exceeds the plan's max_tokens %u", T,
                    p->g.max_tokens);
    return NVMOE_OK;
}

int post_launch(nvmoe_plan* p, const char* what) {
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return fail(p->device, NVMOE_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(err));
    return NVMOE_OK;
}

#define NVMOE_TRY(expr)              \
    do {                             \
        int rc__ = (expr);           \
        if (rc__ != NVMOE_OK) return rc__; \
    } while (0)

bool use_tensor_path(const nvmoe_plan* p) {
    if (p->expert_path == 1) return false;
    if (!tc_shape_supported(p->g)) return false;
    if (p->expert_path == 2) return true;
    return tc_enabled_by_default();
}

int validate_geometry(const nvmoe_geometry& g) {
    auto bad = [](const char* fmt, ...) {
        char text[256];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(text, sizeof(text), fmt, ap);
        va_end(ap);
        g_open_error = text;
        return (int)NVMOE_ERR_INVALID_ARGUMENT;
    };
    if (g.hidden_size == 0u || g.hidden_size % 32u) return bad("hidden_size %u must be a positive multiple of 32", g.hidden_size);
    if (g.intermediate_size == 0u || g.intermediate_size % 32u)
        return bad("intermediate_size %u must be a positive multiple of 32", g.intermediate_size);
    if (!(0u < g.routed_k && g.routed_k <= g.routed_experts && g.routed_experts <= kMaxExperts))
        return bad("invalid routing geometry r%u k%u", g.routed_experts, g.routed_k);
    if (g.router_kind > NVMOE_ROUTER_PRESELECTED) return bad("unknown router_kind %u", g.router_kind);
    if (g.router_kind == NVMOE_ROUTER_PRESELECTED && g.activation == NVMOE_ACT_SOFTMAX)
        return bad("a preselected router needs an activation that is evaluated per resource (sigmoid or sqrt-softplus)");
    if (g.activation > NVMOE_ACT_SQRT_SOFTPLUS) return bad("unknown router activation %u", g.activation);
    if (g.router_kind == NVMOE_ROUTER_TOPK_ROUTED && g.activation == NVMOE_ACT_SQRT_SOFTPLUS)
        return bad("the routed top-k router scores with sigmoid or softmax only");
    if (g.bias_dtype > NVMOE_BIAS_BF16) return bad("unknown bias dtype %u", g.bias_dtype);
    if (g.always_count && g.router_kind != NVMOE_ROUTER_SCORE_TOPK && g.router_kind != NVMOE_ROUTER_PRESELECTED)
        return bad("always-selected resources need the score_topk or the preselected router");
    if (g.always_count && !(g.always_weight > 0.0f) ) return bad("always-selected weight must be positive and finite");
    if (g.routed_experts + g.always_count > kMaxExperts) return bad("total resource count exceeds %u", kMaxExperts);
    if (g.routed_k + g.always_count > kMaxTopK) return bad("more than %u routes per token", kMaxTopK);
    if (g.n_group) {
        if (g.n_group > 32u || g.routed_experts % g.n_group || g.topk_group == 0u || g.topk_group > g.n_group ||
            (g.routed_experts / g.n_group) * g.topk_group < g.routed_k)
            return bad("invalid group-limited routing n_group %u topk_group %u", g.n_group, g.topk_group);
    }
    if (g.act_block == 0u || g.act_block % 32u || g.hidden_size % g.act_block || g.intermediate_size % g.act_block)
        return bad("act_block %u must be a multiple of 32 dividing hidden and intermediate sizes", g.act_block);
    if (g.gate_tile_rows == 0u || g.down_tile_rows == 0u) return bad("tile rows must be positive");
    if (g.max_tokens == 0u) return bad("max_tokens is zero");
    if (g.native_fp8_resources > g.routed_experts + g.always_count)
        return bad("%u native FP8 resources among %u", g.native_fp8_resources, g.routed_experts + g.always_count);
    if ((uint64_t)g.max_tokens * (g.routed_k + g.always_count) > 0x7fffffffull) return bad("max_tokens * routes overflows");
    return NVMOE_OK;
}

__global__ void write_control_kernel(uint32_t* control, uint32_t T, uint32_t start, uint32_t count) {
    if (threadIdx.x < 7u) control[threadIdx.x] = threadIdx.x == 0u ? T : threadIdx.x == 1u ? start : threadIdx.x == 2u ? count : 0u;
}

}  // namespace

extern "C" {

void nvmoe_geometry_default(nvmoe_geometry* g, uint32_t hidden, uint32_t intermediate, uint32_t experts, uint32_t k) {
    std::memset(g, 0, sizeof(*g));
    g->hidden_size = hidden;
    g->intermediate_size = intermediate;
    g->routed_experts = experts;
    g->routed_k = k;
    g->always_weight = 1.0f;
    g->router_kind = NVMOE_ROUTER_SCORE_TOPK;
    g->activation = NVMOE_ACT_SOFTMAX;
    g->normalize_selected = 1;
    g->routed_scale = 1.0f;
    g->swiglu_alpha = 1.0f;
    g->act_block = 128;
    g->gate_tile_rows = 32;
    g->down_tile_rows = 64;
    g->reduce_scale = 1.0f;
    g->max_tokens = 1;
}

int nvmoe_device_open(int cuda_ordinal, nvmoe_device** out) {
    if (!out) return fail(nullptr, NVMOE_ERR_INVALID_ARGUMENT, "out pointer is null");
    *out = nullptr;
    int count = 0;
    cudaError_t err = cudaGetDeviceCount(&count);
    if (err != cudaSuccess) return fail(nullptr, NVMOE_ERR_CUDA, "no CUDA device: %s", cudaGetErrorString(err));
    if (cuda_ordinal < 0 || cuda_ordinal >= count)
        return fail(nullptr, NVMOE_ERR_INVALID_ARGUMENT, "CUDA ordinal %d out of range (%d devices)", cuda_ordinal, count);
    cudaDeviceProp prop;
    NVMOE_CUDA(nullptr, cudaGetDeviceProperties(&prop, cuda_ordinal));
    if (prop.major != 10)
        return fail(nullptr, NVMOE_ERR_UNSUPPORTED, "device %d is sm_%d%d; this backend is built for sm_100a only",
                    cuda_ordinal, prop.major, prop.minor);
    NVMOE_CUDA(nullptr, cudaSetDevice(cuda_ordinal));
    nvmoe_device* d = new (std::nothrow) nvmoe_device();
    if (!d) return fail(nullptr, NVMOE_ERR_OUT_OF_MEMORY, "out of host memory");
    d->ordinal = cuda_ordinal;
    cudaError_t e1 = cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking);
    cudaError_t e2 = e1 == cudaSuccess ? cudaEventCreateWithFlags(&d->sync_event, cudaEventDisableTiming) : e1;
    if (e2 != cudaSuccess) {
        if (d->stream) cudaStreamDestroy(d->stream);
        delete d;
        return fail(nullptr, NVMOE_ERR_CUDA, "stream setup failed: %s", cudaGetErrorString(e2));
    }
    d->own_stream = d->stream;
    *out = d;
    return NVMOE_OK;
}

void nvmoe_device_close(nvmoe_device* d) {
    if (!d) return;
    cudaSetDevice(d->ordinal);
    cudaStreamSynchronize(d->stream);
    cudaEventDestroy(d->sync_event);
    cudaStreamDestroy(d->own_stream);
    delete d;
}

int nvmoe_device_set_stream(nvmoe_device* d, void* stream) {
    if (!d) return NVMOE_ERR_INVALID_ARGUMENT;
    NVMOE_CUDA(d, cudaSetDevice(d->ordinal));
    NVMOE_CUDA(d, cudaStreamSynchronize(d->stream));  // nothing may straddle the switch
    d->stream = stream ? (cudaStream_t)stream : d->own_stream;
    return NVMOE_OK;
}

const char* nvmoe_last_error(const nvmoe_device* d) { return d ? d->error.c_str() : g_open_error.c_str(); }

void* nvmoe_device_stream(const nvmoe_device* d) { return d ? (void*)d->stream : nullptr; }

int nvmoe_buffer_create(nvmoe_device* d, size_t bytes, nvmoe_buffer** out) {
    if (!d || !out) return fail(d, NVMOE_ERR_INVALID_ARGUMENT, "null device or out pointer");
    *out = nullptr;
    if (bytes == 0) return fail(d, NVMOE_ERR_INVALID_ARGUMENT, "resident buffer of zero bytes");
    NVMOE_CUDA(d, cudaSetDevice(d->ordinal));
    nvmoe_buffer* b = new (std::nothrow) nvmoe_buffer();
    if (!b) return fail(d, NVMOE_ERR_OUT_OF_MEMORY, "out of host memory");
    cudaError_t err = cudaMalloc(&b->ptr, bytes);
    if (err != cudaSuccess) {
        delete b;
        return fail(d, NVMOE_ERR_OUT_OF_MEMORY, "cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(err));
    }
    err = cudaMemsetAsync(b->ptr, 0, bytes, d->stream);
    if (err != cudaSuccess) {
        cudaFree(b->ptr);
        delete b;
        return fail(d, NVMOE_ERR_CUDA, "zero fill failed: %s", cudaGetErrorString(err));
    }
    b->device = d;
    b->bytes = bytes;
    b->uid = g_next_buffer_uid.fetch_add(1);
    *out = b;
    return NVMOE_OK;
}

int nvmoe_buffer_wrap(nvmoe_device* d, void* device_ptr, size_t bytes, nvmoe_buffer** out) {
    if (!d || !out) return fail(d, NVMOE_ERR_INVALID_ARGUMENT, "null device or out pointer");
    *out = nullptr;
    if (!device_ptr || bytes == 0) return fail(d, NVMOE_ERR_INVALID_ARGUMENT, "cannot wrap a null or empty range");
    NVMOE_CUDA(d, cudaSetDevice(d->ordinal));
    cudaPointerAttributes attr;
    NVMOE_CUDA(d, cudaPointerGetAttributes(&attr, device_ptr));
    if (attr.type != cudaMemoryTypeDevice || attr.device != d->ordinal)
        return fail(d, NVMOE_ERR_INVALID_ARGUMENT, "the pointer is not device memory of CUDA ordinal %d", d->ordinal);
    nvmoe_buffer* b = new (std::nothrow) nvmoe_buffer();
    if (!b) return fail(d, NVMOE_ERR_OUT_OF_MEMORY, "out of host memory");
    b->device = d;
    b->ptr = device_ptr;
    b->bytes = bytes;
    b->owned = false;
    // handles over the same memory share an identity: a table that is wrapped afresh for every call keeps its
    // place (and its derived copies) in a plan's cache instead of claiming a new one each time
    b->uid = (1ull << 63) | (uint64_t)(uintptr_t)device_ptr;
    *out = b;
    return NVMOE_OK;
}

void nvmoe_buffer_destroy(nvmoe_buffer* b) {
    if (!b) return;
    if (b->owned) {
        cudaSetDevice(b->device->ordinal);
        cudaStreamSynchronize(b->device->stream);
        cudaFree(b->ptr);
    }
    delete b;
}

static int range_ok(nvmoe_buffer* b, size_t offset, size_t bytes, const void* host) {
    if (!b) return NVMOE_ERR_INVALID_ARGUMENT;
    if (!host && bytes) return fail(b->device, NVMOE_ERR_INVALID_ARGUMENT, "host pointer is null");
    if (offset > b->bytes || bytes > b->bytes - offset)
        return fail(b->device, NVMOE_ERR_INVALID_ARGUMENT, "range [%zu, %zu) overflows a buffer of %zu bytes", offset,
                    offset + bytes, b->bytes);
    return NVMOE_OK;
}

int nvmoe_buffer_write(nvmoe_buffer* b, size_t offset, const void* src, size_t bytes) {
    NVMOE_TRY(range_ok(b, offset, bytes, src));
    if (bytes == 0) return NVMOE_OK;
    nvmoe_device* d = b->device;
    b->version++;
    NVMOE_CUDA(d, cudaSetDevice(d->ordinal));
    NVMOE_CUDA(d, cudaMemcpyAsync((char*)b->ptr + offset, src, bytes, cudaMemcpyHostToDevice, d->stream));
    NVMOE_CUDA(d, cudaStreamSynchronize(d->stream));  // the caller may reuse src at once
    return NVMOE_OK;
}

int nvmoe_buffer_read(nvmoe_buffer* b, size_t offset, void* dst, size_t bytes) {
    NVMOE_TRY(range_ok(b, offset, bytes, dst));
    if (bytes == 0) return NVMOE_OK;
    nvmoe_device* d = b->device;
    NVMOE_CUDA(d, cudaSetDevice(d->ordinal));
    NVMOE_CUDA(d, cudaMemcpyAsync(dst, (const char*)b->ptr + offset, bytes, cudaMemcpyDeviceToHost, d->stream));
    NVMOE_CUDA(d, cudaStreamSynchronize(d->stream));
    return NVMOE_OK;
}

int nvmoe_buffer_fill(nvmoe_buffer* b, size_t offset, int byte_value, size_t bytes) {
    NVMOE_TRY(range_ok(b, offset, bytes, b));
    if (bytes == 0) return NVMOE_OK;
    nvmoe_device* d = b->device;
    b->version++;
    NVMOE_CUDA(d, cudaSetDevice(d->ordinal));
    NVMOE_CUDA(d, cudaMemsetAsync((char*)b->ptr + offset, byte_value, bytes, d->stream));
    return NVMOE_OK;
}

uint64_t nvmoe_buffer_device_address(const nvmoe_buffer* b) { return b ? (uint64_t)(uintptr_t)b->ptr : 0u; }

int nvmoe_buffer_mark_dirty(nvmoe_buffer* b) {
    if (!b) return NVMOE_ERR_INVALID_ARGUMENT;
    b->version++;
    return NVMOE_OK;
}
size_t nvmoe_buffer_byte_capacity(const nvmoe_buffer* b) { return b ? b->bytes : 0u; }

int nvmoe_sync(nvmoe_device* d, uint64_t timeout_ns) {
    if (!d) return NVMOE_ERR_INVALID_ARGUMENT;
    NVMOE_CUDA(d, cudaSetDevice(d->ordinal));
    NVMOE_CUDA(d, cudaEventRecord(d->sync_event, d->stream));
    auto deadline = std::chrono::steady_clock::now() + std::chrono::nanoseconds(timeout_ns);
    for (;;) {
        cudaError_t q = cudaEventQuery(d->sync_event);
        if (q == cudaSuccess) return NVMOE_OK;
        if (q != cudaErrorNotReady) return fail(d, NVMOE_ERR_CUDA, "device failed while waiting: %s", cudaGetErrorString(q));
        if (std::chrono::steady_clock::now() >= deadline)
            return fail(d, NVMOE_ERR_TIMEOUT, "device did not finish within %llu ns", (unsigned long long)timeout_ns);
        std::this_thread::yield();
    }
}

// ---- plan ------------------------------------------------------------------------------------

int nvmoe_plan_create(nvmoe_device* d, const nvmoe_geometry* geometry, nvmoe_plan** out) {
    if (!d || !geometry || !out) return fail(d, NVMOE_ERR_INVALID_ARGUMENT, "null argument");
    *out = nullptr;
    int rc = validate_geometry(*geometry);
    if (rc != NVMOE_OK) return fail(d, rc, "%s", g_open_error.c_str());
    NVMOE_CUDA(d, cudaSetDevice(d->ordinal));
    nvmoe_plan* p = new (std::nothrow) nvmoe_plan();
    if (!p) return fail(d, NVMOE_ERR_OUT_OF_MEMORY, "out of host memory");
    p->device = d;
    p->g = *geometry;
    const nvmoe_geometry& g = p->g;
    p->K = g.routed_k + g.always_count;
    p->experts = g.routed_experts + g.always_count;
    p->frame_words = p->K * (g.intermediate_size / 2u) + p->K;
    const size_t T = g.max_tokens, R = T * p->K, H = g.hidden_size, I = g.intermediate_size;
    cudaError_t err = cudaSuccess;
    auto want = [&](DeviceArray& a, size_t bytes) {
        if (err == cudaSuccess) err = a.ensure(bytes);
    };
    want(p->status, 256);
    for (int i = 0; i < 2; i++) {
        want(p->grouped[i], sizeof(uint32_t) * R);
        want(p->offsets[i], sizeof(uint32_t) * (p->experts + 2u));
    }
    want(p->block_hist, sizeof(uint32_t) * scratch_blocks(p) * (p->experts + 1u));
    want(p->bucket_base, sizeof(uint32_t) * (p->experts + 2u));
    want(p->xq, T * H);
    want(p->x_scales, sizeof(float) * T * (H / g.act_block));
    want(p->x_e8m0, sizeof(uint32_t) * T * ((H + 127u) / 128u));
    want(p->iq, R * I);
    want(p->i_scales, sizeof(float) * R * (I / g.act_block));
    want(p->i_e8m0, sizeof(uint32_t) * R * ((I + 127u) / 128u));
    want(p->tile_list, sizeof(uint32_t) * 2u * tile_region_words(p));
    want(p->position[0], sizeof(uint32_t) * R);
    want(p->position[1], sizeof(uint32_t) * R);
    if (tc_shape_supported(g)) {
        want(p->grouped_q[0], R * H);
        want(p->grouped_q[1], R * I);
        want(p->grouped_e8m0[0], sizeof(uint32_t) * R * ((H + 127u) / 128u));
        want(p->grouped_e8m0[1], sizeof(uint32_t) * R * ((I + 127u) / 128u));
        want(p->act_maps, 8u * 128u);
        if (err == cudaSuccess) {
            unsigned char maps[8 * 128];
            bool ok = true;
            for (uint32_t set = 0; set < 2u && ok; set++)
                for (uint32_t i = 0; i < 4u && ok; i++)
                    ok = tc_encode_activation_map(maps + (set * 4u + i) * 128u, p->grouped_q[set].ptr, (uint32_t)R,
                                                  (uint32_t)(set == 0u ? H : I), i < 3u ? 16u << i : 96u);
            if (ok) {
                err = cudaMemcpyAsync(p->act_maps.ptr, maps, sizeof maps, cudaMemcpyHostToDevice, d->stream);
                if (err == cudaSuccess) err = cudaStreamSynchronize(d->stream);  // `maps` is a stack buffer
            } else {
                p->act_maps.release();  // no tensor maps on this system: the tensor path copies with cp.async
            }
        }
        want(p->tmap_templates, 512);
        if (err == cudaSuccess) {
            // per stage: the map of the compact form, then the map of the one-byte-per-element forms (left zero
            // when the shape has no whole 128-column blocks: such resources are then treated as not resident)
            unsigned char maps[512] = {0};
            p->tma[0] = tc_encode_weight_map(maps, p->tmap_templates.ptr, g.intermediate_size, g.hidden_size);
            p->tma[1] = tc_encode_weight_map(maps + 256, p->tmap_templates.ptr, g.hidden_size, g.intermediate_size);
            tc_encode_weight_map_bytes(maps + 128, p->tmap_templates.ptr, g.intermediate_size, g.hidden_size);
            tc_encode_weight_map_bytes(maps + 384, p->tmap_templates.ptr, g.hidden_size, g.intermediate_size);
            if (!p->act_maps.ptr) p->tma[0] = p->tma[1] = false;
            err = cudaMemcpyAsync(p->tmap_templates.ptr, maps, 512, cudaMemcpyHostToDevice, d->stream);
            if (err == cudaSuccess) err = cudaStreamSynchronize(d->stream);  // `maps` is a stack buffer
        }
    }
    if (err == cudaSuccess) err = cudaMemsetAsync(p->status.ptr, 0, 256, d->stream);
    for (int i = 0; i <= kStageCount && err == cudaSuccess; i++) err = cudaEventCreate(&p->ev[i]);
    for (int i = 0; i < 4 && err == cudaSuccess; i++) err = cudaEventCreate(&p->kernel_ev[i / 2][i % 2]);
    if (err != cudaSuccess) {
        int code = err == cudaErrorMemoryAllocation ? NVMOE_ERR_OUT_OF_MEMORY : NVMOE_ERR_CUDA;
        fail(d, code, "plan scratch allocation failed: %s", cudaGetErrorString(err));
        nvmoe_plan_destroy(p);
        return code;
    }
    configure_simt_kernels();
    tc_configure_kernels();
    *out = p;
    return NVMOE_OK;
}

void nvmoe_plan_destroy(nvmoe_plan* p) {
    if (!p) return;
    cudaSetDevice(p->device->ordinal);
    cudaStreamSynchronize(p->device->stream);
    for (auto& dl : p->dense) {
        nvmoe_plan_destroy(dl.plan);
        nvmoe_buffer_destroy(dl.addresses);
        nvmoe_buffer_destroy(dl.slots);
        dl.unit_routes.release();
    }
    for (auto& stage_sets : p->sets)
        for (auto& es : stage_sets) es->release();
    DeviceArray* all[] = {&p->status, &p->grouped[0], &p->grouped[1], &p->offsets[0],
                          &p->offsets[1], &p->block_hist, &p->bucket_base, &p->xq, &p->x_scales, &p->x_e8m0, &p->iq,
                          &p->i_scales, &p->i_e8m0, &p->tile_list, &p->ep_source, &p->tmap_templates, &p->cta_trace, &p->grouped_q[0], &p->grouped_q[1],
                          &p->grouped_e8m0[0], &p->grouped_e8m0[1], &p->position[0], &p->position[1], &p->act_maps, &p->logits, &p->routes, &p->frames, &p->expert_outputs,
                          &p->controls, &p->hidden_dev, &p->output_dev};
    for (DeviceArray* a : all) a->release();
    if (p->pinned_in) cudaFreeHost(p->pinned_in);
    if (p->pinned_out) cudaFreeHost(p->pinned_out);
    for (int i = 0; i <= kStageCount; i++)
        if (p->ev[i]) cudaEventDestroy(p->ev[i]);
    for (int i = 0; i < 4; i++)
        if (p->kernel_ev[i / 2][i % 2]) cudaEventDestroy(p->kernel_ev[i / 2][i % 2]);
    delete p;
}

int nvmoe_plan_status(nvmoe_plan* p, uint32_t* status_bits) {
    if (!p || !status_bits) return NVMOE_ERR_INVALID_ARGUMENT;
    nvmoe_device* d = p->device;
    NVMOE_CUDA(d, cudaSetDevice(d->ordinal));
    NVMOE_CUDA(d, cudaMemcpyAsync(status_bits, p->status.ptr, 4, cudaMemcpyDeviceToHost, d->stream));
    NVMOE_CUDA(d, cudaMemsetAsync(p->status.ptr, 0, 4, d->stream));
    NVMOE_CUDA(d, cudaStreamSynchronize(d->stream));
    return NVMOE_OK;
}

int nvmoe_plan_set_expert_path(nvmoe_plan* p, int path) {
    if (!p) return NVMOE_ERR_INVALID_ARGUMENT;
    if (path < 0 || path > 2) return fail(p->device, NVMOE_ERR_INVALID_ARGUMENT, "expert path %d is not 0, 1 or 2", path);
    if (path == 2 && !tc_shape_supported(p->g))
        return fail(p->device, NVMOE_ERR_UNSUPPORTED, "the tensor-core path needs a power-of-two activation scale per 32-column block layout this geometry lacks");
    p->expert_path = path;
    return NVMOE_OK;
}

int nvmoe_plan_set_wait_limit(nvmoe_plan* p, uint64_t clock_cycles) {
    if (!p) return NVMOE_ERR_INVALID_ARGUMENT;
    if (clock_cycles > (1ull << 40)) return fail(p->device, NVMOE_ERR_INVALID_ARGUMENT, "wait limit of %llu cycles is beyond 2^40",
                                               (unsigned long long)clock_cycles);
    p->wait_cycles = clock_cycles ? (long long)clock_cycles : 4000000000ll;
    return NVMOE_OK;
}

int nvmoe_plan_debug_withhold_arrival(nvmoe_plan* p, int enabled) {
    if (!p) return NVMOE_ERR_INVALID_ARGUMENT;
    p->debug_flags = enabled ? (p->debug_flags | 1u) : (p->debug_flags & ~1u);
    return NVMOE_OK;
}

int nvmoe_plan_set_profiling(nvmoe_plan* p, int enabled) {
    if (!p) return NVMOE_ERR_INVALID_ARGUMENT;
    p->profile_stages = enabled != 0;
    return NVMOE_OK;
}

// ---- node-granular operators -----------------------------------------------------------------

int nvmoe_router_linear(nvmoe_plan* p, uint32_t T, const nvmoe_buffer* hidden, nvmoe_buffer* logits,
                        const nvmoe_buffer* router_weights, const nvmoe_buffer* router_bias) {
    if (!p) return NVMOE_ERR_INVALID_ARGUMENT;
    NVMOE_TRY(check_tokens(p, T));
    const nvmoe_geometry& g = p->g;
    NVMOE_TRY(check_buffer(p, hidden, (size_t)T * g.hidden_size * 2u, "hidden"));
    NVMOE_TRY(check_buffer(p, logits, (size_t)T * ((g.routed_experts + 1u) / 2u) * 4u, "logits"));
    NVMOE_TRY(check_buffer(p, router_weights, (size_t)g.routed_experts * g.hidden_size * 2u, "router weights"));
    if (router_bias) NVMOE_TRY(check_buffer(p, router_bias, (size_t)g.routed_experts * 2u, "router bias"));
    NVMOE_CUDA(p->device, cudaSetDevice(p->device->ordinal));
    launch_router_linear((const uint16_t*)hidden->ptr, (const uint16_t*)router_weights->ptr,
                         router_bias ? (const uint16_t*)router_bias->ptr : nullptr, (uint32_t*)logits->ptr, T,
                         g.hidden_size, g.routed_experts, p->device->stream);
    p->launches++;
    return post_launch(p, "router projection");
}

int nvmoe_route(nvmoe_plan* p, uint32_t T, const nvmoe_buffer* logits, nvmoe_buffer* routes,
                const nvmoe_buffer* bias, nvmoe_buffer* telemetry) {
    if (!p) return NVMOE_ERR_INVALID_ARGUMENT;
    NVMOE_TRY(check_tokens(p, T));
    const nvmoe_geometry& g = p->g;
    NVMOE_TRY(check_buffer(p, logits, (size_t)T * ((g.routed_experts + 1u) / 2u) * 4u, "logits"));
    NVMOE_TRY(check_buffer(p, routes, (size_t)T * p->K * 4u, "routes"));
    if (g.router_kind == NVMOE_ROUTER_PRESELECTED)
        return fail(p->device, NVMOE_ERR_INVALID_ARGUMENT, "this plan's router takes preselected resources: call nvmoe_route_preselected");
    const bool uses_bias = g.bias_dtype != NVMOE_BIAS_NONE && g.router_kind != NVMOE_ROUTER_TOPK_SOFTMAX;
    if (uses_bias)
        NVMOE_TRY(check_buffer(p, bias, (size_t)g.routed_experts * (g.bias_dtype == NVMOE_BIAS_F32 ? 4u : 2u), "selection bias"));
    if (telemetry) {
        const size_t r = p->experts;
        NVMOE_TRY(check_buffer(p, telemetry, (r + r * (r - 1u) / 2u) * 4u, "telemetry"));
    }
    NVMOE_CUDA(p->device, cudaSetDevice(p->device->ordinal));
    RouterLaunch rl{};
    rl.logits = (const uint32_t*)logits->ptr;
    rl.bias = uses_bias ? bias->ptr : nullptr;
    rl.routes = (uint32_t*)routes->ptr;
    rl.telemetry = telemetry ? (uint32_t*)telemetry->ptr : nullptr;
    rl.status = p->status.as<uint32_t>();
    rl.tokens = T;
    rl.g = g;
    if (!uses_bias) rl.g.bias_dtype = NVMOE_BIAS_NONE;
    launch_router(rl, p->device->stream);
    p->launches++;
    return post_launch(p, "router");
}

static int check_slots(nvmoe_plan* p, const nvmoe_buffer* slots) {
    if (slots && slots->device != p->device) return fail(p->device, NVMOE_ERR_INVALID_ARGUMENT, "slot table belongs to another device");
    return NVMOE_OK;
}

int nvmoe_route_compact(nvmoe_plan* p, uint32_t T, const nvmoe_buffer* routes, nvmoe_buffer* intermediates,
                        const nvmoe_buffer* gate_up_slots, nvmoe_buffer* control) {
    if (!p) return NVMOE_ERR_INVALID_ARGUMENT;
    NVMOE_TRY(check_tokens(p, T));
    NVMOE_TRY(check_buffer(p, routes, (size_t)T * p->K * 4u, "routes"));
    NVMOE_TRY(check_buffer(p, intermediates, (size_t)T * p->frame_words * 4u, "intermediates"));
    NVMOE_TRY(check_buffer(p, control, 28u, "control"));
    NVMOE_TRY(check_slots(p, gate_up_slots));
    NVMOE_CUDA(p->device, cudaSetDevice(p->device->ordinal));
    const nvmoe_geometry& g = p->g;
    const uint32_t tiles = (g.intermediate_size + g.gate_tile_rows - 1u) / g.gate_tile_rows;
    launch_route_compact((const uint32_t*)routes->ptr, (uint32_t*)intermediates->ptr,
                         gate_up_slots ? (const uint32_t*)gate_up_slots->ptr : nullptr,
                         gate_up_slots ? (uint32_t)(gate_up_slots->bytes / 4u) : 0u, 4u, (uint32_t*)control->ptr, T, p->K,
                         g.intermediate_size, tiles, p->experts, sort_scratch(p), p->device->stream);
    p->launches += (size_t)T * p->K <= 4096u ? 1u : 3u;
    return post_launch(p, "route compact");
}

int nvmoe_route_count(nvmoe_plan* p, uint32_t T, const nvmoe_buffer* routes, const nvmoe_buffer* down_slots,
                      nvmoe_buffer* control) {
    if (!p) return NVMOE_ERR_INVALID_ARGUMENT;
    NVMOE_TRY(check_tokens(p, T));
    NVMOE_TRY(check_buffer(p, routes, (size_t)T * p->K * 4u, "routes"));
    NVMOE_TRY(check_buffer(p, control, 28u, "control"));
    NVMOE_TRY(check_slots(p, down_slots));
    NVMOE_CUDA(p->device, cudaSetDevice(p->device->ordinal));
    const nvmoe_geometry& g = p->g;
    const uint32_t tiles = (g.hidden_size + g.down_tile_rows - 1u) / g.down_tile_rows;
    launch_route_count((const uint32_t*)routes->ptr, down_slots ? (const uint32_t*)down_slots->ptr : nullptr,
                       down_slots ? (uint32_t)(down_slots->bytes / 4u) : 0u, 2u, (uint32_t*)control->ptr, T, p->K, tiles,
                       p->device->stream);
    p->launches++;
    return post_launch(p, "route count");
}

int nvmoe_quantize_fp8(nvmoe_plan* p, uint32_t rows, uint32_t columns, const nvmoe_buffer* input,
                       nvmoe_buffer* quantized, nvmoe_buffer* scales) {
    if (!p) return NVMOE_ERR_INVALID_ARGUMENT;
    const uint32_t block = p->g.act_block;
    if (rows == 0u || columns == 0u || columns % block)
        return fail(p->device, NVMOE_ERR_INVALID_ARGUMENT, "quantize: %u x %u is not a whole number of %u-column blocks", rows, columns, block);
    NVMOE_TRY(check_buffer(p, input, (size_t)rows * columns * 2u, "input"));
    NVMOE_TRY(check_buffer(p, quantized, (size_t)rows * columns, "quantized"));
    NVMOE_TRY(check_buffer(p, scales, (size_t)rows * (columns / block) * 4u, "scales"));
    NVMOE_CUDA(p->device, cudaSetDevice(p->device->ordinal));
    launch_quantize((const uint16_t*)input->ptr, rows, columns, block, columns, (uint8_t*)quantized->ptr,
                    (float*)scales->ptr, nullptr, p->device->stream);
    p->launches++;
    return post_launch(p, "quantize");
}

// The resolved state for this pair of tables: the cached one when neither table has been written
// since, else a (re)built one in the least recently used place.
static int expert_set_for(nvmoe_plan* p, int set, const nvmoe_buffer* addresses, const nvmoe_buffer* slots, bool tensor,
                          ExpertSet** out) {
    const uint64_t key[4] = {addresses->uid, addresses->version, slots->uid, slots->version};
    const bool cacheable = addresses->owned && slots->owned;
    auto& sets = p->sets[set];
    ExpertSet* found = nullptr;
    for (auto& es : sets)
        if (es->key[0] == key[0] && es->key[2] == key[2]) found = es.get();  // same tables: same place, maybe stale
    if (!found) {
        if (sets.size() < kMaxExpertSets) {
            sets.emplace_back(new (std::nothrow) ExpertSet());
            if (!sets.back()) {
                sets.pop_back();
                return fail(p->device, NVMOE_ERR_OUT_OF_MEMORY, "out of host memory");
            }
            found = sets.back().get();
        } else {
            found = sets[0].get();
            for (auto& es : sets)
                if (es->last_use < found->last_use) found = es.get();
            // kernels of earlier calls may still read the place that is being reused
            NVMOE_CUDA(p->device, cudaStreamSynchronize(p->device->stream));
        }
        found->resolved = found->tensor_ready = false;
    }
    if (!cacheable || found->key[1] != key[1] || found->key[3] != key[3]) found->resolved = found->tensor_ready = false;
    for (int i = 0; i < 4; i++) found->key[i] = key[i];
    found->cacheable = cacheable;
    found->last_use = ++p->use_clock;
    const nvmoe_geometry& g = p->g;
    const uint32_t matrices = set == 0 ? 2u : 1u;
    NVMOE_CUDA(p->device, found->ptrs.ensure(sizeof(ExpertPtrs) * p->experts));
    if (tensor && !found->derived.ptr) {
        const size_t per_matrix = set == 0 ? tc_derived_scale_bytes(g.intermediate_size, g.hidden_size)
                                           : tc_derived_scale_bytes(g.hidden_size, g.intermediate_size);
        NVMOE_CUDA(p->device, found->derived.ensure((size_t)p->experts * matrices * per_matrix));
        NVMOE_CUDA(p->device, found->stamps.ensure((size_t)p->experts * matrices * 16u));
        NVMOE_CUDA(p->device, found->tmaps.ensure((size_t)p->experts * matrices * 128u));
        NVMOE_CUDA(p->device, cudaMemsetAsync(found->stamps.ptr, 0, found->stamps.bytes, p->device->stream));
        found->resolved = found->tensor_ready = false;  // the resolved pointers name the derived copies
    }
    *out = found;
    return NVMOE_OK;
}

// shared tail of the two gate/up entry points and of down
// The resolved expert set of a table pair, with everything the kernels of this call need from it on
// the device: validated pointers and, for the tensor path, re-tiled scales and tensor maps. Launches
// only what the cached state lacks.
static int prepare_expert_set(nvmoe_plan* p, bool gate_up, const nvmoe_buffer* addresses, const nvmoe_buffer* slots,
                              bool tensor, ExpertSet** out) {
    const nvmoe_geometry& g = p->g;
    cudaStream_t st = p->device->stream;
    const int set = gate_up ? 0 : 1;
    ExpertSet* es = nullptr;
    NVMOE_TRY(expert_set_for(p, set, addresses, slots, tensor, &es));
    const uint64_t rows = gate_up ? g.intermediate_size : g.hidden_size;
    const uint64_t cols = gate_up ? g.hidden_size : g.intermediate_size;
    if (!es->resolved || es->resolved_for_tensor != tensor) {
        es->resolved_for_tensor = tensor;
        launch_resolve_experts((const uint32_t*)addresses->ptr, (uint32_t)(addresses->bytes / 4u), (const uint32_t*)slots->ptr,
                               (uint32_t)(slots->bytes / 4u), gate_up ? 4u : 2u, p->experts, (uint32_t)rows, (uint32_t)cols,
                               p->experts - g.native_fp8_resources, tensor, es->derived.as<uint8_t>(),
                               tc_derived_scale_bytes((uint32_t)rows, (uint32_t)cols), es->ptrs.as<ExpertPtrs>(), st);
        p->launches++;
        es->resolved = es->cacheable;
    }
    if (tensor && !es->tensor_ready) {
        ExpertLaunch el{};
        el.work = GroupedWork{nullptr, nullptr, es->ptrs.as<ExpertPtrs>(), p->experts};
        el.scale_stamps = es->stamps.as<uint64_t>();
        el.tmaps = p->tma[set] ? es->tmaps.as<uint8_t>() : nullptr;
        el.g = g;
        launch_derive_scales_tc(el, gate_up, st);
        p->launches += 2;
        if (el.tmaps) {
            launch_build_tensormaps_tc(el, gate_up, p->tmap_templates.as<uint8_t>() + set * 256, st);
            p->launches++;
        }
        es->tensor_ready = es->cacheable;
    }
    *out = es;
    return post_launch(p, gate_up ? "gate/up expert tables" : "down expert tables");
}

// Groups the routes of one expert stage by expert (and, for the tensor path, records where each route
// landed and lists the (expert, token tile) pairs).
static int schedule_stage(nvmoe_plan* p, bool gate_up, ExpertSet* es, uint32_t T, const uint32_t* routes,
                          const uint32_t* intermediates, const uint32_t* control, bool tensor) {
    const int set = gate_up ? 0 : 1;
    cudaStream_t st = p->device->stream;
    launch_group_slots(routes, intermediates, control, es->ptrs.as<ExpertPtrs>(), p->experts, T, p->K, p->g.intermediate_size,
                       p->grouped[set].as<uint32_t>(), p->offsets[set].as<uint32_t>(), p->position[set].as<uint32_t>(),
                       p->status.as<uint32_t>(), sort_scratch(p), st);
    p->launches += (size_t)T * p->K <= 4096u ? 1u : 3u;
    if (tensor) {
        uint32_t* region = p->tile_list.as<uint32_t>() + set * tile_region_words(p);
        launch_build_tiles(p->offsets[set].as<uint32_t>(), p->experts, tc_token_tile_for(T, p->K, p->experts, gate_up), region + 64,
                           region, st);
        p->launches++;
    }
    return post_launch(p, gate_up ? "gate/up schedule" : "down schedule");
}

// Quantises the activations of one expert stage into the form its kernels read: expert-grouped rows
// with E8M0 scales for the tensor path (after the stage has been scheduled), token- or route-ordered
// rows with f32 scales for the CUDA-core path. `source` is the bf16 hidden matrix (gate/up) or the
// intermediates frames (down).
static int quantise_operands(nvmoe_plan* p, bool gate_up, uint32_t T, const void* source, bool tensor) {
    const nvmoe_geometry& g = p->g;
    const int set = gate_up ? 0 : 1;
    cudaStream_t st = p->device->stream;
    if (tensor) {
        launch_quantize_grouped(source, !gate_up, p->grouped[set].as<uint32_t>(), p->offsets[set].as<uint32_t>(), p->experts,
                                T * p->K, p->K, gate_up ? g.hidden_size : g.intermediate_size, g.intermediate_size,
                                g.act_block, p->grouped_q[set].as<uint8_t>(), p->grouped_e8m0[set].as<uint32_t>(), st);
    } else if (gate_up) {
        launch_quantize((const uint16_t*)source, T, g.hidden_size, g.act_block, g.hidden_size, p->xq.as<uint8_t>(),
                        p->x_scales.as<float>(), p->x_e8m0.as<uint32_t>(), st);
    } else {
        launch_quantize_frames((const uint32_t*)source, T, p->K, g.intermediate_size, g.act_block, p->iq.as<uint8_t>(),
                               p->i_scales.as<float>(), p->i_e8m0.as<uint32_t>(), st);
    }
    p->launches++;
    return post_launch(p, gate_up ? "quantize hidden" : "quantize intermediates");
}

struct ExpertCall {
    bool gate_up = true;
    uint32_t T = 0;
    const void* source = nullptr;          // bf16 activations to quantise first (null: operands are ready)
    const uint8_t* pre_q = nullptr;        // pre-quantised contract (CUDA-core path only)
    const float* pre_scales = nullptr;
    const uint32_t* routes = nullptr;
    uint32_t* intermediates = nullptr;
    uint16_t* outputs = nullptr;
    float* partial_outputs = nullptr;      // down only: raw f32 sums instead of weighted bf16 rows
    const nvmoe_buffer* addresses = nullptr;
    const nvmoe_buffer* slots = nullptr;
    const uint32_t* control = nullptr;
    bool allow_tensor_path = true;
    ExpertSet* prepared = nullptr;
    bool scheduled = false;         // grouping (and tile list) already built for this call
    bool fuse_quantise = false;     // gate/up on the tensor path: the epilogue also writes the down stage's operands
};

// shared tail of the two gate/up entry points and of down
static int run_experts(nvmoe_plan* p, const ExpertCall& c) {
    const nvmoe_geometry& g = p->g;
    cudaStream_t st = p->device->stream;
    const bool gate_up = c.gate_up;
    const int set = gate_up ? 0 : 1;
    const uint32_t T = c.T;
    const bool tensor = c.allow_tensor_path && use_tensor_path(p);
    ExpertSet* es = c.prepared;
    if (!es) NVMOE_TRY(prepare_expert_set(p, gate_up, c.addresses, c.slots, tensor, &es));
    if (!c.scheduled) NVMOE_TRY(schedule_stage(p, gate_up, es, T, c.routes, c.intermediates, c.control, tensor));
    if (c.source) NVMOE_TRY(quantise_operands(p, gate_up, T, c.source, tensor));
    ExpertLaunch el{};
    el.work = GroupedWork{p->grouped[set].as<uint32_t>(), p->offsets[set].as<uint32_t>(), es->ptrs.as<ExpertPtrs>(), p->experts};
    if (tensor) {
        el.act_q = p->grouped_q[set].as<uint8_t>();
        el.act_e8m0 = p->grouped_e8m0[set].as<uint32_t>();
    } else if (c.pre_q) {
        el.act_q = c.pre_q;
        el.act_scales = c.pre_scales;
    } else {
        el.act_q = (gate_up ? p->xq : p->iq).as<uint8_t>();
        el.act_scales = (gate_up ? p->x_scales : p->i_scales).as<float>();
        el.act_e8m0 = (gate_up ? p->x_e8m0 : p->i_e8m0).as<uint32_t>();
    }
    el.routes = c.routes;
    el.intermediates = c.intermediates;
    el.outputs = c.outputs;
    el.partial_outputs = c.partial_outputs;
    el.status = p->status.as<uint32_t>();
    el.scale_stamps = es->stamps.as<uint64_t>();
    el.cta_trace = p->cta_trace.as<uint64_t>();
    el.tmaps = tensor && p->tma[set] ? es->tmaps.as<uint8_t>() : nullptr;
    el.tile_count = p->tile_list.as<uint32_t>() + set * tile_region_words(p);  // first word of the stage's region
    el.tile_list = el.tile_count + 64;
    el.tokens = T;
    el.g = g;
    el.wait_cycles = p->wait_cycles;
    el.debug_flags = p->debug_flags;
    if (tensor) {
        const uint32_t size_index = tc_token_tile_index(tc_token_tile_for(T, p->K, p->experts, gate_up));
        el.act_tmap = el.tmaps ? p->act_maps.as<uint8_t>() + (set * 4u + size_index) * 128u : nullptr;
        if (c.fuse_quantise && gate_up) {
            el.q_out = p->grouped_q[1].as<uint8_t>();
            el.q_e8m0 = p->grouped_e8m0[1].as<uint32_t>();
            el.down_position = p->position[1].as<uint32_t>();
        }
    }
    if (p->profile_stages) cudaEventRecord(p->kernel_ev[set][0], st);
    if (tensor) {
        if (gate_up) {
            launch_gate_up_tc(el, st);
        } else {
            launch_down_tc(el, st);
        }
    } else {
        if (gate_up) {
            launch_gate_up_simt(el, st);
        } else {
            launch_down_simt(el, st);
        }
    }
    if (p->profile_stages) cudaEventRecord(p->kernel_ev[set][1], st);
    p->report.tensor_path = tensor ? 1u : 0u;
    p->launches++;
    return post_launch(p, gate_up ? "gate/up" : "down");
}

static int check_expert_tables(nvmoe_plan* p, const nvmoe_buffer* addresses, const nvmoe_buffer* slots, uint32_t params) {
    if (!addresses || !slots) return fail(p->device, NVMOE_ERR_INVALID_ARGUMENT, "address or slot table is null");
    if (addresses->device != p->device || slots->device != p->device)
        return fail(p->device, NVMOE_ERR_INVALID_ARGUMENT, "address or slot table belongs to another device");
    if (addresses->bytes % 32u) return fail(p->device, NVMOE_ERR_INVALID_ARGUMENT, "address table is not a whole number of 32-byte records");
    if (slots->bytes < (size_t)p->experts * params * 4u)
        return fail(p->device, NVMOE_ERR_INVALID_ARGUMENT, "slot table holds %zu bytes, %u experts x %u parameters need %zu",
                    slots->bytes, p->experts, params, (size_t)p->experts * params * 4u);
    return NVMOE_OK;
}

int nvmoe_gate_up(nvmoe_plan* p, uint32_t T, const nvmoe_buffer* hidden, const nvmoe_buffer* routes,
                  nvmoe_buffer* intermediates, const nvmoe_buffer* addresses, const nvmoe_buffer* slots,
                  const nvmoe_buffer* control) {
    if (!p) return NVMOE_ERR_INVALID_ARGUMENT;
    NVMOE_TRY(check_tokens(p, T));
    const nvmoe_geometry& g = p->g;
    NVMOE_TRY(check_buffer(p, hidden, (size_t)T * g.hidden_size * 2u, "hidden"));
    NVMOE_TRY(check_buffer(p, routes, (size_t)T * p->K * 4u, "routes"));
    NVMOE_TRY(check_buffer(p, intermediates, (size_t)T * p->frame_words * 4u, "intermediates"));
    NVMOE_TRY(check_buffer(p, control, 28u, "control"));
    NVMOE_TRY(check_expert_tables(p, addresses, slots, 4u));
    NVMOE_CUDA(p->device, cudaSetDevice(p->device->ordinal));
    ExpertCall c;
    c.gate_up = true;
    c.T = T;
    c.source = hidden->ptr;
    c.routes = (const uint32_t*)routes->ptr;
    c.intermediates = (uint32_t*)intermediates->ptr;
    c.addresses = addresses;
    c.slots = slots;
    c.control = (const uint32_t*)control->ptr;
    return run_experts(p, c);
}

int nvmoe_gate_up_prequant(nvmoe_plan* p, uint32_t T, const nvmoe_buffer* quantized_hidden,
                           const nvmoe_buffer* hidden_scales, const nvmoe_buffer* routes, nvmoe_buffer* intermediates,
                           const nvmoe_buffer* addresses, const nvmoe_buffer* slots, const nvmoe_buffer* control) {
    if (!p) return NVMOE_ERR_INVALID_ARGUMENT;
    NVMOE_TRY(check_tokens(p, T));
    const nvmoe_geometry& g = p->g;
    NVMOE_TRY(check_buffer(p, quantized_hidden, (size_t)T * g.hidden_size, "quantized hidden"));
    NVMOE_TRY(check_buffer(p, hidden_scales, (size_t)T * (g.hidden_size / g.act_block) * 4u, "hidden scales"));
    NVMOE_TRY(check_buffer(p, routes, (size_t)T * p->K * 4u, "routes"));
    NVMOE_TRY(check_buffer(p, intermediates, (size_t)T * p->frame_words * 4u, "intermediates"));
    NVMOE_TRY(check_buffer(p, control, 28u, "control"));
    NVMOE_TRY(check_expert_tables(p, addresses, slots, 4u));
    NVMOE_CUDA(p->device, cudaSetDevice(p->device->ordinal));
    // the f32 scales of this contract need not be powers of two: the CUDA-core kernels take them as they are
    ExpertCall c;
    c.gate_up = true;
    c.T = T;
    c.pre_q = (const uint8_t*)quantized_hidden->ptr;
    c.pre_scales = (const float*)hidden_scales->ptr;
    c.routes = (const uint32_t*)routes->ptr;
    c.intermediates = (uint32_t*)intermediates->ptr;
    c.addresses = addresses;
    c.slots = slots;
    c.control = (const uint32_t*)control->ptr;
    c.allow_tensor_path = false;
    return run_experts(p, c);
}

int nvmoe_down(nvmoe_plan* p, uint32_t T, const nvmoe_buffer* intermediates, const nvmoe_buffer* routes,
               nvmoe_buffer* outputs, const nvmoe_buffer* addresses, const nvmoe_buffer* slots,
               const nvmoe_buffer* control) {
    if (!p) return NVMOE_ERR_INVALID_ARGUMENT;
    NVMOE_TRY(check_tokens(p, T));
    const nvmoe_geometry& g = p->g;
    NVMOE_TRY(check_buffer(p, intermediates, (size_t)T * p->frame_words * 4u, "intermediates"));
    NVMOE_TRY(check_buffer(p, routes, (size_t)T * p->K * 4u, "routes"));
    NVMOE_TRY(check_buffer(p, outputs, (size_t)T * p->K * g.hidden_size * 2u, "expert outputs"));
    NVMOE_TRY(check_buffer(p, control, 28u, "control"));
    NVMOE_TRY(check_expert_tables(p, addresses, slots, 2u));
    NVMOE_CUDA(p->device, cudaSetDevice(p->device->ordinal));
    ExpertCall c;
    c.gate_up = false;
    c.T = T;
    c.source = intermediates->ptr;
    c.routes = (const uint32_t*)routes->ptr;
    c.intermediates = (uint32_t*)intermediates->ptr;
    c.outputs = (uint16_t*)outputs->ptr;
    c.addresses = addresses;
    c.slots = slots;
    c.control = (const uint32_t*)control->ptr;
    return run_experts(p, c);
}

int nvmoe_down_partial(nvmoe_plan* p, uint32_t T, const nvmoe_buffer* intermediates, const nvmoe_buffer* routes,
                       nvmoe_buffer* partial_outputs, const nvmoe_buffer* addresses, const nvmoe_buffer* slots,
                       const nvmoe_buffer* control) {
    if (!p) return NVMOE_ERR_INVALID_ARGUMENT;
    NVMOE_TRY(check_tokens(p, T));
    const nvmoe_geometry& g = p->g;
    const size_t out_bytes = (size_t)T * p->K * g.hidden_size * 4u;
    NVMOE_TRY(check_buffer(p, intermediates, (size_t)T * p->frame_words * 4u, "intermediates"));
    NVMOE_TRY(check_buffer(p, routes, (size_t)T * p->K * 4u, "routes"));
    NVMOE_TRY(check_buffer(p, partial_outputs, out_bytes, "partial expert outputs"));
    NVMOE_TRY(check_buffer(p, control, 28u, "control"));
    NVMOE_TRY(check_expert_tables(p, addresses, slots, 2u));
    NVMOE_CUDA(p->device, cudaSetDevice(p->device->ordinal));
    // a route this participant skips contributes a plane of zeros to the sum
    NVMOE_CUDA(p->device, cudaMemsetAsync(partial_outputs->ptr, 0, out_bytes, p->device->stream));
    ExpertCall c;
    c.gate_up = false;
    c.T = T;
    c.source = intermediates->ptr;
    c.routes = (const uint32_t*)routes->ptr;
    c.intermediates = (uint32_t*)intermediates->ptr;
    c.partial_outputs = (float*)partial_outputs->ptr;
    c.addresses = addresses;
    c.slots = slots;
    c.control = (const uint32_t*)control->ptr;
    return run_experts(p, c);
}

int nvmoe_sum_f32_scale_packed_bf16(nvmoe_plan* p, const nvmoe_buffer* partials, const nvmoe_buffer* scales, nvmoe_buffer* output,
                                    uint32_t element_count, uint32_t participant_count, uint32_t lane_count,
                                    uint32_t elements_per_scale, uint32_t scale_bit_offset) {
    if (!p) return NVMOE_ERR_INVALID_ARGUMENT;
    if (element_count == 0u || element_count % 2u || participant_count == 0u || lane_count == 0u || elements_per_scale == 0u ||
        element_count % elements_per_scale || elements_per_scale % 2u || (scale_bit_offset != 0u && scale_bit_offset != 16u))
        return fail(p->device, NVMOE_ERR_INVALID_ARGUMENT,
                    "sum_f32_scale_packed_bf16: %u elements (even), %u participants, %u lanes, one scale per %u elements (an even "
                    "divisor), bit offset %u (0 or 16)", element_count, participant_count, lane_count, elements_per_scale, scale_bit_offset);
    NVMOE_TRY(check_buffer(p, partials, (size_t)participant_count * lane_count * element_count * 4u, "partial planes"));
    NVMOE_TRY(check_buffer(p, scales, (size_t)lane_count * (element_count / elements_per_scale) * 4u, "packed scales"));
    NVMOE_TRY(check_buffer(p, output, (size_t)lane_count * element_count * 2u, "output"));
    NVMOE_CUDA(p->device, cudaSetDevice(p->device->ordinal));
    launch_sum_f32_scale_packed_bf16((const float*)partials->ptr, (const uint32_t*)scales->ptr, (uint32_t*)output->ptr, element_count,
                                     participant_count, lane_count, elements_per_scale, scale_bit_offset, p->device->stream);
    p->launches++;
    return post_launch(p, "sum_f32_scale_packed_bf16");
}

int nvmoe_reduce(nvmoe_plan* p, uint32_t T, const nvmoe_buffer* expert_outputs, nvmoe_buffer* output) {
    if (!p) return NVMOE_ERR_INVALID_ARGUMENT;
    NVMOE_TRY(check_tokens(p, T));
    const nvmoe_geometry& g = p->g;
    NVMOE_TRY(check_buffer(p, expert_outputs, (size_t)T * p->K * g.hidden_size * 2u, "expert outputs"));
    NVMOE_TRY(check_buffer(p, output, (size_t)T * g.hidden_size * 2u, "output"));
    NVMOE_CUDA(p->device, cudaSetDevice(p->device->ordinal));
    launch_reduce((const uint16_t*)expert_outputs->ptr, (uint16_t*)output->ptr, T, p->K, g.hidden_size, g.reduce_scale,
                  nullptr, p->device->stream);
    p->launches++;
    return post_launch(p, "reduce");
}

// ---- token-id table routing -----------------------------------------------------------------------

int nvmoe_resource_preselect_table(nvmoe_plan* p, uint32_t T, const nvmoe_buffer* token_ids, nvmoe_buffer* resource_routes,
                                   const nvmoe_buffer* table, uint32_t vocab_size, uint32_t table_word_stride,
                                   nvmoe_buffer* telemetry) {
    if (!p) return NVMOE_ERR_INVALID_ARGUMENT;
    NVMOE_TRY(check_tokens(p, T));
    const nvmoe_geometry& g = p->g;
    if (vocab_size == 0u || (table_word_stride != 1u && table_word_stride != 2u))
        return fail(p->device, NVMOE_ERR_INVALID_ARGUMENT, "preselection table of %u rows with %u-word elements (1 = I32, 2 = I64)",
                    vocab_size, table_word_stride);
    NVMOE_TRY(check_buffer(p, token_ids, (size_t)T * 4u, "token ids"));
    NVMOE_TRY(check_buffer(p, resource_routes, (size_t)T * p->K * 4u, "resource routes"));
    NVMOE_TRY(check_buffer(p, table, (size_t)vocab_size * g.routed_k * table_word_stride * 4u, "preselection table"));
    if (telemetry) {
        const size_t r = p->experts;
        NVMOE_TRY(check_buffer(p, telemetry, (r + r * (r - 1u) / 2u) * 4u, "telemetry"));
    }
    NVMOE_CUDA(p->device, cudaSetDevice(p->device->ordinal));
    launch_preselect_table((const uint32_t*)token_ids->ptr, (const uint32_t*)table->ptr, table_word_stride, vocab_size,
                           g.routed_experts, g.routed_k, g.always_count, T, (uint32_t*)resource_routes->ptr,
                           telemetry ? (uint32_t*)telemetry->ptr : nullptr, p->status.as<uint32_t>(), p->device->stream);
    p->launches++;
    return post_launch(p, "resource preselection");
}

int nvmoe_route_preselected(nvmoe_plan* p, uint32_t T, const nvmoe_buffer* logits, const nvmoe_buffer* resource_routes,
                            nvmoe_buffer* routes) {
    if (!p) return NVMOE_ERR_INVALID_ARGUMENT;
    NVMOE_TRY(check_tokens(p, T));
    const nvmoe_geometry& g = p->g;
    if (g.router_kind != NVMOE_ROUTER_PRESELECTED)
        return fail(p->device, NVMOE_ERR_INVALID_ARGUMENT, "this plan's router selects by score: call nvmoe_route");
    NVMOE_TRY(check_buffer(p, logits, (size_t)T * ((g.routed_experts + 1u) / 2u) * 4u, "logits"));
    NVMOE_TRY(check_buffer(p, resource_routes, (size_t)T * p->K * 4u, "resource routes"));
    NVMOE_TRY(check_buffer(p, routes, (size_t)T * p->K * 4u, "routes"));
    NVMOE_CUDA(p->device, cudaSetDevice(p->device->ordinal));
    launch_route_preselected((const uint32_t*)logits->ptr, (const uint32_t*)resource_routes->ptr, T, (uint32_t*)routes->ptr,
                             p->status.as<uint32_t>(), g, p->device->stream);
    p->launches++;
    return post_launch(p, "preselected router");
}

// ---- the nodes either side of the MoE chain ----------------------------------------------------------

int nvmoe_rms_norm(nvmoe_plan* p, uint32_t rows, uint32_t element_count, const nvmoe_buffer* input, nvmoe_buffer* output,
                   const nvmoe_buffer* weight, float eps, float weight_offset) {
    if (!p) return NVMOE_ERR_INVALID_ARGUMENT;
    if (rows == 0u || element_count == 0u || element_count % 2u)
        return fail(p->device, NVMOE_ERR_INVALID_ARGUMENT, "rms_norm: %u rows of %u elements (an even, positive count is required)", rows,
                    element_count);
    if (!(eps >= 0.0f)) return fail(p->device, NVMOE_ERR_INVALID_ARGUMENT, "rms_norm: epsilon must not be negative");
    NVMOE_TRY(check_buffer(p, input, (size_t)rows * element_count * 2u, "input"));
    NVMOE_TRY(check_buffer(p, output, (size_t)rows * element_count * 2u, "output"));
    NVMOE_TRY(check_buffer(p, weight, (size_t)element_count * 2u, "norm weight"));
    NVMOE_CUDA(p->device, cudaSetDevice(p->device->ordinal));
    launch_rms_norm((const uint16_t*)input->ptr, (const uint16_t*)weight->ptr, (uint16_t*)output->ptr, rows, element_count, eps,
                    weight_offset, p->device->stream);
    p->launches++;
    return post_launch(p, "rms_norm");
}

static int pairwise_checks(nvmoe_plan* p, uint32_t rows, uint32_t element_count, const nvmoe_buffer* a, const nvmoe_buffer* b,
                           const nvmoe_buffer* out, const char* what) {
    if (rows == 0u || element_count == 0u || element_count % 2u)
        return fail(p->device, NVMOE_ERR_INVALID_ARGUMENT, "%s: %u rows of %u elements (an even, positive count is required)", what,
                    rows, element_count);
    const size_t bytes = (size_t)rows * element_count * 2u;
    NVMOE_TRY(check_buffer(p, a, bytes, "first input"));
    NVMOE_TRY(check_buffer(p, b, bytes, "second input"));
    NVMOE_TRY(check_buffer(p, out, bytes, "output"));
    return NVMOE_OK;
}

int nvmoe_silu_multiply(nvmoe_plan* p, uint32_t rows, uint32_t element_count, const nvmoe_buffer* gate, const nvmoe_buffer* up,
                        nvmoe_buffer* output, float limit) {
    if (!p) return NVMOE_ERR_INVALID_ARGUMENT;
    if (!(limit >= 0.0f)) return fail(p->device, NVMOE_ERR_INVALID_ARGUMENT, "silu_multiply: the clamp limit must not be negative");
    NVMOE_TRY(pairwise_checks(p, rows, element_count, gate, up, output, "silu_multiply"));
    NVMOE_CUDA(p->device, cudaSetDevice(p->device->ordinal));
    launch_silu_multiply((const uint16_t*)gate->ptr, (const uint16_t*)up->ptr, (uint16_t*)output->ptr, (size_t)rows * element_count,
                         limit, p->device->stream);
    p->launches++;
    return post_launch(p, "silu_multiply");
}

int nvmoe_residual_add(nvmoe_plan* p, uint32_t rows, uint32_t element_count, const nvmoe_buffer* a, const nvmoe_buffer* b,
                       nvmoe_buffer* output) {
    if (!p) return NVMOE_ERR_INVALID_ARGUMENT;
    NVMOE_TRY(pairwise_checks(p, rows, element_count, a, b, output, "residual_add"));
    NVMOE_CUDA(p->device, cudaSetDevice(p->device->ordinal));
    launch_add_bf16((const uint16_t*)a->ptr, (const uint16_t*)b->ptr, (uint16_t*)output->ptr, (size_t)rows * element_count,
                    p->device->stream);
    p->launches++;
    return post_launch(p, "residual_add");
}

// A dense linear over packaged MXFP4 weights is the down projection of one always-selected resource
// with route weight one: the same quantisation, kernels and rounding as an expert's, on a plan of the
// linear's own shape that this plan keeps.
int nvmoe_dense_linear(nvmoe_plan* p, uint32_t T, const nvmoe_buffer* input, nvmoe_buffer* output, const nvmoe_buffer* weights,
                       const nvmoe_buffer* scales, uint32_t rows, uint32_t cols) {
    if (!p) return NVMOE_ERR_INVALID_ARGUMENT;
    NVMOE_TRY(check_tokens(p, T));
    nvmoe_device* d = p->device;
    if (rows == 0u || cols == 0u || rows % 32u || cols % 32u || cols % p->g.act_block)
        return fail(d, NVMOE_ERR_INVALID_ARGUMENT, "dense linear %u x %u: both sizes must be multiples of 32 and the input size of the "
                    "activation block %u", rows, cols, p->g.act_block);
    NVMOE_TRY(check_buffer(p, input, (size_t)T * cols * 2u, "input"));
    NVMOE_TRY(check_buffer(p, output, (size_t)T * rows * 2u, "output"));
    NVMOE_TRY(check_buffer(p, weights, (size_t)rows * (cols / 2u), "weights"));
    NVMOE_TRY(check_buffer(p, scales, (size_t)rows * (cols / 32u), "weight scales"));
    NVMOE_CUDA(d, cudaSetDevice(d->ordinal));
    nvmoe_plan::DenseLinear* dl = nullptr;
    for (auto& entry : p->dense)
        if (entry.rows == rows && entry.cols == cols) dl = &entry;
    if (!dl) {
        nvmoe_plan::DenseLinear fresh;
        fresh.rows = rows;
        fresh.cols = cols;
        nvmoe_geometry g{};
        nvmoe_geometry_default(&g, rows, cols, 1u, 1u);
        g.act_block = p->g.act_block;
        g.max_tokens = p->g.max_tokens;
        NVMOE_TRY(nvmoe_plan_create(d, &g, &fresh.plan));
        fresh.plan->expert_path = p->expert_path;
        int rc = nvmoe_buffer_create(d, 64u, &fresh.addresses);
        if (rc == NVMOE_OK) rc = nvmoe_buffer_create(d, 8u, &fresh.slots);
        const uint32_t slot_words[2] = {0u, 1u};
        if (rc == NVMOE_OK) rc = nvmoe_buffer_write(fresh.slots, 0, slot_words, 8u);
        if (rc == NVMOE_OK && fresh.unit_routes.ensure((size_t)g.max_tokens * 4u) != cudaSuccess)
            rc = fail(d, NVMOE_ERR_OUT_OF_MEMORY, "dense linear: out of device memory");
        if (rc == NVMOE_OK) {
            std::vector<uint32_t> ones(g.max_tokens, 0x3f80u << 16);  // weight 1.0, resource 0
            if (cudaMemcpy(fresh.unit_routes.ptr, ones.data(), ones.size() * 4u, cudaMemcpyHostToDevice) != cudaSuccess)
                rc = fail(d, NVMOE_ERR_CUDA, "dense linear: could not write the unit routes");
        }
        if (rc != NVMOE_OK) {
            nvmoe_plan_destroy(fresh.plan);
            nvmoe_buffer_destroy(fresh.addresses);
            nvmoe_buffer_destroy(fresh.slots);
            fresh.unit_routes.release();
            return rc;
        }
        p->dense.push_back(fresh);
        dl = &p->dense.back();
    }
    nvmoe_plan* sub = dl->plan;
    sub->expert_path = p->expert_path;
    sub->wait_cycles = p->wait_cycles;
    if (dl->weights != weights->ptr || dl->scales != scales->ptr || dl->weights_version != weights->version ||
        dl->scales_version != scales->version) {
        // the two address records of the one resource: {address, byte count, generation, resident, representation}
        uint64_t records[8] = {(uint64_t)(uintptr_t)weights->ptr, (uint64_t)rows * (cols / 2u), 1u + weights->version, 1u,
                               (uint64_t)(uintptr_t)scales->ptr,  (uint64_t)rows * (cols / 32u), 1u + scales->version, 1u};
        NVMOE_TRY(nvmoe_buffer_write(dl->addresses, 0, records, sizeof records));
        dl->weights = weights->ptr;
        dl->scales = scales->ptr;
        dl->weights_version = weights->version;
        dl->scales_version = scales->version;
    }
    cudaStream_t st = d->stream;
    const bool tensor = use_tensor_path(sub);
    ExpertSet* es = nullptr;
    NVMOE_TRY(prepare_expert_set(sub, false, dl->addresses, dl->slots, tensor, &es));
    uint32_t* region = sub->tile_list.as<uint32_t>() + tile_region_words(sub);
    launch_dense_schedule(T, tc_token_tile_for(T, 1u, 1u, false), sub->grouped[1].as<uint32_t>(), sub->offsets[1].as<uint32_t>(),
                          sub->position[1].as<uint32_t>(), tensor ? region + 64 : nullptr, tensor ? region : nullptr, st);
    sub->launches++;
    NVMOE_TRY(post_launch(sub, "dense linear schedule"));
    if (tensor) {
        launch_quantize_grouped(input->ptr, false, sub->grouped[1].as<uint32_t>(), sub->offsets[1].as<uint32_t>(), 1u, T, 1u, cols, cols,
                                sub->g.act_block, sub->grouped_q[1].as<uint8_t>(), sub->grouped_e8m0[1].as<uint32_t>(), st);
    } else {
        launch_quantize((const uint16_t*)input->ptr, T, cols, sub->g.act_block, cols, sub->iq.as<uint8_t>(), sub->i_scales.as<float>(),
                        sub->i_e8m0.as<uint32_t>(), st);
    }
    sub->launches++;
    NVMOE_TRY(post_launch(sub, "dense linear quantise"));
    ExpertCall call;
    call.gate_up = false;
    call.T = T;
    call.routes = dl->unit_routes.as<uint32_t>();
    call.outputs = (uint16_t*)output->ptr;
    call.prepared = es;
    call.scheduled = true;
    NVMOE_TRY(run_experts(sub, call));
    p->launches += sub->launches;
    sub->launches = 0;
    return NVMOE_OK;
}

// ---- expert-parallel exchange helpers -----------------------------------------------------------

int nvmoe_ep_pack(nvmoe_plan* p, uint32_t T, const nvmoe_buffer* hidden, const nvmoe_buffer* routes,
                  const nvmoe_buffer* owner_table, uint32_t world, uint32_t rank, nvmoe_buffer* send_rows,
                  nvmoe_buffer* send_routes, nvmoe_buffer* send_index, nvmoe_buffer* dest_counts, uint32_t segment_rows) {
    if (!p) return NVMOE_ERR_INVALID_ARGUMENT;
    NVMOE_TRY(check_tokens(p, T));
    const nvmoe_geometry& g = p->g;
    if (world == 0u || world > 1024u || rank >= world)
        return fail(p->device, NVMOE_ERR_INVALID_ARGUMENT, "rank %u of %u is not a valid expert-parallel position", rank, world);
    const size_t R = (size_t)T * p->K;
    NVMOE_TRY(check_buffer(p, hidden, (size_t)T * g.hidden_size * 2u, "hidden"));
    NVMOE_TRY(check_buffer(p, routes, R * 4u, "routes"));
    NVMOE_TRY(check_buffer(p, owner_table, (size_t)p->experts * 4u, "owner table"));
    const size_t send_slots = segment_rows ? (size_t)world * segment_rows : R;
    NVMOE_TRY(check_buffer(p, send_rows, send_slots * g.hidden_size * 2u, "send rows"));
    NVMOE_TRY(check_buffer(p, send_routes, send_slots * 4u, "send routes"));
    NVMOE_TRY(check_buffer(p, send_index, R * 4u, "send index"));
    NVMOE_TRY(check_buffer(p, dest_counts, (size_t)world * 4u, "destination counts"));
    NVMOE_CUDA(p->device, cudaSetDevice(p->device->ordinal));
    cudaError_t err = p->ep_source.ensure(((size_t)p->g.max_tokens * p->K * 2u + 64u) * 4u);
    if (err != cudaSuccess) return fail(p->device, NVMOE_ERR_OUT_OF_MEMORY, "exchange scratch allocation failed: %s", cudaGetErrorString(err));
    if ((size_t)world > (size_t)p->experts + 1u)
        return fail(p->device, NVMOE_ERR_INVALID_ARGUMENT, "more ranks (%u) than resources (%u)", world, p->experts);
    uint32_t* total = p->ep_source.as<uint32_t>();
    launch_ep_pack((const uint16_t*)hidden->ptr, (const uint32_t*)routes->ptr, (const uint32_t*)owner_table->ptr, T, p->K,
                   g.hidden_size, p->experts, world, rank, (uint16_t*)send_rows->ptr, (uint32_t*)send_routes->ptr,
                   (uint32_t*)send_index->ptr, total + 64, (uint32_t*)dest_counts->ptr, total, segment_rows,
                   total + 64 + (size_t)p->g.max_tokens * p->K, p->status.as<uint32_t>(), sort_scratch(p), p->device->stream);
    p->launches += segment_rows ? 2 : 3;
    return post_launch(p, "expert-parallel pack");
}

int nvmoe_ep_unpack(nvmoe_plan* p, uint32_t T, const nvmoe_buffer* returned_rows, const nvmoe_buffer* send_index,
                    nvmoe_buffer* expert_outputs) {
    // (returned_rows holds at least T*K rows; in the padded layout it holds world * segment_rows and the
    // positions in send_index are slots of that layout)
    if (!p) return NVMOE_ERR_INVALID_ARGUMENT;
    NVMOE_TRY(check_tokens(p, T));
    const size_t R = (size_t)T * p->K;
    NVMOE_TRY(check_buffer(p, returned_rows, R * p->g.hidden_size * 2u, "returned rows"));
    NVMOE_TRY(check_buffer(p, send_index, R * 4u, "send index"));
    NVMOE_TRY(check_buffer(p, expert_outputs, R * p->g.hidden_size * 2u, "expert outputs"));
    NVMOE_CUDA(p->device, cudaSetDevice(p->device->ordinal));
    launch_ep_unpack((const uint16_t*)returned_rows->ptr, (const uint32_t*)send_index->ptr, T, p->K, p->g.hidden_size,
                     (uint16_t*)expert_outputs->ptr, p->device->stream);
    p->launches++;
    return post_launch(p, "expert-parallel unpack");
}

// ---- fused layer -------------------------------------------------------------------------------

static int ensure_layer_scratch(nvmoe_plan* p) {
    const nvmoe_geometry& g = p->g;
    const size_t T = g.max_tokens;
    cudaError_t err = cudaSuccess;
    auto want = [&](DeviceArray& a, size_t bytes) {
        if (err == cudaSuccess) err = a.ensure(bytes);
    };
    const bool fresh_frames = p->frames.ptr == nullptr;
    want(p->logits, T * ((g.routed_experts + 1u) / 2u) * 4u);
    want(p->routes, T * p->K * 4u);
    want(p->frames, T * (size_t)p->frame_words * 4u);
    want(p->expert_outputs, T * p->K * (size_t)g.hidden_size * 2u);
    want(p->controls, 64u);
    if (err == cudaSuccess && fresh_frames) err = cudaMemsetAsync(p->frames.ptr, 0, p->frames.bytes, p->device->stream);
    if (err != cudaSuccess)
        return fail(p->device, err == cudaErrorMemoryAllocation ? NVMOE_ERR_OUT_OF_MEMORY : NVMOE_ERR_CUDA,
                    "layer scratch allocation failed: %s", cudaGetErrorString(err));
    return NVMOE_OK;
}

int nvmoe_layer(nvmoe_plan* p, const nvmoe_layer_args* a) {
    if (!p || !a) return NVMOE_ERR_INVALID_ARGUMENT;
    const uint32_t T = a->batch_width;
    NVMOE_TRY(check_tokens(p, T));
    const nvmoe_geometry& g = p->g;
    nvmoe_device* d = p->device;
    if (!a->router_weights && !a->logits && !a->routes_in)
        return fail(d, NVMOE_ERR_INVALID_ARGUMENT, "the layer needs router weights, precomputed logits or preselected routes");
    if (a->expert_count && (uint64_t)a->expert_start + a->expert_count > p->experts)
        return fail(d, NVMOE_ERR_INVALID_ARGUMENT, "expert range [%u, %u) exceeds %u resources", a->expert_start,
                    a->expert_start + a->expert_count, p->experts);
    NVMOE_TRY(check_buffer(p, a->hidden, (size_t)T * g.hidden_size * 2u, "hidden"));
    if (a->expert_outputs) {
        NVMOE_TRY(check_buffer(p, a->expert_outputs, (size_t)T * p->K * g.hidden_size * 2u, "expert outputs"));
    } else {
        NVMOE_TRY(check_buffer(p, a->output, (size_t)T * g.hidden_size * 2u, "output"));
    }
    if (a->routes_in) NVMOE_TRY(check_buffer(p, a->routes_in, (size_t)T * p->K * 4u, "routes"));
    NVMOE_TRY(check_expert_tables(p, a->gate_up_addresses, a->gate_up_slots, 4u));
    NVMOE_TRY(check_expert_tables(p, a->down_addresses, a->down_slots, 2u));
    if (a->routes_out) NVMOE_TRY(check_buffer(p, a->routes_out, (size_t)T * p->K * 4u, "routes"));
    NVMOE_CUDA(d, cudaSetDevice(d->ordinal));
    NVMOE_TRY(ensure_layer_scratch(p));
    cudaStream_t st = d->stream;
    const uint32_t launches_before = p->launches;
    const bool prof = p->profile_stages;
    auto mark = [&](int i) {
        if (prof || i == 0 || i == kStageCount) cudaEventRecord(p->ev[i], st);
    };

    nvmoe_buffer logits_view{d, p->logits.ptr, p->logits.bytes};
    nvmoe_buffer* logits = a->logits ? a->logits : &logits_view;
    nvmoe_buffer routes_view{d, p->routes.ptr, p->routes.bytes};
    nvmoe_buffer* routes = a->routes_in ? const_cast<nvmoe_buffer*>(a->routes_in) : a->routes_out ? a->routes_out : &routes_view;
    nvmoe_buffer frames{d, p->frames.ptr, p->frames.bytes};
    nvmoe_buffer outs{d, p->expert_outputs.ptr, p->expert_outputs.bytes};
    if (a->expert_outputs) outs = *a->expert_outputs;
    nvmoe_buffer gate_control{d, p->controls.ptr, 28u};
    nvmoe_buffer down_control{d, (char*)p->controls.ptr + 32u, 28u};

    mark(kStageLinear);
    if (a->router_weights && !a->routes_in)
        NVMOE_TRY(nvmoe_router_linear(p, T, a->hidden, logits, a->router_weights, a->router_bias));
    mark(kStageRoute);
    if (!a->routes_in) NVMOE_TRY(nvmoe_route(p, T, logits, routes, a->bias, a->telemetry));
    mark(kStageSchedule);
    const bool tensor = use_tensor_path(p);
    // with 32-wide scale blocks the tensor-path gate/up epilogue quantises its own output for the down stage
    const bool fused_quantise = tensor && g.act_block == 32u;
    ExpertSet* sets[2] = {nullptr, nullptr};
    NVMOE_TRY(prepare_expert_set(p, true, a->gate_up_addresses, a->gate_up_slots, tensor, &sets[0]));
    NVMOE_TRY(prepare_expert_set(p, false, a->down_addresses, a->down_slots, tensor, &sets[1]));
    if (layer_schedule_is_small(T, p->K, p->experts)) {
        LayerSchedule ls{};
        ls.routes = (const uint32_t*)routes->ptr;
        ls.intermediates = (uint32_t*)frames.ptr;
        ls.slots[0] = (const uint32_t*)a->gate_up_slots->ptr;
        ls.slots[1] = (const uint32_t*)a->down_slots->ptr;
        ls.slot_words[0] = (uint32_t)(a->gate_up_slots->bytes / 4u);
        ls.slot_words[1] = (uint32_t)(a->down_slots->bytes / 4u);
        ls.control[0] = (uint32_t*)gate_control.ptr;
        ls.control[1] = (uint32_t*)down_control.ptr;
        for (int i = 0; i < 2; i++) {
            ls.experts[i] = sets[i]->ptrs.as<ExpertPtrs>();
            ls.grouped[i] = p->grouped[i].as<uint32_t>();
            ls.offsets[i] = p->offsets[i].as<uint32_t>();
            ls.position[i] = p->position[i].as<uint32_t>();
            ls.tile_count[i] = tensor ? p->tile_list.as<uint32_t>() + i * tile_region_words(p) : nullptr;
            ls.tiles[i] = tensor ? ls.tile_count[i] + 64 : nullptr;
        }
        ls.status = p->status.as<uint32_t>();
        ls.tokens = T;
        ls.expert_start = a->expert_start;
        ls.expert_count = a->expert_count;
        ls.K = p->K;
        ls.I = g.intermediate_size;
        ls.tiles_per_route[0] = (g.intermediate_size + g.gate_tile_rows - 1u) / g.gate_tile_rows;
        ls.tiles_per_route[1] = (g.hidden_size + g.down_tile_rows - 1u) / g.down_tile_rows;
        ls.num_experts = p->experts;
        ls.n_tile[0] = tc_token_tile_for(T, p->K, p->experts, true);
        ls.n_tile[1] = tc_token_tile_for(T, p->K, p->experts, false);
        launch_layer_schedule_small(ls, st);
        p->launches++;
        NVMOE_TRY(post_launch(p, "layer schedule"));
    } else {
        write_control_kernel<<<1, 32, 0, st>>>((uint32_t*)gate_control.ptr, T, a->expert_start, a->expert_count);
        write_control_kernel<<<1, 32, 0, st>>>((uint32_t*)down_control.ptr, T, a->expert_start, a->expert_count);
        p->launches += 2;
        NVMOE_TRY(nvmoe_route_compact(p, T, routes, &frames, a->gate_up_slots, &gate_control));
        NVMOE_TRY(nvmoe_route_count(p, T, routes, a->down_slots, &down_control));
        // both stages are grouped before the first runs: gate/up's epilogue needs to know where the down
        // stage will look for each route's activations
        NVMOE_TRY(schedule_stage(p, true, sets[0], T, (const uint32_t*)routes->ptr, (const uint32_t*)frames.ptr,
                                 (const uint32_t*)gate_control.ptr, tensor));
        NVMOE_TRY(schedule_stage(p, false, sets[1], T, (const uint32_t*)routes->ptr, (const uint32_t*)frames.ptr,
                                 (const uint32_t*)down_control.ptr, tensor));
    }
    mark(kStageQuantX);
    NVMOE_TRY(quantise_operands(p, true, T, a->hidden->ptr, tensor));
    mark(kStageGateUp);
    ExpertCall call;
    call.T = T;
    call.routes = (const uint32_t*)routes->ptr;
    call.intermediates = (uint32_t*)frames.ptr;
    call.scheduled = true;
    call.gate_up = true;
    call.addresses = a->gate_up_addresses;
    call.slots = a->gate_up_slots;
    call.control = (const uint32_t*)gate_control.ptr;
    call.prepared = sets[0];
    call.fuse_quantise = fused_quantise;
    NVMOE_TRY(run_experts(p, call));
    mark(kStageQuantI);
    if (!fused_quantise) NVMOE_TRY(quantise_operands(p, false, T, frames.ptr, tensor));
    mark(kStageDown);
    // routes that are skipped (owned by another device, expert not resident) leave their rows untouched:
    // the combine below reads the down stage's position table and counts them as zeros; rows handed to
    // the caller instead start at zero
    if (a->expert_outputs) cudaMemsetAsync(outs.ptr, 0, (size_t)T * p->K * g.hidden_size * 2u, st);
    call.gate_up = false;
    call.outputs = (uint16_t*)outs.ptr;
    call.addresses = a->down_addresses;
    call.slots = a->down_slots;
    call.control = (const uint32_t*)down_control.ptr;
    call.prepared = sets[1];
    call.fuse_quantise = false;
    NVMOE_TRY(run_experts(p, call));
    mark(kStageReduce);
    if (!a->expert_outputs) {
        launch_reduce((const uint16_t*)outs.ptr, (uint16_t*)a->output->ptr, T, p->K, g.hidden_size, g.reduce_scale,
                      p->position[1].as<uint32_t>(), st);
        p->launches++;
        NVMOE_TRY(post_launch(p, "reduce"));
    }
    mark(kStageCount);
    p->events_valid = true;
    p->report.batch_width = T;
    p->report.routes = T * p->K;
    p->report.kernel_launches = p->launches - launches_before;
    return NVMOE_OK;
}

int nvmoe_layer_host(nvmoe_plan* p, const nvmoe_layer_args* args, const void* hidden_host, void* output_host) {
    if (!p || !args || !hidden_host || !output_host) return NVMOE_ERR_INVALID_ARGUMENT;
    const uint32_t T = args->batch_width;
    NVMOE_TRY(check_tokens(p, T));
    nvmoe_device* d = p->device;
    NVMOE_CUDA(d, cudaSetDevice(d->ordinal));
    const size_t bytes = (size_t)T * p->g.hidden_size * 2u;
    const size_t cap = (size_t)p->g.max_tokens * p->g.hidden_size * 2u;
    if (!p->pinned_in) {
        NVMOE_CUDA(d, cudaMallocHost(&p->pinned_in, cap));
        NVMOE_CUDA(d, cudaMallocHost(&p->pinned_out, cap));
        p->pinned_bytes = cap;
    }
    cudaError_t err = p->hidden_dev.ensure(cap);
    if (err == cudaSuccess) err = p->output_dev.ensure(cap);
    if (err != cudaSuccess) return fail(d, NVMOE_ERR_OUT_OF_MEMORY, "staging allocation failed: %s", cudaGetErrorString(err));
    // page-locked caller memory is read and written by the copy engine directly; anything else goes
    // through the plan's own page-locked staging buffers
    auto page_locked = [](const void* ptr) {
        cudaPointerAttributes attr{};
        if (cudaPointerGetAttributes(&attr, ptr) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        return attr.type == cudaMemoryTypeHost;
    };
    const bool direct_in = page_locked(hidden_host), direct_out = page_locked(output_host);
    if (!direct_in) std::memcpy(p->pinned_in, hidden_host, bytes);
    NVMOE_CUDA(d, cudaMemcpyAsync(p->hidden_dev.ptr, direct_in ? hidden_host : p->pinned_in, bytes, cudaMemcpyHostToDevice,
                                  d->stream));
    nvmoe_buffer hidden{d, p->hidden_dev.ptr, cap};
    nvmoe_buffer output{d, p->output_dev.ptr, cap};
    nvmoe_layer_args local = *args;
    local.hidden = &hidden;
    local.output = &output;
    NVMOE_TRY(nvmoe_layer(p, &local));
    NVMOE_CUDA(d, cudaMemcpyAsync(direct_out ? output_host : p->pinned_out, p->output_dev.ptr, bytes, cudaMemcpyDeviceToHost,
                                  d->stream));
    // The caller waits for this result. A decode step is over in well under a millisecond, so poll for it
    // first (a blocking wait would add the wake-up of a sleeping thread to every step); after two
    // milliseconds yield the core between polls; and give up after kHostWaitSeconds, like nvmoe_sync.
    NVMOE_CUDA(d, cudaEventRecord(d->sync_event, d->stream));
    {
        const auto start = std::chrono::steady_clock::now();
        const auto spin_until = start + std::chrono::milliseconds(2);
        const auto give_up = start + std::chrono::seconds(kHostWaitSeconds);
        for (;;) {
            const cudaError_t q = cudaEventQuery(d->sync_event);
            if (q == cudaSuccess) break;
            if (q != cudaErrorNotReady) return fail(d, NVMOE_ERR_CUDA, "device failed while waiting: %s", cudaGetErrorString(q));
            const auto now = std::chrono::steady_clock::now();
            if (now >= give_up)
                return fail(d, NVMOE_ERR_TIMEOUT, "the layer did not finish within %d s", kHostWaitSeconds);
            if (now >= spin_until) std::this_thread::sleep_for(std::chrono::microseconds(50));
        }
    }
    if (!direct_out) std::memcpy(output_host, p->pinned_out, bytes);
    return NVMOE_OK;
}

uint64_t nvmoe_plan_launch_count(const nvmoe_plan* p) { return p ? p->launches : 0u; }

int nvmoe_probe_mma_rate(nvmoe_device* d, uint32_t n_tile, uint32_t k_groups, nvmoe_mma_probe* out) {
    if (!d || !out) return fail(d, NVMOE_ERR_INVALID_ARGUMENT, "null device or result pointer");
    if (n_tile < 16u || n_tile > 128u || n_tile % 16u || k_groups == 0u || k_groups > (1u << 20))
        return fail(d, NVMOE_ERR_INVALID_ARGUMENT, "probe: token tile %u (16..128 by 16) or %u K groups (1..2^20) out of range",
                    n_tile, k_groups);
    NVMOE_CUDA(d, cudaSetDevice(d->ordinal));
    int sms = 0;
    NVMOE_CUDA(d, cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, d->ordinal));
    int khz = 0;
    NVMOE_CUDA(d, cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, d->ordinal));
    DeviceArray scratch;
    NVMOE_CUDA(d, scratch.ensure((size_t)sms * sizeof(long long) + 64u));
    uint32_t* status = reinterpret_cast<uint32_t*>(scratch.as<long long>() + sms);
    cudaEvent_t ev[2] = {nullptr, nullptr};
    cudaError_t err = cudaMemsetAsync(scratch.ptr, 0, scratch.bytes, d->stream);
    for (int i = 0; i < 2 && err == cudaSuccess; i++) err = cudaEventCreate(&ev[i]);
    float best_ms = 0.0f;
    for (int run = 0; run < 3 && err == cudaSuccess; run++) {  // the first run also loads the kernel
        err = cudaEventRecord(ev[0], d->stream);
        if (err == cudaSuccess) err = launch_mma_rate_probe(n_tile, k_groups, (uint32_t)sms, scratch.as<long long>(), status, d->stream);
        if (err == cudaSuccess) err = cudaEventRecord(ev[1], d->stream);
        if (err == cudaSuccess) err = cudaStreamSynchronize(d->stream);
        float ms = 0.0f;
        if (err == cudaSuccess) err = cudaEventElapsedTime(&ms, ev[0], ev[1]);
        if (run > 0 && (best_ms == 0.0f || ms < best_ms)) best_ms = ms;
    }
    std::vector<long long> cycles((size_t)sms + 8u);
    if (err == cudaSuccess) err = cudaMemcpy(cycles.data(), scratch.ptr, (size_t)sms * sizeof(long long) + 4u, cudaMemcpyDeviceToHost);
    for (cudaEvent_t e : ev)
        if (e) cudaEventDestroy(e);
    const uint32_t raised = err == cudaSuccess ? *reinterpret_cast<uint32_t*>(cycles.data() + sms) : 0u;
    scratch.release();
    if (err != cudaSuccess) return fail(d, NVMOE_ERR_CUDA, "tensor-pipe probe failed: %s", cudaGetErrorString(err));
    if (raised) return fail(d, NVMOE_ERR_DEVICE_STATUS, "tensor-pipe probe: a bounded wait gave up (status %u)", raised);
    long long slowest = 0;
    for (int i = 0; i < sms; i++) slowest = cycles[i] > slowest ? cycles[i] : slowest;
    const double mmas = (double)k_groups * 8.0;  // four K steps into each of two accumulators per group
    out->n_tile = n_tile;
    out->ctas = (uint32_t)sms;
    out->mmas_per_cta = (uint64_t)mmas;
    out->elapsed_ms = best_ms;
    out->cycles_per_mma = (double)slowest / mmas;
    out->tflops = 2.0 * 128.0 * n_tile * 32.0 * mmas * sms / ((double)best_ms * 1e-3) / 1e12;
    out->sm_clock_mhz_nominal = (double)khz / 1e3;
    return NVMOE_OK;
}

int nvmoe_plan_debug_counters(nvmoe_plan* p, uint64_t* out24) {
    uint64_t* out8 = out24;
    if (!p || !out8) return NVMOE_ERR_INVALID_ARGUMENT;
    nvmoe_device* d = p->device;
    NVMOE_CUDA(d, cudaSetDevice(d->ordinal));
    NVMOE_CUDA(d, cudaStreamSynchronize(d->stream));
    NVMOE_CUDA(d, cudaMemcpy(out8, p->tile_list.as<uint32_t>() + 16, 96, cudaMemcpyDeviceToHost));
    NVMOE_CUDA(d, cudaMemcpy(out8 + 12, p->tile_list.as<uint32_t>() + tile_region_words(p) + 16 + 24, 96, cudaMemcpyDeviceToHost));
    return NVMOE_OK;
}

int nvmoe_plan_debug_cta_trace(nvmoe_plan* p, uint64_t* out, uint32_t max_ctas, uint32_t* ctas) {
    if (!p || !ctas) return NVMOE_ERR_INVALID_ARGUMENT;
    nvmoe_device* d = p->device;
    NVMOE_CUDA(d, cudaSetDevice(d->ordinal));
    int sms = 0;
    NVMOE_CUDA(d, cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, d->ordinal));
    *ctas = (uint32_t)sms;
    const size_t bytes = (size_t)sms * 2u * 4u * sizeof(uint64_t);
    NVMOE_CUDA(d, cudaStreamSynchronize(d->stream));
    if (!p->cta_trace.ptr) {  // first request: arm the trace, the next calls fill it
        NVMOE_CUDA(d, p->cta_trace.ensure(bytes));
        NVMOE_CUDA(d, cudaMemset(p->cta_trace.ptr, 0, bytes));
        return NVMOE_OK;
    }
    if (out && max_ctas >= (uint32_t)sms) NVMOE_CUDA(d, cudaMemcpy(out, p->cta_trace.ptr, bytes, cudaMemcpyDeviceToHost));
    return NVMOE_OK;
}

int nvmoe_plan_last_report(nvmoe_plan* p, nvmoe_work_report* report) {
    if (!p || !report) return NVMOE_ERR_INVALID_ARGUMENT;
    nvmoe_device* d = p->device;
    if (!p->events_valid) return fail(d, NVMOE_ERR_INVALID_ARGUMENT, "no layer call has run on this plan");
    NVMOE_CUDA(d, cudaSetDevice(d->ordinal));
    NVMOE_CUDA(d, cudaStreamSynchronize(d->stream));
    NVMOE_CUDA(d, cudaEventElapsedTime(&p->report.total_ms, p->ev[0], p->ev[kStageCount]));
    for (int i = 0; i < kStageCount; i++) {
        p->report.stage_ms[i] = 0.0f;
        if (p->profile_stages) cudaEventElapsedTime(&p->report.stage_ms[i], p->ev[i], p->ev[i + 1]);
    }
    p->report.gate_up_kernel_ms = p->report.down_kernel_ms = 0.0f;
    if (p->profile_stages) {
        cudaEventElapsedTime(&p->report.gate_up_kernel_ms, p->kernel_ev[0][0], p->kernel_ev[0][1]);
        cudaEventElapsedTime(&p->report.down_kernel_ms, p->kernel_ev[1][0], p->kernel_ev[1][1]);
    }
    std::vector<uint32_t> offsets(p->experts + 1u);
    NVMOE_CUDA(d, cudaMemcpy(offsets.data(), p->offsets[0].ptr, offsets.size() * 4u, cudaMemcpyDeviceToHost));
    uint32_t distinct = 0;
    for (uint32_t e = 0; e < p->experts; e++) distinct += offsets[e + 1u] > offsets[e];
    p->report.distinct_experts = distinct;
    const uint64_t per_expert = 3ull * p->g.hidden_size * p->g.intermediate_size * 17ull / 32ull;
    p->report.weight_bytes_touched = per_expert * distinct;
    *report = p->report;
    return NVMOE_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Expert-parallel layer with the collectives issued by the library.
//
// NCCL is bound at run time: the copy already loaded into the process (a framework's) if there is
// one, else the system's libnccl.so.2. Only point-to-point calls inside groups are used, so the two
// exchanges of a step are one NCCL kernel each, on the stream the compute kernels use.
// ---------------------------------------------------------------------------------------------
namespace {

struct NcclApi {
    void* lib = nullptr;
    decltype(&ncclGetUniqueId) get_unique_id = nullptr;
    decltype(&ncclCommInitRank) comm_init_rank = nullptr;
    decltype(&ncclCommDestroy) comm_destroy = nullptr;
    decltype(&ncclGroupStart) group_start = nullptr;
    decltype(&ncclGroupEnd) group_end = nullptr;
    decltype(&ncclSend) send = nullptr;
    decltype(&ncclRecv) recv = nullptr;
    decltype(&ncclGetErrorString) error_string = nullptr;
    decltype(&ncclCommGetAsyncError) comm_get_async_error = nullptr;
    decltype(&ncclCommAbort) comm_abort = nullptr;
    std::string problem;
};

const NcclApi& nccl_api() {
    static const NcclApi api = [] {
        NcclApi a;
        // the copy already in the process (a framework's), else the one NVMOE_NCCL_LIBRARY names, else the system's.
        // A process that will load a framework with its own NCCL later must do that first (or name that
        // copy here): the loader shares one libnccl.so.2 per process, whichever comes first.
        a.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
        if (const char* path = getenv("NVMOE_NCCL_LIBRARY"))
            if (!a.lib && path[0]) a.lib = dlopen(path, RTLD_NOW | RTLD_LOCAL);
        if (!a.lib) a.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
        if (!a.lib) {
            a.problem = std::string("libnccl.so.2 could not be loaded: ") + dlerror();
            return a;
        }
        auto bind = [&](auto& fn, const char* name) {
            fn = reinterpret_cast<std::remove_reference_t<decltype(fn)>>(dlsym(a.lib, name));
            if (!fn && a.problem.empty()) a.problem = std::string("libnccl.so.2 lacks ") + name;
        };
        bind(a.get_unique_id, "ncclGetUniqueId");
        bind(a.comm_init_rank, "ncclCommInitRank");
        bind(a.comm_destroy, "ncclCommDestroy");
        bind(a.group_start, "ncclGroupStart");
        bind(a.group_end, "ncclGroupEnd");
        bind(a.send, "ncclSend");
        bind(a.recv, "ncclRecv");
        bind(a.error_string, "ncclGetErrorString");
        bind(a.comm_get_async_error, "ncclCommGetAsyncError");
        bind(a.comm_abort, "ncclCommAbort");
        return a;
    }();
    return api;
}

}  // namespace

struct nvmoe_ep {
    nvmoe_device* device = nullptr;
    ncclComm_t comm = nullptr;
    bool aborted = false;  // the communicator was aborted after a failure: every later call is refused
    uint32_t rank = 0, world = 1;
    // exchange buffers, sized on first use from the plans' geometry
    DeviceArray logits, routes, send_rows, send_routes, recv_rows, recv_routes, work_out, returned, send_index,
        dest_counts, expert_outputs;
};

namespace {

#define NVMOE_NCCL(d, call)                                                                               \
    do {                                                                                                  \
        ncclResult_t r__ = (call);                                                                        \
        if (r__ != ncclSuccess)                                                                           \
            return fail((d), NVMOE_ERR_COLLECTIVE, "%s failed: %s", #call, nccl_api().error_string(r__)); \
    } while (0)

// every rank sends segment `peer` of `send` to rank `peer` and receives segment `peer` of `recv` from it
// A group that was opened is always closed, whatever a call inside it returned: an open group would swallow
// every later NCCL call of the thread. The first failure is what is reported.
int exchange_segments(nvmoe_ep* ep, const void* send_a, void* recv_a, size_t bytes_a, const void* send_b, void* recv_b,
                      size_t bytes_b) {
    const NcclApi& n = nccl_api();
    nvmoe_device* d = ep->device;
    NVMOE_NCCL(d, n.group_start());
    ncclResult_t first = ncclSuccess;
    const char* what = "";
    auto note = [&](ncclResult_t r, const char* call) {
        if (r != ncclSuccess && first == ncclSuccess) {
            first = r;
            what = call;
        }
    };
    for (uint32_t peer = 0; peer < ep->world && first == ncclSuccess; peer++) {
        note(n.send((const char*)send_a + peer * bytes_a, bytes_a, ncclInt8, (int)peer, ep->comm, d->stream), "ncclSend");
        note(n.recv((char*)recv_a + peer * bytes_a, bytes_a, ncclInt8, (int)peer, ep->comm, d->stream), "ncclRecv");
        if (send_b) {
            note(n.send((const char*)send_b + peer * bytes_b, bytes_b, ncclInt8, (int)peer, ep->comm, d->stream), "ncclSend");
            note(n.recv((char*)recv_b + peer * bytes_b, bytes_b, ncclInt8, (int)peer, ep->comm, d->stream), "ncclRecv");
        }
    }
    note(n.group_end(), "ncclGroupEnd");
    if (first != ncclSuccess) return fail(d, NVMOE_ERR_COLLECTIVE, "%s failed: %s", what, n.error_string(first));
    return NVMOE_OK;
}

}  // namespace

extern "C" {

int nvmoe_ep_unique_id(void* id128) {
    if (!id128) return NVMOE_ERR_INVALID_ARGUMENT;
    const NcclApi& n = nccl_api();
    if (!n.problem.empty()) return fail(nullptr, NVMOE_ERR_COLLECTIVE, "%s", n.problem.c_str());
    static_assert(sizeof(ncclUniqueId) == 128, "the id travels as 128 bytes");
    ncclUniqueId id;
    ncclResult_t r = n.get_unique_id(&id);
    if (r != ncclSuccess) return fail(nullptr, NVMOE_ERR_COLLECTIVE, "ncclGetUniqueId failed: %s", n.error_string(r));
    std::memcpy(id128, &id, 128);
    return NVMOE_OK;
}

int nvmoe_ep_create(nvmoe_device* d, const void* id128, uint32_t rank, uint32_t world, nvmoe_ep** out) {
    if (!d || !id128 || !out) return fail(d, NVMOE_ERR_INVALID_ARGUMENT, "null argument");
    *out = nullptr;
    if (world == 0u || world > 1024u || rank >= world)
        return fail(d, NVMOE_ERR_INVALID_ARGUMENT, "rank %u of %u is not a valid expert-parallel position", rank, world);
    const NcclApi& n = nccl_api();
    if (!n.problem.empty()) return fail(d, NVMOE_ERR_COLLECTIVE, "%s", n.problem.c_str());
    NVMOE_CUDA(d, cudaSetDevice(d->ordinal));
    nvmoe_ep* ep = new (std::nothrow) nvmoe_ep();
    if (!ep) return fail(d, NVMOE_ERR_OUT_OF_MEMORY, "out of host memory");
    ep->device = d;
    ep->rank = rank;
    ep->world = world;
    ncclUniqueId id;
    std::memcpy(&id, id128, 128);
    ncclResult_t r = n.comm_init_rank(&ep->comm, (int)world, id, (int)rank);
    if (r != ncclSuccess) {
        delete ep;
        return fail(d, NVMOE_ERR_COLLECTIVE, "ncclCommInitRank failed: %s", n.error_string(r));
    }
    *out = ep;
    return NVMOE_OK;
}

void nvmoe_ep_destroy(nvmoe_ep* ep) {
    if (!ep) return;
    cudaSetDevice(ep->device->ordinal);
    cudaStreamSynchronize(ep->device->stream);
    if (ep->comm && !ep->aborted) nccl_api().comm_destroy(ep->comm);
    DeviceArray* all[] = {&ep->logits, &ep->routes, &ep->send_rows, &ep->send_routes, &ep->recv_rows, &ep->recv_routes,
                          &ep->work_out, &ep->returned, &ep->send_index, &ep->dest_counts, &ep->expert_outputs};
    for (DeviceArray* a : all) a->release();
    delete ep;
}

int nvmoe_ep_layer(nvmoe_ep* ep, nvmoe_plan* home, nvmoe_plan* work, const nvmoe_ep_layer_args* a) {
    if (!ep || !home || !work || !a) return NVMOE_ERR_INVALID_ARGUMENT;
    nvmoe_device* d = ep->device;
    if (home->device != d || work->device != d)
        return fail(d, NVMOE_ERR_INVALID_ARGUMENT, "the plans belong to another device than the communicator");
    const uint32_t T = a->batch_width, K = home->K, G = ep->world;
    NVMOE_TRY(check_tokens(home, T));
    const size_t H = home->g.hidden_size;
    // slots per peer, the same on every rank: the worst case unless the caller bounds it
    const size_t worst = (size_t)home->g.max_tokens * K;
    const size_t S = (a->capacity_rows != 0u && a->capacity_rows < worst) ? a->capacity_rows : worst;
    if (work->K != 1u || work->g.hidden_size != home->g.hidden_size || work->g.intermediate_size != home->g.intermediate_size ||
        work->experts != home->experts || (size_t)work->g.max_tokens < S * G)
        return fail(d, NVMOE_ERR_INVALID_ARGUMENT,
                    "the owner-side plan must be top-1 over the same experts and sizes with room for %zu rows", S * G);
    if (!a->owner_table || !a->hidden || !a->output || !a->router_weights)
        return fail(d, NVMOE_ERR_INVALID_ARGUMENT, "hidden, router weights, owner table and output are required");
    NVMOE_CUDA(d, cudaSetDevice(d->ordinal));
    cudaError_t err = cudaSuccess;
    auto want = [&](DeviceArray& arr, size_t bytes) {
        if (err == cudaSuccess) err = arr.ensure(bytes);
    };
    const size_t Tm = home->g.max_tokens;
    want(ep->logits, Tm * ((home->g.routed_experts + 1u) / 2u) * 4u);
    want(ep->routes, Tm * K * 4u);
    want(ep->send_rows, G * S * H * 2u);
    want(ep->send_routes, G * S * 4u);
    want(ep->recv_rows, G * S * H * 2u);
    want(ep->recv_routes, G * S * 4u);
    want(ep->work_out, G * S * H * 2u);
    want(ep->returned, (G * S > worst ? G * S : worst) * H * 2u);
    want(ep->send_index, worst * 4u);
    want(ep->dest_counts, (size_t)G * 4u);
    want(ep->expert_outputs, worst * H * 2u);
    if (err != cudaSuccess)
        return fail(d, err == cudaErrorMemoryAllocation ? NVMOE_ERR_OUT_OF_MEMORY : NVMOE_ERR_CUDA,
                    "exchange buffer allocation failed: %s", cudaGetErrorString(err));
    auto view = [&](DeviceArray& arr) { return nvmoe_buffer{d, arr.ptr, arr.bytes}; };
    nvmoe_buffer logits = view(ep->logits), routes = view(ep->routes), send_rows = view(ep->send_rows),
                 send_routes = view(ep->send_routes), recv_rows = view(ep->recv_rows), recv_routes = view(ep->recv_routes),
                 work_out = view(ep->work_out), returned = view(ep->returned), send_index = view(ep->send_index),
                 dest_counts = view(ep->dest_counts), expert_outputs = view(ep->expert_outputs);

    if (ep->aborted) return fail(d, NVMOE_ERR_COLLECTIVE, "the communicator was aborted after an earlier failure");
    // Everything that can allocate, synchronise or fail on this rank alone happens before the first exchange:
    // the owner-side scratch and the resolution of both table pairs. Between the two exchanges nothing returns
    // early, because a rank that posted the first exchange and not the second leaves its peers waiting for rows
    // that never come.
    NVMOE_TRY(ensure_layer_scratch(work));
    {
        const bool tensor = use_tensor_path(work);
        ExpertSet* unused = nullptr;
        NVMOE_TRY(check_expert_tables(work, a->gate_up_addresses, a->gate_up_slots, 4u));
        NVMOE_TRY(check_expert_tables(work, a->down_addresses, a->down_slots, 2u));
        NVMOE_TRY(prepare_expert_set(work, true, a->gate_up_addresses, a->gate_up_slots, tensor, &unused));
        NVMOE_TRY(prepare_expert_set(work, false, a->down_addresses, a->down_slots, tensor, &unused));
    }
    // this rank's tokens: route, then place every route's row in the segment of the rank owning its expert
    NVMOE_TRY(nvmoe_router_linear(home, T, a->hidden, &logits, a->router_weights, a->router_bias));
    NVMOE_TRY(nvmoe_route(home, T, &logits, &routes, a->bias, a->telemetry));
    NVMOE_TRY(nvmoe_ep_pack(home, T, a->hidden, &routes, a->owner_table, G, ep->rank, &send_rows, &send_routes, &send_index,
                            &dest_counts, (uint32_t)S));
    int first_error = exchange_segments(ep, send_rows.ptr, recv_rows.ptr, S * H * 2u, send_routes.ptr, recv_routes.ptr, S * 4u);
    std::string first_text = first_error != NVMOE_OK ? d->error : std::string();
    auto keep_first = [&](int rc) {
        if (rc != NVMOE_OK && first_error == NVMOE_OK) {
            first_error = rc;
            first_text = d->error;
        }
    };
    // the rows this rank owns the experts of: every resource in range, the slot tables keep the owned ones
    nvmoe_layer_args owner{};
    owner.batch_width = (uint32_t)(S * G);
    owner.expert_start = 0u;
    owner.expert_count = work->experts;
    owner.hidden = &recv_rows;
    owner.routes_in = &recv_routes;
    owner.expert_outputs = &work_out;
    owner.gate_up_addresses = a->gate_up_addresses;
    owner.gate_up_slots = a->gate_up_slots;
    owner.down_addresses = a->down_addresses;
    owner.down_slots = a->down_slots;
    if (first_error == NVMOE_OK) keep_first(nvmoe_layer(work, &owner));
    // the return exchange is posted whatever happened above (the peers are already waiting for it)
    keep_first(exchange_segments(ep, work_out.ptr, returned.ptr, S * H * 2u, nullptr, nullptr, 0u));
    if (first_error != NVMOE_OK) {
        d->error = first_text;
        return first_error;
    }
    // the combine reads the returned rows through the positions the pack step recorded; shapes it cannot take
    // that way go through the explicit unpack
    NVMOE_TRY(check_buffer(home, a->output, (size_t)T * H * 2u, "output"));
    if (launch_reduce_gather((const uint16_t*)returned.ptr, (const uint32_t*)send_index.ptr, (uint16_t*)a->output->ptr, T, K,
                             (uint32_t)H, home->g.reduce_scale, d->stream)) {
        home->launches++;
        return post_launch(home, "combine of returned rows");
    }
    NVMOE_TRY(nvmoe_ep_unpack(home, T, &returned, &send_index, &expert_outputs));
    return nvmoe_reduce(home, T, &expert_outputs, a->output);
}

// Bounded wait for everything queued on the communicator's stream. While it waits it asks NCCL for
// asynchronous errors; on such an error, or when the time runs out (a peer that never posted its half of an
// exchange), the communicator is aborted so that the kernels spinning on the peer give up and the stream
// drains: the host thread and the device both come back. The communicator is unusable afterwards.
int nvmoe_ep_sync(nvmoe_ep* ep, uint64_t timeout_ns) {
    if (!ep) return NVMOE_ERR_INVALID_ARGUMENT;
    nvmoe_device* d = ep->device;
    const NcclApi& n = nccl_api();
    NVMOE_CUDA(d, cudaSetDevice(d->ordinal));
    NVMOE_CUDA(d, cudaEventRecord(d->sync_event, d->stream));
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::nanoseconds(timeout_ns);
    for (;;) {
        const cudaError_t q = cudaEventQuery(d->sync_event);
        if (q == cudaSuccess) return NVMOE_OK;
        if (q != cudaErrorNotReady) return fail(d, NVMOE_ERR_CUDA, "device failed while waiting: %s", cudaGetErrorString(q));
        ncclResult_t async = ncclSuccess;
        const bool asked = !ep->aborted && n.comm_get_async_error && n.comm_get_async_error(ep->comm, &async) == ncclSuccess;
        const bool failed = asked && async != ncclSuccess && async != ncclInProgress;
        const bool late = std::chrono::steady_clock::now() >= deadline;
        if (failed || late) {
            if (!ep->aborted && n.comm_abort) {
                n.comm_abort(ep->comm);
                ep->comm = nullptr;
            }
            ep->aborted = true;
            if (failed)
                return fail(d, NVMOE_ERR_COLLECTIVE, "the communicator reported %s; it was aborted", n.error_string(async));
            return fail(d, NVMOE_ERR_TIMEOUT, "the exchange did not finish within %llu ns; the communicator was aborted",
                        (unsigned long long)timeout_ns);
        }
        std::this_thread::yield();
    }
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Route scheduler that allocates nothing.
//
// Some callers cannot let a call reach the device allocator: a serving loop that has handed all free
// device memory to a key/value cache, a library whose caller holds the allocator's lock, or code that runs
// where an allocation would synchronise the device. For them the scratch of the multi-block counting
// sort (per-block histograms and bucket bases) lives in a fixed array in the module's own device
// memory, which the loader places when the library is loaded on a device; its address comes from the
// runtime's symbol table once per device and is then handed to the kernels as an ordinary pointer.
// ---------------------------------------------------------------------------------------------
namespace {

constexpr uint32_t kStaticHistWords = 65536u;  // per-block histograms: blocks * (experts + 1) words
constexpr uint32_t kStaticBaseWords = 1024u;   // bucket bases: experts + 2 words
static __device__ __align__(256) uint32_t g_static_sort_scratch[kStaticHistWords + kStaticBaseWords];

constexpr int kStaticScratchDevices = 64;
std::mutex g_static_scratch_mutex;
uint32_t* g_static_scratch_address[kStaticScratchDevices] = {nullptr};

// Device address of the array on the plan's device (which must be current). Looked up on the first
// call for a device and remembered.
int static_scratch_for(nvmoe_plan* p, uint32_t** out) {
    nvmoe_device* d = p->device;
    if (d->ordinal < 0 || d->ordinal >= kStaticScratchDevices)
        return fail(d, NVMOE_ERR_INVALID_ARGUMENT, "device ordinal beyond the static scratch table");
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (!g_static_scratch_address[d->ordinal]) {
        void* address = nullptr;
        const cudaError_t err = cudaGetSymbolAddress(&address, g_static_sort_scratch);
        if (err != cudaSuccess || address == nullptr)
            return fail(d, NVMOE_ERR_CUDA, "static sort scratch: address lookup failed: %s", cudaGetErrorString(err));
        g_static_scratch_address[d->ordinal] = static_cast<uint32_t*>(address);
    }
    *out = g_static_scratch_address[d->ordinal];
    return NVMOE_OK;
}

}  // namespace

extern "C" int nvmoe_route_compact_static(nvmoe_plan* p, uint32_t T, const nvmoe_buffer* routes,
                                          nvmoe_buffer* intermediates, const nvmoe_buffer* gate_up_slots,
                                          nvmoe_buffer* control) {
    if (!p) return NVMOE_ERR_INVALID_ARGUMENT;
    NVMOE_TRY(check_tokens(p, T));
    NVMOE_TRY(check_buffer(p, routes, (size_t)T * p->K * 4u, "routes"));
    NVMOE_TRY(check_buffer(p, intermediates, (size_t)T * p->frame_words * 4u, "intermediates"));
    NVMOE_TRY(check_buffer(p, control, 28u, "control"));
    NVMOE_TRY(check_slots(p, gate_up_slots));
    const uint64_t count = (uint64_t)T * p->K;
    const uint64_t blocks = (count + kSortChunk - 1u) / kSortChunk;
    const uint64_t buckets = (uint64_t)p->experts + 1u;
    if (blocks * buckets > kStaticHistWords || buckets + 1u > kStaticBaseWords)
        return fail(p->device, NVMOE_ERR_INVALID_ARGUMENT,
                    "route compact (static scratch): %llu routes in %llu blocks x %llu buckets exceed the fixed scratch of "
                    "%u histogram words / %u bucket words",
                    (unsigned long long)count, (unsigned long long)blocks, (unsigned long long)buckets, kStaticHistWords,
                    kStaticBaseWords);
    NVMOE_CUDA(p->device, cudaSetDevice(p->device->ordinal));
    uint32_t* scratch = nullptr;
    NVMOE_TRY(static_scratch_for(p, &scratch));
    const nvmoe_geometry& g = p->g;
    const uint32_t tiles = (g.intermediate_size + g.gate_tile_rows - 1u) / g.gate_tile_rows;
    const SortScratch fixed{scratch, scratch + kStaticHistWords, (uint32_t)(kStaticHistWords / buckets), (uint32_t)buckets};
    launch_route_compact((const uint32_t*)routes->ptr, (uint32_t*)intermediates->ptr,
                         gate_up_slots ? (const uint32_t*)gate_up_slots->ptr : nullptr,
                         gate_up_slots ? (uint32_t)(gate_up_slots->bytes / 4u) : 0u, 4u, (uint32_t*)control->ptr, T, p->K,
                         g.intermediate_size, tiles, p->experts, fixed, p->device->stream);
    p->launches += count <= 4096u ? 1u : 3u;
    return post_launch(p, "route compact (static scratch)");
}
