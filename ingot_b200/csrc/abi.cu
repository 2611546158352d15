// C ABI of libingot_cuda.so: the handle, buffers, argument validation, and
// the mapping from CUDA / device-status errors to ingot_status codes.
#include "../../include/ingot_cuda.h"

#include <math.h>
#include <stdio.h>
#include <string.h>

#include <map>
#include <new>
#include <string>
#include <unordered_map>
#include <vector>

#include "gemv_core.cuh"
#include "kernels.h"

using namespace ingot;

struct ingot_gpu {
    int device = 0;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;
    int *status = nullptr;            // device status word
    int *status_host = nullptr;       // pinned mirror
    void *workspace = nullptr;        // scratch for packed activations
    size_t workspace_bytes = 0;
    std::vector<void *> retired;      // outgrown scratch blocks: recorded commands may still hold their addresses
    void *tc_scratch = nullptr;       // tile counters and partial rows of the tcgen05 GEMV
    bool use_tc = false;
    uint32_t ep_world = 1;
    uint32_t sm_count = 0;
    bool failed = false;              // sticky device failure
    bool pdl = true;
    bool force_plain = false;
    bool no_mma = false;
    bool group_scope = true;
    bool wide_rows = false;           // fused-norm rows with four digits even when rounding to bfloat16
    bool capturing = false;
    // independent-projection scope: launches rotate over the main stream and side streams
    static constexpr int SIDE_STREAMS = 3;
    cudaStream_t side[SIDE_STREAMS] = {};
    cudaEvent_t fork_event = nullptr, join_event[SIDE_STREAMS] = {};
    bool in_scope = false;
    int scope_next = 0;               // stream of the next launch inside the scope: 0 = main, i > 0 = side[i - 1]
    int scope_used = 0;               // side streams touched in this scope (bit mask)
    std::vector<GemvCall> pending;    // one-token tensor-core projections of the open scope: they share one launch at its end
    // the size-keyed pool of output buffers (the reference's Workspace: src/metal.rs:1278-1337)
    size_t pool_limit = 0, pool_managed = 0, pool_peak = 0;
    uint64_t pool_allocations = 0, pool_reuses = 0;
    std::map<size_t, std::vector<void *>> pool_free;      // idle buffers by length
    struct PoolEntry { size_t length; bool leased; };
    std::unordered_map<void *, PoolEntry> pool_lengths;   // every buffer the pool manages, idle or leased
    // links of the next fused-norm projection to a tensor-parallel group (ingot_tp_signal_next / ingot_tp_wait_next)
    ingot_group *tp_signal_group = nullptr, *tp_wait_group = nullptr;
    uint32_t tp_signal_slot = 0, tp_wait_slot[2] = {0, 0};
    bool chain_recording = false;     // fused-norm projections are being collected for one persistent kernel
    std::vector<GemvCall> chain_calls;
    std::string error;
};

// A tensor-parallel group as one rank sees it: its window (the activations other ranks write into, then a
// control area: the step counter and one arrival counter per exchange slot) and the other ranks' windows.
struct ingot_group {
    ingot_gpu *gpu = nullptr;
    uint32_t rank = 0, world = 1, slots = 0;
    // the allocation: the window of plain vectors | the tagged twins (8 bytes per float of the window) | the step counter
    size_t window_bytes = 0, twin_off = 0, ctrl_off = 0, total_bytes = 0;
    uint8_t *peer[TP_MAX_RANKS] = {};                 // base of every rank's window; peer[rank] is the own one
    bool opened[TP_MAX_RANKS] = {};                   // mapped through an IPC handle (closed again on destroy)
    struct Shard { size_t off = 0; uint32_t rows = 0; };
    std::vector<Shard> shard;                         // per slot: where this rank's rows of the slot's vector lie (known once its projection was issued)
    uint32_t *step_counter() const { return reinterpret_cast<uint32_t *>(peer[rank] + ctrl_off); }
    uint64_t *twin(uint32_t r, size_t off) const { return reinterpret_cast<uint64_t *>(peer[r] + twin_off + 2u * off); }
};
static constexpr uint32_t TP_NO_SLOT = 0xffffffffu;

struct ingot_chain {
    ChainLaunch launch;
    int device = 0;
};

struct ingot_graph {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
};

namespace {

ingot_status fail(ingot_gpu *g, ingot_status code, const std::string &msg) {
    if (g) g->error = msg;
    return code;
}

ingot_status cuda_fail(ingot_gpu *g, cudaError_t e, const char *what) {
    if (g) {
        g->failed = true;
        g->error = std::string(what) + ": " + cudaGetErrorString(e) + " (device failure; requires reload)";
    }
    return INGOT_DEVICE;
}

// Common entry check: handle present, not failed, right device current.
ingot_status enter(ingot_gpu *g) {
    if (!g) return INGOT_INVALID;
    if (g->failed) return fail(g, INGOT_DEVICE, "device failed earlier; requires reload");
    cudaError_t e = cudaSetDevice(g->device);
    if (e != cudaSuccess) return cuda_fail(g, e, "cudaSetDevice");
    return INGOT_OK;
}

constexpr size_t TC_SCRATCH_BYTES = 8u << 20;

// The stream of the next launch: inside an independent-projection scope launches take the
// main stream and the side streams in turn.
cudaStream_t next_stream(ingot_gpu *g) {
    if (!g->in_scope) return g->stream;
    const int i = g->scope_next;
    g->scope_next = (i + 1) % (ingot_gpu::SIDE_STREAMS + 1);
    if (i == 0) return g->stream;
    if (!(g->scope_used & (1 << (i - 1)))) {            // first use in this scope: order it after the fork point
        if (cudaStreamWaitEvent(g->side[i - 1], g->fork_event, 0) != cudaSuccess) return g->stream;
        g->scope_used |= 1 << (i - 1);
    }
    return g->side[i - 1];
}

LaunchCtx ctx_on(ingot_gpu *g, cudaStream_t stream);
LaunchCtx ctx_of(ingot_gpu *g) { return ctx_on(g, next_stream(g)); }

LaunchCtx ctx_on(ingot_gpu *g, cudaStream_t stream) {
    LaunchCtx c;
    c.stream = stream;
    c.status = g->status;
    c.sm_count = g->sm_count;
    c.pdl = g->pdl;
    c.force_plain = g->force_plain;
    c.no_mma = g->no_mma;
    c.workspace = g->workspace;
    c.workspace_bytes = g->workspace_bytes;
    c.use_tc = g->use_tc;
    c.ep_world = g->ep_world;
    c.tc_scratch = g->tc_scratch;
    c.tc_scratch_bytes = TC_SCRATCH_BYTES;
    if (g->in_scope) {            // concurrent launches must not share the handle's scratch areas
        c.workspace = nullptr;
        c.workspace_bytes = 0;
        c.tc_scratch = nullptr;
        c.tc_scratch_bytes = 0;
    }
    return c;
}

ingot_status after_launch(ingot_gpu *g, cudaError_t e, const char *what) {
    if (e == cudaErrorInvalidValue) return fail(g, INGOT_INVALID, std::string(what) + ": invalid launch arguments");
    if (e != cudaSuccess) return cuda_fail(g, e, what);
    return INGOT_OK;
}

bool x_kind_ok(uint32_t k) {
    return k == INGOT_KIND_F32 || k == INGOT_KIND_BF16 || k == INGOT_X_PACKED || k == INGOT_X_DIGITS || k == INGOT_X_PACKED_HI;
}

constexpr size_t WORKSPACE_BYTES = 16u << 20;

// validate_matrix (src/metal.rs:1602-1621) on the integer parameters.
ingot_status check_matrix(ingot_gpu *g, uint32_t kind, uint64_t cols, uint64_t rows, uint64_t stride) {
    uint32_t block, bytes;
    if (!geometry(kind, block, bytes)) return fail(g, INGOT_UNSUPPORTED, "GGML type " + std::to_string(kind) + " is unsupported");
    if (cols == 0 || rows == 0 || cols % block || stride != cols / block * bytes || cols > 0xffffffffull ||
        rows > 0xffffffffull || stride > 0xffffffffull)
        return fail(g, INGOT_INVALID, "invalid quantized matrix layout");
    return INGOT_OK;
}

}  // namespace

extern "C" {

ingot_status ingot_geometry(uint32_t kind, uint32_t *block, uint32_t *bytes) {
    uint32_t b, s;
    if (!block || !bytes) return INGOT_INVALID;
    if (!geometry(kind, b, s)) return INGOT_UNSUPPORTED;
    *block = b;
    *bytes = s;
    return INGOT_OK;
}

ingot_status ingot_tensor_layout(uint32_t kind, uint64_t cols, uint64_t rows, uint64_t count, uint64_t *stride,
                                 uint64_t *bytes) {
    uint32_t b, s;
    if (!stride || !bytes) return INGOT_INVALID;
    if (!geometry(kind, b, s)) return INGOT_UNSUPPORTED;
    if (cols == 0 || rows == 0 || count == 0 || cols % b) return INGOT_INVALID;
    unsigned __int128 st = (unsigned __int128)(cols / b) * s;
    unsigned __int128 total = st * rows;
    if (st > 0xffffffffffffffffull || total > 0xffffffffffffffffull) return INGOT_INVALID;
    total *= count;
    if (total > 0xffffffffffffffffull) return INGOT_INVALID;
    *stride = (uint64_t)st;
    *bytes = (uint64_t)total;
    return INGOT_OK;
}

ingot_status ingot_gpu_create(int32_t device, ingot_gpu **out) {
    if (!out) return INGOT_INVALID;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || device < 0 || device >= n) return INGOT_DEVICE;
    if (cudaSetDevice(device) != cudaSuccess) return INGOT_DEVICE;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return INGOT_DEVICE;
    if (prop.major != 10) return INGOT_DEVICE;       // the kernels are built for sm_100a only
    ingot_gpu *g = new (std::nothrow) ingot_gpu();
    if (!g) return INGOT_DEVICE;
    g->device = device;
    g->sm_count = (uint32_t)prop.multiProcessorCount;
    if (cudaStreamCreateWithFlags(&g->own_stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaMalloc(&g->status, 64) != cudaSuccess || cudaMemset(g->status, 0, 64) != cudaSuccess ||
        cudaHostAlloc(&g->status_host, 64, cudaHostAllocDefault) != cudaSuccess ||
        cudaMalloc(&g->workspace, WORKSPACE_BYTES) != cudaSuccess ||
        cudaMalloc(&g->tc_scratch, TC_SCRATCH_BYTES) != cudaSuccess || cudaMemset(g->tc_scratch, 0, TC_COUNTER_BYTES) != cudaSuccess) {
        ingot_gpu_destroy(g);
        return INGOT_DEVICE;
    }
    g->workspace_bytes = WORKSPACE_BYTES;
    g->stream = g->own_stream;
    *out = g;
    return INGOT_OK;
}

void ingot_gpu_destroy(ingot_gpu *g) {
    if (!g) return;
    cudaSetDevice(g->device);
    if (g->own_stream) { cudaStreamSynchronize(g->own_stream); cudaStreamDestroy(g->own_stream); }
    for (int i = 0; i < ingot_gpu::SIDE_STREAMS; ++i) {
        if (g->side[i]) cudaStreamDestroy(g->side[i]);
        if (g->join_event[i]) cudaEventDestroy(g->join_event[i]);
    }
    if (g->fork_event) cudaEventDestroy(g->fork_event);
    if (g->status) cudaFree(g->status);
    if (g->workspace) cudaFree(g->workspace);
    for (void *p : g->retired) cudaFree(p);
    for (auto &kv : g->pool_free)
        for (void *p : kv.second) cudaFree(p);            // (leased output buffers belong to their holders)
    if (g->tc_scratch) cudaFree(g->tc_scratch);
    if (g->status_host) cudaFreeHost(g->status_host);
    delete g;
}

const char *ingot_last_error(const ingot_gpu *g) { return g ? g->error.c_str() : "null handle"; }

ingot_status ingot_gpu_set_stream(ingot_gpu *g, void *cuda_stream) {
    if (!g) return INGOT_INVALID;
    if (g->capturing) return fail(g, INGOT_INVALID, "cannot change stream while recording");
    g->stream = cuda_stream ? static_cast<cudaStream_t>(cuda_stream) : g->own_stream;
    return INGOT_OK;
}

ingot_status ingot_gpu_set_option(ingot_gpu *g, int32_t option, int32_t value) {
    if (!g) return INGOT_INVALID;
    switch (option) {
    case INGOT_OPT_PDL: g->pdl = value != 0; return INGOT_OK;
    case INGOT_OPT_FORCE_PLAIN: g->force_plain = value != 0; return INGOT_OK;
    case INGOT_OPT_NO_MMA: g->no_mma = value != 0; return INGOT_OK;
    case INGOT_OPT_TCGEN05_GEMV: g->use_tc = value != 0; return INGOT_OK;
    case INGOT_OPT_EP_WORLD: g->ep_world = value > 1 ? (uint32_t)value : 1u; return INGOT_OK;
    case INGOT_OPT_GROUP_SCOPE: g->group_scope = value != 0; return INGOT_OK;
    case INGOT_OPT_WIDE_ROWS: g->wide_rows = value != 0; return INGOT_OK;
    default: return fail(g, INGOT_INVALID, "unknown option");
    }
}

ingot_status ingot_synchronize(ingot_gpu *g) {
    ingot_status st = enter(g);
    if (st) return st;
    if (g->capturing) return fail(g, INGOT_INVALID, "cannot synchronize while recording");
    if (g->in_scope) return fail(g, INGOT_INVALID, "cannot synchronize inside an independent scope");
    cudaError_t e = cudaMemcpyAsync(g->status_host, g->status, sizeof(int), cudaMemcpyDeviceToHost, g->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(g->stream);
    if (e != cudaSuccess) return cuda_fail(g, e, "synchronize");
    const int code = *g->status_host;
    if (code == KERNEL_OK) return INGOT_OK;
    e = cudaMemsetAsync(g->status, 0, sizeof(int), g->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(g->stream);
    if (e != cudaSuccess) return cuda_fail(g, e, "status reset");
    switch (code) {
    case KERNEL_ERR_EXPERT_RANGE: return fail(g, INGOT_INVALID, "expert id out of range");
    case KERNEL_ERR_ROUTER_INPUT: return fail(g, INGOT_INVALID, "invalid router scores or expert count");
    case KERNEL_ERR_PRODUCER_TIMEOUT: return fail(g, INGOT_TIMEOUT, "GEMV producer wait ran out");
    case KERNEL_ERR_CONSUMER_TIMEOUT: return fail(g, INGOT_TIMEOUT, "GEMV consumer wait ran out");
    case KERNEL_ERR_GEMM_TIMEOUT: return fail(g, INGOT_TIMEOUT, "GEMM pipeline wait ran out");
    case KERNEL_ERR_CHAIN_TIMEOUT: return fail(g, INGOT_TIMEOUT, "chain kernel: a projection never saw the one it depends on finish");
    case KERNEL_ERR_PEER_TIMEOUT: return fail(g, INGOT_TIMEOUT, "row-sharded projection: a rank's shard of the input never arrived");
    default: return fail(g, INGOT_DEVICE, "unknown device status " + std::to_string(code));
    }
}

// ---- buffers ----------------------------------------------------------------

ingot_status ingot_buffer_alloc(ingot_gpu *g, size_t bytes, void **p) {
    ingot_status st = enter(g);
    if (st) return st;
    if (!p) return fail(g, INGOT_INVALID, "null output pointer");
    *p = nullptr;
    cudaError_t e = cudaMalloc(p, bytes ? bytes : 16);
    if (e == cudaErrorMemoryAllocation) { cudaGetLastError(); return fail(g, INGOT_INVALID, "out of device memory"); }
    if (e != cudaSuccess) return cuda_fail(g, e, "cudaMalloc");
    return INGOT_OK;
}

ingot_status ingot_buffer_free(ingot_gpu *g, void *p) {
    if (!g) return INGOT_INVALID;
    if (!p) return INGOT_OK;
    cudaSetDevice(g->device);
    cudaError_t e = cudaFree(p);
    if (e != cudaSuccess && !g->failed) return cuda_fail(g, e, "cudaFree");
    return INGOT_OK;
}

// ---- output buffers from a size-keyed pool (Gpu::output / configure_workspace: src/metal.rs:1278-1337) ----

static size_t allocation_charge(size_t length) { return (length + 16383u) / 16384u * 16384u; }      // charged by 16 KiB pages

ingot_status ingot_gpu_configure_workspace(ingot_gpu *g, size_t limit_bytes) {
    if (!g) return INGOT_INVALID;
    g->pool_limit = limit_bytes;
    return INGOT_OK;
}

ingot_status ingot_output_alloc(ingot_gpu *g, size_t count_f32, float **out) {
    ingot_status st = enter(g);
    if (st) return st;
    if (!out) return fail(g, INGOT_INVALID, "null output pointer");
    *out = nullptr;
    if (count_f32 == 0 || count_f32 > (size_t)-1 / 4u) return fail(g, INGOT_INVALID, "output size overflow");
    const size_t bytes = count_f32 * 4u;
    if (g->pool_limit == 0) return ingot_buffer_alloc(g, bytes, reinterpret_cast<void **>(out));      // no budget: a plain allocation
    auto idle = g->pool_free.find(bytes);
    if (idle != g->pool_free.end() && !idle->second.empty()) {
        *out = static_cast<float *>(idle->second.back());
        idle->second.pop_back();
        g->pool_lengths[*out].leased = true;
        g->pool_reuses += 1;
        return INGOT_OK;
    }
    const size_t charge = allocation_charge(bytes);
    // give up only as much idle capacity as this allocation needs, largest buffers first
    while (g->pool_managed + charge > g->pool_limit) {
        auto largest = g->pool_free.end();
        for (auto it = g->pool_free.begin(); it != g->pool_free.end(); ++it)
            if (!it->second.empty()) largest = it;                     // (ordered by length: the last non-empty one)
        if (largest == g->pool_free.end()) break;
        void *victim = largest->second.back();
        largest->second.pop_back();
        g->pool_managed -= allocation_charge(largest->first);
        g->pool_lengths.erase(victim);
        cudaFree(victim);                                              // (waits for the device: nothing enqueued still uses it)
    }
    if (g->pool_managed + charge > g->pool_limit)
        return fail(g, INGOT_INVALID, "workspace live allocation exceeds budget: " + std::to_string(g->pool_managed) + " + " +
                                          std::to_string(charge) + " > " + std::to_string(g->pool_limit));
    void *p = nullptr;
    if ((st = ingot_buffer_alloc(g, bytes, &p))) return st;
    g->pool_managed += charge;
    if (g->pool_managed > g->pool_peak) g->pool_peak = g->pool_managed;
    g->pool_allocations += 1;
    g->pool_lengths[p] = {bytes, true};
    *out = static_cast<float *>(p);
    return INGOT_OK;
}

ingot_status ingot_output_release(ingot_gpu *g, float *p) {
    if (!g) return INGOT_INVALID;
    if (!p) return INGOT_OK;
    auto it = g->pool_lengths.find(p);
    if (it == g->pool_lengths.end()) return ingot_buffer_free(g, p);   // allocated while no budget was set
    if (!it->second.leased) return fail(g, INGOT_INVALID, "output_release: this buffer is already back in the pool");
    // back on the idle list of its length; work already enqueued on the handle's stream runs before any later user's
    it->second.leased = false;
    g->pool_free[it->second.length].push_back(p);
    return INGOT_OK;
}

ingot_status ingot_workspace_statistics(const ingot_gpu *g, uint64_t *allocations, uint64_t *reuses, size_t *managed, size_t *peak) {
    if (!g) return INGOT_INVALID;
    if (allocations) *allocations = g->pool_allocations;
    if (reuses) *reuses = g->pool_reuses;
    if (managed) *managed = g->pool_managed;
    if (peak) *peak = g->pool_peak;
    return INGOT_OK;
}

ingot_status ingot_buffer_upload(ingot_gpu *g, void *dst, const void *host, size_t bytes) {
    ingot_status st = enter(g);
    if (st) return st;
    if (bytes == 0) return INGOT_OK;
    if (!dst || !host) return fail(g, INGOT_INVALID, "null pointer");
    cudaError_t e = cudaMemcpyAsync(dst, host, bytes, cudaMemcpyHostToDevice, g->stream);
    if (e != cudaSuccess) return cuda_fail(g, e, "upload");
    return INGOT_OK;
}

ingot_status ingot_buffer_read(ingot_gpu *g, void *host, const void *src, size_t bytes) {
    ingot_status st = enter(g);
    if (st) return st;
    if (bytes == 0) return INGOT_OK;
    if (!src || !host) return fail(g, INGOT_INVALID, "null pointer");
    cudaError_t e = cudaMemcpyAsync(host, src, bytes, cudaMemcpyDeviceToHost, g->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(g->stream);
    if (e != cudaSuccess) return cuda_fail(g, e, "read");
    return INGOT_OK;
}

ingot_status ingot_buffer_zero(ingot_gpu *g, void *p, size_t bytes) {
    ingot_status st = enter(g);
    if (st) return st;
    if (bytes == 0) return INGOT_OK;
    cudaError_t e = cudaMemsetAsync(p, 0, bytes, g->stream);
    if (e != cudaSuccess) return cuda_fail(g, e, "memset");
    return INGOT_OK;
}

ingot_status ingot_host_alloc(ingot_gpu *g, size_t bytes, void **p) {
    ingot_status st = enter(g);
    if (st) return st;
    if (!p) return fail(g, INGOT_INVALID, "null output pointer");
    cudaError_t e = cudaHostAlloc(p, bytes ? bytes : 16, cudaHostAllocDefault);
    if (e != cudaSuccess) { cudaGetLastError(); return fail(g, INGOT_INVALID, "out of pinned host memory"); }
    return INGOT_OK;
}

ingot_status ingot_host_free(ingot_gpu *g, void *p) {
    if (!g) return INGOT_INVALID;
    if (p) cudaFreeHost(p);
    return INGOT_OK;
}

ingot_status ingot_weight_upload(ingot_gpu *g, const void *host, uint32_t kind, uint64_t cols, uint64_t rows,
                                 uint64_t count, size_t bytes, void **p) {
    ingot_status st = enter(g);
    if (st) return st;
    uint64_t stride, total;
    st = ingot_tensor_layout(kind, cols, rows, count, &stride, &total);
    if (st == INGOT_UNSUPPORTED) return fail(g, st, "GGML type " + std::to_string(kind) + " is unsupported");
    if (st || total != bytes || !host) return fail(g, INGOT_INVALID, "tensor bytes do not match its shape");
    st = ingot_buffer_alloc(g, bytes, p);
    if (st) return st;
    st = ingot_buffer_upload(g, *p, host, bytes);
    if (st) { cudaFree(*p); *p = nullptr; }
    return st;
}

// ---- operators --------------------------------------------------------------

ingot_status ingot_dequant_rows(ingot_gpu *g, const void *w, uint32_t cols, uint64_t rows, uint32_t stride,
                                uint32_t kind, float *y) {
    ingot_status st = enter(g);
    if (st) return st;
    if ((st = check_matrix(g, kind, cols, rows ? 1 : 0, stride))) return st;
    if (!w || !y) return fail(g, INGOT_INVALID, "null pointer");
    return after_launch(g, launch_dequant(static_cast<const uint8_t *>(w), cols, rows, stride, kind, y, ctx_of(g)), "dequant_rows");
}

// Inside an independent scope a one-token tensor-core projection is not launched at once: the
// scope's projections are launched together, as one grid, when it closes.
static bool defer_in_scope(ingot_gpu *g, const GemvCall &c) {
    if (!g->in_scope || !g->group_scope || g->no_mma || g->force_plain) return false;
    if (!gemv_mma_group_eligible(c, ctx_on(g, g->stream))) return false;
    g->pending.push_back(c);
    return true;
}

static ingot_status flush_pending(ingot_gpu *g) {
    std::vector<GemvCall> calls;
    calls.swap(g->pending);
    const LaunchCtx ctx = ctx_on(g, g->stream);
    for (size_t i = 0; i < calls.size();) {
        const uint32_t n = (uint32_t)(calls.size() - i < 4 ? calls.size() - i : 4);
        cudaError_t e = cudaSuccess;
        if (n >= 2 && try_launch_gemv_mma_group(&calls[i], n, ctx, e)) {
            if (e != cudaSuccess) return cuda_fail(g, e, "independent projections");
        } else {
            for (uint32_t k = 0; k < n; ++k) {
                if (!try_launch_gemv_mma(calls[i + k], ctx, e)) return fail(g, INGOT_UNSUPPORTED, "independent projections: no kernel for a deferred call");
                if (e != cudaSuccess) return cuda_fail(g, e, "independent projections");
            }
        }
        i += n;
    }
    return INGOT_OK;
}

static ingot_status gemv_common(ingot_gpu *g, GemvCall &c, uint32_t x_kind, const char *what) {
    ingot_status st = enter(g);
    if (st) return st;
    if (g->chain_recording) return fail(g, INGOT_INVALID, std::string(what) + ": only ingot_matmul_normed and ingot_gate_up_normed can be recorded into a chain");
    if ((st = check_matrix(g, c.kind, c.cols, c.rows, c.stride))) return st;
    if (!x_kind_ok(x_kind)) return fail(g, INGOT_UNSUPPORTED, "activations must be F32 (0), BF16 (30) or packed");
    if (!c.w[0] || (c.nmat == 2 && !c.w[1]) || !c.x || !c.y) return fail(g, INGOT_INVALID, "null pointer");
    c.x_bf16 = x_kind == INGOT_KIND_BF16;
    c.x_packed = x_kind == INGOT_X_PACKED ? 1u : x_kind == INGOT_X_DIGITS ? 3u : x_kind == INGOT_X_PACKED_HI ? 4u : 0u;
    if (c.x_packed == 4u) {
        // high-part rows: one token takes the one-token kernel, more take the multi-token one
        cudaError_t e = cudaSuccess;
        const bool routed = c.ids != nullptr;
        if (((uintptr_t)c.x % 16u) == 0 && defer_in_scope(g, c)) return INGOT_OK;
        const bool taken = ((uintptr_t)c.x % 16u) == 0 && !g->no_mma && !g->force_plain &&
                           ((routed || c.count == 1) ? try_launch_gemv_mma(c, ctx_of(g), e) : try_launch_gemv_mt(c, ctx_of(g), e));
        if (!taken) return fail(g, INGOT_UNSUPPORTED, std::string(what) + ": no tensor-core GEMV for these high-part rows and this weight");
        return after_launch(g, e, what);
    }
    if (c.x_packed == 3u) {
        cudaError_t e = cudaSuccess;
        if (!try_launch_gemv_tc(c, ctx_of(g), e))
            return fail(g, INGOT_UNSUPPORTED, std::string(what) + ": digit rows need one token and a weight type the tcgen05 GEMV takes");
        return after_launch(g, e, what);
    }
    if (c.x_packed) {
        // packed rows only feed the tensor-core GEMV: one token, a block-quantised type, 16-byte aligned rows
        cudaError_t e = cudaSuccess;
        if (((uintptr_t)c.x % 16u) == 0 && defer_in_scope(g, c)) return INGOT_OK;
        if (((uintptr_t)c.x % 16u) || !try_launch_gemv_mma(c, ctx_of(g), e))
            return fail(g, INGOT_UNSUPPORTED, std::string(what) + ": packed activations need one token and a quantised weight");
        return after_launch(g, e, what);
    }
    return after_launch(g, launch_gemv(c, ctx_of(g)), what);
}

ingot_status ingot_matmul(ingot_gpu *g, const void *w, uint32_t cols, uint32_t rows, uint32_t stride, uint32_t kind,
                          uint32_t expert, const void *x, uint32_t x_kind, uint32_t count, float *y) {
    GemvCall c = {};
    c.w[0] = static_cast<const uint8_t *>(w);
    c.x = x; c.y = y; c.cols = cols; c.rows = rows; c.stride = stride; c.kind = kind;
    c.expert = expert; c.count = count; c.nmat = 1;
    // more than four tokens: the reference switches to its GEMM (src/metal_generic.rs:182-206)
    // (inside an independent scope the projections run concurrently and the GEMM's scratch is the handle's
    // one workspace: such calls take the GEMV in groups of four tokens, as the reference's project() does
    // for any count inside independent_projections, src/qwen.rs:822)
    if (g && !g->no_mma && !g->force_plain && !g->in_scope && count > 4 && (kind == INGOT_KIND_Q4_K || kind == INGOT_KIND_Q6_K || kind == INGOT_KIND_Q4_0) && cols % 256u == 0 &&
        ((uintptr_t)w % 16u) == 0 && (x_kind == INGOT_KIND_F32 || x_kind == INGOT_KIND_BF16))
        return ingot_gemm(g, w, cols, rows, stride, kind, expert, x, x_kind, count, y);
    return gemv_common(g, c, x_kind, "matmul");
}

// Grows the handle's scratch (never while recording: cudaMalloc cannot be captured).
static ingot_status ensure_workspace(ingot_gpu *g, size_t bytes) {
    if (bytes <= g->workspace_bytes) return INGOT_OK;
    if (g->capturing) return fail(g, INGOT_INVALID, "scratch too small for this call while recording; run it once before recording");
    cudaError_t e = cudaStreamSynchronize(g->stream);
    if (e != cudaSuccess) return cuda_fail(g, e, "synchronize");
    void *p = nullptr;
    e = cudaMalloc(&p, bytes);
    if (e == cudaErrorMemoryAllocation) { cudaGetLastError(); return fail(g, INGOT_INVALID, "out of device memory"); }
    if (e != cudaSuccess) return cuda_fail(g, e, "cudaMalloc");
    // the old block is kept until the handle goes: a command recorded earlier has its address in its
    // kernel arguments and must stay replayable
    g->retired.push_back(g->workspace);
    g->workspace = p;
    g->workspace_bytes = bytes;
    return INGOT_OK;
}

ingot_status ingot_gemm(ingot_gpu *g, const void *w, uint32_t cols, uint32_t rows, uint32_t stride, uint32_t kind,
                        uint32_t expert, const void *x, uint32_t x_kind, uint32_t count, float *y) {
    ingot_status st = enter(g);
    if (!st && g->in_scope) return fail(g, INGOT_INVALID, "gemm: not inside an independent scope (it uses the handle's scratch)");
    
    if (st) return st;
    if ((st = check_matrix(g, kind, cols, rows, stride))) return st;
    if (x_kind != INGOT_KIND_F32 && x_kind != INGOT_KIND_BF16) return fail(g, INGOT_UNSUPPORTED, "gemm: activations must be F32 or BF16");
    if (!w || !x || !y || count == 0) return fail(g, INGOT_INVALID, "gemm: bad arguments");
    if ((kind != INGOT_KIND_Q4_K && kind != INGOT_KIND_Q6_K && kind != INGOT_KIND_Q4_0) || cols % 256u || ((uintptr_t)w % 16u))
        return fail(g, INGOT_UNSUPPORTED, "gemm: no tensor-core kernel for this type or shape");
    if ((st = ensure_workspace(g, gemm_scratch_bytes(cols, rows, count, g->sm_count)))) return st;
    cudaError_t e = launch_gemm_dequant(static_cast<const uint8_t *>(w), cols, rows, stride, kind, expert, x,
                                        x_kind == INGOT_KIND_BF16, count, y, g->workspace, ctx_of(g));
    if (e == cudaErrorNotSupported) { cudaGetLastError(); return fail(g, INGOT_UNSUPPORTED, "gemm: no tensor-core kernel for this type or shape"); }
    return after_launch(g, e, "gemm");
}

ingot_status ingot_gate_up(ingot_gpu *g, const void *gate, const void *up, uint32_t cols, uint32_t rows,
                           uint32_t stride, uint32_t kind, const void *x, uint32_t x_kind, uint32_t count,
                           uint32_t gelu, float *y) {
    GemvCall c = {};
    c.w[0] = static_cast<const uint8_t *>(gate);
    c.w[1] = static_cast<const uint8_t *>(up);
    c.x = x; c.y = y; c.cols = cols; c.rows = rows; c.stride = stride; c.kind = kind;
    c.count = count; c.nmat = 2; c.glu = gelu ? 2 : 1;
    // more than four tokens: two tensor-core GEMMs and the activation, as the reference's generic_gate_up
    // falls back to separate projections + glu for wide batches (src/metal_generic.rs:231-261)
    if (g && !g->no_mma && !g->force_plain && !g->in_scope && count > 4 && (kind == INGOT_KIND_Q4_K || kind == INGOT_KIND_Q6_K || kind == INGOT_KIND_Q4_0) &&
        cols % 256u == 0 && ((uintptr_t)gate % 16u) == 0 && ((uintptr_t)up % 16u) == 0 &&
        (x_kind == INGOT_KIND_F32 || x_kind == INGOT_KIND_BF16) && gate && up && x && y) {
        ingot_status st = enter(g);
        if (st) return st;
        if ((st = check_matrix(g, kind, cols, rows, stride))) return st;
        // scratch: binary16 activations, then the two projection outputs
        const size_t xh = (gemm_scratch_bytes(cols, rows, count, g->sm_count) + 255u) & ~(size_t)255u, out = (size_t)count * rows * 4u;
        if ((st = ensure_workspace(g, xh + 2u * out))) return st;
        uint8_t *ws = static_cast<uint8_t *>(g->workspace);
        float *yg = reinterpret_cast<float *>(ws + xh), *yu = reinterpret_cast<float *>(ws + xh + out);
        cudaError_t e = launch_gemm_dequant(static_cast<const uint8_t *>(gate), cols, rows, stride, kind, 0, x,
                                            x_kind == INGOT_KIND_BF16, count, yg, ws, ctx_of(g));
        if (e == cudaSuccess)
            e = launch_gemm_dequant(static_cast<const uint8_t *>(up), cols, rows, stride, kind, 0, x, x_kind == INGOT_KIND_BF16, count,
                                    yu, ws, ctx_of(g));
        if (e == cudaSuccess) e = launch_activation(yg, yu, (uint64_t)count * rows, gelu, y, ctx_of(g));
        if (e != cudaErrorNotSupported) return after_launch(g, e, "gate_up");
        cudaGetLastError();
    }
    return gemv_common(g, c, x_kind, "gate_up");
}

// Consumes the links ingot_tp_signal_next / ingot_tp_wait_next set for this projection.
static ingot_status apply_tp_links(ingot_gpu *g, GemvCall &c, const float *a, const float *b, const char *what) {
    ingot_group *sg = g->tp_signal_group, *wg = g->tp_wait_group;
    g->tp_signal_group = g->tp_wait_group = nullptr;
    if (sg) {
        const uint8_t *base = sg->peer[sg->rank];
        const uint8_t *y = reinterpret_cast<const uint8_t *>(c.y);
        if (y < base || y + (size_t)c.rows * 4u > base + sg->window_bytes || ((size_t)(y - base) % 4u))
            return fail(g, INGOT_INVALID, std::string(what) + ": the output of a signalling projection must lie inside the group's window");
        const size_t off = (size_t)(y - base);
        for (uint32_t r = 0; r < sg->world; ++r) {
            if (!sg->peer[r]) return fail(g, INGOT_INVALID, std::string(what) + ": the group is not connected");
            c.tp.out[r] = sg->twin(r, off);
        }
        c.tp.n_out = sg->world;
        c.tp.out_tag = g->tp_signal_slot + 1u;
        c.tp.tag_mul = sg->slots + 1u;
        c.tp.step = sg->step_counter();
        sg->shard[g->tp_signal_slot] = {off, c.rows};
    }
    if (wg) {
        const uint8_t *base = wg->peer[wg->rank];
        const float *in[2] = {a, b};
        for (int i = 0; i < 2; ++i) {
            const uint32_t slot = g->tp_wait_slot[i];
            if (slot == TP_NO_SLOT) continue;
            const ingot_group::Shard &sh = wg->shard[slot];
            if (sh.rows == 0) return fail(g, INGOT_INVALID, std::string(what) + ": waits for a slot no projection has signalled yet");
            // which of the two normalised inputs the slot's vector is: the one that contains this rank's rows of it
            int k = -1;
            for (int v = 0; v < 2 && k < 0; ++v) {
                const uint8_t *x = reinterpret_cast<const uint8_t *>(in[v]);
                if (x && x >= base && x + (size_t)c.cols * 4u <= base + wg->window_bytes && (size_t)(x - base) <= sh.off &&
                    sh.off + (size_t)sh.rows * 4u <= (size_t)(x - base) + (size_t)c.cols * 4u && !c.tp.in[v])
                    k = v;
            }
            if (k < 0) return fail(g, INGOT_INVALID, std::string(what) + ": the awaited slot's vector is not one of this projection's inputs");
            c.tp.in[k] = wg->twin(wg->rank, (size_t)(reinterpret_cast<const uint8_t *>(in[k]) - base));
            c.tp.in_tag[k] = slot + 1u;
        }
        c.tp.tag_mul = wg->slots + 1u;
        c.tp.step = wg->step_counter();
    }
    return INGOT_OK;
}

// add_rms fused into the projection that consumes it (one token, tensor-core GEMV only).
static ingot_status normed_common(ingot_gpu *g, GemvCall &c, const float *a, const float *b, const float *norm_w, float *s,
                                  float eps, uint32_t add, uint32_t round_bf16, const char *what) {
    ingot_status st = enter(g);
    if (st) return st;
    if ((st = check_matrix(g, c.kind, c.cols, c.rows, c.stride))) return st;
    if (!c.w[0] || (c.nmat == 2 && !c.w[1]) || !a || (add && !b) || !c.y) return fail(g, INGOT_INVALID, "null pointer");
    if (s && (s == a || s == b)) return fail(g, INGOT_INVALID, std::string(what) + ": the sum cannot be stored over an input that every CTA still reads");
    if (((uintptr_t)a % 16u) || (b && ((uintptr_t)b % 16u)) || (s && ((uintptr_t)s % 16u)) || (norm_w && ((uintptr_t)norm_w % 16u)))
        return fail(g, INGOT_INVALID, std::string(what) + ": vectors must be 16-byte aligned");
    c.norm_a = a; c.norm_b = add ? b : nullptr; c.norm_w = norm_w; c.norm_s = add ? s : nullptr;
    c.norm_eps = eps; c.norm_round_bf16 = round_bf16; c.norm_wide = g->wide_rows ? 1u : 0u;
    c.count = 1;
    if ((st = apply_tp_links(g, c, a, add ? b : nullptr, what))) return st;
    if (g->chain_recording) {
        if (c.tp.n_out || c.tp.in[0] || c.tp.in[1]) return fail(g, INGOT_UNSUPPORTED, std::string(what) + ": tensor-parallel links cannot be recorded into a chain");
        if (g->no_mma || g->force_plain || !chain_call_eligible(c))
            return fail(g, INGOT_UNSUPPORTED, std::string(what) + ": this projection cannot be part of a chain (weight type, alignment or shape)");
        g->chain_calls.push_back(c);
        return INGOT_OK;
    }
    cudaError_t e = cudaSuccess;
    const bool aligned = ((uintptr_t)c.w[0] % 16u) == 0 && (c.nmat < 2 || ((uintptr_t)c.w[1] % 16u) == 0) && ((size_t)c.rows * c.stride) % 16u == 0;
    if (aligned && defer_in_scope(g, c)) return INGOT_OK;
    if (g->no_mma || g->force_plain || !aligned || !try_launch_gemv_mma(c, ctx_of(g), e))
        return fail(g, INGOT_UNSUPPORTED, std::string(what) + ": no fused kernel for this weight; use add_rms and the plain projection");
    return after_launch(g, e, what);
}

ingot_status ingot_matmul_normed(ingot_gpu *g, const void *w, uint32_t cols, uint32_t rows, uint32_t stride, uint32_t kind,
                                 uint32_t expert, const float *a, const float *b, const float *norm_w, float *s, float eps,
                                 uint32_t add, uint32_t round_bf16, float *y) {
    GemvCall c = {};
    c.w[0] = static_cast<const uint8_t *>(w);
    c.y = y; c.cols = cols; c.rows = rows; c.stride = stride; c.kind = kind; c.expert = expert; c.nmat = 1;
    return normed_common(g, c, a, b, norm_w, s, eps, add, round_bf16, "matmul_normed");
}

ingot_status ingot_gate_up_normed(ingot_gpu *g, const void *gate, const void *up, uint32_t cols, uint32_t rows, uint32_t stride,
                                  uint32_t kind, const float *a, const float *b, const float *norm_w, float *s, float eps,
                                  uint32_t add, uint32_t round_bf16, uint32_t gelu, float *y) {
    GemvCall c = {};
    c.w[0] = static_cast<const uint8_t *>(gate);
    c.w[1] = static_cast<const uint8_t *>(up);
    c.y = y; c.cols = cols; c.rows = rows; c.stride = stride; c.kind = kind; c.nmat = 2; c.glu = gelu ? 2 : 1;
    return normed_common(g, c, a, b, norm_w, s, eps, add, round_bf16, "gate_up_normed");
}

ingot_status ingot_routed(ingot_gpu *g, const void *w, uint32_t cols, uint32_t rows, uint32_t stride, uint32_t kind,
                          uint32_t experts, const void *x, uint32_t x_kind, const uint32_t *ids, uint32_t per_pair,
                          uint32_t top, uint32_t pairs, float *y) {
    if (g && (!ids || top == 0 || experts == 0)) return fail(g, INGOT_INVALID, "routed projection needs ids, top and experts");
    GemvCall c = {};
    c.w[0] = static_cast<const uint8_t *>(w);
    c.x = x; c.y = y; c.ids = ids; c.cols = cols; c.rows = rows; c.stride = stride; c.kind = kind;
    c.pairs = pairs; c.top = top; c.per_pair = per_pair; c.n_experts = experts; c.nmat = 1;
    return gemv_common(g, c, x_kind, "routed");
}

ingot_status ingot_routed_gate_up(ingot_gpu *g, const void *gate, const void *up, uint32_t cols, uint32_t rows,
                                  uint32_t stride, uint32_t kind, uint32_t experts, const void *x, uint32_t x_kind,
                                  const uint32_t *ids, uint32_t top, uint32_t pairs, float *y) {
    if (g && (!ids || top == 0 || experts == 0)) return fail(g, INGOT_INVALID, "routed projection needs ids, top and experts");
    GemvCall c = {};
    c.w[0] = static_cast<const uint8_t *>(gate);
    c.w[1] = static_cast<const uint8_t *>(up);
    c.x = x; c.y = y; c.ids = ids; c.cols = cols; c.rows = rows; c.stride = stride; c.kind = kind;
    c.pairs = pairs; c.top = top; c.per_pair = 0; c.n_experts = experts; c.nmat = 2; c.glu = 1;
    return gemv_common(g, c, x_kind, "routed_gate_up");
}

// Per-expert projections over the expert grouping (Generic::moe_packed, src/generic.rs:578-660).
static ingot_status expert_tiles_common(ingot_gpu *g, GemvCall &c, const uint32_t *tiles, const uint32_t *pairs, uint32_t tile_capacity,
                                        bool gather, const char *what) {
    ingot_status st = enter(g);
    if (st) return st;
    if (g->chain_recording) return fail(g, INGOT_INVALID, std::string(what) + ": only ingot_matmul_normed and ingot_gate_up_normed can be recorded into a chain");
    if ((st = check_matrix(g, c.kind, c.cols, c.rows, c.stride))) return st;
    if (!c.w[0] || (c.nmat == 2 && !c.w[1]) || !c.x || !c.y || !tiles || !pairs || c.top == 0 || c.n_experts == 0 || tile_capacity == 0)
        return fail(g, INGOT_INVALID, std::string(what) + ": bad arguments");
    cudaError_t e = cudaSuccess;
    if (g->no_mma || g->force_plain || !try_launch_gemv_tiles(c, tiles, pairs, tile_capacity, gather, ctx_of(g), e))
        return fail(g, INGOT_UNSUPPORTED, std::string(what) + ": no grouped kernel for this weight type or alignment; project pair by pair");
    return after_launch(g, e, what);
}

ingot_status ingot_expert_project(ingot_gpu *g, const void *w, uint32_t cols, uint32_t rows, uint32_t stride, uint32_t kind,
                                  uint32_t experts, const float *x, const uint32_t *tiles, const uint32_t *pairs, uint32_t tile_capacity,
                                  uint32_t top, uint32_t n_pairs, uint32_t gather, float *y_packed) {
    GemvCall c = {};
    c.w[0] = static_cast<const uint8_t *>(w);
    c.x = x; c.y = y_packed; c.cols = cols; c.rows = rows; c.stride = stride; c.kind = kind;
    c.pairs = n_pairs; c.top = top; c.n_experts = experts; c.nmat = 1;
    return expert_tiles_common(g, c, tiles, pairs, tile_capacity, gather != 0, "expert_project");
}

ingot_status ingot_expert_gate_up(ingot_gpu *g, const void *gate, const void *up, uint32_t cols, uint32_t rows, uint32_t stride,
                                  uint32_t kind, uint32_t experts, const float *x, const uint32_t *tiles, const uint32_t *pairs,
                                  uint32_t tile_capacity, uint32_t top, uint32_t n_pairs, float *y_packed) {
    GemvCall c = {};
    c.w[0] = static_cast<const uint8_t *>(gate);
    c.w[1] = static_cast<const uint8_t *>(up);
    c.x = x; c.y = y_packed; c.cols = cols; c.rows = rows; c.stride = stride; c.kind = kind;
    c.pairs = n_pairs; c.top = top; c.n_experts = experts; c.nmat = 2; c.glu = 1;
    return expert_tiles_common(g, c, tiles, pairs, tile_capacity, true, "expert_gate_up");
}

ingot_status ingot_route_topk(ingot_gpu *g, const float *logits, uint32_t experts, uint32_t top, uint32_t tokens,
                              uint32_t *ids, float *weights) {
    ingot_status st = enter(g);
    if (st) return st;
    if (top == 0 || top > experts || experts > 512) return fail(g, INGOT_INVALID, "invalid router scores or expert count");
    if (!logits || !ids || !weights) return fail(g, INGOT_INVALID, "null pointer");
    return after_launch(g, launch_route_topk(logits, experts, top, tokens, ids, weights, ctx_of(g)), "route_topk");
}

ingot_status ingot_moe_sum(ingot_gpu *g, const float *routed, const float *weights, uint32_t width, uint32_t top,
                           uint32_t tokens, float *y) {
    ingot_status st = enter(g);
    if (st) return st;
    if (!routed || !weights || !y || width % 4u) return fail(g, INGOT_INVALID, "moe_sum: bad arguments");
    return after_launch(g, launch_moe_sum(routed, weights, width, top, tokens, y, ctx_of(g)), "moe_sum");
}

ingot_status ingot_activation(ingot_gpu *g, const float *gate, const float *up, uint64_t n, uint32_t gelu, float *y) {
    ingot_status st = enter(g);
    if (st) return st;
    if (!gate || !up || !y) return fail(g, INGOT_INVALID, "null pointer");
    return after_launch(g, launch_activation(gate, up, n, gelu, y, ctx_of(g)), "activation");
}

// ---- architecture glue of the generic path (kernels/generic_arch.metal:2-17) ----

static ingot_status glue_common(ingot_gpu *g, uint32_t op, const float *x, uint64_t n, uint32_t width, uint32_t offset, uint32_t stride,
                                float value, float *y, const char *what) {
    ingot_status st = enter(g);
    if (st) return st;
    if (g->chain_recording) return fail(g, INGOT_INVALID, std::string(what) + ": only ingot_matmul_normed and ingot_gate_up_normed can be recorded into a chain");
    if (!x || !y) return fail(g, INGOT_INVALID, "null pointer");
    return after_launch(g, launch_glue(op, x, n, width, offset, stride, value, y, ctx_of(g)), what);
}

ingot_status ingot_scale_rows(ingot_gpu *g, const float *x, uint64_t n, float scale, float *y) {
    return glue_common(g, 0, x, n, 1, 0, 0, scale, y, "scale_rows");
}

ingot_status ingot_softcap_rows(ingot_gpu *g, const float *x, uint64_t n, float cap, float *y) {
    if (g && !(cap != 0.0f)) return fail(g, INGOT_INVALID, "softcap_rows: the cap must not be zero");
    return glue_common(g, 1, x, n, 1, 0, 0, cap, y, "softcap_rows");
}

ingot_status ingot_swiglu_fused(ingot_gpu *g, const float *x, uint32_t tokens, uint32_t ff, float *y) {
    if (g && ff == 0) return fail(g, INGOT_INVALID, "swiglu_fused: zero width");
    return glue_common(g, 2, x, (uint64_t)tokens * ff, ff, 0, 0, 0.f, y, "swiglu_fused");
}

ingot_status ingot_copy_columns(ingot_gpu *g, const float *x, uint32_t rows, uint32_t width, uint32_t offset, uint32_t stride, float *y) {
    if (g && (width == 0 || (uint64_t)offset + width > stride)) return fail(g, INGOT_INVALID, "copy_columns: the columns must lie inside a row");
    return glue_common(g, 3, x, (uint64_t)rows * width, width, offset, stride, 0.f, y, "copy_columns");
}

ingot_status ingot_merge(ingot_gpu *g, const float *routed, const float *shared, const float *weights,
                         const float *shared_logit, uint32_t width, uint32_t top, float *y) {
    ingot_status st = enter(g);
    if (st) return st;
    if (!routed || !shared || !weights || !shared_logit || !y) return fail(g, INGOT_INVALID, "null pointer");
    return after_launch(g, launch_merge(routed, shared, weights, shared_logit, width, top, y, ctx_of(g)), "merge");
}

ingot_status ingot_add_rms(ingot_gpu *g, const float *a, const float *b, const float *w, float *s, float *y,
                           void *y_bf16, uint32_t width, uint32_t rows, float eps, uint32_t add) {
    return ingot_add_rms_packed(g, a, b, w, s, y, y_bf16, nullptr, 0, width, rows, eps, add);
}

ingot_status ingot_add_rms_packed(ingot_gpu *g, const float *a, const float *b, const float *w, float *s, float *y,
                                  void *y_bf16, void *y_packed, uint32_t pack_from_bf16, uint32_t width, uint32_t rows,
                                  float eps, uint32_t add) {
    ingot_status st = enter(g);
    if (st) return st;
    if (!a || (add && !b) || width % 4u || width == 0 || pack_from_bf16 > 3u || (y_packed && (width % 64u || ((uintptr_t)y_packed % 16u))))
        return fail(g, INGOT_INVALID, "add_rms: bad arguments");
    return after_launch(g, launch_add_rms(a, b, w, s, y, width, rows, eps, add, y_bf16, y_packed, pack_from_bf16, ctx_of(g)),
                        "add_rms");
}

ingot_status ingot_expert_layout(ingot_gpu *g, const uint32_t *ids, uint32_t pairs, uint32_t experts,
                                 uint32_t tile_capacity, uint32_t *layout, uint32_t *tiles, uint32_t *packed,
                                 uint32_t *inverse) {
    ingot_status st = enter(g);
    if (st) return st;
    if (!ids || !layout || !tiles || !packed || !inverse || experts == 0 || experts > 512)
        return fail(g, INGOT_INVALID, "expert_layout: bad arguments");
    return after_launch(g, launch_expert_layout(ids, pairs, experts, tile_capacity, layout, tiles, packed, inverse, ctx_of(g)),
                        "expert_layout");
}

// ---- the packed MoE path at prefill width: per-expert tensor-core GEMMs over the grouping's packed rows ----

ingot_status ingot_gather_rows(ingot_gpu *g, const float *x, const uint32_t *packed, uint32_t pairs, uint32_t top, uint32_t width, float *y) {
    ingot_status st = enter(g);
    if (st) return st;
    if (g->chain_recording) return fail(g, INGOT_INVALID, "gather_rows: only ingot_matmul_normed and ingot_gate_up_normed can be recorded into a chain");
    if (!x || !packed || !y || top == 0 || width % 4u || ((uintptr_t)x % 16u) || ((uintptr_t)y % 16u))
        return fail(g, INGOT_INVALID, "gather_rows: rows of 4 n floats, 16-byte aligned");
    return after_launch(g, launch_gather_rows(x, packed, pairs, top, width, y, ctx_of(g)), "gather_rows");
}

// The (count, first) table of ingot_expert_layout on the host: the loop over the experts below is driven from here,
// as the reference's host drives one tiled GEMM per expert tile.  Waits for the stream (not while recording).
static ingot_status read_layout(ingot_gpu *g, const uint32_t *layout, uint32_t experts, uint32_t pairs, std::vector<uint32_t> &host, const char *what) {
    if (g->capturing || g->in_scope || g->chain_recording)
        return fail(g, INGOT_INVALID, std::string(what) + ": reads the grouping back to the host; not inside a recording, a scope or a chain");
    host.resize(2u * (size_t)experts);
    ingot_status st = ingot_buffer_read(g, host.data(), layout, host.size() * 4u);
    if (st) return st;
    uint64_t total = 0;
    for (uint32_t e = 0; e < experts; ++e) {
        if (host[2u * e + 1u] != total) return fail(g, INGOT_INVALID, std::string(what) + ": the layout table is not an expert grouping");
        total += host[2u * e];
    }
    if (total > pairs) return fail(g, INGOT_INVALID, std::string(what) + ": the layout table holds more pairs than given");
    return INGOT_OK;
}

ingot_status ingot_expert_gemm(ingot_gpu *g, const void *w, uint32_t cols, uint32_t rows, uint32_t stride, uint32_t kind, uint32_t experts,
                               const float *x_packed, const uint32_t *layout, uint32_t pairs, float *y_packed) {
    ingot_status st = enter(g);
    if (st) return st;
    if (!w || !x_packed || !layout || !y_packed || experts == 0) return fail(g, INGOT_INVALID, "expert_gemm: bad arguments");
    if ((st = check_matrix(g, kind, cols, rows, stride))) return st;
    std::vector<uint32_t> table;
    if ((st = read_layout(g, layout, experts, pairs, table, "expert_gemm"))) return st;
    const uint8_t *base = static_cast<const uint8_t *>(w);
    for (uint32_t e = 0; e < experts && !st; ++e) {
        const uint32_t n = table[2u * e], first = table[2u * e + 1u];
        if (n) st = ingot_matmul(g, base, cols, rows, stride, kind, e, x_packed + (size_t)first * cols, INGOT_KIND_F32, n, y_packed + (size_t)first * rows);
    }
    return st;
}

ingot_status ingot_expert_gemm_gate_up(ingot_gpu *g, const void *gate, const void *up, uint32_t cols, uint32_t rows, uint32_t stride,
                                       uint32_t kind, uint32_t experts, const float *x_packed, const uint32_t *layout, uint32_t pairs,
                                       uint32_t gelu, float *y_packed) {
    ingot_status st = enter(g);
    if (st) return st;
    if (!gate || !up || !x_packed || !layout || !y_packed || experts == 0) return fail(g, INGOT_INVALID, "expert_gemm_gate_up: bad arguments");
    if ((st = check_matrix(g, kind, cols, rows, stride))) return st;
    std::vector<uint32_t> table;
    if ((st = read_layout(g, layout, experts, pairs, table, "expert_gemm_gate_up"))) return st;
    const size_t slab = (size_t)rows * stride;
    for (uint32_t e = 0; e < experts && !st; ++e) {
        const uint32_t n = table[2u * e], first = table[2u * e + 1u];
        if (n) st = ingot_gate_up(g, static_cast<const uint8_t *>(gate) + e * slab, static_cast<const uint8_t *>(up) + e * slab, cols, rows, stride,
                                  kind, x_packed + (size_t)first * cols, INGOT_KIND_F32, n, gelu, y_packed + (size_t)first * rows);
    }
    return st;
}

ingot_status ingot_combine_packed(ingot_gpu *g, const float *routed, const float *weights, const uint32_t *inverse,
                                  uint32_t width, uint32_t top, uint32_t tokens, float *y) {
    ingot_status st = enter(g);
    if (st) return st;
    if (!routed || !weights || !inverse || !y || width % 4u) return fail(g, INGOT_INVALID, "combine_packed: bad arguments");
    return after_launch(g, launch_combine_packed(routed, weights, inverse, width, top, tokens, y, ctx_of(g)), "combine_packed");
}

ingot_status ingot_ep_localize(ingot_gpu *g, const uint32_t *ids, const float *weights, uint32_t pairs, uint32_t first_expert,
                               uint32_t local_experts, uint32_t *ids_out, float *weights_out) {
    ingot_status st = enter(g);
    if (st) return st;
    if (!ids || !weights || !ids_out || !weights_out || local_experts == 0) return fail(g, INGOT_INVALID, "ep_localize: bad arguments");
    return after_launch(g, launch_ep_localize(ids, weights, pairs, first_expert, local_experts, ids_out, weights_out, ctx_of(g)),
                        "ep_localize");
}

ingot_status ingot_convert_bf16(ingot_gpu *g, const float *x, uint64_t n, void *y) {
    ingot_status st = enter(g);
    if (st) return st;
    if (!x || !y) return fail(g, INGOT_INVALID, "null pointer");
    return after_launch(g, launch_convert_bf16(x, n, y, ctx_of(g)), "convert_bf16");
}

// ---- the rest of a generic decode step ---------------------------------------------------------

ingot_status ingot_embedding_batch(ingot_gpu *g, const void *w, const uint32_t *ids, uint32_t width, uint32_t rows, uint32_t stride,
                                   uint32_t kind, uint32_t count, float *y) {
    ingot_status st = enter(g);
    if (st) return st;
    if (g->chain_recording) return fail(g, INGOT_INVALID, "embedding_batch: only ingot_matmul_normed and ingot_gate_up_normed can be recorded into a chain");
    if ((st = check_matrix(g, kind, width, rows, stride))) return st;
    if (!w || !ids || !y) return fail(g, INGOT_INVALID, "null pointer");
    return after_launch(g, launch_embedding(static_cast<const uint8_t *>(w), ids, width, stride, kind, count, rows, y, ctx_of(g)), "embedding_batch");
}

ingot_status ingot_qk_rope_cache(ingot_gpu *g, const float *q, const float *k, const float *v, const float *q_norm, const float *k_norm,
                                 const float *factors, float *q_out, float *k_cache, float *v_cache, const ingot_rope_params *p,
                                 uint32_t tokens) {
    ingot_status st = enter(g);
    if (st) return st;
    if (g->chain_recording) return fail(g, INGOT_INVALID, "qk_rope_cache: only ingot_matmul_normed and ingot_gate_up_normed can be recorded into a chain");
    if (!p || !q || !k || !v || !q_out || !k_cache || !v_cache) return fail(g, INGOT_INVALID, "null pointer");
    if (p->head_dim == 0 || p->head_dim > 512 || p->heads == 0 || p->kv_heads == 0 || p->rotated > p->head_dim || (p->rotated & 1u) ||
        (p->qk_norm && (!q_norm || !k_norm)) || (p->use_factors && !factors))
        return fail(g, INGOT_INVALID, "qk_rope_cache: bad geometry");
    RopeParams rp = {p->head_dim, p->heads, p->kv_heads, p->rotated, p->position, p->base, p->neox, p->use_factors, p->qk_norm, p->eps,
                     p->value_norm, p->q_scale};
    return after_launch(g, launch_rope_cache(q, k, v, q_norm, k_norm, factors, q_out, k_cache, v_cache, rp, tokens, ctx_of(g)), "qk_rope_cache");
}

ingot_status ingot_attention_decode(ingot_gpu *g, const float *q, const float *k_cache, const float *v_cache, float *out, uint32_t head_dim,
                                    uint32_t heads, uint32_t kv_heads, uint32_t position, uint32_t window, uint32_t tokens) {
    ingot_status st = enter(g);
    if (st) return st;
    if (g->chain_recording) return fail(g, INGOT_INVALID, "attention_decode: only ingot_matmul_normed and ingot_gate_up_normed can be recorded into a chain");
    if (!q || !k_cache || !v_cache || !out) return fail(g, INGOT_INVALID, "null pointer");
    if (heads == 0 || kv_heads == 0 || heads % kv_heads || tokens > 4) return fail(g, INGOT_INVALID, "attention_decode: bad geometry (one to four query tokens)");
    cudaError_t e = launch_attention_decode(q, k_cache, v_cache, out, head_dim, heads, kv_heads, position, window, tokens, ctx_of(g));
    if (e == cudaErrorNotSupported) { cudaGetLastError(); return fail(g, INGOT_UNSUPPORTED, "attention_decode: head dimension must be 64, 96, 128, 256 or 512"); }
    return after_launch(g, e, "attention_decode");
}

// flash_prefill_<D> (kernels/generic.metal:19-136; Generic::flash, src/generic.rs:421-470): causal attention of `rows` query rows,
// the first at `position`, over the first `length` rows of the float32 caches.
ingot_status ingot_attention_prefill(ingot_gpu *g, const float *q, const float *k_cache, const float *v_cache, float *out, uint32_t head_dim,
                                     uint32_t heads, uint32_t kv_heads, uint32_t length, uint32_t position, uint32_t rows, uint32_t window) {
    ingot_status st = enter(g);
    if (st) return st;
    if (g->chain_recording) return fail(g, INGOT_INVALID, "attention_prefill: only ingot_matmul_normed and ingot_gate_up_normed can be recorded into a chain");
    if (!q || !k_cache || !v_cache || !out) return fail(g, INGOT_INVALID, "null pointer");
    if (heads == 0 || kv_heads == 0 || heads % kv_heads || rows > 65535u || (uint64_t)position + rows > length)
        return fail(g, INGOT_INVALID, "attention_prefill: bad geometry (position + rows must lie within length; at most 65535 rows)");
    cudaError_t e = launch_attention_decode(q, k_cache, v_cache, out, head_dim, heads, kv_heads, position, window, rows, ctx_of(g));
    if (e == cudaErrorNotSupported) { cudaGetLastError(); return fail(g, INGOT_UNSUPPORTED, "attention_prefill: head dimension must be 64, 96, 128, 256 or 512"); }
    return after_launch(g, e, "attention_prefill");
}

ingot_status ingot_greedy_select(ingot_gpu *g, const float *logits, const uint32_t *mapping, uint32_t rows, uint32_t vocab, uint32_t *scratch,
                                 uint32_t *out) {
    ingot_status st = enter(g);
    if (st) return st;
    if (g->chain_recording) return fail(g, INGOT_INVALID, "greedy_select: only ingot_matmul_normed and ingot_gate_up_normed can be recorded into a chain");
    if (!logits || !scratch || !out || vocab == 0) return fail(g, INGOT_INVALID, "greedy_select: bad arguments");
    return after_launch(g, launch_greedy(logits, mapping, rows, vocab, scratch, out, ctx_of(g)), "greedy_select");
}

ingot_status ingot_packed_x_bytes(uint32_t cols, uint64_t *bytes) {
    if (!bytes || cols == 0 || cols % 64u) return INGOT_INVALID;
    *bytes = packed_x_bytes(cols);
    return INGOT_OK;
}

ingot_status ingot_pack_x(ingot_gpu *g, const void *x, uint32_t x_kind, uint32_t rows, uint32_t cols, void *packed) {
    ingot_status st = enter(g);
    if (st) return st;
    if (!x || !packed || cols == 0 || cols % 64u || ((uintptr_t)packed % 16u)) return fail(g, INGOT_INVALID, "pack_x: bad arguments");
    if (x_kind != INGOT_KIND_F32 && x_kind != INGOT_KIND_BF16) return fail(g, INGOT_UNSUPPORTED, "pack_x: activations must be F32 or BF16");
    return after_launch(g, launch_pack_x(x, x_kind == INGOT_KIND_BF16, rows, cols, packed, ctx_of(g)), "pack_x");
}

ingot_status ingot_packed_hi_bytes(uint32_t cols, uint64_t *bytes) {
    if (!bytes || cols == 0 || cols % 64u) return INGOT_INVALID;
    *bytes = packed_hi_bytes(cols);
    return INGOT_OK;
}

ingot_status ingot_pack_x_hi(ingot_gpu *g, const void *x_bf16, uint32_t rows, uint32_t cols, void *packed) {
    ingot_status st = enter(g);
    if (st) return st;
    if (!x_bf16 || !packed || cols == 0 || cols % 64u || ((uintptr_t)packed % 16u)) return fail(g, INGOT_INVALID, "pack_x_hi: bad arguments");
    return after_launch(g, launch_pack_x_hi(x_bf16, rows, cols, packed, ctx_of(g)), "pack_x_hi");
}

ingot_status ingot_packed_digits_bytes(uint32_t cols, uint64_t *bytes) {
    if (!bytes || cols == 0 || cols % 256u) return INGOT_INVALID;
    *bytes = packed_digits_bytes(cols);
    return INGOT_OK;
}

ingot_status ingot_pack_digits(ingot_gpu *g, const void *x, uint32_t x_kind, uint32_t rows, uint32_t cols, void *packed) {
    ingot_status st = enter(g);
    if (st) return st;
    if (!x || !packed || cols == 0 || cols % 256u || ((uintptr_t)packed % 16u)) return fail(g, INGOT_INVALID, "pack_digits: bad arguments");
    if (x_kind != INGOT_KIND_F32 && x_kind != INGOT_KIND_BF16) return fail(g, INGOT_UNSUPPORTED, "pack_digits: activations must be F32 or BF16");
    return after_launch(g, launch_pack_digits(x, x_kind == INGOT_KIND_BF16, rows, cols, packed, ctx_of(g)), "pack_digits");
}

// ---- independent projections ----------------------------------------------------------------

ingot_status ingot_independent_begin(ingot_gpu *g) {
    ingot_status st = enter(g);
    if (st) return st;
    if (g->in_scope) return fail(g, INGOT_INVALID, "independent scope already open");
    if (!g->fork_event) {
        cudaError_t e = cudaEventCreateWithFlags(&g->fork_event, cudaEventDisableTiming);
        for (int i = 0; i < ingot_gpu::SIDE_STREAMS && e == cudaSuccess; ++i) {
            e = cudaStreamCreateWithFlags(&g->side[i], cudaStreamNonBlocking);
            if (e == cudaSuccess) e = cudaEventCreateWithFlags(&g->join_event[i], cudaEventDisableTiming);
        }
        if (e != cudaSuccess) return cuda_fail(g, e, "independent scope setup");
    }
    cudaError_t e = cudaEventRecord(g->fork_event, g->stream);
    if (e != cudaSuccess) return cuda_fail(g, e, "independent scope fork");
    g->in_scope = true;
    g->pending.clear();
    g->scope_next = 0;
    g->scope_used = 0;
    return INGOT_OK;
}

ingot_status ingot_independent_end(ingot_gpu *g) {
    if (!g) return INGOT_INVALID;
    if (!g->in_scope) return fail(g, INGOT_INVALID, "no independent scope open");
    g->in_scope = false;
    ingot_status st = g->pending.empty() ? INGOT_OK : flush_pending(g);
    for (int i = 0; i < ingot_gpu::SIDE_STREAMS; ++i) {
        if (!(g->scope_used & (1 << i))) continue;
        cudaError_t e = cudaEventRecord(g->join_event[i], g->side[i]);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(g->stream, g->join_event[i], 0);
        if (e != cudaSuccess) return cuda_fail(g, e, "independent scope join");
    }
    return st;
}

// ---- tensor-parallel groups: row shards over several GPUs, exchanged by the projections themselves ----

ingot_status ingot_group_create(ingot_gpu *g, uint32_t rank, uint32_t world, size_t window_bytes, uint32_t slots, ingot_group **out,
                                void *handle64) {
    ingot_status st = enter(g);
    if (st) return st;
    if (!out || world == 0 || world > TP_MAX_RANKS || rank >= world || slots == 0) return fail(g, INGOT_INVALID, "group_create: bad arguments");
    *out = nullptr;
    ingot_group *gr = new (std::nothrow) ingot_group();
    if (!gr) return fail(g, INGOT_DEVICE, "out of host memory");
    gr->gpu = g; gr->rank = rank; gr->world = world; gr->slots = slots;
    gr->window_bytes = window_bytes;
    gr->twin_off = (window_bytes + 255u) & ~(size_t)255u;
    gr->ctrl_off = gr->twin_off + 2u * gr->twin_off;
    gr->total_bytes = gr->ctrl_off + 256u;
    gr->shard.assign(slots, {});
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, gr->total_bytes);
    if (e == cudaSuccess) e = cudaMemset(p, 0, gr->total_bytes);
    if (e == cudaSuccess && handle64) {
        static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
        e = cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t *>(handle64), p);
    }
    if (e != cudaSuccess) {
        if (p) cudaFree(p);
        delete gr;
        if (e == cudaErrorMemoryAllocation) { cudaGetLastError(); return fail(g, INGOT_INVALID, "out of device memory"); }
        return cuda_fail(g, e, "group_create");
    }
    gr->peer[rank] = static_cast<uint8_t *>(p);
    if ((e = preload_exchange_kernels()) != cudaSuccess) {      // a first step must not spend a peer's bounded wait loading modules
        cudaFree(p);
        delete gr;
        return cuda_fail(g, e, "group_create");
    }
    *out = gr;
    return INGOT_OK;
}

ingot_status ingot_group_connect(ingot_group *gr, const void *handles) {
    if (!gr || !handles) return INGOT_INVALID;
    ingot_gpu *g = gr->gpu;
    ingot_status st = enter(g);
    if (st) return st;
    for (uint32_t r = 0; r < gr->world; ++r) {
        if (r == gr->rank || gr->peer[r]) continue;
        void *p = nullptr;
        cudaIpcMemHandle_t h;
        memcpy(&h, static_cast<const uint8_t *>(handles) + 64u * r, 64);
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) { cudaGetLastError(); return fail(g, INGOT_DEVICE, std::string("group_connect: cannot map the window of rank ") + std::to_string(r) + ": " + cudaGetErrorString(e)); }
        gr->peer[r] = static_cast<uint8_t *>(p);
        gr->opened[r] = true;
    }
    return INGOT_OK;
}

ingot_status ingot_group_connect_local(ingot_group **groups, uint32_t world) {
    if (!groups || world == 0 || world > TP_MAX_RANKS) return INGOT_INVALID;
    for (uint32_t a = 0; a < world; ++a) {
        ingot_group *ga = groups[a];
        if (!ga || ga->world != world || ga->rank != a) return INGOT_INVALID;
        if (cudaSetDevice(ga->gpu->device) != cudaSuccess) return INGOT_DEVICE;
        for (uint32_t b = 0; b < world; ++b) {
            if (a == b) continue;
            if (groups[b]->gpu->device != ga->gpu->device) {
                cudaError_t e = cudaDeviceEnablePeerAccess(groups[b]->gpu->device, 0);
                if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
                else if (e != cudaSuccess) { cudaGetLastError(); return fail(ga->gpu, INGOT_DEVICE, std::string("group_connect_local: ") + cudaGetErrorString(e)); }
            }
            ga->peer[b] = groups[b]->peer[b];
        }
    }
    return INGOT_OK;
}

ingot_status ingot_group_window(const ingot_group *gr, uint32_t rank, void **base) {
    if (!gr || !base || rank >= gr->world || !gr->peer[rank]) return INGOT_INVALID;
    *base = gr->peer[rank];
    return INGOT_OK;
}

ingot_status ingot_group_step(ingot_group *gr) {
    if (!gr) return INGOT_INVALID;
    ingot_gpu *g = gr->gpu;
    ingot_status st = enter(g);
    if (st) return st;
    if (g->in_scope || g->chain_recording) return fail(g, INGOT_INVALID, "group_step: not inside an independent scope or a chain recording");
    return after_launch(g, launch_increment(gr->step_counter(), ctx_on(g, g->stream)), "group_step");
}

ingot_status ingot_group_wait(ingot_group *gr, uint32_t slot, float *whole, uint32_t n) {
    if (!gr || slot >= gr->slots) return INGOT_INVALID;
    ingot_gpu *g = gr->gpu;
    ingot_status st = enter(g);
    if (st) return st;
    const ingot_group::Shard &sh = gr->shard[slot];
    if (sh.rows == 0) return fail(g, INGOT_INVALID, "group_wait: no projection has signalled this slot yet");
    const uint8_t *base = gr->peer[gr->rank], *x = reinterpret_cast<const uint8_t *>(whole);
    if (!whole || x < base || x + (size_t)n * 4u > base + gr->window_bytes || (size_t)(x - base) > sh.off ||
        sh.off + (size_t)sh.rows * 4u > (size_t)(x - base) + (size_t)n * 4u)
        return fail(g, INGOT_INVALID, "group_wait: the vector must lie inside the window and contain this rank's rows of the slot");
    return after_launch(g, launch_collect_tagged(gr->twin(gr->rank, (size_t)(x - base)), whole, n, gr->step_counter(), gr->slots + 1u, slot + 1u,
                                                 ctx_on(g, g->stream)),
                        "group_wait");
}

ingot_status ingot_tp_signal_next(ingot_group *gr, uint32_t slot) {
    if (!gr || slot >= gr->slots) return INGOT_INVALID;
    gr->gpu->tp_signal_group = gr;
    gr->gpu->tp_signal_slot = slot;
    return INGOT_OK;
}

ingot_status ingot_tp_wait_next(ingot_group *gr, uint32_t slot_a, uint32_t slot_b) {
    if (!gr || slot_a >= gr->slots || (slot_b != TP_NO_SLOT && slot_b >= gr->slots)) return INGOT_INVALID;
    gr->gpu->tp_wait_group = gr;
    gr->gpu->tp_wait_slot[0] = slot_a;
    gr->gpu->tp_wait_slot[1] = slot_b;
    return INGOT_OK;
}

// ---- expert-parallel token exchange --------------------------------------------------------------

// The exchange areas (all inside the own window) as every rank sees them.
static ingot_status ep_link(ingot_group *gr, uint32_t slot, const ingot_ep_buffers *b, uint32_t cap, uint32_t hidden, uint32_t counter,
                            EpLink &l, const char *what) {
    ingot_gpu *g = gr->gpu;
    if (!b || !b->rx_rows || !b->rx_meta || !b->rx_ready || !b->ret_rows || !b->ret_ready || cap == 0 || hidden == 0)
        return fail(g, INGOT_INVALID, std::string(what) + ": bad arguments");
    const uint8_t *base = gr->peer[gr->rank];
    auto inside = [&](const void *p, size_t bytes, size_t align) {
        const uint8_t *x = static_cast<const uint8_t *>(p);
        return x >= base && x + bytes <= base + gr->window_bytes && ((uintptr_t)x % align) == 0;
    };
    const size_t places = (size_t)gr->world * cap;
    if (!inside(b->rx_rows, places * hidden * 4u, 16) || !inside(b->rx_meta, places * 4u, 4) || !inside(b->rx_ready, gr->world * 8u, 8) ||
        !inside(b->ret_rows, (size_t)cap * hidden * 4u, 16) || !inside(b->ret_ready, gr->world * 8u, 8))
        return fail(g, INGOT_INVALID, std::string(what) + ": the exchange areas must lie inside the group's window (rows 16-byte aligned)");
    l = {};
    for (uint32_t r = 0; r < gr->world; ++r) {
        if (!gr->peer[r]) return fail(g, INGOT_INVALID, std::string(what) + ": the group is not connected");
        auto at = [&](const void *p) { return gr->peer[r] + (static_cast<const uint8_t *>(p) - base); };
        l.rx_rows[r] = reinterpret_cast<float *>(at(b->rx_rows));
        l.rx_meta[r] = reinterpret_cast<uint32_t *>(at(b->rx_meta));
        l.rx_ready[r] = reinterpret_cast<uint64_t *>(at(b->rx_ready));
        l.ret_rows[r] = reinterpret_cast<float *>(at(b->ret_rows));
        l.ret_ready[r] = reinterpret_cast<uint64_t *>(at(b->ret_ready));
    }
    l.launch_count = reinterpret_cast<uint32_t *>(gr->peer[gr->rank] + gr->ctrl_off + 64u * (1u + counter));
    l.step = gr->step_counter();
    l.tag_mul = gr->slots + 1u;
    l.tag_add = slot + 1u;
    l.world = gr->world;
    l.rank = gr->rank;
    return INGOT_OK;
}

static ingot_status ep_enter(ingot_group *gr, uint32_t slot, const char *what) {
    if (!gr || slot >= gr->slots) return INGOT_INVALID;
    ingot_gpu *g = gr->gpu;
    ingot_status st = enter(g);
    if (st) return st;
    if (g->in_scope || g->chain_recording) return fail(g, INGOT_INVALID, std::string(what) + ": not inside an independent scope or a chain recording");
    return INGOT_OK;
}

ingot_status ingot_ep_dispatch(ingot_group *gr, uint32_t slot, const ingot_ep_buffers *bufs, const float *x, const uint32_t *ids,
                               uint32_t tokens, uint32_t top, uint32_t hidden, uint32_t cap, uint32_t experts_per_rank) {
    ingot_status st = ep_enter(gr, slot, "ep_dispatch");
    if (st) return st;
    ingot_gpu *g = gr->gpu;
    EpLink l;
    if ((st = ep_link(gr, slot, bufs, cap, hidden, 0, l, "ep_dispatch"))) return st;
    const uint64_t pairs = (uint64_t)tokens * top;
    if (!x || !ids || top == 0 || pairs > cap || pairs > EP_MAX_PAIRS || hidden % 4u || experts_per_rank == 0 || ((uintptr_t)x % 16u))
        return fail(g, INGOT_INVALID, "ep_dispatch: tokens x top must fit the capacity (at most 4096 pairs per rank); rows of 4 n floats, 16-byte aligned");
    return after_launch(g, launch_ep_dispatch(l, x, ids, (uint32_t)pairs, top, hidden, cap, experts_per_rank, ctx_on(g, g->stream)), "ep_dispatch");
}

ingot_status ingot_ep_receive(ingot_group *gr, uint32_t slot, const ingot_ep_buffers *bufs, uint32_t hidden, uint32_t cap, uint32_t *ids_out) {
    ingot_status st = ep_enter(gr, slot, "ep_receive");
    if (st) return st;
    ingot_gpu *g = gr->gpu;
    EpLink l;
    if ((st = ep_link(gr, slot, bufs, cap, hidden, 0, l, "ep_receive"))) return st;
    if (!ids_out) return fail(g, INGOT_INVALID, "ep_receive: null pointer");
    return after_launch(g, launch_ep_receive(l, cap, ids_out, ctx_on(g, g->stream)), "ep_receive");
}

ingot_status ingot_ep_return(ingot_group *gr, uint32_t slot, const ingot_ep_buffers *bufs, const float *rows, const uint32_t *inverse,
                             uint32_t hidden, uint32_t cap) {
    ingot_status st = ep_enter(gr, slot, "ep_return");
    if (st) return st;
    ingot_gpu *g = gr->gpu;
    EpLink l;
    if ((st = ep_link(gr, slot, bufs, cap, hidden, 1, l, "ep_return"))) return st;
    if (!rows || hidden % 4u || ((uintptr_t)rows % 16u)) return fail(g, INGOT_INVALID, "ep_return: rows of 4 n floats, 16-byte aligned");
    return after_launch(g, launch_ep_return(l, rows, inverse, cap, hidden, ctx_on(g, g->stream)), "ep_return");
}

ingot_status ingot_ep_combine(ingot_group *gr, uint32_t slot, const ingot_ep_buffers *bufs, const float *weights, uint32_t hidden,
                              uint32_t top, uint32_t tokens, uint32_t cap, float *y) {
    ingot_status st = ep_enter(gr, slot, "ep_combine");
    if (st) return st;
    ingot_gpu *g = gr->gpu;
    EpLink l;
    if ((st = ep_link(gr, slot, bufs, cap, hidden, 1, l, "ep_combine"))) return st;
    if (!weights || !y || hidden % 4u || (uint64_t)tokens * top > cap || ((uintptr_t)y % 16u))
        return fail(g, INGOT_INVALID, "ep_combine: bad arguments");
    return after_launch(g, launch_ep_combine(l, weights, hidden, top, tokens, y, ctx_on(g, g->stream)), "ep_combine");
}

void ingot_group_destroy(ingot_group *gr) {
    if (!gr) return;
    cudaSetDevice(gr->gpu->device);
    cudaStreamSynchronize(gr->gpu->stream);
    for (uint32_t r = 0; r < gr->world; ++r)
        if (gr->opened[r]) cudaIpcCloseMemHandle(gr->peer[r]);
    if (gr->peer[gr->rank]) cudaFree(gr->peer[gr->rank]);
    if (gr->gpu->tp_signal_group == gr) gr->gpu->tp_signal_group = nullptr;
    if (gr->gpu->tp_wait_group == gr) gr->gpu->tp_wait_group = nullptr;
    delete gr;
}

// ---- chains: a sequence of fused-norm projections as one persistent kernel ------------

ingot_status ingot_chain_begin(ingot_gpu *g) {
    ingot_status st = enter(g);
    if (st) return st;
    if (g->chain_recording) return fail(g, INGOT_INVALID, "already recording a chain");
    if (g->capturing || g->in_scope) return fail(g, INGOT_INVALID, "a chain cannot start inside a command recording or an independent scope");
    g->chain_recording = true;
    g->chain_calls.clear();
    return INGOT_OK;
}

ingot_status ingot_chain_end(ingot_gpu *g, ingot_chain **out) {
    if (!g || !out) return INGOT_INVALID;
    *out = nullptr;
    if (!g->chain_recording) return fail(g, INGOT_INVALID, "not recording a chain");
    g->chain_recording = false;
    std::vector<GemvCall> calls;
    calls.swap(g->chain_calls);
    ingot_status st = enter(g);
    if (st) return st;
    if (g->in_scope) return fail(g, INGOT_INVALID, "independent scope still open");
    ingot_chain *ch = new (std::nothrow) ingot_chain();
    if (!ch) return fail(g, INGOT_DEVICE, "out of host memory");
    ch->device = g->device;
    const char *why = "";
    cudaError_t e = chain_build(calls.data(), (uint32_t)calls.size(), ctx_on(g, g->stream), ch->launch, why);
    if (e != cudaSuccess) {
        delete ch;
        if (e == cudaErrorNotSupported || e == cudaErrorInvalidValue) {
            cudaGetLastError();
            return fail(g, e == cudaErrorNotSupported ? INGOT_UNSUPPORTED : INGOT_INVALID, std::string("chain: ") + why);
        }
        if (e == cudaErrorMemoryAllocation) { cudaGetLastError(); return fail(g, INGOT_INVALID, "out of device memory"); }
        return cuda_fail(g, e, "chain build");
    }
    *out = ch;
    return INGOT_OK;
}

ingot_status ingot_chain_submit(ingot_gpu *g, ingot_chain *ch) {
    ingot_status st = enter(g);
    if (st) return st;
    if (!ch || !ch->launch.ops_dev) return fail(g, INGOT_INVALID, "null chain");
    if (ch->device != g->device) return fail(g, INGOT_INVALID, "chain was built on another device");
    if (g->chain_recording || g->in_scope) return fail(g, INGOT_INVALID, "chain: cannot submit inside a chain recording or an independent scope");
    return after_launch(g, chain_launch(ch->launch, ctx_on(g, g->stream)), "chain");
}

ingot_status ingot_chain_info(const ingot_chain *ch, uint32_t *projections, uint32_t *waits, uint32_t *stages, uint32_t *stage_bytes) {
    if (!ch) return INGOT_INVALID;
    if (projections) *projections = ch->launch.n_ops;
    if (waits) *waits = ch->launch.waits;
    if (stages) *stages = ch->launch.slots;
    if (stage_bytes) *stage_bytes = ch->launch.slot_bytes;
    return INGOT_OK;
}

void ingot_chain_destroy(ingot_chain *ch) {
    if (!ch) return;
    cudaSetDevice(ch->device);
    chain_free(ch->launch);
    delete ch;
}

// ---- command recording --------------------------------------------------------

ingot_status ingot_command_begin(ingot_gpu *g) {
    ingot_status st = enter(g);
    if (st) return st;
    if (g->capturing) return fail(g, INGOT_INVALID, "already recording");
    cudaError_t e = cudaStreamBeginCapture(g->stream, cudaStreamCaptureModeThreadLocal);
    if (e != cudaSuccess) return cuda_fail(g, e, "begin capture");
    g->capturing = true;
    return INGOT_OK;
}

ingot_status ingot_command_end(ingot_gpu *g, ingot_graph **out) {
    if (!g || !out) return INGOT_INVALID;
    if (!g->capturing) return fail(g, INGOT_INVALID, "not recording");
    if (g->in_scope) return fail(g, INGOT_INVALID, "independent scope still open");
    g->capturing = false;
    ingot_graph *gr = new (std::nothrow) ingot_graph();
    if (!gr) return fail(g, INGOT_DEVICE, "out of host memory");
    cudaError_t e = cudaStreamEndCapture(g->stream, &gr->graph);
    if (e == cudaSuccess) e = cudaGraphInstantiate(&gr->exec, gr->graph, 0);
    if (e != cudaSuccess) {
        if (gr->graph) cudaGraphDestroy(gr->graph);
        delete gr;
        return cuda_fail(g, e, "end capture");
    }
    *out = gr;
    return INGOT_OK;
}

ingot_status ingot_command_submit(ingot_gpu *g, ingot_graph *gr) {
    ingot_status st = enter(g);
    if (st) return st;
    if (!gr || !gr->exec) return fail(g, INGOT_INVALID, "null graph");
    cudaError_t e = cudaGraphLaunch(gr->exec, g->stream);
    if (e != cudaSuccess) return cuda_fail(g, e, "graph launch");
    return INGOT_OK;
}

void ingot_command_destroy(ingot_graph *gr) {
    if (!gr) return;
    if (gr->exec) cudaGraphExecDestroy(gr->exec);
    if (gr->graph) cudaGraphDestroy(gr->graph);
    delete gr;
}

// ---- host-vector conveniences -------------------------------------------------

static ingot_status check_host_matrix(ingot_gpu *g, size_t data_bytes, uint64_t cols, uint64_t rows, uint64_t count,
                                      uint32_t kind, uint64_t stride) {
    uint32_t block, bytes;
    if (!geometry(kind, block, bytes)) return fail(g, INGOT_UNSUPPORTED, "GGML type " + std::to_string(kind) + " is unsupported");
    unsigned __int128 total = (unsigned __int128)stride * rows * count;
    if (cols == 0 || rows == 0 || count == 0 || cols % block || stride != cols / block * bytes ||
        total != (unsigned __int128)data_bytes || cols > 0xffffffffull || rows > 0xffffffffull ||
        count > 0xffffffffull || stride > 0xffffffffull)
        return fail(g, INGOT_INVALID, "invalid quantized matrix layout");
    return INGOT_OK;
}

ingot_status ingot_dequant_host(ingot_gpu *g, const void *data, size_t data_bytes, uint64_t cols, uint64_t rows,
                                uint64_t count, uint32_t kind, uint64_t stride, float *out) {
    ingot_status st = enter(g);
    if (st) return st;
    if ((st = check_host_matrix(g, data_bytes, cols, rows, count, kind, stride))) return st;
    if (!data || !out) return fail(g, INGOT_INVALID, "null pointer");
    void *w = nullptr, *y = nullptr;
    const size_t out_bytes = (size_t)cols * rows * count * sizeof(float);
    if ((st = ingot_buffer_alloc(g, data_bytes, &w))) return st;
    if ((st = ingot_buffer_alloc(g, out_bytes, &y))) { cudaFree(w); return st; }
    st = ingot_buffer_upload(g, w, data, data_bytes);
    if (!st) st = ingot_dequant_rows(g, w, (uint32_t)cols, rows * count, (uint32_t)stride, kind, static_cast<float *>(y));
    if (!st) st = ingot_buffer_read(g, out, y, out_bytes);
    if (!st) st = ingot_synchronize(g);
    cudaFree(w);
    cudaFree(y);
    return st;
}

ingot_status ingot_project_host(ingot_gpu *g, const void *data, size_t data_bytes, uint64_t cols, uint64_t rows,
                                uint64_t count, uint32_t kind, uint64_t stride, const float *input, size_t input_len,
                                float *out) {
    ingot_status st = enter(g);
    if (st) return st;
    if ((st = check_host_matrix(g, data_bytes, cols, rows, count, kind, stride))) return st;
    if (!data || !input || !out) return fail(g, INGOT_INVALID, "null pointer");
    bool finite = true;
    for (size_t i = 0; i < input_len; ++i) finite = finite && isfinite(input[i]);
    if (!finite || count != 1 || cols != input_len) return fail(g, INGOT_INVALID, "projection shape mismatch");
    void *w = nullptr, *x = nullptr, *y = nullptr;
    if ((st = ingot_buffer_alloc(g, data_bytes, &w))) return st;
    if ((st = ingot_buffer_alloc(g, cols * sizeof(float), &x))) { cudaFree(w); return st; }
    if ((st = ingot_buffer_alloc(g, rows * sizeof(float), &y))) { cudaFree(w); cudaFree(x); return st; }
    st = ingot_buffer_upload(g, w, data, data_bytes);
    if (!st) st = ingot_buffer_upload(g, x, input, cols * sizeof(float));
    if (!st) st = ingot_matmul(g, w, (uint32_t)cols, (uint32_t)rows, (uint32_t)stride, kind, 0, x, INGOT_KIND_F32, 1, static_cast<float *>(y));
    if (!st) st = ingot_buffer_read(g, out, y, rows * sizeof(float));
    if (!st) st = ingot_synchronize(g);
    cudaFree(w);
    cudaFree(x);
    cudaFree(y);
    if (!st)
        for (uint64_t i = 0; i < rows; ++i)
            if (!isfinite(out[i])) return fail(g, INGOT_INVALID, "output contains non-finite values");
    return st;
}

// Gpu::ffn (src/metal.rs:1634-1661) on device buffers: every stacked expert's SwiGLU FFN of the same input.
ingot_status ingot_ffn(ingot_gpu *g, const void *gate, const void *up, const void *down, uint32_t width, uint32_t inner,
                       uint32_t count, uint32_t kind, const float *x, float *scratch, const uint32_t *expert_ids, float *out) {
    ingot_status st = enter(g);
    if (st) return st;
    if (!gate || !up || !down || !x || !scratch || !expert_ids || !out || count == 0)
        return fail(g, INGOT_INVALID, "ffn: null pointer");
    uint32_t block, bytes;
    if (!geometry(kind, block, bytes)) return fail(g, INGOT_UNSUPPORTED, "GGML type " + std::to_string(kind) + " is unsupported");
    if (width % block || inner % block || (uint64_t)inner * count > 0xffffffffull) return fail(g, INGOT_INVALID, "FFN matrix shapes do not match");
    const uint32_t in_stride = width / block * bytes, down_stride = inner / block * bytes, n = inner * count;
    // gate and up of the stacked experts are one tall matrix each over the same input
    float *gv = scratch, *uv = scratch + n, *act = scratch + 2u * (size_t)n;
    if ((st = ingot_matmul(g, gate, width, n, in_stride, kind, 0, x, INGOT_KIND_F32, 1, gv))) return st;
    if ((st = ingot_matmul(g, up, width, n, in_stride, kind, 0, x, INGOT_KIND_F32, 1, uv))) return st;
    if ((st = ingot_activation(g, gv, uv, n, 0, act))) return st;
    // down: expert e multiplies its own slice of the activation (one input row per expert)
    return ingot_routed(g, down, inner, width, down_stride, kind, count, act, INGOT_KIND_F32, expert_ids, 1, 1, count, out);
}

// Gpu::moe (src/metal.rs:1663-1713) with host vectors: the FFNs of the selected experts (stacked in `routed`, one
// weight each) and of the shared expert, merged as sum_e w_e routed_e + sigmoid(shared_gate . x) shared.
ingot_status ingot_moe_host(ingot_gpu *g, const ingot_host_matrix routed[3], const ingot_host_matrix shared[3],
                            const ingot_host_matrix *shared_gate, const float *input, size_t width, const float *weights,
                            size_t n_weights, float *out) {
    ingot_status st = enter(g);
    if (st) return st;
    if (!routed || !shared || !shared_gate || !input || !weights || !out) return fail(g, INGOT_INVALID, "null pointer");
    const ingot_host_matrix *all[7] = {&routed[0], &routed[1], &routed[2], &shared[0], &shared[1], &shared[2], shared_gate};
    for (const ingot_host_matrix *m : all) {
        if (!m->data) return fail(g, INGOT_INVALID, "null pointer");
        if ((st = check_host_matrix(g, m->bytes, m->cols, m->rows, m->count, m->kind, m->stride))) return st;
    }
    bool finite = true;
    for (size_t i = 0; i < width; ++i) finite = finite && isfinite(input[i]);
    for (size_t i = 0; i < n_weights; ++i) finite = finite && isfinite(weights[i]);
    if (!finite || routed[0].cols != width || shared[0].cols != width || shared[0].count != 1 || routed[0].count != n_weights ||
        shared_gate->cols != width || shared_gate->rows != 1 || shared_gate->count != 1)
        return fail(g, INGOT_INVALID, "MoE input shape mismatch");
    for (const ingot_host_matrix *f : {routed, shared}) {
        if (f[1].cols != f[0].cols || f[1].rows != f[0].rows || f[1].count != f[0].count || f[1].kind != f[0].kind ||
            f[2].cols != f[0].rows || f[2].rows != f[0].cols || f[2].count != f[0].count || f[2].kind != f[0].kind)
            return fail(g, INGOT_INVALID, "FFN matrix shapes do not match");
    }
    const uint32_t top = (uint32_t)n_weights, w32 = (uint32_t)width;
    std::vector<void *> owned;
    auto dev = [&](size_t bytes, const void *host) -> void * {
        void *p = nullptr;
        if (st) return p;
        if ((st = ingot_buffer_alloc(g, bytes, &p))) return nullptr;
        owned.push_back(p);
        if (host) st = ingot_buffer_upload(g, p, host, bytes);
        return p;
    };
    void *wdev[7];
    for (int i = 0; i < 7; ++i) wdev[i] = dev(all[i]->bytes, all[i]->data);
    float *x = static_cast<float *>(dev(width * 4u, input));
    float *wts = static_cast<float *>(dev(n_weights * 4u, weights));
    std::vector<uint32_t> iota(top > 1u ? top : 1u);
    for (uint32_t i = 0; i < iota.size(); ++i) iota[i] = i;
    uint32_t *ids = static_cast<uint32_t *>(dev(iota.size() * 4u, iota.data()));
    const size_t n_r = (size_t)routed[0].rows * routed[0].count, n_s = (size_t)shared[0].rows;
    float *scr_r = static_cast<float *>(dev(3u * n_r * 4u, nullptr)), *scr_s = static_cast<float *>(dev(3u * n_s * 4u, nullptr));
    float *out_r = static_cast<float *>(dev((size_t)top * width * 4u, nullptr)), *out_s = static_cast<float *>(dev(width * 4u, nullptr));
    float *logit = static_cast<float *>(dev(4u, nullptr)), *y = static_cast<float *>(dev(width * 4u, nullptr));
    if (!st) st = ingot_ffn(g, wdev[0], wdev[1], wdev[2], w32, (uint32_t)routed[0].rows, top, routed[0].kind, x, scr_r, ids, out_r);
    if (!st) st = ingot_ffn(g, wdev[3], wdev[4], wdev[5], w32, (uint32_t)shared[0].rows, 1, shared[0].kind, x, scr_s, ids, out_s);
    if (!st) st = ingot_matmul(g, wdev[6], w32, 1, (uint32_t)shared_gate->stride, shared_gate->kind, 0, x, INGOT_KIND_F32, 1, logit);
    if (!st) st = ingot_merge(g, out_r, out_s, wts, logit, w32, top, y);
    if (!st) st = ingot_buffer_read(g, out, y, width * 4u);
    if (!st) st = ingot_synchronize(g);
    for (void *p : owned) cudaFree(p);
    if (!st)
        for (size_t i = 0; i < width; ++i)
            if (!isfinite(out[i])) return fail(g, INGOT_INVALID, "output contains non-finite values");
    return st;
}

}  // extern "C"
