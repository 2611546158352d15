// A quantised matrix-vector product for callers that must not allocate.
//
// Who cannot allocate: a decode loop that runs after its host application has already
// handed every remaining byte of HBM to its own pool (an inference server that sizes
// its KV cache to "whatever is left" at start-up leaves nothing for a later cudaMalloc),
// and latency-critical loops that cannot afford the implicit device-wide
// synchronisation and the failure modes of cudaMalloc / cudaFree in the middle of a
// token step.  The regular entry points need a handle (ingot_gpu_create allocates a
// status word and a workspace); this one needs nothing but the library itself: the
// scratch the tensor-core GEMV uses for its packed activations (written when x is not
// 16-byte aligned; an aligned x is packed in shared memory inside the kernel), and the word
// its kernels report errors through, are file-scope __device__ arrays that every GPU
// loading the library carries until the process exits.
#include "../../include/ingot_cuda.h"

#include <stdio.h>

#include <mutex>

#include "gemv_core.cuh"
#include "kernels.h"

using namespace ingot;

namespace {

// Largest row length served: 16384 columns (packed: 4.25 bytes per column + 16).
constexpr uint32_t STATIC_MAX_COLS = 16384;
constexpr size_t STATIC_SCRATCH_BYTES = (size_t)STATIC_MAX_COLS * 4u + STATIC_MAX_COLS / 4u + 16u;

static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];
static __device__ __align__(256) int g_static_status[16];

struct DeviceState {
    bool ready;
    void *scratch;      // device address of g_static_scratch on this device
    int *status;        // device address of g_static_status on this device
    uint32_t sm_count;
};
constexpr int MAX_DEVICES = 64;
DeviceState g_state[MAX_DEVICES];
std::mutex g_setup_lock;          // first calls from several host threads: one of them fills a device's entry
thread_local char g_error[256] = "";

ingot_status fail(ingot_status code, const char *msg) {
    snprintf(g_error, sizeof g_error, "%s", msg);
    return code;
}

// In host code the array names are host-side stand-ins, not device addresses: the
// addresses kernels can use come from cudaGetSymbolAddress, once per device, with
// that device current.
ingot_status setup(int device, DeviceState **out) {
    if (device < 0 || device >= MAX_DEVICES) return fail(INGOT_DEVICE, "device ordinal out of range");
    std::lock_guard<std::mutex> guard(g_setup_lock);
    DeviceState &s = g_state[device];
    if (!s.ready) {
        void *scratch = nullptr, *status = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&scratch, g_static_scratch);
        if (e == cudaSuccess) e = cudaGetSymbolAddress(&status, g_static_status);
        int sms = 0, major = 0;
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
        if (e != cudaSuccess) {
            snprintf(g_error, sizeof g_error, "static scratch set-up failed: %s", cudaGetErrorString(e));
            return INGOT_DEVICE;
        }
        if (major != 10) return fail(INGOT_DEVICE, "the kernels are built for sm_100 devices only");
        s.scratch = scratch;
        s.status = static_cast<int *>(status);
        s.sm_count = (uint32_t)sms;
        s.ready = true;
    }
    *out = &s;
    return INGOT_OK;
}

}  // namespace

extern "C" {

const char *ingot_matvec_static_error(void) { return g_error; }

ingot_status ingot_matvec_static(const void *w, uint32_t cols, uint32_t rows, uint32_t stride, uint32_t kind,
                                 uint32_t expert, const float *x, float *y, void *cuda_stream, int32_t wait) {
    g_error[0] = 0;
    uint32_t block, bytes;
    if (!geometry(kind, block, bytes)) return fail(INGOT_UNSUPPORTED, "GGML type is unsupported");
    if (block == 1) return fail(INGOT_UNSUPPORTED, "static-scratch GEMV serves the block-quantised types (2, 8, 12, 14)");
    if (!w || !x || !y || cols == 0 || rows == 0 || cols % block || stride != cols / block * bytes)
        return fail(INGOT_INVALID, "invalid quantized matrix layout");
    if (cols > STATIC_MAX_COLS) {
        snprintf(g_error, sizeof g_error, "cols = %u exceeds the static scratch (at most %u columns)", cols, STATIC_MAX_COLS);
        return INGOT_INVALID;
    }
    if (cols % 64u || stride % 16u || ((uintptr_t)w % 16u) || ((uintptr_t)x % 4u))
        return fail(INGOT_UNSUPPORTED, "static-scratch GEMV needs cols % 64 == 0 and 16-byte aligned rows");
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return fail(INGOT_DEVICE, "no current CUDA device");
    DeviceState *s = nullptr;
    ingot_status st = setup(device, &s);
    if (st) return st;

    LaunchCtx ctx = {};
    ctx.stream = static_cast<cudaStream_t>(cuda_stream);
    ctx.status = s->status;
    ctx.sm_count = s->sm_count;
    ctx.pdl = false;
    // an x that is 16-byte aligned is turned into the kernel's operand form inside the kernel (shared
    // memory only); any other x (4-byte aligned) is packed into the static array by a first small launch
    ctx.workspace = s->scratch;
    ctx.workspace_bytes = STATIC_SCRATCH_BYTES;
    GemvCall c = {};
    c.w[0] = static_cast<const uint8_t *>(w);
    c.x = x; c.y = y; c.cols = cols; c.rows = rows; c.stride = stride; c.kind = kind;
    c.expert = expert; c.count = 1; c.nmat = 1;
    cudaError_t e = cudaSuccess;
    if (!try_launch_gemv_mma(c, ctx, e)) return fail(INGOT_UNSUPPORTED, "shape not served by the static-scratch GEMV");
    if (e != cudaSuccess) {
        snprintf(g_error, sizeof g_error, "launch failed: %s", cudaGetErrorString(e));
        return INGOT_DEVICE;
    }
    if (!wait) return INGOT_OK;
    int code = 0;
    e = cudaMemcpyAsync(&code, s->status, sizeof(int), cudaMemcpyDeviceToHost, ctx.stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx.stream);
    if (e != cudaSuccess) {
        snprintf(g_error, sizeof g_error, "wait failed: %s", cudaGetErrorString(e));
        return INGOT_DEVICE;
    }
    if (code != KERNEL_OK) {
        cudaMemsetAsync(s->status, 0, sizeof(int), ctx.stream);      // the word is shared: clear it for the next call
        cudaStreamSynchronize(ctx.stream);
        return fail(INGOT_TIMEOUT, "a bounded device-side wait ran out");
    }
    return INGOT_OK;
}

}  // extern "C"
