// production_mul_mat_q4_k_decode_noalloc: the decode mul_mat for callers that must not allocate.
//
// Some hosts cannot call cudaMalloc once they are running: an inference server that has handed all device
// memory to its own pool, a process held to a fixed memory budget with allocations frozen after start-up,
// or a latency-critical loop for which the device-wide synchronisation inside cudaMalloc is itself the
// problem.  The regular entry points stage host-side activations and outputs through a device arena that
// they grow on demand; this variant stages them through a fixed array that is part of the library image
// instead, so nothing is allocated, now or later -- no cudaMalloc, no stream or event creation, no pinned
// host memory.  It runs on the legacy default stream and returns when the result is in place.
//
// Limits and rules:
//   * W must already be device memory (weights are too large to stage); X, Xq and Y may each be host or
//     device memory.  The host-side ones, plus a 256-byte control block, must fit WEFT_B200_NOALLOC_BYTES
//     (1 MiB); larger calls are refused with a message, nothing is truncated.
//   * The array is shared by every call in the process and keeps the previous call's bytes.  The control
//     word is cleared at the start of each call; every other byte the kernels read is written first.
//     Two calls that overlap on the GPU would race on it, so calls are serialised under a lock and each
//     call waits for its own work before returning.
//   * The first call on a device looks the array's device address up (cudaGetSymbolAddress).  Make that
//     first call outside any stream capture.
#include "../../include/weft_b200.h"

#include "common.cuh"
#include "kernels.h"

#include <cstdio>
#include <mutex>

using namespace weft;

namespace {

constexpr size_t kControlBytes = 256;
constexpr int kMaxDevices = 64;

// Scratch for staged arguments.  In host code this name is only a handle for cudaGetSymbolAddress: it is
// not a device address and must never be handed to a kernel or a memcpy directly.
static __device__ __align__(256) unsigned char g_noalloc_scratch[WEFT_B200_NOALLOC_BYTES];

std::mutex g_lock;
unsigned char *g_scratch_on[kMaxDevices];   // device address of the array, per device ordinal
int g_sm_count[kMaxDevices];
thread_local char t_message[256];

int refuse(const char *text) {
    snprintf(t_message, sizeof(t_message), "%s", text);
    return 1;
}

// 1: device (or managed) memory usable from `device`; 0: host memory; -1: device memory of another GPU
int where_is(const void *p, int device) {
    cudaPointerAttributes attr{};
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) { cudaGetLastError(); return 0; }
    if (attr.type == cudaMemoryTypeManaged) return 1;
    if (attr.type != cudaMemoryTypeDevice) return 0;
    return attr.device == device ? 1 : -1;
}

}  // namespace

extern "C" const char *weft_b200_noalloc_last_error(void) { return t_message; }

extern "C" int production_mul_mat_q4_k_decode_noalloc(const uint8_t *W, const float *X, uint8_t *Xq, float *Y,
                                                      size_t N, size_t K, size_t M) {
    std::lock_guard<std::mutex> guard(g_lock);
    t_message[0] = 0;
    if (K == 0 || K % 256) return refuse("K must be a positive multiple of 256 (complete Q4_K / Q8_K records)");
    if (N == 0 || M == 0) return 0;
    if (!W || !X || !Xq || !Y) return refuse("a required buffer is NULL");
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return refuse("no CUDA device is available; there is no CPU fallback");
    if (device < 0 || device >= kMaxDevices) return refuse("device ordinal out of range");
    if (!g_scratch_on[device]) {   // once per device, with that device current
        void *address = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&address, g_noalloc_scratch);
        if (e != cudaSuccess) { snprintf(t_message, sizeof(t_message), "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e)); return 1; }
        int sms = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (e != cudaSuccess || sms <= 0) return refuse("cannot read the multiprocessor count");
        g_scratch_on[device] = static_cast<unsigned char *>(address);
        g_sm_count[device] = sms;
    }
    if (where_is(W, device) != 1) return refuse("W must be device memory of the current device for the no-allocation entry point");
    // extents that could not fit the fixed scratch anyway are refused before any size is multiplied out
    constexpr size_t kMaxExtent = WEFT_B200_NOALLOC_BYTES / 4;
    const bool host_x = where_is(X, device) == 0, host_xq = where_is(Xq, device) == 0, host_y = where_is(Y, device) == 0;
    if (where_is(X, device) < 0 || where_is(Xq, device) < 0 || where_is(Y, device) < 0)
        return refuse("X, Xq and Y must be host memory or memory of the current device");
    if ((host_x || host_xq || host_y) && (M > kMaxExtent || K > kMaxExtent || N > kMaxExtent || M * K > kMaxExtent || (host_y && M * N > kMaxExtent))) {
        snprintf(t_message, sizeof(t_message), "this call needs more staging than the fixed scratch of %d bytes holds; use the regular entry point", WEFT_B200_NOALLOC_BYTES);
        return 1;
    }
    if ((reinterpret_cast<uintptr_t>(W) & 15u)) return refuse("W must be 16-byte aligned");

    // carve the staged arguments out of the fixed array
    unsigned char *base = g_scratch_on[device];
    size_t used = kControlBytes;
    auto place = [&](const void *user, size_t bytes, bool is_host, bool &staged) -> void * {
        staged = is_host;
        if (!staged) return const_cast<void *>(user);
        void *slot = base + used;
        used = (used + bytes + 255) & ~size_t(255);
        return slot;
    };
    const size_t x_bytes = M * K * sizeof(float), xq_bytes = M * (K / 256) * 292, y_bytes = M * N * sizeof(float);
    bool x_staged, xq_staged, y_staged;
    float *x = static_cast<float *>(place(X, x_bytes, host_x, x_staged));
    uint8_t *xq = static_cast<uint8_t *>(place(Xq, xq_bytes, host_xq, xq_staged));
    float *y = static_cast<float *>(place(Y, y_bytes, host_y, y_staged));
    if (used > WEFT_B200_NOALLOC_BYTES) {
        snprintf(t_message, sizeof(t_message), "this call needs %zu bytes of staging, the fixed scratch holds %d; use the regular entry point",
                 used, WEFT_B200_NOALLOC_BYTES);
        return 1;
    }
    if ((reinterpret_cast<uintptr_t>(x) & 15u) || (reinterpret_cast<uintptr_t>(xq) & 3u) || (reinterpret_cast<uintptr_t>(y) & 3u))
        return refuse("X must be 16-byte aligned, Xq and Y 4-byte aligned");

    cudaStream_t stream = 0;
    int *status = reinterpret_cast<int *>(base);
    cudaError_t e = cudaMemsetAsync(status, 0, kControlBytes, stream);            // the one thing that must start at zero
    if (e == cudaSuccess && x_staged) e = cudaMemcpyAsync(x, X, x_bytes, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) {
        GemvArgs args{F_Q4_K, W, xq, x, nullptr, nullptr, nullptr, y, (long long)N, (long long)K, (long long)M, (long long)N, status};
        e = launch_gemv(args, g_sm_count[device], stream);
    }
    int device_status = 0;
    if (e == cudaSuccess && xq_staged) e = cudaMemcpyAsync(Xq, xq, xq_bytes, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess && y_staged) e = cudaMemcpyAsync(Y, y, y_bytes, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(&device_status, status, sizeof(int), cudaMemcpyDeviceToHost, stream);
    // Always wait, also after a failed enqueue: copies already in the stream name the caller's host buffers and the
    // shared scratch, and neither may be touched again while they are in flight.
    const cudaError_t waited = cudaStreamSynchronize(stream);
    if (e == cudaSuccess) e = waited;
    if (e != cudaSuccess) { snprintf(t_message, sizeof(t_message), "CUDA call failed: %s", cudaGetErrorString(e)); return 1; }
    if (device_status != 0) return refuse("device-side failure: a bounded wait on an asynchronous copy ran out");
    return 0;
}
