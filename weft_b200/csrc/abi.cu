// extern "C" surface of libweft_b200.so (declared in include/weft_b200.h).
//
// Host logic only: argument checks, host/device pointer handling, stream and status plumbing.
// All arithmetic happens in the kernels behind launch_*; there is no CPU fallback -- a missing or
// unusable GPU is an error.
#include "../../include/weft_b200.h"

#include "common.cuh"
#include "kernels.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <vector>

using namespace weft;

namespace {

thread_local char t_error[512] = "";

int fail(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof(t_error), fmt, ap);
    va_end(ap);
    return 1;
}

struct Resident { void *device; size_t bytes; };

struct State {
    std::recursive_mutex lock;
    bool ready = false;
    int device = -1;
    cudaDeviceProp prop{};
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;
    bool async = false;
    int *status_host = nullptr;   // mapped, pinned: the kernels write here only on failure
    int *status_dev = nullptr;
    unsigned long long launches = 0;
    std::map<uintptr_t, Resident> resident;   // keyed by host base address
    uint8_t *arena = nullptr;                 // staging for host-pointer arguments; grows, never shrinks
    size_t arena_bytes = 0;
};
State g;

#define CU(call)                                                                                   \
    do {                                                                                           \
        cudaError_t e_ = (call);                                                                   \
        if (e_ != cudaSuccess) return fail("%s failed: %s", #call, cudaGetErrorString(e_));        \
    } while (0)

int ensure_init(int device) {
    if (g.ready) {
        if (device >= 0 && device != g.device) return fail("weft_b200 is already bound to device %d", g.device);
        cudaSetDevice(g.device);
        return 0;
    }
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return fail("no CUDA device is available (%s); weft_b200 has no CPU fallback", cudaGetErrorString(e));
    if (device < 0) { if (cudaGetDevice(&device) != cudaSuccess) device = 0; }
    CU(cudaSetDevice(device));
    CU(cudaGetDeviceProperties(&g.prop, device));
    if (g.prop.major != 10)
        return fail("device %d (%s) is compute capability %d.%d; this library carries sm_100a code only",
                    device, g.prop.name, g.prop.major, g.prop.minor);
    CU(cudaStreamCreateWithFlags(&g.own_stream, cudaStreamNonBlocking));
    g.stream = g.own_stream;
    CU(cudaHostAlloc(reinterpret_cast<void **>(&g.status_host), sizeof(int), cudaHostAllocMapped));
    *g.status_host = 0;
    CU(cudaHostGetDevicePointer(reinterpret_cast<void **>(&g.status_dev), g.status_host, 0));
    g.device = device;
    g.ready = true;
    return 0;
}

int device_status() {
    const int s = *g.status_host;
    if (s == ST_OK) return 0;
    *g.status_host = 0;
    if (s & 0x40000000) return fail("device-side failure: tensor memory allocation returned base 0x%08x", (unsigned)(s & 0x3fffffff));
    return fail("device-side failure: %s", s == ST_WAIT_TIMEOUT ? "a bounded wait on an asynchronous copy or MMA ran out"
                                           : s == ST_TMEM_ALLOC ? "tensor memory allocation failed" : "unknown status");
}

// One argument of a call: where the caller's bytes live and where the kernel will find them.
struct Arg {
    const void *user = nullptr;
    void *dev = nullptr;
    void *mapped = nullptr;    // the user's buffer as the device sees it, when it is pinned and mapped host memory
    size_t bytes = 0;
    bool written = false, overflow = false;
};

// Host arguments up to this size in pinned, mapped memory move by a copy kernel instead of the copy engine.
constexpr size_t kKernelCopyMax = size_t(1) << 18;

// Host-pointer arguments are staged in one device arena owned by the library (256-byte aligned slices).
// An argument that does not fit gets a one-off allocation, and the arena is regrown after the call so
// that the same call fits next time.  Calls that stage anything always end with a stream synchronize,
// so the arena is free again when the next call starts.
class Call {
  public:
    ~Call() {
        for (Arg &a : args_)
            if (a.overflow && a.dev) { cudaStreamSynchronize(g.stream); cudaFree(a.dev); }
    }
    // Returns the device address for `ptr` (bytes long). read: copy in when host; written: copy back.
    // direct: a written host argument in pinned, mapped memory that the kernels only ever store to (never read back)
    // is handed to them as it is -- their stores go to the caller's buffer, no staging slice and no copy back.
    int map(const void *ptr, size_t bytes, bool read, bool written, void **out, bool direct = false) {
        *out = nullptr;
        direct_ = false;
        if (bytes == 0) { *out = const_cast<void *>(ptr); return 0; }
        if (!ptr) return fail("a required buffer is NULL");
        cudaPointerAttributes attr{};
        cudaError_t e = cudaPointerGetAttributes(&attr, ptr);
        if (e != cudaSuccess) { cudaGetLastError(); attr.type = cudaMemoryTypeUnregistered; }
        if (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) {
            if (attr.type == cudaMemoryTypeDevice && attr.device != g.device)
                return fail("buffer lives on device %d, the library is bound to device %d", attr.device, g.device);
            *out = const_cast<void *>(ptr);
            return 0;
        }
        any_host_ = true;
        if (!written) {   // registered resident weights: no copy
            const uintptr_t a = reinterpret_cast<uintptr_t>(ptr);
            auto it = g.resident.upper_bound(a);
            if (it != g.resident.begin()) {
                --it;
                if (a >= it->first && a + bytes <= it->first + it->second.bytes) {
                    *out = static_cast<uint8_t *>(it->second.device) + (a - it->first);
                    return 0;
                }
            }
        }
        Arg arg;
        arg.user = ptr; arg.bytes = bytes; arg.written = written;
        if (attr.type == cudaMemoryTypeHost && attr.devicePointer && bytes <= kKernelCopyMax) arg.mapped = attr.devicePointer;
        if (direct && written && !read && arg.mapped) { *out = arg.mapped; direct_ = true; return 0; }
        if (slice(arg)) return 1;
        if (read) {
            if (arg.mapped) CU(launch_copy_bytes(arg.dev, arg.mapped, bytes, g.stream));
            else CU(cudaMemcpyAsync(arg.dev, ptr, bytes, cudaMemcpyHostToDevice, g.stream));
        }
        *out = arg.dev;
        return 0;
    }
    // A read-only device argument at an address the kernels cannot load from (an Encoding with byte alignment
    // whose records hold 16-bit fields, at an odd address): move it to an aligned slice.
    int realign(void **dev, size_t bytes) {
        Arg arg;
        arg.bytes = bytes;
        if (slice(arg)) return 1;
        any_host_ = true;   // the slice is reused by the next call: end this one with a synchronize
        CU(cudaMemcpyAsync(arg.dev, *dev, bytes, cudaMemcpyDeviceToDevice, g.stream));
        *dev = arg.dev;
        return 0;
    }
    // Copy written host arguments back and decide whether to wait.
    int finish() {
        for (Arg &a : args_)
            if (a.written) {
                if (a.mapped) CU(launch_copy_bytes(a.mapped, a.dev, a.bytes, g.stream));
                else CU(cudaMemcpyAsync(const_cast<void *>(a.user), a.dev, a.bytes, cudaMemcpyDeviceToHost, g.stream));
            }
        if (any_host_ || !g.async) {
            CU(cudaStreamSynchronize(g.stream));
            if (wanted_ > g.arena_bytes) {   // make the next identical call fit
                if (g.arena) cudaFree(g.arena);
                g.arena = nullptr;
                g.arena_bytes = 0;
                const size_t want = (wanted_ + wanted_ / 4 + (size_t(1) << 16)) & ~size_t(255);
                if (cudaMalloc(reinterpret_cast<void **>(&g.arena), want) == cudaSuccess) g.arena_bytes = want;
                else cudaGetLastError();
            }
            return device_status();
        }
        return 0;
    }

    // true when the latest map() handed the caller's pinned buffer to the kernels as it is
    bool direct() const { return direct_; }

  private:
    bool direct_ = false;
    int slice(Arg &arg) {
        const size_t offset = (used_ + 255) & ~size_t(255);
        wanted_ = ((wanted_ + 255) & ~size_t(255)) + arg.bytes;
        if (offset + arg.bytes <= g.arena_bytes) {
            arg.dev = g.arena + offset;
            used_ = offset + arg.bytes;
        } else {
            CU(cudaMalloc(&arg.dev, arg.bytes));
            arg.overflow = true;
        }
        args_.push_back(arg);
        return 0;
    }
    std::vector<Arg> args_;
    size_t used_ = 0, wanted_ = 0;
    bool any_host_ = false;
};

size_t row_bytes(int fmt, size_t k) { return k / record_elements(fmt) * record_bytes(fmt); }

int check_k(int fmt, size_t k) {
    if (k % record_elements(fmt)) return fail("K = %zu does not contain complete %d-element records", k, record_elements(fmt));
    return 0;
}

int launched(cudaError_t e, const char *what, unsigned count = 1) {
    if (e != cudaSuccess) return fail("%s launch failed: %s", what, cudaGetErrorString(e));
    g.launches += count;
    return 0;
}

// bytes of the codebook a format's kernels take as an argument (int8[256][8], int8[512][8], int8[256][4]); the sign
// table is int8[128][8] for all three
size_t codebook_bytes(int fmt) { return fmt == F_IQ2_XXS ? 2048 : fmt == F_IQ2_XS ? 4096 : fmt == F_IQ3_XXS ? 1024 : fmt == F_IQ2_S ? 8192 : fmt == F_IQ3_S ? 2048 : (fmt == F_IQ1_S || fmt == F_IQ1_M) ? 16384 : 0; }
// IQ2_S and IQ3_S carry their sign bits in the record
bool has_sign_table(int fmt) { return fmt == F_IQ2_XXS || fmt == F_IQ2_XS || fmt == F_IQ3_XXS; }

int do_dequantize(int fmt, const void *W, const int8_t *grid, const int8_t *signs, const uint32_t *powers, float *Y, size_t N, size_t K) {
    std::lock_guard<std::recursive_mutex> guard(g.lock);
    if (ensure_init(-1)) return 1;
    if (check_k(fmt, K)) return 1;
    Call call;
    void *w, *y, *gr = nullptr, *sg = nullptr, *pw = nullptr;
    if (call.map(W, N * row_bytes(fmt, K), true, false, &w)) return 1;
    if ((fmt == F_Q6_K || fmt == F_IQ1_M) && (reinterpret_cast<uintptr_t>(w) & 1u) && call.realign(&w, N * row_bytes(fmt, K))) return 1;
    if (codebook_bytes(fmt) && (call.map(grid, codebook_bytes(fmt), true, false, &gr) || (has_sign_table(fmt) && call.map(signs, 1024, true, false, &sg)))) return 1;
    if (fmt == F_TQ1_0 && call.map(powers, 20, true, false, &pw)) return 1;
    if (fmt == F_IQ1_M && call.map(powers, 65536 * sizeof(float), true, false, &pw)) return 1;   // the caller's float[65536] table of f16 bit patterns
    if (call.map(Y, N * K * sizeof(float), false, true, &y)) return 1;
    if (launched(launch_dequantize(fmt, w, (const int8_t *)gr, (const int8_t *)sg, (const uint32_t *)pw, (float *)y,
                                   (long long)(N * K), g.prop.multiProcessorCount, g.stream), "row_dequantize"))
        return 1;
    return call.finish();
}

int do_quantize(int act, const float *X, uint8_t *Y, size_t M, size_t K) {
    std::lock_guard<std::recursive_mutex> guard(g.lock);
    if (ensure_init(-1)) return 1;
    if (check_k(act, K)) return 1;
    Call call;
    void *x, *y;
    if (call.map(X, M * K * sizeof(float), true, false, &x)) return 1;
    if (call.map(Y, M * row_bytes(act, K), false, true, &y)) return 1;
    if ((reinterpret_cast<uintptr_t>(y) & (act == F_Q8_K ? 3u : 1u)) || (reinterpret_cast<uintptr_t>(x) & 3u))
        return fail("activation buffers do not meet their Encoding alignment");
    if (launched(launch_quantize(act, (const float *)x, y, (long long)M, (long long)K, g.prop.multiProcessorCount, g.stream), "quantize"))
        return 1;
    return call.finish();
}

// mode 0: GEMV per activation row; mode 1: tensor-core contraction when the shape allows, else GEMV.
int do_mul_mat(int fmt, int mode, const void *W, const float *X, void *Xq, const int8_t *grid, const int8_t *signs,
               const uint32_t *powers, float *Y, size_t N, size_t K, size_t M, size_t ldy, unsigned flags, bool vec_dot_only,
               const GatherArgs *gather = nullptr) {
    std::lock_guard<std::recursive_mutex> guard(g.lock);
    if (ensure_init(-1)) return 1;
    const int act = activation_of(fmt);
    if (check_k(fmt, K) || check_k(act, K)) return 1;
    if (K == 0 || N == 0 || M == 0) return 0;
    if (ldy < N) return fail("Y row pitch %zu is smaller than N = %zu", ldy, N);
    if (fmt == F_Q4_K_I16 && N % 16 != 0) return fail("Q4K_I[16] holds whole cohorts of 16 rows; N = %zu", N);
    const bool have_xq = vec_dot_only || (flags & 1u);
    Call call;
    void *w, *x = nullptr, *xq, *y, *gr = nullptr, *sg = nullptr, *pw = nullptr;
    if (call.map(W, N * row_bytes(fmt, K), true, false, &w)) return 1;
    if ((fmt == F_Q6_K || fmt == F_IQ1_M) && (reinterpret_cast<uintptr_t>(w) & 1u) && call.realign(&w, N * row_bytes(fmt, K))) return 1;
    if (!have_xq && call.map(X, M * K * sizeof(float), true, false, &x)) return 1;
    // Decode quantizes X inside the GEMV (its first CTA stores the records, nobody loads them again), so a pinned Xq can
    // be written in place; a call that may take the tensor-core path or the separate quantize kernel reads Xq back.
    const bool may_contract = mode == 1 && M >= 32 && K % 256 == 0;
    const bool xq_in_place = !have_xq && !may_contract && K % 256 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
    if (call.map(Xq, M * row_bytes(act, K), have_xq, !have_xq, &xq, xq_in_place)) return 1;
    if (codebook_bytes(fmt) && (call.map(grid, codebook_bytes(fmt), true, false, &gr) || (has_sign_table(fmt) && call.map(signs, 1024, true, false, &sg)))) return 1;
    if (fmt == F_TQ1_0 && call.map(powers, 20, true, false, &pw)) return 1;
    if (fmt == F_IQ1_M && call.map(powers, 65536 * sizeof(float), true, false, &pw)) return 1;   // the caller's float[65536] table of f16 bit patterns
    // a host Y with a pitch is staged whole (pitch * M floats); device Y is written in place; a small pinned Y too
    const size_t y_floats = (M - 1) * ldy + N;
    if (call.map(Y, y_floats * sizeof(float), ldy != N, true, &y, ldy == N && gather == nullptr)) return 1;
    const bool y_on_host = call.direct();
    if ((reinterpret_cast<uintptr_t>(w) & (fmt == F_Q4_K_I16 ? 15u : 1u)) || (reinterpret_cast<uintptr_t>(xq) & (act == F_Q8_K ? 3u : 1u)) ||
        (reinterpret_cast<uintptr_t>(y) & 3u) || (x && (reinterpret_cast<uintptr_t>(x) & 3u)))
        return fail("a buffer does not meet its Encoding alignment");
    const int sms = g.prop.multiProcessorCount;
    const bool by_blocks = mode == 1 && prefill_blocks_supported(fmt, (long long)N, (long long)K, (long long)M, w, xq);
    const bool by_codebook = mode == 1 && gr && sg && prefill_codebook_supported(fmt, (long long)N, (long long)K, (long long)M, w, xq);
    const bool to_prefill = by_blocks || by_codebook || (mode == 1 && (prefill_supported(fmt, (long long)N, (long long)K, (long long)M, w, xq) ||
                                                                       prefill_pair_supported(fmt, (long long)N, (long long)K, (long long)M, w, xq)));
    // decode: the GEMV's own prologue quantizes X (one launch) when the fp32 rows allow 16-byte loads
    const bool fuse_quantize = !have_xq && !to_prefill && K % 256 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
    if (!have_xq && !fuse_quantize &&
        launched(launch_quantize(act, (const float *)x, xq, (long long)M, (long long)K, sms, g.stream), "activation quantize"))
        return 1;
    if (to_prefill) {
        PrefillArgs pa{fmt, w, xq, (const uint32_t *)pw, (float *)y, (long long)N, (long long)K, (long long)M, (long long)ldy, g.status_dev};
        const bool pair = prefill_pair_supported(fmt, (long long)N, (long long)K, (long long)M, w, xq);
        if (launched(by_codebook ? launch_prefill_codebook(pa, (const int8_t *)gr, (const int8_t *)sg, sms, g.stream) : by_blocks ? launch_prefill_blocks(pa, sms, g.stream) : pair ? launch_prefill_pair(pa, sms, g.stream) : launch_prefill(pa, sms, g.stream), "prefill mul_mat",
                     pair ? prefill_pair_launches(fmt) : 1)) return 1;   // the pair paths launch their plane kernel first
        if (gather && launched(launch_gather_push(*gather, (long long)M, (long long)N, (long long)ldy, g.status_dev, sms, g.stream), "peer all-gather")) return 1;
    } else {
        GemvArgs ga{fmt, w, xq, fuse_quantize ? (const float *)x : nullptr, (const int8_t *)gr, (const int8_t *)sg, (const uint32_t *)pw,
                    (float *)y, (long long)N, (long long)K, (long long)M, (long long)ldy, g.status_dev, y_on_host};
        const bool fused = gather && gemv_gathers(ga);
        if (fused) ga.gather = *gather;
        if (launched(launch_gemv(ga, sms, g.stream), "decode mul_mat")) return 1;
        if (gather && !fused && launched(launch_gather_push(*gather, (long long)M, (long long)N, (long long)ldy, g.status_dev, sms, g.stream), "peer all-gather")) return 1;
    }
    return call.finish();
}

}  // namespace

extern "C" {

const char *weft_b200_last_error(void) { return t_error; }

int weft_b200_init(int device) {
    std::lock_guard<std::recursive_mutex> guard(g.lock);
    return ensure_init(device);
}

int weft_b200_device_info(int *cc_major, int *cc_minor, int *sm_count, size_t *total_bytes, char *name, size_t name_len) {
    std::lock_guard<std::recursive_mutex> guard(g.lock);
    if (ensure_init(-1)) return 1;
    if (cc_major) *cc_major = g.prop.major;
    if (cc_minor) *cc_minor = g.prop.minor;
    if (sm_count) *sm_count = g.prop.multiProcessorCount;
    if (total_bytes) *total_bytes = g.prop.totalGlobalMem;
    if (name && name_len) { strncpy(name, g.prop.name, name_len - 1); name[name_len - 1] = 0; }
    return 0;
}

int weft_b200_set_stream(void *cuda_stream) {
    std::lock_guard<std::recursive_mutex> guard(g.lock);
    if (ensure_init(-1)) return 1;
    g.stream = cuda_stream ? static_cast<cudaStream_t>(cuda_stream) : g.own_stream;
    return 0;
}

int weft_b200_set_async(int enabled) {
    std::lock_guard<std::recursive_mutex> guard(g.lock);
    g.async = enabled != 0;
    return 0;
}

int weft_b200_synchronize(void) {
    std::lock_guard<std::recursive_mutex> guard(g.lock);
    if (ensure_init(-1)) return 1;
    CU(cudaStreamSynchronize(g.stream));
    return device_status();
}

unsigned long long weft_b200_launch_count(void) { return g.launches; }

int weft_b200_peek_status(void) { return g.status_host ? *g.status_host : 0; }

int weft_b200_weights_resident(const void *host, size_t bytes) {
    std::lock_guard<std::recursive_mutex> guard(g.lock);
    if (ensure_init(-1)) return 1;
    if (!host || !bytes) return fail("weights_resident needs a buffer");
    const uintptr_t a = reinterpret_cast<uintptr_t>(host);
    if (g.resident.count(a)) return fail("this host buffer is already resident");
    Resident r{nullptr, bytes};
    CU(cudaMalloc(&r.device, bytes));
    cudaError_t e = cudaMemcpy(r.device, host, bytes, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) { cudaFree(r.device); return fail("upload failed: %s", cudaGetErrorString(e)); }
    g.resident[a] = r;
    return 0;
}

int weft_b200_weights_release(const void *host) {
    std::lock_guard<std::recursive_mutex> guard(g.lock);
    auto it = g.resident.find(reinterpret_cast<uintptr_t>(host));
    if (it == g.resident.end()) return fail("this host buffer is not resident");
    cudaStreamSynchronize(g.stream);
    cudaFree(it->second.device);
    g.resident.erase(it);
    return 0;
}

// Tensor-core issue rate of this device: tera-operations per second of a bare tcgen05.mma loop on every SM.
int weft_b200_mma_peak(int mode, double *tera_ops) {
    std::lock_guard<std::recursive_mutex> guard(g.lock);
    if (ensure_init(-1)) return 1;
    if (mode < 0 || mode > 2 || !tera_ops) return fail("mode must be 0 (int8), 1 (int8, CTA pairs) or 2 (f16), and the result slot non-NULL");
    const int sms = g.prop.multiProcessorCount, iterations = 8192;
    unsigned long long *spans = nullptr;
    CU(cudaMalloc(reinterpret_cast<void **>(&spans), sizeof(unsigned long long) * sms));
    cudaError_t e = cudaMemsetAsync(spans, 0, sizeof(unsigned long long) * sms, g.stream);
    double ops = 0.0;
    for (int pass = 0; pass < 2 && e == cudaSuccess; ++pass)   // the first pass warms the clocks up
        e = measure_mma_peak(mode, iterations, sms, spans, g.status_dev, g.stream, &ops);
    std::vector<unsigned long long> host(sms, 0);
    if (e == cudaSuccess) e = cudaStreamSynchronize(g.stream);
    if (e == cudaSuccess) e = cudaMemcpy(host.data(), spans, sizeof(unsigned long long) * sms, cudaMemcpyDeviceToHost);
    cudaFree(spans);
    if (e != cudaSuccess) return fail("tensor-core peak measurement failed: %s", cudaGetErrorString(e));
    if (device_status()) return 1;
    unsigned long long slowest = 0;
    for (unsigned long long v : host) slowest = v > slowest ? v : slowest;
    if (!slowest) return fail("tensor-core peak measurement recorded no time");
    g.launches += 2;
    *tera_ops = ops / (double)slowest * 1e-3;    // operations per nanosecond = giga-ops; / 1e3 = tera
    return 0;
}

// ---- vec_dot
#define VEC_DOT(name, fmt, TABLE_PARAMS, GRID, SIGNS, POWERS)                                                          \
    int name(const uint8_t *W, const uint8_t *X TABLE_PARAMS, float *Y, size_t K) {                                   \
        return do_mul_mat(fmt, 0, W, nullptr, const_cast<uint8_t *>(X), GRID, SIGNS, POWERS, Y, 1, K, 1, 1, 0, true); \
    }                                                                                                                  \
    int name##_rows(const uint8_t *W, const uint8_t *X TABLE_PARAMS, float *Y, size_t N, size_t K) {                  \
        return do_mul_mat(fmt, 0, W, nullptr, const_cast<uint8_t *>(X), GRID, SIGNS, POWERS, Y, N, K, 1, N, 0, true); \
    }
#define NO_TABLES
#define IQ_TABLES , const int8_t *grid, const int8_t *signs
#define TQ_TABLES , const uint32_t *powers
VEC_DOT(quantized_vec_dot_q4_0_q8_0, F_Q4_0, NO_TABLES, nullptr, nullptr, nullptr)
VEC_DOT(quantized_vec_dot_q8_0_q8_0, F_Q8_0, NO_TABLES, nullptr, nullptr, nullptr)
VEC_DOT(quantized_vec_dot_q4_k_q8_k, F_Q4_K, NO_TABLES, nullptr, nullptr, nullptr)
VEC_DOT(quantized_vec_dot_q2_k_q8_k, F_Q2_K, NO_TABLES, nullptr, nullptr, nullptr)
VEC_DOT(quantized_vec_dot_q3_k_q8_k, F_Q3_K, NO_TABLES, nullptr, nullptr, nullptr)
VEC_DOT(quantized_vec_dot_q5_k_q8_k, F_Q5_K, NO_TABLES, nullptr, nullptr, nullptr)
VEC_DOT(quantized_vec_dot_q6_k_q8_k, F_Q6_K, NO_TABLES, nullptr, nullptr, nullptr)
VEC_DOT(quantized_vec_dot_iq2_xxs_q8_k, F_IQ2_XXS, IQ_TABLES, grid, signs, nullptr)
VEC_DOT(quantized_vec_dot_iq2_xs_q8_k, F_IQ2_XS, IQ_TABLES, grid, signs, nullptr)
VEC_DOT(quantized_vec_dot_iq3_xxs_q8_k, F_IQ3_XXS, IQ_TABLES, grid, signs, nullptr)
#define GRID_ONLY , const int8_t *grid
VEC_DOT(quantized_vec_dot_iq2_s_q8_k, F_IQ2_S, GRID_ONLY, grid, nullptr, nullptr)
VEC_DOT(quantized_vec_dot_iq3_s_q8_k, F_IQ3_S, GRID_ONLY, grid, nullptr, nullptr)
VEC_DOT(quantized_vec_dot_iq1_s_q8_k, F_IQ1_S, GRID_ONLY, grid, nullptr, nullptr)
// IQ1_M: the reference passes a float[65536] table of f16 bit patterns; it travels in the slot of the TQ1_0 powers
#define IQ1M_TABLES , const int8_t *grid, const float *f16_bits
VEC_DOT(quantized_vec_dot_iq1_m_q8_k, F_IQ1_M, IQ1M_TABLES, grid, nullptr, reinterpret_cast<const uint32_t *>(f16_bits))
VEC_DOT(quantized_vec_dot_iq1_m_q8_k_lane16, F_IQ1_M, IQ1M_TABLES, grid, nullptr, reinterpret_cast<const uint32_t *>(f16_bits))
VEC_DOT(quantized_vec_dot_tq1_0_q8_k, F_TQ1_0, TQ_TABLES, nullptr, nullptr, powers)
// The reference's second statement of the same dot product with sixteen-wide partial sums (a vector-length plan of
// its target; the integer sum per block, and so every result bit, is the same): examples/kernels/vec_dot/tq1_0_q8_k_lane16.py:9-54
VEC_DOT(quantized_vec_dot_tq1_0_q8_k_lane16, F_TQ1_0, TQ_TABLES, nullptr, nullptr, powers)

// ---- dequantize
#define DEQUANT(name, fmt, TABLE_PARAMS, GRID, SIGNS, POWERS)                                                          \
    int name(const uint8_t *W TABLE_PARAMS, float *Y, size_t K) { return do_dequantize(fmt, W, GRID, SIGNS, POWERS, Y, 1, K); } \
    int name##_rows(const uint8_t *W TABLE_PARAMS, float *Y, size_t N, size_t K) { return do_dequantize(fmt, W, GRID, SIGNS, POWERS, Y, N, K); }
DEQUANT(row_dequantize_q4_0, F_Q4_0, NO_TABLES, nullptr, nullptr, nullptr)
DEQUANT(row_dequantize_q8_0, F_Q8_0, NO_TABLES, nullptr, nullptr, nullptr)
DEQUANT(row_dequantize_q4_k, F_Q4_K, NO_TABLES, nullptr, nullptr, nullptr)
DEQUANT(row_dequantize_q2_k, F_Q2_K, NO_TABLES, nullptr, nullptr, nullptr)
DEQUANT(row_dequantize_q3_k, F_Q3_K, NO_TABLES, nullptr, nullptr, nullptr)
DEQUANT(row_dequantize_q5_k, F_Q5_K, NO_TABLES, nullptr, nullptr, nullptr)
DEQUANT(row_dequantize_q6_k, F_Q6_K, NO_TABLES, nullptr, nullptr, nullptr)
DEQUANT(row_dequantize_iq2_xxs, F_IQ2_XXS, IQ_TABLES, grid, signs, nullptr)
DEQUANT(row_dequantize_iq2_xs, F_IQ2_XS, IQ_TABLES, grid, signs, nullptr)
DEQUANT(row_dequantize_iq3_xxs, F_IQ3_XXS, IQ_TABLES, grid, signs, nullptr)
DEQUANT(row_dequantize_iq2_s, F_IQ2_S, GRID_ONLY, grid, nullptr, nullptr)
DEQUANT(row_dequantize_iq3_s, F_IQ3_S, GRID_ONLY, grid, nullptr, nullptr)
DEQUANT(row_dequantize_iq1_s, F_IQ1_S, GRID_ONLY, grid, nullptr, nullptr)
DEQUANT(row_dequantize_iq1_m, F_IQ1_M, IQ1M_TABLES, grid, nullptr, reinterpret_cast<const uint32_t *>(f16_bits))
DEQUANT(row_dequantize_tq1_0, F_TQ1_0, TQ_TABLES, nullptr, nullptr, powers)

// ---- quantize
int q8_0_quantize(const float *X, uint8_t *Y, size_t K) { return do_quantize(F_Q8_0, X, Y, 1, K); }
int q8_K_quantize(const float *X, uint8_t *Y, size_t K) { return do_quantize(F_Q8_K, X, Y, 1, K); }
int q8_1_quantize(const float *X, uint8_t *Y, size_t K) { return do_quantize(F_Q8_1, X, Y, 1, K); }
int q8_1_quantize_rows(const float *X, uint8_t *Y, size_t M, size_t K) { return do_quantize(F_Q8_1, X, Y, M, K); }
int q8_0_quantize_rows(const float *X, uint8_t *Y, size_t M, size_t K) { return do_quantize(F_Q8_0, X, Y, M, K); }
int q8_K_quantize_rows(const float *X, uint8_t *Y, size_t M, size_t K) { return do_quantize(F_Q8_K, X, Y, M, K); }

// ---- mul_mat
#define MUL_MAT(name, fmt, mode, TABLE_PARAMS, GRID, SIGNS, POWERS)                                                    \
    int name(const uint8_t *W, const float *X, uint8_t *Xq TABLE_PARAMS, float *Y, size_t N, size_t K, size_t M) {    \
        return do_mul_mat(fmt, mode, W, X, Xq, GRID, SIGNS, POWERS, Y, N, K, M, N, 0, false);                         \
    }
MUL_MAT(production_mul_mat_q4_0_decode, F_Q4_0, 0, NO_TABLES, nullptr, nullptr, nullptr)
MUL_MAT(production_mul_mat_q8_0_decode, F_Q8_0, 0, NO_TABLES, nullptr, nullptr, nullptr)
MUL_MAT(production_mul_mat_q4_k_decode, F_Q4_K, 0, NO_TABLES, nullptr, nullptr, nullptr)
MUL_MAT(production_mul_mat_q2_k_decode, F_Q2_K, 0, NO_TABLES, nullptr, nullptr, nullptr)
MUL_MAT(production_mul_mat_q3_k_decode, F_Q3_K, 0, NO_TABLES, nullptr, nullptr, nullptr)
MUL_MAT(production_mul_mat_q5_k_decode, F_Q5_K, 0, NO_TABLES, nullptr, nullptr, nullptr)
MUL_MAT(production_mul_mat_q6_k_decode, F_Q6_K, 0, NO_TABLES, nullptr, nullptr, nullptr)
MUL_MAT(production_mul_mat_iq2_xxs_decode, F_IQ2_XXS, 0, IQ_TABLES, grid, signs, nullptr)
MUL_MAT(production_mul_mat_tq1_0_decode, F_TQ1_0, 0, TQ_TABLES, nullptr, nullptr, powers)
// same functions under the names of the reference's alternative lowering plans (examples/kernels/mul_mat/
// tq1_0_lane16_decode.py:10-23, q3_k_predecoded_scales_decode.py:10-21, q3_k_predecoded_scales.py:10-61)
MUL_MAT(production_mul_mat_tq1_0_lane16_decode, F_TQ1_0, 0, TQ_TABLES, nullptr, nullptr, powers)
MUL_MAT(production_mul_mat_q3_k_predecoded_scales_decode, F_Q3_K, 0, NO_TABLES, nullptr, nullptr, nullptr)
MUL_MAT(production_mul_mat_q3_k_predecoded_scales, F_Q3_K, 1, NO_TABLES, nullptr, nullptr, nullptr)
MUL_MAT(production_mul_mat_q4_0, F_Q4_0, 1, NO_TABLES, nullptr, nullptr, nullptr)
MUL_MAT(production_mul_mat_q8_0, F_Q8_0, 1, NO_TABLES, nullptr, nullptr, nullptr)
MUL_MAT(production_mul_mat_q4_k_staged, F_Q4_K, 1, NO_TABLES, nullptr, nullptr, nullptr)
MUL_MAT(production_mul_mat_q2_k, F_Q2_K, 1, NO_TABLES, nullptr, nullptr, nullptr)
MUL_MAT(production_mul_mat_q3_k, F_Q3_K, 1, NO_TABLES, nullptr, nullptr, nullptr)
MUL_MAT(production_mul_mat_q5_k, F_Q5_K, 1, NO_TABLES, nullptr, nullptr, nullptr)
MUL_MAT(production_mul_mat_q6_k, F_Q6_K, 1, NO_TABLES, nullptr, nullptr, nullptr)
MUL_MAT(production_mul_mat_tq1_0, F_TQ1_0, 1, TQ_TABLES, nullptr, nullptr, powers)
MUL_MAT(production_mul_mat_iq2_xxs_staged, F_IQ2_XXS, 1, IQ_TABLES, grid, signs, nullptr)
MUL_MAT(production_mul_mat_iq2_xxs, F_IQ2_XXS, 1, IQ_TABLES, grid, signs, nullptr)
// IQ2_XS (examples/kernels/mul_mat/iq2_xs.py:27-33, iq2_xs_staged.py:30-36) and IQ3_XXS (iq3_xxs.py:11-17): the GEMV per
// token row at any token count
MUL_MAT(production_mul_mat_iq2_xs, F_IQ2_XS, 1, IQ_TABLES, grid, signs, nullptr)
MUL_MAT(production_mul_mat_iq2_xs_staged, F_IQ2_XS, 1, IQ_TABLES, grid, signs, nullptr)
MUL_MAT(production_mul_mat_iq3_xxs, F_IQ3_XXS, 1, IQ_TABLES, grid, signs, nullptr)
// IQ2_S (examples/kernels/mul_mat/iq2_s.py:10-16, iq2_s_staged.py:29-35) and IQ3_S (iq3_s.py:10-16): one table argument
MUL_MAT(production_mul_mat_iq2_s, F_IQ2_S, 1, GRID_ONLY, grid, nullptr, nullptr)
MUL_MAT(production_mul_mat_iq2_s_staged, F_IQ2_S, 1, GRID_ONLY, grid, nullptr, nullptr)
MUL_MAT(production_mul_mat_iq3_s, F_IQ3_S, 1, GRID_ONLY, grid, nullptr, nullptr)
// IQ1_S (examples/kernels/mul_mat/iq1_s.py:9-15, iq1_s_decode.py:10-16) and IQ1_M (iq1_m.py:10-17, iq1_m_decode.py:10-17,
// iq1_m_lane16_decode.py:10-17)
MUL_MAT(production_mul_mat_iq1_s, F_IQ1_S, 1, GRID_ONLY, grid, nullptr, nullptr)
MUL_MAT(production_mul_mat_iq1_s_decode, F_IQ1_S, 0, GRID_ONLY, grid, nullptr, nullptr)
MUL_MAT(production_mul_mat_iq1_m, F_IQ1_M, 1, IQ1M_TABLES, grid, nullptr, reinterpret_cast<const uint32_t *>(f16_bits))
MUL_MAT(production_mul_mat_iq1_m_decode, F_IQ1_M, 0, IQ1M_TABLES, grid, nullptr, reinterpret_cast<const uint32_t *>(f16_bits))
MUL_MAT(production_mul_mat_iq1_m_lane16_decode, F_IQ1_M, 0, IQ1M_TABLES, grid, nullptr, reinterpret_cast<const uint32_t *>(f16_bits))

// ---- persistent interleaved layout Q4K_I[16]: artifact functions and the kernels that consume it
static size_t q4ki_packed_size(size_t rows, size_t K) { return K % 256 == 0 && rows % 16 == 0 ? rows * (K / 256) * 144 : 0; }
static int q4ki_pack(const uint8_t *source, uint8_t *target, size_t rows, size_t K) {
    std::lock_guard<std::recursive_mutex> guard(g.lock);
    if (ensure_init(-1)) return 1;
    if (K % 256 != 0) return fail("K = %zu does not hold whole Q4_K records", K);
    if (rows % 16 != 0) return fail("Q4K_I[16] holds whole cohorts of 16 rows; rows = %zu", rows);
    if (rows == 0 || K == 0) return 0;
    Call call;
    void *src, *dst;
    const size_t bytes = q4ki_packed_size(rows, K);
    if (call.map(source, bytes, true, false, &src) || call.map(target, bytes, false, true, &dst)) return 1;
    if ((reinterpret_cast<uintptr_t>(src) & 1u) || (reinterpret_cast<uintptr_t>(dst) & 15u)) return fail("a buffer does not meet its Encoding alignment");
    if (launched(launch_interleave_q4k(src, dst, (long long)rows, (long long)K, g.prop.multiProcessorCount, g.stream), "Q4K_I[16] pack")) return 1;
    return call.finish();
}
size_t q4_k_q8_k_gemv_W_packed_size(size_t M, size_t K) { return q4ki_packed_size(M, K); }
int q4_k_q8_k_gemv_W_pack(const uint8_t *source, uint8_t *target, size_t M, size_t K) { return q4ki_pack(source, target, M, K); }
int q4_k_q8_k_gemv(const uint8_t *W, const uint8_t *X, float *Y, size_t M, size_t K) {
    return do_mul_mat(F_Q4_K_I16, 0, W, nullptr, const_cast<uint8_t *>(X), nullptr, nullptr, nullptr, Y, M, K, 1, M, 0, true);
}
// The reference's two other statements of this GEMV (four 16-bit partial groups per sub-block; a 32-bit contraction
// per sub-block) differ in the vector plan only: same layout, same integer sums, same float op tree
// (examples/kernels/gemv/q4_k_groups4.py:8-27, q4_k_contract.py:8-27; examples/repro/weft/q4_k_gemv_runtime.cpp:12-25).
#define Q4KI_GEMV_ALIAS(name)                                                                                          \
    size_t name##_W_packed_size(size_t M, size_t K) { return q4ki_packed_size(M, K); }                                \
    int name##_W_pack(const uint8_t *source, uint8_t *target, size_t M, size_t K) { return q4ki_pack(source, target, M, K); } \
    int name(const uint8_t *W, const uint8_t *X, float *Y, size_t M, size_t K) {                                       \
        return do_mul_mat(F_Q4_K_I16, 0, W, nullptr, const_cast<uint8_t *>(X), nullptr, nullptr, nullptr, Y, M, K, 1, M, 0, true); \
    }
Q4KI_GEMV_ALIAS(q4_k_q8_k_gemv_groups4)
Q4KI_GEMV_ALIAS(q4_k_q8_k_gemv_contract)
size_t production_mul_mat_q4_k_persistent_W_packed_size(size_t N, size_t K) { return q4ki_packed_size(N, K); }
int production_mul_mat_q4_k_persistent_W_pack(const uint8_t *source, uint8_t *target, size_t N, size_t K) { return q4ki_pack(source, target, N, K); }
int production_mul_mat_q4_k_persistent(const uint8_t *W, const float *X, uint8_t *Xq, float *Y, size_t M, size_t K, size_t N) {
    return do_mul_mat(F_Q4_K_I16, 0, W, X, Xq, nullptr, nullptr, nullptr, Y, N, K, M, N, 0, false);
}

// Steps i .. i + count - 1 of a chain as one grouped launch: same activations, same K, one activation row, Q4_K
// weights already on the device.  Returns -1 when the steps do not qualify (the caller then issues them one by one).
static int do_mul_mat_group(const weft_b200_mul_mat_step *steps, int count) {
    if (ensure_init(-1)) return 1;
    const weft_b200_mul_mat_step &first = steps[0];
    Call call;
    GemvArgs ga{};
    ga.fmt = F_Q4_K; ga.k = (long long)first.K; ga.m = 1; ga.segments = count; ga.status = g.status_dev;
    for (int i = 0; i < count; ++i) {
        void *w, *y;
        if (call.map(steps[i].W, steps[i].N * row_bytes(F_Q4_K, first.K), true, false, &w)) return 1;
        if (call.map(steps[i].Y, steps[i].N * sizeof(float), false, true, &y)) return 1;
        ga.seg_w[i] = w; ga.seg_y[i] = static_cast<float *>(y); ga.seg_rows[i] = (long long)steps[i].N;
        if (reinterpret_cast<uintptr_t>(y) & 3u) return fail("a buffer does not meet its Encoding alignment");
    }
    const bool have_xq = (first.flags & 1u) != 0;
    void *x = nullptr, *xq;
    if (!have_xq && call.map(first.X, first.K * sizeof(float), true, false, &x)) return 1;
    if (call.map(first.Xq, row_bytes(F_Q8_K, first.K), have_xq, !have_xq, &xq)) return 1;
    if ((reinterpret_cast<uintptr_t>(xq) & 3u) || (x && (reinterpret_cast<uintptr_t>(x) & 3u))) return fail("a buffer does not meet its Encoding alignment");
    const int sms = g.prop.multiProcessorCount;
    const bool fuse_quantize = !have_xq && (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
    ga.xq = xq;
    ga.x = fuse_quantize ? static_cast<const float *>(x) : nullptr;
    if (!gemv_q4k_groups(ga)) return -1;
    if (!have_xq && !fuse_quantize &&
        launched(launch_quantize(F_Q8_K, (const float *)x, xq, 1, (long long)first.K, sms, g.stream), "activation quantize"))
        return 1;
    if (launched(launch_gemv(ga, sms, g.stream), "grouped decode mul_mat")) return 1;
    return call.finish();
}

int weft_b200_mul_mat_chain(const weft_b200_mul_mat_step *steps, size_t count) {
    if (!steps && count) return fail("the step table is NULL");
    std::lock_guard<std::recursive_mutex> guard(g.lock);
    for (size_t i = 0; i < count; ++i) {
        const weft_b200_mul_mat_step &s = steps[i];
        // consecutive Q4_K steps on the same activations (the later ones marked as reusing Xq) go out as one launch
        size_t run = 1;
        if (s.format == F_Q4_K && s.M == 1 && s.N && s.K && s.K % 256 == 0)
            while (i + run < count && run < (size_t)GEMV_MAX_SEGMENTS && steps[i + run].format == F_Q4_K && steps[i + run].M == 1 &&
                   steps[i + run].K == s.K && steps[i + run].Xq == s.Xq && (steps[i + run].flags & 1u) && steps[i + run].N)
                ++run;
        if (run > 1) {
            const int grouped = do_mul_mat_group(steps + i, (int)run);
            if (grouped > 0) return 1;
            if (grouped == 0) { i += run - 1; continue; }
        }
        if (s.format != F_Q4_0 && s.format != F_Q8_0 && s.format != F_Q2_K && s.format != F_Q3_K && s.format != F_Q4_K && s.format != F_Q5_K &&
            s.format != F_Q6_K && s.format != F_IQ2_XXS && s.format != F_TQ1_0)  /* chains: the formats of the first version */
            return fail("step %zu: unknown weight format id %d", i, s.format);
        if (do_mul_mat(s.format, 0, s.W, s.X, s.Xq, s.grid, s.signs, s.powers, s.Y, s.N, s.K, s.M, s.N, s.flags, false)) return 1;
    }
    return 0;
}

// ---- peer memory (CUDA IPC) and the row-sharded mul_mat that gathers through it
int weft_b200_peer_alloc(size_t bytes, void **ptr, unsigned char *handle) {
    std::lock_guard<std::recursive_mutex> guard(g.lock);
    if (ensure_init(-1)) return 1;
    if (!ptr || !handle || !bytes) return fail("peer_alloc needs a size, a pointer slot and a 64-byte handle buffer");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    void *p = nullptr;
    CU(cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) { cudaFree(p); return fail("peer_alloc: %s", cudaGetErrorString(e)); }
    memcpy(handle, &h, 64);
    *ptr = p;
    return 0;
}

int weft_b200_peer_open(const unsigned char *handle, void **ptr) {
    std::lock_guard<std::recursive_mutex> guard(g.lock);
    if (ensure_init(-1)) return 1;
    if (!ptr || !handle) return fail("peer_open needs a handle and a pointer slot");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    CU(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return 0;
}

int weft_b200_peer_close(void *ptr) {
    std::lock_guard<std::recursive_mutex> guard(g.lock);
    if (!g.ready) return fail("weft_b200 is not initialised");
    cudaStreamSynchronize(g.stream);
    CU(cudaIpcCloseMemHandle(ptr));
    return 0;
}

int weft_b200_peer_free(void *ptr) {
    std::lock_guard<std::recursive_mutex> guard(g.lock);
    if (!g.ready) return fail("weft_b200 is not initialised");
    cudaStreamSynchronize(g.stream);
    CU(cudaFree(ptr));
    return 0;
}

int weft_b200_peer_read(void *host, const void *device, size_t bytes) {
    std::lock_guard<std::recursive_mutex> guard(g.lock);
    if (ensure_init(-1)) return 1;
    CU(cudaStreamSynchronize(g.stream));
    CU(cudaMemcpy(host, device, bytes, cudaMemcpyDeviceToHost));
    return device_status();
}

int weft_b200_mul_mat_shard_gather(int format, int mode, const uint8_t *W_local, const float *X, uint8_t *Xq,
                                   const int8_t *grid, const int8_t *signs, const uint32_t *powers,
                                   float *const *Y_ranks, int *const *sync_ranks, void *const *stage_ranks, int world, int rank,
                                   size_t n0, size_t N_local, size_t N, size_t K, size_t M, unsigned flags) {
    if (format != F_Q4_0 && format != F_Q8_0 && format != F_Q2_K && format != F_Q3_K && format != F_Q4_K && format != F_Q5_K &&
        format != F_Q6_K && format != F_IQ2_XXS && format != F_IQ2_XS && format != F_IQ3_XXS && format != F_IQ2_S && format != F_IQ3_S && format != F_IQ1_S && format != F_IQ1_M && format != F_TQ1_0 && format != F_Q4_K_I16)
        return fail("unknown weight format id %d", format);
    if (mode != 0 && mode != 1) return fail("mode must be 0 (decode) or 1 (prefill)");
    if (world < 2 || world > GATHER_MAX_RANKS || rank < 0 || rank >= world) return fail("world %d / rank %d out of range (2..%d ranks)", world, rank, GATHER_MAX_RANKS);
    if (!Y_ranks || !sync_ranks) return fail("the per-rank buffer tables are NULL");
    if (n0 + N_local > N) return fail("columns [%zu, %zu) exceed N = %zu", n0, n0 + N_local, N);
    if (!N_local || !K || !M) return fail("every rank must take part in the gather with a non-empty shard");
    GatherArgs ga{};
    ga.world = world;
    ga.rank = rank;
    ga.n0 = (long long)n0;
    ga.values = (long long)(M * N);
    ga.ll = stage_ranks != nullptr && (long long)(M * N) <= GATHER_LL_MAX_VALUES;
    for (int r = 0; r < world; ++r) {
        if (!Y_ranks[r] || !sync_ranks[r]) return fail("rank %d has no buffer", r);
        ga.y[r] = Y_ranks[r] + n0;
        ga.sync[r] = sync_ranks[r];
        if (ga.ll) {
            if (!stage_ranks[r] || (reinterpret_cast<uintptr_t>(stage_ranks[r]) & 7u)) return fail("rank %d has no 8-byte aligned staging area", r);
            ga.stage[r] = static_cast<uint2 *>(stage_ranks[r]);
        }
    }
    return do_mul_mat(format, mode, W_local, X, Xq, grid, signs, powers, ga.y[rank], N_local, K, M, N, flags, false, &ga);
}

int weft_b200_mul_mat_shard(int format, int mode, const uint8_t *W_local, const float *X, uint8_t *Xq,
                            const int8_t *grid, const int8_t *signs, const uint32_t *powers,
                            float *Y_columns, size_t N_local, size_t K, size_t M, size_t ldy, unsigned flags) {
    if (format != F_Q4_0 && format != F_Q8_0 && format != F_Q2_K && format != F_Q3_K && format != F_Q4_K && format != F_Q5_K && format != F_Q6_K && format != F_IQ2_XXS && format != F_IQ2_XS && format != F_IQ3_XXS && format != F_IQ2_S && format != F_IQ3_S && format != F_IQ1_S && format != F_IQ1_M && format != F_TQ1_0 && format != F_Q4_K_I16)
        return fail("unknown weight format id %d", format);
    if (mode != 0 && mode != 1) return fail("mode must be 0 (decode) or 1 (prefill)");
    return do_mul_mat(format, mode, W_local, X, Xq, grid, signs, powers, Y_columns, N_local, K, M, ldy, flags, false);
}

}  // extern "C"
