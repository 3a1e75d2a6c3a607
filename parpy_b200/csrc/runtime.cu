// Native runtime of the parpy_b200 library: device buffers, copies and
// synchronisation behind the seven symbols the reference's Python layer binds
// from its per-backend runtime library (python/parpy/runtime.py:11-26,
// python/parpy/native/parpy_cuda.cpp:3-39), plus the library-wide error text.
#include <cstdarg>
#include <map>
#include <mutex>

#include "../../include/parpy_b200.h"
#include "common.cuh"

namespace pb {

static thread_local char g_err[512] = "no error";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

const char *last_error() { return g_err; }

int32_t cuda_fail(cudaError_t err, const char *what) {
    set_error("%s (%s) in %s", cudaGetErrorString(err), cudaGetErrorName(err), what);
    cudaGetLastError();  // clear the sticky-free error slot like the reference's getter does
    return static_cast<int32_t>(err);
}

static std::mutex g_mu;
static constexpr int kMaxDevices = 64;
static DeviceInfo g_info[kMaxDevices];

int32_t device_info(DeviceInfo *out) {
    int dev = 0;
    PB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) {
        set_error("device ordinal %d out of range", dev);
        return PB_ERR_ARGUMENT;
    }
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceInfo &d = g_info[dev];
    if (d.device < 0) {
        cudaDeviceProp prop;
        PB_CUDA(cudaGetDeviceProperties(&prop, dev));
        d.sm_count = prop.multiProcessorCount;
        d.cc_major = prop.major;
        d.cc_minor = prop.minor;
        d.smem_optin = prop.sharedMemPerBlockOptin;
        d.device = dev;
    }
    *out = d;
    return PB_OK;
}

// Scratch blocks are keyed by (device, stream, kind) so that calls queued on
// different streams never share one. Blocks only grow and live until exit.
struct WsKey {
    int dev;
    cudaStream_t stream;
    int kind;
    bool operator<(const WsKey &o) const {
        if (dev != o.dev) return dev < o.dev;
        if (stream != o.stream) return stream < o.stream;
        return kind < o.kind;
    }
};
struct WsBlock {
    void *ptr = nullptr;
    size_t bytes = 0;
};
static std::map<WsKey, WsBlock> g_ws;

int32_t workspace(size_t bytes, void **ptr, cudaStream_t stream, int kind) {
    int dev = 0;
    PB_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(g_mu);
    WsBlock &b = g_ws[WsKey{dev, stream, kind}];
    if (b.bytes < bytes) {
        if (b.ptr) {
            // work already queued on this stream may still use the old block
            PB_CUDA(cudaStreamSynchronize(stream));
            PB_CUDA(cudaFree(b.ptr));
            b.ptr = nullptr;
            b.bytes = 0;
        }
        const size_t want = bytes < (size_t(1) << 20) ? (size_t(1) << 20) : bytes;
        PB_CUDA(cudaMalloc(&b.ptr, want));
        b.bytes = want;
    }
    *ptr = b.ptr;
    return PB_OK;
}

int32_t zeroed_workspace(size_t zero_bytes, size_t extra_bytes, void **ptr, cudaStream_t stream) {
    int32_t rc = workspace(zero_bytes + extra_bytes, ptr, stream, 1);
    if (rc) return rc;
    PB_CUDA(cudaMemsetAsync(*ptr, 0, zero_bytes, stream));
    return PB_OK;
}

}  // namespace pb

extern "C" {

void parpy_init(int64_t) {}

int32_t parpy_sync(void) {
    PB_CUDA(cudaDeviceSynchronize());
    return 0;
}

void *parpy_alloc_buffer(int64_t nbytes) {
    void *ptr = nullptr;
    if (nbytes < 0) {
        pb::set_error("parpy_alloc_buffer: negative size %lld", (long long)nbytes);
        return nullptr;
    }
    cudaError_t err = cudaMallocAsync(&ptr, static_cast<size_t>(nbytes), 0);
    if (err != cudaSuccess) {
        pb::cuda_fail(err, "cudaMallocAsync");
        return nullptr;
    }
    return ptr;
}

int32_t parpy_memcpy(void *dst, void *src, int64_t nbytes, int64_t kind) {
    cudaMemcpyKind k = kind == 0   ? cudaMemcpyHostToHost
                       : kind == 1 ? cudaMemcpyHostToDevice
                       : kind == 2 ? cudaMemcpyDeviceToHost
                                   : cudaMemcpyDeviceToDevice;
    PB_CUDA(cudaMemcpyAsync(dst, src, static_cast<size_t>(nbytes), k, 0));
    return 0;
}

int32_t parpy_memset(void *ptr, int64_t nbytes, int8_t value) {
    PB_CUDA(cudaMemsetAsync(ptr, value, static_cast<size_t>(nbytes), 0));
    return 0;
}

int32_t parpy_free_buffer(void *ptr) {
    PB_CUDA(cudaFreeAsync(ptr, 0));
    return 0;
}

const char *parpy_get_error_message(void) { return pb::last_error(); }

int32_t parpy_b200_device_summary(int32_t *sm_count, int32_t *cc_major, int32_t *cc_minor) {
    pb::DeviceInfo d;
    int32_t rc = pb::device_info(&d);
    if (rc != 0) return rc;
    if (sm_count) *sm_count = d.sm_count;
    if (cc_major) *cc_major = d.cc_major;
    if (cc_minor) *cc_minor = d.cc_minor;
    return 0;
}

}  // extern "C"
