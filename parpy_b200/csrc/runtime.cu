// Native runtime of the parpy_b200 library: device buffers, copies and
// synchronisation behind the seven symbols the reference's Python layer binds
// from its per-backend runtime library (python/parpy/runtime.py:11-26,
// python/parpy/native/parpy_cuda.cpp:3-39), plus the library-wide error text.
#include <cstdarg>
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
static void *g_ws[kMaxDevices];
static size_t g_ws_bytes[kMaxDevices];

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

int32_t workspace(size_t bytes, void **ptr) {
    int dev = 0;
    PB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) {
        set_error("device ordinal %d out of range", dev);
        return PB_ERR_ARGUMENT;
    }
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_ws_bytes[dev] < bytes) {
        // Work already queued against the old block must finish before it goes.
        if (g_ws[dev]) {
            PB_CUDA(cudaDeviceSynchronize());
            PB_CUDA(cudaFree(g_ws[dev]));
            g_ws[dev] = nullptr;
            g_ws_bytes[dev] = 0;
        }
        size_t want = bytes < (size_t(1) << 20) ? (size_t(1) << 20) : bytes;
        PB_CUDA(cudaMalloc(&g_ws[dev], want));
        g_ws_bytes[dev] = want;
    }
    *ptr = g_ws[dev];
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
