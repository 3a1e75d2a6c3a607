// Shared host-side helpers for the parpy_b200 native library: error capture in
// the style of the reference runtime (entry points return 0 on success and a
// non-zero code otherwise; the text is fetched with parpy_get_error_message,
// python/parpy/native/parpy_cuda.h:22-25) and small device utilities.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstring>

enum : int32_t {
    PB_OK = 0,
    PB_ERR_ARGUMENT = 10001,   // rejected before any launch
    PB_ERR_UNSUPPORTED = 10002,
    PB_ERR_DEVICE_STATUS = 10003,
};

namespace pb {

// Last error text of the calling thread. Set by every failing entry point.
void set_error(const char *fmt, ...);
const char *last_error();

// Records a CUDA failure as the thread's error text and returns its code.
int32_t cuda_fail(cudaError_t err, const char *what);

#define PB_CUDA(expr)                                       \
    do {                                                    \
        cudaError_t pb_err__ = (expr);                      \
        if (pb_err__ != cudaSuccess) {                      \
            return ::pb::cuda_fail(pb_err__, #expr);        \
        }                                                   \
    } while (0)

#define PB_REQUIRE(cond, ...)                               \
    do {                                                    \
        if (!(cond)) {                                      \
            ::pb::set_error(__VA_ARGS__);                   \
            return PB_ERR_ARGUMENT;                         \
        }                                                   \
    } while (0)

// Per-device facts queried once.
struct DeviceInfo {
    int device = -1;
    int sm_count = 0;
    int cc_major = 0;
    int cc_minor = 0;
    size_t smem_optin = 0;
};
int32_t device_info(DeviceInfo *out);

// Grow-only device scratch owned by the library, one block per (device, stream,
// kind). Used for scheduling scratch and reduction partials; never for caller
// data. `zeroed_workspace` returns a block whose first `zero_bytes` are cleared
// (stream-ordered) before the caller's kernel runs.
int32_t workspace(size_t bytes, void **ptr, cudaStream_t stream = nullptr, int kind = 0);
int32_t zeroed_workspace(size_t zero_bytes, size_t extra_bytes, void **ptr, cudaStream_t stream);

#ifdef __CUDACC__
#define PB_HD __host__ __device__
#else
#define PB_HD
#endif
PB_HD inline long long ll_min(long long a, long long b) { return a < b ? a : b; }
PB_HD inline long long ll_max(long long a, long long b) { return a > b ? a : b; }

PB_HD inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- device helpers -------------------------------------------------------
#ifdef __CUDACC__
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float lg2_approx(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int i = 16; i > 0; i >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, i));
    return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
    for (int i = 16; i > 0; i >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, i));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int i = 16; i > 0; i >>= 1) v += __shfl_xor_sync(0xffffffffu, v, i);
    return v;
}
__device__ __forceinline__ float warp_prod(float v) {
#pragma unroll
    for (int i = 16; i > 0; i >>= 1) v *= __shfl_xor_sync(0xffffffffu, v, i);
    return v;
}
#endif

}  // namespace pb
