// Device-side preparation of the HMM inputs, replacing the host loops of the
// reference's loader (benchmarks/forward.py:20-87): log of the probability
// tables, the base-reversal permutation of the emission columns (:29-38), the
// [4,K] -> [K,4] transpose of the transition table (:51), the initial
// distribution (:20-27) and the padded int8 observation matrix (:74-79).
#include <algorithm>

#include "../../include/parpy_b200.h"
#include "common.cuh"

namespace {

// Reverses the k base-4 digits of i (benchmarks/forward.py:29-30).
__device__ __forceinline__ long long reverse_base4(long long i, int k) {
    long long r = 0;
    for (int x = 0; x < k; ++x) {
        r = (r << 2) | (i & 3);
        i >>= 2;
    }
    return r;
}

// The reference takes logs in the file's dtype and then stores float32.
template <typename T>
__device__ __forceinline__ float log_as_stored(T p);
template <>
__device__ __forceinline__ float log_as_stored<float>(float p) { return logf(p); }
template <>
__device__ __forceinline__ float log_as_stored<double>(double p) { return (float)log(p); }

template <typename T>
__global__ void prepare_tables(const T *__restrict__ obs, const T *__restrict__ trans,
                               const T *__restrict__ dur, int k, long long K, long long n_obs,
                               float *__restrict__ output_prob, float *__restrict__ trans1,
                               float *__restrict__ trans2, float *__restrict__ initial_prob) {
    const long long total = n_obs * K;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const long long j = idx / K, i = idx % K;
        output_prob[idx] = log_as_stored<T>(obs[j * K + reverse_base4(i, k)]);   // log(0) = -inf
    }
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < 4 * K; idx += stride) {
        const long long s = idx >> 2, c = idx & 3;
        trans1[idx] = log_as_stored<T>(trans[c * K + s]);
    }
    const float init0 = (float)log(1.0 / (double)K);
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < 16 * K; idx += stride)
        initial_prob[idx] = idx < K ? init0 : -INFINITY;
    if (blockIdx.x == 0 && threadIdx.x < 16) trans2[threadIdx.x] = log_as_stored<T>(dur[threadIdx.x]);
}

__global__ void pad_signals(const int16_t *__restrict__ flat, const int64_t *__restrict__ offsets,
                            long long B, long long maxlen, int8_t *__restrict__ data,
                            int64_t *__restrict__ lens) {
    const long long b = blockIdx.y;
    const long long start = offsets[b], len = offsets[b + 1] - offsets[b];
    if (blockIdx.x == 0 && threadIdx.x == 0) lens[b] = len;
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < maxlen; t += (long long)gridDim.x * blockDim.x)
        data[b * maxlen + t] = t < len ? (int8_t)flat[start + t] : (int8_t)0;
}

}  // namespace

extern "C" {

int32_t parpy_b200_hmm_prepare_tables(const void *obs_prob, const void *trans_prob, const void *dur_prob,
                                      int32_t is_f64, int32_t k, int64_t n_obs, float *output_prob,
                                      float *trans1, float *trans2, float *initial_prob, void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    PB_REQUIRE(k >= 1 && k <= 12, "hmm_prepare_tables: k=%d out of range", k);
    PB_REQUIRE(n_obs >= 1, "hmm_prepare_tables: n_obs must be positive");
    PB_REQUIRE(obs_prob && trans_prob && dur_prob && output_prob && trans1 && trans2 && initial_prob,
               "hmm_prepare_tables: null pointer");
    const long long K = 1LL << (2 * k);
    pb::DeviceInfo dev;
    int32_t rc = pb::device_info(&dev);
    if (rc) return rc;
    const unsigned grid = (unsigned)std::min<long long>((n_obs * K + 255) / 256, 8LL * dev.sm_count);
    if (is_f64)
        prepare_tables<double><<<grid, 256, 0, stream>>>(
            static_cast<const double *>(obs_prob), static_cast<const double *>(trans_prob),
            static_cast<const double *>(dur_prob), k, K, n_obs, output_prob, trans1, trans2, initial_prob);
    else
        prepare_tables<float><<<grid, 256, 0, stream>>>(
            static_cast<const float *>(obs_prob), static_cast<const float *>(trans_prob),
            static_cast<const float *>(dur_prob), k, K, n_obs, output_prob, trans1, trans2, initial_prob);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

int32_t parpy_b200_hmm_pad_signals(const int16_t *flat, const int64_t *offsets, int64_t num_signals,
                                   int64_t maxlen, int8_t *data, int64_t *lens, void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    PB_REQUIRE(num_signals >= 0 && maxlen >= 1, "hmm_pad_signals: bad sizes");
    if (num_signals == 0) return PB_OK;
    PB_REQUIRE(flat && offsets && data && lens, "hmm_pad_signals: null pointer");
    PB_REQUIRE(num_signals <= 65535, "hmm_pad_signals: at most 65535 signals per call");
    dim3 grid((unsigned)std::min<long long>((maxlen + 255) / 256, 64), (unsigned)num_signals, 1);
    pad_signals<<<grid, 256, 0, stream>>>(flat, offsets, num_signals, maxlen, data, lens);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

}  // extern "C"
