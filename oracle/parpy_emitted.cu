/*
 * The CUDA program ParPy's compiler emits for benchmarks/forward.py `forward_kernel`
 * with p = {'inst': threads(B), 'state': threads(nthreads)}, nthreads > 1024 —
 * written out by hand from the code-generation rules, because the compiler itself
 * (a Rust cdylib) cannot be built where there is no cargo.
 *
 * TEST AND MEASUREMENT INFRASTRUCTURE ONLY: the "ParPy-generated CUDA" arm of the
 * benchmark and a cross-check in the GPU tests. Nothing in the shipped package
 * calls it.
 *
 * What the rules give (citations into the reference checkout):
 *  - one kernel per outermost parallel loop; the innermost parallel loop ('state',
 *    nthreads > tpb = 1024) maps to blockIdx.x * 1024 + threadIdx.x with a grid-stride
 *    loop `for (s = idx; s < N; s += nthreads)`, the outer one ('inst') to blockIdx.y:
 *    grid (nthreads / 1024, B, 1) x (1024, 1, 1), __launch_bounds__(1024)
 *    (src/gpu/par.rs:256-296, src/gpu/codegen.rs:141-173,377-414);
 *  - a parallel loop that needs more than one block inside a sequential loop forces
 *    the sequential loop (t = 1 .. maxlen-1) out to the host: one launch per time step,
 *    each followed by cudaGetLastError (src/gpu/inter_block.rs:466-563,1070-1116,
 *    src/cuda/error.rs:56-73);
 *  - a reduction over more than one block becomes two kernels: per-block partials into
 *    a cudaMallocAsync temporary, then one block that reduces the partials
 *    (src/gpu/inter_block.rs:150-293,380-433); locals that cross kernels (maxp, psum)
 *    live in cudaMallocAsync temporaries freed with cudaFreeAsync (:999-1053);
 *  - block reduce = per-thread accumulate, __shfl_xor_sync butterfly, __shared__
 *    stemp[32] exchange, second butterfly (src/gpu/reduce.rs:401-435,
 *    src/cuda/reduce.rs:7-56);
 *  - fp32 exp/log print as __expf/__logf, max as fmaxf, inf as HUGE_VALF
 *    (src/cuda/pprint.rs:71-82,185-198); index arithmetic is int64 except the explicit
 *    int32 casts of the source; shapes and 0-d arguments are compile-time constants
 *    (src/py/inline_const.rs:97-148) — here the state-space size is a template
 *    parameter so that every // and % is by a constant, the other scalars are kernel
 *    parameters;
 *  - everything runs on stream 0 (src/cuda/pprint.rs:348-355).
 * The benchmark's wrapper zero-fills result, alpha1 and alpha2 on every call inside the
 * timed region (benchmarks/forward.py:189-198); `zero_fill` reproduces that.
 */
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace {

constexpr int kTpb = 1024;

struct Hmm {
    float gamma;
    const float *initial_prob;
    const float *output_prob;
    float synthetic_248;
    const float *trans1;
    const float *trans2;
};
struct Seqs {
    const int8_t *data;
    const int64_t *lens;
    int64_t maxlen;
    int64_t num_instances;
};

/* benchmarks/forward.py:94-101 */
template <int64_t N>
__global__ void __launch_bounds__(kTpb) forward_kernel_init(Hmm hmm, Seqs seqs, float *__restrict__ alpha_src,
                                                            int64_t nthreads) {
    const int64_t inst = blockIdx.y;
    const int64_t o = seqs.data[inst * seqs.maxlen + 0];
    for (int64_t state = (int64_t)blockIdx.x * kTpb + threadIdx.x; state < N; state += nthreads) {
        const int64_t num_kmers = N / 16;
        alpha_src[inst * N + state] = hmm.initial_prob[state] + hmm.output_prob[o * num_kmers + state % num_kmers];
    }
}

/* benchmarks/forward.py:103-158 */
template <int64_t N>
__global__ void __launch_bounds__(kTpb) forward_kernel_step(Hmm hmm, Seqs seqs, float *__restrict__ alpha1,
                                                            float *__restrict__ alpha2, int64_t t, int64_t nthreads) {
    const int64_t inst = blockIdx.y;
    float *alpha_src = alpha2;
    float *alpha_dst = alpha1;
    if (t & 1) {
        alpha_src = alpha1;
        alpha_dst = alpha2;
    }
    const int64_t o = seqs.data[inst * seqs.maxlen + t];
    for (int64_t state = (int64_t)blockIdx.x * kTpb + threadIdx.x; state < N; state += nthreads) {
        if (t < seqs.lens[inst]) {
            const int64_t num_kmers = N / 16;
            const int32_t pred1 = (int32_t)((state / 4) % (N / 64));
            const int32_t pred2 = (int32_t)(N / 64 + (state / 4) % (N / 64));
            const int32_t pred3 = (int32_t)(2 * N / 64 + (state / 4) % (N / 64));
            const int32_t pred4 = (int32_t)(3 * N / 64 + (state / 4) % (N / 64));
            const float t11 = hmm.trans1[(pred1 % num_kmers) * 4 + state % 4];
            const float t12 = hmm.trans1[(pred2 % num_kmers) * 4 + state % 4];
            const float t13 = hmm.trans1[(pred3 % num_kmers) * 4 + state % 4];
            const float t14 = hmm.trans1[(pred4 % num_kmers) * 4 + state % 4];
            const float t2 = hmm.trans2[state / num_kmers];
            const float p1 = t11 + t2 + alpha_src[inst * N + pred1];
            const float p2 = t12 + t2 + alpha_src[inst * N + pred2];
            const float p3 = t13 + t2 + alpha_src[inst * N + pred3];
            const float p4 = t14 + t2 + alpha_src[inst * N + pred4];
            int32_t pred5 = 0;
            float p5 = 0.0f;
            if (state / num_kmers == 15) {
                pred5 = (int32_t)state;
                p5 = hmm.gamma;
            } else if (state / num_kmers == 14) {
                pred5 = (int32_t)((state / num_kmers + 1) * num_kmers + state % num_kmers);
                p5 = hmm.synthetic_248;
            } else {
                pred5 = (int32_t)((state / num_kmers + 1) * num_kmers + state % num_kmers);
                p5 = 0.0f;
            }
            p5 = p5 + alpha_src[inst * N + pred5];
            float maxp = fmaxf(p1, p2);
            maxp = fmaxf(maxp, p3);
            maxp = fmaxf(maxp, p4);
            maxp = fmaxf(maxp, p5);
            float lsexp = maxp + __logf(__expf(p1 - maxp) + __expf(p2 - maxp) + __expf(p3 - maxp) +
                                        __expf(p4 - maxp) + __expf(p5 - maxp));
            lsexp = fmaxf(lsexp, -HUGE_VALF);
            alpha_dst[inst * N + state] = lsexp + hmm.output_prob[o * num_kmers + state % num_kmers];
        }
    }
}

/* Block reduce as emitted: butterfly, stemp[32], butterfly (src/gpu/reduce.rs:401-435). */
template <bool MAX>
__device__ __forceinline__ float combine(float a, float b) { return MAX ? fmaxf(a, b) : a + b; }
template <bool MAX>
__device__ __forceinline__ float block_reduce(float v) {
    __shared__ float stemp[32];
    for (int i = 16; i > 0; i /= 2) v = combine<MAX>(v, __shfl_xor_sync(0xFFFFFFFF, v, i));
    if (threadIdx.x < 32) stemp[threadIdx.x] = MAX ? -HUGE_VALF : 0.0f;
    __syncthreads();
    if (threadIdx.x % 32 == 0) stemp[threadIdx.x / 32] = v;
    __syncthreads();
    v = stemp[threadIdx.x % 32];
    for (int i = 16; i > 0; i /= 2) v = combine<MAX>(v, __shfl_xor_sync(0xFFFFFFFF, v, i));
    __syncthreads();
    return v;
}

/* benchmarks/forward.py:160-173, first stage of the two reductions: one partial per block. */
template <int64_t N, bool MAX>
__global__ void __launch_bounds__(kTpb) forward_kernel_lse_partial(Seqs seqs, const float *__restrict__ alpha1,
                                                                   const float *__restrict__ alpha2,
                                                                   const float *__restrict__ maxp,
                                                                   float *__restrict__ partial, int64_t nthreads) {
    const int64_t inst = blockIdx.y;
    const float *alpha = alpha2;
    if ((seqs.lens[inst] & 1) != 0) alpha = alpha1;
    float acc = MAX ? -HUGE_VALF : 0.0f;
    for (int64_t state = (int64_t)blockIdx.x * kTpb + threadIdx.x; state < N; state += nthreads) {
        if (MAX) acc = fmaxf(acc, alpha[inst * N + state]);
        else acc = acc + __expf(alpha[inst * N + state] - maxp[inst]);
    }
    acc = block_reduce<MAX>(acc);
    if (threadIdx.x == 0) partial[inst * gridDim.x + blockIdx.x] = acc;
}

/* Second stage: one block per instance reduces the partials into the cross-kernel local. */
template <bool MAX>
__global__ void __launch_bounds__(kTpb) forward_kernel_lse_final(const float *__restrict__ partial, int64_t nblocks,
                                                                 float *__restrict__ out) {
    const int64_t inst = blockIdx.y;
    float acc = MAX ? -HUGE_VALF : 0.0f;
    for (int64_t i = threadIdx.x; i < nblocks; i += kTpb) acc = combine<MAX>(acc, partial[inst * nblocks + i]);
    acc = block_reduce<MAX>(acc);
    if (threadIdx.x == 0) out[inst] = acc;
}

/* benchmarks/forward.py:173 */
__global__ void forward_kernel_store(const float *__restrict__ maxp, const float *__restrict__ psum,
                                     float *__restrict__ result, int64_t num_instances) {
    const int64_t inst = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (inst < num_instances) result[inst] = maxp[inst] + __logf(psum[inst]);
}

#define CHECK(expr)                          \
    do {                                     \
        cudaError_t e__ = (expr);            \
        if (e__ != cudaSuccess) return (int32_t)e__; \
    } while (0)

template <int64_t N>
int32_t run(Hmm hmm, Seqs seqs, float *result, float *alpha1, float *alpha2, int64_t nthreads, int32_t zero_fill) {
    const int64_t B = seqs.num_instances;
    if (nthreads <= kTpb || nthreads % kTpb != 0 || nthreads > N || B < 1 || B > 65535) return -1;
    if (zero_fill) {   /* torch.zeros of result, alpha1, alpha2: benchmarks/forward.py:190-192 */
        CHECK(cudaMemsetAsync(result, 0, sizeof(float) * B, 0));
        CHECK(cudaMemsetAsync(alpha1, 0, sizeof(float) * B * N, 0));
        CHECK(cudaMemsetAsync(alpha2, 0, sizeof(float) * B * N, 0));
    }
    const int64_t nblocks = nthreads / kTpb;
    const dim3 grid((unsigned)nblocks, (unsigned)B, 1), block(kTpb, 1, 1);
    forward_kernel_init<N><<<grid, block>>>(hmm, seqs, alpha1, nthreads);
    CHECK(cudaGetLastError());
    for (int64_t t = 1; t < seqs.maxlen; ++t) {
        forward_kernel_step<N><<<grid, block>>>(hmm, seqs, alpha1, alpha2, t, nthreads);
        CHECK(cudaGetLastError());
    }
    float *maxp, *psum, *partial;
    CHECK(cudaMallocAsync(&maxp, sizeof(float) * B, 0));
    CHECK(cudaMallocAsync(&psum, sizeof(float) * B, 0));
    CHECK(cudaMallocAsync(&partial, sizeof(float) * B * nblocks, 0));
    forward_kernel_lse_partial<N, true><<<grid, block>>>(seqs, alpha1, alpha2, nullptr, partial, nthreads);
    CHECK(cudaGetLastError());
    forward_kernel_lse_final<true><<<dim3(1, (unsigned)B, 1), block>>>(partial, nblocks, maxp);
    CHECK(cudaGetLastError());
    forward_kernel_lse_partial<N, false><<<grid, block>>>(seqs, alpha1, alpha2, maxp, partial, nthreads);
    CHECK(cudaGetLastError());
    forward_kernel_lse_final<false><<<dim3(1, (unsigned)B, 1), block>>>(partial, nblocks, psum);
    CHECK(cudaGetLastError());
    forward_kernel_store<<<(unsigned)((B + 255) / 256), 256>>>(maxp, psum, result, B);
    CHECK(cudaGetLastError());
    CHECK(cudaFreeAsync(partial, 0));
    CHECK(cudaFreeAsync(psum, 0));
    CHECK(cudaFreeAsync(maxp, 0));
    return 0;
}

}  // namespace

/* Flattened like the entry the compiler generates (dict arguments in sorted-key order, 0-d
 * values by value; python/parpy/compile.py:140-178), plus the thread count of the 'state'
 * label and the wrapper's zero fill. Returns 0, a cudaError_t, or -1 for a state space or
 * thread count this transcription was not instantiated for (num_states 4096, 16384 or 262144;
 * nthreads a multiple of 1024 above 1024). Asynchronous on stream 0. */
extern "C" int32_t parpy_emitted_forward_kernel(float gamma, float *initial_prob, int64_t num_states,
                                                float *output_prob, float synthetic_248, float *trans1,
                                                float *trans2, int8_t *data, int64_t *lens, int64_t maxlen,
                                                int64_t num_instances, float *result, float *alpha1, float *alpha2,
                                                int64_t nthreads, int32_t zero_fill) {
    Hmm hmm{gamma, initial_prob, output_prob, synthetic_248, trans1, trans2};
    Seqs seqs{data, lens, maxlen, num_instances};
    switch (num_states) {
        case 4096: return run<4096>(hmm, seqs, result, alpha1, alpha2, nthreads, zero_fill);
        case 16384: return run<16384>(hmm, seqs, result, alpha1, alpha2, nthreads, zero_fill);
        case 262144: return run<262144>(hmm, seqs, result, alpha1, alpha2, nthreads, zero_fill);
        default: return -1;
    }
}
