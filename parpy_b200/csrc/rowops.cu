// Row-wise softmax and sum / prod / max / min reductions for sm_100a.
//
// All of these are HBM-bound streaming kernels: the design goal is one global
// read of the input (plus one write of the output for softmax), 128-bit loads,
// and enough bytes in flight per SM. What the reference's compiler emits for
// the same Python functions reads the row from global memory up to four times
// (softmax: test/test_softmax.py:11-26) or uses two kernels with a temporary
// (reductions over more than 1024 threads: src/gpu/inter_block.rs:380-433).
//
//   softmax      rows <= 2048 floats: one warp per row, row held in registers;
//                rows <= 48K floats: one CTA per row, row staged in shared
//                memory; longer rows: one CTA per row, two passes over global.
//   reductions   short rows: one warp per row; long rows / full reductions:
//                grid-wide partials + a last-block finish (one launch, fixed
//                combination order, deterministic).
#include <algorithm>
#include <cfloat>

#include "../../include/parpy_b200.h"
#include "common.cuh"

namespace {

constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float fast_exp(float x) { return pb::ex2_approx(x * kLog2e); }

// ---------------------------------------------- softmax and its relatives ----
// One family of single-read / single-write row kernels with three modes:
//   kSoftmax    out = exp(x - max) / sum(exp(x - max))          (test/test_softmax.py:11-26)
//   kNormalize  out = x / sum(x)                                 (test/test_normalize.py:7-15)
//   kExpSum     out = exp(x), rowsum = sum(exp(x))               (test/test_sync.py:59-69)
// `out` may alias `x` (normalize_rows and sum_exp_3d work in place).
enum RowMode { kSoftmax = 0, kNormalize = 1, kExpSum = 2 };

template <int MODE>
__device__ __forceinline__ float row_map(float v, float m) {
    return MODE == kSoftmax ? fast_exp(v - m) : MODE == kExpSum ? fast_exp(v) : v;
}
template <int MODE>
__device__ __forceinline__ float row_finish(float v, float s, float inv) {
    return MODE == kSoftmax ? v * inv : MODE == kNormalize ? v / s : v;
}

__device__ __forceinline__ float block_max(float v, float *s_red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = pb::warp_max(v);
    __syncthreads();
    if (lane == 0) s_red[warp] = v;
    __syncthreads();
    float r = -INFINITY;
    for (int w = 0; w < nw; ++w) r = fmaxf(r, s_red[w]);
    return r;
}

__device__ __forceinline__ float block_sum(float v, float *s_red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = pb::warp_sum(v);
    __syncthreads();
    if (lane == 0) s_red[warp] = v;
    __syncthreads();
    float r = 0.0f;
    for (int w = 0; w < nw; ++w) r += s_red[w];
    return r;
}

// One warp per row; the row lives in registers (VEC float4 per lane).
template <int MODE, int VEC>
__global__ void __launch_bounds__(256) rowmap_warp_rows(const float *x, float *out,
                                                        float *__restrict__ rowsum, long long N, int M) {
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= N) return;
    const float4 *src = reinterpret_cast<const float4 *>(x + row * M);
    float4 *dst = reinterpret_cast<float4 *>(out + row * M);
    const int nvec = M >> 2;
    float4 v[VEC];
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        const int idx = lane + 32 * i;
        if (idx < nvec) {
            v[i] = __ldcs(src + idx);
            if (MODE == kSoftmax) m = fmaxf(m, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
        }
    }
    if (MODE == kSoftmax) m = pb::warp_max(m);
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        const int idx = lane + 32 * i;
        if (idx < nvec) {
            v[i].x = row_map<MODE>(v[i].x, m);
            v[i].y = row_map<MODE>(v[i].y, m);
            v[i].z = row_map<MODE>(v[i].z, m);
            v[i].w = row_map<MODE>(v[i].w, m);
            s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        }
    }
    s = pb::warp_sum(s);
    const float inv = 1.0f / s;
    if (MODE == kExpSum && lane == 0) rowsum[row] = s;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        const int idx = lane + 32 * i;
        if (idx < nvec) {
            v[i].x = row_finish<MODE>(v[i].x, s, inv);
            v[i].y = row_finish<MODE>(v[i].y, s, inv);
            v[i].z = row_finish<MODE>(v[i].z, s, inv);
            v[i].w = row_finish<MODE>(v[i].w, s, inv);
            __stcs(dst + idx, v[i]);
        }
    }
}

// One CTA per row, the row held in registers (VEC float4 per thread): a single
// global read and a single write for rows of up to blockDim * 4 * VEC floats.
template <int MODE, int VEC>
__global__ void __launch_bounds__(1024) rowmap_block_regs(const float *x, float *out,
                                                          float *__restrict__ rowsum, long long N, int M) {
    __shared__ float s_red[32];
    const int nvec = M >> 2;
    for (long long row = blockIdx.x; row < N; row += gridDim.x) {
        const float4 *src = reinterpret_cast<const float4 *>(x + row * M);
        float4 *dst = reinterpret_cast<float4 *>(out + row * M);
        float4 v[VEC];
        float m = -INFINITY;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            const int idx = threadIdx.x + blockDim.x * i;
            if (idx < nvec) {
                v[i] = __ldcs(src + idx);
                if (MODE == kSoftmax) m = fmaxf(m, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
            }
        }
        if (MODE == kSoftmax) m = block_max(m, s_red);
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            const int idx = threadIdx.x + blockDim.x * i;
            if (idx < nvec) {
                v[i].x = row_map<MODE>(v[i].x, m);
                v[i].y = row_map<MODE>(v[i].y, m);
                v[i].z = row_map<MODE>(v[i].z, m);
                v[i].w = row_map<MODE>(v[i].w, m);
                s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
            }
        }
        s = block_sum(s, s_red);
        const float inv = 1.0f / s;
        if (MODE == kExpSum && threadIdx.x == 0) rowsum[row] = s;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            const int idx = threadIdx.x + blockDim.x * i;
            if (idx < nvec) {
                v[i].x = row_finish<MODE>(v[i].x, s, inv);
                v[i].y = row_finish<MODE>(v[i].y, s, inv);
                v[i].z = row_finish<MODE>(v[i].z, s, inv);
                v[i].w = row_finish<MODE>(v[i].w, s, inv);
                __stcs(dst + idx, v[i]);
            }
        }
    }
}

// One CTA per row (grid-stride over rows) for everything else: unaligned or very
// long rows. STAGE: keep the row in dynamic shared memory between the passes;
// otherwise re-read it from global memory (the input is only overwritten in the
// last pass, so in-place use stays correct).
template <int MODE, bool STAGE>
__global__ void __launch_bounds__(1024) rowmap_block_rows(const float *x, float *out,
                                                          float *__restrict__ rowsum, long long N,
                                                          long long M) {
    extern __shared__ __align__(16) float s_row[];
    __shared__ float s_red[32];
    for (long long row = blockIdx.x; row < N; row += gridDim.x) {
        const float *src = x + row * M;
        float *dst = out + row * M;
        float m = -INFINITY;
        if (MODE == kSoftmax || STAGE) {
            for (long long i = threadIdx.x; i < M; i += blockDim.x) {
                const float v = src[i];
                if (STAGE) s_row[i] = v;
                m = fmaxf(m, v);
            }
            if (MODE == kSoftmax) m = block_max(m, s_red);
            else __syncthreads();
        }
        float s = 0.0f;
        for (long long i = threadIdx.x; i < M; i += blockDim.x) {
            const float e = row_map<MODE>(STAGE ? s_row[i] : src[i], m);
            if (STAGE) s_row[i] = e;
            s += e;
        }
        s = block_sum(s, s_red);
        const float inv = 1.0f / s;
        if (MODE == kExpSum && threadIdx.x == 0) rowsum[row] = s;
        for (long long i = threadIdx.x; i < M; i += blockDim.x) {
            const float e = STAGE ? s_row[i] : row_map<MODE>(src[i], m);
            dst[i] = row_finish<MODE>(e, s, inv);
        }
        __syncthreads();
    }
}

template <int MODE>
int32_t launch_rowmap(const float *x, float *out, float *rowsum, int64_t N, int64_t M, cudaStream_t stream,
                      const char *what) {
    PB_REQUIRE(N >= 0 && M >= 0, "%s: negative shape (%lld, %lld)", what, (long long)N, (long long)M);
    if (N == 0 || M == 0) return PB_OK;
    PB_REQUIRE(x && out && (MODE != kExpSum || rowsum), "%s: null pointer", what);
    pb::DeviceInfo dev;
    int32_t rc = pb::device_info(&dev);
    if (rc) return rc;
    const bool vec_ok = (M % 4 == 0) && pb::aligned16(x) && pb::aligned16(out);
    if (vec_ok && M <= 2048) {
        const int wpb = 4;
        const long long blocks = (N + wpb - 1) / wpb;
        PB_REQUIRE(blocks <= 0x7fffffffLL, "%s: too many rows", what);
        const int nvec = (int)(M / 4);
        if (nvec <= 32 * 2) rowmap_warp_rows<MODE, 2><<<(unsigned)blocks, wpb * 32, 0, stream>>>(x, out, rowsum, N, (int)M);
        else if (nvec <= 32 * 4) rowmap_warp_rows<MODE, 4><<<(unsigned)blocks, wpb * 32, 0, stream>>>(x, out, rowsum, N, (int)M);
        else if (nvec <= 32 * 8) rowmap_warp_rows<MODE, 8><<<(unsigned)blocks, wpb * 32, 0, stream>>>(x, out, rowsum, N, (int)M);
        else rowmap_warp_rows<MODE, 16><<<(unsigned)blocks, wpb * 32, 0, stream>>>(x, out, rowsum, N, (int)M);
        PB_CUDA(cudaGetLastError());
        return PB_OK;
    }
    if (vec_ok && M <= 32768) {
        // row in registers of one CTA: threads x VEC float4
        const int nvec = (int)(M / 4);
        const int threads = nvec <= 2048 ? 256 : nvec <= 4096 ? 512 : 1024;
        const int per = (nvec + threads - 1) / threads;
        // one resident wave: CTA b takes rows b, b + grid, ..., so the rows in flight are neighbours
#define PB_ROWMAP_REGS(V)                                                                                   \
    do {                                                                                                    \
        int per_sm = 0;                                                                                     \
        PB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, rowmap_block_regs<MODE, V>, threads, 0)); \
        const long long g = std::min<long long>(N, (long long)dev.sm_count * std::max(per_sm, 1));          \
        rowmap_block_regs<MODE, V><<<(unsigned)g, threads, 0, stream>>>(x, out, rowsum, N, (int)M);         \
    } while (0)
        if (per <= 2) PB_ROWMAP_REGS(2);
        else if (per <= 4) PB_ROWMAP_REGS(4);
        else PB_ROWMAP_REGS(8);
#undef PB_ROWMAP_REGS
        PB_CUDA(cudaGetLastError());
        return PB_OK;
    }
    const long long grid = std::min<long long>(N, 8LL * dev.sm_count);
    const size_t smem = (size_t)M * sizeof(float);
    const int threads = M >= 4096 ? 1024 : 256;
    if (smem <= 192 * 1024) {
        PB_CUDA(cudaFuncSetAttribute(rowmap_block_rows<MODE, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     192 * 1024));
        rowmap_block_rows<MODE, true><<<(unsigned)grid, threads, smem, stream>>>(x, out, rowsum, N, M);
    } else {
        rowmap_block_rows<MODE, false><<<(unsigned)grid, threads, 0, stream>>>(x, out, rowsum, N, M);
    }
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

// ------------------------------------------------------------- reductions ----
enum Op { kSum = 0, kProd = 1, kMax = 2, kMin = 3 };

template <int OP>
struct Red {
    // neutral elements: src/utils/reduce.rs:75-88
    __device__ static float neutral() {
        return OP == kSum ? 0.0f : OP == kProd ? 1.0f : OP == kMax ? -INFINITY : INFINITY;
    }
    __device__ static float apply(float a, float b) {
        return OP == kSum ? a + b : OP == kProd ? a * b : OP == kMax ? fmaxf(a, b) : fminf(a, b);
    }
    __device__ static float warp(float v) {
        return OP == kSum ? pb::warp_sum(v) : OP == kProd ? pb::warp_prod(v)
             : OP == kMax ? pb::warp_max(v) : pb::warp_min(v);
    }
};

// Reduces the part of x[0, n) that belongs to CTA `part` of `parts`: tiles of
// 4 x blockDim float4 dealt round-robin to the CTAs (so that the CTAs of a row read
// one contiguous region at any moment), 4 independent accumulators per thread,
// 128-bit streaming loads; CTA 0 also takes the unaligned ends. Every thread returns
// the CTA-wide value.
template <int OP>
__device__ float block_reduce_tiles(const float *__restrict__ x, long long n, int part, int parts,
                                    float *s_red) {
    using R = Red<OP>;
    float a0 = R::neutral(), a1 = R::neutral(), a2 = R::neutral(), a3 = R::neutral();
    long long head = 0;
    while (head < n && (reinterpret_cast<uintptr_t>(x + head) & 15u)) ++head;
    const long long nvec = (n - head) >> 2;
    const float4 *xv = reinterpret_cast<const float4 *>(x + head);
    const long long bd = blockDim.x, tile = 4 * bd;
    for (long long base = part * tile; base < nvec; base += (long long)parts * tile) {
        const long long i = base + threadIdx.x;
        if (base + tile <= nvec) {
            const float4 p = __ldcs(xv + i);
            const float4 q = __ldcs(xv + i + bd);
            const float4 r = __ldcs(xv + i + 2 * bd);
            const float4 t = __ldcs(xv + i + 3 * bd);
            a0 = R::apply(a0, R::apply(R::apply(p.x, p.y), R::apply(p.z, p.w)));
            a1 = R::apply(a1, R::apply(R::apply(q.x, q.y), R::apply(q.z, q.w)));
            a2 = R::apply(a2, R::apply(R::apply(r.x, r.y), R::apply(r.z, r.w)));
            a3 = R::apply(a3, R::apply(R::apply(t.x, t.y), R::apply(t.z, t.w)));
        } else {
            for (long long j = i; j < nvec; j += bd) {
                const float4 p = __ldcs(xv + j);
                a0 = R::apply(a0, R::apply(R::apply(p.x, p.y), R::apply(p.z, p.w)));
            }
        }
    }
    if (part == 0) {
        for (long long j = threadIdx.x; j < head; j += bd) a1 = R::apply(a1, x[j]);
        for (long long j = head + (nvec << 2) + threadIdx.x; j < n; j += bd) a1 = R::apply(a1, x[j]);
    }
    float v = R::apply(R::apply(a0, a1), R::apply(a2, a3));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = R::warp(v);
    __syncthreads();
    if (lane == 0) s_red[warp] = v;
    __syncthreads();
    float r = R::neutral();
    for (int w = 0; w < nw; ++w) r = R::apply(r, s_red[w]);
    return r;
}

// One warp per row, for rows up to a few thousand elements.
template <int OP>
__global__ void __launch_bounds__(256) reduce_warp_rows(const float *__restrict__ x,
                                                        float *__restrict__ out, long long N,
                                                        long long M) {
    using R = Red<OP>;
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= N) return;
    const float *src = x + row * M;
    float a = R::neutral(), b = R::neutral();
    if ((M & 3) == 0 && pb::aligned16(src)) {
        const float4 *sv = reinterpret_cast<const float4 *>(src);
        const long long nvec = M >> 2;
        long long i = lane;
        for (; i + 96 < nvec; i += 128) {   // four 128-bit loads in flight per lane
            const float4 p = __ldcs(sv + i), q = __ldcs(sv + i + 32), r = __ldcs(sv + i + 64), t = __ldcs(sv + i + 96);
            a = R::apply(a, R::apply(R::apply(p.x, p.y), R::apply(p.z, p.w)));
            b = R::apply(b, R::apply(R::apply(q.x, q.y), R::apply(q.z, q.w)));
            a = R::apply(a, R::apply(R::apply(r.x, r.y), R::apply(r.z, r.w)));
            b = R::apply(b, R::apply(R::apply(t.x, t.y), R::apply(t.z, t.w)));
        }
        for (; i < nvec; i += 32) {
            const float4 p = __ldcs(sv + i);
            a = R::apply(a, R::apply(R::apply(p.x, p.y), R::apply(p.z, p.w)));
        }
    } else {
        for (long long i = lane; i < M; i += 32) a = R::apply(a, src[i]);
    }
    const float v = R::warp(R::apply(a, b));
    if (lane == 0) out[row] = v;
}

// Rows split over `parts` CTAs each. Every CTA stores its partial, takes a
// ticket for its row, and the CTA that draws the last ticket combines the
// partials in index order. `tickets` must be zero on entry; the finishing CTA
// zeroes its row's ticket again, so the scratch is reusable without a memset.
template <int OP>
__global__ void __launch_bounds__(512) reduce_split_rows(const float *__restrict__ x,
                                                         float *__restrict__ out, long long M,
                                                         int parts, float *__restrict__ partials,
                                                         unsigned *__restrict__ tickets) {
    using R = Red<OP>;
    __shared__ float s_red[32];
    __shared__ bool s_last;
    const long long row = blockIdx.y;
    const int part = blockIdx.x;
    const float v = block_reduce_tiles<OP>(x + row * M, M, part, parts, s_red);
    if (parts == 1) {
        if (threadIdx.x == 0) out[row] = v;
        return;
    }
    if (threadIdx.x == 0) {
        partials[row * parts + part] = v;
        __threadfence();
        const unsigned t = atomicAdd(&tickets[row], 1u);
        s_last = (t == (unsigned)parts - 1u);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    float a = R::neutral();
    for (int i = threadIdx.x; i < parts; i += blockDim.x) a = R::apply(a, __ldcg(partials + row * parts + i));
    // fixed combination order: per-thread strided, then warp tree, then warp order
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    a = R::warp(a);
    __syncthreads();
    if (lane == 0) s_red[warp] = a;
    __syncthreads();
    if (threadIdx.x == 0) {
        float r = R::neutral();
        for (int w = 0; w < nw; ++w) r = R::apply(r, s_red[w]);
        out[row] = r;
        tickets[row] = 0;
    }
}

// Fused sum and max of one long vector in a single pass (4 B/element).
__global__ void __launch_bounds__(512) sum_max_fused(const float *__restrict__ x, long long n,
                                                     float *__restrict__ out_sum,
                                                     float *__restrict__ out_max, int parts,
                                                     float *__restrict__ partials,
                                                     unsigned *__restrict__ ticket) {
    __shared__ float s_a[32], s_b[32];
    __shared__ bool s_last;
    const int part = blockIdx.x;
    // Tiles of 4 x blockDim float4 dealt round-robin to the CTAs, so that at any moment the
    // whole grid reads one contiguous region of the vector. CTA 0 takes the unaligned ends.
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f, m0 = -INFINITY, m1 = -INFINITY;
    long long head = 0;
    while (head < n && (reinterpret_cast<uintptr_t>(x + head) & 15u)) ++head;
    const long long nvec = (n - head) >> 2;
    const float4 *xv = reinterpret_cast<const float4 *>(x + head);
    const long long bd = blockDim.x, tile = 4 * bd;
    for (long long base = part * tile; base < nvec; base += (long long)parts * tile) {
        const long long i = base + threadIdx.x;
        if (base + tile <= nvec) {
            const float4 p = __ldcs(xv + i);
            const float4 q = __ldcs(xv + i + bd);
            const float4 r = __ldcs(xv + i + 2 * bd);
            const float4 t = __ldcs(xv + i + 3 * bd);
            s0 += (p.x + p.y) + (p.z + p.w);
            s1 += (q.x + q.y) + (q.z + q.w);
            s2 += (r.x + r.y) + (r.z + r.w);
            s3 += (t.x + t.y) + (t.z + t.w);
            m0 = fmaxf(m0, fmaxf(fmaxf(fmaxf(p.x, p.y), fmaxf(p.z, p.w)), fmaxf(fmaxf(q.x, q.y), fmaxf(q.z, q.w))));
            m1 = fmaxf(m1, fmaxf(fmaxf(fmaxf(r.x, r.y), fmaxf(r.z, r.w)), fmaxf(fmaxf(t.x, t.y), fmaxf(t.z, t.w))));
        } else {
            for (long long j = i; j < nvec; j += bd) {
                const float4 p = __ldcs(xv + j);
                s0 += (p.x + p.y) + (p.z + p.w);
                m0 = fmaxf(m0, fmaxf(fmaxf(p.x, p.y), fmaxf(p.z, p.w)));
            }
        }
    }
    if (part == 0) {
        for (long long j = threadIdx.x; j < head; j += bd) {
            s1 += x[j];
            m1 = fmaxf(m1, x[j]);
        }
        for (long long j = head + (nvec << 2) + threadIdx.x; j < n; j += bd) {
            s1 += x[j];
            m1 = fmaxf(m1, x[j]);
        }
    }
    float s = (s0 + s1) + (s2 + s3), m = fmaxf(m0, m1);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    s = pb::warp_sum(s);
    m = pb::warp_max(m);
    if (lane == 0) {
        s_a[warp] = s;
        s_b[warp] = m;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float ts = 0.f, tm = -INFINITY;
        for (int w = 0; w < nw; ++w) {
            ts += s_a[w];
            tm = fmaxf(tm, s_b[w]);
        }
        partials[2 * part] = ts;
        partials[2 * part + 1] = tm;
        __threadfence();
        const unsigned t = atomicAdd(ticket, 1u);
        s_last = (t == (unsigned)parts - 1u);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // the finishing CTA sums the partials in double precision, in index order per thread
    double ds = 0.0;
    float dm = -INFINITY;
    for (int k = threadIdx.x; k < parts; k += blockDim.x) {
        ds += (double)__ldcg(partials + 2 * k);
        dm = fmaxf(dm, __ldcg(partials + 2 * k + 1));
    }
    __shared__ double s_d[32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ds += __shfl_xor_sync(0xffffffffu, ds, o);
    }
    dm = pb::warp_max(dm);
    __syncthreads();
    if (lane == 0) {
        s_d[warp] = ds;
        s_b[warp] = dm;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        double r = 0.0;
        float rm = -INFINITY;
        for (int w = 0; w < nw; ++w) {
            r += s_d[w];
            rm = fmaxf(rm, s_b[w]);
        }
        *out_sum = (float)r;
        *out_max = rm;
        *ticket = 0;
    }
}

template <int OP>
int32_t launch_reduce(const float *x, float *out, long long N, long long M, cudaStream_t stream,
                      const pb::DeviceInfo &dev) {
    if (M <= 16384 && N >= 8LL * dev.sm_count) {
        const int wpb = 8;
        const long long blocks = (N + wpb - 1) / wpb;
        reduce_warp_rows<OP><<<(unsigned)blocks, wpb * 32, 0, stream>>>(x, out, N, M);
        PB_CUDA(cudaGetLastError());
        return PB_OK;
    }
    // CTAs per row so that the grid is one resident wave
    int per_sm = 1;
    PB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, reduce_split_rows<OP>, 512, 0));
    const long long target = (long long)std::max(per_sm, 1) * dev.sm_count;
    long long parts = std::max<long long>(1, std::min<long long>((target + N - 1) / N, (M + 8191) / 8192));
    parts = std::min<long long>(parts, 1024);
    PB_REQUIRE(N <= 65535, "reduce: more than 65535 rows of more than 4096 elements are not supported");
    void *ws = nullptr;
    const size_t tick_bytes = ((size_t)N * sizeof(unsigned) + 255) & ~size_t(255);
    const size_t part_bytes = (size_t)N * (size_t)parts * sizeof(float);
    int32_t rc = pb::zeroed_workspace(tick_bytes, part_bytes, &ws, stream);
    if (rc) return rc;
    unsigned *tickets = static_cast<unsigned *>(ws);
    float *partials = reinterpret_cast<float *>(static_cast<char *>(ws) + tick_bytes);
    dim3 grid((unsigned)parts, (unsigned)N, 1);
    reduce_split_rows<OP><<<grid, 512, 0, stream>>>(x, out, M, (int)parts, partials, tickets);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

}  // namespace

extern "C" {

int32_t parpy_b200_softmax(const float *x, int64_t N, int64_t M, float *out, void *stream_) {
    return launch_rowmap<kSoftmax>(x, out, nullptr, N, M, static_cast<cudaStream_t>(stream_), "softmax");
}

int32_t parpy_b200_normalize_rows(float *t, int64_t nrows, int64_t ncols, void *stream_) {
    return launch_rowmap<kNormalize>(t, t, nullptr, nrows, ncols, static_cast<cudaStream_t>(stream_),
                                     "normalize_rows");
}

int32_t normalize_rows(float *t, int64_t nrows, int64_t ncols) {
    return parpy_b200_normalize_rows(t, nrows, ncols, nullptr);
}

int32_t parpy_b200_sum_exp_rows(float *x, int64_t nrows, int64_t ncols, float *out, void *stream_) {
    return launch_rowmap<kExpSum>(x, x, out, nrows, ncols, static_cast<cudaStream_t>(stream_), "sum_exp");
}

int32_t softmax(float *x, int64_t N, int64_t M, float *out) {
    return parpy_b200_softmax(x, N, M, out, nullptr);
}

int32_t parpy_b200_reduce_rows(int32_t op, const float *x, float *out, int64_t N, int64_t M,
                               void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    PB_REQUIRE(op >= 0 && op <= 3, "reduce: unknown operator %d", op);
    PB_REQUIRE(N >= 0 && M >= 0, "reduce: negative shape (%lld, %lld)", (long long)N, (long long)M);
    if (N == 0) return PB_OK;
    PB_REQUIRE(x || M == 0, "reduce: null input");
    PB_REQUIRE(out, "reduce: null output");
    pb::DeviceInfo dev;
    int32_t rc = pb::device_info(&dev);
    if (rc) return rc;
    switch (op) {
        case kSum: return launch_reduce<kSum>(x, out, N, M, stream, dev);
        case kProd: return launch_reduce<kProd>(x, out, N, M, stream, dev);
        case kMax: return launch_reduce<kMax>(x, out, N, M, stream, dev);
        default: return launch_reduce<kMin>(x, out, N, M, stream, dev);
    }
}

int32_t parpy_b200_sum_max(const float *x, int64_t n, float *out_sum, float *out_max, void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    PB_REQUIRE(n >= 1, "sum_max: needs at least one element, got %lld", (long long)n);
    PB_REQUIRE(x && out_sum && out_max, "sum_max: null pointer");
    pb::DeviceInfo dev;
    int32_t rc = pb::device_info(&dev);
    if (rc) return rc;
    // one resident wave: as many CTAs as the kernel's registers allow per SM
    int per_sm = 1;
    PB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, sum_max_fused, 512, 0));
    long long parts = std::min<long long>((long long)std::max(per_sm, 1) * dev.sm_count, (n + 16383) / 16384);
    parts = std::max<long long>(parts, 1);
    void *ws = nullptr;
    rc = pb::zeroed_workspace(256, (size_t)parts * 2 * sizeof(float), &ws, stream);
    if (rc) return rc;
    unsigned *ticket = static_cast<unsigned *>(ws);
    float *partials = reinterpret_cast<float *>(static_cast<char *>(ws) + 256);
    sum_max_fused<<<(unsigned)parts, 512, 0, stream>>>(x, n, out_sum, out_max, (int)parts, partials, ticket);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

}  // extern "C"
