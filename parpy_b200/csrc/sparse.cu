// CSR SpMV and SDDMM for sm_100a. Both are FFMA kernels bound by memory
// traffic; neither is a dense contraction worth tensor cores.
//
// SpMV (test/test_spmv.py:12-18): y[row] += sum_i values[i] * x[cols[i]] over
// the row's non-zeros, int64 row pointers and column indices as torch CSR
// tensors carry them. The reference maps one 128-thread CTA to every row,
// whatever its length. Here the non-zeros are cut into equal chunks, one CTA per
// chunk: values and column indices stream in fully coalesced, the products go to
// shared memory, and a segmented reduction hands them to their rows (one thread
// per short row, one warp per long row). Work per CTA is the same whatever the
// row-length distribution, which is what a power-law matrix needs.
//
// SDDMM (benchmarks/sddmm.py:21-41,63-70): D[i] = alpha * dot(A[row_i,:],
// B[:,col_i]) + beta * Cvalues[i]. The reference reads B[:,col] with a stride of
// ncols floats per element (one 32-byte sector per 4 useful bytes). Here B is
// transposed once per call into library scratch so that both operands of every
// dot product are contiguous; half a warp serves one non-zero with 128-bit loads.
#include <algorithm>

#include "../../include/parpy_b200.h"
#include "common.cuh"

namespace {

// ------------------------------------------------------------------- SpMV ----
constexpr int kLongRow = 64;   // segments above this get a warp

// first_row[c] = the row that contains non-zero c * kSpmvChunk, i.e. the largest
// r with rows[r] <= c * kSpmvChunk. One thread per row writes the entries of the
// chunk starts that fall inside its row (none for an empty row), so the table is
// built with one coalesced pass over the row pointers and no search; the pass
// also leaves the row pointers in L2 for the main kernel.
__global__ void spmv_first_rows(const int64_t *__restrict__ rows, long long nrows,
                                int *__restrict__ first_row, int kSpmvChunk) {
    const long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= nrows) return;
    const long long start = __ldg(rows + r), end = __ldg(rows + r + 1);
    if (end <= start) return;
    for (long long c = (start + kSpmvChunk - 1) / kSpmvChunk; c * kSpmvChunk < end; ++c)
        first_row[c] = (int)r;
}

template <int kSpmvThreads, int kSpmvPerThread>
__global__ void __launch_bounds__(kSpmvThreads) spmv_chunks(const float *__restrict__ values,
                                                            const int64_t *__restrict__ cols,
                                                            const int64_t *__restrict__ rows,
                                                            long long nrows, long long nnz,
                                                            const float *__restrict__ x,
                                                            float *__restrict__ y,
                                                            const int *__restrict__ first_row) {
    constexpr int kSpmvChunk = kSpmvThreads * kSpmvPerThread;   // non-zeros per CTA
    constexpr int kMaxLong = kSpmvChunk / kLongRow;
    __shared__ float s_prod[kSpmvChunk];
    __shared__ int s_nlong;
    __shared__ long long s_long_row[kMaxLong];
    __shared__ int s_long_a[kMaxLong], s_long_b[kMaxLong];
    const int tid = threadIdx.x;
    const long long lo = (long long)blockIdx.x * kSpmvChunk;
    const long long hi = pb::ll_min(nnz, lo + kSpmvChunk);
    if (tid == 0) s_nlong = 0;

    // stream this chunk's non-zeros: loads first, then the gathers, then smem
    float v[kSpmvPerThread];
    long long c[kSpmvPerThread];
#pragma unroll
    for (int i = 0; i < kSpmvPerThread; ++i) {
        const long long idx = lo + i * kSpmvThreads + tid;
        if (idx < hi) {
            v[i] = __ldcs(values + idx);
            c[i] = __ldcs(cols + idx);
        }
    }
    // the rows this thread will own, fetched while the non-zeros are in flight
    const long long r0 = (long long)__ldg(first_row + blockIdx.x) + tid;
    long long start0 = 0, end0 = 0;
    if (r0 < nrows) {
        start0 = __ldg(rows + r0);
        end0 = __ldg(rows + r0 + 1);
    }
#pragma unroll
    for (int i = 0; i < kSpmvPerThread; ++i) {
        const long long idx = lo + i * kSpmvThreads + tid;
        if (idx < hi) s_prod[i * kSpmvThreads + tid] = v[i] * __ldg(x + c[i]);
    }
    __syncthreads();

    // rows that own a piece of this chunk: one thread per row
    for (long long r = r0; r < nrows; r += kSpmvThreads) {
        const long long start = r == r0 ? start0 : __ldg(rows + r);
        if (start >= hi) break;
        const long long end = r == r0 ? end0 : __ldg(rows + r + 1);
        const long long a = pb::ll_max(start, lo), b = pb::ll_min(end, hi);
        if (b <= a) continue;
        const int ia = (int)(a - lo), ib = (int)(b - lo);
        if (ib - ia > kLongRow) {
            const int slot = atomicAdd(&s_nlong, 1);
            s_long_row[slot] = r;
            s_long_a[slot] = ia;
            s_long_b[slot] = ib;
            continue;
        }
        float sum = 0.0f;
        for (int j = ia; j < ib; ++j) sum += s_prod[j];
        if (start >= lo && end <= hi) y[r] = y[r] + sum;   // the row lies inside this chunk
        else atomicAdd(y + r, sum);                        // shared with a neighbouring chunk
    }
    __syncthreads();
    const int nlong = s_nlong;
    const int lane = tid & 31, warp = tid >> 5;
    for (int k = warp; k < nlong; k += kSpmvThreads / 32) {
        const int ia = s_long_a[k], ib = s_long_b[k];
        float sum = 0.0f;
        for (int j = ia + lane; j < ib; j += 32) sum += s_prod[j];
        sum = pb::warp_sum(sum);
        if (lane == 0) {
            const long long r = s_long_row[k];
            const long long start = __ldg(rows + r), end = __ldg(rows + r + 1);
            if (start >= lo && end <= hi) y[r] = y[r] + sum;
            else atomicAdd(y + r, sum);
        }
    }
}

// ------------------------------------------------------------------ SDDMM ----
// rows[i] = row for every non-zero of a CSR matrix (benchmarks/sddmm.py:21-26).
__global__ void sddmm_decompress(const int64_t *__restrict__ crows, int64_t *__restrict__ rows, long long N) {
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= N) return;
    const long long a = __ldg(crows + row), b = __ldg(crows + row + 1);
    for (long long i = a + lane; i < b; i += 32) rows[i] = row;
}

// One launch for both passes that precede the dot products: the first `tblocks` CTAs
// transpose a 32 x 32 tile of B each, the others expand 8 CSR rows each into per-non-zero
// row indices (crows == nullptr: rows are given, nothing to expand).
__global__ void __launch_bounds__(256) sddmm_prepare(const float *__restrict__ B, float *__restrict__ Bt,
                                                     long long K, long long ncols, unsigned tiles_x,
                                                     unsigned tblocks, const int64_t *__restrict__ crows,
                                                     int64_t *__restrict__ rows, long long N) {
    if (blockIdx.x < tblocks) {
        __shared__ float tile[32][33];
        const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
        const long long c0 = (long long)(blockIdx.x % tiles_x) * 32, k0 = (long long)(blockIdx.x / tiles_x) * 32;
        for (int j = ty; j < 32; j += 8) {
            const long long k = k0 + j, c = c0 + tx;
            if (k < K && c < ncols) tile[j][tx] = B[k * ncols + c];
        }
        __syncthreads();
        for (int j = ty; j < 32; j += 8) {
            const long long c = c0 + j, k = k0 + tx;
            if (k < K && c < ncols) Bt[c * K + k] = tile[tx][j];
        }
    } else {
        const int lane = threadIdx.x & 31;
        const long long row = (long long)(blockIdx.x - tblocks) * 8 + (threadIdx.x >> 5);
        if (row >= N) return;
        const long long a = __ldg(crows + row), b = __ldg(crows + row + 1);
        for (long long i = a + lane; i < b; i += 32) rows[i] = row;
    }
}

// A warp takes W = (32 / LPN) * U consecutive non-zeros per trip: lane l loads row and column
// index l (one coalesced request each, the next trip's while this trip's operands travel),
// groups of LPN lanes then work on U non-zeros each, every lane holding K / LPN elements of the
// two operand rows, H 128-bit pieces per operand and non-zero in flight (all loads of a trip
// are issued before the math, so their L2 round trips overlap), a log2(LPN)-step shuffle sum
// per non-zero, and lane l stores non-zero l of the trip (coalesced). The grid is one resident
// wave. VEC: 128-bit loads (K % 4 == 0, 16-byte aligned rows).
template <bool VEC, int LPN, int U, int H>
__global__ void __launch_bounds__(256) sddmm_nnz(const float *__restrict__ A, const float *__restrict__ Bt,
                                                 const int64_t *__restrict__ rows,
                                                 const int64_t *__restrict__ cols,
                                                 const float *__restrict__ cvalues, float *__restrict__ D,
                                                 long long nnz, int K, float alpha, float beta) {
    constexpr int G = 32 / LPN;   // non-zeros a warp works on at once
    constexpr int W = G * U;      // non-zeros per warp and trip
    static_assert(W <= 32, "one index per lane");
    const int lane = threadIdx.x & 31;
    const int sub = lane % LPN, grp = lane / LPN;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    auto load_index = [&](long long base, long long &r, long long &c) {
        r = 0;
        c = 0;
        if (lane < W && base < nnz) {
            const long long i = base + lane < nnz ? base + lane : nnz - 1;   // clamp: harmless duplicate work
            r = __ldg(rows + i);
            c = __ldg(cols + i);
        }
    };
    long long my_row, my_col;
    load_index(warp * W, my_row, my_col);
    // the trip count depends on the warp only, so the full-mask shuffles below are safe
    for (long long base = warp * W; base < nnz; base += nwarps * W) {
        long long next_row, next_col;
        load_index(base + nwarps * W, next_row, next_col);
        const float *a[U], *b[U];
        float acc[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int src = u * G + grp;
            a[u] = A + __shfl_sync(0xffffffffu, my_row, src) * K;
            b[u] = Bt + __shfl_sync(0xffffffffu, my_col, src) * K;
            acc[u] = 0.0f;
        }
        if (VEC) {
            for (int k = 4 * sub; k < K; k += 4 * LPN * H) {
                float4 p[U][H], q[U][H];
#pragma unroll
                for (int u = 0; u < U; ++u) {
#pragma unroll
                    for (int h = 0; h < H; ++h) {
                        const int kk = k + 4 * LPN * h;
                        const bool in = h == 0 || kk < K;
                        q[u][h] = in ? __ldg(reinterpret_cast<const float4 *>(b[u] + kk)) : make_float4(0.f, 0.f, 0.f, 0.f);
                        p[u][h] = in ? __ldg(reinterpret_cast<const float4 *>(a[u] + kk)) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
#pragma unroll
                    for (int h = 0; h < H; ++h) {
                        acc[u] = fmaf(p[u][h].x, q[u][h].x, acc[u]);
                        acc[u] = fmaf(p[u][h].y, q[u][h].y, acc[u]);
                        acc[u] = fmaf(p[u][h].z, q[u][h].z, acc[u]);
                        acc[u] = fmaf(p[u][h].w, q[u][h].w, acc[u]);
                    }
                }
            }
        } else {
            for (int k = sub; k < K; k += LPN) {
#pragma unroll
                for (int u = 0; u < U; ++u) acc[u] = fmaf(__ldg(a[u] + k), __ldg(b[u] + k), acc[u]);
            }
        }
        float mine = 0.0f;
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
            for (int o = LPN / 2; o > 0; o >>= 1) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], o);
            // non-zero u * G + g of the trip sits in group g: hand it to lane u * G + g
            const float v = __shfl_sync(0xffffffffu, acc[u], (lane % G) * LPN);
            if (lane / G == u) mine = v;
        }
        if (lane < W && base + lane < nnz) D[base + lane] = alpha * mine + beta * __ldg(cvalues + base + lane);
        my_row = next_row;
        my_col = next_col;
    }
}


// ------------------------------------------------------------------- SpMM ----
// C[i, j] += sum over the non-zeros a of row i of values[a] * B[cols[a], j]
// (test/test_spmm.py:16-24). The reference gives every cell (i, j) its own
// 32-thread block. Here a warp owns one row and a run of up to 128 columns: LPR
// lanes cover the run with one float4 each, so every non-zero is one coalesced
// read of a B row segment, and the 32 / LPR lane groups take different non-zeros
// of the row at the same time (narrow B: all lanes busy, several gathers in
// flight); the groups' partial sums meet in a shuffle butterfly and group 0
// updates C once.
template <int LPR>
__global__ void __launch_bounds__(256) spmm_warp_rows(const float *__restrict__ values,
                                                      const int64_t *__restrict__ rows,
                                                      const int64_t *__restrict__ cols,
                                                      const float *__restrict__ B, long long nrows,
                                                      long long K, int chunks, float *__restrict__ C) {
    constexpr int G = 32 / LPR;   // non-zeros in flight per warp and trip
    const int lane = threadIdx.x & 31, sub = lane % LPR, grp = lane / LPR;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long i = warp / chunks;
    if (i >= nrows) return;
    const long long j = (warp % chunks) * (4 * LPR) + 4 * sub;
    const bool live = j < K;   // K % 4 == 0: a float4 is inside or outside as a whole
    const long long a0 = __ldg(rows + i), a1 = __ldg(rows + i + 1);
    float4 acc0 = make_float4(0.f, 0.f, 0.f, 0.f), acc1 = acc0;
    long long a = a0 + grp;
    for (; a + G < a1; a += 2 * G) {   // two non-zeros per group in flight
        const float v0 = __ldg(values + a), v1 = __ldg(values + a + G);
        const long long c0 = __ldg(cols + a), c1 = __ldg(cols + a + G);
        if (live) {
            const float4 b0 = __ldg(reinterpret_cast<const float4 *>(B + c0 * K + j));
            const float4 b1 = __ldg(reinterpret_cast<const float4 *>(B + c1 * K + j));
            acc0.x = fmaf(v0, b0.x, acc0.x); acc0.y = fmaf(v0, b0.y, acc0.y);
            acc0.z = fmaf(v0, b0.z, acc0.z); acc0.w = fmaf(v0, b0.w, acc0.w);
            acc1.x = fmaf(v1, b1.x, acc1.x); acc1.y = fmaf(v1, b1.y, acc1.y);
            acc1.z = fmaf(v1, b1.z, acc1.z); acc1.w = fmaf(v1, b1.w, acc1.w);
        }
    }
    if (a < a1 && live) {
        const float v0 = __ldg(values + a);
        const float4 b0 = __ldg(reinterpret_cast<const float4 *>(B + __ldg(cols + a) * K + j));
        acc0.x = fmaf(v0, b0.x, acc0.x); acc0.y = fmaf(v0, b0.y, acc0.y);
        acc0.z = fmaf(v0, b0.z, acc0.z); acc0.w = fmaf(v0, b0.w, acc0.w);
    }
    acc0.x += acc1.x; acc0.y += acc1.y; acc0.z += acc1.z; acc0.w += acc1.w;
#pragma unroll
    for (int o = LPR; o < 32; o <<= 1) {   // across the lane groups
        acc0.x += __shfl_xor_sync(0xffffffffu, acc0.x, o);
        acc0.y += __shfl_xor_sync(0xffffffffu, acc0.y, o);
        acc0.z += __shfl_xor_sync(0xffffffffu, acc0.z, o);
        acc0.w += __shfl_xor_sync(0xffffffffu, acc0.w, o);
    }
    if (grp == 0 && live) {
        float4 *dst = reinterpret_cast<float4 *>(C + i * K + j);
        float4 c = *dst;
        c.x += acc0.x; c.y += acc0.y; c.z += acc0.z; c.w += acc0.w;
        *dst = c;
    }
}

// Any width and alignment: one thread per cell of a row's column run.
__global__ void __launch_bounds__(128) spmm_rows_scalar(const float *__restrict__ values,
                                                        const int64_t *__restrict__ rows,
                                                        const int64_t *__restrict__ cols,
                                                        const float *__restrict__ B, long long K, int chunks,
                                                        float *__restrict__ C) {
    const long long i = blockIdx.x / chunks;
    const long long j = (long long)(blockIdx.x % chunks) * blockDim.x + threadIdx.x;
    if (j >= K) return;
    const long long a0 = __ldg(rows + i), a1 = __ldg(rows + i + 1);
    float acc = 0.f;
    for (long long a = a0; a < a1; ++a) acc = fmaf(__ldg(values + a), __ldg(B + __ldg(cols + a) * K + j), acc);
    C[i * K + j] += acc;
}

int32_t sddmm_common(const float *A, const float *B, const int64_t *crows, int64_t N, const int64_t *rows,
                     const int64_t *cols, const float *cvalues, float *D, int64_t K, int64_t ncols,
                     int64_t nnz, double alpha, double beta, cudaStream_t stream) {
    PB_REQUIRE(K >= 1 && K <= 0x7fffffffLL && ncols >= 1, "sddmm: bad inner size K=%lld or ncols=%lld",
               (long long)K, (long long)ncols);
    if (nnz == 0) return PB_OK;
    PB_REQUIRE(A && B && rows && cols && cvalues && D, "sddmm: null pointer");
    pb::DeviceInfo dev;
    int32_t rc = pb::device_info(&dev);
    if (rc) return rc;
    void *ws = nullptr;
    rc = pb::workspace((size_t)K * (size_t)ncols * sizeof(float), &ws, stream, 2);
    if (rc) return rc;
    float *Bt = static_cast<float *>(ws);
    const long long tiles_x = (ncols + 31) / 32, tiles = tiles_x * ((K + 31) / 32);
    const long long expand = crows ? (N + 7) / 8 : 0;
    PB_REQUIRE(tiles + expand <= 0x7fffffffLL, "sddmm: K=%lld x ncols=%lld too large", (long long)K, (long long)ncols);
    sddmm_prepare<<<(unsigned)(tiles + expand), 256, 0, stream>>>(B, Bt, K, ncols, (unsigned)tiles_x, (unsigned)tiles,
                                                                 crows, const_cast<int64_t *>(rows), N);
    PB_CUDA(cudaGetLastError());
    const bool vec = (K % 4 == 0) && pb::aligned16(A) && pb::aligned16(Bt);
    static const int cfg_env = [] { const char *e = getenv("PARPY_B200_SDDMM_CFG"); return e ? atoi(e) : -1; }();
    const int cfg = cfg_env >= 0 ? cfg_env : 0;
#define PB_SDDMM(V, L, U, H)                                                                                  \
    do {                                                                                                      \
        int per_sm = 0;                                                                                       \
        PB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, sddmm_nnz<V, L, U, H>, 256, 0));       \
        const long long per_block = (256 / 32) * (32 / L) * U;                                                \
        const long long blocks = std::max<long long>(                                                         \
            1, std::min<long long>((nnz + per_block - 1) / per_block, (long long)std::max(per_sm, 1) * dev.sm_count)); \
        sddmm_nnz<V, L, U, H><<<(unsigned)blocks, 256, 0, stream>>>(A, Bt, rows, cols, cvalues, D, nnz,       \
                                                                    (int)K, (float)alpha, (float)beta);       \
    } while (0)
    // measured at 8192 x 8192, 1 %, K = 64: <4,2,2> 38.9 us for the whole call, <8,4,2> 40.0,
    // <8,8,1> 46, <16,8,1> 73 (the old half-warp-per-non-zero kernel: 64)
    // K = 1024 (the reference's other inner size, benchmarks/bench.py:206-244): 0.29 ms, i.e. 2.75 GB of
    // gathered B^T rows at 9.5 TB/s out of the L2. A variant that keeps the A row of a run of non-zeros in
    // registers (one warp per run, only B^T rows move) measured 0.284 ms and was not kept.
    if (!vec) PB_SDDMM(false, 8, 4, 1);
    else if (cfg == 1) PB_SDDMM(true, 8, 4, 2);
    else PB_SDDMM(true, 4, 2, 2);
#undef PB_SDDMM
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

}  // namespace

extern "C" {

int32_t parpy_b200_spmv(const float *values, const int64_t *rows, const int64_t *cols, int64_t nrows,
                        int64_t nnz, const float *x, float *y, void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    PB_REQUIRE(nrows >= 0 && nnz >= 0, "spmv: negative size (nrows=%lld, nnz=%lld)", (long long)nrows, (long long)nnz);
    if (nrows == 0 || nnz == 0) return PB_OK;
    PB_REQUIRE(values && rows && cols && x && y, "spmv: null pointer");
    // CTA shape: 128 threads x 16 non-zeros measured best on B200 (the kernel is bound by the
    // L2 sector traffic of the x gathers, so the differences are a few percent)
    int cfg = 3;
    if (const char *env = getenv("PARPY_B200_SPMV_CFG")) cfg = atoi(env);
    const int threads = cfg == 2 ? 512 : cfg == 3 ? 128 : 256;
    const int per = cfg == 1 || cfg == 3 ? 16 : 8;
    const int chunk = threads * per;
    const long long blocks = (nnz + chunk - 1) / chunk;
    PB_REQUIRE(blocks <= 0x7fffffffLL && nrows <= 0x7fffffffLL, "spmv: matrix too large");
    void *ws = nullptr;
    int32_t rc = pb::workspace((size_t)blocks * sizeof(int), &ws, stream, 3);
    if (rc) return rc;
    int *first_row = static_cast<int *>(ws);
    spmv_first_rows<<<(unsigned)((nrows + 255) / 256), 256, 0, stream>>>(rows, nrows, first_row, chunk);
    PB_CUDA(cudaGetLastError());
    if (cfg == 1) spmv_chunks<256, 16><<<(unsigned)blocks, 256, 0, stream>>>(values, cols, rows, nrows, nnz, x, y, first_row);
    else if (cfg == 2) spmv_chunks<512, 8><<<(unsigned)blocks, 512, 0, stream>>>(values, cols, rows, nrows, nnz, x, y, first_row);
    else if (cfg == 3) spmv_chunks<128, 16><<<(unsigned)blocks, 128, 0, stream>>>(values, cols, rows, nrows, nnz, x, y, first_row);
    else spmv_chunks<256, 8><<<(unsigned)blocks, 256, 0, stream>>>(values, cols, rows, nrows, nnz, x, y, first_row);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

int32_t spmv_row(int64_t *cols, int64_t nrows, int64_t *rows, float *values, float *x, float *y) {
    PB_REQUIRE(nrows >= 0, "spmv_row: negative nrows");
    if (nrows == 0) return PB_OK;
    PB_REQUIRE(rows != nullptr, "spmv_row: null row pointer array");
    // The reference bakes the number of non-zeros into the generated code; here
    // it is read back from rows[nrows] (one 8-byte copy, synchronises stream 0).
    int64_t nnz = 0;
    PB_CUDA(cudaMemcpyAsync(&nnz, rows + nrows, sizeof(nnz), cudaMemcpyDeviceToHost, 0));
    PB_CUDA(cudaStreamSynchronize(0));
    return parpy_b200_spmv(values, rows, cols, nrows, nnz, x, y, nullptr);
}


int32_t parpy_b200_spmm(const float *values, const int64_t *rows, const int64_t *cols, int64_t nrows,
                        const float *B, int64_t ncols, float *C, void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    PB_REQUIRE(nrows >= 0 && ncols >= 0, "spmm: negative size");
    if (nrows == 0 || ncols == 0) return PB_OK;
    PB_REQUIRE(values && rows && cols && B && C, "spmm: null pointer");
    const bool vec = (ncols % 4 == 0) && pb::aligned16(B) && pb::aligned16(C);
    if (vec) {
        // lanes per column run: as many as the row of B needs, up to a full warp
        const int lpr = ncols >= 128 ? 32 : ncols > 32 ? 16 : ncols > 16 ? 8 : 4;
        const long long chunks = (ncols + 4 * lpr - 1) / (4 * lpr);
        const long long warps = nrows * chunks;
        const long long blocks = (warps + 7) / 8;
        PB_REQUIRE(blocks <= 0x7fffffffLL, "spmm: %lld rows x %lld columns is too large", (long long)nrows, (long long)ncols);
        if (lpr == 32) spmm_warp_rows<32><<<(unsigned)blocks, 256, 0, stream>>>(values, rows, cols, B, nrows, ncols, (int)chunks, C);
        else if (lpr == 16) spmm_warp_rows<16><<<(unsigned)blocks, 256, 0, stream>>>(values, rows, cols, B, nrows, ncols, (int)chunks, C);
        else if (lpr == 8) spmm_warp_rows<8><<<(unsigned)blocks, 256, 0, stream>>>(values, rows, cols, B, nrows, ncols, (int)chunks, C);
        else spmm_warp_rows<4><<<(unsigned)blocks, 256, 0, stream>>>(values, rows, cols, B, nrows, ncols, (int)chunks, C);
    } else {
        const long long chunks = (ncols + 127) / 128;
        PB_REQUIRE(nrows * chunks <= 0x7fffffffLL, "spmm: %lld rows x %lld columns is too large", (long long)nrows, (long long)ncols);
        spmm_rows_scalar<<<(unsigned)(nrows * chunks), 128, 0, stream>>>(values, rows, cols, B, ncols, (int)chunks, C);
    }
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

int32_t spmm_cell(int64_t *A_cols, int64_t A_nrows, int64_t *A_rows, float *A_values, int64_t B_ncols,
                  float *B_values, float *C) {
    return parpy_b200_spmm(A_values, A_rows, A_cols, A_nrows, B_values, B_ncols, C, nullptr);
}

int32_t parpy_b200_sddmm_decompress_csr(const int64_t *crows, int64_t *rows_out, int64_t N, void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    PB_REQUIRE(N >= 0, "sddmm_decompress_csr: negative N");
    if (N == 0) return PB_OK;
    PB_REQUIRE(crows && rows_out, "sddmm_decompress_csr: null pointer");
    const long long blocks = (N + 7) / 8;
    sddmm_decompress<<<(unsigned)blocks, 256, 0, stream>>>(crows, rows_out, N);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

int32_t parpy_sddmm_decompress_csr(int64_t *C_crows, int64_t *C_rows, int64_t N) {
    return parpy_b200_sddmm_decompress_csr(C_crows, C_rows, N, nullptr);
}

int32_t parpy_b200_sddmm_coo(const float *A, const float *B, const int64_t *rows, const int64_t *cols,
                             const float *cvalues, float *D, int64_t K, int64_t ncols, int64_t nnz,
                             double alpha, double beta, void *stream_) {
    PB_REQUIRE(nnz >= 0, "sddmm: negative nnz");
    return sddmm_common(A, B, nullptr, 0, rows, cols, cvalues, D, K, ncols, nnz, alpha, beta,
                        static_cast<cudaStream_t>(stream_));
}

int32_t parpy_b200_sddmm_csr(const float *A, const float *B, const int64_t *crows, int64_t *rows_out,
                             const int64_t *cols, const float *cvalues, float *D, int64_t N, int64_t K,
                             int64_t ncols, int64_t nnz, double alpha, double beta, void *stream_) {
    PB_REQUIRE(nnz >= 0 && N >= 0, "sddmm: negative size");
    if (nnz == 0) return parpy_b200_sddmm_decompress_csr(crows, rows_out, N, stream_);
    PB_REQUIRE(N == 0 || (crows && rows_out), "sddmm: null pointer");
    return sddmm_common(A, B, N > 0 ? crows : nullptr, N, rows_out, cols, cvalues, D, K, ncols, nnz, alpha, beta,
                        static_cast<cudaStream_t>(stream_));
}

}  // extern "C"
