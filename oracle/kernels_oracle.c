/*
 * CPU restatements of the reduction-heavy kernels that surround the HMM
 * forward path: softmax, row reductions, CSR SpMV and SDDMM.
 *
 * TEST INFRASTRUCTURE ONLY (see hmm_oracle.c). Parity pin: these follow the
 * reference's Python function bodies line by line; the reference checks the
 * same functions against torch.softmax (test/test_softmax.py:35-40), NumPy
 * (test/test_reduce.py:72-85), torch CSR matmul (test/test_spmv.py:46-53) and
 * torch.sparse.sampled_addmm (benchmarks/sddmm.py:18-19), and the CPU test
 * suite repeats exactly those comparisons for this file.
 */
#include <math.h>
#include <stdint.h>

/* test/test_softmax.py:11-26: m = max(x[i,:]); out = exp(x - m); s = sum(out); out /= s */
void oracle_softmax(const float *x, int64_t N, int64_t M, float *out) {
#pragma omp parallel for
    for (int64_t i = 0; i < N; ++i) {
        const float *r = x + i * M;
        float *o = out + i * M;
        float m = -INFINITY;
        for (int64_t j = 0; j < M; ++j) m = fmaxf(m, r[j]);
        float s = 0.0f;
        for (int64_t j = 0; j < M; ++j) {
            o[j] = expf(r[j] - m);
            s += o[j];
        }
        for (int64_t j = 0; j < M; ++j) o[j] = o[j] / s;
    }
}

/* test/test_reduce.py:12-54: out[i] = op(x[i,:]); op 0 sum, 1 prod, 2 max, 3 min.
 * Accumulated in double so that the oracle is order-independent; neutral
 * elements as in src/utils/reduce.rs:75-88. */
void oracle_reduce_rows(int32_t op, const float *x, float *out, int64_t N, int64_t M) {
#pragma omp parallel for
    for (int64_t i = 0; i < N; ++i) {
        const float *r = x + i * M;
        double acc = op == 0 ? 0.0 : op == 1 ? 1.0 : op == 2 ? -INFINITY : INFINITY;
        for (int64_t j = 0; j < M; ++j) {
            const double v = r[j];
            if (op == 0) acc += v;
            else if (op == 1) acc *= v;
            else if (op == 2) acc = v > acc ? v : acc;
            else acc = v < acc ? v : acc;
        }
        out[i] = (float)acc;
    }
}

/* test/test_spmv.py:12-18: y[row] += values[i] * x[cols[i]] in index order, fp32 */
void oracle_spmv(const float *values, const int64_t *rows, const int64_t *cols, int64_t nrows,
                 const float *x, float *y) {
#pragma omp parallel for schedule(dynamic, 1024)
    for (int64_t r = 0; r < nrows; ++r) {
        float acc = y[r];
        for (int64_t i = rows[r]; i < rows[r + 1]; ++i) acc += values[i] * x[cols[i]];
        y[r] = acc;
    }
}

/* benchmarks/sddmm.py:21-26 */
void oracle_sddmm_decompress(const int64_t *crows, int64_t *rows, int64_t N) {
    for (int64_t r = 0; r < N; ++r)
        for (int64_t i = crows[r]; i < crows[r + 1]; ++i) rows[i] = r;
}

/* benchmarks/sddmm.py:33-41,63-70: t = sum_k A[row,k] * B[k,col] (fp32, k order);
 * D[i] = alpha * t + beta * C[i] with the Python-float scalars in double. */
void oracle_sddmm(const float *A, const float *B, const int64_t *rows, const int64_t *cols,
                  const float *cvalues, float *D, int64_t K, int64_t ncols, int64_t nnz,
                  double alpha, double beta) {
#pragma omp parallel for
    for (int64_t i = 0; i < nnz; ++i) {
        const float *a = A + rows[i] * K;
        const int64_t c = cols[i];
        float t = 0.0f;
        for (int64_t k = 0; k < K; ++k) t += a[k] * B[k * ncols + c];
        D[i] = (float)(alpha * (double)t + beta * (double)cvalues[i]);
    }
}

/* test/test_normalize.py:7-15: s = sum(t[i,:]) (double accumulator, order-free); t[i,:] /= s */
void oracle_normalize_rows(float *t, int64_t nrows, int64_t ncols) {
#pragma omp parallel for
    for (int64_t i = 0; i < nrows; ++i) {
        float *r = t + i * ncols;
        double acc = 0.0;
        for (int64_t j = 0; j < ncols; ++j) acc += r[j];
        const float s = (float)acc;
        for (int64_t j = 0; j < ncols; ++j) r[j] = r[j] / s;
    }
}

/* test/test_sync.py:59-69 with rows = N*M: x = exp(x) in place; out[r] = sum(x[r,:]) */
void oracle_sum_exp_rows(float *x, int64_t nrows, int64_t ncols, float *out) {
#pragma omp parallel for
    for (int64_t i = 0; i < nrows; ++i) {
        float *r = x + i * ncols;
        double acc = 0.0;
        for (int64_t j = 0; j < ncols; ++j) {
            r[j] = expf(r[j]);
            acc += r[j];
        }
        out[i] = (float)acc;
    }
}

/* test/test_spmm.py:16-24: C[i,j] += values[a] * B[cols[a], j], non-zeros in index order */
void oracle_spmm(const float *values, const int64_t *rows, const int64_t *cols, int64_t nrows,
                 const float *B, int64_t ncols, float *C) {
#pragma omp parallel for
    for (int64_t i = 0; i < nrows; ++i)
        for (int64_t j = 0; j < ncols; ++j) {
            float acc = C[i * ncols + j];
            for (int64_t a = rows[i]; a < rows[i + 1]; ++a) acc += values[a] * B[cols[a] * ncols + j];
            C[i * ncols + j] = acc;
        }
}
