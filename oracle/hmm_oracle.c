/*
 * CPU restatement of the reference's log-space HMM forward algorithm.
 *
 * TEST INFRASTRUCTURE ONLY: this file is the checker the CUDA kernels are
 * compared against. Nothing in the shipped package may call it; only the
 * tests, the smoke check and the CPU-baseline leg of the benchmark do.
 *
 * Parity pin: checked against the reference's golden vectors
 * test/data/3mer-expected.txt and test/data/5mer-expected.txt (inputs
 * test/data/{3mer,5mer}-model.hdf5 + signals.hdf5) by the CPU test suite.
 *
 * Every function cites the reference lines it follows; the arithmetic keeps
 * the reference's operand order so that fp32 rounding matches:
 *   benchmarks/forward.py:94-101   forward_init_inst
 *   benchmarks/forward.py:103-158  forward_step_inst
 *   benchmarks/forward.py:160-173  forward_lse_inst
 *   benchmarks/forward.py:175-187  forward_kernel (loop nest)
 *   test/test_forward.py:83-160    same maths, scratch-first argument order
 *
 * State numbering: state = layer * K + kmer, K = num_states / 16, layer in
 * 0..15 (remaining-duration counter), kmer read as a big-endian base-4 number.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_LAYERS 16

static inline float f32_max(float a, float b) {
    /* fmaxf semantics: a NaN operand yields the other operand. This is what
     * turns the NaN of (-inf) - (-inf) back into -inf at forward.py:156. */
    return fmaxf(a, b);
}

/* One time step for one sequence; forward.py:112-158 for every state. States
 * of a step do not depend on one another, so `split_states` may hand them to
 * several threads (used when a batch has fewer sequences than threads); the
 * values do not depend on the split. */
static void step_states(float gamma, int64_t N, const float *output_row,
                        float synthetic_248, const float *trans1,
                        const float *trans2, const float *src, float *dst,
                        int split_states) {
    const int64_t K = N / ORACLE_LAYERS;  /* num_kmers, forward.py:115 */
    const int64_t Q = N / 64;             /* num_states // 64, forward.py:117 */
#pragma omp parallel for schedule(static) if (split_states)
    for (int64_t state = 0; state < N; ++state) {
        const int64_t kmer = state % K;
        const int64_t layer = state / K;
        const int64_t low = (state / 4) % Q;
        const int64_t pred1 = low;              /* forward.py:117 */
        const int64_t pred2 = Q + low;          /* forward.py:118 */
        const int64_t pred3 = 2 * N / 64 + low; /* forward.py:119 */
        const int64_t pred4 = 3 * N / 64 + low; /* forward.py:120 */
        const float t11 = trans1[(pred1 % K) * 4 + state % 4];
        const float t12 = trans1[(pred2 % K) * 4 + state % 4];
        const float t13 = trans1[(pred3 % K) * 4 + state % 4];
        const float t14 = trans1[(pred4 % K) * 4 + state % 4];
        const float t2 = trans2[layer];
        const float p1 = (t11 + t2) + src[pred1]; /* forward.py:126-129 */
        const float p2 = (t12 + t2) + src[pred2];
        const float p3 = (t13 + t2) + src[pred3];
        const float p4 = (t14 + t2) + src[pred4];
        int64_t pred5;
        float p5;
        if (layer == 15) { /* forward.py:133-141 */
            pred5 = state;
            p5 = gamma;
        } else if (layer == 14) {
            pred5 = (layer + 1) * K + kmer;
            p5 = synthetic_248;
        } else {
            pred5 = (layer + 1) * K + kmer;
            p5 = 0.0f;
        }
        p5 = p5 + src[pred5]; /* forward.py:142 */
        float maxp = f32_max(p1, p2); /* forward.py:145-148 */
        maxp = f32_max(maxp, p3);
        maxp = f32_max(maxp, p4);
        maxp = f32_max(maxp, p5);
        float lsexp = maxp + logf(expf(p1 - maxp) + expf(p2 - maxp) +
                                  expf(p3 - maxp) + expf(p4 - maxp) +
                                  expf(p5 - maxp)); /* forward.py:149-155 */
        lsexp = f32_max(lsexp, -INFINITY);          /* forward.py:156 */
        dst[state] = lsexp + output_row[kmer];      /* forward.py:158 */
    }
}

/*
 * forward_kernel restated. `data` holds one observation byte per (sequence,
 * time); values are < 101 so int8 and uint8 views agree. Entries at
 * t >= lens[i] are never read (the reference loads them but never uses them).
 * `alpha_final`, when not NULL, receives the alpha vector after the last step
 * of each sequence ([num_instances, num_states]); the reference leaves it in
 * alpha1 when lens[i] is odd and in alpha2 otherwise (forward.py:163-165).
 * Returns 0, or 1 on a bad argument / allocation failure.
 */
int oracle_forward(float gamma, const float *initial_prob, int64_t num_states,
                   const float *output_prob, float synthetic_248,
                   const float *trans1, const float *trans2,
                   const uint8_t *data, const int64_t *lens, int64_t maxlen,
                   int64_t num_instances, float *result, float *alpha_final,
                   int32_t num_threads) {
    const int64_t N = num_states;
    if (N <= 0 || N % 64 != 0 || maxlen < 1 || num_instances < 0) return 1;
    const int64_t K = N / ORACLE_LAYERS;
    int failed = 0;
#ifdef _OPENMP
    if (num_threads > 0) omp_set_num_threads(num_threads);
#else
    (void)num_threads;
#endif
    /* Sequences are independent: one thread each. A batch with fewer sequences
     * than threads splits the states of every step over the threads instead. */
    int split_states = 0;
#ifdef _OPENMP
    split_states = num_instances < omp_get_max_threads() && N >= 4096;
#endif
#pragma omp parallel for schedule(dynamic, 1) if (!split_states)
    for (int64_t inst = 0; inst < num_instances; ++inst) {
        float *a1 = (float *)malloc(sizeof(float) * (size_t)N);
        float *a2 = (float *)malloc(sizeof(float) * (size_t)N);
        if (!a1 || !a2) {
            failed = 1;
            free(a1);
            free(a2);
            continue;
        }
        const uint8_t *obs = data + inst * maxlen;
        int64_t len = lens[inst];
        if (len > maxlen) len = maxlen;
        /* forward.py:96-101 */
        const float *row0 = output_prob + (int64_t)obs[0] * K;
        for (int64_t s = 0; s < N; ++s) a1[s] = initial_prob[s] + row0[s % K];
        memset(a2, 0, sizeof(float) * (size_t)N); /* torch.zeros, forward.py:192 */
        /* forward.py:183-184; steps with t >= len write nothing (:113) */
        for (int64_t t = 1; t < len; ++t) {
            const float *src = (t & 1) ? a1 : a2; /* forward.py:105-109 */
            float *dst = (t & 1) ? a2 : a1;
            step_states(gamma, N, output_prob + (int64_t)obs[t] * K,
                        synthetic_248, trans1, trans2, src, dst, split_states);
        }
        /* forward.py:163-173 */
        const float *alpha = (len & 1) ? a1 : a2;
        float maxp = -INFINITY;
        for (int64_t s = 0; s < N; ++s) maxp = f32_max(maxp, alpha[s]);
        /* parpy.operators.sum is a parallel (tree) reduction on the GPU and a
         * pairwise sum in NumPy; a sequential float accumulator would instead drop
         * small terms once it has grown (N reaches 2^20). The float terms are
         * therefore accumulated in double and rounded once. */
        double acc = 0.0;
        for (int64_t s = 0; s < N; ++s) acc += (double)expf(alpha[s] - maxp);
        const float psum = (float)acc;
        result[inst] = maxp + logf(psum);
        if (alpha_final)
            memcpy(alpha_final + inst * N, alpha, sizeof(float) * (size_t)N);
        free(a1);
        free(a2);
    }
    return failed;
}

int32_t oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
