/*
 * CPU restatement of the windowed Viterbi decoder the reference ships as CUDA
 * for the same k-mer / duration HMM (benchmarks/7mer/hmm.cu).
 *
 * TEST INFRASTRUCTURE ONLY (see hmm_oracle.c). Parity pin: there are no golden
 * vectors for Viterbi in the reference; this file is checked on the GPU box
 * against the reference's own CUDA (benchmarks/5mer/hmm.cu compiled unmodified
 * into oracle/_ref) on the nanopore fixture, bit for bit.
 *
 * It follows the reference literally, quirks included:
 *   hmm.cu:116-176  viterbi_max_predecessor: candidates in the order j = 0..3
 *                   then the duration-chain predecessor, strict '>' (first wins)
 *   hmm.cu:352-376  viterbi_init / viterbi_init_batch (a window after the first
 *                   starts from the state decoded at t-1, everything else -inf)
 *   hmm.cu:378-412  viterbi_forward: chi ping-pong selected by k % 2; at
 *                   t+k == len the vector is copied once, past it zeta = identity
 *   hmm.cu:436-508  viterbi_backward: argmax over the FIRST chi buffer (which
 *                   holds step BATCH-2 when the window is full), then backtrack
 *   hmm.cu:569-657  host loop: windows of BATCH steps advancing by
 *                   BATCH - OVERLAP; later windows overwrite the overlap
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define V_LAYERS 16

/* Best predecessor of `state`; returns the predecessor index. When no candidate beats -inf
 * (the state cannot be reached at this step) the reference stores an uninitialised value
 * (hmm.cu:404-406: `state_t maxs;` is only assigned inside `if (p > *maxp)`); this
 * restatement and the CUDA kernel both take the first k-mer candidate there. The backward
 * pass can meet such a state only where the reference's own output is arbitrary: a sequence
 * of probability zero, or the step after the arg-max of a window that the reference reads
 * one step early. */
static inline uint32_t max_predecessor(const float *chi, int64_t N, int64_t state, float gamma,
                                       float syn, const float *trans1, const float *trans2,
                                       float *best) {
    const int64_t K = N / V_LAYERS;
    const int64_t layer = state / K, kmer = state % K;
    float maxp = -INFINITY;
    uint32_t maxs = (uint32_t)((state / 4) % (K / 4));
    for (int64_t x = 0; x < 4; ++x) {
        const int64_t pred = x * (K / 4) + (state / 4) % (K / 4);
        float p = trans1[(pred % K) * 4 + state % 4] + trans2[layer];
        p = p + chi[pred];
        if (p > maxp) { maxs = (uint32_t)pred; maxp = p; }
    }
    int64_t pred;
    float p;
    if (layer == 15) { pred = state; p = gamma; }
    else if (layer == 14) { pred = (layer + 1) * K + kmer; p = syn; }
    else { pred = (layer + 1) * K + kmer; p = 0.0f; }
    p = p + chi[pred];
    if (p > maxp) { maxs = (uint32_t)pred; maxp = p; }
    *best = maxp;
    return maxs;
}

/*
 * obs: uint8 [B, maxlen] (entries at t >= lens[i] unused); out: uint32 [B, out_stride],
 * positions [0, lens[i]) of every row are defined. Returns 0, or 1 on bad arguments.
 */
int oracle_viterbi(float gamma, const float *initial_prob, int64_t num_states,
                   const float *output_prob, float synthetic, const float *trans1,
                   const float *trans2, const uint8_t *obs, const int64_t *lens, int64_t maxlen,
                   int64_t num_instances, int64_t batch_size, int64_t batch_overlap, uint32_t *out,
                   int64_t out_stride) {
    const int64_t N = num_states, K = N / V_LAYERS;
    if (N < 64 || N % 64 || batch_size < 2 || batch_overlap < 0 || batch_overlap >= batch_size) return 1;
    const int64_t bos = batch_size - batch_overlap;
    int failed = 0;
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t inst = 0; inst < num_instances; ++inst) {
        const int64_t len = lens[inst];
        float *chi1 = (float *)malloc(sizeof(float) * (size_t)N);
        float *chi2 = (float *)malloc(sizeof(float) * (size_t)N);
        uint32_t *zeta = (uint32_t *)malloc(sizeof(uint32_t) * (size_t)N * (size_t)(batch_size - 1));
        if (!chi1 || !chi2 || !zeta) { failed = 1; free(chi1); free(chi2); free(zeta); continue; }
        const uint8_t *o = obs + inst * maxlen;
        uint32_t *res = out + inst * out_stride;
        const int64_t nbatches = (len + bos - 1) / bos;
        for (int64_t b = 0; b < nbatches; ++b) {
            const int64_t t = b * bos;
            if (b == 0) {
                for (int64_t s = 0; s < N; ++s) chi1[s] = initial_prob[s] + output_prob[(int64_t)o[0] * K + s % K];
            } else if (t < len) {
                const uint32_t last = res[t - 1];
                for (int64_t s = 0; s < N; ++s)
                    chi1[s] = ((uint32_t)s == last) ? output_prob[(int64_t)o[t] * K + s % K] : -INFINITY;
            }
            for (int64_t k = 1; k < batch_size; ++k) {
                float *prev = (k % 2 == 0) ? chi2 : chi1, *curr = (k % 2 == 0) ? chi1 : chi2;
                uint32_t *z = zeta + (size_t)(k - 1) * (size_t)N;
                if (t + k < len) {
                    const float *row = output_prob + (int64_t)o[t + k] * K;
                    for (int64_t s = 0; s < N; ++s) {
                        float best;
                        z[s] = max_predecessor(prev, N, s, gamma, synthetic, trans1, trans2, &best);
                        curr[s] = best + row[s % K];
                    }
                } else if (t + k == len) {
                    memcpy(curr, prev, sizeof(float) * (size_t)N);
                    for (int64_t s = 0; s < N; ++s) z[s] = (uint32_t)s;
                } else {
                    for (int64_t s = 0; s < N; ++s) z[s] = (uint32_t)s;
                }
            }
            /* argmax over the first buffer, lowest index among equal maxima */
            uint32_t cur = 0;
            float m = chi1[0];
            for (int64_t s = 1; s < N; ++s) if (chi1[s] > m) { m = chi1[s]; cur = (uint32_t)s; }
            for (int64_t j = batch_size - 1; j >= 0; --j) {
                if (j < batch_size - 1) {
                    cur = zeta[(size_t)j * (size_t)N + cur];
                }
                if (t + j < out_stride) res[t + j] = cur;
            }
        }
        free(chi1); free(chi2); free(zeta);
    }
    return failed;
}
