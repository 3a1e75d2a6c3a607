/*
 * parpy_b200 — C ABI of the B200 (sm_100a) kernel library.
 *
 * Conventions, shared by every entry point and taken from the reference's
 * generated libraries (python/parpy/compile.py:140-182,
 * src/gpu/codegen.rs:529-549): return 0 on success, non-zero on failure; the
 * failure text is read with parpy_get_error_message(); pointers are DEVICE
 * pointers unless a comment says host; launches are asynchronous, nothing
 * synchronises unless stated; the caller owns every buffer it passes.
 *
 * Two families of symbols:
 *   1. Reference-shaped entries carry the name and flattened parameter list
 *      the reference's ctypes wrapper would call for the same Python function
 *      (dict arguments expanded in sorted-key order, 0-d values by value,
 *      Python int -> int64_t, Python float -> double). They run on the legacy
 *      default stream (stream 0), as the reference's generated code does.
 *   2. parpy_b200_* entries take the shapes the reference bakes in at JIT time
 *      as explicit arguments, plus a stream (a cudaStream_t passed as void*;
 *      NULL = legacy default stream) and option flags.
 *
 * Concurrency: entry points may be called from several host threads and on
 * several streams. Library-owned scratch is kept per (device, stream); calls on
 * one stream use it one after another in stream order.
 */
#ifndef PARPY_B200_H
#define PARPY_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- runtime library ---------------------------------------------------
 * Replaces python/parpy/native/parpy_cuda.cpp:3-39 as bound by
 * python/parpy/runtime.py:11-26. kind: 0 H2H, 1 H2D, 2 D2H, 3 D2D. */
void parpy_init(int64_t unused);
int32_t parpy_sync(void);
void *parpy_alloc_buffer(int64_t nbytes);
int32_t parpy_memcpy(void *dst, void *src, int64_t nbytes, int64_t kind);
int32_t parpy_memset(void *ptr, int64_t nbytes, int8_t value);
int32_t parpy_free_buffer(void *ptr);
/* Replaces python/parpy/native/parpy_cuda.h:22-25. Thread-local text of the
 * most recent failure reported by this library on the calling thread. */
const char *parpy_get_error_message(void);

/* Facts about the current device (host pointers, any may be NULL). */
int32_t parpy_b200_device_summary(int32_t *sm_count, int32_t *cc_major, int32_t *cc_minor);

/* ---- HMM forward (log space, k-mer x 16 duration layers) ------------------
 *
 * forward_kernel: the entry the reference generates for
 * benchmarks/forward.py:175-187 `forward_kernel(hmm, seqs, result, alpha1,
 * alpha2)`; hmm fields sorted (gamma, initial_prob, num_states, output_prob,
 * synthetic_248, trans1, trans2), seqs fields sorted (data, lens, maxlen,
 * num_instances). Layouts: initial_prob f32[num_states]; output_prob
 * f32[n_obs, K] with K = num_states/16; trans1 f32[K,4]; trans2 f32[16];
 * data int8/uint8 [num_instances, maxlen] with values < n_obs at t < lens[i];
 * lens i64[num_instances]; result f32[num_instances]. Log 0 is -inf in every
 * table; a sequence the model cannot produce scores NaN, the (-inf) - (-inf)
 * of the reference's final reduction (benchmarks/forward.py:168-173).
 * alpha1/alpha2 f32[num_instances, num_states] are the reference's scratch.
 * The resident kernel keeps alpha on chip and leaves them untouched (they may
 * be NULL); the streaming kernel (state spaces the resident kernel does not
 * cover) needs both.
 *
 * forward_kernel_scratch_first: same computation with the parameter order of
 * test/test_forward.py:83-160 `forward_kernel(hmm, seqs, alpha1, alpha2,
 * result)`.
 */
int32_t forward_kernel(float gamma, float *initial_prob, int64_t num_states,
                       float *output_prob, float synthetic_248, float *trans1,
                       float *trans2, int8_t *data, int64_t *lens, int64_t maxlen,
                       int64_t num_instances, float *result, float *alpha1,
                       float *alpha2);
int32_t forward_kernel_scratch_first(float gamma, float *initial_prob, int64_t num_states,
                                     float *output_prob, float synthetic_248,
                                     float *trans1, float *trans2, int8_t *data,
                                     int64_t *lens, int64_t maxlen,
                                     int64_t num_instances, float *alpha1,
                                     float *alpha2, float *result);

/* Option flags of parpy_b200_forward. Without SCALED, LOG_SPACE, FIVE_TERM,
 * STREAMING or WRITE_ALPHA the library picks the arithmetic by state space:
 * scaled for 4096 k-mers and more (6-mer and up), log space below that, where
 * the reference ships golden vectors that its own test compares at rtol 1e-5
 * with fp32 log-space results. forward_kernel and
 * forward_kernel_scratch_first follow the same rule. The environment variable
 * PARPY_B200_FWD_DEFAULT=log makes log space the rule everywhere. */
#define PARPY_B200_FWD_AUTO 0u
/* Force the streaming kernel: alpha ping-pongs through alpha1/alpha2 in global
 * memory, one launch per time step, the reference's five-term log-sum-exp in
 * the reference's operand order (what ParPy emits for `state: threads(N)`,
 * N > 1024; src/gpu/inter_block.rs:466-563). */
#define PARPY_B200_FWD_STREAMING 1u
/* Also store each sequence's final alpha vector where the reference leaves it:
 * alpha1 if lens[i] is odd, alpha2 otherwise (benchmarks/forward.py:163-165).
 * Needs both buffers. */
#define PARPY_B200_FWD_WRITE_ALPHA 2u
/* Resident kernel only: evaluate every state with the reference's five-term
 * log-sum-exp and operand order instead of the factored 4-way + 2-way form. */
#define PARPY_B200_FWD_FIVE_TERM 4u

/* Resident kernel, at least 1024 k-mers: evaluate the recurrence on probabilities
 * with a per-thread base-2 exponent (extended-range linear arithmetic) instead of
 * on log-probabilities. Mathematically the same quantity; rounding differs: this
 * form agrees with a float64 evaluation to ~1e-8 relative, while fp32 log space
 * (the reference's arithmetic) is itself 1e-6..1e-4 away from float64. States
 * more than about 2^-110 below the largest of their thread's 64 states count as log 0
 * (visible only in alpha written with WRITE_ALPHA). Its layer-0 exchange waits on
 * mbarriers with a bounded number of polls; a wait that runs out raises bit 2 of
 * the status word (parpy_b200_forward_status). */
#define PARPY_B200_FWD_SCALED 8u
/* Resident kernel: evaluate on log-probabilities (the factored log-sum-exp form)
 * whatever the library's default for the state space is. */
#define PARPY_B200_FWD_LOG_SPACE 16u

/* Same computation as forward_kernel with explicit options. `trans2` is a
 * DEVICE pointer to 16 floats like everywhere else. `stream` is a
 * cudaStream_t (NULL = stream 0). Replaces the host stub + kernels the
 * reference emits for benchmarks/forward.py:94-187. */
int32_t parpy_b200_forward(float gamma, const float *initial_prob, int64_t num_states,
                           const float *output_prob, float synthetic_248,
                           const float *trans1, const float *trans2,
                           const void *data, const int64_t *lens, int64_t maxlen,
                           int64_t num_instances, float *result, float *alpha1,
                           float *alpha2, uint32_t flags, void *stream);

/* parpy_b200_forward with the number of rows of output_prob (n_obs, 1..256) given,
 * so that observation bytes can be checked: a byte >= n_obs inside a sequence is
 * read as n_obs - 1 instead of indexing past the table, and bit 1 of the status
 * word (parpy_b200_forward_status) is raised. The reference's generated entry has
 * no such check and no n_obs parameter (an out-of-range byte reads out of bounds
 * there); forward_kernel and parpy_b200_forward keep that signature and accept
 * any byte value the caller guarantees to be valid. n_obs = 0: no check. */
int32_t parpy_b200_forward_ex(float gamma, const float *initial_prob, int64_t num_states,
                              const float *output_prob, int64_t n_obs, float synthetic_248,
                              const float *trans1, const float *trans2, const void *data,
                              const int64_t *lens, int64_t maxlen, int64_t num_instances,
                              float *result, float *alpha1, float *alpha2, uint32_t flags,
                              void *stream);

/* Describes the launch parpy_b200_forward would use for a state space on the
 * current device (host pointers; any may be NULL): kmers per thread, threads
 * per CTA, CTAs per cluster and resident clusters. Returns non-zero when only
 * the streaming kernel applies. */
int32_t parpy_b200_forward_plan(int64_t num_states, int64_t num_instances, int32_t *kmers_per_thread,
                                int32_t *threads_per_cta, int32_t *ctas_per_cluster,
                                int32_t *clusters);

/* The static schedule parpy_b200_forward builds for a batch of up to 4096
 * sequences on `clusters` (1..512) resident clusters: cluster_of[i] (device,
 * int32 [num_instances]) receives the cluster that scores sequence i. lens is
 * the device array the forward entry takes. Sequences are packed longest first
 * into the least loaded cluster, then the fullest cluster is repaired by single
 * exchanges, so the per-cluster sums of lengths (what a launch's duration
 * follows) differ by far less than one sequence. For inspection and tests. */
int32_t parpy_b200_forward_schedule(const int64_t *lens, int64_t num_instances, int64_t clusters,
                                    int32_t *cluster_of, void *stream);

/* Reads and clears the device status word of the current device (host call,
 * synchronises the device). Bit 0: a sequence length outside [1, maxlen] was
 * clamped. Bit 1: an observation byte >= n_obs was clamped (parpy_b200_forward_ex).
 * Bit 2: a bounded wait for another CTA's values ran out inside a kernel (scaled
 * kernel, st.async exchange); the results of the calls since the last read are
 * not valid. A caller that never reads the word still learns of bit 2: the
 * kernel also sets a word in pinned host memory (one per device, allocated by the
 * first forward call on it), and every later forward_kernel / parpy_b200_forward*
 * call on the device returns an error that says so, without launching, until the
 * status has been read. */
int32_t parpy_b200_forward_status(uint32_t *status);
/* Launches one 32-thread CTA that waits, with the scaled kernel's bounded wait,
 * on a barrier nothing completes; after `polls` (0..2^20) polls it gives up and
 * raises bit 2 of the forward status word. Touches no caller data. Lets a caller
 * (or a test) see the give-up path reach parpy_b200_forward_status without any
 * kernel being starved. No counterpart in the reference. */
int32_t parpy_b200_forward_wait_probe(int32_t polls, void *stream);

/* Forward pass for callers that must not trigger a device allocation.
 * No counterpart in the reference: its generated host stub allocates and frees
 * its temporaries with cudaMallocAsync on every call.
 *
 * Who needs this: code that calls the library from a context where cudaMalloc
 * is off limits — a stream-ordered pipeline that must not hit the implicit
 * device synchronisation an allocation can cause, a service whose device memory
 * is fully budgeted up front and which treats any late allocation as a fault, or
 * a plugin host that forbids allocation inside its execute callback.
 * parpy_b200_forward may grow the library's scheduling scratch with cudaMalloc
 * on its first call or when the batch grows; this entry never does. It computes
 * result[] with the resident log-space kernel (factored log-sum-exp, alpha kept on
 * chip: what parpy_b200_forward runs with PARPY_B200_FWD_LOG_SPACE, bit for bit)
 * with its scheduling scratch — the length-sorted sequence order and the work-
 * queue head — in a fixed device array compiled into the library, of
 * 4 * PARPY_B200_NOALLOC_MAX_SEQUENCES + 2560 bytes on every GPU that loads the
 * library, held until the process exits.
 *
 * Limits and rules:
 *  - num_instances above PARPY_B200_NOALLOC_MAX_SEQUENCES is rejected with an
 *    error text that names the limit; so are state spaces that only the
 *    streaming kernel covers (that kernel needs caller scratch).
 *  - It calls no cudaMalloc / cudaFree and no allocating library routine; the
 *    caller passes every input and output, as for parpy_b200_forward.
 *  - The first call on each device looks up the array's device address (one
 *    cudaGetSymbolAddress, with that device current). Make that first call
 *    before any stream capture is begun on the device.
 *  - (The array also holds a 2.5 KB table with each resident cluster's part of
 *    the schedule.)
 *  - All calls on a device share the one array, and it keeps the previous
 *    call's contents; each call rewrites the part it uses before reading it.
 *    Two calls whose kernels overlap on the GPU (different streams) race on it:
 *    serialise them on one stream or with events.
 */
#define PARPY_B200_NOALLOC_MAX_SEQUENCES 16384
int32_t parpy_b200_forward_noalloc(float gamma, const float *initial_prob, int64_t num_states,
                                   const float *output_prob, float synthetic_248,
                                   const float *trans1, const float *trans2, const void *data,
                                   const int64_t *lens, int64_t maxlen, int64_t num_instances,
                                   float *result, void *stream);

/* ---- row-wise softmax ---------------------------------------------------------
 * out[i,:] = exp(x[i,:] - max_i) / sum(exp(x[i,:] - max_i)) for fp32 x[N,M]
 * (row-major, contiguous). `softmax` is the entry the reference generates for
 * test/test_softmax.py:11-26 `softmax(x, N, M, out)`. */
int32_t softmax(float *x, int64_t N, int64_t M, float *out);
int32_t parpy_b200_softmax(const float *x, int64_t N, int64_t M, float *out, void *stream);

/* ---- reductions -------------------------------------------------------------------
 * out[i] = reduce(x[i, 0:M]) for fp32 x[N,M]; op: 0 sum, 1 prod, 2 max, 3 min
 * (neutral elements of src/utils/reduce.rs:75-88 for M = 0). Covers the
 * reference's sum_rows / prod_rows / max_rows / min_rows and *_axis functions
 * (test/test_reduce.py:12-54) and, with N = 1, the full reductions *_2d
 * (:56-70). The reference's generated entries take (x, out, N) only, with M
 * compiled in, so they have no fixed-signature twin here. */
int32_t parpy_b200_reduce_rows(int32_t op, const float *x, float *out, int64_t N, int64_t M,
                               void *stream);
/* Sum and max of one fp32 vector of n >= 1 elements in a single pass. */
int32_t parpy_b200_sum_max(const float *x, int64_t n, float *out_sum, float *out_max, void *stream);

/* ---- CSR SpMV -------------------------------------------------------------------------
 * y[row] += sum_i values[i] * x[cols[i]], i in [rows[row], rows[row+1]); int64
 * row pointers and column indices; y is accumulated into (the caller zeroes it).
 * `spmv_row` is the entry the reference generates for test/test_spmv.py:12-18
 * `spmv_row(A, x, y)` with A = {cols, nrows, rows, values} (sorted keys); it
 * reads the non-zero count back from rows[nrows], which synchronises stream 0. */
int32_t spmv_row(int64_t *cols, int64_t nrows, int64_t *rows, float *values, float *x, float *y);
int32_t parpy_b200_spmv(const float *values, const int64_t *rows, const int64_t *cols, int64_t nrows,
                        int64_t nnz, const float *x, float *y, void *stream);

/* ---- SDDMM -------------------------------------------------------------------------------
 * D[i] = alpha * dot(A[rows[i], 0:K], B[0:K, cols[i]]) + beta * cvalues[i] for
 * every non-zero i of the mask; A fp32 [N,K], B fp32 [K,ncols], int64 indices.
 * parpy_sddmm_decompress_csr: the entry generated for benchmarks/sddmm.py:21-26
 * (rows_out[i] = row of non-zero i). parpy_b200_sddmm_csr replaces
 * parpy_sddmm_csr_kernel (benchmarks/sddmm.py:28-41; it also fills rows_out, as
 * the reference's kernel does), parpy_b200_sddmm_coo replaces
 * parpy_sddmm_coo_kernel (:63-70). K and ncols are compiled into the
 * reference's generated entries, hence the explicit-shape signatures. */
int32_t parpy_sddmm_decompress_csr(int64_t *C_crows, int64_t *C_rows, int64_t N);
int32_t parpy_b200_sddmm_decompress_csr(const int64_t *crows, int64_t *rows_out, int64_t N, void *stream);
int32_t parpy_b200_sddmm_csr(const float *A, const float *B, const int64_t *crows, int64_t *rows_out,
                             const int64_t *cols, const float *cvalues, float *D, int64_t N, int64_t K,
                             int64_t ncols, int64_t nnz, double alpha, double beta, void *stream);
int32_t parpy_b200_sddmm_coo(const float *A, const float *B, const int64_t *rows, const int64_t *cols,
                             const float *cvalues, float *D, int64_t K, int64_t ncols, int64_t nnz,
                             double alpha, double beta, void *stream);

/* ---- row normalisation, exp + row sum, CSR SpMM ---------------------------------------------
 * normalize_rows: t[i,:] /= sum(t[i,:]) in place, the entry generated for
 * test/test_normalize.py:7-15 `normalize_rows(t, nrows, ncols)`.
 * parpy_b200_sum_exp_rows: x = exp(x) in place and out[r] = sum(x[r,:]) for fp32
 * x[nrows, ncols]; with nrows = N*M and ncols = K this is test/test_sync.py:59-69
 * `sum_exp_3d(x, N, M, out)` (whose generated entry has K compiled in).
 * spmm_cell: C[i,j] += sum_a A.values[a] * B.values[A.cols[a], j], the entry
 * generated for test/test_spmm.py:16-24 `spmm_cell(A, B, C)` with A = {cols, nrows,
 * rows, values} and B = {ncols, values} (sorted keys); C fp32 [nrows, ncols]. */
int32_t normalize_rows(float *t, int64_t nrows, int64_t ncols);
int32_t parpy_b200_normalize_rows(float *t, int64_t nrows, int64_t ncols, void *stream);
int32_t parpy_b200_sum_exp_rows(float *x, int64_t nrows, int64_t ncols, float *out, void *stream);
int32_t spmm_cell(int64_t *A_cols, int64_t A_nrows, int64_t *A_rows, float *A_values, int64_t B_ncols,
                  float *B_values, float *C);
int32_t parpy_b200_spmm(const float *values, const int64_t *rows, const int64_t *cols, int64_t nrows,
                        const float *B, int64_t ncols, float *C, void *stream);

/* ---- HMM input preparation on the device ------------------------------------------------
 * Replaces the host loops of the reference's loader (benchmarks/forward.py:20-87,
 * test/test_forward.py:11-78). prepare_tables: from the raw probability tables of
 * a model file (ObservationProbabilities [n_obs, 4^k], TransitionProbabilities
 * [4, 4^k], DurationProbabilities [16]; all float32 or all float64, device
 * memory) to output_prob [n_obs, K] (log, columns permuted by base reversal),
 * trans1 [K, 4] (log, transposed), trans2 [16] (log) and initial_prob [16 K]
 * (log(1/K) in layer 0, -inf elsewhere). pad_signals: from the concatenated int16
 * signals and their offsets [num_signals + 1] to the zero-padded int8 matrix
 * [num_signals, maxlen] and the int64 lengths. */
int32_t parpy_b200_hmm_prepare_tables(const void *obs_prob, const void *trans_prob, const void *dur_prob,
                                      int32_t is_f64, int32_t k, int64_t n_obs, float *output_prob,
                                      float *trans1, float *trans2, float *initial_prob, void *stream);
int32_t parpy_b200_hmm_pad_signals(const int16_t *flat, const int64_t *offsets, int64_t num_signals,
                                   int64_t maxlen, int8_t *data, int64_t *lens, void *stream);

/* ---- windowed Viterbi decoding ------------------------------------------------------------
 * Most likely state sequence of every observation sequence under the same model
 * tables as forward_kernel, with the semantics of the CUDA the reference ships
 * (benchmarks/7mer/hmm.cu:116-176,352-508,569-657, driven by
 * benchmarks/7mer/trellis.py:25-83 with batch_size 1024 and batch_overlap 128):
 * windows of batch_size steps advancing by batch_size - batch_overlap, each later
 * window restarted from the state decoded just before it. out is uint32
 * [num_instances, out_stride] (out_stride >= maxlen); row i holds lens[i] decoded
 * states (state = layer * K + kmer), the rest of the row is unspecified. The
 * reference's entry takes host pointers and returns malloc'ed host memory; this
 * one works on device memory. State spaces from 4^5 to 4^8 k-mers. */
int32_t parpy_b200_viterbi(float gamma, const float *initial_prob, int64_t num_states,
                           const float *output_prob, float synthetic_248, const float *trans1,
                           const float *trans2, const void *data, const int64_t *lens, int64_t maxlen,
                           int64_t num_instances, int64_t batch_size, int64_t batch_overlap,
                           uint32_t *out, int64_t out_stride, void *stream);
/* Same, with the number of rows of output_prob given (1..256; 0: no check): an
 * observation byte >= n_obs inside a sequence is read as n_obs - 1 and bit 1 of
 * the Viterbi status word is raised (the reference's CUDA indexes past the table). */
int32_t parpy_b200_viterbi_ex(float gamma, const float *initial_prob, int64_t num_states,
                              const float *output_prob, int64_t n_obs, float synthetic_248,
                              const float *trans1, const float *trans2, const void *data,
                              const int64_t *lens, int64_t maxlen, int64_t num_instances,
                              int64_t batch_size, int64_t batch_overlap, uint32_t *out, int64_t out_stride,
                              void *stream);
/* Reads and clears the Viterbi status word of the current device (host call,
 * synchronises the device). Bit 0: a bounded wait for another CTA's layer-0
 * values ran out, so the paths written by the calls since the last read are not
 * valid. Bit 1: an observation byte >= n_obs was clamped. No counterpart in the
 * reference, whose kernels cannot time out (one launch per step). */
int32_t parpy_b200_viterbi_status(uint32_t *status);
/* Launches one 32-thread CTA that waits, with the decoding kernel's bounded
 * wait, on a barrier nothing completes; after `polls` (0..2^20) polls it gives up
 * and raises bit 0 of the Viterbi status word. Touches no caller data. Lets a
 * caller (or a test) see the give-up path reach parpy_b200_viterbi_status
 * without any kernel being starved. */
int32_t parpy_b200_viterbi_wait_probe(int32_t polls, void *stream);

#ifdef __cplusplus
}
#endif

#endif /* PARPY_B200_H */
