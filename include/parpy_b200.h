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
 * lens i64[num_instances]; result f32[num_instances].
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

/* Option flags of parpy_b200_forward. */
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

/* Describes the launch parpy_b200_forward would use for a state space on the
 * current device (host pointers; any may be NULL): kmers per thread, threads
 * per CTA, CTAs per cluster and resident clusters. Returns non-zero when only
 * the streaming kernel applies. */
int32_t parpy_b200_forward_plan(int64_t num_states, int64_t num_instances, int32_t *kmers_per_thread,
                                int32_t *threads_per_cta, int32_t *ctas_per_cluster,
                                int32_t *clusters);

/* Reads and clears the device status word of the current device (host call,
 * synchronises the device). Bit 0: a sequence length outside [1, maxlen] was
 * clamped. */
int32_t parpy_b200_forward_status(uint32_t *status);

#ifdef __cplusplus
}
#endif

#endif /* PARPY_B200_H */
