// HMM forward algorithm over a k-mer x 16-duration-layer state space for
// sm_100a. Implementations behind one entry point:
//
//  * resident kernels — a persistent thread-block cluster owns one sequence at
//    a time; every thread keeps the 16 duration layers of its k-mers on chip
//    (registers, tensor memory) for the whole sequence, only layer 0 (K floats)
//    is exchanged per time step through distributed shared memory. In log
//    space (the reference's arithmetic: hmm_forward_packed and its twins, one
//    split barrier.cluster arrive/wait per step hidden behind layers 1..15) or
//    on probabilities with a per-thread base-2 exponent (hmm_forward_scaled*:
//    two multiply-adds per state, st.async + mbarrier exchange), which is what
//    a call without options runs for 4096 k-mers and more.
//  * streaming kernel — alpha ping-pongs through caller scratch in global
//    memory, one launch per time step, the reference's literal five-term
//    log-sum-exp. Covers state spaces the resident kernel cannot hold and is
//    the structural twin of what the reference's compiler emits.
//
// The recurrence (benchmarks/forward.py:103-158), with state = d*K + s:
//   alpha'[d,s] = LSE( trans1[p_j, s%4] + trans2[d] + alpha[0,p_j]  (j=0..3),
//                      c[d] + alpha[min(d+1,15), s] ) + output_prob[o_t, s]
//   p_j = j*K/4 + s/4,  c[15] = gamma, c[14] = synthetic_248, else 0.
// The four k-mer terms do not depend on d apart from the additive trans2[d],
// so the resident kernel evaluates q[s] = LSE_j(trans1[p_j,s%4] + alpha[0,p_j])
// once per k-mer and alpha'[d,s] = LSE2(trans2[d] + q[s], c[d] + alpha[d+1,s]).
#include <cooperative_groups.h>

#include <algorithm>
#include <cstring>
#include <type_traits>
#include <mutex>

#include "../../include/parpy_b200.h"
#include "common.cuh"
#include "cluster.cuh"
#include "tmem.cuh"

namespace {

constexpr int kLayers = 16;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr int kSortLimit = 4096;  // batches up to this size get a static, balanced schedule
constexpr int kMaxBins = 512;     // resident clusters a static schedule is built for
constexpr int kSegInts = kMaxBins + 64;   // ints reserved for the per-cluster segment table

// Device status word. Bit 0: a sequence length outside [1, maxlen] was clamped.
// Bit 1: an observation >= n_obs inside a sequence was clamped to n_obs - 1.
// Bit 2: a bounded wait of the st.async exchange ran out; that call's results are not valid.
__device__ unsigned g_status;

// Fixed scheduling scratch of parpy_b200_forward_noalloc: the sequence order
// (one int per sequence), the work-queue head and the per-cluster segment table.
// It is part of the loaded module, so every GPU that loads the library holds
// these bytes until the process exits. In host code this name is only a handle
// for the symbol, not a device address; host code obtains the address with
// cudaGetSymbolAddress.
constexpr int kNoAllocMaxSequences = PARPY_B200_NOALLOC_MAX_SEQUENCES;
constexpr size_t kNoAllocOrderBytes = size_t(kNoAllocMaxSequences) * sizeof(int);
constexpr size_t kSchedTailBytes = 256 + size_t(kSegInts) * sizeof(int);   // queue head + segment table
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocOrderBytes + kSchedTailBytes];

struct FwdParams {
    const float *initial_prob;  // [16*K]
    const float *output_prob;   // [n_obs, K]
    const float *trans1;        // [K, 4]
    const float *trans2;        // [16]
    const uint8_t *data;        // [B, maxlen]
    const int64_t *lens;        // [B]
    float *result;              // [B]
    float *alpha1;              // optional [B, 16*K]
    float *alpha2;              // optional [B, 16*K]
    const int *order;           // [B] sequence ids: grouped by cluster (static schedule) or longest first
    const int *seg;             // [clusters + 1] bounds of each cluster's part of `order`; NULL: work queue
    int *counter;               // work-queue head (dynamic schedule only)
    long long maxlen;
    int B;
    int K;
    int obs_max;                // n_obs - 1: observations above it are clamped and flagged (255: unknown)
    int write_alpha;
    float gamma;
    float synthetic;
    float gamma_lin;            // exp(gamma), exp(synthetic_248): scaled kernel only
    float synthetic_lin;
    unsigned *host_flag;        // pinned host word set when a bounded wait runs out (NULL: none)
    const float *output_lin;    // exp(output_prob) in library scratch: scaled tensor-memory kernel only (NULL: none)
};

// A bounded wait ran out: status bit 2 on the device and, where the library has one, a word in
// pinned host memory that the next forward call on the device checks before it launches anything.
__device__ __forceinline__ void flag_wait_timeout(unsigned *host_flag) {
    atomicOr(&g_status, 4u);
    if (host_flag != nullptr) {
        *reinterpret_cast<volatile unsigned *>(host_flag) = 1u;
        __threadfence_system();
    }
}

// Observation byte t of a sequence, kept inside the emission table: a value past the last
// row is clamped and remembered in `bad` (no branch in the time loop; the caller raises the
// status bit once per sequence with flag_bad_observation).
__device__ __forceinline__ int obs_at(const FwdParams &p, const uint8_t *obs, int t, bool &bad) {
    const int o = obs[t];
    bad = bad || o > p.obs_max;
    return min(o, p.obs_max);
}
__device__ __forceinline__ void flag_bad_observation(bool bad, bool reporter) {
    if (bad && reporter) atomicOr(&g_status, 2u);
}

// ---- log-sum-exp building blocks -------------------------------------------
// exp and log are the fast intrinsics the reference's CUDA backend prints for
// fp32 (src/cuda/pprint.rs:185-191): ex2.approx(x*log2e), lg2.approx(x)*ln2.
__device__ __forceinline__ float fast_exp(float x) { return pb::ex2_approx(x * kLog2e); }
__device__ __forceinline__ float fast_log(float x) { return pb::lg2_approx(x) * kLn2; }

// log(exp(u) + exp(v)); NaN from (-inf)-(-inf) is folded back to -inf the way
// the reference's trailing max(lsexp, -inf) does (benchmarks/forward.py:156).
__device__ __forceinline__ float lse2(float u, float v) {
    const float mx = fmaxf(u, v);
    const float d = u - v;
    const float ex = pb::ex2_approx(-fabsf(d) * kLog2e);
    const float l = pb::lg2_approx(1.0f + ex);
    return fmaxf(fmaf(l, kLn2, mx), -INFINITY);
}

// 2^t for t <= 0 without the MUFU unit: round-to-nearest split t = n + f with
// the magic-number trick (n integer, f in [-0.5, 0.5]), a degree-5 minimax
// polynomial for 2^f (max relative error 2.2e-7, on par with ex2.approx), and n
// added straight into the exponent field. The forward kernels are bound by the
// MUFU pipe; evaluating a fixed subset of the exponentials on the FMA pipe
// instead balances the two.
__device__ __forceinline__ float ex2_poly(float t) {
    t = fmaxf(t, -126.0f);              // also maps NaN to -126 (result ~0)
    const float magic = 12582912.0f;    // 1.5 * 2^23
    const float r = t + magic;
    const float n = r - magic;
    const float f = t - n;
    float p = 0.001327647129073739f;
    p = fmaf(p, f, 0.009675540961325169f);
    p = fmaf(p, f, 0.05550713092088699f);
    p = fmaf(p, f, 0.24022120237350464f);
    p = fmaf(p, f, 0.6931469440460205f);
    p = fmaf(p, f, 1.0000001192092896f);
    return __int_as_float(__float_as_int(p) + (__float_as_int(r) << 23));
}

// `poly` is a compile-time constant at every call site once the layer loops are
// unrolled, so the unused branch disappears.
__device__ __forceinline__ float lse2_sel(bool poly, float u, float v) {
    const float mx = fmaxf(u, v);
    const float t = -fabsf(u - v) * kLog2e;
    const float ex = poly ? ex2_poly(t) : pb::ex2_approx(t);
    const float l = pb::lg2_approx(1.0f + ex);
    return fmaxf(fmaf(l, kLn2, mx), -INFINITY);
}

__device__ __forceinline__ float lse4(float p0, float p1, float p2, float p3) {
    const float m = fmaxf(fmaxf(p0, p1), fmaxf(p2, p3));
    const float s = fast_exp(p0 - m) + fast_exp(p1 - m) + fast_exp(p2 - m) + fast_exp(p3 - m);
    return fmaxf(fmaf(pb::lg2_approx(s), kLn2, m), -INFINITY);
}

// The reference's five-term form, operand order as written there
// (benchmarks/forward.py:145-156).
__device__ __forceinline__ float lse5_reference(float p1, float p2, float p3, float p4, float p5) {
    float maxp = fmaxf(p1, p2);
    maxp = fmaxf(maxp, p3);
    maxp = fmaxf(maxp, p4);
    maxp = fmaxf(maxp, p5);
    float lsexp = maxp + fast_log(fast_exp(p1 - maxp) + fast_exp(p2 - maxp) + fast_exp(p3 - maxp) +
                                  fast_exp(p4 - maxp) + fast_exp(p5 - maxp));
    return fmaxf(lsexp, -INFINITY);
}

// ---- scheduling prologue ----------------------------------------------------
// One CTA decides, before the forward kernel starts, which resident cluster scores
// which sequences. A cluster's time is the sum of the lengths it is given and the
// launch lasts as long as the busiest cluster, so the lengths are packed into C bins
// of nearly equal sums: longest-first greedy packing (each sequence to the least
// loaded bin), then repeated repair of the fullest bin by the best single exchange
// (or move) of one of its sequences with another bin. Greedy packing alone, which is
// also what a longest-first work queue produces, leaves the bins up to one shortest
// sequence apart: 2 % of the run for 500 sequences of 1000..4000 steps on 33 clusters;
// the repair brings that below 0.1 %. Output: `order` holds the sequence ids grouped
// by bin (longest first inside a bin) and seg[c] .. seg[c+1] delimit bin c.
// Batches above kSortLimit fall back to a work queue in input order (seg unused).
// Smallest 64-bit key of the warp: the smallest high word, then the smallest low word among the
// lanes that hold it (two hardware reductions instead of five rounds of 64-bit shuffles).
__device__ __forceinline__ unsigned long long warp_min_u64(unsigned long long v) {
    const unsigned hi = static_cast<unsigned>(v >> 32);
    const unsigned mh = __reduce_min_sync(0xffffffffu, hi);
    const unsigned ml = __reduce_min_sync(0xffffffffu, hi == mh ? static_cast<unsigned>(v) : 0xffffffffu);
    return (static_cast<unsigned long long>(mh) << 32) | ml;
}

__global__ void __launch_bounds__(1024, 1)
hmm_schedule(const int64_t *__restrict__ lens, int B, int C, int *__restrict__ order,
             int *__restrict__ counter, int *__restrict__ seg, int *__restrict__ cluster_of, int max_rounds) {
    extern __shared__ int s_dyn[];                       // [B] lengths by rank, then two u16 arrays
    __shared__ long long s_load[kMaxBins];
    __shared__ int s_cnt[kMaxBins + 1];
    __shared__ unsigned short s_alist[256];
    __shared__ int s_alen[256];                           // lengths of the listed members
    __shared__ unsigned char s_chunk[kSortLimit / 32];   // members of the fullest bin per chunk of 32 ranks
    __shared__ unsigned long long s_red[32];
    __shared__ int s_a, s_na, s_done;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) *counter = 0;
    if (C <= 0) {   // no static schedule asked for: work queue in input order
        for (int i = tid; i < B; i += blockDim.x) order[i] = i;
        return;
    }
    int *s_len = s_dyn;                                                          // length of the item of rank r
    unsigned short *s_id = reinterpret_cast<unsigned short *>(s_dyn + B);        // its sequence id
    unsigned short *s_bin = s_id + B;                                            // its bin
    constexpr int kLenCap = 1 << 26;    // keeps every sum below 2^38 (64-bit keys below)
    constexpr int kPerThread = kSortLimit / 1024;

    // rank by counting: longest first, lower id first among equal lengths
    for (int i = tid; i < B; i += blockDim.x) {
        const long long l = lens[i];
        s_len[i] = l > kLenCap ? kLenCap : (l < 1 ? 1 : static_cast<int>(l));
    }
    __syncthreads();
    int my_len[kPerThread], my_rank[kPerThread];
#pragma unroll
    for (int k = 0; k < kPerThread; ++k) {
        const int i = tid + k * 1024;
        my_len[k] = 0;
        my_rank[k] = -1;
        if (i < B) {
            const int li = s_len[i];
            int rank = 0;
            for (int j = 0; j < B; ++j) {
                const int lj = s_len[j];
                rank += (lj > li) || (lj == li && j < i);
            }
            my_len[k] = li;
            my_rank[k] = rank;
        }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kPerThread; ++k) {
        if (my_rank[k] >= 0) {
            s_len[my_rank[k]] = my_len[k];
            s_id[my_rank[k]] = static_cast<unsigned short>(tid + k * 1024);
        }
    }
    for (int c = tid; c < C; c += blockDim.x) s_load[c] = 0;
    __syncthreads();

    // greedy packing, one warp: item r to the least loaded bin (lowest bin among equals). Up to 64 bins
    // (two per lane) the sums stay in registers; the general path keeps them in shared memory.
    if (warp == 0 && C <= 64) {
        long long l0 = 0, l1 = 0;   // sums of bins lane and lane + 32
        for (int r = 0; r < B; ++r) {
            int bin;
            if (r < C) {
                bin = r;
            } else {
                const unsigned long long k0 = lane < C ? ((static_cast<unsigned long long>(l0) << 10) | unsigned(lane)) : ~0ull;
                const unsigned long long k1 = lane + 32 < C ? ((static_cast<unsigned long long>(l1) << 10) | unsigned(lane + 32)) : ~0ull;
                bin = static_cast<int>(warp_min_u64(k0 < k1 ? k0 : k1) & 1023u);
            }
            const int len = s_len[r];
            if (bin == lane) l0 += len;
            if (bin == lane + 32) l1 += len;
            if (lane == 0) s_bin[r] = static_cast<unsigned short>(bin);
        }
        if (lane < C) s_load[lane] = l0;
        if (lane + 32 < C) s_load[lane + 32] = l1;
    } else if (warp == 0) {
        for (int r = 0; r < B; ++r) {
            int bin;
            if (r < C) {
                bin = r;
            } else {
                unsigned long long key = ~0ull;
                for (int c = lane; c < C; c += 32) {
                    const unsigned long long k = (static_cast<unsigned long long>(s_load[c]) << 10) | unsigned(c);
                    key = k < key ? k : key;
                }
                bin = static_cast<int>(warp_min_u64(key) & 1023u);
            }
            if (lane == 0) {
                s_load[bin] += s_len[r];
                s_bin[r] = static_cast<unsigned short>(bin);
            }
            __syncwarp();
        }
    }
    __syncthreads();

    // repair of the fullest bin, for a bounded number of rounds
    long long total = 0;
    if (C > 1 && B > C) {
        for (int c = 0; c < C; ++c) total += s_load[c];
    }
    int budget = 0;
    if (C > 1 && B > C) {
        long long top = 0;
        for (int c = 0; c < C; ++c) top = s_load[c] > top ? s_load[c] : top;
        // a round costs about as much as a time step of a small model: spend at most an eighth of
        // the steps that perfect balance could save
        const long long gap = top - total / C;
        budget = static_cast<int>(gap / 8 < max_rounds ? gap / 8 : max_rounds);
    }
    for (int it = 0; it < budget; ++it) {
        if (warp == 0) {
            // fullest bin (lowest index among equals) and its longest members, in rank order
            unsigned long long key = ~0ull;
            for (int c = lane; c < C; c += 32) {
                const unsigned long long k = ((~static_cast<unsigned long long>(s_load[c]) & ((1ull << 40) - 1)) << 10) | unsigned(c);
                key = k < key ? k : key;
            }
            const int a = static_cast<int>(warp_min_u64(key) & 1023u);
            if (lane == 0) {
                s_a = a;
                s_done = 0;
            }
        }
        __syncthreads();
        const int a = s_a;
        // its members in rank order (the first 256): every warp lists those of its own chunks of 32
        // ranks, a warp's position in the list is the number of members in the chunks before its own
        for (int c0 = warp; c0 * 32 < B; c0 += 32) {
            const int r = c0 * 32 + lane;
            const unsigned m = __ballot_sync(0xffffffffu, r < B && s_bin[r] == a);
            if (lane == 0) s_chunk[c0] = static_cast<unsigned char>(__popc(m));
        }
        __syncthreads();
        for (int c0 = warp; c0 * 32 < B; c0 += 32) {
            int before = 0;
            for (int c = lane; c < c0; c += 32) before += s_chunk[c];
            before = __reduce_add_sync(0xffffffffu, before);
            const int r = c0 * 32 + lane;
            const bool in = r < B && s_bin[r] == a;
            const unsigned m = __ballot_sync(0xffffffffu, in);
            const int pos = before + __popc(m & ((1u << lane) - 1u));
            if (in && pos < 256) {
                s_alist[pos] = static_cast<unsigned short>(r);
                s_alen[pos] = s_len[r];
            }
            if (c0 == (B - 1) / 32 && lane == 0) {
                const int n = before + __popc(m);
                s_na = n < 256 ? n : 256;
            }
        }
        __syncthreads();
        const int na = s_na;
        const long long La = s_load[a];
        // candidates: exchange x (fullest bin) with a shorter y of bin b, or move x to bin b;
        // key = new larger sum of the two bins, then a deterministic tie-break
        unsigned long long best = ~0ull;
        if (total < (1ll << 30)) {
            // every sum fits 31 bits: the same search on 32-bit values, the key kept as (sum, tie-break)
            const int La32 = static_cast<int>(La);
            unsigned bm = 0xffffffffu, blo = 0xffffffffu;
            for (int y = tid; y < B; y += blockDim.x) {
                const int b = s_bin[y];
                const int Lb = static_cast<int>(s_load[b]);
                const int d = La32 - Lb;
                if (b == a || d < 2) continue;
                const int ly = s_len[y];
                for (int i = 0; i < na; ++i) {
                    const int dd = s_alen[i] - ly;
                    if (dd > 0 && dd < d) {
                        const unsigned m = static_cast<unsigned>(max(La32 - dd, Lb + dd));
                        const unsigned lo = (unsigned(y) << 12) | unsigned(s_alist[i]);
                        if (m < bm || (m == bm && lo < blo)) {
                            bm = m;
                            blo = lo;
                        }
                    }
                }
            }
            for (int b = tid; b < C; b += blockDim.x) {
                const int Lb = static_cast<int>(s_load[b]);
                const int d = La32 - Lb;
                if (b == a || d < 2) continue;
                for (int i = 0; i < na; ++i) {
                    const int lx = s_alen[i];
                    if (lx < d) {
                        const unsigned m = static_cast<unsigned>(max(La32 - lx, Lb + lx));
                        const unsigned lo = (1u << 24) | (unsigned(b) << 12) | unsigned(s_alist[i]);
                        if (m < bm || (m == bm && lo < blo)) {
                            bm = m;
                            blo = lo;
                        }
                    }
                }
            }
            if (bm != 0xffffffffu) best = (static_cast<unsigned long long>(bm) << 25) | blo;
        } else {
        for (int y = tid; y < B; y += blockDim.x) {
            const int b = s_bin[y];
            const long long d = La - s_load[b];
            if (b == a || d < 2) continue;
            const int ly = s_len[y];
            const long long Lb = s_load[b];
            for (int i = 0; i < na; ++i) {
                const int x = s_alist[i];
                const long long dd = s_len[x] - ly;
                if (dd > 0 && dd < d) {
                    const long long m = La - dd > Lb + dd ? La - dd : Lb + dd;
                    const unsigned long long k = (static_cast<unsigned long long>(m) << 25) | (unsigned(y) << 12) | unsigned(x);
                    best = k < best ? k : best;
                }
            }
        }
        for (int b = tid; b < C; b += blockDim.x) {
            const long long Lb = s_load[b];
            const long long d = La - Lb;
            if (b == a || d < 2) continue;
            for (int i = 0; i < na; ++i) {
                const int x = s_alist[i];
                const long long lx = s_len[x];
                if (lx < d) {
                    const long long m = La - lx > Lb + lx ? La - lx : Lb + lx;
                    const unsigned long long k = (static_cast<unsigned long long>(m) << 25) | (1ull << 24) |
                                                 (static_cast<unsigned long long>(b) << 12) | unsigned(x);
                    best = k < best ? k : best;
                }
            }
        }
        }
        best = warp_min_u64(best);
        if (lane == 0) s_red[warp] = best;
        __syncthreads();
        if (warp == 0) {
            best = warp_min_u64(s_red[lane]);
            if (lane == 0) {
                if (best == ~0ull || static_cast<long long>(best >> 25) >= La) {
                    s_done = 1;
                } else {
                    const int x = static_cast<int>(best & 4095u);
                    if (best & (1ull << 24)) {
                        const int b = static_cast<int>((best >> 12) & 1023u);
                        s_load[a] -= s_len[x];
                        s_load[b] += s_len[x];
                        s_bin[x] = static_cast<unsigned short>(b);
                    } else {
                        const int y = static_cast<int>((best >> 12) & 4095u);
                        const int b = s_bin[y];
                        const int dd = s_len[x] - s_len[y];
                        s_load[a] -= dd;
                        s_load[b] += dd;
                        s_bin[x] = static_cast<unsigned short>(b);
                        s_bin[y] = static_cast<unsigned short>(a);
                    }
                }
            }
        }
        __syncthreads();
        if (s_done) break;
    }

    // group by bin: counts, prefix, then every bin lists its members in rank order
    for (int c = tid; c <= C; c += blockDim.x) s_cnt[c] = 0;
    __syncthreads();
    for (int r = tid; r < B; r += blockDim.x) atomicAdd(&s_cnt[s_bin[r] + 1], 1);
    __syncthreads();
    if (tid == 0) {
        for (int c = 0; c < C; ++c) s_cnt[c + 1] += s_cnt[c];
    }
    __syncthreads();
    for (int c = tid; c <= C; c += blockDim.x) seg[c] = s_cnt[c];
    for (int c = tid; c < C; c += blockDim.x) {
        int at = s_cnt[c];
        for (int r = 0; r < B; ++r)
            if (s_bin[r] == c) order[at++] = s_id[r];
    }
    if (cluster_of != nullptr)
        for (int r = tid; r < B; r += blockDim.x) cluster_of[s_id[r]] = s_bin[r];
}

// The next sequence of this cluster (-1: none left). Static schedule: the CTA's shared word
// `s_seq` holds the position in the cluster's own part of `order` (set up by
// first_position), so that nothing stays in a register across a sequence. Otherwise the
// cluster leader pops the shared queue and hands the id to every CTA through distributed
// shared memory. Either way the cluster barrier here also separates the previous sequence's
// use of the CTA's scratch words from the next one's.
__device__ __forceinline__ void first_position(const FwdParams &p, const unsigned CS, const int tid, int *s_seq) {
    if (p.seg != nullptr && tid == 0) *s_seq = p.seg[blockIdx.x / CS];
}
__device__ __forceinline__ int next_sequence(const FwdParams &p, const unsigned rank, const unsigned CS,
                                             const int tid, int *s_seq) {
    if (p.seg == nullptr && rank == 0 && tid == 0) {
        const int i = atomicAdd(p.counter, 1);
        const int seq = i < p.B ? p.order[i] : -1;
        const unsigned seq_addr = smem_u32(s_seq);
        for (unsigned r = 0; r < CS; ++r) st_cluster_s32(map_to_rank(seq_addr, r), seq);
    }
    cluster_arrive();
    cluster_wait();
    if (p.seg == nullptr) return *s_seq;
    const int qi = *s_seq;
    const int seq = qi < p.seg[blockIdx.x / CS + 1] ? p.order[qi] : -1;
    __syncthreads();   // every thread has read the position
    if (tid == 0) *s_seq = qi + 1;
    return seq;
}

// ---- resident kernel ---------------------------------------------------------
// KPT: consecutive k-mers per thread (4 or 1). FIVE: literal five-term LSE.
// A cluster of CS CTAs x NT threads covers K = CS*NT*KPT k-mers.
template <int KPT, bool FIVE>
__global__ void __launch_bounds__(KPT == 4 ? 512 : 1024, 1)
hmm_forward_resident(const FwdParams p) {
    extern __shared__ __align__(16) float a0s[];  // [2][4][M] layer-0 values this CTA consumes
    __shared__ int s_seq;
    __shared__ float s_warp[32];
    __shared__ float s_cl[16];
    __shared__ float s_tr2[kLayers];              // trans2

    const int tid = threadIdx.x;
    const int NT = blockDim.x;
    const unsigned rank = cluster_ctarank();
    const unsigned CS = cluster_nctarank();
    const int K = p.K;
    const int Kq = K >> 2;
    const int M = (NT * KPT) >> 2;     // predecessor groups per CTA
    const int lk = tid * KPT;          // first local k-mer
    const int g = (rank * NT + tid) * KPT;  // first global k-mer
    const int lane = tid & 31, warp = tid >> 5, nwarps = (NT + 31) >> 5;
    if (tid < kLayers) s_tr2[tid] = __ldg(p.trans2 + tid);
    __syncthreads();

    // Transition log-probs into my k-mers: T[j][c] = trans1[p_j, (g+c)%4].
    float T[4][KPT];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int pj = j * Kq + (g >> 2);
        if constexpr (KPT == 4) {
            const float4 v = __ldg(reinterpret_cast<const float4 *>(p.trans1) + pj);
            T[j][0] = v.x;
            T[j][1] = v.y;
            T[j][2] = v.z;
            T[j][3] = v.w;
        } else {
            T[j][0] = __ldg(p.trans1 + pj * 4 + (g & 3));
        }
    }

    // Where my new layer-0 values go: k-mer g is predecessor j=g/Kq of group
    // (g%Kq), which lives in CTA (g%Kq)/M at slot [j][(g%Kq)%M].
    const unsigned a0_base = smem_u32(a0s);
    unsigned dst0;
    {
        const int dj = g / Kq, rem = g % Kq;
        const int dr = rem / M, di = rem % M;
        dst0 = map_to_rank(a0_base + 4u * (dj * M + di), dr);
    }
    const unsigned buf_bytes = 16u * M;  // 4 segments * M floats
    const unsigned cl_addr = smem_u32(s_cl);

    first_position(p, CS, tid, &s_seq);
    for (;;) {
        const int seq = next_sequence(p, rank, CS, tid, &s_seq);
        if (seq < 0) break;

        long long len = p.lens[seq];
        if (len < 1 || len > p.maxlen) {
            if (tid == 0 && rank == 0) atomicOr(&g_status, 1u);
            len = len < 1 ? 1 : p.maxlen;
        }
        const uint8_t *obs = p.data + static_cast<long long>(seq) * p.maxlen;
        const int T_len = static_cast<int>(len);
        bool bad_obs = false;   // an observation byte outside the emission table was met

        // ---- t = 0 (benchmarks/forward.py:94-101) ------------------------------
        float a[kLayers][KPT];
        float e[KPT], e_next[KPT];
        int o_next;
        {
            const int o0 = obs_at(p, obs, 0, bad_obs);
            const int o1 = obs_at(p, obs, T_len > 1 ? 1 : 0, bad_obs);
            o_next = obs_at(p, obs, T_len > 2 ? 2 : T_len - 1, bad_obs);
            if constexpr (KPT == 4) {
                const float4 v0 = __ldg(reinterpret_cast<const float4 *>(p.output_prob + (long long)o0 * K + g));
                const float4 v1 = __ldg(reinterpret_cast<const float4 *>(p.output_prob + (long long)o1 * K + g));
                e[0] = v0.x; e[1] = v0.y; e[2] = v0.z; e[3] = v0.w;
                e_next[0] = v1.x; e_next[1] = v1.y; e_next[2] = v1.z; e_next[3] = v1.w;
            } else {
                e[0] = __ldg(p.output_prob + (long long)o0 * K + g);
                e_next[0] = __ldg(p.output_prob + (long long)o1 * K + g);
            }
#pragma unroll
            for (int d = 0; d < kLayers; ++d) {
                if constexpr (KPT == 4) {
                    const float4 v = __ldg(reinterpret_cast<const float4 *>(p.initial_prob + d * K + g));
                    a[d][0] = v.x + e[0];
                    a[d][1] = v.y + e[1];
                    a[d][2] = v.z + e[2];
                    a[d][3] = v.w + e[3];
                } else {
                    a[d][0] = __ldg(p.initial_prob + d * K + g) + e[0];
                }
            }
        }
        unsigned buf = 0;
        if constexpr (KPT == 4) st_cluster_v4(dst0, a[0][0], a[0][1], a[0][2], a[0][3]);
        else st_cluster_f32(dst0, a[0][0]);
        cluster_arrive();

        // ---- t = 1 .. len-1 (benchmarks/forward.py:103-158) --------------------
        for (int t = 1; t < T_len; ++t) {
            // emission of o_t was fetched a step ago; fetch o_{t+1}'s row and o_{t+2}
#pragma unroll
            for (int c = 0; c < KPT; ++c) e[c] = e_next[c];
            {
                const float *row = p.output_prob + (long long)o_next * K + g;
                if constexpr (KPT == 4) {
                    const float4 v = __ldg(reinterpret_cast<const float4 *>(row));
                    e_next[0] = v.x; e_next[1] = v.y; e_next[2] = v.z; e_next[3] = v.w;
                } else {
                    e_next[0] = __ldg(row);
                }
                const int tn = t + 2 < T_len ? t + 2 : T_len - 1;
                o_next = obs_at(p, obs, tn, bad_obs);
            }

            cluster_wait();  // layer 0 of step t-1 from every CTA has landed
            const float *seg = a0s + (buf ? 4 * M : 0) + (lk >> 2);
            const float a0 = seg[0], a1 = seg[M], a2 = seg[2 * M], a3 = seg[3 * M];
            const unsigned dst = dst0 + (buf ? 0u : buf_bytes);

            if (!FIVE) {
                float q[KPT];
#pragma unroll
                for (int c = 0; c < KPT; ++c)
                    q[c] = lse4(T[0][c] + a0, T[1][c] + a1, T[2][c] + a2, T[3][c] + a3);
                // layer 0 first: it is what the other CTAs wait for
#pragma unroll
                for (int c = 0; c < KPT; ++c) a[0][c] = lse2(s_tr2[0] + q[c], a[1][c]) + e[c];
                if constexpr (KPT == 4) st_cluster_v4(dst, a[0][0], a[0][1], a[0][2], a[0][3]);
                else st_cluster_f32(dst, a[0][0]);
                cluster_arrive();
#pragma unroll
                for (int d = 1; d < kLayers; ++d) {
#pragma unroll
                    for (int c = 0; c < KPT; ++c) {
                        const float v = d == 15 ? p.gamma + a[15][c]
                                      : d == 14 ? p.synthetic + a[15][c]
                                                : a[d + 1 < kLayers ? d + 1 : 15][c];
                        a[d][c] = lse2(s_tr2[d] + q[c], v) + e[c];
                    }
                }
            } else {
#pragma unroll
                for (int d = 0; d < kLayers; ++d) {
#pragma unroll
                    for (int c = 0; c < KPT; ++c) {
                        const float t2 = s_tr2[d];
                        const float p1 = (T[0][c] + t2) + a0;
                        const float p2 = (T[1][c] + t2) + a1;
                        const float p3 = (T[2][c] + t2) + a2;
                        const float p4 = (T[3][c] + t2) + a3;
                        const float p5 = d == 15 ? p.gamma + a[15][c]
                                       : d == 14 ? p.synthetic + a[15][c]
                                                 : 0.0f + a[d + 1 < kLayers ? d + 1 : 15][c];
                        a[d][c] = lse5_reference(p1, p2, p3, p4, p5) + e[c];
                    }
                    if (d == 0) {
                        if constexpr (KPT == 4) st_cluster_v4(dst, a[0][0], a[0][1], a[0][2], a[0][3]);
                        else st_cluster_f32(dst, a[0][0]);
                        cluster_arrive();
                    }
                }
            }
            buf ^= 1u;
        }
        cluster_wait();  // pairs with the last arrive

        // ---- final log-sum-exp over all states (benchmarks/forward.py:160-173) --
        float tmax = -INFINITY;
#pragma unroll
        for (int d = 0; d < kLayers; ++d)
#pragma unroll
            for (int c = 0; c < KPT; ++c) tmax = fmaxf(tmax, a[d][c]);
        tmax = pb::warp_max(tmax);
        if (lane == 0) s_warp[warp] = tmax;
        __syncthreads();
        if (tid < (int)CS) {
            float m = -INFINITY;
            for (int w = 0; w < nwarps; ++w) m = fmaxf(m, s_warp[w]);
            st_cluster_f32(map_to_rank(cl_addr + 4u * rank, tid), m);
        }
        cluster_arrive();
        cluster_wait();
        float gmax = -INFINITY;
        for (unsigned r = 0; r < CS; ++r) gmax = fmaxf(gmax, s_cl[r]);

        float tsum = 0.0f;
#pragma unroll
        for (int d = 0; d < kLayers; ++d)
#pragma unroll
            for (int c = 0; c < KPT; ++c) tsum += fast_exp(a[d][c] - gmax);
        tsum = pb::warp_sum(tsum);
        cluster_arrive();  // everyone has read s_cl (max) before it is reused
        cluster_wait();
        if (lane == 0) s_warp[warp] = tsum;
        __syncthreads();
        if (tid < (int)CS) {
            float s = 0.0f;
            for (int w = 0; w < nwarps; ++w) s += s_warp[w];
            st_cluster_f32(map_to_rank(cl_addr + 4u * rank, tid), s);
        }
        cluster_arrive();
        cluster_wait();
        if (rank == 0 && tid == 0) {
            float s = 0.0f;
            for (unsigned r = 0; r < CS; ++r) s += s_cl[r];
            p.result[seq] = gmax + fast_log(s);
            flag_bad_observation(bad_obs, true);
        }

        if (p.write_alpha) {
            float *dst_alpha = ((len & 1) ? p.alpha1 : p.alpha2) + (long long)seq * (kLayers * (long long)K);
#pragma unroll
            for (int d = 0; d < kLayers; ++d) {
                if constexpr (KPT == 4) {
                    *reinterpret_cast<float4 *>(dst_alpha + (long long)d * K + g) =
                        make_float4(a[d][0], a[d][1], a[d][2], a[d][3]);
                } else {
                    dst_alpha[(long long)d * K + g] = a[d][0];
                }
            }
        }
        // The pop at the top of the loop starts with a full cluster barrier, so
        // s_cl / s_warp / s_seq are free to be rewritten there.
    }
}


// ---- resident kernel, register/shared split ----------------------------------------
// Same algorithm and arithmetic as hmm_forward_resident<4,false>, laid out for
// twice the k-mers per SM: 1024 threads x 4 k-mers per CTA, duration layers 0..7
// in registers, layers 8..15 and the transition columns in shared memory (each
// thread only ever touches its own float4 slots, so no extra synchronisation).
// A 7-mer sequence then needs a cluster of 4 CTAs instead of 8, and clusters of 4
// pack the GPCs without leaving SMs idle.
constexpr int kRegLayers = 8;

template <unsigned POLY_MASK>   // bit d set: layer d evaluates its exponential on the FMA pipe
__global__ void __launch_bounds__(1024, 1) hmm_forward_split(const FwdParams p) {
    extern __shared__ __align__(16) float smem_dyn[];
    __shared__ int s_seq;
    __shared__ float s_warp[32];
    __shared__ float s_cl[16];
    __shared__ float s_tr2[kLayers];          // trans2

    const int tid = threadIdx.x;
    const int NT = blockDim.x;
    const unsigned rank = cluster_ctarank();
    const unsigned CS = cluster_nctarank();
    const int K = p.K;
    const int Kq = K >> 2;
    const int M = NT;                         // predecessor groups per CTA (4 k-mers per thread)
    const int g = (rank * NT + tid) * 4;      // first global k-mer
    const int lane = tid & 31, warp = tid >> 5, nwarps = (NT + 31) >> 5;
    if (tid < kLayers) s_tr2[tid] = __ldg(p.trans2 + tid);

    float *a0s = smem_dyn;                                             // [2][4][M]
    float4 *Ts = reinterpret_cast<float4 *>(smem_dyn + 8 * M);         // [4][NT] transition columns
    float4 *As = Ts + 4 * NT;                                          // [8][NT] layers 8..15
#pragma unroll
    for (int j = 0; j < 4; ++j)
        Ts[j * NT + tid] = __ldg(reinterpret_cast<const float4 *>(p.trans1) + (j * Kq + (g >> 2)));

    const unsigned a0_base = smem_u32(a0s);
    unsigned dst0;
    {
        const int dj = g / Kq, rem = g % Kq;
        const int dr = rem / M, di = rem % M;
        dst0 = map_to_rank(a0_base + 4u * (dj * M + di), dr);
    }
    const unsigned buf_bytes = 16u * M;
    const unsigned cl_addr = smem_u32(s_cl);

    first_position(p, CS, tid, &s_seq);
    for (;;) {
        const int seq = next_sequence(p, rank, CS, tid, &s_seq);
        if (seq < 0) break;

        long long len = p.lens[seq];
        if (len < 1 || len > p.maxlen) {
            if (tid == 0 && rank == 0) atomicOr(&g_status, 1u);
            len = len < 1 ? 1 : p.maxlen;
        }
        const uint8_t *obs = p.data + static_cast<long long>(seq) * p.maxlen;
        const int T_len = static_cast<int>(len);
        bool bad_obs = false;   // an observation byte outside the emission table was met

        // t = 0
        float a[kRegLayers][4];
        float4 e;
        int o_next;
        {
            const int o0 = obs_at(p, obs, 0, bad_obs);
            o_next = obs_at(p, obs, T_len > 1 ? 1 : 0, bad_obs);
            e = __ldg(reinterpret_cast<const float4 *>(p.output_prob + (long long)o0 * K + g));
#pragma unroll
            for (int d = 0; d < kLayers; ++d) {
                float4 v = __ldg(reinterpret_cast<const float4 *>(p.initial_prob + d * K + g));
                v.x += e.x; v.y += e.y; v.z += e.z; v.w += e.w;
                if (d < kRegLayers) { a[d][0] = v.x; a[d][1] = v.y; a[d][2] = v.z; a[d][3] = v.w; }
                else As[(d - kRegLayers) * NT + tid] = v;
            }
        }
        unsigned buf = 0;
        st_cluster_v4(dst0, a[0][0], a[0][1], a[0][2], a[0][3]);
        cluster_arrive();

        for (int t = 1; t < T_len; ++t) {
            // this step's emission slice; the observation after it
            e = __ldg(reinterpret_cast<const float4 *>(p.output_prob + (long long)o_next * K + g));
            o_next = obs_at(p, obs, t + 1 < T_len ? t + 1 : T_len - 1, bad_obs);
            const float ev[4] = {e.x, e.y, e.z, e.w};

            cluster_wait();
            const float *seg = a0s + (buf ? 4 * M : 0) + tid;
            const float a0 = seg[0], a1 = seg[M], a2 = seg[2 * M], a3 = seg[3 * M];
            const unsigned dst = dst0 + (buf ? 0u : buf_bytes);

            float q[4];
            {
                const float4 t0 = Ts[tid], t1 = Ts[NT + tid], t2 = Ts[2 * NT + tid], t3 = Ts[3 * NT + tid];
                q[0] = lse4(t0.x + a0, t1.x + a1, t2.x + a2, t3.x + a3);
                q[1] = lse4(t0.y + a0, t1.y + a1, t2.y + a2, t3.y + a3);
                q[2] = lse4(t0.z + a0, t1.z + a1, t2.z + a2, t3.z + a3);
                q[3] = lse4(t0.w + a0, t1.w + a1, t2.w + a2, t3.w + a3);
            }
#pragma unroll
            for (int c = 0; c < 4; ++c)
                a[0][c] = lse2_sel((POLY_MASK & 1u) != 0, s_tr2[0] + q[c], a[1][c]) + ev[c];
            st_cluster_v4(dst, a[0][0], a[0][1], a[0][2], a[0][3]);
            cluster_arrive();
#pragma unroll
            for (int d = 1; d < kRegLayers - 1; ++d)
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    a[d][c] = lse2_sel(((POLY_MASK >> d) & 1u) != 0, s_tr2[d] + q[c], a[d + 1][c]) + ev[c];
            // layers 7..15: the "next layer" operand comes from shared memory
            float4 nxt = As[tid];  // layer 8 (old)
            {
                const float nv[4] = {nxt.x, nxt.y, nxt.z, nxt.w};
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    a[kRegLayers - 1][c] = lse2_sel(((POLY_MASK >> (kRegLayers - 1)) & 1u) != 0,
                                               s_tr2[kRegLayers - 1] + q[c], nv[c]) + ev[c];
            }
#pragma unroll
            for (int d = kRegLayers; d < kLayers; ++d) {
                // old alpha[min(d+1,15)]; layers 14 and 15 both read old layer 15
                if (d < kLayers - 1) nxt = As[(d + 1 - kRegLayers) * NT + tid];
                const float nv[4] = {nxt.x, nxt.y, nxt.z, nxt.w};
                float r[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float v = d == 15 ? p.gamma + nv[c] : d == 14 ? p.synthetic + nv[c] : nv[c];
                    r[c] = lse2_sel(((POLY_MASK >> d) & 1u) != 0, s_tr2[d] + q[c], v) + ev[c];
                }
                As[(d - kRegLayers) * NT + tid] = make_float4(r[0], r[1], r[2], r[3]);
            }
            buf ^= 1u;
        }
        cluster_wait();

        // final log-sum-exp over all states
        float tmax = -INFINITY;
#pragma unroll
        for (int d = 0; d < kRegLayers; ++d)
#pragma unroll
            for (int c = 0; c < 4; ++c) tmax = fmaxf(tmax, a[d][c]);
#pragma unroll
        for (int d = 0; d < kLayers - kRegLayers; ++d) {
            const float4 v = As[d * NT + tid];
            tmax = fmaxf(tmax, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
        }
        tmax = pb::warp_max(tmax);
        if (lane == 0) s_warp[warp] = tmax;
        __syncthreads();
        if (tid < (int)CS) {
            float m = -INFINITY;
            for (int w = 0; w < nwarps; ++w) m = fmaxf(m, s_warp[w]);
            st_cluster_f32(map_to_rank(cl_addr + 4u * rank, tid), m);
        }
        cluster_arrive();
        cluster_wait();
        float gmax = -INFINITY;
        for (unsigned r = 0; r < CS; ++r) gmax = fmaxf(gmax, s_cl[r]);
        float tsum = 0.0f;
#pragma unroll
        for (int d = 0; d < kRegLayers; ++d)
#pragma unroll
            for (int c = 0; c < 4; ++c) tsum += fast_exp(a[d][c] - gmax);
#pragma unroll
        for (int d = 0; d < kLayers - kRegLayers; ++d) {
            const float4 v = As[d * NT + tid];
            tsum += fast_exp(v.x - gmax) + fast_exp(v.y - gmax) + fast_exp(v.z - gmax) + fast_exp(v.w - gmax);
        }
        tsum = pb::warp_sum(tsum);
        cluster_arrive();
        cluster_wait();
        if (lane == 0) s_warp[warp] = tsum;
        __syncthreads();
        if (tid < (int)CS) {
            float sacc = 0.0f;
            for (int w = 0; w < nwarps; ++w) sacc += s_warp[w];
            st_cluster_f32(map_to_rank(cl_addr + 4u * rank, tid), sacc);
        }
        cluster_arrive();
        cluster_wait();
        if (rank == 0 && tid == 0) {
            float sacc = 0.0f;
            for (unsigned r = 0; r < CS; ++r) sacc += s_cl[r];
            p.result[seq] = gmax + fast_log(sacc);
            flag_bad_observation(bad_obs, true);
        }
        if (p.write_alpha) {
            float *dst_alpha = ((len & 1) ? p.alpha1 : p.alpha2) + (long long)seq * (kLayers * (long long)K);
#pragma unroll
            for (int d = 0; d < kLayers; ++d) {
                const float4 v = d < kRegLayers ? make_float4(a[d % kRegLayers][0], a[d % kRegLayers][1],
                                                              a[d % kRegLayers][2], a[d % kRegLayers][3])
                                                : As[(d - kRegLayers) * NT + tid];
                *reinterpret_cast<float4 *>(dst_alpha + (long long)d * K + g) = v;
            }
        }
    }
}


// log 0 inside the kernels that run with `finite` arithmetic: every -inf that enters (tables,
// emissions, initial distribution) becomes this value, sums of a few of them stay finite for
// any sequence length an int can hold, anything below kLogZeroTest leaves the kernel as -inf.
constexpr float kLogZero = -1e25f;
constexpr float kLogZeroTest = -1e24f;
__device__ __forceinline__ float4 clamp_log_zero(float4 v) {
    return make_float4(fmaxf(v.x, kLogZero), fmaxf(v.y, kLogZero), fmaxf(v.z, kLogZero), fmaxf(v.w, kLogZero));
}
__device__ __forceinline__ float restore_log_zero(float x) { return x < kLogZeroTest ? -INFINITY : x; }

// ---- resident kernel, register/shared split, packed arithmetic ---------------------
// hmm_forward_split with its additions, multiplications and multiply-adds issued as packed
// pairs (add/sub/mul/fma .f32x2: one issue slot for the same operation on two k-mers of the
// thread, each half rounded exactly like the scalar instruction, so the results are those
// of hmm_forward_split with the same POLY_MASK, bit for bit). The freed issue slots let
// more layers take the polynomial exponential, which in turn unloads the MUFU pipe.
// Values stay in natural-log units like the reference's: keeping them in base-2 units
// would save one multiplication per log-sum-exp, but then alpha is rounded on a different
// grid at every step and the result drifts away from the reference's own fp32 rounding
// (2e-5 relative on the 5-mer golden vectors instead of 2e-6).
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 sub2(float2 a, float2 b) {
    float2 r;
    asm("{\n\t.reg .b64 ra, rb, rr;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "sub.rn.f32x2 rr, ra, rb;\n\tmov.b64 {%0, %1}, rr;\n\t}"
        : "=f"(r.x), "=f"(r.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return r;
}
__device__ __forceinline__ float2 dup2(float x) { return make_float2(x, x); }
__device__ __forceinline__ float2 max2(float2 a, float2 b) { return make_float2(fmaxf(a.x, b.x), fmaxf(a.y, b.y)); }

// 2^-|t| for both halves on the FMA pipe; same split and polynomial as ex2_poly.
__device__ __forceinline__ float2 ex2_poly2_negabs(float2 t2) {
    const float2 t = make_float2(fmaxf(-fabsf(t2.x), -126.0f), fmaxf(-fabsf(t2.y), -126.0f));  // NaN -> -126
    const float2 magic = dup2(12582912.0f);
    const float2 r = add2(t, magic);
    const float2 n = sub2(r, magic);
    const float2 f = sub2(t, n);
    float2 p = dup2(0.001327647129073739f);
    p = fma2(p, f, dup2(0.009675540961325169f));
    p = fma2(p, f, dup2(0.05550713092088699f));
    p = fma2(p, f, dup2(0.24022120237350464f));
    p = fma2(p, f, dup2(0.6931469440460205f));
    p = fma2(p, f, dup2(1.0000001192092896f));
    return make_float2(__int_as_float(__float_as_int(p.x) + (__float_as_int(r.x) << 23)),
                       __int_as_float(__float_as_int(p.y) + (__float_as_int(r.y) << 23)));
}

// ln(1 + x) for x in [0, 1] on the FMA pipe: x * P(x), P of degree 6 (minimax on [0, 1], max
// absolute error 3.3e-7 evaluated in fp32; lg2.approx is specified to 2.4e-7). Folded into the
// final multiply-add of the log-sum-exp, it costs five packed instructions more than the
// MUFU form and takes two MUFU operations per pair off the pipe that bounds the kernel.
// `short6`: the same with P of degree 5 (max absolute error 1.5e-6, mean error 3e-9): one packed
// instruction less per pair; still far below the rounding of an alpha value of magnitude 100 and more.
__device__ __forceinline__ float2 log1p_poly2_times(float2 x, bool short6 = false) {
    if (short6) {
        float2 p = dup2(-0.01833890751004219f);
        p = fma2(p, x, dup2(0.08557005226612091f));
        p = fma2(p, x, dup2(-0.19376108050346375f));
        p = fma2(p, x, dup2(0.31764912605285645f));
        p = fma2(p, x, dup2(-0.4978750944137573f));
        p = fma2(p, x, dup2(0.9999016523361206f));
        return p;
    }
    float2 p = dup2(0.01076451875269413f);
    p = fma2(p, x, dup2(-0.05514521896839142f));
    p = fma2(p, x, dup2(0.1346745640039444f));
    p = fma2(p, x, dup2(-0.22589802742004395f));
    p = fma2(p, x, dup2(0.3282422125339508f));
    p = fma2(p, x, dup2(-0.4994717836380005f));
    p = fma2(p, x, dup2(0.999981164932251f));
    return p;   // ln(1 + x) = x * p
}

// log(exp(u) + exp(v)) for two states, every half rounded exactly like lse2_sel;
// (-inf, -inf) gives -inf. `lgpoly`: the logarithm is the polynomial above.
// `finite`: the caller guarantees finite operands (log 0 is kept as a large negative number, see
// kLogZero), so (-inf) - (-inf) cannot occur and the NaN clamp is dropped.
__device__ __forceinline__ float2 lse2_pair(bool poly, float2 u, float2 v, bool lgpoly = false, bool finite = false,
                                            bool short6 = false) {
    const float2 mx = max2(u, v);
    const float2 t = mul2(sub2(u, v), dup2(kLog2e));   // |t| = |u - v| * log2(e)
    float2 ex;
    if (poly) ex = ex2_poly2_negabs(t);
    else ex = make_float2(pb::ex2_approx(-fabsf(t.x)), pb::ex2_approx(-fabsf(t.y)));
    if (lgpoly) {
        const float2 r = fma2(ex, log1p_poly2_times(ex, short6), mx);
        return (poly || finite) ? r : make_float2(fmaxf(r.x, -INFINITY), fmaxf(r.y, -INFINITY));
    }
    const float2 s = add2(ex, dup2(1.0f));
    const float2 r = fma2(make_float2(pb::lg2_approx(s.x), pb::lg2_approx(s.y)), dup2(kLn2), mx);
    // the polynomial path maps the NaN of (-inf) - (-inf) to a zero term by itself
    return (poly || finite) ? r : make_float2(fmaxf(r.x, -INFINITY), fmaxf(r.y, -INFINITY));
}

// log of the sum of four exponentials, terms added in the order j = 0..3 (lse4 on pairs).
__device__ __forceinline__ float2 lse4_pair(float2 p0, float2 p1, float2 p2, float2 p3, bool finite = false) {
    const float2 m = max2(max2(p0, p1), max2(p2, p3));
    const float2 l2e = dup2(kLog2e);
    const float2 d0 = mul2(sub2(p0, m), l2e), d1 = mul2(sub2(p1, m), l2e);
    const float2 d2 = mul2(sub2(p2, m), l2e), d3 = mul2(sub2(p3, m), l2e);
    float2 sum = add2(make_float2(pb::ex2_approx(d0.x), pb::ex2_approx(d0.y)),
                      make_float2(pb::ex2_approx(d1.x), pb::ex2_approx(d1.y)));
    sum = add2(sum, make_float2(pb::ex2_approx(d2.x), pb::ex2_approx(d2.y)));
    sum = add2(sum, make_float2(pb::ex2_approx(d3.x), pb::ex2_approx(d3.y)));
    const float2 r = fma2(make_float2(pb::lg2_approx(sum.x), pb::lg2_approx(sum.y)), dup2(kLn2), m);
    return finite ? r : make_float2(fmaxf(r.x, -INFINITY), fmaxf(r.y, -INFINITY));
}

// POLY_MASK bit d: layer d evaluates its exponential on the FMA pipe; LG_MASK bit d: its logarithm.
// TMEM: layers RL..15 and the transition columns live in tensor memory instead of shared memory
// (RL = layers kept in registers; the shared-memory layout is fixed at 8).
// FIN: finite arithmetic (kLogZero in place of -inf inside the kernel; no NaN clamps).
template <unsigned POLY_MASK, unsigned LG_MASK = 0u, bool TMEM = false, int RL = kRegLayers, bool FIN = false, bool LG6 = false>
__global__ void __launch_bounds__(1024, 1) hmm_forward_packed(const FwdParams p) {
    static_assert(TMEM ? (RL >= 4 && RL <= 8 && RL % 2 == 0) : RL == kRegLayers, "register layers");
    extern __shared__ __align__(16) float smem_dyn[];
    __shared__ int s_seq;
    __shared__ float s_warp[32];
    __shared__ float s_cl[16];
    __shared__ float2 s_t2[kLayers];   // (trans2[d], trans2[d])
    __shared__ unsigned s_tmem;        // base address of the CTA's tensor memory (TMEM)

    const int tid = threadIdx.x;
    constexpr int NT = 1024;            // this layout always runs 1024 threads per CTA (make_plan)
    const unsigned rank = cluster_ctarank();
    const unsigned CS = cluster_nctarank();
    const int K = p.K;
    const int Kq = K >> 2;
    const int M = NT;                         // predecessor groups per CTA (4 k-mers per thread)
    const int g = (rank * NT + tid) * 4;      // first global k-mer
    const int lane = tid & 31, warp = tid >> 5, nwarps = (NT + 31) >> 5;

    float *a0s = smem_dyn;                                             // [2][4][M]
    float4 *Ts = reinterpret_cast<float4 *>(smem_dyn + 8 * M);         // [4][NT] transition columns
    float4 *As = Ts + 4 * NT;                                          // [8][NT] layers 8..15
    // tensor memory: the 8 warps that share a lane quarter take 64 columns each; a thread's
    // columns 0..31 hold layers 8..15 (4 k-mers each), columns 32..47 the transition columns
    unsigned tm_all = 0, tm = 0;
    if constexpr (TMEM) {
        if (warp == 0) tmem_alloc_all(&s_tmem);
        tmem_publish();
        tm_all = s_tmem;
        tm = tmem_warp_base(tm_all, warp, 64 * (warp >> 2));
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float4 v = __ldg(reinterpret_cast<const float4 *>(p.trans1) + (j * Kq + (g >> 2)));
        if constexpr (FIN) v = clamp_log_zero(v);
        if constexpr (TMEM) tmem_st4(tm + 4 * (kLayers - RL) + 4 * j, v);
        else Ts[j * NT + tid] = v;
    }
    if constexpr (TMEM) tmem_wait_st();
    if (tid < kLayers) s_t2[tid] = dup2(FIN ? fmaxf(__ldg(p.trans2 + tid), kLogZero) : __ldg(p.trans2 + tid));
    const float gamma2 = FIN ? fmaxf(p.gamma, kLogZero) : p.gamma, syn2 = FIN ? fmaxf(p.synthetic, kLogZero) : p.synthetic;

    const unsigned a0_base = smem_u32(a0s);
    unsigned dst0;
    {
        const int dj = g / Kq, rem = g % Kq;
        const int dr = rem / M, di = rem % M;
        dst0 = map_to_rank(a0_base + 4u * (dj * M + di), dr);
    }
    const unsigned buf_bytes = 16u * M;
    const unsigned cl_addr = smem_u32(s_cl);
    __syncthreads();

    first_position(p, CS, tid, &s_seq);
    for (;;) {
        const int seq = next_sequence(p, rank, CS, tid, &s_seq);
        if (seq < 0) break;

        long long len = p.lens[seq];
        if (len < 1 || len > p.maxlen) {
            if (tid == 0 && rank == 0) atomicOr(&g_status, 1u);
            len = len < 1 ? 1 : p.maxlen;
        }
        const uint8_t *obs = p.data + static_cast<long long>(seq) * p.maxlen;
        const int T_len = static_cast<int>(len);
        bool bad_obs = false;   // an observation byte outside the emission table was met

        // t = 0
        float2 a[RL][2];
        float4 e;
        int o_next;
        {
            const int o0 = obs_at(p, obs, 0, bad_obs);
            o_next = obs_at(p, obs, T_len > 1 ? 1 : 0, bad_obs);
            e = __ldg(reinterpret_cast<const float4 *>(p.output_prob + (long long)o0 * K + g));
            if constexpr (FIN) e = clamp_log_zero(e);
#pragma unroll
            for (int d = 0; d < kLayers; ++d) {
                float4 v = __ldg(reinterpret_cast<const float4 *>(p.initial_prob + d * K + g));
                if constexpr (FIN) v = clamp_log_zero(v);
                const float2 lo = make_float2(v.x + e.x, v.y + e.y);
                const float2 hi = make_float2(v.z + e.z, v.w + e.w);
                if (d < RL) { a[d][0] = lo; a[d][1] = hi; }
                else if constexpr (TMEM) tmem_st4(tm + 4 * (d - RL), make_float4(lo.x, lo.y, hi.x, hi.y));
                else As[(d - RL) * NT + tid] = make_float4(lo.x, lo.y, hi.x, hi.y);
            }
            if constexpr (TMEM) tmem_wait_st();
        }
        st_cluster_v4(dst0, a[0][0].x, a[0][0].y, a[0][1].x, a[0][1].y);
        cluster_arrive();

        // One time step; buf = (t - 1) & 1, the buffer that holds the previous step's layer 0, is a compile-time
        // constant (the loop below is unrolled twice), so both buffers are addressed with immediates.
        auto step = [&](const int t, auto btag) {
            constexpr unsigned buf = decltype(btag)::value;
            // this step's emission slice; the observation after it
            e = __ldg(reinterpret_cast<const float4 *>(p.output_prob + (long long)o_next * K + g));
            o_next = obs_at(p, obs, t + 1 < T_len ? t + 1 : T_len - 1, bad_obs);
            if constexpr (FIN) e = clamp_log_zero(e);
            const float2 ev[2] = {make_float2(e.x, e.y), make_float2(e.z, e.w)};
            float4 t0, t1, t2, t3;   // transition columns
            if constexpr (TMEM) tmem_ld16(tm + 4 * (kLayers - RL), t0, t1, t2, t3);   // in flight while the exchange completes

            cluster_wait();
            const float *seg = a0s + (buf ? 4 * M : 0) + tid;
            const float2 a0 = dup2(seg[0]), a1 = dup2(seg[M]), a2 = dup2(seg[2 * M]), a3 = dup2(seg[3 * M]);
            const unsigned dst = dst0 + (buf ? 0u : buf_bytes);

            float2 q[2];
            {
                if constexpr (TMEM) {
                    tmem_wait_ld(t0, t1, t2, t3);
                } else {
                    t0 = Ts[tid], t1 = Ts[NT + tid], t2 = Ts[2 * NT + tid], t3 = Ts[3 * NT + tid];
                }
                q[0] = lse4_pair(add2(make_float2(t0.x, t0.y), a0), add2(make_float2(t1.x, t1.y), a1),
                                 add2(make_float2(t2.x, t2.y), a2), add2(make_float2(t3.x, t3.y), a3), FIN);
                q[1] = lse4_pair(add2(make_float2(t0.z, t0.w), a0), add2(make_float2(t1.z, t1.w), a1),
                                 add2(make_float2(t2.z, t2.w), a2), add2(make_float2(t3.z, t3.w), a3), FIN);
            }
            {
                const float2 w = s_t2[0];
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    a[0][h] = add2(lse2_pair((POLY_MASK & 1u) != 0, add2(w, q[h]), a[1][h], (LG_MASK & 1u) != 0, FIN, LG6), ev[h]);
            }
            st_cluster_v4(dst, a[0][0].x, a[0][0].y, a[0][1].x, a[0][1].y);
            cluster_arrive();
#pragma unroll
            for (int d = 1; d < RL - 1; ++d) {
                const float2 w = s_t2[d];
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    a[d][h] = add2(lse2_pair(((POLY_MASK >> d) & 1u) != 0, add2(w, q[h]), a[d + 1][h], ((LG_MASK >> d) & 1u) != 0, FIN, LG6), ev[h]);
            }
            if constexpr (TMEM) {
                // Layers RL..15 live in tensor memory and are updated in place, two layers per load and
                // per store: pair p = layers (d, d + 1), d = RL + 2p, needs the old values of layers
                // d + 1 and d + 2 (the last pair: old layer 15 twice), which one 8-column load brings;
                // the results replace them in the same registers and leave with one 8-column store.
                // The operands of pair p + 1 are requested as soon as those of pair p have arrived (a
                // wait covers every load in flight), so they travel while pair p is computed; a load
                // never covers columns that a store issued before its wait writes.
                constexpr int NP = (kLayers - RL) / 2;
                float4 o0, pr[2][2];
                tmem_ld4(tm, o0);                       // old layer RL, for the last register layer
                if (NP > 1) tmem_ld8(tm + 4, pr[0][0], pr[0][1]);
                else tmem_ld4(tm + 4, pr[0][0]);
                if (NP > 1) tmem_wait_ld(o0, pr[0][0], pr[0][1]);
                else tmem_wait_ld(o0, pr[0][0]);
                if (NP > 2) tmem_ld8(tm + 4 * 3, pr[1][0], pr[1][1]);
                else if (NP == 2) tmem_ld4(tm + 4 * 3, pr[1][0]);
                {
                    const float2 w = s_t2[RL - 1];
                    a[RL - 1][0] = add2(lse2_pair(((POLY_MASK >> (RL - 1)) & 1u) != 0, add2(w, q[0]),
                                                  make_float2(o0.x, o0.y), ((LG_MASK >> (RL - 1)) & 1u) != 0, FIN, LG6), ev[0]);
                    a[RL - 1][1] = add2(lse2_pair(((POLY_MASK >> (RL - 1)) & 1u) != 0, add2(w, q[1]),
                                                  make_float2(o0.z, o0.w), ((LG_MASK >> (RL - 1)) & 1u) != 0, FIN, LG6), ev[1]);
                }
#pragma unroll
                for (int pp = 0; pp < NP; ++pp) {
                    float4 (&b)[2] = pr[pp & 1];
                    const bool last = pp == NP - 1;
                    if (pp > 0) {
                        if (last) tmem_wait_ld(b[0]);
                        else tmem_wait_ld(b[0], b[1]);
                        if (pp + 2 < NP) tmem_ld8(tm + 4 * (2 * pp + 3), pr[(pp + 1) & 1][0], pr[(pp + 1) & 1][1]);
                        else if (pp + 2 == NP) tmem_ld4(tm + 4 * (2 * pp + 3), pr[(pp + 1) & 1][0]);
                    }
                    const int d = RL + 2 * pp;
                    // second layer of the pair first: in the last pair both read old layer 15 (b[0])
                    {
                        const float4 &old = last ? b[0] : b[1];
                        float2 v0 = make_float2(old.x, old.y), v1 = make_float2(old.z, old.w);
                        if (last) { v0.x += gamma2; v0.y += gamma2; v1.x += gamma2; v1.y += gamma2; }
                        const float2 w = s_t2[d + 1];
                        const float2 r0 = add2(lse2_pair(((POLY_MASK >> (d + 1)) & 1u) != 0, add2(w, q[0]), v0, ((LG_MASK >> (d + 1)) & 1u) != 0, FIN, LG6), ev[0]);
                        const float2 r1 = add2(lse2_pair(((POLY_MASK >> (d + 1)) & 1u) != 0, add2(w, q[1]), v1, ((LG_MASK >> (d + 1)) & 1u) != 0, FIN, LG6), ev[1]);
                        b[1] = make_float4(r0.x, r0.y, r1.x, r1.y);
                    }
                    {
                        float2 v0 = make_float2(b[0].x, b[0].y), v1 = make_float2(b[0].z, b[0].w);
                        if (last) { v0.x += syn2; v0.y += syn2; v1.x += syn2; v1.y += syn2; }
                        const float2 w = s_t2[d];
                        const float2 r0 = add2(lse2_pair(((POLY_MASK >> d) & 1u) != 0, add2(w, q[0]), v0, ((LG_MASK >> d) & 1u) != 0, FIN, LG6), ev[0]);
                        const float2 r1 = add2(lse2_pair(((POLY_MASK >> d) & 1u) != 0, add2(w, q[1]), v1, ((LG_MASK >> d) & 1u) != 0, FIN, LG6), ev[1]);
                        b[0] = make_float4(r0.x, r0.y, r1.x, r1.y);
                    }
                    tmem_st8(tm + 4 * (2 * pp), b[0], b[1]);
                }
            } else {
            // layers RL..15: the "next layer" operand comes from shared memory
            float4 nxt = As[tid];           // layer RL (old)
            {
                const float2 w = s_t2[RL - 1];
                a[RL - 1][0] = add2(lse2_pair(((POLY_MASK >> (RL - 1)) & 1u) != 0, add2(w, q[0]),
                                                      make_float2(nxt.x, nxt.y), ((LG_MASK >> (RL - 1)) & 1u) != 0, FIN, LG6), ev[0]);
                a[RL - 1][1] = add2(lse2_pair(((POLY_MASK >> (RL - 1)) & 1u) != 0, add2(w, q[1]),
                                                      make_float2(nxt.z, nxt.w), ((LG_MASK >> (RL - 1)) & 1u) != 0, FIN, LG6), ev[1]);
            }
#pragma unroll
            for (int d = RL; d < kLayers; ++d) {
                // old alpha[min(d+1,15)]; layers 14 and 15 both read old layer 15
                if (d < kLayers - 1) nxt = As[(d + 1 - RL) * NT + tid];
                float2 v0 = make_float2(nxt.x, nxt.y), v1 = make_float2(nxt.z, nxt.w);
                if (d >= 14) {
                    const float c = d == 15 ? gamma2 : syn2;
                    v0.x += c; v0.y += c; v1.x += c; v1.y += c;
                }
                const float2 w = s_t2[d];
                const float2 r0 = add2(lse2_pair(((POLY_MASK >> d) & 1u) != 0, add2(w, q[0]), v0, ((LG_MASK >> d) & 1u) != 0, FIN, LG6), ev[0]);
                const float2 r1 = add2(lse2_pair(((POLY_MASK >> d) & 1u) != 0, add2(w, q[1]), v1, ((LG_MASK >> d) & 1u) != 0, FIN, LG6), ev[1]);
                As[(d - RL) * NT + tid] = make_float4(r0.x, r0.y, r1.x, r1.y);
            }
            }
            if constexpr (TMEM) tmem_wait_st();   // the next step reads what this one stored

        };
        {
            int t = 1;
            for (; t + 1 < T_len; t += 2) {
                step(t, std::integral_constant<unsigned, 0u>{});
                step(t + 1, std::integral_constant<unsigned, 1u>{});
            }
            if (t < T_len) step(t, std::integral_constant<unsigned, 0u>{});
        }
        cluster_wait();

        // final log-sum-exp over all states
        float tmax = -INFINITY;
#pragma unroll
        for (int d = 0; d < RL; ++d)
            tmax = fmaxf(tmax, fmaxf(fmaxf(a[d][0].x, a[d][0].y), fmaxf(a[d][1].x, a[d][1].y)));
#pragma unroll
        for (int d = 0; d < kLayers - RL; ++d) {
            float4 v;
            if constexpr (TMEM) {
                tmem_ld4(tm + 4 * d, v);
                tmem_wait_ld(v);
            } else {
                v = As[d * NT + tid];
            }
            tmax = fmaxf(tmax, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
        }
        tmax = pb::warp_max(tmax);
        if (lane == 0) s_warp[warp] = tmax;
        __syncthreads();
        if (tid < (int)CS) {
            float m = -INFINITY;
            for (int w = 0; w < nwarps; ++w) m = fmaxf(m, s_warp[w]);
            st_cluster_f32(map_to_rank(cl_addr + 4u * rank, tid), m);
        }
        cluster_arrive();
        cluster_wait();
        float gmax = -INFINITY;
        for (unsigned r = 0; r < CS; ++r) gmax = fmaxf(gmax, s_cl[r]);
        float tsum = 0.0f;
#pragma unroll
        for (int d = 0; d < RL; ++d)
            tsum += fast_exp(a[d][0].x - gmax) + fast_exp(a[d][0].y - gmax) +
                    fast_exp(a[d][1].x - gmax) + fast_exp(a[d][1].y - gmax);
#pragma unroll
        for (int d = 0; d < kLayers - RL; ++d) {
            float4 v;
            if constexpr (TMEM) {
                tmem_ld4(tm + 4 * d, v);
                tmem_wait_ld(v);
            } else {
                v = As[d * NT + tid];
            }
            tsum += fast_exp(v.x - gmax) + fast_exp(v.y - gmax) + fast_exp(v.z - gmax) + fast_exp(v.w - gmax);
        }
        tsum = pb::warp_sum(tsum);
        cluster_arrive();
        cluster_wait();
        if (lane == 0) s_warp[warp] = tsum;
        __syncthreads();
        if (tid < (int)CS) {
            float sacc = 0.0f;
            for (int w = 0; w < nwarps; ++w) sacc += s_warp[w];
            st_cluster_f32(map_to_rank(cl_addr + 4u * rank, tid), sacc);
        }
        cluster_arrive();
        cluster_wait();
        if (rank == 0 && tid == 0) {
            float sacc = 0.0f;
            for (unsigned r = 0; r < CS; ++r) sacc += s_cl[r];
            // an impossible sequence (every state at log 0) scores NaN, as the reference's
            // (-inf) - (-inf) in forward_lse_inst does (benchmarks/forward.py:168-173)
            p.result[seq] = (FIN && gmax < kLogZeroTest) ? __int_as_float(0x7fc00000) : gmax + fast_log(sacc);
            flag_bad_observation(bad_obs, true);
        }
        if (p.write_alpha) {
            float *dst_alpha = ((len & 1) ? p.alpha1 : p.alpha2) + (long long)seq * (kLayers * (long long)K);
#pragma unroll
            for (int d = 0; d < kLayers; ++d) {
                float4 v = make_float4(a[d % RL][0].x, a[d % RL][0].y,
                                       a[d % RL][1].x, a[d % RL][1].y);
                if (d >= RL) {
                    if constexpr (TMEM) {
                        tmem_ld4(tm + 4 * (d - RL), v);
                        tmem_wait_ld(v);
                    } else {
                        v = As[(d - RL) * NT + tid];
                    }
                }
                if constexpr (FIN)
                    v = make_float4(restore_log_zero(v.x), restore_log_zero(v.y), restore_log_zero(v.z), restore_log_zero(v.w));
                *reinterpret_cast<float4 *>(dst_alpha + (long long)d * K + g) = v;
            }
        }
    }
    if constexpr (TMEM) {
        tmem_publish();   // every warp is done with its columns
        if (warp == 0) tmem_free_all(tm_all);
    }
}


// ---- one CTA per sequence, packed arithmetic (K <= 1024) -----------------------------
// The 5-mer state space (16 x 1024) fits the registers of one 256-thread CTA: 4 k-mers x
// 16 layers per thread, the arithmetic of hmm_forward_packed (packed pairs, polynomial
// exponential on the layers of POLY_MASK). Layer 0 is exchanged
// through the CTA's own shared memory, so a time step costs one __syncthreads instead of
// a cluster barrier, which is what bounds the step time of small state spaces.
template <unsigned POLY_MASK, unsigned LG_MASK = 0u, bool FIN = false, bool LG6 = false>
__global__ void __launch_bounds__(256, 1) hmm_forward_packed_cta(const FwdParams p) {
    __shared__ __align__(16) float a0s[2][1024];   // layer 0 of all k-mers, double buffered
    __shared__ int s_seq;
    __shared__ float s_warp[32];
    __shared__ float2 s_t2[kLayers];   // (trans2[d], trans2[d])

    const int tid = threadIdx.x;
    constexpr int NT = 256;             // K / 4: this layout exists for K = 1024 only (make_plan)
    constexpr int K = 1024;
    constexpr int Kq = K >> 2;
    const int g = tid * 4;              // first k-mer
    const int lane = tid & 31, warp = tid >> 5, nwarps = (NT + 31) >> 5;

    float2 T[4][2];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float4 v = __ldg(reinterpret_cast<const float4 *>(p.trans1) + (j * Kq + tid));
        if constexpr (FIN) v = clamp_log_zero(v);
        T[j][0] = make_float2(v.x, v.y);
        T[j][1] = make_float2(v.z, v.w);
    }
    if (tid < kLayers) s_t2[tid] = dup2(FIN ? fmaxf(__ldg(p.trans2 + tid), kLogZero) : __ldg(p.trans2 + tid));
    const float gamma2 = FIN ? fmaxf(p.gamma, kLogZero) : p.gamma, syn2 = FIN ? fmaxf(p.synthetic, kLogZero) : p.synthetic;

    if (p.seg != nullptr && tid == 0) s_seq = p.seg[blockIdx.x];   // position in this CTA's part of the schedule
    for (;;) {
        __syncthreads();   // s_seq, s_warp and a0s of the previous sequence are no longer read
        int seq;
        if (p.seg != nullptr) {
            const int qi = s_seq;
            seq = qi < p.seg[blockIdx.x + 1] ? p.order[qi] : -1;
            __syncthreads();   // every thread has read the position
            if (tid == 0) s_seq = qi + 1;
        } else {
            if (tid == 0) {
                const int i = atomicAdd(p.counter, 1);
                s_seq = i < p.B ? p.order[i] : -1;
            }
            __syncthreads();
            seq = s_seq;
        }
        if (seq < 0) break;

        long long len = p.lens[seq];
        if (len < 1 || len > p.maxlen) {
            if (tid == 0) atomicOr(&g_status, 1u);
            len = len < 1 ? 1 : p.maxlen;
        }
        const uint8_t *obs = p.data + static_cast<long long>(seq) * p.maxlen;
        const int T_len = static_cast<int>(len);
        bool bad_obs = false;   // an observation byte outside the emission table was met

        float2 a[kLayers][2];
        float4 e;
        int o_next;
        {
            const int o0 = obs_at(p, obs, 0, bad_obs);
            o_next = obs_at(p, obs, T_len > 1 ? 1 : 0, bad_obs);
            e = __ldg(reinterpret_cast<const float4 *>(p.output_prob + (long long)o0 * K + g));
            if constexpr (FIN) e = clamp_log_zero(e);
#pragma unroll
            for (int d = 0; d < kLayers; ++d) {
                float4 v = __ldg(reinterpret_cast<const float4 *>(p.initial_prob + d * K + g));
                if constexpr (FIN) v = clamp_log_zero(v);
                a[d][0] = make_float2(v.x + e.x, v.y + e.y);
                a[d][1] = make_float2(v.z + e.z, v.w + e.w);
            }
        }
        unsigned buf = 0;
        *reinterpret_cast<float4 *>(&a0s[0][g]) = make_float4(a[0][0].x, a[0][0].y, a[0][1].x, a[0][1].y);

        for (int t = 1; t < T_len; ++t) {
            e = __ldg(reinterpret_cast<const float4 *>(p.output_prob + (long long)o_next * K + g));
            if constexpr (FIN) e = clamp_log_zero(e);
            o_next = obs_at(p, obs, t + 1 < T_len ? t + 1 : T_len - 1, bad_obs);
            const float2 ev[2] = {make_float2(e.x, e.y), make_float2(e.z, e.w)};

            __syncthreads();   // layer 0 of step t-1 is complete; the other buffer is free
            const float *seg = a0s[buf] + tid;
            const float2 a0 = dup2(seg[0]), a1 = dup2(seg[Kq]), a2 = dup2(seg[2 * Kq]), a3 = dup2(seg[3 * Kq]);
            float2 q[2];
#pragma unroll
            for (int h = 0; h < 2; ++h)
                q[h] = lse4_pair(add2(T[0][h], a0), add2(T[1][h], a1), add2(T[2][h], a2), add2(T[3][h], a3), FIN);
#pragma unroll
            for (int d = 0; d < kLayers; ++d) {
                const float2 w = s_t2[d];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float2 v = a[d + 1 < kLayers ? d + 1 : kLayers - 1][h];   // old values: layers ascend in place
                    if (d >= 14) {
                        const float c = d == 15 ? gamma2 : syn2;
                        v.x += c;
                        v.y += c;
                    }
                    a[d][h] = add2(lse2_pair(((POLY_MASK >> d) & 1u) != 0, add2(w, q[h]), v, ((LG_MASK >> d) & 1u) != 0, FIN, LG6), ev[h]);
                }
                if (d == 0)
                    *reinterpret_cast<float4 *>(&a0s[buf ^ 1u][g]) =
                        make_float4(a[0][0].x, a[0][0].y, a[0][1].x, a[0][1].y);
            }
            buf ^= 1u;
        }

        // final log-sum-exp over all states
        float tmax = -INFINITY;
#pragma unroll
        for (int d = 0; d < kLayers; ++d)
            tmax = fmaxf(tmax, fmaxf(fmaxf(a[d][0].x, a[d][0].y), fmaxf(a[d][1].x, a[d][1].y)));
        tmax = pb::warp_max(tmax);
        if (lane == 0) s_warp[warp] = tmax;
        __syncthreads();
        float gmax = -INFINITY;
        for (int w = 0; w < nwarps; ++w) gmax = fmaxf(gmax, s_warp[w]);
        float tsum = 0.0f;
#pragma unroll
        for (int d = 0; d < kLayers; ++d)
            tsum += fast_exp(a[d][0].x - gmax) + fast_exp(a[d][0].y - gmax) +
                    fast_exp(a[d][1].x - gmax) + fast_exp(a[d][1].y - gmax);
        tsum = pb::warp_sum(tsum);
        __syncthreads();   // every thread has read the maxima
        if (lane == 0) s_warp[warp] = tsum;
        __syncthreads();
        if (tid == 0) {
            float sacc = 0.0f;
            for (int w = 0; w < nwarps; ++w) sacc += s_warp[w];
            // an impossible sequence scores NaN like the reference's (-inf) - (-inf)
            p.result[seq] = (FIN && gmax < kLogZeroTest) ? __int_as_float(0x7fc00000) : gmax + fast_log(sacc);
            flag_bad_observation(bad_obs, true);
        }
        if (p.write_alpha) {
            float *dst_alpha = ((len & 1) ? p.alpha1 : p.alpha2) + (long long)seq * (kLayers * (long long)K);
#pragma unroll
            for (int d = 0; d < kLayers; ++d) {
                float4 v = make_float4(a[d][0].x, a[d][0].y, a[d][1].x, a[d][1].y);
                if constexpr (FIN)
                    v = make_float4(restore_log_zero(v.x), restore_log_zero(v.y), restore_log_zero(v.z), restore_log_zero(v.w));
                *reinterpret_cast<float4 *>(dst_alpha + (long long)d * K + g) = v;
            }
        }
    }
}


// ---- scaled (extended-range linear) kernel ------------------------------------------
// The same recurrence evaluated on probabilities instead of log-probabilities:
//   alpha'[d,s] = (A[d] * Q[s] + C[d] * alpha[d+1,s]) * E[s],   Q[s] = sum_j T[j,s] * alpha[0,p_j]
// with A = exp(trans2), T = exp(trans1), E = exp(output_prob[o_t]), C[15] = exp(gamma),
// C[14] = exp(synthetic_248), else 1. Two multiply-adds per state and no
// transcendental in the inner loop (4 ex2 per thread and step for the emissions).
// Range: every thread keeps one base-2 exponent W for its 64 states, value =
// mantissa * 2^W with fp32 mantissas; W follows the data (largest incoming or own
// magnitude) so mantissas stay near 1, and states more than 2^-126 below their
// thread's largest value flush to zero. Layer 0 travels between CTAs as
// (mantissa, exponent). Log-likelihoods are formed once per sequence. Against a
// float64 evaluation of the reference formula this agrees to ~1e-8 relative; the
// reference's own fp32 log-space result carries more rounding than that.
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ int exponent_of(float x) {   // x >= 0; 0 and denormals give -127
    return (__float_as_int(x) >> 23) - 127;
}
__device__ __forceinline__ float pow2_clamped(int e) {  // 2^e, +0.0 below 2^-126
    e = max(e, -127);
    e = min(e, 127);
    return __int_as_float((e + 127) << 23);
}

constexpr int kExpFloor = -(1 << 28);  // exponent of an all-zero thread
// Exponent that travels with a layer-0 mantissa: thread exponent + exponent of the
// mantissa. A zero mantissa travels with an exponent so low that the receiver's
// scale factor becomes +0.0 (its mantissa bits are rebuilt as 1.0, see below).
__device__ __forceinline__ int export_exponent(float x, int W) {
    return x > 0.0f ? W + exponent_of(x) : kExpFloor - 200;
}

__global__ void __launch_bounds__(512, 1) hmm_forward_scaled(const FwdParams p) {
    extern __shared__ __align__(16) float smem_dyn[];   // [2][4][M] mantissas, then [2][4][M] exponents
    __shared__ int s_seq;
    __shared__ float s_warp[32];
    __shared__ int s_warp_i[32];
    __shared__ float s_cl[16];
    __shared__ int s_cl_i[16];
    __shared__ float s_A[kLayers];      // exp(trans2[d])

    const int tid = threadIdx.x;
    const int NT = blockDim.x;
    const unsigned rank = cluster_ctarank();
    const unsigned CS = cluster_nctarank();
    const int K = p.K;
    const int Kq = K >> 2;
    const int M = NT;
    const int g = (rank * NT + tid) * 4;
    const int lane = tid & 31, warp = tid >> 5, nwarps = (NT + 31) >> 5;
    if (tid < kLayers) s_A[tid] = expf(__ldg(p.trans2 + tid));

    float *a0x = smem_dyn;
    int *a0e = reinterpret_cast<int *>(smem_dyn + 8 * M);

    // T[j][c] = exp(trans1[p_j, (g+c)%4])
    float T[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float4 v = __ldg(reinterpret_cast<const float4 *>(p.trans1) + (j * Kq + (g >> 2)));
        T[j][0] = fast_exp(v.x);
        T[j][1] = fast_exp(v.y);
        T[j][2] = fast_exp(v.z);
        T[j][3] = fast_exp(v.w);
    }
    unsigned dstx0, dste0;
    {
        const int dj = g / Kq, rem = g % Kq;
        const int dr = rem / M, di = rem % M;
        dstx0 = map_to_rank(smem_u32(a0x) + 4u * (dj * M + di), dr);
        dste0 = map_to_rank(smem_u32(a0e) + 4u * (dj * M + di), dr);
    }
    const unsigned buf_bytes = 16u * M;
    const unsigned cl_addr = smem_u32(s_cl);
    const unsigned cli_addr = smem_u32(s_cl_i);

    first_position(p, CS, tid, &s_seq);
    for (;;) {
        const int seq = next_sequence(p, rank, CS, tid, &s_seq);
        if (seq < 0) break;

        long long len = p.lens[seq];
        if (len < 1 || len > p.maxlen) {
            if (tid == 0 && rank == 0) atomicOr(&g_status, 1u);
            len = len < 1 ? 1 : p.maxlen;
        }
        const uint8_t *obs = p.data + static_cast<long long>(seq) * p.maxlen;
        const int T_len = static_cast<int>(len);
        bool bad_obs = false;   // an observation byte outside the emission table was met

        // ---- t = 0: x = exp(initial_prob) * exp(emission), W = 0 ------------------------
        float x[kLayers][4];
        float4 e_next;
        int o_next;
        int W = 0;       // exponent shared by this thread's 64 states
        int kt;          // exponent of the largest mantissa (magnitude hint)
        {
            const int o0 = obs_at(p, obs, 0, bad_obs);
            const int o1 = obs_at(p, obs, T_len > 1 ? 1 : 0, bad_obs);
            o_next = obs_at(p, obs, T_len > 2 ? 2 : T_len - 1, bad_obs);
            const float4 e0 = __ldg(reinterpret_cast<const float4 *>(p.output_prob + (long long)o0 * K + g));
            e_next = __ldg(reinterpret_cast<const float4 *>(p.output_prob + (long long)o1 * K + g));
            const float el[4] = {fast_exp(e0.x), fast_exp(e0.y), fast_exp(e0.z), fast_exp(e0.w)};
            float m = 0.0f;
#pragma unroll
            for (int d = 0; d < kLayers; ++d) {
                const float4 v = __ldg(reinterpret_cast<const float4 *>(p.initial_prob + d * K + g));
                x[d][0] = fast_exp(v.x) * el[0];
                x[d][1] = fast_exp(v.y) * el[1];
                x[d][2] = fast_exp(v.z) * el[2];
                x[d][3] = fast_exp(v.w) * el[3];
                m = max3(m, fmaxf(x[d][0], x[d][1]), fmaxf(x[d][2], x[d][3]));
            }
            kt = exponent_of(m);
        }
        unsigned buf = 0;
        st_cluster_v4(dstx0, x[0][0], x[0][1], x[0][2], x[0][3]);
        st_cluster_v4i(dste0, export_exponent(x[0][0], W), export_exponent(x[0][1], W),
                       export_exponent(x[0][2], W), export_exponent(x[0][3], W));
        cluster_arrive();

        for (int t = 1; t < T_len; ++t) {
            // emission probabilities of o_t (log values were fetched a step ago)
            const float el[4] = {fast_exp(e_next.x), fast_exp(e_next.y), fast_exp(e_next.z), fast_exp(e_next.w)};
            e_next = __ldg(reinterpret_cast<const float4 *>(p.output_prob + (long long)o_next * K + g));
            o_next = obs_at(p, obs, t + 2 < T_len ? t + 2 : T_len - 1, bad_obs);

            cluster_wait();
            const int off = (buf ? 4 * M : 0) + tid;
            const float xa0 = a0x[off], xa1 = a0x[off + M], xa2 = a0x[off + 2 * M], xa3 = a0x[off + 3 * M];
            // each predecessor arrives with "its exponent + exponent of its mantissa" so that
            // the largest incoming magnitude is known without touching the mantissas
            const int ea0 = a0e[off], ea1 = a0e[off + M], ea2 = a0e[off + 2 * M], ea3 = a0e[off + 3 * M];
            const unsigned dstx = dstx0 + (buf ? 0u : buf_bytes);
            const unsigned dste = dste0 + (buf ? 0u : buf_bytes);

            // new exponent: the largest magnitude this thread is about to combine
            int Wn = max(max(ea0, ea1), max(ea2, ea3));
            Wn = max(Wn, W + kt);
            Wn = max(Wn, kExpFloor);
            // incoming layer-0 values relative to 2^Wn (ea = W_p + exponent_of(x) => x*2^(W_p-Wn) =
            // mantissa-normalised x * 2^(ea - Wn))
            const float y0 = __int_as_float((__float_as_int(xa0) & 0x007fffff) | 0x3f800000) * pow2_clamped(ea0 - Wn);
            const float y1 = __int_as_float((__float_as_int(xa1) & 0x007fffff) | 0x3f800000) * pow2_clamped(ea1 - Wn);
            const float y2 = __int_as_float((__float_as_int(xa2) & 0x007fffff) | 0x3f800000) * pow2_clamped(ea2 - Wn);
            const float y3 = __int_as_float((__float_as_int(xa3) & 0x007fffff) | 0x3f800000) * pow2_clamped(ea3 - Wn);
            const float own = pow2_clamped(W - Wn);
            float QE[4], Eo[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float q = fmaf(T[3][c], y3, fmaf(T[2][c], y2, fmaf(T[1][c], y1, T[0][c] * y0)));
                QE[c] = q * el[c];
                Eo[c] = el[c] * own;
            }
            // layer 0 first: it is what the other CTAs wait for
#pragma unroll
            for (int c = 0; c < 4; ++c) x[0][c] = fmaf(s_A[0], QE[c], Eo[c] * x[1][c]);
            st_cluster_v4(dstx, x[0][0], x[0][1], x[0][2], x[0][3]);
            st_cluster_v4i(dste, export_exponent(x[0][0], Wn), export_exponent(x[0][1], Wn),
                           export_exponent(x[0][2], Wn), export_exponent(x[0][3], Wn));
            cluster_arrive();
            float m = max3(fmaxf(x[0][0], x[0][1]), x[0][2], x[0][3]);
#pragma unroll
            for (int d = 1; d < kLayers; ++d) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float nx = d == 15 ? p.gamma_lin * x[15][c]
                                   : d == 14 ? p.synthetic_lin * x[15][c]
                                             : x[d + 1 < kLayers ? d + 1 : 15][c];
                    x[d][c] = fmaf(s_A[d], QE[c], Eo[c] * nx);
                }
                m = max3(m, fmaxf(x[d][0], x[d][1]), fmaxf(x[d][2], x[d][3]));
            }
            kt = exponent_of(m);
            W = Wn;
            buf ^= 1u;
        }
        cluster_wait();

        // ---- log-likelihood: log(sum of all states) with a common exponent --------------
        int gexp = W + kt;
        gexp = __reduce_max_sync(0xffffffffu, gexp);
        if (lane == 0) s_warp_i[warp] = gexp;
        __syncthreads();
        if (tid < (int)CS) {
            int v = kExpFloor - 200;
            for (int w = 0; w < nwarps; ++w) v = max(v, s_warp_i[w]);
            st_cluster_s32(map_to_rank(cli_addr + 4u * rank, tid), v);
        }
        cluster_arrive();
        cluster_wait();
        int G = kExpFloor - 200;
        for (unsigned r = 0; r < CS; ++r) G = max(G, s_cl_i[r]);
        float tsum = 0.0f;
#pragma unroll
        for (int d = 0; d < kLayers; ++d) tsum += (x[d][0] + x[d][1]) + (x[d][2] + x[d][3]);
        tsum *= pow2_clamped(W - G);
        tsum = pb::warp_sum(tsum);
        if (lane == 0) s_warp[warp] = tsum;
        __syncthreads();
        if (tid < (int)CS) {
            float sacc = 0.0f;
            for (int w = 0; w < nwarps; ++w) sacc += s_warp[w];
            st_cluster_f32(map_to_rank(cl_addr + 4u * rank, tid), sacc);
        }
        cluster_arrive();
        cluster_wait();
        if (rank == 0 && tid == 0) {
            double sacc = 0.0;
            for (unsigned r = 0; r < CS; ++r) sacc += (double)s_cl[r];
            // natural log of sum * 2^G; an impossible sequence (sum == 0) gives NaN like the reference's (-inf) - (-inf)
            p.result[seq] = sacc > 0.0 ? (float)(log(sacc) + (double)G * 0.6931471805599453) : __int_as_float(0x7fc00000);
            flag_bad_observation(bad_obs, true);
        }
        if (p.write_alpha) {
            float *dst_alpha = ((len & 1) ? p.alpha1 : p.alpha2) + (long long)seq * (kLayers * (long long)K);
            const float wl = (float)W * kLn2;
#pragma unroll
            for (int d = 0; d < kLayers; ++d) {
                float4 v;
                v.x = fast_log(x[d][0]) + wl;
                v.y = fast_log(x[d][1]) + wl;
                v.z = fast_log(x[d][2]) + wl;
                v.w = fast_log(x[d][3]) + wl;
                *reinterpret_cast<float4 *>(dst_alpha + (long long)d * K + g) = v;
            }
        }
        // the pop at the top of the loop starts with a full cluster barrier
    }
}

// ---- scaled kernel, register/shared split layout --------------------------------------
// hmm_forward_scaled laid out like hmm_forward_packed: 1024 threads x 4 k-mers per CTA,
// layers 0..7 in registers, layers 8..15 and three of the four transition columns in
// shared memory, so a 7-mer sequence takes a cluster of 4 CTAs (33 clusters on 132 SMs,
// 32 warps per SM to hide the exchange) instead of 8. The multiply-adds run as packed
// pairs. Layer 0 travels as the sender's mantissas plus ONE exponent per sending thread
// (its 64 states share it), which the receiver combines with the exponent field of each
// mantissa; that is 20 bytes per thread and step instead of 32 and lets two exchange
// buffers fit beside the state. Same arithmetic as hmm_forward_scaled value for value.
__global__ void __launch_bounds__(1024, 1) hmm_forward_scaled_split(const FwdParams p) {
    extern __shared__ __align__(16) float smem_dyn[];
    __shared__ int s_seq;
    __shared__ float s_warp[32];
    __shared__ int s_warp_i[32];
    __shared__ float s_cl[16];
    __shared__ int s_cl_i[16];
    __shared__ float4 s_A4[kLayers / 4];  // exp(trans2[d]), four layers per 16-byte load

    const int tid = threadIdx.x;
    constexpr int NT = 1024;            // this layout always runs 1024 threads per CTA (make_plan)
    const unsigned rank = cluster_ctarank();
    const unsigned CS = cluster_nctarank();
    const int K = p.K;
    const int Kq = K >> 2;
    const int M = NT;
    const int g = (rank * NT + tid) * 4;
    const int lane = tid & 31, warp = tid >> 5, nwarps = (NT + 31) >> 5;

    float *a0x = smem_dyn;                                            // [2][4][M] mantissas
    int *a0w = reinterpret_cast<int *>(smem_dyn + 8 * M);             // [2][4][M/4] sender exponents
    float4 *Ts = reinterpret_cast<float4 *>(smem_dyn + 10 * M);       // [3][NT] exp(trans1) columns j = 0..2
    float4 *As = Ts + 3 * NT;                                         // [8][NT] layers 8..15

    float2 T3[2];   // column j = 3 stays in registers
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float4 v = __ldg(reinterpret_cast<const float4 *>(p.trans1) + (j * Kq + (g >> 2)));
        const float4 w = make_float4(fast_exp(v.x), fast_exp(v.y), fast_exp(v.z), fast_exp(v.w));
        if (j < 3) {
            Ts[j * NT + tid] = w;
        } else {
            T3[0] = make_float2(w.x, w.y);
            T3[1] = make_float2(w.z, w.w);
        }
    }
    if (tid < kLayers) reinterpret_cast<float *>(s_A4)[tid] = expf(__ldg(p.trans2 + tid));
    unsigned dstx0, dstw0;
    {
        const int dj = g / Kq, rem = g % Kq;
        const int dr = rem / M, di = rem % M;
        dstx0 = map_to_rank(smem_u32(a0x) + 4u * (dj * M + di), dr);
        dstw0 = map_to_rank(smem_u32(a0w) + 4u * (dj * (M >> 2) + (di >> 2)), dr);
    }
    const unsigned bufx_bytes = 16u * M, bufw_bytes = 4u * M;
    const unsigned cl_addr = smem_u32(s_cl);
    const unsigned cli_addr = smem_u32(s_cl_i);

    first_position(p, CS, tid, &s_seq);
    for (;;) {
        const int seq = next_sequence(p, rank, CS, tid, &s_seq);
        if (seq < 0) break;

        long long len = p.lens[seq];
        if (len < 1 || len > p.maxlen) {
            if (tid == 0 && rank == 0) atomicOr(&g_status, 1u);
            len = len < 1 ? 1 : p.maxlen;
        }
        const uint8_t *obs = p.data + static_cast<long long>(seq) * p.maxlen;
        const int T_len = static_cast<int>(len);
        bool bad_obs = false;   // an observation byte outside the emission table was met

        // ---- t = 0: x = exp(initial_prob) * exp(emission), W = 0 ------------------------
        float2 x[kRegLayers][2];
        int o_next;
        int W = 0;       // exponent shared by this thread's 64 states
        int kt;          // exponent of the largest mantissa (magnitude hint)
        {
            const int o0 = obs_at(p, obs, 0, bad_obs);
            o_next = obs_at(p, obs, T_len > 1 ? 1 : 0, bad_obs);
            const float4 e0 = __ldg(reinterpret_cast<const float4 *>(p.output_prob + (long long)o0 * K + g));
            const float el[4] = {fast_exp(e0.x), fast_exp(e0.y), fast_exp(e0.z), fast_exp(e0.w)};
            float m = 0.0f;
#pragma unroll
            for (int d = 0; d < kLayers; ++d) {
                const float4 v = __ldg(reinterpret_cast<const float4 *>(p.initial_prob + d * K + g));
                const float4 r = make_float4(fast_exp(v.x) * el[0], fast_exp(v.y) * el[1], fast_exp(v.z) * el[2],
                                             fast_exp(v.w) * el[3]);
                m = max3(m, fmaxf(r.x, r.y), fmaxf(r.z, r.w));
                if (d < kRegLayers) {
                    x[d][0] = make_float2(r.x, r.y);
                    x[d][1] = make_float2(r.z, r.w);
                } else {
                    As[(d - kRegLayers) * NT + tid] = r;
                }
            }
            kt = exponent_of(m);
        }
        st_cluster_v4(dstx0, x[0][0].x, x[0][0].y, x[0][1].x, x[0][1].y);
        st_cluster_s32(dstw0, W);
        cluster_arrive();

        for (int t = 1; t < T_len; ++t) {
            // this step's emission slice (in flight while the exchange completes); the observation after it
            const float4 e = __ldg(reinterpret_cast<const float4 *>(p.output_prob + (long long)o_next * K + g));
            o_next = obs_at(p, obs, t + 1 < T_len ? t + 1 : T_len - 1, bad_obs);

            cluster_wait();
            const unsigned buf = (t & 1) ^ 1u;   // buffer that holds the previous step's layer 0
            const float *px = a0x + (buf ? 4 * M : 0) + tid;
            const int *pw = a0w + (buf ? M : 0) + (tid >> 2);
            const float xa0 = px[0], xa1 = px[M], xa2 = px[2 * M], xa3 = px[3 * M];
            const int wp0 = pw[0], wp1 = pw[M >> 2], wp2 = pw[2 * (M >> 2)], wp3 = pw[3 * (M >> 2)];
            const unsigned dstx = dstx0 + (buf ? 0u : bufx_bytes);
            const unsigned dstw = dstw0 + (buf ? 0u : bufw_bytes);

            // magnitude of each incoming value = sender exponent + exponent field of its mantissa;
            // the new exponent is the largest magnitude this thread is about to combine
            const int ea0 = xa0 > 0.0f ? wp0 + exponent_of(xa0) : kExpFloor - 200;
            const int ea1 = xa1 > 0.0f ? wp1 + exponent_of(xa1) : kExpFloor - 200;
            const int ea2 = xa2 > 0.0f ? wp2 + exponent_of(xa2) : kExpFloor - 200;
            const int ea3 = xa3 > 0.0f ? wp3 + exponent_of(xa3) : kExpFloor - 200;
            int Wn = max(max(ea0, ea1), max(ea2, ea3));
            Wn = max(Wn, W + kt);
            Wn = max(Wn, kExpFloor);
            // incoming values relative to 2^Wn (a power-of-two factor: exact); Wn >= wp + exponent, so
            // the product stays below 2; below 2^-126 it flushes to zero
            const float2 y0 = dup2(xa0 * pow2_clamped(wp0 - Wn)), y1 = dup2(xa1 * pow2_clamped(wp1 - Wn));
            const float2 y2 = dup2(xa2 * pow2_clamped(wp2 - Wn)), y3 = dup2(xa3 * pow2_clamped(wp3 - Wn));
            const float2 own = dup2(pow2_clamped(W - Wn));
            float2 QE[2], Eo[2];
            {
                const float4 t0 = Ts[tid], t1 = Ts[NT + tid], t2 = Ts[2 * NT + tid];
                const float2 q0 = fma2(T3[0], y3, fma2(make_float2(t2.x, t2.y), y2,
                                  fma2(make_float2(t1.x, t1.y), y1, mul2(make_float2(t0.x, t0.y), y0))));
                const float2 q1 = fma2(T3[1], y3, fma2(make_float2(t2.z, t2.w), y2,
                                  fma2(make_float2(t1.z, t1.w), y1, mul2(make_float2(t0.z, t0.w), y0))));
                const float2 el2[2] = {make_float2(fast_exp(e.x), fast_exp(e.y)), make_float2(fast_exp(e.z), fast_exp(e.w))};
                QE[0] = mul2(q0, el2[0]);
                QE[1] = mul2(q1, el2[1]);
                Eo[0] = mul2(el2[0], own);
                Eo[1] = mul2(el2[1], own);
            }
            // layer 0 first: it is what the other CTAs wait for
            // exp(trans2) of four layers per shared-memory load (the shared-memory pipe bounds this kernel)
            float4 a4 = s_A4[0];
            const auto A_of = [&](int d) { return dup2(d % 4 == 0 ? a4.x : d % 4 == 1 ? a4.y : d % 4 == 2 ? a4.z : a4.w); };
            {
                const float2 a = A_of(0);
                x[0][0] = fma2(a, QE[0], mul2(Eo[0], x[1][0]));
                x[0][1] = fma2(a, QE[1], mul2(Eo[1], x[1][1]));
            }
            st_cluster_v4(dstx, x[0][0].x, x[0][0].y, x[0][1].x, x[0][1].y);
            st_cluster_s32(dstw, Wn);
            cluster_arrive();
            float m = max3(fmaxf(x[0][0].x, x[0][0].y), x[0][1].x, x[0][1].y);
#pragma unroll
            for (int d = 1; d < kRegLayers - 1; ++d) {
                if (d % 4 == 0) a4 = s_A4[d / 4];
                const float2 a = A_of(d);
                x[d][0] = fma2(a, QE[0], mul2(Eo[0], x[d + 1][0]));
                x[d][1] = fma2(a, QE[1], mul2(Eo[1], x[d + 1][1]));
                m = max3(m, x[d][0].x, x[d][0].y);
                m = max3(m, x[d][1].x, x[d][1].y);
            }
            float4 nxt = As[tid];   // layer 8 (old)
            {
                const float2 a = A_of(kRegLayers - 1);
                x[kRegLayers - 1][0] = fma2(a, QE[0], mul2(Eo[0], make_float2(nxt.x, nxt.y)));
                x[kRegLayers - 1][1] = fma2(a, QE[1], mul2(Eo[1], make_float2(nxt.z, nxt.w)));
                m = max3(m, x[kRegLayers - 1][0].x, x[kRegLayers - 1][0].y);
                m = max3(m, x[kRegLayers - 1][1].x, x[kRegLayers - 1][1].y);
            }
#pragma unroll
            for (int d = kRegLayers; d < kLayers; ++d) {
                // old value of layer min(d+1, 15); layers 14 and 15 both read old layer 15
                if (d < kLayers - 1) nxt = As[(d + 1 - kRegLayers) * NT + tid];
                float2 v0 = make_float2(nxt.x, nxt.y), v1 = make_float2(nxt.z, nxt.w);
                if (d >= 14) {
                    const float c = d == 15 ? p.gamma_lin : p.synthetic_lin;
                    v0.x *= c; v0.y *= c; v1.x *= c; v1.y *= c;
                }
                if (d % 4 == 0) a4 = s_A4[d / 4];
                const float2 a = A_of(d);
                const float2 r0 = fma2(a, QE[0], mul2(Eo[0], v0));
                const float2 r1 = fma2(a, QE[1], mul2(Eo[1], v1));
                As[(d - kRegLayers) * NT + tid] = make_float4(r0.x, r0.y, r1.x, r1.y);
                m = max3(m, r0.x, r0.y);
                m = max3(m, r1.x, r1.y);
            }
            kt = exponent_of(m);
            W = Wn;
        }
        cluster_wait();

        // ---- log-likelihood: log(sum of all states) with a common exponent --------------
        int gexp = W + kt;
        gexp = __reduce_max_sync(0xffffffffu, gexp);
        if (lane == 0) s_warp_i[warp] = gexp;
        __syncthreads();
        if (tid < (int)CS) {
            int v = kExpFloor - 200;
            for (int w = 0; w < nwarps; ++w) v = max(v, s_warp_i[w]);
            st_cluster_s32(map_to_rank(cli_addr + 4u * rank, tid), v);
        }
        cluster_arrive();
        cluster_wait();
        int G = kExpFloor - 200;
        for (unsigned r = 0; r < CS; ++r) G = max(G, s_cl_i[r]);
        float tsum = 0.0f;
#pragma unroll
        for (int d = 0; d < kRegLayers; ++d) tsum += (x[d][0].x + x[d][0].y) + (x[d][1].x + x[d][1].y);
#pragma unroll
        for (int d = 0; d < kLayers - kRegLayers; ++d) {
            const float4 v = As[d * NT + tid];
            tsum += (v.x + v.y) + (v.z + v.w);
        }
        tsum *= pow2_clamped(W - G);
        tsum = pb::warp_sum(tsum);
        if (lane == 0) s_warp[warp] = tsum;
        __syncthreads();
        if (tid < (int)CS) {
            float sacc = 0.0f;
            for (int w = 0; w < nwarps; ++w) sacc += s_warp[w];
            st_cluster_f32(map_to_rank(cl_addr + 4u * rank, tid), sacc);
        }
        cluster_arrive();
        cluster_wait();
        if (rank == 0 && tid == 0) {
            double sacc = 0.0;
            for (unsigned r = 0; r < CS; ++r) sacc += (double)s_cl[r];
            // natural log of sum * 2^G; an impossible sequence (sum == 0) gives NaN like the reference's (-inf) - (-inf)
            p.result[seq] = sacc > 0.0 ? (float)(log(sacc) + (double)G * 0.6931471805599453) : __int_as_float(0x7fc00000);
            flag_bad_observation(bad_obs, true);
        }
        if (p.write_alpha) {
            float *dst_alpha = ((len & 1) ? p.alpha1 : p.alpha2) + (long long)seq * (kLayers * (long long)K);
            const float wl = (float)W * kLn2;
#pragma unroll
            for (int d = 0; d < kLayers; ++d) {
                const float4 s4 = d < kRegLayers ? make_float4(x[d % kRegLayers][0].x, x[d % kRegLayers][0].y,
                                                               x[d % kRegLayers][1].x, x[d % kRegLayers][1].y)
                                                 : As[(d - kRegLayers) * NT + tid];
                float4 v;
                v.x = fast_log(s4.x) + wl;
                v.y = fast_log(s4.y) + wl;
                v.z = fast_log(s4.z) + wl;
                v.w = fast_log(s4.w) + wl;
                *reinterpret_cast<float4 *>(dst_alpha + (long long)d * K + g) = v;
            }
        }
        // the next pop starts with a full cluster barrier
    }
}

// ---- scaled kernel, layers 8..15 and the transition columns in tensor memory -----------
// hmm_forward_scaled_split is bound by the shared-memory pipe: per thread and step it reads
// and writes the eight upper layers (2 x 128 bytes) and reads three transition columns through
// a pipe that moves 128 bytes per clock and SM. Tensor memory (256 KB per SM, otherwise the
// accumulator store of the tensor cores) takes their place here: every thread owns 48 of its
// warp's columns (32 for layers 8..15, 16 for exp(trans1)) and moves them with tcgen05.ld/st,
// which reach 3.4 x the shared-memory rate for this access pattern. Shared memory then holds
// only the layer-0 exchange. Arithmetic and results are those of hmm_forward_scaled_split.
// Bounded wait on a CTA-local mbarrier phase (st.async exchange). False: gave up.
constexpr int kFwdWaitLimit = 1 << 22;
__device__ __forceinline__ bool fwd_mbar_wait(unsigned mbar, unsigned parity, int limit = kFwdWaitLimit) {
    for (int i = 0; i < limit; ++i) {
        unsigned ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(mbar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

// exp() of every entry of the emission table, for the scaled kernel: the same fast_exp it would
// take per use (4 per thread and step), taken once per entry here. n4 = number of float4.
__global__ void __launch_bounds__(256) hmm_exp_table(const float4 *__restrict__ in, float4 *__restrict__ out, long long n4) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
        const float4 v = __ldg(in + i);
        out[i] = make_float4(fast_exp(v.x), fast_exp(v.y), fast_exp(v.z), fast_exp(v.w));
    }
}

// One CTA that waits, with the kernel's own bounded wait, on a barrier nothing completes: the wait
// runs out after `polls` polls and status bit 2 is raised exactly as in hmm_forward_scaled_tmem. No
// other CTA, no data in flight; used to check that a wait that gives up reaches the host.
__global__ void fwd_wait_probe(int polls, unsigned *host_flag) {
    __shared__ __align__(8) unsigned long long mbar;
    const unsigned addr = smem_u32(&mbar);
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(addr));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (!fwd_mbar_wait(addr, 0u, polls) && threadIdx.x == 0) flag_wait_timeout(host_flag);
    __syncthreads();
    if (threadIdx.x == 0) asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(addr) : "memory");
}

// RL: layers kept in registers (4, 6 or 8); the others live in tensor memory. ASYNC (clusters of
// 2 to 8 CTAs): layer 0 travels with st.async and is counted in by an mbarrier of the consuming
// CTA (complete_tx), so the sender runs no release fence (the largest stall of the barrier
// version). A CTA's phase completes on the bytes of the quarter of each producer's threads whose
// k-mers it consumes, so a CTA can run ahead of threads elsewhere in the cluster; with up to 8
// CTAs a writer of round r is only ordered after every thread's read of round r - 4, hence four
// buffers and four mbarriers. Every wait is bounded; one that runs out raises status bit 2.
// LIN: emission factors come from the table of exponentials in p.output_lin.
template <int RL, bool ASYNC, bool LIN = false>
__global__ void __launch_bounds__(1024, 1) hmm_forward_scaled_tmem(const FwdParams p) {
    static_assert(RL >= 4 && RL <= 8 && RL % 2 == 0, "register layers");
    extern __shared__ __align__(16) float smem_dyn[];
    __shared__ int s_seq;
    __shared__ float s_warp[32];
    __shared__ int s_warp_i[32];
    __shared__ float s_cl[16];
    __shared__ int s_cl_i[16];
    __shared__ float4 s_A4[kLayers / 4];  // exp(trans2[d]), four layers per 16-byte load
    __shared__ unsigned s_tmem;           // base address of the CTA's tensor memory
    __shared__ __align__(8) unsigned long long s_mbar[4];

    const int tid = threadIdx.x;
    constexpr int NT = 1024;            // this layout always runs 1024 threads per CTA (make_plan)
    const unsigned rank = cluster_ctarank();
    const unsigned CS = cluster_nctarank();
    const int K = p.K;
    const int Kq = K >> 2;
    const int M = NT;
    const int g = (rank * NT + tid) * 4;
    const int lane = tid & 31, warp = tid >> 5, nwarps = (NT + 31) >> 5;

    constexpr unsigned NB = ASYNC ? 4u : 2u;                          // layer-0 buffers
    float *a0x = smem_dyn;                                            // [NB][4][M] mantissas
    int *a0w = reinterpret_cast<int *>(smem_dyn + NB * 4 * M);        // [NB][4][M/4] sender exponents

    // tensor memory: the 8 warps that share a lane quarter take 64 columns each; a thread's
    // columns 0..31 hold layers 8..15 (4 k-mers each), columns 32..47 exp(trans1) for j = 0..3
    if (warp == 0) tmem_alloc_all(&s_tmem);
    tmem_publish();
    const unsigned tm_all = s_tmem;
    const unsigned tm = tmem_warp_base(tm_all, warp, 64 * (warp >> 2));
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float4 v = __ldg(reinterpret_cast<const float4 *>(p.trans1) + (j * Kq + (g >> 2)));
        tmem_st4(tm + 4 * (kLayers - RL) + 4 * j, make_float4(fast_exp(v.x), fast_exp(v.y), fast_exp(v.z), fast_exp(v.w)));
    }
    tmem_wait_st();
    if (tid < kLayers) reinterpret_cast<float *>(s_A4)[tid] = expf(__ldg(p.trans2 + tid));
    unsigned dstx0, dstw0;
    {
        const int dj = g / Kq, rem = g % Kq;
        const int dr = rem / M, di = rem % M;
        dstx0 = map_to_rank(smem_u32(a0x) + 4u * (dj * M + di), dr);
        dstw0 = map_to_rank(smem_u32(a0w) + 4u * (dj * (M >> 2) + (di >> 2)), dr);
    }
    const unsigned bufx_bytes = 16u * M, bufw_bytes = 4u * M;
    const unsigned mbar0 = smem_u32(&s_mbar[0]);
    unsigned rmbar0 = 0;      // mbarrier 0 of the CTA that consumes my layer 0
    unsigned phase = 0;       // bit b: parity to wait for on mbarrier b
    bool dead = false;        // a wait ran out: stop waiting, keep the trip counts
    if constexpr (ASYNC) {
        rmbar0 = map_to_rank(mbar0, (unsigned)((g % Kq) / M));
        if (tid == 0) {
            for (int b2 = 0; b2 < 4; ++b2)
                asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(mbar0 + 8u * b2));
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
    }
    // layer 0 of this thread (4 mantissas and the thread's exponent) to buffer b of its consumer
    auto send = [&](unsigned b2, float v0, float v1, float v2, float v3, int w) {
        if constexpr (ASYNC) {
            if (tid == 0)   // the bytes this CTA will receive in that buffer
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar0 + 8u * b2), "r"(20u * M) : "memory");
            asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];"
                         ::"r"(dstx0 + b2 * bufx_bytes), "f"(v0), "f"(v1), "f"(v2), "f"(v3), "r"(rmbar0 + 8u * b2) : "memory");
            asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.s32 [%0], %1, [%2];"
                         ::"r"(dstw0 + b2 * bufw_bytes), "r"(w), "r"(rmbar0 + 8u * b2) : "memory");
        } else {
            st_cluster_v4(dstx0 + b2 * bufx_bytes, v0, v1, v2, v3);
            st_cluster_s32(dstw0 + b2 * bufw_bytes, w);
            cluster_arrive();
        }
    };
    // layer 0 of every producer has landed in buffer b
    auto receive = [&](unsigned b2) {
        if constexpr (ASYNC) {
            if (!dead && !fwd_mbar_wait(mbar0 + 8u * b2, (phase >> b2) & 1u)) {
                dead = true;
                flag_wait_timeout(p.host_flag);
            }
            phase ^= 1u << b2;
        } else {
            cluster_wait();
        }
    };
    const unsigned cl_addr = smem_u32(s_cl);
    const unsigned cli_addr = smem_u32(s_cl_i);
    // emission factors: from the table of exponentials a prologue kernel left in library scratch
    // (same exponential, taken once per table entry instead of once per use), else from the log table
    const float *etab = LIN ? p.output_lin : p.output_prob;

    first_position(p, CS, tid, &s_seq);
    for (;;) {
        const int seq = next_sequence(p, rank, CS, tid, &s_seq);
        if (seq < 0) break;

        long long len = p.lens[seq];
        if (len < 1 || len > p.maxlen) {
            if (tid == 0 && rank == 0) atomicOr(&g_status, 1u);
            len = len < 1 ? 1 : p.maxlen;
        }
        const uint8_t *obs = p.data + static_cast<long long>(seq) * p.maxlen;
        const int T_len = static_cast<int>(len);
        bool bad_obs = false;   // an observation byte outside the emission table was met

        // ---- t = 0: x = exp(initial_prob) * exp(emission), W = 0 ------------------------
        float2 x[RL][2];
        int o_next;
        int W = 0;       // exponent shared by this thread's 64 states
        int kt;          // exponent of the largest mantissa (magnitude hint)
        {
            const int o0 = obs_at(p, obs, 0, bad_obs);
            o_next = obs_at(p, obs, T_len > 1 ? 1 : 0, bad_obs);
            const float4 e0 = __ldg(reinterpret_cast<const float4 *>(etab + (long long)o0 * K + g));
            const float el[4] = {LIN ? e0.x : fast_exp(e0.x), LIN ? e0.y : fast_exp(e0.y),
                                 LIN ? e0.z : fast_exp(e0.z), LIN ? e0.w : fast_exp(e0.w)};
            float m = 0.0f;
#pragma unroll
            for (int d = 0; d < kLayers; ++d) {
                const float4 v = __ldg(reinterpret_cast<const float4 *>(p.initial_prob + d * K + g));
                const float4 r = make_float4(fast_exp(v.x) * el[0], fast_exp(v.y) * el[1], fast_exp(v.z) * el[2],
                                             fast_exp(v.w) * el[3]);
                m = max3(m, fmaxf(r.x, r.y), fmaxf(r.z, r.w));
                if (d < RL) {
                    x[d][0] = make_float2(r.x, r.y);
                    x[d][1] = make_float2(r.z, r.w);
                } else {
                    tmem_st4(tm + 4 * (d - RL), r);
                }
            }
            kt = exponent_of(m);
            tmem_wait_st();
        }
        send(0u, x[0][0].x, x[0][0].y, x[0][1].x, x[0][1].y, W);

        // One time step; Q = (t - 1) mod 4 is a compile-time constant (the loop below is unrolled four
        // times), so the exchange buffers, their mbarriers and the phase bits are addressed with
        // immediates and the every-fourth-step maximum needs no test.
        auto step = [&](const int t, auto qtag) {
            constexpr unsigned Q = decltype(qtag)::value;
            // this step's emission slice (in flight while the exchange completes); the observation after it
            const float4 e = __ldg(reinterpret_cast<const float4 *>(etab + (long long)o_next * K + g));
            o_next = obs_at(p, obs, t + 1 < T_len ? t + 1 : T_len - 1, bad_obs);
            // the transition columns, in flight while the exchange completes
            float4 t0, t1, t2, t3;
            tmem_ld16(tm + 4 * (kLayers - RL), t0, t1, t2, t3);

            constexpr unsigned buf = Q % NB;   // buffer that holds the previous step's layer 0
            receive(buf);
            const float *px = a0x + buf * 4 * M + tid;
            const int *pw = a0w + buf * M + (tid >> 2);
            const float xa0 = px[0], xa1 = px[M], xa2 = px[2 * M], xa3 = px[3 * M];
            const int wp0 = pw[0], wp1 = pw[M >> 2], wp2 = pw[2 * (M >> 2)], wp3 = pw[3 * (M >> 2)];

            // magnitude of each incoming value = sender exponent + exponent field of its mantissa;
            // the new exponent is the largest magnitude this thread is about to combine
            const int ea0 = xa0 > 0.0f ? wp0 + exponent_of(xa0) : kExpFloor - 200;
            const int ea1 = xa1 > 0.0f ? wp1 + exponent_of(xa1) : kExpFloor - 200;
            const int ea2 = xa2 > 0.0f ? wp2 + exponent_of(xa2) : kExpFloor - 200;
            const int ea3 = xa3 > 0.0f ? wp3 + exponent_of(xa3) : kExpFloor - 200;
            int Wn = max(max(ea0, ea1), max(ea2, ea3));
            Wn = max(Wn, W + kt);
            Wn = max(Wn, kExpFloor);
            // incoming values relative to 2^Wn (a power-of-two factor: exact); Wn >= wp + exponent, so
            // the product stays below 2; below 2^-126 it flushes to zero
            const float2 y0 = dup2(xa0 * pow2_clamped(wp0 - Wn)), y1 = dup2(xa1 * pow2_clamped(wp1 - Wn));
            const float2 y2 = dup2(xa2 * pow2_clamped(wp2 - Wn)), y3 = dup2(xa3 * pow2_clamped(wp3 - Wn));
            const float2 own = dup2(pow2_clamped(W - Wn));
            float2 QE[2], Eo[2];
            {
                tmem_wait_ld(t0, t1, t2, t3);
                const float2 q0 = fma2(make_float2(t3.x, t3.y), y3, fma2(make_float2(t2.x, t2.y), y2,
                                  fma2(make_float2(t1.x, t1.y), y1, mul2(make_float2(t0.x, t0.y), y0))));
                const float2 q1 = fma2(make_float2(t3.z, t3.w), y3, fma2(make_float2(t2.z, t2.w), y2,
                                  fma2(make_float2(t1.z, t1.w), y1, mul2(make_float2(t0.z, t0.w), y0))));
                const float2 el2[2] = {LIN ? make_float2(e.x, e.y) : make_float2(fast_exp(e.x), fast_exp(e.y)),
                                       LIN ? make_float2(e.z, e.w) : make_float2(fast_exp(e.z), fast_exp(e.w))};
                QE[0] = mul2(q0, el2[0]);
                QE[1] = mul2(q1, el2[1]);
                Eo[0] = mul2(el2[0], own);
                Eo[1] = mul2(el2[1], own);
                kt = exponent_of(max3(fmaxf(el2[0].x, el2[0].y), el2[1].x, el2[1].y)) + 4;   // the bound; see below
            }
            // layer 0 first: it is what the other CTAs wait for
            // exp(trans2) of four layers per shared-memory load (the shared-memory pipe bounds this kernel)
            float4 a4 = s_A4[0];
            const auto A_of = [&](int d) { return dup2(d % 4 == 0 ? a4.x : d % 4 == 1 ? a4.y : d % 4 == 2 ? a4.z : a4.w); };
            {
                const float2 a = A_of(0);
                x[0][0] = fma2(a, QE[0], mul2(Eo[0], x[1][0]));
                x[0][1] = fma2(a, QE[1], mul2(Eo[1], x[1][1]));
            }
            send((Q + 1u) % NB, x[0][0].x, x[0][0].y, x[0][1].x, x[0][1].y, Wn);
#pragma unroll
            for (int d = 1; d < RL - 1; ++d) {
                if (d % 4 == 0) a4 = s_A4[d / 4];
                const float2 a = A_of(d);
                x[d][0] = fma2(a, QE[0], mul2(Eo[0], x[d + 1][0]));
                x[d][1] = fma2(a, QE[1], mul2(Eo[1], x[d + 1][1]));
            }
            // Layers RL..15 live in tensor memory and are updated in place, two layers per load and per
            // store: pair p = layers (d, d + 1), d = RL + 2p, needs the old values of layers d + 1 and
            // d + 2 (the last pair: old layer 15 twice), which one 8-column load brings; the results
            // replace them in the same registers and leave with one 8-column store. The operands of
            // pair p + 1 are requested as soon as those of pair p have arrived (a wait covers every
            // load in flight), so they travel while pair p is computed; a load never covers columns
            // that a store issued before its wait writes.
            constexpr int NP = (kLayers - RL) / 2;
            float mt = 0.0f;   // largest new mantissa among the tensor-memory layers (Q == 3 only)
            float4 o0, pr[2][2];
            tmem_ld4(tm, o0);                       // old layer RL, for the last register layer
            if (NP > 1) tmem_ld8(tm + 4, pr[0][0], pr[0][1]);
            else tmem_ld4(tm + 4, pr[0][0]);
            if (NP > 1) tmem_wait_ld(o0, pr[0][0], pr[0][1]);
            else tmem_wait_ld(o0, pr[0][0]);
            if (NP > 2) tmem_ld8(tm + 4 * 3, pr[1][0], pr[1][1]);
            else if (NP == 2) tmem_ld4(tm + 4 * 3, pr[1][0]);
            {
                const float2 a = A_of(RL - 1);
                x[RL - 1][0] = fma2(a, QE[0], mul2(Eo[0], make_float2(o0.x, o0.y)));
                x[RL - 1][1] = fma2(a, QE[1], mul2(Eo[1], make_float2(o0.z, o0.w)));
            }
#pragma unroll
            for (int pp = 0; pp < NP; ++pp) {
                float4 (&b)[2] = pr[pp & 1];
                const bool last = pp == NP - 1;
                if (pp > 0) {
                    if (last) tmem_wait_ld(b[0]);
                    else tmem_wait_ld(b[0], b[1]);
                    if (pp + 2 < NP) tmem_ld8(tm + 4 * (2 * pp + 3), pr[(pp + 1) & 1][0], pr[(pp + 1) & 1][1]);
                    else if (pp + 2 == NP) tmem_ld4(tm + 4 * (2 * pp + 3), pr[(pp + 1) & 1][0]);
                }
                const int d = RL + 2 * pp;
                if (d % 4 == 0) a4 = s_A4[d / 4];   // RL is even: a pair never straddles a group of four
                // second layer of the pair first: in the last pair both read old layer 15 (b[0])
                {
                    const float4 &old = last ? b[0] : b[1];
                    float2 v0 = make_float2(old.x, old.y), v1 = make_float2(old.z, old.w);
                    if (last) {
                        const float c = p.gamma_lin;
                        v0.x *= c; v0.y *= c; v1.x *= c; v1.y *= c;
                    }
                    const float2 a = A_of(d + 1);
                    const float2 r0 = fma2(a, QE[0], mul2(Eo[0], v0));
                    const float2 r1 = fma2(a, QE[1], mul2(Eo[1], v1));
                    b[1] = make_float4(r0.x, r0.y, r1.x, r1.y);
                }
                {
                    float2 v0 = make_float2(b[0].x, b[0].y), v1 = make_float2(b[0].z, b[0].w);
                    if (last) {
                        const float c = p.synthetic_lin;
                        v0.x *= c; v0.y *= c; v1.x *= c; v1.y *= c;
                    }
                    const float2 a = A_of(d);
                    const float2 r0 = fma2(a, QE[0], mul2(Eo[0], v0));
                    const float2 r1 = fma2(a, QE[1], mul2(Eo[1], v1));
                    b[0] = make_float4(r0.x, r0.y, r1.x, r1.y);
                }
                tmem_st8(tm + 4 * (2 * pp), b[0], b[1]);
                if constexpr (Q == 3u) {   // the step that takes the exact maximum: the upper layers on their way out
                    mt = max3(mt, fmaxf(b[0].x, b[0].y), fmaxf(b[0].z, b[0].w));
                    mt = max3(mt, fmaxf(b[1].x, b[1].y), fmaxf(b[1].z, b[1].w));
                }
            }
            W = Wn;
            tmem_wait_st();   // the next step reads what this one stored
            // The thread's exponent for the next step follows the largest of its 64 new mantissas. Every
            // fourth step (and the last two, so that a sequence ends on the exponents the exact maximum
            // gives) finds it; the steps between use a bound instead: inputs are
            // below 2 after rescaling, so with transition and duration factors of at most 1 a new value
            // is below 10 x the largest emission factor. The bound only has to hold loosely (fp32 has
            // 2^127 of headroom and the true maximum follows within three steps), and power-of-two
            // rescaling is exact: the values represented do not depend on which exponent was chosen.
            if (Q == 3u || t >= T_len - 2) {
                float m = mt;
#pragma unroll
                for (int d = 0; d < RL; ++d) {
                    m = max3(m, x[d][0].x, x[d][0].y);
                    m = max3(m, x[d][1].x, x[d][1].y);
                }
                if constexpr (Q != 3u) {   // one of the last two steps: the upper layers are read back
#pragma unroll
                    for (int d = 0; d < kLayers - RL; d += 2) {
                        float4 u, v;
                        tmem_ld8(tm + 4 * d, u, v);
                        tmem_wait_ld(u, v);
                        m = max3(m, fmaxf(u.x, u.y), fmaxf(u.z, u.w));
                        m = max3(m, fmaxf(v.x, v.y), fmaxf(v.z, v.w));
                    }
                }
                kt = exponent_of(m);
            }
        };
        {
            int t = 1;
            for (; t + 3 < T_len; t += 4) {
                step(t, std::integral_constant<unsigned, 0u>{});
                step(t + 1, std::integral_constant<unsigned, 1u>{});
                step(t + 2, std::integral_constant<unsigned, 2u>{});
                step(t + 3, std::integral_constant<unsigned, 3u>{});
            }
            if (t < T_len) step(t, std::integral_constant<unsigned, 0u>{});
            if (t + 1 < T_len) step(t + 1, std::integral_constant<unsigned, 1u>{});
            if (t + 2 < T_len) step(t + 2, std::integral_constant<unsigned, 2u>{});
        }
        receive((unsigned)(T_len - 1) % NB);   // the last round is not used, but it must have landed

        // ---- log-likelihood: log(sum of all states) with a common exponent --------------
        int gexp = W + kt;
        gexp = __reduce_max_sync(0xffffffffu, gexp);
        if (lane == 0) s_warp_i[warp] = gexp;
        __syncthreads();
        if (tid < (int)CS) {
            int v = kExpFloor - 200;
            for (int w = 0; w < nwarps; ++w) v = max(v, s_warp_i[w]);
            st_cluster_s32(map_to_rank(cli_addr + 4u * rank, tid), v);
        }
        cluster_arrive();
        cluster_wait();
        int G = kExpFloor - 200;
        for (unsigned r = 0; r < CS; ++r) G = max(G, s_cl_i[r]);
        float tsum = 0.0f;
#pragma unroll
        for (int d = 0; d < RL; ++d) tsum += (x[d][0].x + x[d][0].y) + (x[d][1].x + x[d][1].y);
#pragma unroll
        for (int d = 0; d < kLayers - RL; ++d) {
            float4 v;
            tmem_ld4(tm + 4 * d, v);
            tmem_wait_ld(v);
            tsum += (v.x + v.y) + (v.z + v.w);
        }
        tsum *= pow2_clamped(W - G);
        tsum = pb::warp_sum(tsum);
        if (lane == 0) s_warp[warp] = tsum;
        __syncthreads();
        if (tid < (int)CS) {
            float sacc = 0.0f;
            for (int w = 0; w < nwarps; ++w) sacc += s_warp[w];
            st_cluster_f32(map_to_rank(cl_addr + 4u * rank, tid), sacc);
        }
        cluster_arrive();
        cluster_wait();
        if (rank == 0 && tid == 0) {
            double sacc = 0.0;
            for (unsigned r = 0; r < CS; ++r) sacc += (double)s_cl[r];
            // natural log of sum * 2^G; an impossible sequence (sum == 0) gives NaN like the reference's (-inf) - (-inf)
            p.result[seq] = sacc > 0.0 ? (float)(log(sacc) + (double)G * 0.6931471805599453) : __int_as_float(0x7fc00000);
            flag_bad_observation(bad_obs, true);
        }
        if (p.write_alpha) {
            float *dst_alpha = ((len & 1) ? p.alpha1 : p.alpha2) + (long long)seq * (kLayers * (long long)K);
            const float wl = (float)W * kLn2;
#pragma unroll
            for (int d = 0; d < kLayers; ++d) {
                float4 s4 = make_float4(x[d % RL][0].x, x[d % RL][0].y,
                                        x[d % RL][1].x, x[d % RL][1].y);
                if (d >= RL) {
                    tmem_ld4(tm + 4 * (d - RL), s4);
                    tmem_wait_ld(s4);
                }
                float4 v;
                v.x = fast_log(s4.x) + wl;
                v.y = fast_log(s4.y) + wl;
                v.z = fast_log(s4.z) + wl;
                v.w = fast_log(s4.w) + wl;
                *reinterpret_cast<float4 *>(dst_alpha + (long long)d * K + g) = v;
            }
        }
        // the next pop starts with a full cluster barrier
    }
    tmem_publish();   // every warp is done with its columns
    if (warp == 0) tmem_free_all(tm_all);
}

// ---- streaming kernels --------------------------------------------------------
__global__ void hmm_stream_init(const FwdParams p) {
    const long long N = (long long)kLayers * p.K;
    const long long state = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int inst = blockIdx.y;
    if (state >= N) return;
    bool bad_obs = false;
    const int o = obs_at(p, p.data + (long long)inst * p.maxlen, 0, bad_obs);
    flag_bad_observation(bad_obs, state == 0);
    p.alpha1[inst * N + state] = p.initial_prob[state] + p.output_prob[(long long)o * p.K + state % p.K];
}

__global__ void hmm_stream_step(const FwdParams p, int t) {
    const int K = p.K;
    const long long N = (long long)kLayers * K;
    const long long state = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int inst = blockIdx.y;
    if (state >= N) return;
    if (t >= p.lens[inst]) return;  // benchmarks/forward.py:113: no write past the end
    const float *src = ((t & 1) ? p.alpha1 : p.alpha2) + inst * N;
    float *dst = ((t & 1) ? p.alpha2 : p.alpha1) + inst * N;
    bool bad_obs = false;
    const int o = obs_at(p, p.data + (long long)inst * p.maxlen, t, bad_obs);
    flag_bad_observation(bad_obs, state == 0);
    const int s = static_cast<int>(state % K);
    const int d = static_cast<int>(state / K);
    const int Kq = K >> 2;
    const int low = s >> 2;
    const float t2 = __ldg(p.trans2 + d);
    const float p1 = (p.trans1[(0 * Kq + low) * 4 + (s & 3)] + t2) + src[0 * Kq + low];
    const float p2 = (p.trans1[(1 * Kq + low) * 4 + (s & 3)] + t2) + src[1 * Kq + low];
    const float p3 = (p.trans1[(2 * Kq + low) * 4 + (s & 3)] + t2) + src[2 * Kq + low];
    const float p4 = (p.trans1[(3 * Kq + low) * 4 + (s & 3)] + t2) + src[3 * Kq + low];
    float p5;
    if (d == 15) p5 = p.gamma + src[state];
    else if (d == 14) p5 = p.synthetic + src[state + K];
    else p5 = 0.0f + src[state + K];
    dst[state] = lse5_reference(p1, p2, p3, p4, p5) + p.output_prob[(long long)o * K + s];
}

__global__ void hmm_stream_final(const FwdParams p) {
    __shared__ float s_red[32];
    __shared__ float s_bcast;
    const int inst = blockIdx.x;
    const long long N = (long long)kLayers * p.K;
    long long len = p.lens[inst];
    const float *alpha = ((len & 1) ? p.alpha1 : p.alpha2) + inst * N;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float m = -INFINITY;
    for (long long i = threadIdx.x; i < N; i += blockDim.x) m = fmaxf(m, alpha[i]);
    m = pb::warp_max(m);
    if (lane == 0) s_red[warp] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float v = -INFINITY;
        for (int w = 0; w < nw; ++w) v = fmaxf(v, s_red[w]);
        s_bcast = v;
    }
    __syncthreads();
    const float gmax = s_bcast;
    float s = 0.0f;
    for (long long i = threadIdx.x; i < N; i += blockDim.x) s += fast_exp(alpha[i] - gmax);
    s = pb::warp_sum(s);
    __syncthreads();
    if (lane == 0) s_red[warp] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float v = 0.0f;
        for (int w = 0; w < nw; ++w) v += s_red[w];
        p.result[inst] = gmax + fast_log(v);
    }
}

// ---- host side ------------------------------------------------------------------
struct Plan {
    int kpt = 0, nt = 0, cs = 0;
    bool split = false;  // layers 8..15 in shared memory, 1024 threads per CTA
    bool scaled = false; // extended-range linear arithmetic instead of log space
    bool cta = false;    // one 256-thread CTA per sequence, packed arithmetic (K = 1024)
    bool tmem = false;   // scaled split layout with layers 8..15 and transition columns in tensor memory
    bool exptab = false; // scaled tensor-memory kernel reads exp(output_prob) from a table prepared per call
};

// Picks (k-mers per thread, threads per CTA, CTAs per cluster) with
// K = kpt*nt*cs, or returns false when only the streaming kernel applies.
// `allow_split` permits the register/shared split layout (factored log form
// only); `need_kpt4` is set by the scaled kernel, which owns 4 k-mers per thread.
// Shapes for K <= 1024 follow measurements on the 100-sequence 5-mer workload:
// small CTAs in clusters of 4 spread one sequence over several SMs.
bool make_plan(long long K, Plan *pl, bool allow_split, bool need_kpt4 = false) {
    if (K < 4 || (K & (K - 1)) != 0) return false;  // K = 4^k
    long long kpt = (K >= 4096 || need_kpt4) ? 4 : 1;
    if (need_kpt4 && K < 1024) return false;
    long long nt_max = kpt == 4 ? (K <= 1024 ? 64 : 512) : (K == 1024 ? 256 : 1024);
    if (const char *env = getenv("PARPY_B200_FWD_KPT")) {
        const int v = atoi(env);
        if ((v == 1 || v == 4) && K >= 16 && !(need_kpt4 && v != 4)) {
            kpt = v;
            nt_max = kpt == 4 ? 512 : 1024;
        }
    }
    if (const char *env = getenv("PARPY_B200_FWD_NT")) {
        const long long w = atoll(env);
        if (w >= 32 && w <= (kpt == 4 ? 512 : 1024) && (w & (w - 1)) == 0) nt_max = w;
    }
    const long long threads = K / kpt;
    if (threads < 32) return false;  // whole warps only; tiny state spaces stream
    long long nt = std::min<long long>(threads, nt_max);
    long long cs = threads / nt;
    bool split = false;
    // Large state spaces: the split layout (1024 threads x 4 k-mers per CTA) halves
    // the CTAs a sequence needs, so clusters pack the GPCs without idle SMs.
    bool want_split = allow_split && kpt == 4 && K >= 4096;
    if (const char *env = getenv(need_kpt4 ? "PARPY_B200_SCALED_SPLIT" : "PARPY_B200_FWD_SPLIT"))
        want_split = want_split && atoi(env) != 0;
    if (want_split) {
        nt = 1024;
        cs = K / 4 / 1024;
        split = true;
    }
    if (cs > 16) return false;
    bool cta = false;
    if (allow_split && !need_kpt4 && K == 1024 && !getenv("PARPY_B200_FWD_KPT") && !getenv("PARPY_B200_FWD_NT")) {
        int packed = 1;
        if (const char *env = getenv("PARPY_B200_FWD_PACKED")) packed = atoi(env);
        if (packed) {
            kpt = 4;
            nt = 256;
            cs = 1;
            cta = true;
        }
    }
    pl->kpt = (int)kpt;
    pl->nt = (int)nt;
    pl->cs = (int)cs;
    pl->split = split;
    pl->cta = cta;
    return true;
}

using ResidentKernel = void (*)(const FwdParams);

// Completes a plan made by make_plan: where tensor memory takes the place of shared memory.
// Every entry point calls this, so that the same state space always runs the same kernel.
// PARPY_B200_FWD_POLY (the scalar-twin comparisons of the tests) selects the kernels that keep
// layers 8..15 in shared memory; PARPY_B200_FWD_TMEM=0 / PARPY_B200_SCALED_TMEM=0 do so too.
void finish_plan(Plan *pl, bool five, bool scaled) {
    pl->scaled = scaled;
    pl->tmem = false;
    if (!pl->split || five) return;
    int packed = 1;
    if (const char *env = getenv("PARPY_B200_FWD_PACKED")) packed = atoi(env);
    const char *env = getenv(scaled ? "PARPY_B200_SCALED_TMEM" : "PARPY_B200_FWD_TMEM");
    pl->tmem = (env == nullptr || atoi(env) != 0) && (scaled || (packed && getenv("PARPY_B200_FWD_POLY") == nullptr));
}

ResidentKernel pick_kernel(const Plan &pl, bool five) {
    const int kpt = pl.kpt;
    int rl = 0;   // layers kept in registers by the tensor-memory kernels (0: the kernel's default)
    if (const char *env = getenv("PARPY_B200_FWD_REGLAYERS")) rl = atoi(env);
    if (pl.scaled && pl.tmem) {
        // Measured on the benchmark workload (state-steps/s), layers in registers / exchange:
        // 6 / st.async 4.76e12, 4 / st.async 4.65e12, 8 / st.async 4.46e12, 6 / barrier 4.44e12,
        // 4 / barrier 4.22e12, 8 / barrier 4.14e12; shared memory instead of tensor memory 3.77e12.
        bool async_x = pl.cs >= 2 && pl.cs <= 8;
        if (const char *env = getenv("PARPY_B200_SCALED_ASYNC")) async_x = async_x && atoi(env) != 0;
        if (async_x && pl.exptab && rl != 8) return rl == 4 ? hmm_forward_scaled_tmem<4, true, true> : hmm_forward_scaled_tmem<6, true, true>;
        if (async_x) return rl == 4 ? hmm_forward_scaled_tmem<4, true> : rl == 8 ? hmm_forward_scaled_tmem<8, true> : hmm_forward_scaled_tmem<6, true>;
        return rl == 4 ? hmm_forward_scaled_tmem<4, false> : rl == 8 ? hmm_forward_scaled_tmem<8, false> : hmm_forward_scaled_tmem<6, false>;
    }
    if (pl.scaled) return pl.split ? hmm_forward_scaled_split : hmm_forward_scaled;
    if (pl.cta && !five) {
        if (const char *mk = getenv("PARPY_B200_FWD_MASKS")) {
            unsigned ex = 0, lg = 0;
            if (sscanf(mk, "%x:%x", &ex, &lg) == 2) {
#define PB_MASKS(E, L) if (ex == E && lg == L) return hmm_forward_packed_cta<E, L>
                PB_MASKS(0x0000u, 0xEEECu);
                PB_MASKS(0x0000u, 0xFFFEu);
                PB_MASKS(0xAAAAu, 0x5554u);
                PB_MASKS(0xAAAAu, 0x5555u);
                PB_MASKS(0x0000u, 0xAAAAu);
                PB_MASKS(0x8888u, 0x7776u);
#undef PB_MASKS
            }
        }
        // Measured on 100 sequences x 2000 steps: logarithm of 11 layers as polynomial (mask 0xEEEC, all
        // exponentials on the MUFU pipe) 2.64 ms; of the odd layers 2.71; of all but layer 0 2.69;
        // exponential of the odd layers as polynomial (the earlier default) 2.72; both kinds mixed 2.84-2.93.
        if (getenv("PARPY_B200_FWD_POLY") == nullptr) {
            const char *fin = getenv("PARPY_B200_FWD_FINITE");   // finite arithmetic unless set to 0
            if (fin && atoi(fin) == 0) return hmm_forward_packed_cta<0x0000u, 0xEEECu>;
            // finite arithmetic 2.54 -> 2.48 ms, degree-5 logarithm polynomial 2.42 ms (with 13 layers: 2.44)
            if (const char *l6 = getenv("PARPY_B200_FWD_LG6")) {
                if (atoi(l6) == 0) return hmm_forward_packed_cta<0x0000u, 0xEEECu, true>;
                if (atoi(l6) == 2) return hmm_forward_packed_cta<0x0000u, 0xFEFCu, true, true>;
            }
            return hmm_forward_packed_cta<0x0000u, 0xEEECu, true, true>;
        }
        const int npoly = atoi(getenv("PARPY_B200_FWD_POLY"));   // exponential masks only
        switch (npoly) {
            case 0: return hmm_forward_packed_cta<0x0000u>;
            case 5: return hmm_forward_packed_cta<0x2492u>;
            case 12: return hmm_forward_packed_cta<0xEEEEu>;
            case 14: return hmm_forward_packed_cta<0xFEFEu>;
            case 16: return hmm_forward_packed_cta<0xFFFFu>;
            case 7: return hmm_forward_packed_cta<0x5554u>;
            case 10: return hmm_forward_packed_cta<0x6DB6u>;
            default: return hmm_forward_packed_cta<0xAAAAu>;
        }
    }
    if (pl.split && !five) {
        int packed = 1;
        if (const char *env = getenv("PARPY_B200_FWD_PACKED")) packed = atoi(env);
        // "PARPY_B200_FWD_MASKS=<exp mask>:<log mask>" (hex) picks, among the compiled combinations,
        // which layers take their exponential / their logarithm on the FMA pipe
        unsigned ex = 0, lg = 0;
        bool masks = false;
        if (const char *mk = getenv("PARPY_B200_FWD_MASKS")) masks = sscanf(mk, "%x:%x", &ex, &lg) == 2;
        if (packed && pl.tmem) {
            // The log-space kernel for 4096 k-mers and more. Measured on the benchmark workload (state-steps/s):
            // logarithm of layers 2,3,5,6,7,9,10,11,13,14,15 as polynomial, 4 layers in registers
            // 1.911e12; same with 8 in registers 1.905e12, 6: 1.891e12; layers 1,2,3,5,... (12) 1.897e12;
            // exponential of the even layers but 0 as polynomial and no logarithm (the earlier
            // default) 1.835e12 in tensor memory, 1.817e12 in shared memory.
            // Finite arithmetic (log 0 kept as -1e25 inside the kernel, -inf again in what it writes)
            // drops the NaN clamps of every log-sum-exp: 1.999e12 against 1.923e12 state-steps/s.
            // PARPY_B200_FWD_FINITE=0 selects the kernel that computes on -inf itself.
            const char *fin = getenv("PARPY_B200_FWD_FINITE");
            if (masks && !(fin && atoi(fin) == 0)) {
                // finite arithmetic with other masks (degree-6 polynomial; measured: 0xEEE8 2.012e12, 0xEEEC
                // 2.001e12, 0xEEEE 1.986e12, 0xFEFE 1.983e12, 0xEEC8 1.984e12, 0xFFFE 1.969e12, 0xECC8
                // 1.961e12, 0xAAAA 1.950e12) and the degree-5 polynomial on all layers but 0
                const char *l6 = getenv("PARPY_B200_FWD_LG6");
                if (l6 && atoi(l6) != 0 && ex == 0 && lg == 0xFFFEu) return hmm_forward_packed<0x0000u, 0xFFFEu, true, 4, true, true>;
                if (ex == 0 && lg == 0xEEEEu) return hmm_forward_packed<0x0000u, 0xEEEEu, true, 4, true>;
                if (ex == 0 && lg == 0xAAAAu) return hmm_forward_packed<0x0000u, 0xAAAAu, true, 4, true>;
            }
            if (masks) {
                if (ex == 0x0000u && lg == 0xEEEEu) return rl == 8 ? hmm_forward_packed<0x0000u, 0xEEEEu, true, 8> : hmm_forward_packed<0x0000u, 0xEEEEu, true, 4>;
                if (ex == 0x5554u && lg == 0x0000u) return rl == 4 ? hmm_forward_packed<0x5554u, 0x0000u, true, 4> : hmm_forward_packed<0x5554u, 0x0000u, true, 8>;
            }
            if ((rl == 0 || rl == 4) && !(fin && atoi(fin) == 0)) {
                // With the shorter logarithm polynomial (degree 5) 13 layers take it: 2.050e12; the same
                // masks measured with it: 0xFEFE 2.049e12, 0xFFFC 2.047e12, 0xEEFC 2.041e12, 0xFFFE 2.037e12,
                // 0xFCFC 2.037e12, 0xFEEC 2.032e12, 0xEEEC 2.025e12. PARPY_B200_FWD_LG6=0: degree 6, 11 layers.
                const char *l6 = getenv("PARPY_B200_FWD_LG6");
                if (l6 && atoi(l6) == 0) return hmm_forward_packed<0x0000u, 0xEEECu, true, 4, true>;
                return hmm_forward_packed<0x0000u, 0xFEFCu, true, 4, true, true>;
            }
            return rl == 8 ? hmm_forward_packed<0x0000u, 0xEEECu, true, 8>
                 : rl == 6 ? hmm_forward_packed<0x0000u, 0xEEECu, true, 6> : hmm_forward_packed<0x0000u, 0xEEECu, true, 4>;
        }
        if (packed) {
            // layers 8..15 in shared memory. Measured (state-steps/s), logarithm masks with all
            // exponentials on the MUFU pipe: 0xEEEC 1.888e12, 0x6EEE 1.881e12, 0x3FFC 1.876e12, 0xEEEE
            // 1.870e12, 0xFEFE 1.863e12, 0xFFF0 1.862e12, 0xAAAA 1.859e12, 0x7FFE 1.858e12, 0xFFFE 1.845e12,
            // 0xFFFF 1.841e12; with exponentials as well: 0x1110:0xEEEE 1.785e12, 0x5554:0xAAAA 1.724e12.
            // Exponential masks alone: even layers but 0 (7 layers) 1.817e12, layers 1..8 1.793e12, odd
            // layers 1.764e12, 9 layers 1.747e12, 10 layers 1.751e12, 11 layers 1.712e12.
            if (masks) {
#define PB_MASKS(E, L) if (ex == E && lg == L) return hmm_forward_packed<E, L>
                PB_MASKS(0x0000u, 0xEEEEu);
                PB_MASKS(0x0000u, 0xFEFEu);
                PB_MASKS(0x0000u, 0xFFFEu);
                PB_MASKS(0x0000u, 0xFFFFu);
                PB_MASKS(0x5554u, 0xAAAAu);
                PB_MASKS(0x0000u, 0xAAAAu);
                PB_MASKS(0x0000u, 0x6EEEu);
#undef PB_MASKS
            }
            if (const char *env = getenv("PARPY_B200_FWD_POLY")) {
                switch (atoi(env)) {   // exponential masks only: the scalar kernel's twins
                    case 0: return hmm_forward_packed<0x0000u>;
                    case 5: return hmm_forward_packed<0x2492u>;   // layers 1,4,7,10,13
                    case 8: return hmm_forward_packed<0xAAAAu>;   // odd layers
                    case 9: return hmm_forward_packed<0xAD5Au>;   // all but 0,2,5,7,9,12,14
                    case 10: return hmm_forward_packed<0x6DB6u>;  // all but 0,3,6,9,12,15
                    case 11: return hmm_forward_packed<0xDB6Eu>;  // all but 0,4,7,10,13
                    case 12: return hmm_forward_packed<0xEEEEu>;  // all but 0,4,8,12
                    default: return hmm_forward_packed<0x5554u>;  // 7: even layers but 0
                }
            }
            return hmm_forward_packed<0x0000u, 0xEEECu>;
        }
        int npoly = 5;   // how many of the 16 layers take the polynomial exponential
        if (const char *env = getenv("PARPY_B200_FWD_POLY")) npoly = atoi(env);
        switch (npoly) {
            case 0: return hmm_forward_split<0x0000u>;
            case 4: return hmm_forward_split<0x2222u>;   // layers 1,5,9,13
            case 6: return hmm_forward_split<0x4A52u>;   // layers 1,4,6,9,11,14
            case 8: return hmm_forward_split<0xAAAAu>;   // odd layers
            default: return hmm_forward_split<0x2492u>;  // layers 1,4,7,10,13
        }
    }
    if (kpt == 4) return five ? hmm_forward_resident<4, true> : hmm_forward_resident<4, false>;
    return five ? hmm_forward_resident<1, true> : hmm_forward_resident<1, false>;
}

int32_t resident_config(const Plan &pl, bool five, cudaLaunchConfig_t *cfg,
                        cudaLaunchAttribute *attr, int *max_clusters, ResidentKernel *kern) {
    ResidentKernel k = pick_kernel(pl, five);
    size_t smem = size_t(2) * 4 * (size_t(pl.nt) * pl.kpt / 4) * sizeof(float);
    if (pl.cta && !five && !pl.scaled) smem = 0;  // static shared memory only
    else if (pl.scaled && pl.tmem)    // the exchange only: mantissas + sender exponents, up to four buffers
        smem = size_t(20) * pl.nt * sizeof(float);
    else if (pl.scaled && pl.split)   // mantissas + sender exponents, 3 transition columns, layers 8..15
        smem = size_t(10) * pl.nt * sizeof(float) + size_t(3 + 8) * pl.nt * sizeof(float4);
    else if (pl.scaled) smem *= 2;  // mantissas + exponents
    else if (pl.split && !five && !pl.tmem) smem += size_t(4 + 8) * pl.nt * sizeof(float4);  // transition columns + layers 8..15
    if (pl.cs > 8) PB_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    PB_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    memset(cfg, 0, sizeof(*cfg));
    cfg->gridDim = dim3(pl.cs, 1, 1);
    cfg->blockDim = dim3(pl.nt, 1, 1);
    cfg->dynamicSmemBytes = smem;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = pl.cs;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg->attrs = attr;
    cfg->numAttrs = 1;
    int n = 0;
    PB_CUDA(cudaOccupancyMaxActiveClusters(&n, k, cfg));
    if (n < 1) {
        pb::set_error("no resident cluster of %d CTAs x %d threads fits this device", pl.cs, pl.nt);
        return PB_ERR_UNSUPPORTED;
    }
    *max_clusters = n;
    *kern = k;
    return PB_OK;
}

// Scheduling scratch of one call: order[B] (256-byte aligned), the queue head, the segment table.
struct SchedScratch {
    int *order, *counter, *seg;
};
size_t sched_bytes(int B) { return ((size_t(B) * sizeof(int) + 255) & ~size_t(255)) + kSchedTailBytes; }
SchedScratch sched_layout(void *base, size_t order_bytes) {
    char *c = static_cast<char *>(base);
    return {reinterpret_cast<int *>(c), reinterpret_cast<int *>(c + order_bytes),
            reinterpret_cast<int *>(c + order_bytes + 256)};
}

// Launches the scheduling prologue for `clusters` resident clusters and fills in the
// schedule fields of `p`. Batches up to kSortLimit get the static balanced schedule.
int32_t launch_schedule(FwdParams *p, const SchedScratch &sc, int clusters, int *cluster_of,
                        cudaStream_t stream) {
    const bool fixed = p->B <= kSortLimit && clusters <= kMaxBins;
    p->order = sc.order;
    p->counter = sc.counter;
    p->seg = fixed ? sc.seg : nullptr;
    const size_t smem = fixed ? size_t(p->B) * 8 : 0;
    int max_rounds = 512;   // repair rounds at most
    if (const char *env = getenv("PARPY_B200_SCHED_ROUNDS")) max_rounds = atoi(env);
    hmm_schedule<<<1, 1024, smem, stream>>>(p->lens, p->B, fixed ? clusters : 0, sc.order, sc.counter, sc.seg,
                                             cluster_of, max_rounds);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

// One word of pinned host memory per device that a kernel sets when a bounded wait runs out
// (flag_wait_timeout). The forward entry looks at it before launching: a call whose exchange
// timed out returned without an error (launches are asynchronous), so the next call on the device
// reports it instead of letting invalid results pass silently; reading the status word clears it.
// Allocated on the first call per device; without it (allocation refused) only the status word is left.
unsigned *host_timeout_flag(int device) {
    static std::mutex mu;
    static unsigned *flags[64] = {};
    static bool tried[64] = {};
    if (device < 0 || device >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!tried[device]) {
        tried[device] = true;
        void *ptr = nullptr;
        if (cudaHostAlloc(&ptr, sizeof(unsigned), cudaHostAllocPortable | cudaHostAllocMapped) == cudaSuccess) {
            flags[device] = static_cast<unsigned *>(ptr);
            *flags[device] = 0u;
        } else {
            (void)cudaGetLastError();
        }
    }
    return flags[device];
}

// Arithmetic of a call that names none (flags without SCALED / LOG_SPACE / FIVE_TERM / STREAMING /
// WRITE_ALPHA) on 4096 k-mers and more: the scaled kernel. On the benchmark batch at full length it is
// 2.3e-6 from the fp32 oracle where the log-space kernel is 1.5e-6 (the oracle's own distance from a
// float64 evaluation is of that order), and it scores the batch 2.7 times as fast. State spaces of
// 1024 k-mers and fewer keep log-space arithmetic: the reference ships golden vectors for them and its
// own test asks for rtol 1e-5 against fp32 log-space results, which rounding-for-rounding agreement
// needs. A call that asks for alpha gets log space too (the scaled kernel flushes states more than
// about 2^-110 below their thread's largest to log 0). PARPY_B200_FWD_DEFAULT=log restores log space everywhere.
bool default_is_scaled() {
    if (const char *env = getenv("PARPY_B200_FWD_DEFAULT")) return strcmp(env, "log") != 0;
    return true;
}

int32_t forward_impl(float gamma, const float *initial_prob, int64_t num_states,
                     const float *output_prob, float synthetic_248, const float *trans1,
                     const float *trans2, const void *data, const int64_t *lens, int64_t maxlen,
                     int64_t num_instances, float *result, float *alpha1, float *alpha2,
                     uint32_t flags, int64_t n_obs, cudaStream_t stream) {
    PB_REQUIRE(num_states >= 64 && num_states % 64 == 0,
               "forward: num_states=%lld must be a positive multiple of 64", (long long)num_states);
    PB_REQUIRE(num_states <= (1LL << 30), "forward: num_states=%lld too large", (long long)num_states);
    PB_REQUIRE(num_instances >= 0 && num_instances <= 0x7fffffffLL,
               "forward: num_instances=%lld out of range", (long long)num_instances);
    PB_REQUIRE(maxlen >= 1 && maxlen <= 0x7fffffffLL, "forward: maxlen=%lld out of range", (long long)maxlen);
    PB_REQUIRE(n_obs >= 0, "forward: n_obs=%lld is negative", (long long)n_obs);
    if (num_instances == 0) return PB_OK;
    PB_REQUIRE(initial_prob && output_prob && trans1 && trans2 && data && lens && result,
               "forward: null table, observation or result pointer");
    const long long K = num_states / kLayers;
    const bool streaming_forced = flags & PARPY_B200_FWD_STREAMING;
    const bool write_alpha = flags & PARPY_B200_FWD_WRITE_ALPHA;
    const bool five = flags & PARPY_B200_FWD_FIVE_TERM;
    const bool log_space = flags & PARPY_B200_FWD_LOG_SPACE;
    bool scaled = flags & PARPY_B200_FWD_SCALED;
    PB_REQUIRE(!(five && scaled), "forward: FIVE_TERM and SCALED exclude each other");
    PB_REQUIRE(!(log_space && scaled), "forward: LOG_SPACE and SCALED exclude each other");
    // Which arithmetic a call without an explicit choice gets: see default_is_scaled().
    const bool scaled_by_default = !scaled && !log_space && !five && !streaming_forced && !write_alpha &&
                                   K >= 4096 && default_is_scaled();
    scaled = scaled || scaled_by_default;
    PB_REQUIRE(!write_alpha || (alpha1 && alpha2), "forward: WRITE_ALPHA needs alpha1 and alpha2");

    pb::DeviceInfo dev;
    int32_t rc = pb::device_info(&dev);
    if (rc) return rc;
    PB_REQUIRE(dev.cc_major >= 10, "forward: needs compute capability 10.x, found %d.%d",
               dev.cc_major, dev.cc_minor);

    FwdParams p{};
    p.initial_prob = initial_prob;
    p.output_prob = output_prob;
    p.trans1 = trans1;
    p.trans2 = trans2;
    p.data = static_cast<const uint8_t *>(data);
    p.lens = lens;
    p.result = result;
    p.alpha1 = alpha1;
    p.alpha2 = alpha2;
    p.maxlen = maxlen;
    p.B = static_cast<int>(num_instances);
    p.K = static_cast<int>(K);
    p.obs_max = n_obs >= 1 && n_obs <= 256 ? static_cast<int>(n_obs) - 1 : 255;
    p.gamma = gamma;
    p.synthetic = synthetic_248;
    p.gamma_lin = expf(gamma);
    p.synthetic_lin = expf(synthetic_248);
    p.write_alpha = write_alpha ? 1 : 0;
    p.host_flag = host_timeout_flag(dev.device);
    PB_REQUIRE(p.host_flag == nullptr || *reinterpret_cast<volatile unsigned *>(p.host_flag) == 0u,
               "forward: a bounded wait inside an earlier forward kernel on this device ran out, so results "
               "computed since the last parpy_b200_forward_status read are not valid; read the status word "
               "(that clears this condition) and repeat those calls");

    Plan pl;
    bool resident = !streaming_forced && make_plan(K, &pl, !five, scaled);
    if (scaled_by_default && !(resident && pl.kpt == 4 && pl.split)) {   // no 1024-thread layout for this size
        scaled = false;
        resident = make_plan(K, &pl, true, false);
    }
    PB_REQUIRE(!scaled || (resident && pl.kpt == 4),
               "forward: the scaled kernel needs at least 1024 k-mers (num_states=%lld)", (long long)num_states);
    if (resident) finish_plan(&pl, five, scaled);
    // scaled tensor-memory kernel with a known table height: exponentials of the emission table once per
    // call (6.6 MB for the 7-mer table, a few microseconds) instead of four per thread and step
    if (resident)
        pl.exptab = pl.scaled && pl.tmem && n_obs >= 1 && n_obs <= 256 && getenv("PARPY_B200_SCALED_EXPTAB_OFF") == nullptr;
    if (resident) {
        PB_REQUIRE(pl.kpt == 1 || (pb::aligned16(initial_prob) && pb::aligned16(output_prob) &&
                                   pb::aligned16(trans1) &&
                                   (!write_alpha || (pb::aligned16(alpha1) && pb::aligned16(alpha2)))),
                   "forward: tables must be 16-byte aligned");
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute attr[1];
        int max_clusters = 0;
        ResidentKernel kern = nullptr;
        rc = resident_config(pl, five, &cfg, attr, &max_clusters, &kern);
        if (rc) return rc;
        int clusters = std::min(max_clusters, p.B);
        if (const char *env = getenv("PARPY_B200_FWD_CLUSTERS")) {
            const int v = atoi(env);
            if (v >= 1 && v <= clusters) clusters = v;
        }
        // scratch from the library workspace: sequence order, queue head, segment table
        void *ws = nullptr;
        rc = pb::workspace(sched_bytes(p.B), &ws, stream, 0);
        if (rc) return rc;
        rc = launch_schedule(&p, sched_layout(ws, sched_bytes(p.B) - kSchedTailBytes), clusters, nullptr, stream);
        if (rc) return rc;
        if (pl.exptab) {
            void *tab = nullptr;
            const long long n4 = n_obs * K / 4;
            rc = pb::workspace((size_t)n4 * sizeof(float4), &tab, stream, 5);
            if (rc) return rc;
            const int blocks = (int)std::min<long long>((n4 + 255) / 256, 148 * 8);
            hmm_exp_table<<<blocks, 256, 0, stream>>>(reinterpret_cast<const float4 *>(output_prob),
                                                      static_cast<float4 *>(tab), n4);
            PB_CUDA(cudaGetLastError());
            p.output_lin = static_cast<const float *>(tab);
        }
        cfg.gridDim = dim3(pl.cs * clusters, 1, 1);
        cfg.stream = stream;
        PB_CUDA(cudaLaunchKernelEx(&cfg, kern, p));
        return PB_OK;
    }

    // streaming path
    PB_REQUIRE(alpha1 && alpha2, "forward: the streaming kernel needs alpha1 and alpha2 scratch (%s)",
               streaming_forced ? "streaming was requested" : "this state space has no resident mapping");
    PB_REQUIRE(num_instances <= 65535, "forward: streaming kernel supports at most 65535 sequences");
    const int tpb = 256;
    dim3 grid((unsigned)((num_states + tpb - 1) / tpb), (unsigned)num_instances, 1);
    hmm_stream_init<<<grid, tpb, 0, stream>>>(p);
    PB_CUDA(cudaGetLastError());
    for (int t = 1; t < maxlen; ++t) {
        hmm_stream_step<<<grid, tpb, 0, stream>>>(p, t);
        PB_CUDA(cudaGetLastError());
    }
    hmm_stream_final<<<(unsigned)num_instances, 512, 0, stream>>>(p);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

}  // namespace

extern "C" {

int32_t parpy_b200_forward(float gamma, const float *initial_prob, int64_t num_states,
                           const float *output_prob, float synthetic_248, const float *trans1,
                           const float *trans2, const void *data, const int64_t *lens,
                           int64_t maxlen, int64_t num_instances, float *result, float *alpha1,
                           float *alpha2, uint32_t flags, void *stream) {
    return forward_impl(gamma, initial_prob, num_states, output_prob, synthetic_248, trans1, trans2,
                        data, lens, maxlen, num_instances, result, alpha1, alpha2, flags, 0,
                        static_cast<cudaStream_t>(stream));
}

int32_t parpy_b200_forward_ex(float gamma, const float *initial_prob, int64_t num_states,
                              const float *output_prob, int64_t n_obs, float synthetic_248,
                              const float *trans1, const float *trans2, const void *data,
                              const int64_t *lens, int64_t maxlen, int64_t num_instances, float *result,
                              float *alpha1, float *alpha2, uint32_t flags, void *stream) {
    return forward_impl(gamma, initial_prob, num_states, output_prob, synthetic_248, trans1, trans2,
                        data, lens, maxlen, num_instances, result, alpha1, alpha2, flags, n_obs,
                        static_cast<cudaStream_t>(stream));
}

int32_t forward_kernel(float gamma, float *initial_prob, int64_t num_states, float *output_prob,
                       float synthetic_248, float *trans1, float *trans2, int8_t *data,
                       int64_t *lens, int64_t maxlen, int64_t num_instances, float *result,
                       float *alpha1, float *alpha2) {
    return forward_impl(gamma, initial_prob, num_states, output_prob, synthetic_248, trans1, trans2,
                        data, lens, maxlen, num_instances, result, alpha1, alpha2,
                        PARPY_B200_FWD_AUTO, 0, nullptr);
}

int32_t forward_kernel_scratch_first(float gamma, float *initial_prob, int64_t num_states,
                                     float *output_prob, float synthetic_248, float *trans1,
                                     float *trans2, int8_t *data, int64_t *lens, int64_t maxlen,
                                     int64_t num_instances, float *alpha1, float *alpha2,
                                     float *result) {
    return forward_impl(gamma, initial_prob, num_states, output_prob, synthetic_248, trans1, trans2,
                        data, lens, maxlen, num_instances, result, alpha1, alpha2,
                        PARPY_B200_FWD_AUTO, 0, nullptr);
}

int32_t parpy_b200_forward_plan(int64_t num_states, int64_t num_instances, int32_t *kmers_per_thread,
                                int32_t *threads_per_cta, int32_t *ctas_per_cluster,
                                int32_t *clusters) {
    Plan pl;
    if (num_states < 64 || num_states % 64 != 0 || !make_plan(num_states / kLayers, &pl, true)) {
        pb::set_error("forward_plan: num_states=%lld has no resident mapping", (long long)num_states);
        return PB_ERR_UNSUPPORTED;
    }
    finish_plan(&pl, false, false);
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    int max_clusters = 0;
    ResidentKernel kern = nullptr;
    int32_t rc = resident_config(pl, false, &cfg, attr, &max_clusters, &kern);
    if (rc) return rc;
    if (kmers_per_thread) *kmers_per_thread = pl.kpt;
    if (threads_per_cta) *threads_per_cta = pl.nt;
    if (ctas_per_cluster) *ctas_per_cluster = pl.cs;
    if (clusters) *clusters = (int32_t)std::min<int64_t>(max_clusters, std::max<int64_t>(num_instances, 1));
    return PB_OK;
}

int32_t parpy_b200_forward_schedule(const int64_t *lens, int64_t num_instances, int64_t clusters,
                                    int32_t *cluster_of, void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    PB_REQUIRE(num_instances >= 1 && num_instances <= kSortLimit,
               "forward_schedule: the static schedule covers 1..%d sequences (got %lld); larger batches "
               "use a work queue", kSortLimit, (long long)num_instances);
    PB_REQUIRE(clusters >= 1 && clusters <= kMaxBins, "forward_schedule: clusters=%lld outside 1..%d",
               (long long)clusters, kMaxBins);
    PB_REQUIRE(lens && cluster_of, "forward_schedule: null pointer");
    FwdParams p{};
    p.lens = lens;
    p.B = static_cast<int>(num_instances);
    void *ws = nullptr;
    int32_t rc = pb::workspace(sched_bytes(p.B), &ws, stream, 0);
    if (rc) return rc;
    const int c = static_cast<int>(std::min<int64_t>(clusters, num_instances));
    return launch_schedule(&p, sched_layout(ws, sched_bytes(p.B) - kSchedTailBytes), c, cluster_of, stream);
}

int32_t parpy_b200_forward_status(uint32_t *status) {
    PB_REQUIRE(status != nullptr, "forward_status: null output pointer");
    unsigned v = 0, zero = 0;
    PB_CUDA(cudaDeviceSynchronize());
    PB_CUDA(cudaMemcpyFromSymbol(&v, g_status, sizeof(v)));
    PB_CUDA(cudaMemcpyToSymbol(g_status, &zero, sizeof(zero)));
    int device = -1;
    PB_CUDA(cudaGetDevice(&device));
    if (unsigned *flag = host_timeout_flag(device)) *reinterpret_cast<volatile unsigned *>(flag) = 0u;
    *status = v;
    return PB_OK;
}

int32_t parpy_b200_forward_wait_probe(int32_t polls, void *stream) {
    PB_REQUIRE(polls >= 0 && polls <= (1 << 20), "forward_wait_probe: polls=%d outside 0..2^20", polls);
    int device = -1;
    PB_CUDA(cudaGetDevice(&device));
    fwd_wait_probe<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(polls, host_timeout_flag(device));
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

}  // extern "C"

// ---- entry point that allocates nothing --------------------------------------------
namespace {

std::mutex g_noalloc_mu;
void *g_noalloc_addr[64];  // device address of g_noalloc_scratch, per device ordinal

// Looks up (once per device, with that device current) where the module's copy
// of g_noalloc_scratch lives on the current device.
int32_t noalloc_scratch_address(void **out) {
    int dev = 0;
    PB_CUDA(cudaGetDevice(&dev));
    PB_REQUIRE(dev >= 0 && dev < 64, "forward_noalloc: device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    if (g_noalloc_addr[dev] == nullptr) {
        void *p = nullptr;
        PB_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        g_noalloc_addr[dev] = p;
    }
    *out = g_noalloc_addr[dev];
    return PB_OK;
}

}  // namespace

extern "C" int32_t parpy_b200_forward_noalloc(float gamma, const float *initial_prob,
                                              int64_t num_states, const float *output_prob,
                                              float synthetic_248, const float *trans1,
                                              const float *trans2, const void *data,
                                              const int64_t *lens, int64_t maxlen,
                                              int64_t num_instances, float *result, void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    PB_REQUIRE(num_states >= 64 && num_states % 64 == 0,
               "forward_noalloc: num_states=%lld must be a positive multiple of 64", (long long)num_states);
    PB_REQUIRE(num_instances >= 0, "forward_noalloc: negative num_instances");
    PB_REQUIRE(num_instances <= kNoAllocMaxSequences,
               "forward_noalloc: num_instances=%lld exceeds the fixed scratch capacity of %d sequences; "
               "split the batch or call parpy_b200_forward",
               (long long)num_instances, kNoAllocMaxSequences);
    PB_REQUIRE(maxlen >= 1 && maxlen <= 0x7fffffffLL, "forward_noalloc: maxlen=%lld out of range", (long long)maxlen);
    if (num_instances == 0) return PB_OK;
    PB_REQUIRE(initial_prob && output_prob && trans1 && trans2 && data && lens && result,
               "forward_noalloc: null table, observation or result pointer");
    const long long K = num_states / kLayers;
    Plan pl;
    PB_REQUIRE(make_plan(K, &pl, true),
               "forward_noalloc: num_states=%lld has no resident mapping (the streaming kernel needs "
               "caller scratch: use parpy_b200_forward)", (long long)num_states);
    finish_plan(&pl, false, false);
    PB_REQUIRE(pl.kpt == 1 || (pb::aligned16(initial_prob) && pb::aligned16(output_prob) && pb::aligned16(trans1)),
               "forward_noalloc: tables must be 16-byte aligned");
    pb::DeviceInfo dev;
    int32_t rc = pb::device_info(&dev);
    if (rc) return rc;
    PB_REQUIRE(dev.cc_major >= 10, "forward_noalloc: needs compute capability 10.x, found %d.%d",
               dev.cc_major, dev.cc_minor);
    void *scratch = nullptr;
    rc = noalloc_scratch_address(&scratch);
    if (rc) return rc;

    FwdParams p{};
    p.initial_prob = initial_prob;
    p.output_prob = output_prob;
    p.trans1 = trans1;
    p.data = static_cast<const uint8_t *>(data);
    p.lens = lens;
    p.result = result;
    p.maxlen = maxlen;
    p.B = static_cast<int>(num_instances);
    p.K = static_cast<int>(K);
    p.gamma = gamma;
    p.synthetic = synthetic_248;
    p.write_alpha = 0;
    p.trans2 = trans2;
    p.obs_max = 255;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    int max_clusters = 0;
    ResidentKernel kern = nullptr;
    rc = resident_config(pl, false, &cfg, attr, &max_clusters, &kern);
    if (rc) return rc;
    // The array keeps whatever the previous call left in it. hmm_schedule rewrites
    // all num_instances order entries, the queue head and the segment table before the
    // forward kernel (same stream) reads any of them, so nothing stale is ever used.
    const int clusters = std::min(max_clusters, p.B);
    rc = launch_schedule(&p, sched_layout(scratch, kNoAllocOrderBytes), clusters, nullptr, stream);
    if (rc) return rc;
    cfg.gridDim = dim3(pl.cs * clusters, 1, 1);
    cfg.stream = stream;
    PB_CUDA(cudaLaunchKernelEx(&cfg, kern, p));
    return PB_OK;
}
