// Windowed Viterbi decoding over the k-mer x 16-duration-layer HMM for sm_100a,
// with the semantics of the CUDA the reference ships for the same model
// (benchmarks/7mer/hmm.cu:116-176, 352-508, 569-657): windows of `batch` time
// steps that advance by `batch - overlap`, a window after the first restarts from
// the state decoded at t-1, candidates compared in the order j = 0..3 then the
// duration-chain predecessor with a strict '>', and the final arg-max of a full
// window taken one step before its end, as the reference's buffer swap has it.
//
// Layout: the resident design of the forward kernel. A cluster owns one sequence
// at a time, each thread keeps the 16 layers of its 4 k-mers (64 chi values) in
// registers, only layer 0 crosses CTAs (distributed shared memory, one split
// barrier.cluster per step). The reference stores a 4-byte back pointer per state
// and step (1 MiB per step for the 7-mer model); here a back pointer is one of
// five choices, stored as a nibble: 32 bytes per thread and step, 128 KiB per
// step for the 7-mer model, written with two 16-byte stores. The cluster leader
// walks the window backwards through these nibbles.
#include <algorithm>
#include <atomic>

#include "../../include/parpy_b200.h"
#include "common.cuh"
#include "cluster.cuh"
#include "tmem.cuh"

namespace {

constexpr int kLayers = 16;

struct VitParams {
    const float *initial_prob;  // [16*K]
    const float *output_prob;   // [n_obs, K]
    const float *trans1;        // [K, 4]
    const float *trans2;        // [16]
    const uint8_t *data;        // [B, maxlen]
    const int64_t *lens;        // [B]
    uint32_t *out;              // [B, out_stride] decoded states
    const int *order;           // [B] sequence ids, longest first
    int *counter;               // work-queue head
    uint4 *codes;               // back-pointer nibbles, one block per resident cluster
    long long codes_per_cluster;  // uint4 elements per cluster block
    long long maxlen;
    long long out_stride;
    int B;
    int K;
    int batch;
    int overlap;
    int obs_max;                // n_obs - 1: observations above it are clamped and flagged
    float gamma;
    float synthetic;
};

__global__ void vit_schedule(const int64_t *__restrict__ lens, int B, int *__restrict__ order,
                             int *__restrict__ counter) {
    extern __shared__ int s_len[];
    if (B <= 4096) {
        for (int i = threadIdx.x; i < B; i += blockDim.x) {
            long long l = lens[i];
            s_len[i] = l > 0x7fffffffLL ? 0x7fffffff : (l < 0 ? 0 : static_cast<int>(l));
        }
        __syncthreads();
        for (int i = threadIdx.x; i < B; i += blockDim.x) {
            const int li = s_len[i];
            int rank = 0;
            for (int j = 0; j < B; ++j) rank += (s_len[j] > li) || (s_len[j] == li && j < i);
            order[rank] = i;
        }
    } else {
        for (int i = threadIdx.x; i < B; i += blockDim.x) order[i] = i;
    }
    if (threadIdx.x == 0) *counter = 0;
}

// Packed fp32 pairs (add.rn.f32x2: one issue slot, each half rounded like a scalar add).
__device__ __forceinline__ float2 vadd2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 vdup2(float x) { return make_float2(x, x); }

__device__ __forceinline__ float vmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// Winner among the four k-mer candidates c0..c3 and the duration-chain candidate p5, in the
// reference's order (j = 0..3, then p5, each taken only if strictly greater than the best so
// far): the first candidate equal to the maximum. The compare-and-select instructions run on
// the ALU pipe, which bounds this kernel; two 3-input maxima and one equality test per
// candidate need fewer of them than a running (value, index) pair. The code comes out
// already shifted to its nibble (SHIFT), so packing eight of them is a few ORs.
// A state that no candidate reaches (all -inf) gets code 0. The reference leaves its back
// pointer uninitialised (hmm.cu:404-406); the backward pass only ever visits reachable
// states unless the whole sequence has probability zero, where the reference's path is
// arbitrary as well.
template <int SHIFT>
__device__ __forceinline__ void pick5(float c0, float c1, float c2, float c3, float p5, float &best,
                                      unsigned &code) {
    const float m = vmax3(vmax3(c0, c1, c2), c3, p5);
    unsigned c = c3 == m ? (3u << SHIFT) : (4u << SHIFT);
    c = c2 == m ? (2u << SHIFT) : c;
    c = c1 == m ? (1u << SHIFT) : c;
    c = c0 == m ? 0u : c;
    code = c;
    best = m;
}

// The four k-mer candidates of a state differ between duration layers only by the additive
// trans2[d], so in exact arithmetic their winner does not depend on the layer. With fp32
// rounding it can, but only when the two best are closer than the rounding errors. `decide4`
// evaluates s_j = T_j + a_j once per k-mer and reports the winner j* together with `safe`:
// true when s_best - s_second exceeds a bound on every rounding error involved, in which case
// fl(fl(T_j + trans2[d]) + a_j) has the same strict winner j* at every layer and only that one
// candidate needs to be evaluated per layer (bit-identical to evaluating all four).
//   error of one layer's candidate:  <= 1.0001 u (|T_j| + 2 t2max + |s_j|),  u = 2^-24
//   error of s_j itself:             <= 1.0001 u |s_j|
// so  s_b - s_k > 2^-22 (|s_b| + |s_k| + Tmax + 2 t2max)  leaves a factor two in hand; the
// left side grows faster than the right as s_k falls, so testing the second best covers the
// rest. -inf among the candidates, NaN or an infinite bound make `safe` false (except a lone
// finite candidate), and the caller then evaluates all candidates at every layer as before.
struct Decide4 {
    unsigned j;    // winner (first index among equal maxima of s)
    bool safe;
};
__device__ __forceinline__ Decide4 decide4(float s0, float s1, float s2, float s3, float slack) {
    const float hi01 = fmaxf(s0, s1), lo01 = fminf(s0, s1);
    const float hi23 = fmaxf(s2, s3), lo23 = fminf(s2, s3);
    const float best = fmaxf(hi01, hi23);
    const float second = fmaxf(fminf(hi01, hi23), hi01 >= hi23 ? lo01 : lo23);
    unsigned j = s2 == best ? 2u : 3u;
    j = s1 == best ? 1u : j;
    j = s0 == best ? 0u : j;
    const float bound = 0x1p-22f * (fabsf(best) + fabsf(second) + slack);
    Decide4 r;
    r.j = j;
    r.safe = (best - second > bound) || (second == -INFINITY && best > -INFINITY && slack < INFINITY);
    return r;
}
__device__ __forceinline__ float sel4(unsigned j, float v0, float v1, float v2, float v3) {
    float r = j == 2u ? v2 : v3;
    r = j == 1u ? v1 : r;
    return j == 0u ? v0 : r;
}

// (value, index) arg-max with the lowest index among equal values.
__device__ __forceinline__ void argmax_combine(float &v, unsigned &i, float ov, unsigned oi) {
    if (ov > v || (ov == v && oi < i)) {
        v = ov;
        i = oi;
    }
}

// ASYNC (clusters of 2 to 8 CTAs): layer 0 travels with st.async and is counted in by an
// mbarrier of the consuming CTA (complete_tx) instead of st.shared::cluster + barrier.cluster,
// so the sender runs no release fence. A CTA's phase completes on the bytes of a quarter of
// each producer's threads (the quarter whose k-mers it consumes), so a CTA can run ahead of a
// thread elsewhere in the cluster: in a cluster of 8 a writer of round r is only ordered after
// every thread's read of round r - 4 (three hops through the "feeds" relation reach every
// CTA), hence four buffers and four mbarriers. Waits are bounded.
constexpr int kVitWaitLimit = 1 << 22;
// Device status word. Bit 0: a wait for layer 0 ran out; the paths of that call are not
// valid. Bit 1: an observation >= n_obs inside a sequence was clamped to n_obs - 1.
__device__ unsigned g_vit_status;

__device__ __forceinline__ bool vit_mbar_wait(unsigned mbar, unsigned parity, int limit = kVitWaitLimit) {
    for (int i = 0; i < limit; ++i) {
        unsigned ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(mbar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

// Observation byte t of a sequence, kept inside the emission table (no branch in the time loop:
// `bad` is raised into the status word once per sequence).
__device__ __forceinline__ int vit_obs(const VitParams &p, const uint8_t *obs, int t, bool &bad) {
    const int o = obs[t];
    bad = bad || o > p.obs_max;
    return min(o, p.obs_max);
}

// One CTA waits, with the kernel's bounded wait, on an mbarrier that nothing ever completes:
// the wait runs out after `polls` polls and the status bit is raised exactly as in the
// decoding kernel. No other CTA, no data in flight; used to check that a wait that gives up
// reaches the host.
__global__ void vit_wait_probe(int polls) {
    __shared__ __align__(8) unsigned long long mbar;
    const unsigned addr = smem_u32(&mbar);
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(addr));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (!vit_mbar_wait(addr, 0u, polls) && threadIdx.x == 0) atomicOr(&g_vit_status, 1u);
    __syncthreads();
    if (threadIdx.x == 0) asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(addr) : "memory");
}

// Layer 0 of one thread to the consuming CTA: buffer b of its shared memory.
template <bool ASYNC>
__device__ __forceinline__ void vit_send_layer0(unsigned dst, unsigned rmbar, unsigned my_mbar, bool elected,
                                                unsigned round_bytes, float v0, float v1, float v2, float v3) {
    if (ASYNC) {
        // one thread per CTA and round announces the bytes its own CTA will receive in this buffer
        if (elected)
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(my_mbar), "r"(round_bytes) : "memory");
        asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];"
                     ::"r"(dst), "f"(v0), "f"(v1), "f"(v2), "f"(v3), "r"(rmbar) : "memory");
    } else {
        st_cluster_v4(dst, v0, v1, v2, v3);
    }
}

// TM (4096 k-mers and more): 1024 threads per CTA; a thread keeps layers 0..3 of its four k-mers in
// registers and layers 4..15 in tensor memory (48 of its warp's columns, one float2 per k-mer pair
// and layer, moved with tcgen05.ld/st), its transition values and decision slack in shared memory.
// A 7-mer sequence then takes a cluster of 4 CTAs instead of 8 (33 clusters on 132 SMs instead of
// 15 on 120) with 8 warps per scheduler instead of 4. Same arithmetic, same paths.
// MAXT: the largest CTA the instantiation is launched with (256 for the one-CTA 5-mer layout, which
// then has 255 registers per thread to work with and keeps everything in them).
template <bool ASYNC, bool TM, int MAXT = (TM ? 1024 : 512)>
__global__ void __launch_bounds__(MAXT, 1) hmm_viterbi_resident(const VitParams p) {
    constexpr unsigned NB = ASYNC ? 4u : 2u;      // layer-0 buffers
    constexpr int RL = TM ? 4 : kLayers;          // layers kept in registers
    extern __shared__ __align__(16) float a0s[];  // [NB][4][M] layer-0 values this CTA consumes; TM: + Ts, slack
    __shared__ unsigned s_tmem;                   // TM: base address of the CTA's tensor memory
    __shared__ __align__(8) unsigned long long s_mbar[4];
    __shared__ float2 s_t2[kLayers];   // (trans2[d], trans2[d])
    __shared__ int s_seq;
    __shared__ unsigned s_last;
    __shared__ float s_warp_v[32];
    __shared__ unsigned s_warp_i[32];
    __shared__ float s_cl_v[16];
    __shared__ unsigned s_cl_i[16];

    const int tid = threadIdx.x;
    const int NT = TM ? 1024 : static_cast<int>(blockDim.x);   // the tensor-memory layout always runs 1024 threads (vit_plan)
    const unsigned rank = cluster_ctarank();
    const unsigned CS = cluster_nctarank();
    // One CTA per sequence (small state spaces): the hardware cluster barrier is replaced by
    // the CTA barrier at the points where the split barrier completes.
    auto arrive = [&]() { if (CS > 1) cluster_arrive(); };
    auto wait = [&]() { if (CS > 1) cluster_wait(); else __syncthreads(); };
    const int K = p.K;
    const int Kq = K >> 2;
    const int M = NT;
    const int gthread = rank * NT + tid;     // thread index within the sequence, 0 .. K/4-1
    const int g = gthread * 4;               // first global k-mer
    const int lane = tid & 31, warp = tid >> 5, nwarps = (NT + 31) >> 5;
    const int bos = p.batch - p.overlap;
    uint4 *codes = p.codes + (long long)(blockIdx.x / CS) * p.codes_per_cluster;

    if (tid < kLayers) s_t2[tid] = vdup2(__ldg(p.trans2 + tid));
    float4 *Ts = reinterpret_cast<float4 *>(a0s + NB * 4 * M);   // TM: [4][NT] transition values
    float4 *Ss = Ts + 4 * NT;                                    // TM: [NT] decision slack
    unsigned tm_all = 0, tm = 0;
    if constexpr (TM) {
        if (warp == 0) tmem_alloc_all(&s_tmem);
        tmem_publish();
        tm_all = s_tmem;
        tm = tmem_warp_base(tm_all, warp, 64 * (warp >> 2));
    }
    float2 T[4][2];   // transition log-probabilities into the thread's two k-mer pairs
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float4 v = __ldg(reinterpret_cast<const float4 *>(p.trans1) + (j * Kq + (g >> 2)));
        T[j][0] = make_float2(v.x, v.y);
        T[j][1] = make_float2(v.z, v.w);
        if constexpr (TM) Ts[j * NT + tid] = v;
    }
    // Tmax + 2 t2max per k-mer of the thread (see decide4); infinite when a table holds -inf
    float slack[4];
    {
        float t2max = 0.0f;
        for (int d = 0; d < kLayers; ++d) t2max = fmaxf(t2max, fabsf(__ldg(p.trans2 + d)));
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float mx = 0.0f, my = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                // a transition of probability zero makes its candidate -inf at every layer: no error to bound
                mx = fmaxf(mx, T[j][h].x == -INFINITY ? 0.0f : fabsf(T[j][h].x));
                my = fmaxf(my, T[j][h].y == -INFINITY ? 0.0f : fabsf(T[j][h].y));
            }
            slack[2 * h] = mx + 2.0f * t2max;
            slack[2 * h + 1] = my + 2.0f * t2max;
        }
        if constexpr (TM) Ss[tid] = make_float4(slack[0], slack[1], slack[2], slack[3]);
    }
    const unsigned a0_base = smem_u32(a0s);
    unsigned dst0;
    {
        const int dj = g / Kq, rem = g % Kq;
        dst0 = map_to_rank(a0_base + 4u * (dj * M + rem % M), rem / M);
    }
    const unsigned buf_bytes = 16u * M;
    const unsigned mbar0 = smem_u32(&s_mbar[0]);
    unsigned rmbar0 = 0;            // mbarrier 0 of the CTA that consumes my layer 0
    unsigned phase = 0;             // bit b: parity to wait for on mbarrier b
    bool dead = false;
    if (ASYNC) {
        rmbar0 = map_to_rank(smem_u32(&s_mbar[0]), (unsigned)((g % Kq) / M));
        if (tid == 0) {
            for (int b = 0; b < 4; ++b)
                asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&s_mbar[b])));
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
    }
    const unsigned seq_addr = smem_u32(&s_seq);
    const unsigned last_addr = smem_u32(&s_last);
    const unsigned clv_addr = smem_u32(s_cl_v);
    const unsigned cli_addr = smem_u32(s_cl_i);
    __syncthreads();

    for (;;) {
        if (rank == 0 && tid == 0) {
            const int i = atomicAdd(p.counter, 1);
            const int seq = i < p.B ? p.order[i] : -1;
            for (unsigned r = 0; r < CS; ++r) st_cluster_s32(map_to_rank(seq_addr, r), seq);
        }
        arrive();
        wait();
        const int seq = s_seq;
        if (seq < 0) break;
        long long len64 = p.lens[seq];
        len64 = len64 < 1 ? 1 : (len64 > p.maxlen ? p.maxlen : len64);
        const int len = static_cast<int>(len64);
        const uint8_t *obs = p.data + (long long)seq * p.maxlen;
        uint32_t *res = p.out + (long long)seq * p.out_stride;
        bool bad_obs = false;   // an observation byte outside the emission table was met

        for (int t = 0; t < len; t += bos) {
            const int L = min(len - t, p.batch);        // positions of this window that exist
            // The step whose chi the arg-max reads: the reference takes it from its first chi
            // buffer, which after a full window with an odd last step holds the step before.
            const int karg = (L == p.batch && ((p.batch - 1) & 1)) ? p.batch - 2 : L - 1;

            // ---- window start (hmm.cu:352-376) ------------------------------------------
            float chi[RL][4];   // TM: layers RL..15 live in tensor memory
            float e[4];
            // layer d of this thread's four k-mers, wherever it lives (d is a constant after unrolling)
            auto put_layer = [&](const int d, const float4 v) {
                if (d < RL) { chi[d % RL][0] = v.x; chi[d % RL][1] = v.y; chi[d % RL][2] = v.z; chi[d % RL][3] = v.w; }
                else if constexpr (TM) tmem_st4(tm + 4 * (d - RL), v);
            };
            auto get_layer = [&](const int d) {
                float4 v = make_float4(chi[d % RL][0], chi[d % RL][1], chi[d % RL][2], chi[d % RL][3]);
                if constexpr (TM) {
                    if (d >= RL) {
                        tmem_ld4(tm + 4 * (d - RL), v);
                        tmem_wait_ld(v);
                    }
                }
                return v;
            };
            {
                const float4 v = __ldg(reinterpret_cast<const float4 *>(p.output_prob + (long long)vit_obs(p, obs, t, bad_obs) * K + g));
                e[0] = v.x; e[1] = v.y; e[2] = v.z; e[3] = v.w;
            }
            if (t == 0) {
#pragma unroll
                for (int d = 0; d < kLayers; ++d) {
                    const float4 v = __ldg(reinterpret_cast<const float4 *>(p.initial_prob + d * K + g));
                    put_layer(d, make_float4(v.x + e[0], v.y + e[1], v.z + e[2], v.w + e[3]));
                }
            } else {
                const unsigned last = s_last;
#pragma unroll
                for (int d = 0; d < kLayers; ++d) {
                    float w[4];
#pragma unroll
                    for (int c = 0; c < 4; ++c) w[c] = (unsigned)(d * K + g + c) == last ? e[c] : -INFINITY;
                    put_layer(d, make_float4(w[0], w[1], w[2], w[3]));
                }
            }
            if constexpr (TM) tmem_wait_st();
            unsigned buf = 0;   // buffer that holds the previous step's layer 0
            vit_send_layer0<ASYNC>(dst0, rmbar0, mbar0, tid == 0, 16u * M, chi[0][0], chi[0][1], chi[0][2], chi[0][3]);
            if (!ASYNC) arrive();

            float best_v = -INFINITY;
            unsigned best_i = 0;
            // Arg-max over all states of the cluster, lowest index among equal maxima. Must be
            // entered with no arrive pending; leaves none pending.
            auto cluster_argmax = [&]() {
                float v = chi[0][0];
                unsigned i = (unsigned)g;
#pragma unroll
                for (int d = 0; d < kLayers; ++d) {
                    const float4 l4 = get_layer(d);
                    const float w[4] = {l4.x, l4.y, l4.z, l4.w};
#pragma unroll
                    for (int c = 0; c < 4; ++c) argmax_combine(v, i, w[c], (unsigned)(d * K + g + c));
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
                    const unsigned oi = __shfl_xor_sync(0xffffffffu, i, o);
                    argmax_combine(v, i, ov, oi);
                }
                if (lane == 0) { s_warp_v[warp] = v; s_warp_i[warp] = i; }
                __syncthreads();
                if (tid < (int)CS) {
                    float bv = s_warp_v[0];
                    unsigned bi = s_warp_i[0];
                    for (int w = 1; w < nwarps; ++w) argmax_combine(bv, bi, s_warp_v[w], s_warp_i[w]);
                    st_cluster_f32(map_to_rank(clv_addr + 4u * rank, tid), bv);
                    st_cluster_s32(map_to_rank(cli_addr + 4u * rank, tid), (int)bi);
                }
                arrive();
                wait();
                best_v = s_cl_v[0];
                best_i = s_cl_i[0];
                for (unsigned r = 1; r < CS; ++r) argmax_combine(best_v, best_i, s_cl_v[r], s_cl_i[r]);
                arrive();   // everyone has read s_cl_* before it can be rewritten
                wait();
            };
            if (karg == 0) {
                if (ASYNC) {
                    cluster_argmax();
                } else {
                    wait();
                    cluster_argmax();
                    arrive();
                }
            }

            // ---- forward steps with back pointers (hmm.cu:116-176, 378-412) ----------------
            for (int k = 1; k < L; ++k) {
                {
                    const float4 v = __ldg(reinterpret_cast<const float4 *>(p.output_prob + (long long)vit_obs(p, obs, t + k, bad_obs) * K + g));
                    e[0] = v.x; e[1] = v.y; e[2] = v.z; e[3] = v.w;
                }
                if (ASYNC) {
                    if (!dead && !vit_mbar_wait(mbar0 + 8u * buf, (phase >> buf) & 1u)) {
                        dead = true;
                        atomicOr(&g_vit_status, 1u);
                    }
                    phase ^= 1u << buf;
                } else {
                    wait();
                }
                const float *seg = a0s + buf * 4 * M + tid;
                const float2 a[4] = {vdup2(seg[0]), vdup2(seg[M]), vdup2(seg[2 * M]), vdup2(seg[3 * M])};
                const unsigned nbuf = (buf + 1u) % NB;   // where this step's layer 0 goes
                unsigned words[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) words[i] = 0u;
                // winner of the k-mer candidates, once per k-mer (decide4); a pair of k-mers takes
                // the short path when it is safe for both in every lane of the warp
                Decide4 dec[4];
                bool fast[2];
                // TM: the transition values come out of shared memory for the decision and the winner's
                // selection only (the rare all-candidates path fetches them again)
                float2 Tq[4][2];
                float sl[4];
                if constexpr (TM) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float4 v = Ts[j * NT + tid];
                        Tq[j][0] = make_float2(v.x, v.y);
                        Tq[j][1] = make_float2(v.z, v.w);
                    }
                    const float4 s4 = Ss[tid];
                    sl[0] = s4.x; sl[1] = s4.y; sl[2] = s4.z; sl[3] = s4.w;
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) { Tq[j][0] = T[j][0]; Tq[j][1] = T[j][1]; }
#pragma unroll
                    for (int c = 0; c < 4; ++c) sl[c] = slack[c];
                }
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float2 sj[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) sj[j] = vadd2(Tq[j][h], a[j]);
                    dec[2 * h] = decide4(sj[0].x, sj[1].x, sj[2].x, sj[3].x, sl[2 * h]);
                    dec[2 * h + 1] = decide4(sj[0].y, sj[1].y, sj[2].y, sj[3].y, sl[2 * h + 1]);
                    fast[h] = __all_sync(0xffffffffu, dec[2 * h].safe && dec[2 * h + 1].safe);
                }
                // the winner's transition value and layer-0 value of each k-mer pair, chosen here so that
                // the four candidates' values are dead before the layers start
                float2 Tw[2], aw[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const unsigned jx = dec[2 * h].j, jy = dec[2 * h + 1].j;
                    Tw[h] = make_float2(sel4(jx, Tq[0][h].x, Tq[1][h].x, Tq[2][h].x, Tq[3][h].x),
                                        sel4(jy, Tq[0][h].y, Tq[1][h].y, Tq[2][h].y, Tq[3][h].y));
                    aw[h] = make_float2(sel4(jx, a[0].x, a[1].x, a[2].x, a[3].x),
                                        sel4(jy, a[0].x, a[1].x, a[2].x, a[3].x));
                }
                // layers [d_lo, d_hi) of pair h, ascending (a layer reads the old value of the next)
                auto layers = [&](const int h, const int d_lo, const int d_hi) {
                    // TM: old values of the layers above the register layers, requested one layer ahead
                    // (pair h of layer d sits in columns 4 (d - RL) + 2 h, 2 h + 1)
                    float2 nA = make_float2(0.f, 0.f), nB = nA;
                    if constexpr (TM) {
                        if (d_hi > RL - 1) tmem_ld2(tm + 2 * h, nA);   // layer RL
                    }
                    // old value of layer min(d + 1, 15) for pair h; called once per d, in ascending order
                    auto old_next = [&](const int d) {
                        if constexpr (!TM) {
                            return make_float2(chi[(d + 1 < kLayers ? d + 1 : 15) % RL][2 * h],
                                               chi[(d + 1 < kLayers ? d + 1 : 15) % RL][2 * h + 1]);
                        } else {
                            if (d + 1 < RL) return make_float2(chi[(d + 1) % RL][2 * h], chi[(d + 1) % RL][2 * h + 1]);
                            if (d == RL - 1) {
                                tmem_wait_ld(nA);
                                tmem_ld2(tm + 4 + 2 * h, nB);   // layer RL + 1
                                return nA;
                            }
                            if (d < kLayers - 1) {
                                float2 &cur = (d & 1) ? nA : nB, &ahead = (d & 1) ? nB : nA;
                                tmem_wait_ld(cur);
                                // requested before layer d is written: a load has completed before
                                // anything overwrites its columns
                                if (d + 2 < kLayers) tmem_ld2(tm + 4 * (d + 2 - RL) + 2 * h, ahead);
                                return cur;
                            }
                            return (d & 1) ? nB : nA;   // layer 15 reads its own old value, fetched for layer 14
                        }
                    };
                    auto put_pair = [&](const int d, const float2 r) {
                        if (d < RL) {
                            chi[d % RL][2 * h] = r.x;
                            chi[d % RL][2 * h + 1] = r.y;
                        } else if constexpr (TM) {
                            tmem_st2(tm + 4 * (d - RL) + 2 * h, r);
                        }
                    };
                    if (fast[h]) {
                        const unsigned jx = dec[2 * h].j, jy = dec[2 * h + 1].j;
                        const unsigned ex = jx << (8 * h), ey = jy << (8 * h + 4);     // even layers
                        const unsigned ox = ex << 16, oy = ey << 16;                     // odd layers
#pragma unroll
                        for (int d = d_lo; d < d_hi; ++d) {
                            const float2 val = vadd2(vadd2(Tw[h], s_t2[d]), aw[h]);
                            const float2 nx = old_next(d);
                            const float2 p5 = d == 15 ? vadd2(vdup2(p.gamma), nx)
                                            : d == 14 ? vadd2(vdup2(p.synthetic), nx) : nx;
                            const unsigned sh = 8 * h + 16 * (d & 1);
                            const unsigned cx = p5.x > val.x ? (4u << sh) : ((d & 1) ? ox : ex);
                            const unsigned cy = p5.y > val.y ? (4u << (sh + 4)) : ((d & 1) ? oy : ey);
                            const float2 r = vadd2(make_float2(fmaxf(val.x, p5.x), fmaxf(val.y, p5.y)),
                                                   make_float2(e[2 * h], e[2 * h + 1]));
                            put_pair(d, r);
                            words[d >> 1] |= cx | cy;
                        }
                    } else {
#pragma unroll
                        for (int d = d_lo; d < d_hi; ++d) {
                            const float2 t2 = s_t2[d];
                            // all four k-mer candidates: (T + t2) + a, as the reference adds them
                            float2 cand[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                float2 Tj = T[j][h];
                                if constexpr (TM) {
                                    const float4 v = Ts[j * NT + tid];
                                    Tj = h == 0 ? make_float2(v.x, v.y) : make_float2(v.z, v.w);
                                }
                                cand[j] = vadd2(vadd2(Tj, t2), a[j]);
                            }
                            const float2 nx = old_next(d);
                            // duration-chain candidate; below layer 14 its log-probability is 0
                            const float2 p5 = d == 15 ? vadd2(vdup2(p.gamma), nx)
                                            : d == 14 ? vadd2(vdup2(p.synthetic), nx) : nx;
                            float bx, by;
                            unsigned cx, cy;
                            if (h == 0) {
                                if (d & 1) {
                                    pick5<16>(cand[0].x, cand[1].x, cand[2].x, cand[3].x, p5.x, bx, cx);
                                    pick5<20>(cand[0].y, cand[1].y, cand[2].y, cand[3].y, p5.y, by, cy);
                                } else {
                                    pick5<0>(cand[0].x, cand[1].x, cand[2].x, cand[3].x, p5.x, bx, cx);
                                    pick5<4>(cand[0].y, cand[1].y, cand[2].y, cand[3].y, p5.y, by, cy);
                                }
                            } else {
                                if (d & 1) {
                                    pick5<24>(cand[0].x, cand[1].x, cand[2].x, cand[3].x, p5.x, bx, cx);
                                    pick5<28>(cand[0].y, cand[1].y, cand[2].y, cand[3].y, p5.y, by, cy);
                                } else {
                                    pick5<8>(cand[0].x, cand[1].x, cand[2].x, cand[3].x, p5.x, bx, cx);
                                    pick5<12>(cand[0].y, cand[1].y, cand[2].y, cand[3].y, p5.y, by, cy);
                                }
                            }
                            const float2 r = vadd2(make_float2(bx, by), make_float2(e[2 * h], e[2 * h + 1]));
                            put_pair(d, r);
                            words[d >> 1] |= cx | cy;
                        }
                    }
                };
                // layer 0 of both pairs first: it is what the other CTAs wait for
                layers(0, 0, 1);
                layers(1, 0, 1);
                vit_send_layer0<ASYNC>(dst0 + nbuf * buf_bytes, rmbar0 + 8u * nbuf, mbar0 + 8u * nbuf, tid == 0, 16u * M,
                                       chi[0][0], chi[0][1], chi[0][2], chi[0][3]);
                if (!ASYNC) arrive();
                layers(0, 1, kLayers);
                layers(1, 1, kLayers);
                if constexpr (TM) tmem_wait_st();   // the next step (and the arg-max) read what this one stored
                uint4 *slot = codes + ((long long)(k - 1) * Kq + gthread) * 2;
                __stcg(slot, make_uint4(words[0], words[1], words[2], words[3]));
                __stcg(slot + 1, make_uint4(words[4], words[5], words[6], words[7]));
                buf = nbuf;
                if (k == karg && k < L - 1) {   // full window: arg-max one step before the end
                    if (ASYNC) {
                        cluster_argmax();
                    } else {
                        wait();
                        cluster_argmax();
                        arrive();
                    }
                }
            }
            if (ASYNC) {   // the last round is not used, but it must have landed
                if (!dead && !vit_mbar_wait(mbar0 + 8u * buf, (phase >> buf) & 1u)) {
                    dead = true;
                    atomicOr(&g_vit_status, 1u);
                }
                phase ^= 1u << buf;
            } else {
                wait();
            }
            if (karg == L - 1 && karg > 0) cluster_argmax();

            // ---- backward pass (hmm.cu:436-508) -----------------------------------------------
            __threadfence();   // the nibbles of every CTA must be visible to the leader
            arrive();
            wait();
            if (rank == 0) {
                // positions L-1 .. batch-1 all hold the arg-max state (identity back pointers)
                const long long hi = min((long long)t + p.batch, p.out_stride);
                for (long long pos = t + L - 1 + tid; pos < hi; pos += NT) res[pos] = best_i;
                if (tid < 32) {
                    // One warp walks the window backwards. A hop is a dependent load, so the warp
                    // speculates: a k-mer is usually left through its duration chain (back pointer
                    // 4: same k-mer, one layer up), and then the next 32 hops read words whose
                    // addresses are known in advance. Lane i fetches the word of hop i under that
                    // assumption, all 32 loads travel together, and the hops are resolved from
                    // registers until one of them changes the k-mer (the rest is fetched again).
                    unsigned cur = best_i;
                    unsigned anchor = cur;
                    int j = L - 2;
                    while (j >= 0) {
                        const unsigned s = cur % (unsigned)K, d0 = cur / (unsigned)K;
                        const int jj = j - tid;                       // my hop's step
                        const unsigned dd = min(d0 + (unsigned)tid, 15u);   // its layer if the chain holds
                        unsigned word = 0;
                        if (jj >= 0)
                            word = __ldcg(reinterpret_cast<const unsigned *>(codes + ((long long)jj * Kq + (s >> 2)) * 2) +
                                          (dd >> 1));
                        const unsigned mine = (word >> (16 * (dd & 1) + 4 * (s & 3))) & 15u;
                        // hops that follow the chain, up to the first that does not (or the window start)
                        const unsigned off_chain = __ballot_sync(0xffffffffu, mine != 4u || jj < 0);
                        const int n_chain = off_chain ? __ffs(off_chain) - 1 : 32;
                        // lane i < n_chain writes the state after i + 1 chain hops
                        if (tid < n_chain) {
                            const unsigned st = min(d0 + (unsigned)tid + 1u, 15u) * (unsigned)K + s;
                            res[t + jj] = st;
                            if (jj == bos - 1) anchor = st;
                        }
                        const unsigned d_end = min(d0 + (unsigned)n_chain, 15u);
                        cur = d_end * (unsigned)K + s;
                        j -= n_chain;
                        if (n_chain < 32 && j >= 0) {
                            // the hop that left the chain: a k-mer predecessor (codes 0..3)
                            const unsigned code = __shfl_sync(0xffffffffu, mine, n_chain);
                            cur = code * (unsigned)Kq + (s >> 2);
                            if (tid == 0) res[t + j] = cur;
                            if (j == bos - 1) anchor = cur;
                            --j;
                        }
                    }
                    // whichever lane met position bos-1 holds the anchor
                    const unsigned has = __ballot_sync(0xffffffffu, anchor != best_i);
                    if (has) anchor = __shfl_sync(0xffffffffu, anchor, __ffs(has) - 1);
                    if (L - 1 == bos - 1) anchor = best_i;
                    // the next window restarts from the state decoded at its t-1
                    if (tid == 0)
                        for (unsigned r = 0; r < CS; ++r) st_cluster_s32(map_to_rank(last_addr, r), (int)anchor);
                }
            }
            arrive();
            wait();
        }
        if (bad_obs && tid == 0) atomicOr(&g_vit_status, 2u);
    }
    if constexpr (TM) {
        tmem_publish();   // every warp is done with its columns
        if (warp == 0) tmem_free_all(tm_all);
    }
}

struct VitPlan {
    int nt = 0, cs = 0;
    bool tm = false;   // 1024-thread CTAs with the upper layers in tensor memory
};

bool vit_plan(long long K, VitPlan *pl) {
    if (K < 1024 || (K & (K - 1)) != 0) return false;
    const long long threads = K / 4;
    // 5-mer: one 256-thread CTA per sequence (CTA barrier per step; 5.4 ms for 100 sequences of 2000
    // steps against 6.3 ms for clusters of 4 x 64 threads); larger models: clusters of 512-thread CTAs
    long long nt = K <= 1024 ? K / 4 : 512;
    if (const char *env = getenv("PARPY_B200_VIT_NT")) {
        const long long v = atoll(env);
        if (v >= 32 && v <= 512 && (v & (v - 1)) == 0 && v <= threads) nt = v;
    }
    // 4096 k-mers and more: 1024 threads per CTA, layers 4..15 in tensor memory (7-mer: clusters of 4 on
    // 132 SMs instead of clusters of 8 on 120, twice the warps per scheduler)
    bool tm = threads >= 1024 && getenv("PARPY_B200_VIT_NT") == nullptr;
    if (const char *env = getenv("PARPY_B200_VIT_TMEM")) tm = tm && atoi(env) != 0;
    if (tm) nt = 1024;
    long long cs = threads / nt;
    if (cs > 16) return false;
    pl->nt = (int)nt;
    pl->cs = (int)cs;
    pl->tm = tm;
    return true;
}

}  // namespace

static int32_t viterbi_impl(float gamma, const float *initial_prob, int64_t num_states,
                            const float *output_prob, int64_t n_obs, float synthetic_248,
                            const float *trans1, const float *trans2, const void *data,
                            const int64_t *lens, int64_t maxlen, int64_t num_instances,
                            int64_t batch_size, int64_t batch_overlap, uint32_t *out,
                            int64_t out_stride, void *stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    PB_REQUIRE(n_obs >= 0, "viterbi: n_obs=%lld is negative", (long long)n_obs);
    PB_REQUIRE(num_states >= 64 && num_states % 64 == 0, "viterbi: num_states=%lld must be a positive multiple of 64",
               (long long)num_states);
    PB_REQUIRE(num_instances >= 0 && num_instances <= 0x7fffffffLL, "viterbi: num_instances out of range");
    PB_REQUIRE(maxlen >= 1 && maxlen <= 0x7fffffffLL, "viterbi: maxlen=%lld out of range", (long long)maxlen);
    PB_REQUIRE(batch_size >= 2 && batch_size <= 65536 && batch_overlap >= 0 && batch_overlap < batch_size,
               "viterbi: window of %lld steps with overlap %lld is not valid", (long long)batch_size,
               (long long)batch_overlap);
    PB_REQUIRE(out_stride >= maxlen, "viterbi: out_stride=%lld is smaller than maxlen=%lld", (long long)out_stride,
               (long long)maxlen);
    if (num_instances == 0) return PB_OK;
    PB_REQUIRE(initial_prob && output_prob && trans1 && trans2 && data && lens && out, "viterbi: null pointer");
    PB_REQUIRE(pb::aligned16(initial_prob) && pb::aligned16(output_prob) && pb::aligned16(trans1),
               "viterbi: tables must be 16-byte aligned");
    const long long K = num_states / kLayers;
    VitPlan pl;
    PB_REQUIRE(vit_plan(K, &pl), "viterbi: needs 4^k k-mers with 5 <= k <= 8 (num_states=%lld)", (long long)num_states);
    pb::DeviceInfo dev;
    int32_t rc = pb::device_info(&dev);
    if (rc) return rc;
    PB_REQUIRE(dev.cc_major >= 10, "viterbi: needs compute capability 10.x, found %d.%d", dev.cc_major, dev.cc_minor);

    // layer 0 by st.async + mbarriers in clusters of 2 to 8 CTAs (7mer: 30.0 against 36.4 ms)
    bool async_x = true;
    if (const char *env = getenv("PARPY_B200_VIT_ASYNC")) async_x = atoi(env) != 0;
    async_x = async_x && pl.cs >= 2 && pl.cs <= 8;
    void (*kernel)(const VitParams) = pl.tm ? (async_x ? hmm_viterbi_resident<true, true> : hmm_viterbi_resident<false, true>)
                                            : (async_x ? hmm_viterbi_resident<true, false> : hmm_viterbi_resident<false, false>);
    // One CTA of at most 256 threads per sequence: with no more sequences than SMs every CTA has an SM to
    // itself, and the instantiation bounded to 256 threads keeps all 64 values and the transition
    // table in its 253 registers (no spills); larger batches keep the 128-register one, two CTAs per SM.
    if (!pl.tm && !async_x && pl.nt <= 256 && num_instances <= dev.sm_count) kernel = hmm_viterbi_resident<false, false, 256>;
    // layer-0 buffers; with tensor memory also the transition values and the decision slack of every thread
    const size_t smem = size_t(async_x ? 4 : 2) * 4 * pl.nt * sizeof(float) + (pl.tm ? size_t(5) * pl.nt * sizeof(float4) : 0);
    if (pl.cs > 8) PB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    PB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = pl.cs;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.gridDim = dim3(pl.cs, 1, 1);
    cfg.blockDim = dim3(pl.nt, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cfg.stream = stream;
    int max_clusters = 0;
    PB_CUDA(cudaOccupancyMaxActiveClusters(&max_clusters, kernel, &cfg));
    PB_REQUIRE(max_clusters >= 1, "viterbi: no cluster of %d CTAs x %d threads fits this device", pl.cs, pl.nt);

    // back-pointer nibbles: (batch - 1) steps x K/4 threads x 32 bytes per resident cluster,
    // at most ~6 GiB in total (33 clusters of a 7-mer model with 1024-step windows: 4.4 GB)
    const long long per_cluster = (batch_size - 1) * (K / 4) * 2;   // uint4 elements
    const long long budget = (6LL << 30) / (per_cluster * (long long)sizeof(uint4));
    long long clusters = std::min<long long>(std::min<long long>(max_clusters, num_instances), std::max<long long>(budget, 1));
    void *ws_codes = nullptr, *ws = nullptr;
    rc = pb::workspace((size_t)clusters * (size_t)per_cluster * sizeof(uint4), &ws_codes, stream, 4);
    if (rc) return rc;
    const size_t order_bytes = ((size_t)num_instances * sizeof(int) + 255) & ~size_t(255);
    rc = pb::workspace(order_bytes + 512, &ws, stream, 0);
    if (rc) return rc;

    VitParams p{};
    p.initial_prob = initial_prob;
    p.output_prob = output_prob;
    p.trans1 = trans1;
    p.trans2 = trans2;
    p.data = static_cast<const uint8_t *>(data);
    p.lens = lens;
    p.out = out;
    p.order = static_cast<int *>(ws);
    p.counter = reinterpret_cast<int *>(static_cast<char *>(ws) + order_bytes);
    p.codes = static_cast<uint4 *>(ws_codes);
    p.codes_per_cluster = per_cluster;
    p.maxlen = maxlen;
    p.out_stride = out_stride;
    p.B = (int)num_instances;
    p.K = (int)K;
    p.batch = (int)batch_size;
    p.overlap = (int)batch_overlap;
    p.obs_max = n_obs >= 1 && n_obs <= 256 ? (int)n_obs - 1 : 255;
    p.gamma = gamma;
    p.synthetic = synthetic_248;
    const size_t sched_smem = p.B <= 4096 ? size_t(p.B) * sizeof(int) : 0;
    vit_schedule<<<1, 1024, sched_smem, stream>>>(lens, p.B, const_cast<int *>(p.order), p.counter);
    PB_CUDA(cudaGetLastError());
    cfg.gridDim = dim3(pl.cs * (unsigned)clusters, 1, 1);
    PB_CUDA(cudaLaunchKernelEx(&cfg, kernel, p));
    return PB_OK;
}

extern "C" {

int32_t parpy_b200_viterbi(float gamma, const float *initial_prob, int64_t num_states,
                           const float *output_prob, float synthetic_248, const float *trans1,
                           const float *trans2, const void *data, const int64_t *lens, int64_t maxlen,
                           int64_t num_instances, int64_t batch_size, int64_t batch_overlap,
                           uint32_t *out, int64_t out_stride, void *stream) {
    return viterbi_impl(gamma, initial_prob, num_states, output_prob, 0, synthetic_248, trans1, trans2, data, lens,
                        maxlen, num_instances, batch_size, batch_overlap, out, out_stride, stream);
}

int32_t parpy_b200_viterbi_ex(float gamma, const float *initial_prob, int64_t num_states,
                              const float *output_prob, int64_t n_obs, float synthetic_248,
                              const float *trans1, const float *trans2, const void *data,
                              const int64_t *lens, int64_t maxlen, int64_t num_instances,
                              int64_t batch_size, int64_t batch_overlap, uint32_t *out, int64_t out_stride,
                              void *stream) {
    return viterbi_impl(gamma, initial_prob, num_states, output_prob, n_obs, synthetic_248, trans1, trans2, data,
                        lens, maxlen, num_instances, batch_size, batch_overlap, out, out_stride, stream);
}

int32_t parpy_b200_viterbi_status(uint32_t *status) {
    PB_REQUIRE(status != nullptr, "viterbi_status: null output pointer");
    unsigned v = 0, zero = 0;
    PB_CUDA(cudaDeviceSynchronize());
    PB_CUDA(cudaMemcpyFromSymbol(&v, g_vit_status, sizeof(v)));
    PB_CUDA(cudaMemcpyToSymbol(g_vit_status, &zero, sizeof(zero)));
    *status = v;
    return PB_OK;
}

int32_t parpy_b200_viterbi_wait_probe(int32_t polls, void *stream) {
    PB_REQUIRE(polls >= 0 && polls <= (1 << 20), "viterbi_wait_probe: polls=%d outside 0..2^20", polls);
    vit_wait_probe<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(polls);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

}  // extern "C"
