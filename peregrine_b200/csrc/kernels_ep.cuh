// Expert parallelism over the GPUs of one node: the exchange kernels (sm_100a).
//
// Rank r of G owns routed experts [r*E/G, (r+1)*E/G); router, shared expert and dense layers are
// replicated; the decode batch is data-parallel (M/G home tokens per rank).  One MoE layer step:
//
//   1. every rank routes ITS home tokens (exact chains, top-k) and stores their picks into every
//      rank's copy of the batch-wide pick table (ep_select_scatter_kernel);
//   2. with all picks present every rank derives the same batch-union order and pair layout
//      (ep_plan_kernel: crates/peregrine-model/src/router.rs:420-430, mlp.rs:83-95), then sends, for
//      each (home token, picked expert) pair, the token's int8 row, scale and block corrections
//      straight into the owner's receive buffer at the pair's row (ep_dispatch_kernel): 6.5 KB per
//      pair instead of the 24 KB of the fp32 row, and exact, because quantisation is deterministic;
//   3. the owner waits for the rows of its experts (ep_wait_rows_kernel), runs gate/up + SwiGLU and
//      down on them with the same kernels as a single device, and stores each un-weighted output row
//      straight into the home rank's pair buffer (ep_return_kernel);
//   4. the home rank waits for the rows of its tokens and sums them with the gate weights in
//      batch-union order, shared expert last (ep_combine_kernel) — the fixed-order rule of
//      docs/scale-out-design.md:62-67: partial results are never added in arrival order.
//
// All transfers are plain stores into peer memory (NVLink) followed by a release store of a flag
// that carries the step number; the consumer polls its own memory with a bounded wait.  No TMA or
// bulk load ever names peer memory.  Buffers exist twice and alternate with the step number: a rank
// can run at most one exchange step ahead of another (its next step waits for every rank's picks of
// that step), so the set being written never is the set still being read.
#pragma once
#include "kernels.cuh"

namespace pgb {

constexpr int kEpMaxRanks = 16;
constexpr long long kEpWaitCycles = 2000000000LL;

// Byte offsets of the parts of one parity set inside a rank's exchange block.
struct EpLayout {
    unsigned long long idx, keff, ix_flag, sx, rx_flag, ry_flag, cs, xq, y, set_bytes;
};

struct EpPeers {
    unsigned char *base[kEpMaxRanks];  // exchange block of every rank (own included), this rank's addresses
};

__device__ __forceinline__ unsigned ep_ld_acquire_sys(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void ep_st_release_sys(unsigned *p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// One thread polls until *p == want; false after ~1 s.  `failed` is a word of this rank's own block
// that the first wait to run out sets: every later wait of the rank then gives up at once, so a
// rank that has lost step with the others (they must enter a step within the wait limit of each
// other) drains its queued launches in microseconds instead of a second per wait.
__device__ __forceinline__ bool ep_wait_flag(const unsigned *p, unsigned want, unsigned *failed) {
    const long long t0 = clock64();
    while (ep_ld_acquire_sys(p) != want) {
        const long long dt = clock64() - t0;
        if (dt > 4000) {
            if (*reinterpret_cast<volatile unsigned *>(failed)) return false;
            if (dt > kEpWaitCycles) {
                atomicExch(failed, 1u);
                return false;
            }
            __nanosleep(200);
        }
    }
    return true;
}

// ---- 1. per-token selection of the home tokens + publication of the picks.
// One CTA; warp w selects tokens w, w + nwarp, ... with the arithmetic of route_select_kernel
// (crates/peregrine-model/src/router.rs:86-150).  idx / keff go to every rank's pick table at the
// token's batch-wide index, the weights stay local; then every rank's flag for this rank is set.
struct EpSelectArgs {
    const float *logits;  // [m_loc, E] of the home tokens
    const float *bias;
    int m_loc, home_lo, E, k, norm_topk;
    float routed_scale;
    float *w;             // local [M, k]: gate weights, rows of the home tokens filled
    EpPeers peers;
    EpLayout lay;
    unsigned long long set_off;  // byte offset of the step's parity set
    int rank, world;
    unsigned epoch;
};

// (a device routine so that the routing launch's last chain CTA can run it without a launch of its own)
__device__ __forceinline__ void ep_select_scatter_body(const EpSelectArgs &A, unsigned char *es_smem) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    float *sig = reinterpret_cast<float *>(es_smem) + warp * 2 * A.E;
    unsigned *key = reinterpret_cast<unsigned *>(sig + A.E);
    for (int sl = warp; sl < A.m_loc; sl += nwarp) {
        for (int e = lane; e < A.E; e += 32) {
            const float sg = sigmoid32(__ldcg(A.logits + (long long)sl * A.E + e));
            sig[e] = sg;
            const float c = __fadd_rn(sg, A.bias[e]);
            unsigned u = 0u;
            if (c > -INFINITY) {  // false for NaN and -inf
                u = __float_as_uint(c == 0.0f ? 0.0f : c);
                u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
            }
            key[e] = u;
        }
        __syncwarp();
        int kept = A.k, my_idx = 0;
        float my_w = 0.0f;
        for (int kk = 0; kk < A.k; ++kk) {
            unsigned bu = 0u;
            int bi = 0x7fffffff;
            for (int e = lane; e < A.E; e += 32) {
                const unsigned u = key[e];
                if (u > bu) {
                    bu = u;
                    bi = e;
                }
            }
            const unsigned top = __reduce_max_sync(0xffffffffu, bu);
            if (top == 0u) {
                kept = kk;
                break;
            }
            const int best = (int)__reduce_min_sync(0xffffffffu, (unsigned)(bu == top ? bi : 0x7fffffff));
            if (lane == kk) {
                my_idx = best;
                my_w = sig[best];
            }
            if (lane == 0) key[best] = 0u;
            __syncwarp();
        }
        if (A.norm_topk) {
            float sm = 0.0f;
            for (int j = 0; j < A.k; ++j) sm = __fadd_rn(sm, __shfl_sync(0xffffffffu, my_w, j));
            sm = __fadd_rn(sm, 1e-20f);
            my_w = __fdiv_rn(my_w, sm);
        }
        my_w = __fmul_rn(my_w, A.routed_scale);
        const int s = A.home_lo + sl;  // batch-wide token index
        if (lane < A.k) A.w[s * A.k + lane] = my_w;
        for (int r = 0; r < A.world; ++r) {
            unsigned char *set = A.peers.base[r] + A.set_off;
            if (lane < A.k) reinterpret_cast<int *>(set + A.lay.idx)[s * A.k + lane] = my_idx;
            if (lane == 0) reinterpret_cast<int *>(set + A.lay.keff)[s] = kept;
        }
        __syncwarp();
    }
    __threadfence_system();
    __syncthreads();
    if ((int)threadIdx.x < A.world)
        ep_st_release_sys(reinterpret_cast<unsigned *>(A.peers.base[threadIdx.x] + A.set_off + A.lay.ix_flag) + A.rank,
                          A.epoch);
}

__global__ void __launch_bounds__(512) ep_select_scatter_kernel(const EpSelectArgs A) {
    extern __shared__ __align__(16) unsigned char es_smem[];
    ep_select_scatter_body(A, es_smem);
}

// Routing launch of an expert-parallel rank: the exact chains and int8 rows of the home tokens
// (route_fused_kernel without a plan); the chain CTA that finishes last selects and publishes the picks.
__global__ void __launch_bounds__(kRtThreads, 1) route_fused_ep_kernel(const RouteArgs A, const EpSelectArgs S) {
    extern __shared__ __align__(128) unsigned char rt_smem[];
    if ((int)blockIdx.x >= A.n_chain_ctas) {
        route_quantise_row(A, blockIdx.x - A.n_chain_ctas, rt_smem);
        return;
    }
    if (route_chain_role(A, rt_smem, blockIdx.x)) {  // uniform over the CTA: this one saw all logits written
        __syncthreads();
        ep_select_scatter_body(S, rt_smem);
    }
}

// ---- 2a. batch-wide plan once every rank's picks are here (one CTA).
__global__ void __launch_bounds__(256) ep_plan_kernel(const unsigned *ix_flag, int world, unsigned epoch, int M, int E,
                                                      int k, int has_shared, const ExpertDev *__restrict__ experts,
                                                      RoutePlan plan, int *err, unsigned *failed) {
    extern __shared__ __align__(16) unsigned char ep_smem[];
    int bad = 0;
    if ((int)threadIdx.x < world && !ep_wait_flag(ix_flag + threadIdx.x, epoch, failed)) {
        report_error(err, kErrBarrierTimeout);
        bad = 1;
    }
    // without every rank's picks there is nothing to plan (and nothing valid to index with)
    if (__syncthreads_or(bad)) {
        if (threadIdx.x == 0) {
            *plan.n_slots = 0;
            *plan.n_pairs = 0;
            *plan.n_union = 0;
            *plan.shared_pair0 = -1;
        }
        return;
    }
    route_plan_body(nullptr, nullptr, M, E, k, 0, 0.0f, has_shared, experts, plan, ep_smem, true);
}

// ---- 2b. dispatch: CTA (home token sl, kk) sends the token's quantised row to the owner of its
// kk-th pick (kk == k: the shared expert's row, which stays on this rank).  `chunk_major` selects
// the layout the expert kernels of this batch size read (see qrow_i8_kernel).
struct EpDispatchArgs {
    const int8_t *xq;   // [m_loc, kp] rows of the home tokens, as quantised by the routing launch
    const int *xcs;     // [m_loc, nblk]
    const float *sx;    // [m_loc]
    int kp, nblk, m_loc, home_lo, k, E, world, has_shared, chunk_major;
    long long pcap;
    const int *idx, *keff, *tok_pair, *shared_pair0, *n_pairs;  // batch-wide plan (local copies)
    EpPeers peers;
    EpLayout lay;
    unsigned long long set_off;
    int rank;
    unsigned epoch;
};

__global__ void __launch_bounds__(256) ep_dispatch_kernel(const EpDispatchArgs A) {
    const int sl = blockIdx.x / (A.k + 1), kk = blockIdx.x % (A.k + 1);
    const int s = A.home_lo + sl;
    if (*A.n_pairs <= 0) return;  // no plan (a wait ran out): nothing may be indexed
    int p, dst;
    if (kk < A.k) {
        if (kk >= A.keff[s]) return;
        const int e = A.idx[s * A.k + kk];
        const int per = (A.E + A.world - 1) / A.world;
        dst = e / per;
        p = A.tok_pair[s * A.k + kk];
    } else {
        const int sp0 = *A.shared_pair0;
        if (!A.has_shared || sp0 < 0) return;
        dst = A.rank;
        p = sp0 + s;
    }
    unsigned char *set = A.peers.base[dst] + A.set_off;
    int8_t *xq_d = reinterpret_cast<int8_t *>(set + A.lay.xq);
    int *cs_d = reinterpret_cast<int *>(set + A.lay.cs);
    const uint4 *src = reinterpret_cast<const uint4 *>(A.xq + (long long)sl * A.kp);
    for (int u = threadIdx.x; u < (A.kp >> 4); u += blockDim.x) {
        const int chunk = u >> 4, unit = u & 15;
        const long long off = A.chunk_major ? ((long long)chunk * A.pcap + p) * kXqChunkRowBytes + unit * 16
                                            : (long long)p * A.kp + (long long)u * 16;
        *reinterpret_cast<uint4 *>(xq_d + off) = __ldg(src + u);
    }
    const int4 *csrc = reinterpret_cast<const int4 *>(A.xcs + (long long)sl * A.nblk);
    for (int u = threadIdx.x; u < (A.nblk >> 2); u += blockDim.x) {
        const int chunk = u >> 1;
        const long long off = A.chunk_major ? ((long long)chunk * A.pcap + p) * kChunkBlocks + (u & 1) * 4
                                            : (long long)p * A.nblk + (long long)u * 4;
        *reinterpret_cast<int4 *>(cs_d + off) = __ldg(csrc + u);
    }
    if (threadIdx.x == 0) reinterpret_cast<float *>(set + A.lay.sx)[p] = A.sx[sl];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) ep_st_release_sys(reinterpret_cast<unsigned *>(set + A.lay.rx_flag) + p, A.epoch);
}

// ---- 3a. the owner waits for every row of its experts (slots with rows).  One CTA; thread t takes
// slots t, t + blockDim, ...
__global__ void __launch_bounds__(256) ep_wait_rows_kernel(const GemvSlot *__restrict__ slots, const int *n_slots,
                                                           const unsigned *rx_flag, unsigned epoch, int *err,
                                                           unsigned *failed) {
    const int n = *n_slots;
    for (int sl = threadIdx.x; sl < n; sl += blockDim.x) {
        const int r0 = slots[sl].row0, nr = slots[sl].nrows;
        for (int r = 0; r < nr; ++r)
            if (!ep_wait_flag(rx_flag + r0 + r, epoch, failed)) {
                report_error(err, kErrBarrierTimeout);
                return;
            }
    }
}

// ---- 3b. return: CTA p looks its pair row up in the step's down slots; if this rank computed it,
// the row goes into the home rank's pair buffer (rows of this rank's own tokens are already in
// place: the down launch writes into this rank's buffer) and the row's flag is set there.
struct EpReturnArgs {
    const GemvSlot *slots;  // down slots of the step (rows of experts this rank does not own: nrows 0)
    const int *n_slots, *n_pairs, *pair_token;
    const float *y;         // this rank's pair buffer [P, D]
    int D, m_per_rank;
    EpPeers peers;
    EpLayout lay;
    unsigned long long set_off;
    int rank;
    unsigned epoch;
};

__global__ void __launch_bounds__(288) ep_return_kernel(const EpReturnArgs A) {
    const int p = blockIdx.x;
    if (p >= *A.n_pairs) return;
    const int n = *A.n_slots;
    int mine = 0;
    for (int sl = threadIdx.x; sl < n; sl += blockDim.x) {
        const int r0 = A.slots[sl].row0, nr = A.slots[sl].nrows;
        mine |= (p >= r0 && p < r0 + nr);
    }
    if (!__syncthreads_or(mine)) return;
    const int home = A.pair_token[p] / A.m_per_rank;  // the shared expert's rows belong to home tokens of this rank
    unsigned char *set = A.peers.base[home] + A.set_off;
    if (home != A.rank) {
        const float4 *src = reinterpret_cast<const float4 *>(A.y + (long long)p * A.D);
        float4 *dst = reinterpret_cast<float4 *>(reinterpret_cast<float *>(set + A.lay.y) + (long long)p * A.D);
        for (int u = threadIdx.x; u < (A.D >> 2); u += blockDim.x) dst[u] = __ldcg(src + u);
        __threadfence_system();
    } else {
        __threadfence();
    }
    __syncthreads();
    if (threadIdx.x == 0) ep_st_release_sys(reinterpret_cast<unsigned *>(set + A.lay.ry_flag) + p, A.epoch);
}

// ---- 4. ordered combine of the home tokens once their rows are here
// (crates/peregrine-model/src/mlp.rs:111-127, concurrent.rs:1866-1929): out starts at zero, each
// expert's row is added as out + (w * y) in batch-union order, the shared expert's row last.
__global__ void __launch_bounds__(256) ep_combine_kernel(const float *__restrict__ y, int D, int k, RoutePlan plan,
                                                         const unsigned *ry_flag, unsigned epoch,
                                                         float *__restrict__ out, int first_token, int *err,
                                                         unsigned *failed) {
    const int s = first_token + blockIdx.y;
    const int ke = plan.keff[s];
    const int sp0 = *plan.shared_pair0;
    __shared__ int s_ok;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if ((int)threadIdx.x <= ke) {
        const int j = threadIdx.x;
        bool ok = true;
        if (j < ke)
            ok = ep_wait_flag(ry_flag + plan.comb_pair[s * k + j], epoch, failed);
        else if (sp0 >= 0)
            ok = ep_wait_flag(ry_flag + sp0 + s, epoch, failed);
        if (!ok) {
            report_error(err, kErrBarrierTimeout);
            s_ok = 0;
        }
    }
    __syncthreads();
    if (!s_ok) return;
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= D) return;
    float acc = 0.0f;
    for (int j = 0; j < ke; ++j) {
        const int p = plan.comb_pair[s * k + j];
        acc = __fadd_rn(acc, __fmul_rn(plan.comb_w[s * k + j], __ldcg(y + (long long)p * D + d)));
    }
    if (sp0 >= 0) acc = __fadd_rn(acc, __ldcg(y + (long long)(sp0 + s) * D + d));
    out[(long long)blockIdx.y * D + d] = acc;
}

}  // namespace pgb
