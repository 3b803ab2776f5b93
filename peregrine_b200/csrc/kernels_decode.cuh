// One launch for a whole single-token decode step of the MoE layer (sm_100a).
//
//   router logits -> top-k -> gate/up + SwiGLU -> quantise h -> down -> ordered combine
//
// The grid is one CTA per SM in two roles:
//   chain CTAs [0, n_chain): the exact router of the reference — one strictly sequential fp32
//     chain per expert (crates/peregrine-kernels/src/matmul.rs:18-30) and the exact plan
//     (crates/peregrine-model/src/router.rs:86-150) — exactly the code of route_fused_kernel; the
//     CTA that finishes the plan publishes a flag;
//   worker CTAs: stream the expert weights.  They cannot wait ~35 us for the exact chains, so they
//     pick the experts from parallel-sum logits they compute themselves (every worker CTA a few
//     experts, then a grid-wide counter), and only the *combine* waits for the exact plan: its gate
//     weights come from there, and the selection is compared with it.  When the two selections
//     differ (rare: the sums differ from the chains in the last bits only) every worker CTA sees
//     the same mismatch and the step is done again inside the kernel from the exact selection.
//     Nothing numerical ever comes from the speculative logits.
// Inside a worker CTA every warp owns a ring of bulk-copied weight chunks (kernels.cuh) that keeps
// running across the phases: the shared expert, which needs no routing, streams while the logits
// are formed; the down weights of a warp's first item are already in its ring when the grid-wide
// "gate/up complete" counter releases the down phase.
//
// Code that runs once per step runs cold: a step streams far more than the L2 holds, so the
// instructions of every phase come from DRAM again, and a long straight-line stretch costs
// microseconds in instruction fetches alone (measured: a 2000-add loop ran at full clock while a
// 700-instruction staging routine beside it took 9 us).  Hence the shape of the worker: ONE copy of
// the streaming loop serves the three phases (it is warm after the shared expert's items), one small
// routine quantises both the token row and the h rows, and the h rows' maxima are taken from the
// data by the CTA that quantises them instead of a thousand atomics on one line.
//
// Grid-wide waits are legal here because the launch is sized to one CTA per SM with a shared-memory
// footprint that admits no second CTA, so all CTAs are resident together; every wait is bounded and
// reports through the device error word instead of hanging.
#pragma once
#include "kernels.cuh"

namespace pgb {

constexpr int kDecEPC = 3;       // experts whose logits a worker CTA forms per round trip
constexpr int kDecU = 5;         // float4 per lane and expert: hidden size up to 11 * 32 * 5 * 4 = 7040
constexpr int kDecMaxK = 32;     // top-k bound (one lane per pick)
constexpr int kDecSlotBytes = ((kDecMaxK + 1) * (int)sizeof(GemvSlot) + 15) & ~15;
constexpr int kDecCtlInts = 64;  // [0,32) picks, 32 kept, 33 selection ready, 34 mismatch, 35 active slots,
                                 // 36 token row ready, 37 last CTA
constexpr long long kDecWaitCycles = 2000000000LL;

struct DecodeArgs {
    RouteArgs route;     // exact chains and plan (M = 1, small_plan)
    GemvParams gu, dn;   // layout fields of the two phases; rowmap of gu maps every pair row to token 0
    ExpertDev shared;    // streams of the shared expert (has_shared)
    int has_shared, n_chain;
    float *spec_logits;  // [E] parallel-sum logits
    float spec_sign;     // -1 turns the speculative pick upside down (self-test of the redo path)
    float *h;            // [2][(k + 1) * I] SwiGLU rows per attempt; row j = pick j, row k = shared expert
    float *y;            // [(k + 1) * D]   un-weighted expert outputs, same row numbering
    unsigned *sync;      // zero at launch: [0] CTAs whose logits are written, [1] CTAs that left,
                         // [2 + a] warps done with gate/up of attempt a, [8 + a * n_col + t] column tiles
    int n_col;
    unsigned *exact_flag;  // set to the step number by the chain CTA that wrote the exact plan
    unsigned *epoch_word;  // the step number, in device memory: read at the start of a launch, advanced by the last
                           // worker CTA to leave, so the same arguments serve every launch (graph replays too)
    float *out;            // [D]
    unsigned long long *timeline;  // optional [gridDim.x][16] globaltimer stamps (ns) per CTA, see decode_stamp
};

// Timeline slots of a worker CTA: 0 start, 1 token row quantised, 2 logits written, 3 selection known,
// 4 gate/up done (latest warp), 5 gate/up complete grid-wide, 6 h row quantised, 7 down done (latest
// warp), 8 leaving, 9 first wait for the exact plan began, 10 it ended, 14 logits of all CTAs seen,
// 15 picks made; of a chain CTA: 0 start, 1 chains and (in one CTA) plan done.
__device__ __forceinline__ void decode_stamp(const DecodeArgs &A, int slot) {
    if (A.timeline == nullptr) return;
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    atomicMax(A.timeline + (size_t)blockIdx.x * 16 + slot, t);
}

__host__ __device__ inline size_t decode_smem_bytes(int E, int k, int kp_gu, int nblk_gu, int kp_dn, int nblk_dn) {
    const size_t fixed = (size_t)kRingBytes + kGemvBarBytes + 2 * kDecSlotBytes + kDecCtlInts * 4 +
                         ((kDecEPC * kGemvWarps + 15) & ~15) * 4 + 16 * 4 + (((size_t)E * 4 + 15) & ~(size_t)15);
    const size_t a0 = (((size_t)kp_gu + 15) & ~(size_t)15) + (size_t)nblk_gu * 4 + 16;
    const size_t a1 = ((((size_t)(k + 1) * kp_dn) + 15) & ~(size_t)15) + (size_t)(k + 1) * nblk_dn * 4 + (size_t)(k + 1) * 8 + 16;
    return fixed + a0 + a1 + 128;
}

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_u32(unsigned *p, unsigned v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Lane 0 polls until *p >= target (or == when `exact`), all lanes get the verdict.  Bounded.
__device__ __forceinline__ bool warp_wait_counter(const unsigned *p, unsigned target, bool exact, int lane) {
    int ok = 1;
    if (lane == 0) {
        const long long t0 = clock64();
        for (;;) {
            const unsigned v = ld_acquire_u32(p);
            if (exact ? v == target : v >= target) break;
            if (clock64() - t0 > kDecWaitCycles) {
                ok = 0;
                break;
            }
            if (clock64() - t0 > 4000) __nanosleep(100);  // poll back to back at first, then back off
        }
    }
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

__device__ __forceinline__ void named_barrier(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// One fp32 row -> int8 in shared memory with its scale and the -8*sum block corrections
// (crates/peregrine-kernels/src/quant.rs:14-33); the maximum is taken from the data.  Called by the
// first `nthr` threads of the CTA (a multiple of 32; they meet on named barrier 1 twice);
// n4 = row length / 4 <= kDecQ * nthr; the row must be 16-byte aligned.  One copy of this code
// serves the token row and the h rows.
constexpr int kDecQ = 5;
__device__ __noinline__ void decode_quantise_row(const float4 *src4, int n4, int8_t *dst, int *cs, float *sx,
                                                 float *red, int nthr) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    float4 v[kDecQ];
#pragma unroll
    for (int u = 0; u < kDecQ; ++u) {
        const int i = tid + u * nthr;
        v[u] = i < n4 ? __ldcg(src4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float amax = 0.0f;
#pragma unroll
    for (int u = 0; u < kDecQ; ++u)
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[u].x), fabsf(v[u].y)), fmaxf(fabsf(v[u].z), fabsf(v[u].w))));
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    named_barrier(1, nthr);  // `red` may still be read from an earlier call
    if (lane == 0) red[warp] = amax;
    named_barrier(1, nthr);
    float m = red[0];
    for (int w = 1; w < (nthr >> 5); ++w) m = fmaxf(m, red[w]);
    float sc = __fdiv_rn(m, 127.0f);
    if (sc < 1e-12f) sc = 1e-12f;
    const float inv = __fdiv_rn(1.0f, sc);
    if (tid == 0) *sx = sc;
    uint32_t *q32 = reinterpret_cast<uint32_t *>(dst);
#pragma unroll
    for (int u = 0; u < kDecQ; ++u) {
        const int i = tid + u * nthr;
        const int q0 = max(-128, min(127, __float2int_rn(__fmul_rn(v[u].x, inv))));
        const int q1 = max(-128, min(127, __float2int_rn(__fmul_rn(v[u].y, inv))));
        const int q2 = max(-128, min(127, __float2int_rn(__fmul_rn(v[u].z, inv))));
        const int q3 = max(-128, min(127, __float2int_rn(__fmul_rn(v[u].w, inv))));
        if (i < n4)
            q32[i] = (uint32_t)(q0 & 255) | ((uint32_t)(q1 & 255) << 8) | ((uint32_t)(q2 & 255) << 16) |
                     ((uint32_t)(q3 & 255) << 24);
        int sum = (q0 + q1) + (q2 + q3);
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
        if ((lane & 7) == 0 && i < n4) cs[i >> 3] = -8 * sum;
    }
}

// Top-k of one token by one warp from parallel-sum logits: scores from the fast exponential, the
// rules of crates/peregrine-model/src/router.rs:86-150 (strict '>' from -inf, ties to the lowest
// index, NaN / -inf never chosen).  Lane kk returns pick kk in my_idx; `kept` = picks made.  With
// `dry` set nothing is read from memory: the call only brings the code in (the routine runs once per
// step, long after the L2 has been swept, so its first pass pays for its instruction fetches).
__device__ __noinline__ void decode_select(const float *spec_logits, const float *bias, const float (&bias_r)[8], int E,
                                           int k, unsigned *keys, int dry, int &my_idx_out, int &kept_out) {
    const int lane = threadIdx.x & 31;
    int kept = k, my_idx = 0;
    if (E <= 256) {
        // keys in registers: lane l holds experts l, 32 + l, ...; a round is a local maximum, a warp
        // maximum and a warp minimum over the indices that reach it
        unsigned kr[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int e = u * 32 + lane;
            const float lgv = (e < E && !dry) ? __ldcg(spec_logits + e) : (float)(e & 7);
            const float c = __fdividef(1.0f, 1.0f + __expf(-lgv)) + (dry ? 0.0f : bias_r[u]);
            unsigned q = 0u;
            if (e < E && c > -INFINITY) {  // false for NaN and -inf: never selectable
                q = __float_as_uint(c == 0.0f ? 0.0f : c);
                q = (q & 0x80000000u) ? ~q : (q | 0x80000000u);
            }
            kr[u] = q;
        }
        for (int kk = 0; kk < k; ++kk) {
            unsigned bu = 0u;
            int bi = 0x7fffffff;
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (kr[u] > bu) {  // ascending index within a lane: the first maximum keeps the lowest
                    bu = kr[u];
                    bi = u * 32 + lane;
                }
            const unsigned top = __reduce_max_sync(0xffffffffu, bu);
            if (top == 0u) {
                kept = kk;
                break;
            }
            const int best = (int)__reduce_min_sync(0xffffffffu, (unsigned)(bu == top ? bi : 0x7fffffff));
            if (lane == kk) my_idx = best;
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (u * 32 + lane == best) kr[u] = 0u;  // never chosen again
        }
    } else {
        for (int e = lane; e < E; e += 32) {
            const float lgv = dry ? (float)(e & 7) : __ldcg(spec_logits + e);
            const float c = __fdividef(1.0f, 1.0f + __expf(-lgv)) + (dry ? 0.0f : __ldg(bias + e));
            unsigned q = 0u;
            if (c > -INFINITY) {
                q = __float_as_uint(c == 0.0f ? 0.0f : c);
                q = (q & 0x80000000u) ? ~q : (q | 0x80000000u);
            }
            keys[e] = q;
        }
        __syncwarp();
        for (int kk = 0; kk < k; ++kk) {
            unsigned bu = 0u;
            int bi = 0x7fffffff;
            for (int e = lane; e < E; e += 32) {
                const unsigned u = keys[e];
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
            if (lane == kk) my_idx = best;
            if (lane == 0) keys[best] = 0u;
            __syncwarp();
        }
    }
    my_idx_out = my_idx;
    kept_out = kept;
}

template <bool GROUPED, int BPG>
__global__ void __launch_bounds__(kGemvThreads, 1) decode_step_kernel(const DecodeArgs A) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    unsigned epoch = 0;  // lane 0 of every warp holds it (only lane 0 ever compares or publishes it)
    if (lane == 0) epoch = __ldcg(A.epoch_word);
    if ((int)blockIdx.x < A.n_chain) {
        if (tid == 0) decode_stamp(A, 0);
        const bool planned = route_chain_role(A.route, smem, blockIdx.x);
        if (tid == 0) decode_stamp(A, 1);
        if (planned) {  // uniform over the CTA
            __threadfence();
            __syncthreads();
            if (tid == 0) st_release_u32(A.exact_flag, epoch);
        }
        return;
    }
    // ------------------------------------------------------------------ worker role
    const int W = gridDim.x - A.n_chain, wb = blockIdx.x - A.n_chain;
    const int k = A.route.k, E = A.route.E, D = A.route.D;
    const int I = A.gu.O;  // rows of a gate matrix = width of h
    uint8_t *p = smem + kRingBytes + kGemvBarBytes;
    GemvSlot *vs_gu = reinterpret_cast<GemvSlot *>(p);  // [0] shared expert, [1 + j] pick j
    GemvSlot *vs_dn = reinterpret_cast<GemvSlot *>(p + kDecSlotBytes);
    volatile int *ctl = reinterpret_cast<volatile int *>(p + 2 * kDecSlotBytes);
    float *part = reinterpret_cast<float *>(p + 2 * kDecSlotBytes + kDecCtlInts * 4);
    float *red = part + ((kDecEPC * kGemvWarps + 15) & ~15);
    unsigned *keys = reinterpret_cast<unsigned *>(red + 16);
    uint8_t *area = reinterpret_cast<uint8_t *>(keys) + (((size_t)E * 4 + 15) & ~(size_t)15);
    // the token's int8 row (kept for a second attempt), then the k + 1 quantised h rows (a CTA fills
    // only the row of the slot it is dealt)
    int8_t *xs0 = reinterpret_cast<int8_t *>(area);
    int *cs0 = reinterpret_cast<int *>(area + ((A.gu.xq_stride + 15) & ~15));
    float *sx0 = reinterpret_cast<float *>(cs0 + A.gu.cs_stride);
    uint8_t *area1 = reinterpret_cast<uint8_t *>(sx0 + 4);
    int8_t *xs1 = reinterpret_cast<int8_t *>(area1);
    int *cs1 = reinterpret_cast<int *>(area1 + (((k + 1) * A.dn.xq_stride + 15) & ~15));
    float *sx1 = reinterpret_cast<float *>(cs1 + (k + 1) * A.dn.cs_stride);

    WarpStream S;
    stream_init(S, smem, warp, lane);
    if (tid == 0) decode_stamp(A, 0);
    if (tid == 0) {
        GemvSlot g{A.shared.gate, A.shared.up, A.shared.gate_rs, A.shared.up_rs, k, A.has_shared ? 1 : 0};
        GemvSlot d{A.shared.down, nullptr, A.shared.down_rs, nullptr, k, A.has_shared ? 1 : 0};
        vs_gu[0] = g;
        vs_dn[0] = d;
        ctl[33] = 0;
        ctl[34] = 0;
        ctl[36] = 0;
        ctl[37] = 0;
    }
    __syncthreads();
    const int stride = W * kGemvWarps, first = wb + W * warp;  // a warp's rank in the grid (combine tiles)
    // Gate/up: the worker CTAs are dealt to the k (+1 with a shared expert) slots, so that a CTA
    // streams the two matrices of ONE expert (few pages per SM) and the shared expert's group can
    // start before anything is selected; inside a group the row tiles go round the warps.
    const int gu_slots = k + (A.has_shared ? 1 : 0);
    const int gu_a = wb % gu_slots;
    const int gu_slot = A.has_shared ? gu_a : gu_a + 1;
    const int gu_gsz = (W - gu_a + gu_slots - 1) / gu_slots;
    const int gu_first = gu_slot * A.gu.warp_tiles + wb / gu_slots + gu_gsz * warp;
    const int gu_total = (gu_slot + 1) * A.gu.warp_tiles;
    const int gu_stride = gu_gsz * kGemvWarps;
    const bool pre_cta = gu_slot == 0;  // this CTA streams the shared expert: no selection needed

    // ---- the shared expert's gate/up chunks start to arrive while the logits are formed
    stream_begin<1, GROUPED, BPG>(S, A.gu, vs_gu, gu_first, pre_cta ? gu_total : 0, gu_stride, lane);
    // what the selection will read in a dependent chain (bias, expert table) is pulled into L2 now:
    // after a cold start each would be a DRAM round trip on the critical path
    {
        const int table_lines = (int)(((size_t)(E + 1) * sizeof(ExpertDev) + 127) / 128);
        const int bias_lines = (E * 4 + 127) / 128;
        const int line = wb * 2 + (tid >> 5);  // warps 0 and 1 of every CTA: two lines per CTA
        if (lane == 0 && warp < 2) {
            for (int l = line; l < table_lines + bias_lines; l += 2 * W) {
                const char *q = l < table_lines ? reinterpret_cast<const char *>(A.route.experts) + (size_t)l * 128
                                                : reinterpret_cast<const char *>(A.route.bias) + (size_t)(l - table_lines) * 128;
                prefetch_l2(q);
            }
        }
    }
    float bias_r[8];  // selection warp: the first 256 experts' bias, fetched long before it is needed
#pragma unroll
    for (int u = 0; u < 8; ++u) bias_r[u] = 0.0f;
    if (warp == kGemvWarps - 1) {
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (u * 32 + lane < E) bias_r[u] = __ldg(A.route.bias + u * 32 + lane);
    }
    // ---- warps 0-10: parallel-sum logits of this CTA's experts (every warp one contiguous part of D,
    // all loads of a round issued before the first use), published at once; then the token's int8
    // row, which only the streaming below needs.  Meanwhile the selection warp runs its routine once
    // without data, so that the real selection finds its code in place.
    constexpr int kDotWarps = kGemvWarps - 1, kDotThreads = kDotWarps * 32;
    if (warp < kDotWarps) {
        const int n4 = D >> 2;
        const int per = (n4 + kDotWarps - 1) / kDotWarps;
        const int lo = warp * per, hi = min(n4, lo + per);
        const float4 *x4 = reinterpret_cast<const float4 *>(A.route.x);
        for (int e0 = wb; e0 < E; e0 += W * kDecEPC) {
            float4 xv[kDecU], wv[kDecEPC][kDecU];
#pragma unroll
            for (int u = 0; u < kDecU; ++u) {
                const int i = lo + u * 32 + lane;
                const bool in = i < hi;
#pragma unroll
                for (int j = 0; j < kDecEPC; ++j) {
                    const int e = e0 + j * W;
                    wv[j][u] = (in && e < E) ? __ldg(reinterpret_cast<const float4 *>(A.route.rw + (long long)e * D) + i)
                                             : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                xv[u] = in ? __ldg(x4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int j = 0; j < kDecEPC; ++j) {
                float acc = 0.0f;
#pragma unroll
                for (int u = 0; u < kDecU; ++u)
                    acc += (xv[u].x * wv[j][u].x + xv[u].y * wv[j][u].y) + (xv[u].z * wv[j][u].z + xv[u].w * wv[j][u].w);
                for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                if (lane == 0) part[j * kGemvWarps + warp] = acc;
            }
            named_barrier(2, kDotThreads);
            if (tid < kDecEPC) {
                const int e = e0 + tid * W;
                if (e < E) {
                    float sum = 0.0f;
                    for (int q = 0; q < kDotWarps; ++q) sum += part[tid * kGemvWarps + q];
                    A.spec_logits[e] = sum * A.spec_sign;
                    __threadfence();  // the writer publishes; the CTA's arrival below follows a barrier
                }
            }
            named_barrier(2, kDotThreads);
        }
        if (tid == 0) atomicAdd(A.sync + 0, 1u);  // this CTA's logits are visible
        if (tid == 0) decode_stamp(A, 2);
        decode_quantise_row(x4, n4, xs0, cs0, sx0, red, kDotThreads);
        named_barrier(2, kDotThreads);  // the row is complete for these warps; the selection warp is told below
        if (tid == 0) {
            __threadfence_block();
            ctl[36] = 1;
            decode_stamp(A, 1);
        }
    } else {
        int d_idx, d_kept;
        decode_select(A.spec_logits, A.route.bias, bias_r, E, k, keys, 1, d_idx, d_kept);
        if (d_kept < 0) A.out[0] = (float)d_idx;  // never true; keeps the dry call alive
    }

    // Fills the routed entries of both slot tables from a selection: lane j holds pick j.
    auto build_tables = [&](int my_idx, int kept) {
        ExpertDev ex = {};
        if (lane < kept) ex = A.route.experts[my_idx];
        if (lane < k) {
            const int nrows = lane < kept ? 1 : 0;
            GemvSlot g{ex.gate, ex.up, ex.gate_rs, ex.up_rs, lane, nrows};
            GemvSlot d{ex.down, nullptr, ex.down_rs, nullptr, lane, nrows};
            vs_gu[1 + lane] = g;
            vs_dn[1 + lane] = d;
            ctl[lane] = my_idx;
        }
        if (lane == 0) {
            ctl[32] = kept;
            ctl[35] = kept + (A.has_shared ? 1 : 0);
        }
        __syncwarp();
    };

    if (warp == kGemvWarps - 1) {
        // ---- speculative selection (one warp per CTA, every CTA the same result): scores from the fast
        // exponential, the rules of crates/peregrine-model/src/router.rs:86-150
        if (!warp_wait_counter(A.sync + 0, (unsigned)W, false, lane) && lane == 0)
            report_error(A.route.err, kErrBarrierTimeout);
        if (lane == 0) decode_stamp(A, 14);
        int kept, my_idx;
        decode_select(A.spec_logits, A.route.bias, bias_r, E, k, keys, 0, my_idx, kept);
        if (lane == 0) decode_stamp(A, 15);
        build_tables(my_idx, kept);
        __threadfence_block();
        if (lane == 0) ctl[33] = 1;
        if (lane == 0) decode_stamp(A, 3);
        {  // the token row written by the other warps
            const long long t0 = clock64();
            while (ctl[36] == 0) {
                if (clock64() - t0 > kDecWaitCycles) {
                    if (lane == 0) report_error(A.route.err, kErrBarrierTimeout);
                    break;
                }
                __nanosleep(40);
            }
            __syncwarp();
            __threadfence_block();
        }
    }

    bool exact_seen = false;  // this warp has observed the exact plan's flag and holds its picks and weights
    int e_idx = 0, ke = 0;
    float wj = 0.0f;
    auto fetch_exact = [&]() {
        e_idx = lane < k ? __ldcg(A.route.plan.idx + lane) : 0;
        ke = __ldcg(A.route.plan.keff);
        wj = lane < k ? __ldcg(A.route.plan.w + lane) : 0.0f;
        exact_seen = true;
    };
    for (int attempt = 0; attempt < 2; ++attempt) {
        float *h_att = A.h + (size_t)attempt * (k + 1) * I;
        unsigned *col_done = A.sync + 8 + attempt * A.n_col;
        int n_active = 0, dn_row = 0, dn_first = 0, dn_total = 0, dn_stride = 1;
        if (attempt == 1) {
            // ---- the step again, from the exact selection
            if (warp == kGemvWarps - 1) {
                const int my_idx = lane < k ? __ldcg(A.route.plan.idx + lane) : 0;
                const int kept = __ldcg(A.route.plan.keff);
                build_tables(my_idx, kept);
            }
            __syncthreads();
        }
        // phase 0: the shared expert's gate/up items (first attempt; they need no selection)
        // phase 1: gate/up + SwiGLU of the picks       phase 2: down + ordered combine
        // One copy of the streaming code serves all three.
        for (int ph = attempt == 0 ? 0 : 1; ph < 3; ++ph) {
            const bool down = ph == 2;
            if (ph == 1) {
                if (attempt == 0) {
                    const long long t0 = clock64();
                    while (ctl[33] == 0) {
                        if (clock64() - t0 > kDecWaitCycles) {
                            if (lane == 0) report_error(A.route.err, kErrBarrierTimeout);
                            break;
                        }
                        __nanosleep(40);
                    }
                    __syncwarp();
                    __threadfence_block();  // the tables written before the flag
                }
                // (first attempt: the shared expert's group has already done its items in phase 0)
                stream_begin<1, GROUPED, BPG>(S, A.gu, vs_gu, gu_first, (attempt == 0 && pre_cta) ? 0 : gu_total,
                                              gu_stride, lane);
            }
            if (down) {
                __threadfence();  // every lane publishes the h values it stored
                if (lane == 0) decode_stamp(A, 4);
                // The worker CTAs are dealt to the slots that have rows, so that a CTA needs one row of
                // h only; inside a slot's group of CTAs the column-tile pairs go round the warps.  The
                // first down chunks of this warp arrive while the rest of the grid finishes gate/up.
                n_active = ctl[35];
                if (n_active > 0) {
                    const int a_idx = wb % n_active;
                    const int slot = A.has_shared ? a_idx : a_idx + 1;
                    const int gsz = (W - a_idx + n_active - 1) / n_active;  // CTAs dealt to this slot
                    dn_row = slot == 0 ? k : slot - 1;
                    // as many warps of the group as give every one of them the same number of items:
                    // a last round that only a few warps run is a tail the whole grid waits for
                    const int rounds = (A.dn.warp_tiles + gsz * kGemvWarps - 1) / (gsz * kGemvWarps);
                    const int active = (A.dn.warp_tiles + rounds - 1) / rounds;
                    const int r_idx = wb / n_active + gsz * warp;  // consecutive items go to different CTAs
                    dn_stride = active;
                    dn_first = slot * A.dn.warp_tiles + r_idx;
                    dn_total = r_idx < active ? (slot + 1) * A.dn.warp_tiles : 0;
                }
                stream_begin<1, GROUPED, BPG>(S, A.dn, vs_dn, dn_first, dn_total, dn_stride, lane);
                __syncthreads();
                // one arrival and one poller per CTA
                if (warp == 0) {
                    if (lane == 0) atomicAdd(A.sync + 2 + attempt, 1u);
                    if (!warp_wait_counter(A.sync + 2 + attempt, (unsigned)W, false, lane) && lane == 0)
                        report_error(A.route.err, kErrBarrierTimeout);
                }
                __syncthreads();
                if (tid == 0) decode_stamp(A, 5);
                if (n_active > 0)
                    decode_quantise_row(reinterpret_cast<const float4 *>(h_att + (size_t)dn_row * I), I >> 2,
                                        xs1 + (size_t)dn_row * A.dn.xq_stride, cs1 + dn_row * A.dn.cs_stride,
                                        sx1 + dn_row, red, kGemvThreads);
                else  // nothing selectable and no shared expert: the combine of nothing is zero
                    for (int col = wb * kGemvThreads + tid; col < D; col += W * kGemvThreads) A.out[col] = 0.0f;
                __syncthreads();
                if (tid == 0) decode_stamp(A, 6);
                // the warps that will combine fetch the exact plan now if it is there already (it
                // normally is, long since), so the end of the step does not wait for these round trips
                if (first < A.n_col && !exact_seen) {
                    int there = 0;
                    if (lane == 0) there = ld_acquire_u32(A.exact_flag) == epoch;
                    if (__shfl_sync(0xffffffffu, there, 0)) fetch_exact();
                }
            }
            GemvParams P;
            if (down)
                P = A.dn;
            else
                P = A.gu;
            const GemvSlot *slots = down ? vs_dn : vs_gu;
            const int total = down ? dn_total : (((ph == 0) == pre_cta || attempt == 1) ? gu_total : 0);
            const int strd = down ? dn_stride : gu_stride;
            stream_run<1, GROUPED, BPG, 1, false>(
                S, P, slots, total, strd, down ? xs1 : xs0, down ? cs1 : cs0, down ? sx1 : sx0, down ? A.y : h_att, nullptr,
                lane, [&](int tile) {
                    // (down phase only) one more slot has stored its part of this 32-column tile
                    __threadfence();
                    __syncwarp();
                    if (lane == 0) atomicAdd(col_done + tile, 1u);
                });
            if (S.failed) stream_drain(S);
        }
        // ---- ordered combine, the column tiles dealt round the warps of the whole grid:
        // out = sum_j w_j * y_j in pick order (a single token's batch-union order), the shared expert
        // last (crates/peregrine-model/src/mlp.rs:111-127); weights and the checked selection come
        // from the exact plan
        if (n_active > 0 && first < A.n_col) {
            bool go = true;
            if (lane == 0) decode_stamp(A, 9);
            if (!exact_seen) {
                if (!warp_wait_counter(A.exact_flag, epoch, true, lane)) {
                    if (lane == 0) report_error(A.route.err, kErrBarrierTimeout);
                    go = false;
                } else {
                    fetch_exact();
                }
            }
            if (go && attempt == 0) {
                const int s_idx = lane < k ? ctl[lane] : 0;
                if (__any_sync(0xffffffffu, e_idx != s_idx) || ke != ctl[32]) go = false;  // redone below
            }
            for (int tile = first; go && tile < A.n_col; tile += stride) {
                if (!warp_wait_counter(col_done + tile, (unsigned)n_active, false, lane)) {
                    if (lane == 0) report_error(A.route.err, kErrBarrierTimeout);
                    break;
                }
                __threadfence();
                const int col = tile * 32 + lane;
                const bool in = col < D;
                const float ysh = (A.has_shared && in) ? __ldcg(A.y + (long long)k * D + col) : 0.0f;
                float a = 0.0f;
                for (int j0 = 0; j0 < ke; j0 += 8) {
                    float yv[8], wv[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int j = j0 + u;
                        wv[u] = __shfl_sync(0xffffffffu, wj, j & 31);
                        yv[u] = (j < ke && in) ? __ldcg(A.y + (long long)j * D + col) : 0.0f;
                    }
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        if (j0 + u < ke) a = __fadd_rn(a, __fmul_rn(wv[u], yv[u]));
                }
                if (A.has_shared) a = __fadd_rn(a, ysh);
                if (in) A.out[col] = a;
            }
            if (lane == 0) decode_stamp(A, 10);
        }
        if (lane == 0) decode_stamp(A, 7);
        // ---- every CTA decides alike whether the step has to be done again
        __syncthreads();
        if (warp == 0) {
            int mismatch = 0;
            if (attempt == 0) {
                if (!warp_wait_counter(A.exact_flag, epoch, true, lane)) {
                    if (lane == 0) report_error(A.route.err, kErrBarrierTimeout);
                } else {
                    const int e_idx = lane < k ? __ldcg(A.route.plan.idx + lane) : 0;
                    const int s_idx = lane < k ? ctl[lane] : 0;
                    mismatch = (__any_sync(0xffffffffu, e_idx != s_idx) || __ldcg(A.route.plan.keff) != ctl[32]) ? 1 : 0;
                }
            }
            if (lane == 0) ctl[34] = mismatch;
        }
        __syncthreads();
        if (ctl[34] == 0) break;
    }
    // ---- leave: the last worker CTA out re-zeroes the counters for the next launch
    __syncthreads();
    if (tid == 0) decode_stamp(A, 8);
    if (tid == 0) {
        __threadfence();
        ctl[37] = (atomicAdd(A.sync + 1, 1u) == (unsigned)(W - 1)) ? 1 : 0;
    }
    __syncthreads();
    if (ctl[37]) {
        for (int i = tid; i < 8 + 2 * A.n_col; i += blockDim.x) A.sync[i] = 0u;
        // every CTA of this launch has read the step number (the workers have all arrived here, the
        // chain CTAs finished before the plan the workers waited for); zero is never a step number
        if (tid == 0) *A.epoch_word = (epoch + 1u != 0u) ? epoch + 1u : 1u;
    }
}

}  // namespace pgb
