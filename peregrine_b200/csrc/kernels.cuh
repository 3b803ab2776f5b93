// Device kernels of the MoE expert-FFN path for sm_100a.
//
// Arithmetic contract (identical to the CPU reference kernels, file:line given
// at each kernel): IEEE fp32, round-to-nearest-even, no FMA contraction (the
// translation unit is compiled with -fmad=false and the order-sensitive steps
// use __fmul_rn/__fadd_rn/__fdiv_rn explicitly), integer dots exact in int32.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "w4_layout.h"

namespace pgb {

// ------------------------------------------------------------------ PTX glue
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
// 1-D bulk copy global -> shared (TMA engine), completion counted on an mbarrier.
// Source, destination and size must be multiples of 16 bytes.  One destination CTA.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
// Programmatic dependent launch: a launch made with the programmatic-serialisation attribute may
// start while its predecessor in the stream is still running; it must not touch anything the
// predecessor writes before griddep_wait().  Both are no-ops in an ordinary launch.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// Bulk prefetch of a global range into L2 (source 16-byte aligned, size a multiple of 16 bytes).
__device__ __forceinline__ void bulk_prefetch_l2(const void *src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void prefetch_l2(const void *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

// unsigned bytes of `a` times signed bytes of `b`, accumulated into c
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// The exponential both sides of the parity check use: the fp64 exponential
// rounded once to fp32.
__device__ __forceinline__ float exp32(float v) { return __double2float_rn(exp((double)v)); }
// crates/peregrine-model/src/math.rs:103-110
__device__ __forceinline__ float sigmoid32(float v) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, exp32(-v))); }
__device__ __forceinline__ float silu32(float v) { return __fdiv_rn(v, __fadd_rn(1.0f, exp32(-v))); }

// The per-device error word lives in page-locked host memory that the device can address, so the
// host reads it after a synchronise without queueing a copy.  It is only written on a failure.
__device__ __forceinline__ void report_error(int *err, int code) {
    *reinterpret_cast<volatile int *>(err) = code;
    __threadfence_system();
}
// Error codes written to the per-device error word.
enum : int { kErrNone = 0, kErrBarrierTimeout = 1 };

// ------------------------------------------------------- activation quantiser
// Layout of the quantised activations a launch consumes.
//   row-major  (dp4a kernel): xq[row][kp], csum[row][nblk]
//   chunk-major (tensor-core kernel): xq[chunk][pcap][272] (256 bytes of the chunk + 16 bytes of
//     skew so that 8 consecutive rows land on distinct shared-memory banks), csum[chunk][pcap][8];
//     the rows of one expert are consecutive, so one bulk copy fetches a pass's rows of a chunk.
constexpr int kXqChunkRowBytes = kChunkElems + 16;

// crates/peregrine-kernels/src/quant.rs:14-33, one CTA per row.  Besides the
// int8 row (zero padded) and its scale it writes, per 32-element block,
// -8 * sum(q): the term that turns the stream's stored nibbles (v+8) back into
// signed weights inside the integer dot.  `rowmap` (optional) names the source row
// of output row r; `pcap` > 0 selects the chunk-major layout with that row capacity, `pcap` < 0
// the core-matrix layout of the tcgen05 kernel with capacity -pcap.
__global__ void __launch_bounds__(256) qrow_i8_kernel(const float *__restrict__ x, long long ldx, int K, int kp,
                                                      int nblk, int8_t *__restrict__ xq, float *__restrict__ sx,
                                                      int *__restrict__ csum, const int *__restrict__ n_rows_dev,
                                                      int n_rows, const int *__restrict__ rowmap, long long pcap,
                                                      const unsigned *__restrict__ amax_bits) {
    const int row = blockIdx.x;
    const int limit = n_rows_dev ? *n_rows_dev : n_rows;
    if (row >= limit) return;
    const float *xr = x + (long long)(rowmap ? rowmap[row] : row) * ldx;
    __shared__ float red[8];
    __shared__ float s_inv;
    // amax_bits (optional, indexed by output row): the row maximum the producing launch already
    // left (bit pattern of max|x|, NaN never recorded), which saves the first pass over the row
    float amax = amax_bits ? __uint_as_float(amax_bits[row]) : 0.0f;
    if (!amax_bits) {
        for (int i = threadIdx.x; i < K; i += blockDim.x) {
            float a = fabsf(xr[i]);
            if (a > amax) amax = a;
        }
        for (int o = 16; o > 0; o >>= 1) {
            float other = __shfl_xor_sync(0xffffffffu, amax, o);
            if (other > amax) amax = other;
        }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) red[warp] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
        float m = red[0];
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
            if (red[w] > m) m = red[w];
        float s = __fdiv_rn(m, 127.0f);
        if (s < 1e-12f) s = 1e-12f;
        sx[row] = s;
        s_inv = __fdiv_rn(1.0f, s);
    }
    __syncthreads();
    const float inv = s_inv;
    for (int blk = warp; blk < nblk; blk += (int)(blockDim.x >> 5)) {
        const int i = blk * 32 + lane;
        int q = 0;
        if (i < K) {
            q = __float2int_rn(__fmul_rn(xr[i], inv));
            q = max(-128, min(127, q));
        }
        int sum = q;
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (pcap < 0) {
            // core-matrix order for the tcgen05 kernel: [chunk][16-element unit][row][16 bytes]
            const long long cap = -pcap;
            const int kk = (blk & 7) * 32 + lane;
            xq[((((long long)(blk >> 3) * 16 + (kk >> 4)) * cap + row) << 4) + (kk & 15)] = (int8_t)q;
            if (lane == 0) csum[((long long)(blk >> 3) * cap + row) * kChunkBlocks + (blk & 7)] = -8 * sum;
        } else if (pcap > 0) {
            const long long cr = (long long)(blk >> 3) * pcap + row;
            xq[cr * kXqChunkRowBytes + (blk & 7) * 32 + lane] = (int8_t)q;
            if (lane == 0) csum[cr * kChunkBlocks + (blk & 7)] = -8 * sum;
        } else {
            xq[(long long)row * kp + i] = (int8_t)q;
            if (lane == 0) csum[(long long)row * nblk + blk] = -8 * sum;
        }
    }
}

// Pair-ordered copy of already quantised token rows for the tensor-core kernels: output row p is
// token pair_token[p], in the chunk-major layout (pcap > 0) or the core-matrix layout (pcap < 0)
// described at qrow_i8_kernel.  Quantising once per token and copying int8 rows replaces
// quantising every (token, expert) pair from fp32 again.  One CTA per pair row.
__global__ void __launch_bounds__(256) gather_pair_rows_kernel(const int8_t *__restrict__ xq_tok,
                                                               const int *__restrict__ cs_tok,
                                                               const float *__restrict__ sx_tok, int kp, int nblk,
                                                               const int *__restrict__ pair_token,
                                                               const int *__restrict__ n_pairs_dev,
                                                               int8_t *__restrict__ xqp, int *__restrict__ csp,
                                                               float *__restrict__ sxp, long long pcap) {
    const int p = blockIdx.x;
    if (p >= *n_pairs_dev) return;
    const int tok = pair_token[p];
    const long long cap = pcap < 0 ? -pcap : pcap;
    const uint4 *src = reinterpret_cast<const uint4 *>(xq_tok + (long long)tok * kp);
    for (int u = threadIdx.x; u < (kp >> 4); u += blockDim.x) {
        const int chunk = u >> 4, unit = u & 15;
        const long long off = pcap < 0 ? ((((long long)chunk * 16 + unit) * cap + p) << 4)
                                       : ((long long)chunk * cap + p) * kXqChunkRowBytes + unit * 16;
        *reinterpret_cast<uint4 *>(xqp + off) = __ldg(src + u);
    }
    const int nchunk = nblk >> 3;
    const int4 *csrc = reinterpret_cast<const int4 *>(cs_tok + (long long)tok * nblk);
    for (int u = threadIdx.x; u < 2 * nchunk; u += blockDim.x) {
        const int chunk = u >> 1;
        *reinterpret_cast<int4 *>(csp + ((long long)chunk * cap + p) * kChunkBlocks + (u & 1) * 4) = __ldg(csrc + u);
    }
    if (threadIdx.x == 0) sxp[p] = sx_tok[tok];
}

// ------------------------------------------------------------ int4 x int8 GEMV
#ifndef PGB_GEMV_WARPS
#define PGB_GEMV_WARPS 12
#endif
#ifndef PGB_GEMV_STAGES
#define PGB_GEMV_STAGES 3
#endif
constexpr int kGemvWarps = PGB_GEMV_WARPS;
constexpr int kGemvStages = PGB_GEMV_STAGES;
constexpr int kGemvThreads = kGemvWarps * 32;
constexpr int kStageBytes = 2 * kChunkMaxBytes;  // two half-warp chunks
constexpr int kRingBytes = kGemvWarps * kGemvStages * kStageBytes;
constexpr int kGemvBarBytes = ((kGemvWarps * kGemvStages * 8 + 127) / 128) * 128;

// The wait every kernel here uses, with the limit as a parameter, on a barrier that never
// completes: exercises give-up, error report and a clean return.
__global__ void selftest_bounded_wait_kernel(long long limit_cycles, int *err) {
    __shared__ __align__(8) unsigned long long bar;
    const uint32_t b = smem_u32(&bar);
    if (threadIdx.x == 0) {
        mbar_init(b, 1);
        fence_mbar_init();
    }
    __syncthreads();
    const long long t0 = clock64();
    bool done = false;
    while (!(done = mbar_try_wait(b, 0u)))
        if (clock64() - t0 > limit_cycles) break;
    if (!done && threadIdx.x == 0) report_error(err, kErrBarrierTimeout);
}

// Bounded wait on an mbarrier phase; false after ~2e9 cycles.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity))
        if (clock64() - t0 > 2000000000LL) return false;
    return true;
}

// One expert's share of a launch.
struct GemvSlot {
    const uint8_t *a;   // tile stream: gate (mode 0) or down (mode 1)
    const uint8_t *b;   // tile stream: up (mode 0); unused in mode 1
    const float *a_rs;  // per-row scales, padded to ntile*16 (per-row format only)
    const float *b_rs;
    int row0;   // first pair row (output row; activation row unless rowmap is given)
    int nrows;  // pair rows of this expert
};

// The ordered combine a down launch can finish with (device-resident layer only).
struct CombineArgs {
    int *col_done;           // [warp_tiles] arrival counters, zero at launch (nullptr: no fused combine)
    const int *keff;         // [M]
    const int *comb_pair;    // [M*k] pair rows of token s in batch-union order
    const float *comb_w;     // [M*k] their gate weights
    const int *shared_pair0; // [1] first pair row of the shared expert, -1 if none
    float *out;              // [M, D]
    long long ldo;
    int M, k;
};

struct GemvParams {
    const GemvSlot *slots;
    const int *n_slots;  // device scalar
    int mode;            // 0: gate/up + SwiGLU -> h ; 1: down -> y
    int nchunk, chunk_bytes, ntile, warp_tiles, O;
    int ng_tap;          // groups per row in the tap layout (ceil(K/gs); 1 for per-row scales)
    unsigned long long tile_bytes;
    const int8_t *xq;  // activation rows, int8, natural element order, padded to nchunk*256
    int xq_stride;     // bytes per activation row (= kp)
    const int *csum;   // -8*sum per 32-block
    int cs_stride;     // ints per activation row (= nblk)
    const float *sx;   // activation row scales
    const int *rowmap; // activation row of pair p (nullptr: p itself)
    int n_xrows;       // activation rows staged in shared memory (XS kernels)
    long long pcap;    // row capacity of the chunk-major activation layout (tensor-core kernel)
    // QS kernels quantise the activation rows themselves while staging them:
    const float *x_f32;   // [n_xrows, K] fp32 rows (row stride x_ld)
    long long x_ld;
    int K;                // logical row length
    const unsigned *amax_bits;  // [n_xrows] bit pattern of max|x| per row
    // speculative routing: the launch compares two selections (spec_n ids and spec_m counts).  Equal:
    // a mode-0 launch has nothing to repair and returns; a mode-1 launch reads amax_bits.  Different:
    // the mode-0 launch recomputes under its (exact) slots, the mode-1 launch reads amax_alt.
    const int *spec_a, *spec_b, *spec_ka, *spec_kb;
    int spec_n, spec_m;
    const unsigned *amax_alt;
    float neg_zero;  // -0.0f, as a run-time value: the fold's product is an FMA onto it (see fold_pair)
    int grid;  // host only: CTAs to launch (0 = one per SM)
    int pdl;   // host only: launch with programmatic stream serialisation (see griddep_wait)
    int tile_rb;  // host only: > 0 selects the large-batch tile kernel with this many row blocks in the grid
    int blk_rpp;  // shared-row kernel: rows per work unit (32, 16 or 8); 0: chosen by the kernel
    int umma;     // host only: with tile_rb > 0, take the tcgen05 kernel (activations in core-matrix order)
    const int *n_xrows_dev;     // rows actually valid (device scalar; nullptr: n_xrows)
    unsigned *amax_out;   // mode 0: per pair row, atomicMax of |h| bits (nullptr: off)
    float *out;
    long long out_stride;
    CombineArgs comb;
    int *tap;  // optional per-group int32 accumulators (TAP kernels)
    int *err;
};

struct TileCursor {
    int i, tile, pass, chunk, npass, row0, nrows;
    const uint8_t *a, *b;
    const float *a_rs, *b_rs;
};

// `slots` is the launch's slot table: P.slots, or a table a kernel keeps in shared memory.
template <int RMAX>
__device__ __forceinline__ void cursor_seek(TileCursor &c, const GemvParams &P, const GemvSlot *slots, int total,
                                            int stride) {
    // position on the first tile at or after c.i that has rows to compute
    while (c.i < total) {
        const int slot = c.i / P.warp_tiles;
        const int t = c.i - slot * P.warp_tiles;
        const GemvSlot *s = slots + slot;
        c.nrows = s->nrows;
        c.npass = (c.nrows + RMAX - 1) / RMAX;
        if (c.npass > 0) {
            c.tile = t;
            c.row0 = s->row0;
            c.a_rs = s->a_rs;
            c.b_rs = s->b_rs;
            if (P.mode == 0) {
                c.a = s->a + (unsigned long long)t * P.tile_bytes;
                c.b = s->b + (unsigned long long)t * P.tile_bytes;
            } else {
                c.a = s->a + (unsigned long long)(2 * t) * P.tile_bytes;
                c.b = (2 * t + 1 < P.ntile) ? s->a + (unsigned long long)(2 * t + 1) * P.tile_bytes : nullptr;
            }
            return;
        }
        c.i += stride;
    }
}

template <int RMAX>
__device__ __forceinline__ void cursor_next(TileCursor &c, const GemvParams &P, const GemvSlot *slots, int total,
                                            int stride) {
    if (++c.chunk < P.nchunk) return;
    c.chunk = 0;
    if (++c.pass < c.npass) return;
    c.pass = 0;
    c.i += stride;
    cursor_seek<RMAX>(c, P, slots, total, stride);
}

// Ordered combine of one 32-column tile by the warp whose arrival completes it (down launches of
// the device-resident layer): out starts at zero, each expert's row is added as out + (w * y) in
// batch-union order, the shared expert last (crates/peregrine-model/src/mlp.rs:111-127,
// concurrent.rs:1866-1929).  The lists of a token are read once by the warp (lane j holds entry j;
// k <= 32) and the rows of a token are fetched eight at a time before the first is used, so the
// tail of the launch is a few round trips to L2 rather than one per expert.
__device__ __forceinline__ void ordered_combine_tile(const GemvParams &P, int tile, int lane, int n_slots) {
    __threadfence();
    __syncwarp();
    int last = 0;
    if (lane == 0) last = (atomicAdd(P.comb.col_done + tile, 1) == n_slots - 1);
    last = __shfl_sync(0xffffffffu, last, 0);
    if (!last) return;
    __threadfence();
    const int col = tile * 32 + lane;
    const bool in = col < P.O;
    const int sp0 = *P.comb.shared_pair0;
    for (int s = 0; s < P.comb.M; ++s) {
        const int ke = P.comb.keff[s];
        const int pj = lane < P.comb.k ? P.comb.comb_pair[s * P.comb.k + lane] : 0;
        const float wj = lane < P.comb.k ? P.comb.comb_w[s * P.comb.k + lane] : 0.0f;
        const float ysh = (sp0 >= 0 && in) ? __ldcg(P.out + (long long)(sp0 + s) * P.out_stride + col) : 0.0f;
        float a = 0.0f;
        for (int j0 = 0; j0 < ke; j0 += 8) {
            float yv[8], wv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int j = j0 + u;
                const int p = __shfl_sync(0xffffffffu, pj, j & 31);
                wv[u] = __shfl_sync(0xffffffffu, wj, j & 31);
                yv[u] = (j < ke && in) ? __ldcg(P.out + (long long)p * P.out_stride + col) : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (j0 + u < ke) a = __fadd_rn(a, __fmul_rn(wv[u], yv[u]));
        }
        if (sp0 >= 0) a = __fadd_rn(a, ysh);
        if (in) P.comb.out[(long long)s * P.comb.ldo + col] = a;
    }
}

// Each warp streams two 16-row tiles (lanes 0-15 / 16-31) through a private
// ring of kGemvStages shared-memory stages filled by bulk copies of one
// 256-element chunk each; lane L owns one weight row for the whole K extent, so
// the fp32 fold over groups runs in ascending group order exactly as
// crates/peregrine-kernels/src/idot.rs:98-110 and matmul.rs:93-106 (grouped) /
// :75-87 (per-row scale) prescribe.
//   mode 0: half 0 = gate tile t, half 1 = up tile t; epilogue
//           h = silu(g) * u (crates/peregrine-model/src/math.rs:108-118)
//   mode 1: halves = down tiles 2t, 2t+1; epilogue y = acc * sx
// RMAX activation rows are processed per pass over a tile; an expert with more
// rows re-streams its tile (from L2) once per extra pass.  BPG = 32-element
// blocks per scale group (gs/32); a chunk always holds 8 blocks, so the inner
// loops have constant trip counts and fold into immediates.
//   XS = 0: activation rows are read from global memory (read-only path)
//   XS = 1: the launch's int8 rows are first copied into shared memory
//   XS = 2: the launch's fp32 rows are quantised into shared memory by the CTA
//           itself (crates/peregrine-kernels/src/quant.rs:14-33) from a row
//           maximum the producing launch left in amax_bits
//
// The pieces below are shared by the plain GEMV launch and by the fused decode step, which runs
// several phases (gate/up, down) over one ring without leaving the kernel.

// A warp's ring and its position in the stream of work items; lives across the phases of a kernel.
struct WarpStream {
    uint8_t *ring;
    uint32_t ring_u32, bar_u32;
    uint32_t fq, cq;  // chunks fetched / consumed so far (stage = q % kGemvStages)
    TileCursor fc, cc;
    bool failed;
};

__device__ __forceinline__ void stream_init(WarpStream &S, uint8_t *smem, int warp, int lane) {
    S.ring = smem + warp * (kGemvStages * kStageBytes);
    S.ring_u32 = smem_u32(S.ring);
    S.bar_u32 = smem_u32(smem + kRingBytes) + warp * (kGemvStages * 8);
    S.fq = S.cq = 0;
    S.failed = false;
    if (lane == 0) {
        for (int s = 0; s < kGemvStages; ++s) mbar_init(S.bar_u32 + s * 8, 1);
        fence_mbar_init();
        fence_proxy_async();
    }
    __syncwarp();
}

template <bool GROUPED, int BPG>
__device__ __forceinline__ void stream_issue(const WarpStream &S, const TileCursor &c, uint32_t q) {
    constexpr int CHUNK_BYTES = kChunkSlabBytes + (GROUPED ? (kChunkBlocks / BPG) * 64 : 0);
    const uint32_t stage = q % kGemvStages;
    const uint32_t bar = S.bar_u32 + stage * 8;
    const uint32_t dst = S.ring_u32 + stage * kStageBytes;
    const size_t off = (size_t)c.chunk * CHUNK_BYTES;
    mbar_expect_tx(bar, c.b ? 2 * CHUNK_BYTES : CHUNK_BYTES);
    bulk_g2s(dst, c.a + off, CHUNK_BYTES, bar);
    if (c.b) bulk_g2s(dst + kChunkMaxBytes, c.b + off, CHUNK_BYTES, bar);
}

// Positions the warp on its first work item in [first, total) (items `stride` apart) and fills the
// ring.  Everything fetched by an earlier phase must have been consumed (fq == cq).
template <int RMAX, bool GROUPED, int BPG>
__device__ __forceinline__ void stream_begin(WarpStream &S, const GemvParams &P, const GemvSlot *slots, int first,
                                             int total, int stride, int lane) {
    S.fc.i = first;
    S.fc.pass = 0;
    S.fc.chunk = 0;
    cursor_seek<RMAX>(S.fc, P, slots, total, stride);
    S.cc = S.fc;
    if (lane == 0 && S.fc.i < total) fence_proxy_async();
    while (S.fc.i < total && S.fq < S.cq + kGemvStages) {
        if (lane == 0) stream_issue<GROUPED, BPG>(S, S.fc, S.fq);
        cursor_next<RMAX>(S.fc, P, slots, total, stride);
        ++S.fq;
    }
}

// After a failed wait: give copies already in flight a bounded chance to land before the CTA retires.
__device__ __forceinline__ void stream_drain(WarpStream &S) {
    for (uint32_t q = S.cq; q < S.fq; ++q) {
        const uint32_t stage = q % kGemvStages, parity = (q / kGemvStages) & 1u;
        const long long t0 = clock64();
        while (!mbar_try_wait(S.bar_u32 + stage * 8, parity))
            if (clock64() - t0 > 200000000LL) break;
    }
    S.cq = S.fq;
}

// The XS = 2 staging: the CTA quantises `nrows_valid` fp32 rows (row stride x_ld, logical length K)
// into shared memory as int8 rows of stride P.xq_stride with their -8*sum block corrections and
// scales, from row maxima already known (amax_src, bit patterns, global memory).  crates/peregrine-kernels/src/quant.rs:14-33.  All threads of the CTA call it; it ends
// with a CTA barrier.
struct NoStamp {
    __device__ __forceinline__ void operator()(int) const {}
};
template <typename Stamp = NoStamp>
__device__ __forceinline__ void stage_quantise_rows(const GemvParams &P, const float *x_f32, long long x_ld, int K,
                                                    int nrows_valid, const unsigned *amax_src, int8_t *xs, int *cs_s,
                                                    float *sx_s, float *inv_s, Stamp stamp = Stamp()) {
    // four consecutive elements per thread and step; eight neighbouring lanes cover one
    // 32-element block, so the block sum is three shuffles.  Loads of a whole step batch are
    // issued before any of them is used, and the first batch goes out before the row scales
    // are known (its addresses do not depend on them).
    const int q4_per_row = P.xq_stride >> 2;
    const int total4 = nrows_valid * q4_per_row;
    const bool vec_ok = ((x_ld & 3) == 0) && ((reinterpret_cast<uintptr_t>(x_f32) & 15) == 0);
    constexpr int kBatch = 12;  // a decode step's 9 rows of 2048 are one batch: a single round trip to L2
    float4 v[kBatch];
    int rowv[kBatch], c4v[kBatch];
    auto load_batch = [&](int base4) {
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int i4 = base4 + u * (int)blockDim.x + (int)threadIdx.x;
            v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            rowv[u] = -1;
            c4v[u] = 0;
            if (i4 < total4) {
                const int row = i4 / q4_per_row, c4 = i4 - row * q4_per_row;
                rowv[u] = row;
                c4v[u] = c4;
                const float *src = x_f32 + (long long)row * x_ld + 4 * c4;
                if (vec_ok && 4 * c4 + 3 < K) {
                    v[u] = __ldcg(reinterpret_cast<const float4 *>(src));
                } else {
                    if (4 * c4 + 0 < K) v[u].x = __ldcg(src + 0);
                    if (4 * c4 + 1 < K) v[u].y = __ldcg(src + 1);
                    if (4 * c4 + 2 < K) v[u].z = __ldcg(src + 2);
                    if (4 * c4 + 3 < K) v[u].w = __ldcg(src + 3);
                }
            }
        }
    };
    auto quant_batch = [&]() {
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            // all 32 lanes take part in the shuffles; lanes past the end carry zeros
            const float inv = rowv[u] >= 0 ? inv_s[rowv[u]] : 0.0f;
            const int q0 = max(-128, min(127, __float2int_rn(__fmul_rn(v[u].x, inv))));
            const int q1 = max(-128, min(127, __float2int_rn(__fmul_rn(v[u].y, inv))));
            const int q2 = max(-128, min(127, __float2int_rn(__fmul_rn(v[u].z, inv))));
            const int q3 = max(-128, min(127, __float2int_rn(__fmul_rn(v[u].w, inv))));
            int sum = q0 + q1 + q2 + q3;
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            sum += __shfl_xor_sync(0xffffffffu, sum, 4);
            if (rowv[u] >= 0) {
                const uint32_t packed = (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) |
                                        ((uint32_t)(q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24);
                *reinterpret_cast<uint32_t *>(xs + (size_t)rowv[u] * P.xq_stride + 4 * c4v[u]) = packed;
                if ((c4v[u] & 7) == 0) cs_s[rowv[u] * P.cs_stride + (c4v[u] >> 3)] = -8 * sum;
            }
        }
    };
    load_batch(0);
    for (int row = threadIdx.x; row < nrows_valid; row += blockDim.x) {
        float s = __fdiv_rn(__uint_as_float(__ldcg(amax_src + row)), 127.0f);
        if (s < 1e-12f) s = 1e-12f;
        sx_s[row] = s;
        inv_s[row] = __fdiv_rn(1.0f, s);
    }
    stamp(11);
    __syncthreads();
    stamp(12);
    quant_batch();
    stamp(13);
    for (int base4 = kBatch * (int)blockDim.x; base4 < total4; base4 += kBatch * (int)blockDim.x) {
        load_batch(base4);
        quant_batch();
    }
    __syncthreads();
}

// Consumes the warp's items of [.., total): integer dots, fold, epilogue.  `out` / `amax_out` are
// the phase's output rows and (mode 0, optional) row-maximum words; `on_tile_done(tile)` runs when
// the last pass of a mode-1 item has been stored (all lanes call it).
template <int RMAX, bool GROUPED, int BPG, int XS, bool TAP, typename OnTileDone>
__device__ __forceinline__ void stream_run(WarpStream &S, const GemvParams &P, const GemvSlot *slots, int total,
                                           int stride, const int8_t *xbase, const int *csbase, const float *sxbase,
                                           float *out, unsigned *amax_out, int lane, OnTileDone on_tile_done) {
    constexpr int GPC = kChunkBlocks / BPG;
    const int half = lane >> 4, r16 = lane & 15;
    TileCursor &fc = S.fc, &cc = S.cc;
    float acc[RMAX];
    int iacc[RMAX];
    int arow[RMAX];

    while (cc.i < total) {
        // keep the ring full: the stage being refilled was consumed one iteration ago
        if (fc.i < total && S.fq < S.cq + kGemvStages) {
            if (lane == 0) {
                fence_proxy_async();
                stream_issue<GROUPED, BPG>(S, fc, S.fq);
            }
            cursor_next<RMAX>(fc, P, slots, total, stride);
            ++S.fq;
        }
        const uint32_t stage = S.cq % kGemvStages;
        const uint32_t parity = (S.cq / kGemvStages) & 1u;
        {
            const bool ok = mbar_wait_bounded(S.bar_u32 + stage * 8, parity);
            if (__any_sync(0xffffffffu, !ok)) {
                if (lane == 0) report_error(P.err, kErrBarrierTimeout);
                S.failed = true;
                break;
            }
        }
        if (cc.chunk == 0) {
#pragma unroll
            for (int r = 0; r < RMAX; ++r) {
                acc[r] = 0.0f;
                iacc[r] = 0;
                const int ridx = min(cc.pass * RMAX + r, cc.nrows - 1);
                const int p = cc.row0 + ridx;
                arow[r] = P.rowmap ? P.rowmap[p] : p;
            }
        }
        const uint8_t *wp = S.ring + stage * kStageBytes + half * kChunkMaxBytes + r16 * 16;
        const int o_half = (P.mode == 0) ? (cc.tile * 16 + r16) : (cc.tile * 32 + lane);

        float sc[GPC];
        if (GROUPED) {
            const float *sp =
                reinterpret_cast<const float *>(S.ring + stage * kStageBytes + half * kChunkMaxBytes + kChunkSlabBytes) +
                r16 * GPC;
            if constexpr (GPC >= 4) {
#pragma unroll
                for (int j = 0; j < GPC / 4; ++j) {
                    const float4 v = *reinterpret_cast<const float4 *>(sp + 4 * j);
                    sc[4 * j + 0] = v.x;
                    sc[4 * j + 1] = v.y;
                    sc[4 * j + 2] = v.z;
                    sc[4 * j + 3] = v.w;
                }
            } else {
#pragma unroll
                for (int j = 0; j < GPC; ++j) sc[j] = sp[j];
            }
        }
#pragma unroll
        for (int r = 0; r < RMAX; ++r) {
            // one activation row at a time keeps the live register set small
            const int8_t *xr = xbase + (size_t)arow[r] * P.xq_stride + cc.chunk * kChunkElems;
            const int *cp = csbase + (size_t)arow[r] * P.cs_stride + cc.chunk * kChunkBlocks;
            int4 c0, c1;
            if (XS) {
                c0 = *reinterpret_cast<const int4 *>(cp);
                c1 = *reinterpret_cast<const int4 *>(cp + 4);
            } else {
                c0 = __ldg(reinterpret_cast<const int4 *>(cp));
                c1 = __ldg(reinterpret_cast<const int4 *>(cp + 4));
            }
            const int cs[kChunkBlocks] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
            for (int gi = 0; gi < GPC; ++gi) {
                int dsum = 0;
#pragma unroll
                for (int b = 0; b < BPG; ++b) {
                    const int blk = gi * BPG + b;
                    const uint4 wv = *reinterpret_cast<const uint4 *>(wp + blk * kSlabBytes);
                    uint4 x0, x1;
                    if (XS) {
                        x0 = *reinterpret_cast<const uint4 *>(xr + blk * 32);
                        x1 = *reinterpret_cast<const uint4 *>(xr + blk * 32 + 16);
                    } else {
                        x0 = __ldg(reinterpret_cast<const uint4 *>(xr + blk * 32));
                        x1 = __ldg(reinterpret_cast<const uint4 *>(xr + blk * 32 + 16));
                    }
                    int lo = cs[blk];
                    lo = dp4a_us(wv.x & 0x0F0F0F0Fu, x0.x, lo);
                    lo = dp4a_us(wv.y & 0x0F0F0F0Fu, x0.y, lo);
                    lo = dp4a_us(wv.z & 0x0F0F0F0Fu, x0.z, lo);
                    lo = dp4a_us(wv.w & 0x0F0F0F0Fu, x0.w, lo);
                    int hi = dp4a_us(wv.x & 0xF0F0F0F0u, x1.x, 0);
                    hi = dp4a_us(wv.y & 0xF0F0F0F0u, x1.y, hi);
                    hi = dp4a_us(wv.z & 0xF0F0F0F0u, x1.z, hi);
                    hi = dp4a_us(wv.w & 0xF0F0F0F0u, x1.w, hi);
                    dsum += lo + (hi >> 4);  // hi is exactly 16x the upper-half dot
                }
                if (GROUPED) {
                    acc[r] = __fadd_rn(acc[r], __fmul_rn(sc[gi], (float)dsum));
                    if (TAP) {
                        const int g = cc.chunk * GPC + gi;
                        const int ridx = cc.pass * RMAX + r;
                        if (P.tap != nullptr && o_half < P.O && g < P.ng_tap && ridx < cc.nrows) {
                            // mode 0 taps gate (half 0) and up (half 1) side by side: [pair][2][O][ng]
                            const long long base =
                                (P.mode == 0) ? ((long long)(cc.row0 + ridx) * 2 + half) * P.O + o_half
                                              : (long long)(cc.row0 + ridx) * P.O + o_half;
                            P.tap[base * P.ng_tap + g] = dsum;
                        }
                    }
                } else {
                    iacc[r] += dsum;
                }
            }
        }
        __syncwarp();
        if (cc.chunk == P.nchunk - 1) {
            float rs = 0.0f;
            if (!GROUPED) {
                const float *rsp = (P.mode == 0 && half) ? cc.b_rs : cc.a_rs;
                rs = (o_half < P.ntile * 16) ? rsp[o_half] : 0.0f;
            }
#pragma unroll
            for (int r = 0; r < RMAX; ++r) {
                const int ridx = cc.pass * RMAX + r;
                const bool valid = ridx < cc.nrows;
                const float sxa = sxbase[arow[r]];
                float v;
                if (GROUPED) {
                    v = __fmul_rn(acc[r], sxa);
                } else {
                    if (TAP && P.tap != nullptr && valid && o_half < P.O) {
                        const long long base = (P.mode == 0) ? ((long long)(cc.row0 + ridx) * 2 + half) * P.O + o_half
                                                             : (long long)(cc.row0 + ridx) * P.O + o_half;
                        P.tap[base] = iacc[r];
                    }
                    v = __fmul_rn(__fmul_rn((float)iacc[r], rs), sxa);
                }
                if (P.mode == 0) {
                    const float u = __shfl_down_sync(0xffffffffu, v, 16);
                    float hval = 0.0f;
                    const bool store = valid && half == 0 && o_half < P.O;
                    if (store) {
                        hval = __fmul_rn(silu32(v), u);
                        out[(long long)(cc.row0 + ridx) * P.out_stride + o_half] = hval;
                    }
                    if (amax_out != nullptr) {
                        // row maximum of |h| for the quantiser of the next launch: max is order-free,
                        // NaN never becomes the maximum (crates/peregrine-kernels/src/quant.rs:17-22)
                        float a = fabsf(hval);
                        if (!(a == a)) a = 0.0f;
                        for (int o = 8; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
                        if (valid && lane == 0 && a > 0.0f) atomicMax(amax_out + cc.row0 + ridx, __float_as_uint(a));
                    }
                } else {
                    if (valid && o_half < P.O) out[(long long)(cc.row0 + ridx) * P.out_stride + o_half] = v;
                }
            }
            if (P.mode == 1 && cc.pass == cc.npass - 1) on_tile_done(cc.tile);
        }
        cursor_next<RMAX>(cc, P, slots, total, stride);
        ++S.cq;
    }
}

template <int RMAX, bool GROUPED, int BPG, int XS, bool TAP>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_w4a8_kernel(const GemvParams P) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // gate/up reads its slot table from the launch before it; a down launch only depends on its
    // predecessor (the repair launch) for the activation rows, see below
    griddep_launch_dependents();
    if (P.mode == 0) griddep_wait();
    // Scalars of the plan are fetched here, together with the selections compared below, so that
    // the dependent steps further down (slot table, staging) do not each start with a round trip
    // of their own: after a cold start every first touch costs a microsecond.
    const int n_slots = __ldcg(P.n_slots);
    const int n_xrows_now = (XS == 2 && P.n_xrows_dev) ? __ldcg(P.n_xrows_dev) : P.n_xrows;
    bool spec_same = true;
    if (P.spec_a) {
        int bad = 0;
        for (int i = threadIdx.x; i < P.spec_n; i += blockDim.x) bad |= (__ldcg(P.spec_a + i) != __ldcg(P.spec_b + i));
        for (int i = threadIdx.x; i < P.spec_m; i += blockDim.x) bad |= (__ldcg(P.spec_ka + i) != __ldcg(P.spec_kb + i));
        spec_same = __syncthreads_or(bad) == 0;
        if (P.mode == 0 && spec_same) return;  // the speculative launch already produced these rows
    }
    int8_t *xs = reinterpret_cast<int8_t *>(smem + kRingBytes + kGemvBarBytes);
    const int xs_bytes = (P.n_xrows * P.xq_stride + 15) & ~15;
    int *cs_s = reinterpret_cast<int *>(xs + xs_bytes);
    float *sx_s = reinterpret_cast<float *>(cs_s + P.n_xrows * P.cs_stride);

    WarpStream S;
    stream_init(S, smem, warp, lane);
    const int total = n_slots * P.warp_tiles;
    const int stride = gridDim.x * kGemvWarps;
    // first fill of the ring overlaps the activation staging below
    stream_begin<RMAX, GROUPED, BPG>(S, P, P.slots, blockIdx.x + gridDim.x * warp, total, stride, lane);

    // everything above (plan, weight prefetch) is independent of the preceding launch; the
    // activation rows and their row maxima are not
    if (P.mode != 0) griddep_wait();
    if (XS == 1) {
        const int n16 = xs_bytes >> 4;
        const uint4 *src = reinterpret_cast<const uint4 *>(P.xq);
        uint4 *dst = reinterpret_cast<uint4 *>(xs);
        for (int i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = src[i];
        const int ncs = P.n_xrows * P.cs_stride;
        for (int i = threadIdx.x; i < ncs; i += blockDim.x) cs_s[i] = P.csum[i];
        for (int i = threadIdx.x; i < P.n_xrows; i += blockDim.x) sx_s[i] = P.sx[i];
        __syncthreads();
    } else if (XS == 2) {
        const unsigned *ab = (P.amax_alt && !spec_same) ? P.amax_alt : P.amax_bits;
        stage_quantise_rows(P, P.x_f32, P.x_ld, P.K, min(n_xrows_now, P.n_xrows), ab, xs, cs_s, sx_s,
                            sx_s + P.n_xrows);
    }
    const int8_t *xbase = XS ? xs : P.xq;
    const int *csbase = XS ? cs_s : P.csum;
    const float *sxbase = XS ? sx_s : P.sx;
    stream_run<RMAX, GROUPED, BPG, XS, TAP>(S, P, P.slots, total, stride, xbase, csbase, sxbase, P.out, P.amax_out,
                                            lane, [&](int tile) {
                                                if (P.comb.col_done != nullptr)
                                                    ordered_combine_tile(P, tile, lane, n_slots);
                                            });
    if (S.failed) stream_drain(S);
}

// -------------------------------------------------------------- f32 experts
// fmt 0 weights, y[row, o] = sum_k x[row, k] * w[o, k]: one warp per output,
// lanes stride K, shuffle-tree sum.  ABI-completeness path for experts the
// caller uploaded dequantised; not order-exact with the CPU's sequential sum.
struct F32Slot {
    const float *w_a;  // [O, K]
    const float *w_b;  // second matrix for mode 0 (up)
    int row0, nrows;
};
__global__ void __launch_bounds__(256) gemv_f32_kernel(const F32Slot *__restrict__ slots, int n_slots, int mode, int O,
                                                       int K, const float *__restrict__ x, long long ldx,
                                                       float *__restrict__ out, long long ldo, int max_rows) {
    const int slot = blockIdx.z;
    if (slot >= n_slots) return;
    const F32Slot s = slots[slot];
    const int row = blockIdx.y;
    if (row >= s.nrows) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int o = blockIdx.x * 8 + warp;
    if (o >= O) return;
    const float *xr = x + (long long)(s.row0 + row) * ldx;
    const float *wa = s.w_a + (long long)o * K;
    float a = 0.0f, b = 0.0f;
    for (int k = lane; k < K; k += 32) a += xr[k] * wa[k];
    if (mode == 0) {
        const float *wb = s.w_b + (long long)o * K;
        for (int k = lane; k < K; k += 32) b += xr[k] * wb[k];
    }
    for (int d = 16; d > 0; d >>= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, d);
        b += __shfl_xor_sync(0xffffffffu, b, d);
    }
    if (lane == 0) out[(long long)(s.row0 + row) * ldo + o] = (mode == 0) ? __fmul_rn(silu32(a), b) : a;
    (void)max_rows;
}

// One-entry slot tables written from kernel arguments: the single-matrix entry points describe
// their launch without any host-to-device copy (a copy from a stack variable is pageable memory,
// which a stream capture cannot record).
__global__ void write_slot_kernel(GemvSlot *slot, int *count, const GemvSlot v) {
    if (threadIdx.x == 0) {
        *slot = v;
        *count = 1;
    }
}
__global__ void write_f32_slot_kernel(F32Slot *slot, const F32Slot v) {
    if (threadIdx.x == 0) *slot = v;
}

// ------------------------------------------------------------------- router
// Router logits, crates/peregrine-kernels/src/matmul.rs:18-30: one strictly
// sequential, unfused fp32 chain acc = acc + x[d]*w[e,d] per (token, expert).
// A CTA owns 8 experts x up to 32 tokens; the operands are streamed through
// shared memory in 256-element slices (register prefetch of the next slice
// while the chains run), one thread per chain.
constexpr int kRlDC = 256, kRlEPB = 8, kRlMT = 32, kRlPad = 4;
constexpr int kRlRow = kRlDC + kRlPad;
constexpr int kRlSmemBytes = 2 * (kRlEPB + kRlMT) * kRlRow * 4;

__global__ void __launch_bounds__(256) route_logits_kernel(const float *__restrict__ x, long long ldx,
                                                           const float *__restrict__ rw, int M, int D, int E,
                                                           float *__restrict__ logits) {
    extern __shared__ __align__(16) float rl_smem[];
    const int e0 = blockIdx.x * kRlEPB, s0 = blockIdx.y * kRlMT;
    const int ne = min(kRlEPB, E - e0), ns = min(kRlMT, M - s0);
    const int tid = threadIdx.x;
    const int el = tid & 7, sl = tid >> 3;
    const bool chain = (el < ne) && (sl < ns);
    constexpr int kPre = (kRlEPB + kRlMT) * kRlDC / 256;
    float pre[kPre];
    const int rows = ne + ns;  // rows 0..ne-1 = router rows, ne.. = token rows
    auto load_slice = [&](int d0) {
        const int dlen = min(kRlDC, D - d0);
#pragma unroll
        for (int j = 0; j < kPre; ++j) {
            const int q = tid + j * 256;
            const int r = q / kRlDC, c = q - r * kRlDC;
            float v = 0.0f;
            if (r < rows && c < dlen)
                v = (r < ne) ? rw[(long long)(e0 + r) * D + d0 + c] : x[(long long)(s0 + r - ne) * ldx + d0 + c];
            pre[j] = v;
        }
    };
    auto store_slice = [&](int buf) {
        float *wb = rl_smem + buf * (kRlEPB + kRlMT) * kRlRow;
#pragma unroll
        for (int j = 0; j < kPre; ++j) {
            const int q = tid + j * 256;
            const int r = q / kRlDC, c = q - r * kRlDC;
            if (r < rows) {
                const int dstrow = (r < ne) ? r : (kRlEPB + r - ne);
                wb[dstrow * kRlRow + c] = pre[j];
            }
        }
    };
    float acc = 0.0f;
    load_slice(0);
    int buf = 0;
    for (int d0 = 0; d0 < D; d0 += kRlDC) {
        store_slice(buf);
        __syncthreads();
        if (d0 + kRlDC < D) load_slice(d0 + kRlDC);
        if (chain) {
            const float *wr = rl_smem + buf * (kRlEPB + kRlMT) * kRlRow + el * kRlRow;
            const float *xr = rl_smem + buf * (kRlEPB + kRlMT) * kRlRow + (kRlEPB + sl) * kRlRow;
            const int dlen = min(kRlDC, D - d0);
            int d = 0;
            for (; d + 4 <= dlen; d += 4) {
                const float4 w4 = *reinterpret_cast<const float4 *>(wr + d);
                const float4 x4 = *reinterpret_cast<const float4 *>(xr + d);
                acc = __fadd_rn(acc, __fmul_rn(x4.x, w4.x));
                acc = __fadd_rn(acc, __fmul_rn(x4.y, w4.y));
                acc = __fadd_rn(acc, __fmul_rn(x4.z, w4.z));
                acc = __fadd_rn(acc, __fmul_rn(x4.w, w4.w));
            }
            for (; d < dlen; ++d) acc = __fadd_rn(acc, __fmul_rn(xr[d], wr[d]));
        }
        buf ^= 1;
    }
    if (chain) logits[(long long)(s0 + sl) * E + e0 + el] = acc;
}

// Everything the layer's later kernels need to know about one routing result.
struct RoutePlan {
    int *idx;         // [M*k] selected expert ids            (router.rs Routed.idx)
    float *w;         // [M*k] gate weights after norm/scale  (Routed.w)
    int *keff;        // [M]   experts kept per token         (Routed.keff)
    int *n_slots;     // [1]   active expert slots incl. shared
    int *n_pairs;     // [1]   (token, expert) pairs incl. shared
    int *n_union;     // [1]   distinct routed experts
    int *union_ids;   // [E]   expert id of routed slot p (batch-union order)
    int *pair_token;  // [P]   token of pair p (the GEMV rowmap for gate/up)
    int *tok_pair;    // [M*k] pair index of (s, kk)
    int *comb_pair;   // [M*k] pair rows of token s in batch-union order (keff[s] entries)
    float *comb_w;    // [M*k] gate weights in the same order
    int *shared_pair0;  // [1] first pair of the shared expert (pairs s.. in token order), -1 if none
    GemvSlot *gu_slots;  // [E+1]
    GemvSlot *dn_slots;  // [E+1]
    // per-step scratch the plan clears for the launches that follow it
    int *col_done;      // [n_col] column-tile arrival counters of the down launch
    int n_col;
    unsigned *amax;     // [n_amax] row maxima of |h| filled by the gate/up launch
    int n_amax;
    // expert-parallel ownership: this device computes routed experts [ep_lo, ep_hi) and the
    // shared expert for tokens [home_lo, home_lo + home_n); other slots are planned with 0 rows
    int ep_lo, ep_hi, home_lo, home_n;
};

// Per-expert device pointers, indexed by expert id; entry E is the shared expert.
struct ExpertDev {
    const uint8_t *gate, *up, *down;
    const float *gate_rs, *up_rs, *down_rs;
};

constexpr int kPlanCacheTokens = 64;  // routing of up to this many tokens is kept in shared memory
__host__ __device__ inline size_t route_plan_smem_bytes(int E, int nwarp, int k) {
    // sig/choice per warp, first_seen, cnt, slot_of, row0 (E+2), base, mask (8E), union (E), nunion,
    // cached idx / w / keff
    return (size_t)(2 * nwarp * E + 13 * E + 8 + E) * 4 + (size_t)kPlanCacheTokens * (2 * k + 1) * 4 + 64;
}

// Top-k selection, batch union and the pair layout, executed by one CTA.
//   selection: crates/peregrine-model/src/router.rs:86-150 (sigmoid scores, bias
//     only for choosing, strict '>' from -inf so ties go to the lowest index and
//     NaN / -inf scores are never chosen, norm over all k slots + 1e-20, scale)
//   union order: router.rs:420-430 (first seen, s ascending then kk ascending)
//   rows of an expert: ascending s (crates/peregrine-model/src/mlp.rs:83-95)
// Pairs are laid out expert by expert in union order, the shared expert last.
// Routing of the first kPlanCacheTokens tokens is mirrored in shared memory so a
// decode-sized batch never waits on its own global writes.
__device__ __forceinline__ void route_plan_body(const float *__restrict__ logits, const float *__restrict__ bias,
                                                int M, int E, int k, int norm_topk, float routed_scale,
                                                int has_shared, const ExpertDev *__restrict__ experts,
                                                const RoutePlan &plan, unsigned char *rp_smem,
                                                bool preselected = false) {
    const int nwarp = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float *sig_all = reinterpret_cast<float *>(rp_smem);
    float *choice_all = sig_all + nwarp * E;
    int *first_seen = reinterpret_cast<int *>(choice_all + nwarp * E);
    int *cnt = first_seen + E;
    int *slot_of = cnt + E;
    int *row0 = slot_of + E;  // E + 2 entries
    int *base = row0 + E + 2;
    unsigned *mask = reinterpret_cast<unsigned *>(base + E);  // E * 8 words: 256 tokens per sweep
    int *union_s = reinterpret_cast<int *>(mask + E * 8);     // E
    int *s_nunion = union_s + E;                              // 1 (+7 pad)
    int *idx_c = s_nunion + 8;                                // kPlanCacheTokens * k
    float *w_c = reinterpret_cast<float *>(idx_c + kPlanCacheTokens * k);
    int *keff_c = reinterpret_cast<int *>(w_c + kPlanCacheTokens * k);
    const bool cached = M <= kPlanCacheTokens && !preselected;
    auto ld_idx = [&](int q) { return cached ? idx_c[q] : plan.idx[q]; };
    auto ld_w = [&](int q) { return cached ? w_c[q] : plan.w[q]; };
    auto ld_keff = [&](int s) { return cached ? keff_c[s] : plan.keff[s]; };

    // clear the per-step scratch of the launches that follow
    for (int i = threadIdx.x; i < plan.n_col; i += blockDim.x) plan.col_done[i] = 0;
    for (int i = threadIdx.x; i < plan.n_amax; i += blockDim.x) plan.amax[i] = 0u;

    // ---- 1. per-token selection.  Tokens are taken nwarp at a time: all threads evaluate the
    // sigmoids of the group (the fp64 exponential is the expensive part), then warp w selects
    // for token g0 + w.  A score is turned into an order-preserving 32-bit key (0 = not
    // selectable: NaN or -inf, which strict '>' from -inf never picks) so that a round is one
    // warp-wide integer max plus one integer min for the lowest index among equals.
    // (preselected: route_select_kernel already wrote idx / w / keff of every token; only for
    // batches too large for the shared-memory mirror)
    for (int g0 = 0; g0 < (preselected ? 0 : M); g0 += nwarp) {
        const int ng = min(nwarp, M - g0);
        for (int i = threadIdx.x; i < ng * E; i += blockDim.x) {
            const int sl = i / E, e = i - sl * E;
            const float sg = sigmoid32(__ldcg(logits + (long long)(g0 + sl) * E + e));
            sig_all[sl * E + e] = sg;
            choice_all[sl * E + e] = __fadd_rn(sg, bias[e]);
        }
        __syncthreads();
        if (warp < ng) {
            const int s = g0 + warp;
            float *sig = sig_all + warp * E;
            unsigned *key = reinterpret_cast<unsigned *>(choice_all + warp * E);
            for (int e = lane; e < E; e += 32) {
                const float c = choice_all[warp * E + e];
                unsigned u = 0u;
                if (c > -INFINITY) {  // false for NaN and -inf
                    u = __float_as_uint(c == 0.0f ? 0.0f : c);
                    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
                }
                key[e] = u;
            }
            __syncwarp();
            int kept = k;
            int my_idx = 0;      // lane kk keeps the kk-th selection (k <= 32)
            float my_w = 0.0f;
            for (int kk = 0; kk < k; ++kk) {
                unsigned bu = 0u;
                int bi = 0x7fffffff;
                for (int e = lane; e < E; e += 32) {
                    const unsigned u = key[e];
                    if (u > bu) {  // ascending e within a lane: the first maximum keeps the lowest index
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
                if (lane == 0) key[best] = 0u;  // never chosen again
                __syncwarp();
            }
            // slots >= kept hold expert 0 with weight 0 (the initial values)
            if (norm_topk) {
                float sm = 0.0f;
                for (int j = 0; j < k; ++j) sm = __fadd_rn(sm, __shfl_sync(0xffffffffu, my_w, j));
                sm = __fadd_rn(sm, 1e-20f);
                my_w = __fdiv_rn(my_w, sm);
            }
            my_w = __fmul_rn(my_w, routed_scale);
            if (lane < k) {
                plan.idx[s * k + lane] = my_idx;
                plan.w[s * k + lane] = my_w;
                if (cached) {
                    idx_c[s * k + lane] = my_idx;
                    w_c[s * k + lane] = my_w;
                }
            }
            if (lane == 0) {
                plan.keff[s] = kept;
                if (cached) keff_c[s] = kept;
            }
        }
        __syncthreads();
    }
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        first_seen[e] = 0x7fffffff;
        cnt[e] = 0;
        base[e] = 0;
    }
    if (threadIdx.x == 0) *s_nunion = 0;
    __syncthreads();

    // ---- 2. first-seen key and row count per expert
    for (int q = threadIdx.x; q < M * k; q += blockDim.x) {
        const int s = q / k, kk = q - s * k;
        if (kk < ld_keff(s)) {
            const int e = ld_idx(q);
            atomicMin(&first_seen[e], q);
            atomicAdd(&cnt[e], 1);
        }
    }
    __syncthreads();

    // ---- 3. union position of each routed expert = rank of its first-seen key
    if (M * k <= (int)blockDim.x) {
        // one thread per selection: the selection that first names an expert owns it, and its
        // rank among such selections (ballot prefix) is the expert's union position
        for (int e = threadIdx.x; e < E; e += blockDim.x) slot_of[e] = -1;
        const int q = threadIdx.x;
        int e_mine = -1;
        bool owner = false;
        if (q < M * k) {
            const int s = q / k, kk = q - s * k;
            if (kk < ld_keff(s)) {
                e_mine = ld_idx(q);
                owner = first_seen[e_mine] == q;
            }
        }
        const unsigned bal = __ballot_sync(0xffffffffu, owner);
        unsigned *wcount = mask;  // scratch: owners per warp
        if (lane == 0) wcount[warp] = __popc(bal);
        __syncthreads();
        int before = 0;
        for (int w2 = 0; w2 < warp; ++w2) before += (int)wcount[w2];
        if (owner) {
            const int pos = before + __popc(bal & ((1u << lane) - 1u));
            union_s[pos] = e_mine;
            plan.union_ids[pos] = e_mine;
            slot_of[e_mine] = pos;
        }
        if (threadIdx.x == 0) {
            int tot = 0;
            for (int w2 = 0; w2 < nwarp; ++w2) tot += (int)wcount[w2];
            *s_nunion = tot;
        }
    } else {
        for (int e = threadIdx.x; e < E; e += blockDim.x) {
            int pos = -1;
            if (cnt[e] > 0) {
                pos = 0;
                const int key = first_seen[e];
                for (int o = 0; o < E; ++o) pos += (first_seen[o] < key) ? 1 : 0;
                union_s[pos] = e;
                plan.union_ids[pos] = e;
                atomicAdd(s_nunion, 1);
            }
            slot_of[e] = pos;
        }
    }
    __syncthreads();
    const int nunion = *s_nunion;
    // ---- 4. first pair row of each slot (serial scan; at most E entries, all in shared memory)
    if (threadIdx.x == 0) {
        int run = 0;
        for (int p = 0; p < nunion; ++p) {
            row0[p] = run;
            run += cnt[union_s[p]];
        }
        row0[nunion] = run;  // routed pairs
        *plan.n_union = nunion;
        *plan.n_slots = nunion + (has_shared ? 1 : 0);
        *plan.n_pairs = run + (has_shared ? M : 0);
        *plan.shared_pair0 = has_shared ? run : -1;
    }
    __syncthreads();
    const int routed_pairs = row0[nunion];

    // ---- 5. pair rows: expert-major, ascending token inside an expert.
    // Tokens are swept 256 at a time; a per-expert bitmask over the sweep gives
    // each (token, expert) its rank among the sweep's tokens of that expert.
    for (int sweep0 = 0; sweep0 < M; sweep0 += 256) {
        for (int i = threadIdx.x; i < E * 8; i += blockDim.x) mask[i] = 0u;
        __syncthreads();
        const int s = sweep0 + threadIdx.x;
        const int ke = (s < M && threadIdx.x < 256) ? ld_keff(s) : 0;
        for (int kk = 0; kk < ke; ++kk) {
            const int e = ld_idx(s * k + kk);
            atomicOr(&mask[e * 8 + (threadIdx.x >> 5)], 1u << (threadIdx.x & 31));
        }
        __syncthreads();
        for (int kk = 0; kk < ke; ++kk) {
            const int e = ld_idx(s * k + kk);
            int rank = 0;
            const int wi = threadIdx.x >> 5;
            for (int w2 = 0; w2 < wi; ++w2) rank += __popc(mask[e * 8 + w2]);
            rank += __popc(mask[e * 8 + wi] & ((1u << (threadIdx.x & 31)) - 1u));
            const int p = row0[slot_of[e]] + base[e] + rank;
            plan.pair_token[p] = s;
            plan.tok_pair[s * k + kk] = p;
            // combine order of token s: its selections sorted by union position
            const int key = slot_of[e];
            int pos = 0;
            for (int j2 = 0; j2 < ke; ++j2) {
                const int key2 = slot_of[ld_idx(s * k + j2)];
                pos += (key2 < key || (key2 == key && j2 < kk)) ? 1 : 0;
            }
            plan.comb_pair[s * k + pos] = p;
            plan.comb_w[s * k + pos] = ld_w(s * k + kk);
        }
        __syncthreads();
        for (int e = threadIdx.x; e < E; e += blockDim.x) {
            int add = 0;
            for (int w2 = 0; w2 < 8; ++w2) add += __popc(mask[e * 8 + w2]);
            base[e] += add;
        }
        __syncthreads();
    }
    // shared expert rows: every token, in token order
    if (has_shared)
        for (int s = threadIdx.x; s < M; s += blockDim.x) plan.pair_token[routed_pairs + s] = s;

    // ---- 6. GEMV slot tables
    for (int p = threadIdx.x; p < nunion + (has_shared ? 1 : 0); p += blockDim.x) {
        const bool sh = p >= nunion;
        const ExpertDev ex = experts[sh ? E : union_s[p]];
        GemvSlot g, d;
        g.a = ex.gate;
        g.b = ex.up;
        g.a_rs = ex.gate_rs;
        g.b_rs = ex.up_rs;
        const int e_id = sh ? E : union_s[p];
        const bool owned = sh || (e_id >= plan.ep_lo && e_id < plan.ep_hi);
        g.row0 = sh ? routed_pairs + plan.home_lo : row0[p];
        g.nrows = sh ? plan.home_n : (owned ? cnt[e_id] : 0);
        d = g;
        d.a = ex.down;
        d.b = nullptr;
        d.a_rs = ex.down_rs;
        d.b_rs = nullptr;
        plan.gu_slots[p] = g;
        plan.dn_slots[p] = d;
    }
}

__global__ void __launch_bounds__(256) route_plan_kernel(const float *__restrict__ logits,
                                                         const float *__restrict__ bias, int M, int E, int k,
                                                         int norm_topk, float routed_scale, int has_shared,
                                                         const ExpertDev *__restrict__ experts, RoutePlan plan,
                                                         int preselected) {
    extern __shared__ __align__(16) unsigned char rp_smem[];
    route_plan_body(logits, bias, M, E, k, norm_topk, routed_scale, has_shared, experts, plan, rp_smem,
                    preselected != 0);
}

// Per-token selection for large batches: one warp per token, any number of CTAs.  Same rules and
// the same arithmetic as step 1 of route_plan_body (crates/peregrine-model/src/router.rs:86-150).
__global__ void __launch_bounds__(256) route_select_kernel(const float *__restrict__ logits,
                                                           const float *__restrict__ bias, int M, int E, int k,
                                                           int norm_topk, float routed_scale, RoutePlan plan) {
    extern __shared__ __align__(16) unsigned char rs_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    const int s = blockIdx.x * nwarp + warp;
    if (s >= M) return;
    float *sig = reinterpret_cast<float *>(rs_smem) + warp * 2 * E;
    unsigned *key = reinterpret_cast<unsigned *>(sig + E);
    for (int e = lane; e < E; e += 32) {
        const float sg = sigmoid32(__ldcg(logits + (long long)s * E + e));
        sig[e] = sg;
        const float c = __fadd_rn(sg, bias[e]);
        unsigned u = 0u;
        if (c > -INFINITY) {  // false for NaN and -inf
            u = __float_as_uint(c == 0.0f ? 0.0f : c);
            u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
        }
        key[e] = u;
    }
    __syncwarp();
    int kept = k, my_idx = 0;
    float my_w = 0.0f;
    for (int kk = 0; kk < k; ++kk) {
        unsigned bu = 0u;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
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
    if (norm_topk) {
        float sm = 0.0f;
        for (int j = 0; j < k; ++j) sm = __fadd_rn(sm, __shfl_sync(0xffffffffu, my_w, j));
        sm = __fadd_rn(sm, 1e-20f);
        my_w = __fdiv_rn(my_w, sm);
    }
    my_w = __fmul_rn(my_w, routed_scale);
    if (lane < k) {
        plan.idx[s * k + lane] = my_idx;
        plan.w[s * k + lane] = my_w;
    }
    if (lane == 0) plan.keff[s] = kept;
}

// ------------------------------------------------- fused routing kernel
// One launch does everything the layer needs before the experts run:
//   chain CTAs (one per 8 experts x up to 32 tokens): the router logits of
//     crates/peregrine-kernels/src/matmul.rs:18-30 — one strictly sequential,
//     unfused fp32 chain acc = acc + x[d]*w[e,d] per (token, expert), one thread
//     per chain — with the operands streamed through a four-stage shared-memory
//     ring by bulk copies issued from a producer warp;
//   quantiser CTAs (one per token): the int8 copy of x for the gate/up launch;
//   the chain CTA that finishes last runs route_plan_body.
constexpr int kRtEPB = 8, kRtMT = 32, kRtMaxStages = 16;
constexpr int kRtThreads = 288;  // 9 warps
constexpr int kRtRingBytes = 160 * 1024;   // the ring uses as many stages as fit here (at most 16)
constexpr int kRtBarOffset = kRtRingBytes; // barriers and flags follow the ring
// slice length along D: long slices for a single token (fewer hand-overs on the critical chain)
// tokens per chain CTA: 16 up to 32 tokens (one chain per thread, 128 chain threads: one warp per
// scheduler, so nothing competes with a chain for its issue slots: a chain is a string of dependent
// adds, and two chain warps on one scheduler took more than twice as long as one), above that 64
// (two independent chains per thread)
__host__ __device__ inline int route_tokens_per_cta(int M) { return M > kRtMT ? 2 * kRtMT : kRtMT / 2; }
__host__ __device__ inline int route_slice(int M) { return M == 1 ? 512 : 256; }
// floats per operand row inside a stage: 16-byte skew so the 8 router rows land on distinct banks
__host__ __device__ inline int route_row_floats(int M) { return route_slice(M) + 4; }
__host__ __device__ inline int route_stage_bytes(int M) {
    return (kRtEPB + (M < route_tokens_per_cta(M) ? M : route_tokens_per_cta(M))) * route_row_floats(M) * 4;
}
__host__ __device__ inline int route_stages(int M) {
    const int n = kRtRingBytes / route_stage_bytes(M);
    return n > kRtMaxStages ? kRtMaxStages : n;
}

struct RouteArgs {
    const float *x;
    long long ldx;
    const float *rw, *bias;
    int M, D, E, k, norm_topk;
    float routed_scale;
    int has_shared;
    float *logits;
    unsigned *done_counter;  // zero before the first launch; the last CTA resets it
    const ExpertDev *experts;
    RoutePlan plan;
    int n_chain_ctas;
    // quantiser role
    int8_t *xq;
    float *sx;
    int *xcs;
    int kp, nblk;
    int *err;
    // Operands re-laid for batches: rwt[e-block][slice][8][260] and xt[slice][M][260] (rows of 256
    // floats + 4 of padding, route_tile_rows_kernel), so a slice's 8 router rows and a CTA's token
    // rows are one bulk copy each instead of one per row; nullptr: copy row by row
    const float *rwt, *xt;
    int small_plan;   // route_fused_kernel: at most kSpecTokens tokens on one device: route_plan_small<true>
    int no_plan;      // route_fused_kernel: logits and quantised rows only (large batches plan separately)
    float spec_sign;  // route_spec_kernel: -1 turns the speculative pick upside down (repair-path self-test)
};

// Plan for at most kSpecTokens tokens on one device, two uses:
//   EXACT = false: plan of a speculative selection.  Only what the gate/up launch reads is produced
//     (selection ids, pair rows, gate/up slots, cleared scratch), with the numbering rules of
//     route_plan_body, so that an agreeing exact plan describes the same rows.  Scores use the fast
//     fp32 exponential: a guess does not need more.
//   EXACT = true: the complete plan with the arithmetic of route_plan_body step 1
//     (crates/peregrine-model/src/router.rs:86-150) and the same layout rules, written for one or
//     two tokens so that no phase is longer than a warp's worth of work: it runs at the end of the
//     exact chains, which the down launch of a decode step waits for.
constexpr int kSpecTokens = 2;
template <bool EXACT>
__device__ __forceinline__ void route_plan_small(const float *__restrict__ logits, const float *__restrict__ bias,
                                                 int M, int E, int k, int norm_topk, float routed_scale,
                                                 int has_shared, const ExpertDev *__restrict__ experts,
                                                 const RoutePlan &plan, unsigned char *rp_smem) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned *key_all = reinterpret_cast<unsigned *>(rp_smem);        // [kSpecTokens][E]
    int *idx_s = reinterpret_cast<int *>(key_all + kSpecTokens * E);  // [kSpecTokens][32]
    int *keff_s = idx_s + kSpecTokens * 32;                           // [kSpecTokens]
    float *w_s = reinterpret_cast<float *>(keff_s + kSpecTokens);     // [kSpecTokens][32]
    float *sig_all = w_s + kSpecTokens * 32;                          // [kSpecTokens][E] (EXACT)
    for (int i = threadIdx.x; i < plan.n_col; i += blockDim.x) plan.col_done[i] = 0;
    for (int i = threadIdx.x; i < plan.n_amax; i += blockDim.x) plan.amax[i] = 0u;
    if (warp < M) {
        const int s = warp;
        unsigned *key = key_all + s * E;
        float *sig = sig_all + s * E;
        // scores: eight experts per lane and round trip to memory
        for (int e0 = 0; e0 < E; e0 += 256) {
            float lg[8], bs[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int e = e0 + u * 32 + lane;
                lg[u] = e < E ? __ldcg(logits + (long long)s * E + e) : 0.0f;
                bs[u] = e < E ? __ldg(bias + e) : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int e = e0 + u * 32 + lane;
                float c;
                if (EXACT) {
                    const float sg = sigmoid32(lg[u]);
                    if (e < E) sig[e] = sg;
                    c = __fadd_rn(sg, bs[u]);
                } else {
                    c = __fdividef(1.0f, 1.0f + __expf(-lg[u])) + bs[u];
                }
                unsigned q = 0u;
                if (c > -INFINITY) {  // false for NaN and -inf: never selectable
                    q = __float_as_uint(c == 0.0f ? 0.0f : c);
                    q = (q & 0x80000000u) ? ~q : (q | 0x80000000u);
                }
                if (e < E) key[e] = q;
            }
        }
        __syncwarp();
        int kept = k;
        int my_idx = 0;
        float my_w = 0.0f;
        for (int kk = 0; kk < k; ++kk) {
            unsigned bu = 0u;
            int bi = 0x7fffffff;
            for (int e = lane; e < E; e += 32) {
                const unsigned u = key[e];
                if (u > bu) {  // ascending e within a lane: the first maximum keeps the lowest index
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
                if (EXACT) my_w = sig[best];
            }
            if (lane == 0) key[best] = 0u;
            __syncwarp();
        }
        if (EXACT) {
            // slots >= kept hold expert 0 with weight 0 (the initial values)
            if (norm_topk) {
                float sm = 0.0f;
                for (int j = 0; j < k; ++j) sm = __fadd_rn(sm, __shfl_sync(0xffffffffu, my_w, j));
                sm = __fadd_rn(sm, 1e-20f);
                my_w = __fdiv_rn(my_w, sm);
            }
            my_w = __fmul_rn(my_w, routed_scale);
        }
        idx_s[s * 32 + lane] = my_idx;
        w_s[s * 32 + lane] = my_w;
        if (lane < k) {
            plan.idx[s * k + lane] = my_idx;
            if (EXACT) plan.w[s * k + lane] = my_w;
        }
        if (lane == 0) {
            keff_s[s] = kept;
            plan.keff[s] = kept;
        }
    }
    __syncthreads();
    if (warp == 0) {
        // Union and pair rows for one or two tokens, lane kk = selection kk.  Token 0's picks are
        // union slots 0..keff0-1 in order; a pick of token 1 either repeats one of them (its row
        // follows token 0's row of that expert) or opens a new slot in kk order.
        const int keff0 = keff_s[0], keff1 = M > 1 ? keff_s[1] : 0;
        const int e0 = lane < keff0 ? idx_s[lane] : -1;
        const int e1 = lane < keff1 ? idx_s[32 + lane] : -2;
        // the expert-table entries are fetched now; they are needed after the scans below
        ExpertDev ex0 = {}, ex1 = {}, exs = {};
        if (e0 >= 0) ex0 = experts[e0];
        if (e1 >= 0) ex1 = experts[e1];
        if (has_shared && lane == 0) exs = experts[E];
        int dup_of = -1;           // slot of token 0 that my token-1 pick repeats
        bool shared_by_1 = false;  // my token-0 pick is repeated by token 1
        for (int j = 0; j < (M > 1 ? k : 0); ++j) {
            const int o0 = __shfl_sync(0xffffffffu, e0, j), o1 = __shfl_sync(0xffffffffu, e1, j);
            if (e1 >= 0 && o0 == e1) dup_of = j;
            if (e0 >= 0 && o1 == e0) shared_by_1 = true;
        }
        // rows of the first group: 1 or 2 per slot; exclusive scan over lanes
        const int c0 = e0 >= 0 ? (shared_by_1 ? 2 : 1) : 0;
        int inc = c0;
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += v;
        }
        const int row_a = inc - c0;
        const int total_a = __shfl_sync(0xffffffffu, inc, 31);
        const bool fresh = e1 >= 0 && dup_of < 0;
        const unsigned fb = __ballot_sync(0xffffffffu, fresh);
        const int rank_b = __popc(fb & ((1u << lane) - 1u));
        const int nfresh = __popc(fb);
        const int nun = keff0 + nfresh, run = total_a + nfresh;
        const int row_dup = __shfl_sync(0xffffffffu, row_a, dup_of < 0 ? 0 : dup_of);
        auto slot_of = [&](const ExpertDev &ex, int r0, int n, int p) {
            GemvSlot g;
            g.a = ex.gate;
            g.b = ex.up;
            g.a_rs = ex.gate_rs;
            g.b_rs = ex.up_rs;
            g.row0 = r0;
            g.nrows = n;
            plan.gu_slots[p] = g;
            if (EXACT) {
                g.a = ex.down;
                g.b = nullptr;
                g.a_rs = ex.down_rs;
                g.b_rs = nullptr;
                plan.dn_slots[p] = g;
            }
        };
        if (e0 >= 0) {
            plan.pair_token[row_a] = 0;
            slot_of(ex0, row_a, c0, lane);
            if (EXACT) {
                plan.union_ids[lane] = e0;
                plan.tok_pair[lane] = row_a;
                plan.comb_pair[lane] = row_a;  // a single token's union order is its selection order
                plan.comb_w[lane] = w_s[lane];
            }
        }
        // token 1: union position and pair row of my pick
        const int slot1 = e1 >= 0 ? (fresh ? keff0 + rank_b : dup_of) : 0x7fffffff;
        const int row1 = fresh ? total_a + rank_b : row_dup + 1;
        if (e1 >= 0) {
            plan.pair_token[row1] = 1;
            if (fresh) slot_of(ex1, row1, 1, keff0 + rank_b);
        }
        if (EXACT && M > 1) {
            // combine order of token 1: its picks by ascending union position
            int pos = 0;
            for (int j = 0; j < k; ++j) {
                const int other = __shfl_sync(0xffffffffu, slot1, j);
                pos += (other < slot1) ? 1 : 0;
            }
            if (e1 >= 0) {
                if (fresh) plan.union_ids[keff0 + rank_b] = e1;
                plan.tok_pair[k + lane] = row1;
                plan.comb_pair[k + pos] = row1;
                plan.comb_w[k + pos] = w_s[32 + lane];
            }
        }
        if (has_shared && lane < M) plan.pair_token[run + lane] = lane;
        if (has_shared && lane == 0) slot_of(exs, run, M, nun);
        if (lane == 0) {
            *plan.n_union = nun;
            *plan.n_slots = nun + (has_shared ? 1 : 0);
            *plan.n_pairs = run + (has_shared ? M : 0);
            *plan.shared_pair0 = has_shared ? run : -1;
        }
    }
}

// Slice-major copy of fp32 rows for the batch router: dst[((r / G) * nslice + slice) * G + r % G][260]
// holds src[r][slice * 256 ..] (zero past D and for rows past `rows`); 4 floats of padding per
// row keep the 8 router rows of a stage on distinct shared-memory banks.  grid = (rows_padded, nslice).
__global__ void __launch_bounds__(64) route_tile_rows_kernel(const float *__restrict__ src, long long ld, int rows,
                                                             int D, int G, float *__restrict__ dst) {
    const int r = blockIdx.x, slice = blockIdx.y, nslice = gridDim.y;
    float *out = dst + (((long long)(r / G) * nslice + slice) * G + (r % G)) * 260;
    for (int j = threadIdx.x; j < 260; j += blockDim.x) {
        const int d = slice * 256 + j;
        out[j] = (j < 256 && d < D && r < rows) ? src[(long long)r * ld + d] : 0.0f;
    }
}

// Quantiser role of the routing launches (crates/peregrine-kernels/src/quant.rs:14-33): one CTA
// turns token `row` into int8 with its scale and the -8*sum correction of every 32-block.
__device__ __forceinline__ void route_quantise_row(const RouteArgs &A, int row, unsigned char *rt_smem) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const float *xr = A.x + (long long)row * A.ldx;
    float *red = reinterpret_cast<float *>(rt_smem);
    const int n4 = A.D >> 2;
    if (A.kp == A.D && (A.D & 31) == 0 && n4 <= 8 * (int)blockDim.x && (blockDim.x & 7) == 0 &&
        ((reinterpret_cast<uintptr_t>(xr) | reinterpret_cast<uintptr_t>(A.xq)) & 15) == 0) {
        // the whole row in registers: one round trip to memory, then maximum, scale and rounding
        // from the registers.  Eight neighbouring lanes hold one 32-element block.
        const float4 *x4 = reinterpret_cast<const float4 *>(xr);
        float4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = tid + u * (int)blockDim.x;
            v[u] = i < n4 ? __ldg(x4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float amax = 0.0f;
#pragma unroll
        for (int u = 0; u < 8; ++u)
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[u].x), fabsf(v[u].y)), fmaxf(fabsf(v[u].z), fabsf(v[u].w))));
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if (lane == 0) red[warp] = amax;
        __syncthreads();
        float m = red[0];
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w) m = fmaxf(m, red[w]);
        float s = __fdiv_rn(m, 127.0f);
        if (s < 1e-12f) s = 1e-12f;
        const float inv = __fdiv_rn(1.0f, s);
        if (tid == 0) A.sx[row] = s;
        uint32_t *xq32 = reinterpret_cast<uint32_t *>(A.xq + (long long)row * A.kp);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = tid + u * (int)blockDim.x;
            const int q0 = max(-128, min(127, __float2int_rn(__fmul_rn(v[u].x, inv))));
            const int q1 = max(-128, min(127, __float2int_rn(__fmul_rn(v[u].y, inv))));
            const int q2 = max(-128, min(127, __float2int_rn(__fmul_rn(v[u].z, inv))));
            const int q3 = max(-128, min(127, __float2int_rn(__fmul_rn(v[u].w, inv))));
            if (i < n4)
                xq32[i] = (uint32_t)(q0 & 255) | ((uint32_t)(q1 & 255) << 8) | ((uint32_t)(q2 & 255) << 16) |
                          ((uint32_t)(q3 & 255) << 24);
            int sum = (q0 + q1) + (q2 + q3);
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            sum += __shfl_xor_sync(0xffffffffu, sum, 4);
            if ((lane & 7) == 0 && i < n4) A.xcs[(long long)row * A.nblk + (i >> 3)] = -8 * sum;
        }
        return;
    }
    float amax = 0.0f;
    for (int i = tid; i < A.D; i += blockDim.x) {
        const float a = fabsf(xr[i]);
        if (a > amax) amax = a;
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, amax, o);
        if (other > amax) amax = other;
    }
    if (lane == 0) red[warp] = amax;
    __syncthreads();
    float m = red[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
        if (red[w] > m) m = red[w];
    float s = __fdiv_rn(m, 127.0f);
    if (s < 1e-12f) s = 1e-12f;
    const float inv = __fdiv_rn(1.0f, s);
    if (tid == 0) A.sx[row] = s;
    for (int blk = warp; blk < A.nblk; blk += (int)(blockDim.x >> 5)) {
        const int i = blk * 32 + lane;
        int q = 0;
        if (i < A.D) {
            q = __float2int_rn(__fmul_rn(xr[i], inv));
            q = max(-128, min(127, q));
        }
        A.xq[(long long)row * A.kp + i] = (int8_t)q;
        int sum = q;
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) A.xcs[(long long)row * A.nblk + blk] = -8 * sum;
    }
}

// Chain role of the routing launches, executed by CTA `cta` of A.n_chain_ctas (block size kRtThreads;
// for a single token any larger block works too, the extra warps idle).  Returns true in the one CTA that finished
// last and therefore wrote the plan (never when A.no_plan is set).
// Returns true (for the whole CTA) in the chain CTA that finished last.
__device__ __forceinline__ bool route_chain_role(const RouteArgs &A, unsigned char *rt_smem, int cta) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_eblk = (A.E + kRtEPB - 1) / kRtEPB;
    const int eb = cta % n_eblk, sb = cta / n_eblk;
    const int tpc = route_tokens_per_cta(A.M);
    const int e0 = eb * kRtEPB, s0 = sb * tpc;
    const int ne = min(kRtEPB, A.E - e0), ns = min(tpc, A.M - s0);
    const int kRtStages = route_stages(A.M), kRtStageBytes = route_stage_bytes(A.M);
    const int kRtSL = route_slice(A.M), kRtRowFloats = route_row_floats(A.M);
    const int xrow0 = kRtEPB;  // token rows follow the 8 router rows inside a stage
    const uint32_t full_u32 = smem_u32(rt_smem + kRtBarOffset);
    const uint32_t empty_u32 = full_u32 + kRtMaxStages * 8;
    if (tid == 0) {
        for (int s = 0; s < kRtStages; ++s) {
            mbar_init(full_u32 + s * 8, 1);
            // a stage is released by the warps that run chains: one (decode), those that hold a token of
            // the block (batches up to 32 tokens), all eight (above)
            mbar_init(empty_u32 + s * 8, A.M == 1 ? 1 : (A.M > kRtMT ? 8 : (ns * kRtEPB + 31) / 32));
            mbar_init(empty_u32 + kRtMaxStages * 8 + s * 8, 2);  // products ready: warps 1 and 3
        }
        fence_mbar_init();
        fence_proxy_async();
    }
    __syncthreads();
    const int nslice = (A.D + kRtSL - 1) / kRtSL;
    bool failed = false;
    const int producer_warp = (A.M == 1) ? 2 : 8;
    if (warp == producer_warp) {
        // producer: one bulk copy per operand row and slice (rows 0..ne-1 router, ne.. tokens)
        const int rows = ne + ns;
        for (int i = 0; i < nslice; ++i) {
            const int st = i % kRtStages;
            if (i >= kRtStages) {
                const bool ok = mbar_wait_bounded(empty_u32 + st * 8, ((i / kRtStages) + 1) & 1u);
                if (__any_sync(0xffffffffu, !ok)) {
                    failed = true;
                    break;
                }
            }
            const int d0 = i * kRtSL;
            const int dlen = min(kRtSL, A.D - d0);
            if (A.xt != nullptr && A.M > 1) {
                // two copies per slice: the e-block's 8 padded router rows, the CTA's padded token rows
                if (lane == 0) {
                    fence_proxy_async();
                    mbar_expect_tx(full_u32 + st * 8, (uint32_t)((kRtEPB + ns) * kRtRowFloats * 4));
                    bulk_g2s(smem_u32(rt_smem + st * kRtStageBytes),
                             A.rwt + ((long long)eb * nslice + i) * kRtEPB * kRtRowFloats,
                             (uint32_t)(kRtEPB * kRtRowFloats * 4), full_u32 + st * 8);
                    bulk_g2s(smem_u32(rt_smem + st * kRtStageBytes + xrow0 * kRtRowFloats * 4),
                             A.xt + ((long long)i * A.M + s0) * kRtRowFloats, (uint32_t)(ns * kRtRowFloats * 4),
                             full_u32 + st * 8);
                }
                __syncwarp();
                continue;
            }
            if (A.rwt != nullptr && A.M > 1) {
                // the e-block's 8 padded router rows in one copy, the CTA's token rows one by one straight
                // from x (up to 32 tokens: no re-laid copy of the tokens, one launch less per step)
                if (lane == 0) {
                    fence_proxy_async();
                    mbar_expect_tx(full_u32 + st * 8, (uint32_t)(kRtEPB * kRtRowFloats * 4 + ns * dlen * 4));
                    bulk_g2s(smem_u32(rt_smem + st * kRtStageBytes),
                             A.rwt + ((long long)eb * nslice + i) * kRtEPB * kRtRowFloats,
                             (uint32_t)(kRtEPB * kRtRowFloats * 4), full_u32 + st * 8);
                }
                __syncwarp();
                for (int r = lane; r < ns; r += 32)
                    bulk_g2s(smem_u32(rt_smem + st * kRtStageBytes + (xrow0 + r) * kRtRowFloats * 4),
                             A.x + (long long)(s0 + r) * A.ldx + d0, (uint32_t)(dlen * 4), full_u32 + st * 8);
                continue;
            }
            if (lane == 0) {
                fence_proxy_async();
                mbar_expect_tx(full_u32 + st * 8, (uint32_t)(rows * dlen * 4));
            }
            __syncwarp();
            for (int r = lane; r < rows; r += 32) {
                const float *src = (r < ne) ? A.rw + (long long)(e0 + r) * A.D + d0
                                            : A.x + (long long)(s0 + r - ne) * A.ldx + d0;
                const int dstrow = (r < ne) ? r : (xrow0 + r - ne);
                bulk_g2s(smem_u32(rt_smem + st * kRtStageBytes + dstrow * kRtRowFloats * 4), src,
                         (uint32_t)(dlen * 4), full_u32 + st * 8);
            }
        }
    } else if (A.M == 1) {
        // Decode: 8 chains in lanes 0-7 of warp 0.  Warps 1 and 3 turn each landed slice into products
        // in place (p[e][d] = x[d] * w[e][d], the same single rounding the reference's
        // `acc += xs[d] * wo[d]` applies before its add), so the chain lanes only load and add:
        // the dependent fp32 add latency is then the only thing on the critical path.  Chain,
        // product (1, 3) and producer (2) warps sit on four different schedulers; the other warps
        // wait at the CTA barrier below without issuing, so nothing competes with the chain.
        const uint32_t prod_u32 = empty_u32 + kRtMaxStages * 8;  // [stage] products ready
        if (warp >= 4) {
            // nothing to do until the plan, except warming what the plan will read
            if (warp == 4 && lane < ne) {
                prefetch_l2(A.bias + e0 + lane);
                prefetch_l2(A.experts + e0 + lane);
                if (cta == 0 && lane == 0) prefetch_l2(A.experts + A.E);
            }
        } else if (warp == 1 || warp == 3) {
            for (int i = 0; i < nslice; ++i) {
                const int st = i % kRtStages;
                const bool ok = mbar_wait_bounded(full_u32 + st * 8, (i / kRtStages) & 1u);
                if (__any_sync(0xffffffffu, !ok)) {
                    failed = true;
                    break;
                }
                float *stage = reinterpret_cast<float *>(rt_smem + st * kRtStageBytes);
                const int dlen = min(kRtSL, A.D - i * kRtSL);
                const int n4 = (dlen + 3) >> 2;  // D is a multiple of 4 on this path
                // warps 1 and 3 split the slice; four float4 products per lane and step, loads first
                const int hsel = (warp == 3) ? 1 : 0;
                const int total4 = ne * n4;
                for (int q0 = hsel * 32 + lane; q0 < total4; q0 += 4 * 64) {
                    float4 wq[4], xq4[4];
                    int off[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int q = q0 + u * 64;
                        const int e = (q < total4) ? q / n4 : 0;
                        const int d4 = (q < total4) ? q - e * n4 : 0;
                        off[u] = (q < total4) ? e * kRtRowFloats + 4 * d4 : -1;
                        wq[u] = *reinterpret_cast<const float4 *>(stage + (off[u] < 0 ? 0 : off[u]));
                        xq4[u] = *reinterpret_cast<const float4 *>(stage + xrow0 * kRtRowFloats + 4 * d4);
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        if (off[u] >= 0) {
                            wq[u].x = __fmul_rn(xq4[u].x, wq[u].x);
                            wq[u].y = __fmul_rn(xq4[u].y, wq[u].y);
                            wq[u].z = __fmul_rn(xq4[u].z, wq[u].z);
                            wq[u].w = __fmul_rn(xq4[u].w, wq[u].w);
                            *reinterpret_cast<float4 *>(stage + off[u]) = wq[u];
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(prod_u32 + st * 8);
            }
        } else {
            const int el = lane & 7;
            const bool chain = (lane < 8) && (el < ne);
            float acc = 0.0f;
            for (int i = 0; i < nslice; ++i) {
                const int st = i % kRtStages;
                const bool ok = mbar_wait_bounded(prod_u32 + st * 8, (i / kRtStages) & 1u);
                if (__any_sync(0xffffffffu, !ok)) {
                    failed = true;
                    break;
                }
                if (chain) {
                    const float *pr = reinterpret_cast<const float *>(rt_smem + st * kRtStageBytes) + el * kRtRowFloats;
                    const int dlen = min(kRtSL, A.D - i * kRtSL);
                    if (dlen == kRtSL) {
                        float4 pv[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) pv[j] = *reinterpret_cast<const float4 *>(pr + 4 * j);
#pragma unroll 1
                        for (int d = 0; d < kRtSL; d += 16) {
                            float4 pn[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                // the load past the last step reads the head of the next row of the
                                // stage (router rows are always followed by the token row) and is unused
                                pn[j] = *reinterpret_cast<const float4 *>(pr + d + 16 + 4 * j);
                                acc = __fadd_rn(acc, pv[j].x);
                                acc = __fadd_rn(acc, pv[j].y);
                                acc = __fadd_rn(acc, pv[j].z);
                                acc = __fadd_rn(acc, pv[j].w);
                            }
#pragma unroll
                            for (int j = 0; j < 4; ++j) pv[j] = pn[j];
                        }
                    } else {
                        for (int d = 0; d < dlen; ++d) acc = __fadd_rn(acc, pr[d]);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_u32 + st * 8);
            }
            if (chain && !failed) A.logits[(long long)s0 * A.E + e0 + el] = acc;
        }
    } else if (A.M > kRtMT) {
        // Large batch: thread (el, sl) runs the chains of expert el for tokens sl and sl + 32.  Each
        // chain is still one strictly ordered multiply-then-add sequence; the two are independent.
        const int el = tid & 7, sl = tid >> 3;
        float acc0 = 0.0f, acc1 = 0.0f;
        for (int i = 0; i < nslice; ++i) {
            const int st = i % kRtStages;
            const bool ok = mbar_wait_bounded(full_u32 + st * 8, (i / kRtStages) & 1u);
            if (__any_sync(0xffffffffu, !ok)) {
                failed = true;
                break;
            }
            const float *stage = reinterpret_cast<const float *>(rt_smem + st * kRtStageBytes);
            const float *wr = stage + el * kRtRowFloats;
            const float *x0 = stage + (xrow0 + sl) * kRtRowFloats;
            const float *x1 = x0 + 32 * kRtRowFloats;  // rows past the block's last token: stale, never stored
            const int dlen = min(kRtSL, A.D - i * kRtSL);
            if (dlen == kRtSL) {
#pragma unroll 4
                for (int d = 0; d < kRtSL; d += 4) {
                    const float4 wv = *reinterpret_cast<const float4 *>(wr + d);
                    const float4 a = *reinterpret_cast<const float4 *>(x0 + d);
                    const float4 b = *reinterpret_cast<const float4 *>(x1 + d);
                    acc0 = __fadd_rn(acc0, __fmul_rn(a.x, wv.x));
                    acc1 = __fadd_rn(acc1, __fmul_rn(b.x, wv.x));
                    acc0 = __fadd_rn(acc0, __fmul_rn(a.y, wv.y));
                    acc1 = __fadd_rn(acc1, __fmul_rn(b.y, wv.y));
                    acc0 = __fadd_rn(acc0, __fmul_rn(a.z, wv.z));
                    acc1 = __fadd_rn(acc1, __fmul_rn(b.z, wv.z));
                    acc0 = __fadd_rn(acc0, __fmul_rn(a.w, wv.w));
                    acc1 = __fadd_rn(acc1, __fmul_rn(b.w, wv.w));
                }
            } else {
                for (int d = 0; d < dlen; ++d) {
                    acc0 = __fadd_rn(acc0, __fmul_rn(x0[d], wr[d]));
                    acc1 = __fadd_rn(acc1, __fmul_rn(x1[d], wr[d]));
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_u32 + st * 8);
        }
        if (!failed && el < ne) {
            if (sl < ns) A.logits[(long long)(s0 + sl) * A.E + e0 + el] = acc0;
            if (sl + 32 < ns) A.logits[(long long)(s0 + sl + 32) * A.E + e0 + el] = acc1;
        }
    } else if (warp < (ns * kRtEPB + 31) / 32) {
        const int el = tid & 7, sl = tid >> 3;
        const bool chain = (el < ne) && (sl < ns);
        float acc = 0.0f;
        for (int i = 0; i < nslice; ++i) {
            const int st = i % kRtStages;
            const bool ok = mbar_wait_bounded(full_u32 + st * 8, (i / kRtStages) & 1u);
            if (__any_sync(0xffffffffu, !ok)) {
                failed = true;
                break;
            }
            if (chain) {
                const float *wr = reinterpret_cast<const float *>(rt_smem + st * kRtStageBytes) + el * kRtRowFloats;
                const float *xr =
                    reinterpret_cast<const float *>(rt_smem + st * kRtStageBytes) + (xrow0 + sl) * kRtRowFloats;
                const int dlen = min(kRtSL, A.D - i * kRtSL);
                if (dlen == kRtSL && (kRtSL & 31) == 0) {
                    // Software pipeline over two register sets (a, b), 16 elements each, written out in
                    // source order: while the 16 dependent adds of one set run, the products of the other
                    // are formed and the operands after those are loaded, so the independent work fills
                    // the issue slots the adds leave free and no value is ever copied between registers.
                    float4 wa[4], xa[4], wb[4], xb[4];
                    float pa[16], pb[16];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        wa[j] = *reinterpret_cast<const float4 *>(wr + 4 * j);
                        xa[j] = *reinterpret_cast<const float4 *>(xr + 4 * j);
                        wb[j] = *reinterpret_cast<const float4 *>(wr + 16 + 4 * j);
                        xb[j] = *reinterpret_cast<const float4 *>(xr + 16 + 4 * j);
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        pa[4 * j + 0] = __fmul_rn(xa[j].x, wa[j].x);
                        pa[4 * j + 1] = __fmul_rn(xa[j].y, wa[j].y);
                        pa[4 * j + 2] = __fmul_rn(xa[j].z, wa[j].z);
                        pa[4 * j + 3] = __fmul_rn(xa[j].w, wa[j].w);
                    }
#pragma unroll 1
                    for (int d = 0; d < kRtSL; d += 32) {
                        // loads past the slice stay inside the padded row of this stage or read the next
                        // row of the stage; values past the slice are never added
                        const int l0 = min(d + 32, kRtSL - 16), l1 = min(d + 48, kRtSL - 16);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            acc = __fadd_rn(acc, pa[4 * j + 0]);
                            pb[4 * j + 0] = __fmul_rn(xb[j].x, wb[j].x);
                            acc = __fadd_rn(acc, pa[4 * j + 1]);
                            pb[4 * j + 1] = __fmul_rn(xb[j].y, wb[j].y);
                            acc = __fadd_rn(acc, pa[4 * j + 2]);
                            pb[4 * j + 2] = __fmul_rn(xb[j].z, wb[j].z);
                            acc = __fadd_rn(acc, pa[4 * j + 3]);
                            pb[4 * j + 3] = __fmul_rn(xb[j].w, wb[j].w);
                            wa[j] = *reinterpret_cast<const float4 *>(wr + l0 + 4 * j);
                            xa[j] = *reinterpret_cast<const float4 *>(xr + l0 + 4 * j);
                        }
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            acc = __fadd_rn(acc, pb[4 * j + 0]);
                            pa[4 * j + 0] = __fmul_rn(xa[j].x, wa[j].x);
                            acc = __fadd_rn(acc, pb[4 * j + 1]);
                            pa[4 * j + 1] = __fmul_rn(xa[j].y, wa[j].y);
                            acc = __fadd_rn(acc, pb[4 * j + 2]);
                            pa[4 * j + 2] = __fmul_rn(xa[j].z, wa[j].z);
                            acc = __fadd_rn(acc, pb[4 * j + 3]);
                            pa[4 * j + 3] = __fmul_rn(xa[j].w, wa[j].w);
                            wb[j] = *reinterpret_cast<const float4 *>(wr + l1 + 4 * j);
                            xb[j] = *reinterpret_cast<const float4 *>(xr + l1 + 4 * j);
                        }
                    }
                } else {
                    for (int d = 0; d < dlen; ++d) acc = __fadd_rn(acc, __fmul_rn(xr[d], wr[d]));
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_u32 + st * 8);
        }
        if (chain && !failed) A.logits[(long long)(s0 + sl) * A.E + e0 + el] = acc;
    }
    if (failed && lane == 0) report_error(A.err, kErrBarrierTimeout);
    // ---------------- the last chain CTA to finish plans the layer
    __threadfence();
    __syncthreads();
    int *s_last = reinterpret_cast<int *>(rt_smem + kRtBarOffset + 3 * kRtMaxStages * 8);
    if (tid == 0) {
        const unsigned old = atomicAdd(A.done_counter, 1u);
        *s_last = (old == (unsigned)A.n_chain_ctas - 1u);
        if (*s_last) *A.done_counter = 0u;
    }
    __syncthreads();
    if (!*s_last) return false;
    __threadfence();
    if (A.no_plan) return true;  // the caller goes on from the complete logits
    if (A.small_plan)
        route_plan_small<true>(A.logits, A.bias, A.M, A.E, A.k, A.norm_topk, A.routed_scale, A.has_shared, A.experts,
                               A.plan, rt_smem);
    else
        route_plan_body(A.logits, A.bias, A.M, A.E, A.k, A.norm_topk, A.routed_scale, A.has_shared, A.experts, A.plan,
                        rt_smem);
    return true;
}

__global__ void __launch_bounds__(kRtThreads, 1) route_fused_kernel(const RouteArgs A) {
    extern __shared__ __align__(128) unsigned char rt_smem[];
    if ((int)blockIdx.x >= A.n_chain_ctas) {
        route_quantise_row(A, blockIdx.x - A.n_chain_ctas, rt_smem);
        return;
    }
    route_chain_role(A, rt_smem, blockIdx.x);
}

// Speculative routing launch.  Same outputs as route_fused_kernel (int8 copy of x, logits, plan)
// but the logits are plain parallel dot products, so they can differ from the reference's
// sequential fp32 chain in the last bits.  The layer starts the expert launches from this plan
// while route_fused_kernel computes the exact chains on other SMs; the selections of the two are
// compared afterwards (see GemvParams::spec_a) and the rare disagreement is recomputed.  Only
// the *selection* of this plan is ever used: weights and combine order come from the exact plan.
//   CTAs [0, n_chain_ctas): kSpEPB experts each; the rest: one token each.
constexpr int kSpEPB = 1, kSpWPE = 8, kSpBatch = 6;
__global__ void __launch_bounds__(kRtThreads) route_spec_kernel(const RouteArgs A) {
    extern __shared__ __align__(128) unsigned char rt_smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    griddep_launch_dependents();
    if ((int)blockIdx.x >= A.n_chain_ctas) {
        route_quantise_row(A, blockIdx.x - A.n_chain_ctas, rt_smem);
        return;
    }
    // kSpEPB experts per CTA, kSpWPE warps per expert, each warp one contiguous part of D with all
    // its loads issued before the first use (one memory round trip per kSpBatch float4 per lane)
    __shared__ float s_part[kSpEPB][kSpWPE][kSpecTokens];
    const int el = warp / kSpWPE, part = warp % kSpWPE;
    const int e = blockIdx.x * kSpEPB + el;
    // the planning CTA reads bias and expert-table entries in a dependent chain at the very end of
    // this launch: pull them into L2 now (after an L2-cold start each would be a DRAM round trip)
    if (tid == 0 && e < A.E) {
        prefetch_l2(A.bias + e);
        prefetch_l2(A.experts + e);
        if (blockIdx.x == 0) prefetch_l2(A.experts + A.E);
    }
    if (warp < kSpEPB * kSpWPE && e < A.E) {
        const float4 *wr = reinterpret_cast<const float4 *>(A.rw + (long long)e * A.D);
        const int n4 = A.D >> 2;
        const int per = (n4 + kSpWPE - 1) / kSpWPE;
        const int lo = part * per, hi = min(n4, lo + per);
        float acc[kSpecTokens];
#pragma unroll
        for (int s = 0; s < kSpecTokens; ++s) acc[s] = 0.0f;
        for (int base = lo; base < hi; base += 32 * kSpBatch) {
            float4 wv[kSpBatch], xv[kSpecTokens][kSpBatch];
#pragma unroll
            for (int u = 0; u < kSpBatch; ++u) {
                const int i = base + u * 32 + lane;
                wv[u] = (i < hi) ? __ldg(wr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int s = 0; s < kSpecTokens; ++s)
                    xv[s][u] = (i < hi && s < A.M)
                                   ? __ldg(reinterpret_cast<const float4 *>(A.x + (long long)s * A.ldx) + i)
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < kSpBatch; ++u)
#pragma unroll
                for (int s = 0; s < kSpecTokens; ++s)
                    acc[s] += (xv[s][u].x * wv[u].x + xv[s][u].y * wv[u].y) + (xv[s][u].z * wv[u].z + xv[s][u].w * wv[u].w);
        }
#pragma unroll
        for (int s = 0; s < kSpecTokens; ++s) {
            float sum = acc[s];
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if (lane == 0) s_part[el][part][s] = sum;
        }
    }
    __syncthreads();
    if (tid < kSpEPB * kSpecTokens) {
        const int el2 = tid / kSpecTokens, s = tid % kSpecTokens;
        const int e2 = blockIdx.x * kSpEPB + el2;
        if (e2 < A.E && s < A.M) {
            float sum = 0.0f;
            for (int q = 0; q < kSpWPE; ++q) sum += s_part[el2][q][s];
            A.logits[(long long)s * A.E + e2] = sum * A.spec_sign;
        }
    }
    __threadfence();
    __syncthreads();
    __shared__ int s_last;
    if (tid == 0) {
        const unsigned old = atomicAdd(A.done_counter, 1u);
        s_last = (old == (unsigned)A.n_chain_ctas - 1u);
        if (s_last) *A.done_counter = 0u;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    route_plan_small<false>(A.logits, A.bias, A.M, A.E, A.k, A.norm_topk, A.routed_scale, A.has_shared, A.experts,
                            A.plan, rt_smem);
}

// Routing-weighted combine, crates/peregrine-model/src/mlp.rs:111-127 and
// crates/peregrine-model/src/concurrent.rs:1866-1929: out starts at zero, each
// expert's row is added as out = out + (w * y) in batch-union order, the shared
// expert's row is added last without a weight.
__global__ void __launch_bounds__(256) combine_kernel(const float *__restrict__ y, long long ldy, int D, int k,
                                                      RoutePlan plan, float *__restrict__ out, long long ldo,
                                                      int first_token) {
    // output row blockIdx.y holds token first_token + blockIdx.y
    const int s = first_token + blockIdx.y;
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= D) return;
    const int ke = plan.keff[s];
    float acc = 0.0f;
    for (int j = 0; j < ke; ++j) {
        const int p = plan.comb_pair[s * k + j];
        acc = __fadd_rn(acc, __fmul_rn(plan.comb_w[s * k + j], y[(long long)p * ldy + d]));
    }
    const int sp0 = *plan.shared_pair0;
    if (sp0 >= 0) acc = __fadd_rn(acc, y[(long long)(sp0 + s) * ldy + d]);
    out[(long long)blockIdx.y * ldo + d] = acc;
}

// CSR combine of the host-pointer ABI (out[s] = sum over the row's listed y-rows
// of rw * y, in the listed order, starting from zero).
__global__ void __launch_bounds__(256) csr_reduce_kernel(const float *__restrict__ y, int D,
                                                         const int *__restrict__ row_ptr,
                                                         const int *__restrict__ row_idx, const float *__restrict__ rw,
                                                         float *__restrict__ out) {
    const int s = blockIdx.y;
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= D) return;
    float acc = 0.0f;
    for (int j = row_ptr[s]; j < row_ptr[s + 1]; ++j) {
        const int kx = row_idx[j];
        acc = __fadd_rn(acc, __fmul_rn(rw[kx], y[(long long)kx * D + d]));
    }
    out[(long long)s * D + d] = acc;
}

}  // namespace pgb
