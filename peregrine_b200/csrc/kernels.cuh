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
// Source, destination and size must be multiples of 16 bytes.  No multicast.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
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

// Error codes written to the per-device error word.
enum : int { kErrNone = 0, kErrBarrierTimeout = 1 };

// ------------------------------------------------------- activation quantiser
// crates/peregrine-kernels/src/quant.rs:14-33, one CTA per row.  Besides the
// int8 row (zero padded to `kp`) and its scale it writes, per 32-element block,
// -8 * sum(q): the term that turns the stream's stored nibbles (v+8) back into
// signed weights inside the integer dot.
__global__ void __launch_bounds__(256) qrow_i8_kernel(const float *__restrict__ x, long long ldx, int K, int kp,
                                                      int nblk, int8_t *__restrict__ xq, float *__restrict__ sx,
                                                      int *__restrict__ csum, const int *__restrict__ n_rows_dev,
                                                      int n_rows) {
    const int row = blockIdx.x;
    const int limit = n_rows_dev ? *n_rows_dev : n_rows;
    if (row >= limit) return;
    const float *xr = x + (long long)row * ldx;
    __shared__ float red[8];
    __shared__ float s_inv;
    float amax = 0.0f;
    for (int i = threadIdx.x; i < K; i += blockDim.x) {
        float a = fabsf(xr[i]);
        if (a > amax) amax = a;
    }
    for (int o = 16; o > 0; o >>= 1) {
        float other = __shfl_xor_sync(0xffffffffu, amax, o);
        if (other > amax) amax = other;
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
        xq[(long long)row * kp + i] = (int8_t)q;
        int sum = q;
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) csum[(long long)row * nblk + blk] = -8 * sum;
    }
}

// ------------------------------------------------------------ int4 x int8 GEMV
constexpr int kGemvWarps = 8;
constexpr int kGemvStages = 4;
constexpr int kStageBytes = 2 * kChunkMaxBytes;
constexpr int kRingBytes = kGemvWarps * kGemvStages * kStageBytes;
constexpr int kGemvBarBytes = kGemvWarps * kGemvStages * 8;

// One expert's share of a launch.
struct GemvSlot {
    const uint8_t *a;   // tile stream: gate (mode 0) or down (mode 1)
    const uint8_t *b;   // tile stream: up (mode 0); unused in mode 1
    const float *a_rs;  // per-row scales, padded to ntile*16 (per-row format only)
    const float *b_rs;
    int row0;   // first pair row (output row; activation row unless rowmap is given)
    int nrows;  // pair rows of this expert
};

struct GemvParams {
    const GemvSlot *slots;
    const int *n_slots;  // device scalar
    int mode;            // 0: gate/up + SwiGLU -> h ; 1: down -> y
    int ng, bpg, gpc, nchunk, group_bytes, ntile, warp_tiles, O;
    unsigned long long tile_bytes;
    const int8_t *xq;  // activation rows, int8, natural element order
    int xq_stride;     // bytes per activation row (= kp)
    const int *csum;   // -8*sum per 32-block
    int cs_stride;     // ints per activation row (= nblk)
    const float *sx;   // activation row scales
    const int *rowmap; // activation row of pair p (nullptr: p itself)
    int n_xrows;       // activation rows staged in shared memory (XS kernels)
    float *out;
    long long out_stride;
    int *tap;  // optional per-block int32 accumulators [pair][O][ng]
    int *err;
};

struct TileCursor {
    int i, tile, pass, chunk, npass, row0, nrows;
    const uint8_t *a, *b;
    const float *a_rs, *b_rs;
};

template <int RMAX>
__device__ __forceinline__ void cursor_seek(TileCursor &c, const GemvParams &P, int total, int stride) {
    // position on the first tile at or after c.i that has rows to compute
    while (c.i < total) {
        const int slot = c.i / P.warp_tiles;
        const int t = c.i - slot * P.warp_tiles;
        const GemvSlot *s = P.slots + slot;
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
__device__ __forceinline__ void cursor_next(TileCursor &c, const GemvParams &P, int total, int stride) {
    if (++c.chunk < P.nchunk) return;
    c.chunk = 0;
    if (++c.pass < c.npass) return;
    c.pass = 0;
    c.i += stride;
    cursor_seek<RMAX>(c, P, total, stride);
}

// Each warp streams two 16-row tiles (lanes 0-15 / 16-31) through a private
// ring of kGemvStages shared-memory stages filled by bulk copies; lane L owns
// one weight row for the whole K extent, so the fp32 fold over groups runs in
// ascending group order exactly as crates/peregrine-kernels/src/idot.rs:98-110
// and matmul.rs:93-106 (grouped) / :75-87 (per-row scale) prescribe.
//   mode 0: half 0 = gate tile t, half 1 = up tile t; epilogue
//           h = silu(g) * u (crates/peregrine-model/src/math.rs:108-118)
//   mode 1: halves = down tiles 2t, 2t+1; epilogue y = acc * sx
// RMAX activation rows are processed per pass over a tile; an expert with more
// rows re-streams its tile (from L2) once per extra pass.
template <int RMAX, bool GROUPED, int BPG, bool XS>
__global__ void __launch_bounds__(kGemvWarps * 32, 1) gemv_w4a8_kernel(const GemvParams P) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = lane >> 4, r16 = lane & 15;
    uint8_t *ring = smem + warp * (kGemvStages * kStageBytes);
    const uint32_t ring_u32 = smem_u32(ring);
    const uint32_t bar_u32 = smem_u32(smem + kRingBytes) + warp * (kGemvStages * 8);
    int8_t *xs = reinterpret_cast<int8_t *>(smem + kRingBytes + kGemvBarBytes);
    const int xs_bytes = (P.n_xrows * P.xq_stride + 15) & ~15;
    int *cs_s = reinterpret_cast<int *>(xs + xs_bytes);

    if (lane == 0) {
        for (int s = 0; s < kGemvStages; ++s) mbar_init(bar_u32 + s * 8, 1);
        fence_mbar_init();
        fence_proxy_async();
    }
    __syncwarp();

    const int bpg = (BPG > 0) ? BPG : P.bpg;
    const int group_bytes = bpg * kSlabBytes + (GROUPED ? kScaleBytes : 0);
    const int half_off = P.gpc * group_bytes;
    const int total = (*P.n_slots) * P.warp_tiles;
    const int stride = gridDim.x * kGemvWarps;

    TileCursor fc, cc;
    fc.i = blockIdx.x + gridDim.x * warp;
    fc.pass = 0;
    fc.chunk = 0;
    cursor_seek<RMAX>(fc, P, total, stride);
    cc = fc;
    uint32_t fq = 0, cq = 0;

    auto issue = [&](const TileCursor &c, uint32_t q) {
        const int g0 = c.chunk * P.gpc;
        const int ngc = min(P.gpc, P.ng - g0);
        const uint32_t bytes = (uint32_t)(ngc * group_bytes);
        const uint32_t stage = q % kGemvStages;
        const uint32_t bar = bar_u32 + stage * 8;
        const uint32_t dst = ring_u32 + stage * kStageBytes;
        const size_t off = (size_t)g0 * group_bytes;
        mbar_expect_tx(bar, c.b ? 2 * bytes : bytes);
        bulk_g2s(dst, c.a + off, bytes, bar);
        if (c.b) bulk_g2s(dst + half_off, c.b + off, bytes, bar);
    };

    // first fill of the ring overlaps the activation staging below
    while (fc.i < total && fq < cq + kGemvStages) {
        if (lane == 0) issue(fc, fq);
        cursor_next<RMAX>(fc, P, total, stride);
        ++fq;
    }

    if (XS) {
        const int n16 = xs_bytes >> 4;
        const uint4 *src = reinterpret_cast<const uint4 *>(P.xq);
        uint4 *dst = reinterpret_cast<uint4 *>(xs);
        for (int i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = src[i];
        const int ncs = P.n_xrows * P.cs_stride;
        for (int i = threadIdx.x; i < ncs; i += blockDim.x) cs_s[i] = P.csum[i];
        __syncthreads();
    }
    const int8_t *xbase = XS ? xs : P.xq;
    const int *csbase = XS ? cs_s : P.csum;

    float acc[RMAX];
    int iacc[RMAX];
    int arow[RMAX];
    bool failed = false;

    while (cc.i < total) {
        // keep the ring full: the stage being refilled was consumed one iteration ago
        while (fc.i < total && fq < cq + kGemvStages) {
            if (lane == 0) {
                fence_proxy_async();
                issue(fc, fq);
            }
            cursor_next<RMAX>(fc, P, total, stride);
            ++fq;
        }
        const uint32_t stage = cq % kGemvStages;
        const uint32_t parity = (cq / kGemvStages) & 1u;
        {
            // bounded wait: give up after ~2e9 cycles, flag the error and leave
            uint32_t done = mbar_try_wait(bar_u32 + stage * 8, parity);
            if (!done) {
                const long long t0 = clock64();
                while (!(done = mbar_try_wait(bar_u32 + stage * 8, parity))) {
                    if (clock64() - t0 > 2000000000LL) break;
                }
            }
            if (__any_sync(0xffffffffu, !done)) {
                if (lane == 0) atomicExch(P.err, kErrBarrierTimeout);
                failed = true;
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
        const int g0 = cc.chunk * P.gpc;
        const int ngc = min(P.gpc, P.ng - g0);
        const uint8_t *sbase = ring + stage * kStageBytes + half * half_off + r16 * 16;
        const int o_half = (P.mode == 0) ? (cc.tile * 16 + r16) : (cc.tile * 32 + lane);
#pragma unroll 2
        for (int gi = 0; gi < ngc; ++gi) {
            const uint8_t *gp = sbase + gi * group_bytes;
            int dsum[RMAX];
#pragma unroll
            for (int r = 0; r < RMAX; ++r) dsum[r] = 0;
#pragma unroll
            for (int b = 0; b < bpg; ++b) {
                const uint4 wv = *reinterpret_cast<const uint4 *>(gp + b * kSlabBytes);
                const int kb = (g0 + gi) * bpg + b;
                const uint32_t l0 = wv.x & 0x0F0F0F0Fu, l1 = wv.y & 0x0F0F0F0Fu, l2 = wv.z & 0x0F0F0F0Fu,
                               l3 = wv.w & 0x0F0F0F0Fu;
                const uint32_t h0 = wv.x & 0xF0F0F0F0u, h1 = wv.y & 0xF0F0F0F0u, h2 = wv.z & 0xF0F0F0F0u,
                               h3 = wv.w & 0xF0F0F0F0u;
#pragma unroll
                for (int r = 0; r < RMAX; ++r) {
                    const int8_t *xr = xbase + (size_t)arow[r] * P.xq_stride + kb * 32;
                    uint4 x0, x1;
                    int lo;
                    if (XS) {
                        x0 = *reinterpret_cast<const uint4 *>(xr);
                        x1 = *reinterpret_cast<const uint4 *>(xr + 16);
                        lo = csbase[arow[r] * P.cs_stride + kb];
                    } else {
                        x0 = __ldg(reinterpret_cast<const uint4 *>(xr));
                        x1 = __ldg(reinterpret_cast<const uint4 *>(xr + 16));
                        lo = __ldg(csbase + (size_t)arow[r] * P.cs_stride + kb);
                    }
                    lo = dp4a_us(l0, x0.x, lo);
                    lo = dp4a_us(l1, x0.y, lo);
                    lo = dp4a_us(l2, x0.z, lo);
                    lo = dp4a_us(l3, x0.w, lo);
                    int hi = dp4a_us(h0, x1.x, 0);
                    hi = dp4a_us(h1, x1.y, hi);
                    hi = dp4a_us(h2, x1.z, hi);
                    hi = dp4a_us(h3, x1.w, hi);
                    dsum[r] += lo + (hi >> 4);  // hi is exactly 16x the upper-half dot
                }
            }
            if (GROUPED) {
                const float sc = *reinterpret_cast<const float *>(gp - r16 * 16 + bpg * kSlabBytes + r16 * 4);
#pragma unroll
                for (int r = 0; r < RMAX; ++r) acc[r] = __fadd_rn(acc[r], __fmul_rn(sc, (float)dsum[r]));
                if (P.tap != nullptr && o_half < P.O && (P.mode == 1 || true)) {
#pragma unroll
                    for (int r = 0; r < RMAX; ++r) {
                        const int ridx = cc.pass * RMAX + r;
                        if (ridx < cc.nrows) {
                            // mode 0 taps gate (half 0) and up (half 1) side by side: [pair][2][O][ng]
                            const long long base =
                                (P.mode == 0) ? ((long long)(cc.row0 + ridx) * 2 + half) * P.O + o_half
                                              : (long long)(cc.row0 + ridx) * P.O + o_half;
                            P.tap[base * P.ng + (g0 + gi)] = dsum[r];
                        }
                    }
                }
            } else {
#pragma unroll
                for (int r = 0; r < RMAX; ++r) iacc[r] += dsum[r];
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
                const float sxa = P.sx[arow[r]];
                float v;
                if (GROUPED) {
                    v = __fmul_rn(acc[r], sxa);
                } else {
                    if (P.tap != nullptr && valid && o_half < P.O) {
                        const long long base = (P.mode == 0) ? ((long long)(cc.row0 + ridx) * 2 + half) * P.O + o_half
                                                             : (long long)(cc.row0 + ridx) * P.O + o_half;
                        P.tap[base] = iacc[r];
                    }
                    v = __fmul_rn(__fmul_rn((float)iacc[r], rs), sxa);
                }
                if (P.mode == 0) {
                    const float u = __shfl_down_sync(0xffffffffu, v, 16);
                    if (valid && half == 0 && o_half < P.O)
                        P.out[(long long)(cc.row0 + ridx) * P.out_stride + o_half] = __fmul_rn(silu32(v), u);
                } else {
                    if (valid && o_half < P.O) P.out[(long long)(cc.row0 + ridx) * P.out_stride + o_half] = v;
                }
            }
        }
        cursor_next<RMAX>(cc, P, total, stride);
        ++cq;
    }
    if (failed) {
        // give copies already in flight a bounded chance to land before the CTA retires
        for (uint32_t q = cq; q < fq; ++q) {
            const uint32_t stage = q % kGemvStages, parity = (q / kGemvStages) & 1u;
            const long long t0 = clock64();
            while (!mbar_try_wait(bar_u32 + stage * 8, parity))
                if (clock64() - t0 > 200000000LL) break;
        }
    }
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
    int *tok_order;   // [M*k] kk values of token s sorted by union position
    int *shared_pair0;  // [1] first pair of the shared expert (pairs s.. in token order), -1 if none
    GemvSlot *gu_slots;  // [E+1]
    GemvSlot *dn_slots;  // [E+1]
};

// Per-expert device pointers, indexed by expert id; entry E is the shared expert.
struct ExpertDev {
    const uint8_t *gate, *up, *down;
    const float *gate_rs, *up_rs, *down_rs;
};

// Top-k selection, batch union and the pair layout, one CTA.
//   selection: crates/peregrine-model/src/router.rs:86-150 (sigmoid scores, bias
//     only for choosing, strict '>' from -inf so ties go to the lowest index and
//     NaN / -inf scores are never chosen, norm over all k slots + 1e-20, scale)
//   union order: router.rs:420-430 (first seen, s ascending then kk ascending)
//   rows of an expert: ascending s (crates/peregrine-model/src/mlp.rs:83-95)
// Pairs are laid out expert by expert in union order, the shared expert last.
__global__ void __launch_bounds__(256) route_plan_kernel(const float *__restrict__ logits,
                                                         const float *__restrict__ bias, int M, int E, int k,
                                                         int norm_topk, float routed_scale, int has_shared,
                                                         const ExpertDev *__restrict__ experts, RoutePlan plan) {
    extern __shared__ __align__(16) unsigned char rp_smem[];
    // layout: per-warp sig[E], choice[E]; then first_seen[E], cnt[E], slot_of[E], row0[E+1], base[E], mask[E*8]
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
    __shared__ int s_nunion;

    // ---- 1. per-token selection, one warp per token
    float *sig = sig_all + warp * E, *choice = choice_all + warp * E;
    for (int s = warp; s < M; s += nwarp) {
        for (int e = lane; e < E; e += 32) {
            const float sg = sigmoid32(logits[(long long)s * E + e]);
            sig[e] = sg;
            choice[e] = __fadd_rn(sg, bias[e]);
        }
        __syncwarp();
        int kept = k;
        for (int kk = 0; kk < k; ++kk) {
            float bv = -INFINITY;
            int best = -1;
            for (int e = lane; e < E; e += 32) {
                const float c = choice[e];
                if (c > bv) {
                    bv = c;
                    best = e;
                }
            }
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, best, o);
                // a valid candidate always has value > -inf; among equals the lower index wins
                if (oi >= 0 && (best < 0 || ov > bv || (ov == bv && oi < best))) {
                    bv = ov;
                    best = oi;
                }
            }
            if (best < 0) {
                kept = kk;
                break;
            }
            if (lane == 0) {
                plan.idx[s * k + kk] = best;
                plan.w[s * k + kk] = sig[best];
                choice[best] = -INFINITY;  // never chosen again
            }
            __syncwarp();
        }
        if (lane == 0) {
            for (int slot = kept; slot < k; ++slot) {
                plan.idx[s * k + slot] = 0;
                plan.w[s * k + slot] = 0.0f;
            }
            plan.keff[s] = kept;
            if (norm_topk) {
                float sm = 0.0f;
                for (int j = 0; j < k; ++j) sm = __fadd_rn(sm, plan.w[s * k + j]);
                sm = __fadd_rn(sm, 1e-20f);
                for (int j = 0; j < k; ++j) plan.w[s * k + j] = __fdiv_rn(plan.w[s * k + j], sm);
            }
            for (int j = 0; j < k; ++j) plan.w[s * k + j] = __fmul_rn(plan.w[s * k + j], routed_scale);
        }
        __syncwarp();
    }
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        first_seen[e] = 0x7fffffff;
        cnt[e] = 0;
        base[e] = 0;
    }
    __syncthreads();

    // ---- 2. first-seen key and row count per expert
    for (int q = threadIdx.x; q < M * k; q += blockDim.x) {
        const int s = q / k, kk = q - s * k;
        if (kk < plan.keff[s]) {
            const int e = plan.idx[q];
            atomicMin(&first_seen[e], q);
            atomicAdd(&cnt[e], 1);
        }
    }
    __syncthreads();

    // ---- 3. union position of each routed expert = rank of its first-seen key
    if (threadIdx.x == 0) s_nunion = 0;
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int pos = -1;
        if (cnt[e] > 0) {
            pos = 0;
            const int key = first_seen[e];
            for (int o = 0; o < E; ++o) pos += (first_seen[o] < key) ? 1 : 0;
            plan.union_ids[pos] = e;
            atomicAdd(&s_nunion, 1);
        }
        slot_of[e] = pos;
    }
    __syncthreads();
    const int nunion = s_nunion;
    // ---- 4. first pair row of each slot (serial scan; at most E entries)
    if (threadIdx.x == 0) {
        int run = 0;
        for (int p = 0; p < nunion; ++p) {
            row0[p] = run;
            run += cnt[plan.union_ids[p]];
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
        const int ke = (s < M && threadIdx.x < 256) ? plan.keff[s] : 0;
        for (int kk = 0; kk < ke; ++kk) {
            const int e = plan.idx[s * k + kk];
            atomicOr(&mask[e * 8 + (threadIdx.x >> 5)], 1u << (threadIdx.x & 31));
        }
        __syncthreads();
        for (int kk = 0; kk < ke; ++kk) {
            const int e = plan.idx[s * k + kk];
            int rank = 0;
            const int wi = threadIdx.x >> 5;
            for (int w2 = 0; w2 < wi; ++w2) rank += __popc(mask[e * 8 + w2]);
            rank += __popc(mask[e * 8 + wi] & ((1u << (threadIdx.x & 31)) - 1u));
            const int p = row0[slot_of[e]] + base[e] + rank;
            plan.pair_token[p] = s;
            plan.tok_pair[s * k + kk] = p;
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

    // ---- 6. combine order of each token: its kk values sorted by union position
    for (int s = threadIdx.x; s < M; s += blockDim.x) {
        const int ke = plan.keff[s];
        for (int j = 0; j < ke; ++j) {
            const int key = slot_of[plan.idx[s * k + j]];
            int pos = 0;
            for (int j2 = 0; j2 < ke; ++j2) {
                const int key2 = slot_of[plan.idx[s * k + j2]];
                pos += (key2 < key || (key2 == key && j2 < j)) ? 1 : 0;
            }
            plan.tok_order[s * k + pos] = j;
        }
    }
    // ---- 7. GEMV slot tables
    for (int p = threadIdx.x; p < nunion + (has_shared ? 1 : 0); p += blockDim.x) {
        const bool sh = p >= nunion;
        const ExpertDev ex = experts[sh ? E : plan.union_ids[p]];
        GemvSlot g, d;
        g.a = ex.gate;
        g.b = ex.up;
        g.a_rs = ex.gate_rs;
        g.b_rs = ex.up_rs;
        g.row0 = sh ? routed_pairs : row0[p];
        g.nrows = sh ? M : cnt[plan.union_ids[p]];
        d = g;
        d.a = ex.down;
        d.b = nullptr;
        d.a_rs = ex.down_rs;
        d.b_rs = nullptr;
        plan.gu_slots[p] = g;
        plan.dn_slots[p] = d;
    }
}

// Routing-weighted combine, crates/peregrine-model/src/mlp.rs:111-127 and
// crates/peregrine-model/src/concurrent.rs:1866-1929: out starts at zero, each
// expert's row is added as out = out + (w * y) in batch-union order, the shared
// expert's row is added last without a weight.
__global__ void __launch_bounds__(256) combine_kernel(const float *__restrict__ y, long long ldy, int D, int k,
                                                      RoutePlan plan, float *__restrict__ out, long long ldo) {
    const int s = blockIdx.y;
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= D) return;
    const int ke = plan.keff[s];
    float acc = 0.0f;
    for (int j = 0; j < ke; ++j) {
        const int kk = plan.tok_order[s * k + j];
        const int p = plan.tok_pair[s * k + kk];
        acc = __fadd_rn(acc, __fmul_rn(plan.w[s * k + kk], y[(long long)p * ldy + d]));
    }
    const int sp0 = *plan.shared_pair0;
    if (sp0 >= 0) acc = __fadd_rn(acc, y[(long long)(sp0 + s) * ldy + d]);
    out[(long long)s * ldo + d] = acc;
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
