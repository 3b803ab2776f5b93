// Small-batch variant of the int4 x int8 expert matmul: 3 to ~32 activation rows
// per expert.  Same tile stream, ring, cursor and epilogues as gemv_w4a8_kernel
// (kernels.cuh); the integer block dots are formed by the warp-level int8 MMA
// (m16n8k32, u8 x s8 -> s32) instead of dp4a, so one instruction covers 16 weight
// rows x 8 activation rows x 32 elements.  The fp32 side is unchanged: per (row,
// activation row) one lane folds the group dots in ascending group order, one
// multiply and one add at a time (crates/peregrine-kernels/src/idot.rs:98-110,
// matmul.rs:75-106).
//
// Fragment fit: lane (g = lane/4, t = lane%4) of an m16n8k32 MMA holds, of the A
// operand, elements [4t, 4t+4) and [16+4t, 16+4t+4) of rows g and g+8.  Word t of
// a row's 16-byte segment in the tile stream is exactly elem[4t..4t+3] in its low
// nibbles and elem[16+4t..] in its high nibbles, so two 32-bit loads and four
// mask/shift operations build the whole A fragment.  Stored nibbles are v+8; the
// accumulator therefore starts from -8*sum(q) of the activation block (the same
// correction the dp4a kernel uses).
#pragma once
#include "kernels.cuh"

namespace pgb {

#ifndef PGB_MMA_WARPS
#define PGB_MMA_WARPS 10
#endif
constexpr int kMmaWarps = PGB_MMA_WARPS;
constexpr int kMmaThreads = kMmaWarps * 32;
// a stage holds two 16-row weight chunks, the pass's activation rows of the same chunk
// (chunk-major layout, 272 bytes per row) and their 8 block sums each
__host__ __device__ constexpr int mma_stages(int nt) { return nt == 1 ? 3 : 2; }
__host__ __device__ constexpr int mma_stage_bytes(int nt) {
    return kStageBytes + 8 * nt * kXqChunkRowBytes + 8 * nt * kChunkBlocks * 4;
}
__host__ __device__ constexpr int mma_ring_bytes(int nt) { return kMmaWarps * mma_stages(nt) * mma_stage_bytes(nt); }
constexpr int kMmaBarBytes = ((kMmaWarps * 3 * 8 + 127) / 128) * 128;

__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Exact int -> float without a conversion instruction: an MMA accumulator that starts from the bit
// pattern of 1.5 * 2^23 (plus the integer -8*sum(q) correction) reads, as a float, 12582912 + d for
// |d| < 2^22; subtracting 12582912.0f gives (float)d exactly.
constexpr uint32_t kMagicBits = 0x4B400000u;  // 1.5 * 2^23
constexpr float kMagicF = 12582912.0f;

// d = a * b + c with c in registers of its own, so a group's first MMA can start from a constant
// without first copying it into the destination.
__device__ __forceinline__ void mma_u8s8_c(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                           uint32_t b1, int c0, int c1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%10,%11};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c0), "r"(c1));
}

// Two accumulators of one weight row (neighbouring activation columns) take one fold step,
// (a0, a1) += sc * ((float)bits(c0, c1) - K), on the packed fp32 pair instructions of sm_100, each
// lane rounded exactly as the scalar subtract / multiply / add of the reference would be
// (crates/peregrine-kernels/src/idot.rs:98-110).  The product must be rounded on its own: the
// assembler contracts a packed multiply that feeds a packed add into one fused multiply-add even
// when both carry an explicit rounding mode, so the multiply is written as a fused multiply-add
// onto negative zero (x + -0 = x for every x, so this *is* the rounded product) with the zero
// taken from a kernel argument, which nothing can fold away and nothing can fuse further.
__device__ __forceinline__ void fold_pair(float &a0, float &a1, int c0, int c1, float sc, float K, float nz) {
    asm("{\n\t.reg .b64 cc, kk, ss, aa, ff, pp, zz;\n\t"
        "mov.b64 cc, {%2, %3};\n\tmov.b64 kk, {%5, %5};\n\tmov.b64 ss, {%4, %4};\n\t"
        "mov.b64 aa, {%0, %1};\n\tmov.b64 zz, {%6, %6};\n\t"
        "sub.rn.f32x2 ff, cc, kk;\n\tfma.rn.f32x2 pp, ff, ss, zz;\n\tadd.rn.f32x2 aa, aa, pp;\n\t"
        "mov.b64 {%0, %1}, aa;\n\t}"
        : "+f"(a0), "+f"(a1)
        : "r"(c0), "r"(c1), "f"(sc), "f"(K), "f"(nz));
}

// NT = 8-row activation groups per pass (rows per pass = 8 * NT).  Activations come in the
// chunk-major layout (kernels.cuh, qrow_i8_kernel): P.xq[chunk][pcap][272], P.csum[chunk][pcap][8],
// P.sx[row]; rows are indexed by pair row (row0 + i), P.rowmap is not used.
template <int NT, bool GROUPED, int BPG, bool TAP>
__global__ void __launch_bounds__(kMmaThreads, 1) gemv_w4a8_mma_kernel(const GemvParams P) {
    constexpr int RMAX = 8 * NT;
    constexpr int STAGES = mma_stages(NT);
    constexpr int STAGE_BYTES = mma_stage_bytes(NT);
    constexpr int X_OFF = kStageBytes, CS_OFF = kStageBytes + RMAX * kXqChunkRowBytes;
    constexpr int GPC = kChunkBlocks / BPG;
    constexpr int CHUNK_BYTES = kChunkSlabBytes + (GROUPED ? GPC * 64 : 0);
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    uint8_t *ring = smem + warp * (STAGES * STAGE_BYTES);
    const uint32_t ring_u32 = smem_u32(ring);
    const uint32_t bar_u32 = smem_u32(smem + mma_ring_bytes(NT)) + warp * (STAGES * 8);

    if (lane == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(bar_u32 + s * 8, 1);
        fence_mbar_init();
        fence_proxy_async();
    }
    __syncwarp();

    const int n_slots = *P.n_slots;
    const int total = n_slots * P.warp_tiles;
    const int stride = gridDim.x * kMmaWarps;

    TileCursor fc, cc;
    fc.i = blockIdx.x + gridDim.x * warp;
    fc.pass = 0;
    fc.chunk = 0;
    cursor_seek<RMAX>(fc, P, P.slots, total, stride);
    cc = fc;
    uint32_t fq = 0, cq = 0;

    auto issue = [&](const TileCursor &c, uint32_t q) {
        const uint32_t stage = q % STAGES;
        const uint32_t bar = bar_u32 + stage * 8;
        const uint32_t dst = ring_u32 + stage * STAGE_BYTES;
        const size_t off = (size_t)c.chunk * CHUNK_BYTES;
        const int first = c.row0 + c.pass * RMAX;
        const int nr = min(RMAX, c.nrows - c.pass * RMAX);
        const long long cr = (long long)c.chunk * P.pcap + first;
        mbar_expect_tx(bar, (c.b ? 2 * CHUNK_BYTES : CHUNK_BYTES) + nr * (kXqChunkRowBytes + kChunkBlocks * 4));
        bulk_g2s(dst, c.a + off, CHUNK_BYTES, bar);
        if (c.b) bulk_g2s(dst + kChunkMaxBytes, c.b + off, CHUNK_BYTES, bar);
        bulk_g2s(dst + X_OFF, P.xq + cr * kXqChunkRowBytes, nr * kXqChunkRowBytes, bar);
        bulk_g2s(dst + CS_OFF, P.csum + cr * kChunkBlocks, nr * kChunkBlocks * 4, bar);
    };
    while (fc.i < total && fq < cq + STAGES) {
        if (lane == 0) issue(fc, fq);
        cursor_next<RMAX>(fc, P, P.slots, total, stride);
        ++fq;
    }

    // accumulators: [half][n-tile][fragment slot]; slot i: row g + 8*(i>>1), column 2t + (i&1)
    float acc[2][NT][4];
    int iacc[2][NT][4];
    bool failed = false;

    while (cc.i < total) {
        if (fc.i < total && fq < cq + STAGES) {
            if (lane == 0) {
                fence_proxy_async();
                issue(fc, fq);
            }
            cursor_next<RMAX>(fc, P, P.slots, total, stride);
            ++fq;
        }
        const uint32_t stage = cq % STAGES;
        const uint32_t parity = (cq / STAGES) & 1u;
        {
            const bool ok = mbar_wait_bounded(bar_u32 + stage * 8, parity);
            if (__any_sync(0xffffffffu, !ok)) {
                if (lane == 0) report_error(P.err, kErrBarrierTimeout);
                failed = true;
                break;
            }
        }
        if (cc.chunk == 0) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        acc[h][nt][i] = 0.0f;
                        iacc[h][nt][i] = 0;
                    }
            }
        }
        const uint8_t *st = ring + stage * STAGE_BYTES;
#pragma unroll
        for (int gi = 0; gi < GPC; ++gi) {
            int c[2][NT][4];
            // -8 * sum(q) of the group's blocks per activation column of this lane; the first MMA of
            // the group starts from bits(1.5 * 2^23) + that correction (grouped formats) or from it
            // alone (per-row format, integer accumulation over the whole K)
            int csg[NT][2], cinit[NT][2];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                csg[nt][0] = csg[nt][1] = 0;
#pragma unroll
                for (int b = 0; b < BPG; ++b)
#pragma unroll
                    for (int j = 0; j < 2; ++j)
                        csg[nt][j] += *reinterpret_cast<const int *>(st + CS_OFF + ((8 * nt + 2 * t + j) * kChunkBlocks + gi * BPG + b) * 4);
                cinit[nt][0] = (GROUPED ? (int)kMagicBits : 0) + csg[nt][0];
                cinit[nt][1] = (GROUPED ? (int)kMagicBits : 0) + csg[nt][1];
            }
#pragma unroll
            for (int b = 0; b < BPG; ++b) {
                const int blk = gi * BPG + b;
                uint32_t b0[NT], b1[NT];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    // columns past the pass's rows read stale shared memory: their results are never stored
                    const uint8_t *xr = st + X_OFF + (8 * nt + g) * kXqChunkRowBytes + blk * 32 + 4 * t;
                    b0[nt] = *reinterpret_cast<const uint32_t *>(xr);
                    b1[nt] = *reinterpret_cast<const uint32_t *>(xr + 16);
                }
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint8_t *wp = st + h * kChunkMaxBytes + blk * kSlabBytes + t * 4;
                    const uint32_t w0 = *reinterpret_cast<const uint32_t *>(wp + g * 16);
                    const uint32_t w1 = *reinterpret_cast<const uint32_t *>(wp + (g + 8) * 16);
                    const uint32_t a0 = w0 & 0x0F0F0F0Fu, a2 = (w0 >> 4) & 0x0F0F0F0Fu;
                    const uint32_t a1 = w1 & 0x0F0F0F0Fu, a3 = (w1 >> 4) & 0x0F0F0F0Fu;
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        if (b == 0)
                            mma_u8s8_c(c[h][nt], a0, a1, a2, a3, b0[nt], b1[nt], cinit[nt][0], cinit[nt][1]);
                        else
                            mma_u8s8(c[h][nt], a0, a1, a2, a3, b0[nt], b1[nt]);
                    }
                }
            }
            if (GROUPED) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const float *sp = reinterpret_cast<const float *>(st + h * kChunkMaxBytes + kChunkSlabBytes);
                    const float sc_lo = sp[g * GPC + gi], sc_hi = sp[(g + 8) * GPC + gi];
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        fold_pair(acc[h][nt][0], acc[h][nt][1], c[h][nt][0], c[h][nt][1], sc_lo, kMagicF, P.neg_zero);
                        fold_pair(acc[h][nt][2], acc[h][nt][3], c[h][nt][2], c[h][nt][3], sc_hi, kMagicF, P.neg_zero);
                        if (TAP) {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int d = c[h][nt][i] - (int)kMagicBits;
                                const int ridx = cc.pass * RMAX + 8 * nt + 2 * t + (i & 1);
                                const int r = g + 8 * (i >> 1);
                                const int o = (P.mode == 0) ? cc.tile * 16 + r : (2 * cc.tile + h) * 16 + r;
                                const int gg = cc.chunk * GPC + gi;
                                if (P.tap != nullptr && ridx < cc.nrows && o < P.O && gg < P.ng_tap && (h == 0 || cc.b)) {
                                    const long long base = (P.mode == 0)
                                                               ? ((long long)(cc.row0 + ridx) * 2 + h) * P.O + o
                                                               : (long long)(cc.row0 + ridx) * P.O + o;
                                    P.tap[base * P.ng_tap + gg] = d;
                                }
                            }
                        }
                    }
                }
            } else {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    // the block corrections entered through the MMA's start value
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int i = 0; i < 4; ++i) iacc[h][nt][i] += c[h][nt][i];
                }
            }
        }
        __syncwarp();
        if (cc.chunk == P.nchunk - 1) {
            // value of accumulator slot (h, nt, i) after the activation scale
            auto value = [&](int h, int nt, int i, int o) -> float {
                const int rr = min(cc.pass * RMAX + 8 * nt + 2 * t + (i & 1), cc.nrows - 1);
                const float sxa = P.sx[cc.row0 + rr];
                if (GROUPED) return __fmul_rn(acc[h][nt][i], sxa);
                const float *rsp = (P.mode == 0 && h) ? cc.b_rs : cc.a_rs;
                const float rs = (o < P.ntile * 16) ? rsp[o] : 0.0f;
                const int d = iacc[h][nt][i];  // block corrections included (they rode in the MMA start values)
                if (TAP && P.tap != nullptr && o < P.O && (h == 0 || cc.b)) {
                    const int ridx = cc.pass * RMAX + 8 * nt + 2 * t + (i & 1);
                    if (ridx < cc.nrows) {
                        const long long base = (P.mode == 0) ? ((long long)(cc.row0 + ridx) * 2 + h) * P.O + o
                                                             : (long long)(cc.row0 + ridx) * P.O + o;
                        P.tap[base] = d;
                    }
                }
                return __fmul_rn(__fmul_rn((float)d, rs), sxa);
            };
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                float amax2[2] = {0.0f, 0.0f};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int ridx = cc.pass * RMAX + 8 * nt + 2 * t + (i & 1);
                    const bool valid = ridx < cc.nrows;
                    const int r = g + 8 * (i >> 1);
                    if (P.mode == 0) {
                        const int o = cc.tile * 16 + r;
                        const float vg = value(0, nt, i, o), vu = value(1, nt, i, o);
                        if (valid && o < P.O) {
                            const float hval = __fmul_rn(silu32(vg), vu);
                            P.out[(long long)(cc.row0 + ridx) * P.out_stride + o] = hval;
                            const float a = fabsf(hval);
                            if (a == a) amax2[i & 1] = fmaxf(amax2[i & 1], a);  // NaN never becomes the maximum
                        }
                    } else {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const int o = (2 * cc.tile + h) * 16 + r;
                            const float v = value(h, nt, i, o);
                            if (valid && o < P.O && (h == 0 || cc.b))
                                P.out[(long long)(cc.row0 + ridx) * P.out_stride + o] = v;
                        }
                    }
                }
                if (P.mode == 0 && P.amax_out != nullptr) {
                    // row maxima of |h|: reduce over the 8 lanes that share this lane's two columns
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        float a = amax2[j];
                        a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 4));
                        a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 8));
                        a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 16));
                        const int ridx = cc.pass * RMAX + 8 * nt + 2 * t + j;
                        if (g == 0 && ridx < cc.nrows && a > 0.0f)
                            atomicMax(P.amax_out + cc.row0 + ridx, __float_as_uint(a));
                    }
                }
            }
            if (P.mode == 1 && P.comb.col_done != nullptr && cc.pass == cc.npass - 1)
                ordered_combine_tile(P, cc.tile, lane, n_slots);
        }
        cursor_next<RMAX>(cc, P, P.slots, total, stride);
        ++cq;
    }
    if (failed) {
        for (uint32_t q = cq; q < fq; ++q) {
            const uint32_t stage = q % STAGES, parity = (q / STAGES) & 1u;
            const long long t0 = clock64();
            while (!mbar_try_wait(bar_u32 + stage * 8, parity))
                if (clock64() - t0 > 200000000LL) break;
        }
    }
}

}  // namespace pgb
