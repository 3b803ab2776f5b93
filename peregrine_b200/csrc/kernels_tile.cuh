// Large-batch (prefill) variant of the int4 x int8 expert matmul: tens to thousands of
// activation rows per expert.  One CTA computes a block of 128 weight rows (64 gate + 64 up
// rows in mode 0, 128 down rows in mode 1) against a block of 128 activation rows of one
// expert, so a weight chunk fetched once is used by 128 rows instead of 8 or 16.
//
// Same tile stream, fragment fit and numerics as gemv_w4a8_mma_kernel (kernels_mma.cuh): the
// integer block dots come from mma.sync m16n8k32 (u8 x s8 -> s32), and per (weight row,
// activation row) the group dots are folded into one fp32 accumulator in ascending group
// order, one multiply and one add at a time (crates/peregrine-kernels/src/idot.rs:98-110,
// matmul.rs:75-106).  The int -> float step of the fold is done without a conversion
// instruction: the MMA accumulator starts from the bit pattern of 1.5 * 2^23, so after the
// group's blocks it *is* the float 12582912 + d (exact for |d| < 2^22; a group dot is below
// 2^19); the -8*sum(q) correction is added to that start value as an integer, and subtracting
// 12582912.0f afterwards gives (float)(d - 8*sum(q)) exactly.
#pragma once
#include "kernels_mma.cuh"

namespace pgb {

constexpr int kTileWarps = 8;
constexpr int kTileThreads = kTileWarps * 32;
constexpr int kTileTokens = 128;   // activation rows per CTA
constexpr int kTileStages = 3;
constexpr int kTileWBytes = 8 * kChunkMaxBytes;                   // 8 sixteen-row weight chunks
constexpr int kTileXOff = kTileWBytes;
constexpr int kTileCsOff = kTileXOff + kTileTokens * kXqChunkRowBytes;
constexpr int kTileStageBytes = kTileCsOff + kTileTokens * kChunkBlocks * 4;
constexpr int kTileSmemBytes = kTileStages * kTileStageBytes + 128;

// Row blocks of at most kTileTokens rows, slot by slot: an upper bound for the launch grid.
__host__ __device__ inline int tile_row_blocks_max(int pairs_max, int slots_max) {
    return (pairs_max + kTileTokens - 1) / kTileTokens + slots_max;
}

// One 256-element chunk of the K extent for one warp: NTC 8-row column tiles (compile-time, so the
// unrolled MMA / fold sequence has no branches) against 2 x 2 sixteen-row weight tiles.
template <bool GROUPED, int BPG, int NTC>
__device__ __forceinline__ void tile_chunk(const uint8_t *st, int wo, int g, int t, int rowoff, float nz,
                                           float (&acc)[2][2][4][4], int (&iacc)[2][2][4][4], int (&csacc)[4][2]) {
    constexpr int GPC = kChunkBlocks / BPG;
    const uint8_t *xb = st + kTileXOff + (rowoff + g) * kXqChunkRowBytes + 4 * t;
    const int *csb = reinterpret_cast<const int *>(st + kTileCsOff) + (rowoff + 2 * t) * kChunkBlocks;

    // the MMAs of scale group gi into c (grouped formats) or onto iacc (per-row format)
    auto mma_group = [&](int gi, int (&c)[2][2][4][4]) {
        // -8 * sum(q) of the group's blocks, per activation column of this lane; for grouped
        // formats it rides in the MMA's start value: bits(1.5 * 2^23) + correction
        int cinit[4][2];
#pragma unroll
        for (int nt = 0; nt < NTC; ++nt) {
            int c0 = 0, c1 = 0;
#pragma unroll
            for (int b = 0; b < BPG; ++b) {
                c0 += csb[(8 * nt) * kChunkBlocks + gi * BPG + b];
                c1 += csb[(8 * nt + 1) * kChunkBlocks + gi * BPG + b];
            }
            if (GROUPED) {
                cinit[nt][0] = (int)kMagicBits + c0;
                cinit[nt][1] = (int)kMagicBits + c1;
            } else {
                csacc[nt][0] += c0;
                csacc[nt][1] += c1;
            }
        }
#pragma unroll
        for (int b = 0; b < BPG; ++b) {
            const int blk = gi * BPG + b;
            uint32_t b0[4], b1[4];
#pragma unroll
            for (int nt = 0; nt < NTC; ++nt) {
                // rows past the block's last one read stale shared memory: never stored
                const uint8_t *xr = xb + 8 * nt * kXqChunkRowBytes + blk * 32;
                b0[nt] = *reinterpret_cast<const uint32_t *>(xr);
                b1[nt] = *reinterpret_cast<const uint32_t *>(xr + 16);
            }
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    const uint8_t *wp = st + (h * 4 + 2 * wo + mt) * kChunkMaxBytes + blk * kSlabBytes + t * 4;
                    const uint32_t w0 = *reinterpret_cast<const uint32_t *>(wp + g * 16);
                    const uint32_t w1 = *reinterpret_cast<const uint32_t *>(wp + (g + 8) * 16);
                    const uint32_t a0 = w0 & 0x0F0F0F0Fu, a2 = (w0 >> 4) & 0x0F0F0F0Fu;
                    const uint32_t a1 = w1 & 0x0F0F0F0Fu, a3 = (w1 >> 4) & 0x0F0F0F0Fu;
#pragma unroll
                    for (int nt = 0; nt < NTC; ++nt) {
                        if (!GROUPED)
                            mma_u8s8(iacc[h][mt][nt], a0, a1, a2, a3, b0[nt], b1[nt]);
                        else if (b == 0)
                            mma_u8s8_c(c[h][mt][nt], a0, a1, a2, a3, b0[nt], b1[nt], cinit[nt][0], cinit[nt][1]);
                        else
                            mma_u8s8(c[h][mt][nt], a0, a1, a2, a3, b0[nt], b1[nt]);
                    }
                }
        }
    };
    // the fp32 fold of group gi's dots
    auto fold_group = [&](int gi, int (&c)[2][2][4][4]) {
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
                const float *sp =
                    reinterpret_cast<const float *>(st + (h * 4 + 2 * wo + mt) * kChunkMaxBytes + kChunkSlabBytes);
                const float sc_lo = sp[g * GPC + gi], sc_hi = sp[(g + 8) * GPC + gi];
#pragma unroll
                for (int nt = 0; nt < NTC; ++nt) {
                    fold_pair(acc[h][mt][nt][0], acc[h][mt][nt][1], c[h][mt][nt][0], c[h][mt][nt][1], sc_lo, kMagicF, nz);
                    fold_pair(acc[h][mt][nt][2], acc[h][mt][nt][3], c[h][mt][nt][2], c[h][mt][nt][3], sc_hi, kMagicF, nz);
                }
            }
    };

    int ca[2][2][4][4];
    if (!GROUPED) {
        // integer accumulation over the whole K: nothing to fold per group
#pragma unroll 1
        for (int gi = 0; gi < GPC; ++gi) mma_group(gi, ca);
        return;
    }
    if (BPG == 1) {
        // one block per group: the first dots of a group can be folded while its last MMAs are
        // still running, so the plain order already overlaps the two (measured faster here)
#pragma unroll 1
        for (int gi = 0; gi < GPC; ++gi) {
            mma_group(gi, ca);
            fold_group(gi, ca);
        }
        return;
    }
    // Several blocks per group: a group's fold has to wait for all of its MMAs, so the MMAs of
    // group gi + 1 are issued before group gi is folded, on two alternating result sets.  Two groups
    // per loop trip (not more): the body has to stay inside the instruction cache.
    int cb[2][2][4][4];
    mma_group(0, ca);
#pragma unroll 1
    for (int gi = 0; gi < GPC; gi += 2) {
        if (gi + 1 < GPC) mma_group(gi + 1, cb);
        fold_group(gi, ca);
        if (gi + 2 < GPC) mma_group(gi + 2, ca);
        if (gi + 1 < GPC) fold_group(gi + 1, cb);
    }
}

// grid: x = block of weight rows, y = row block (blocks past the last one return at once).
template <bool GROUPED, int BPG>
__global__ void __launch_bounds__(kTileThreads, 1) ffn_w4a8_tile_kernel(const GemvParams P) {
    constexpr int GPC = kChunkBlocks / BPG;
    constexpr int CHUNK_BYTES = kChunkSlabBytes + (GROUPED ? GPC * 64 : 0);
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int s_slot, s_first, s_per;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int wo = warp & 1, wn = warp >> 1;  // 2 x 4 warps: 32 weight rows (of each half) x 32 activation rows
    const uint32_t bar_u32 = smem_u32(smem + kTileStages * kTileStageBytes);

    // ---- which row block: prefix over the slots' block counts (one warp)
    const int n_slots = *P.n_slots;
    if (warp == 0) {
        int base = 0, found = -1, first = 0, per = kTileTokens;
        for (int j0 = 0; j0 < n_slots && found < 0; j0 += 32) {
            const int j = j0 + lane;
            const int nrj = j < n_slots ? P.slots[j].nrows : 0;
            const int nb = (nrj + kTileTokens - 1) / kTileTokens;
            int inc = nb;
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += v;
            }
            const int lo = base + inc - nb;
            const bool mine = nb > 0 && (int)blockIdx.y >= lo && (int)blockIdx.y < lo + nb;
            const unsigned bal = __ballot_sync(0xffffffffu, mine);
            if (bal) {
                const int src = __ffs(bal) - 1;
                found = j0 + src;
                // the slot's rows are dealt to its blocks evenly, in units of 8 rows
                const int n_src = __shfl_sync(0xffffffffu, nrj, src), nb_src = __shfl_sync(0xffffffffu, nb, src);
                per = 8 * (((n_src + 7) / 8 + nb_src - 1) / nb_src);
                first = ((int)blockIdx.y - __shfl_sync(0xffffffffu, lo, src)) * per;
            }
            base += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (lane == 0) {
            s_slot = found;
            s_first = first;
            s_per = per;
            for (int s = 0; s < kTileStages; ++s) mbar_init(bar_u32 + s * 8, 1);
            fence_mbar_init();
            fence_proxy_async();
        }
    }
    __syncthreads();
    if (s_slot < 0) return;
    const GemvSlot slot = P.slots[s_slot];
    const int first = s_first;
    const int nr = min(s_per, slot.nrows - first);
    if (nr <= 0) return;
    const int prow0 = slot.row0 + first;  // first pair row of the block
    // 8-row column tiles of the block, dealt to the four warp columns: warp column wn owns
    // tiles [wn * q, wn * q + ntc)
    const int q = ((nr + 7) / 8 + 3) / 4;
    const int ntc = max(0, min(q, (nr + 7) / 8 - wn * q));
    const int rowoff = 8 * q * wn;

    // ---- weight tiles of this CTA: stage slot s = half * 4 + i
    const int ob = blockIdx.x;
    const uint8_t *wsrc[8];
#pragma unroll
    for (int s = 0; s < 8; ++s) {
        const int half = s >> 2, i = s & 3;
        const int tile = (P.mode == 0) ? ob * 4 + i : ob * 8 + s;
        const uint8_t *mat = (P.mode == 0 && half) ? slot.b : slot.a;
        wsrc[s] = (tile < P.ntile) ? mat + (unsigned long long)tile * P.tile_bytes : nullptr;
    }
    int n_wt = 0;
#pragma unroll
    for (int s = 0; s < 8; ++s) n_wt += wsrc[s] ? 1 : 0;

    // A bulk copy holds the issuing warp for ~130 cycles, one copy after the other, so the ten copies
    // of a stage are shared out: lane 0 of warp w issues weight tile w, warp 0 also sets the stage's
    // byte count, warps 1 and 2 also fetch the activation rows and their block sums.  (Copies of the
    // other warps may land before the count is set; the phase cannot complete before that arrival.)
    const uint8_t *w_mine = nullptr;
#pragma unroll
    for (int s = 0; s < 8; ++s)
        if (s == warp) w_mine = wsrc[s];
    auto issue = [&](int chunk) {  // lane 0 of every warp
        const int stage = chunk % kTileStages;
        const uint32_t bar = bar_u32 + stage * 8;
        const uint32_t dst = smem_u32(smem + stage * kTileStageBytes);
        const long long cr = (long long)chunk * P.pcap + prow0;
        if (warp == 0) mbar_expect_tx(bar, n_wt * CHUNK_BYTES + nr * (kXqChunkRowBytes + kChunkBlocks * 4));
        if (w_mine) bulk_g2s(dst + warp * kChunkMaxBytes, w_mine + (size_t)chunk * CHUNK_BYTES, CHUNK_BYTES, bar);
        if (warp == 1) bulk_g2s(dst + kTileXOff, P.xq + cr * kXqChunkRowBytes, nr * kXqChunkRowBytes, bar);
        if (warp == 2) bulk_g2s(dst + kTileCsOff, P.csum + cr * kChunkBlocks, nr * kChunkBlocks * 4, bar);
    };
    if (lane == 0)
        for (int c = 0; c < kTileStages - 1 && c < P.nchunk; ++c) issue(c);

    // accumulators [half][m-tile][n-tile][slot]; slot i: row g + 8*(i>>1), column 2t + (i&1)
    float acc[2][2][4][4];
    int iacc[2][2][4][4];  // per-row format: integer sum over the whole K
    int csacc[4][2];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    acc[h][mt][nt][i] = 0.0f;
                    iacc[h][mt][nt][i] = 0;
                }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) csacc[nt][0] = csacc[nt][1] = 0;

    int fail_chunk = -1;
    for (int chunk = 0; chunk < P.nchunk; ++chunk) {
        // every warp is past chunk - 1, so its stage may be refilled
        __syncthreads();
        if (lane == 0 && chunk + kTileStages - 1 < P.nchunk) {
            fence_proxy_async();
            issue(chunk + kTileStages - 1);
        }
        __syncwarp();
        const int stage = chunk % kTileStages;
        {
            const bool ok = mbar_wait_bounded(bar_u32 + stage * 8, (chunk / kTileStages) & 1u);
            if (__any_sync(0xffffffffu, !ok)) {
                if (lane == 0) report_error(P.err, kErrBarrierTimeout);
                fail_chunk = chunk;
                break;
            }
        }
        const uint8_t *st = smem + stage * kTileStageBytes;
        switch (ntc) {
            case 4: tile_chunk<GROUPED, BPG, 4>(st, wo, g, t, rowoff, P.neg_zero, acc, iacc, csacc); break;
            case 3: tile_chunk<GROUPED, BPG, 3>(st, wo, g, t, rowoff, P.neg_zero, acc, iacc, csacc); break;
            case 2: tile_chunk<GROUPED, BPG, 2>(st, wo, g, t, rowoff, P.neg_zero, acc, iacc, csacc); break;
            case 1: tile_chunk<GROUPED, BPG, 1>(st, wo, g, t, rowoff, P.neg_zero, acc, iacc, csacc); break;
            default: break;
        }
    }
    if (fail_chunk >= 0) {
        // let the copies still in flight land before the shared memory is released
        if (tid == 0) {
            const int last = min(P.nchunk, fail_chunk + kTileStages);
            for (int q = fail_chunk; q < last; ++q) {
                const long long t0 = clock64();
                while (!mbar_try_wait(bar_u32 + (q % kTileStages) * 8, (q / kTileStages) & 1u))
                    if (clock64() - t0 > 200000000LL) break;
            }
        }
        __syncthreads();
        return;
    }

    // ---- epilogue
    float amax_row[4][2];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) amax_row[nt][0] = amax_row[nt][1] = 0.0f;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int ridx = rowoff + 8 * nt + 2 * t + j;  // row inside the block
            const bool valid = ridx < nr && nt < ntc;  // tiles past ntc belong to the next warp column
            const float sxa = P.sx[prow0 + (valid ? ridx : 0)];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int hi = 0; hi < 2; ++hi) {
                    const int i = 2 * hi + j;
                    const int r = g + 8 * hi;
                    float v[2];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int tile = (P.mode == 0) ? ob * 4 + 2 * wo + mt : ob * 8 + h * 4 + 2 * wo + mt;
                        const int o = tile * 16 + r;
                        if (GROUPED) {
                            v[h] = __fmul_rn(acc[h][mt][nt][i], sxa);
                        } else {
                            const float *rsp = (P.mode == 0 && h) ? slot.b_rs : slot.a_rs;
                            const float rs = (tile < P.ntile) ? rsp[o] : 0.0f;
                            const int d = iacc[h][mt][nt][i] + csacc[nt][j];
                            v[h] = __fmul_rn(__fmul_rn((float)d, rs), sxa);
                        }
                    }
                    if (P.mode == 0) {
                        const int o = (ob * 4 + 2 * wo + mt) * 16 + r;
                        if (valid && o < P.O) {
                            const float hval = __fmul_rn(silu32(v[0]), v[1]);
                            P.out[(long long)(prow0 + ridx) * P.out_stride + o] = hval;
                            const float a = fabsf(hval);
                            if (a == a) amax_row[nt][j] = fmaxf(amax_row[nt][j], a);
                        }
                    } else {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const int o = (ob * 8 + h * 4 + 2 * wo + mt) * 16 + r;
                            if (valid && o < P.O) P.out[(long long)(prow0 + ridx) * P.out_stride + o] = v[h];
                        }
                    }
                }
        }
    if (P.mode == 0 && P.amax_out != nullptr) {
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                float a = amax_row[nt][j];
                a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 4));
                a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 8));
                a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 16));
                const int ridx = rowoff + 8 * nt + 2 * t + j;
                if (g == 0 && ridx < nr && nt < ntc && a > 0.0f) atomicMax(P.amax_out + prow0 + ridx, __float_as_uint(a));
            }
    }
}

}  // namespace pgb
