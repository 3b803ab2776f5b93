// Batched-decode variant of the int4 x int8 expert matmul for experts with 9 to ~32 (and more)
// activation rows: the warps of a CTA work on ONE expert at a time and share its activation rows.
//
// gemv_w4a8_mma_kernel (kernels_mma.cuh) gives every warp a ring of its own, weights and activation
// rows alike; beyond 8 rows per expert the rows of a 256-element chunk (272 bytes each) weigh as much
// as the chunk's packed weights (5 KB for a tile pair), the traffic from L2 into the SM doubles and
// an expert with more than 16 rows is streamed once per 16 rows.  Here a work item is (expert, block
// of 8 tile pairs), run in passes of up to 32 rows: a producer warp fills a CTA-wide ring stage by stage with
// the 8 warps' weight chunks, ONE copy of the pass's activation rows of that chunk and their block
// sums; each consumer warp multiplies its own tile pair with all rows of the pass (m16n8k32 int8
// MMAs, 1 to 4 column groups of 8 rows, chosen per item) and folds the group dots into fp32 in the
// reference's order (crates/peregrine-kernels/src/idot.rs:98-110, matmul.rs:75-106): the same
// arithmetic, accumulator presets and packed fold as gemv_w4a8_mma_kernel.  An expert's weights are
// fetched once per 32 rows, the activation rows once per CTA instead of once per warp.
#pragma once
#include "kernels_mma.cuh"

namespace pgb {

constexpr int kBlkW = 8;                  // consumer warps = tile pairs per work item
constexpr int kBlkThreads = (kBlkW + 1) * 32;
constexpr int kBlkRows = 32;              // activation rows per pass
constexpr int kBlkStages = 4;
constexpr int kBlkXOff = kBlkW * kStageBytes;
constexpr int kBlkCsOff = kBlkXOff + kBlkRows * kXqChunkRowBytes;
constexpr int kBlkStageBytes = kBlkCsOff + kBlkRows * kChunkBlocks * 4;
constexpr int kBlkBarOff = kBlkStages * kBlkStageBytes;
constexpr int kBlkCumOff = kBlkBarOff + 128;
constexpr int kBlkMaxSlots = 320;         // slots of a launch (experts of a layer + the shared one)
constexpr int kBlkSmemBytes = kBlkCumOff + 2 * (kBlkMaxSlots + 1) * 4 + 64;

struct BlkItem {
    int slot, tb, row0, nrows, npass;
    const uint8_t *a, *b;  // this warp's tile streams (nullptr: no tile for this warp)
    const float *a_rs, *b_rs;
    int tile;              // this warp's tile pair index
};

// One chunk of one item for one consumer warp: NT column groups of 8 rows.
template <int NT, bool GROUPED, int BPG>
__device__ __forceinline__ void blk_chunk(const uint8_t *wst, const uint8_t *xst, const uint8_t *cst, int g, int t,
                                          float (&acc)[2][4][4], int (&iacc)[2][4][4], float neg_zero) {
    constexpr int GPC = kChunkBlocks / BPG;
#pragma unroll
    for (int gi = 0; gi < GPC; ++gi) {
        int c[2][NT][4];
        int cinit[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            int cs0 = 0, cs1 = 0;
#pragma unroll
            for (int b = 0; b < BPG; ++b) {
                cs0 += *reinterpret_cast<const int *>(cst + ((8 * nt + 2 * t) * kChunkBlocks + gi * BPG + b) * 4);
                cs1 += *reinterpret_cast<const int *>(cst + ((8 * nt + 2 * t + 1) * kChunkBlocks + gi * BPG + b) * 4);
            }
            cinit[nt][0] = (GROUPED ? (int)kMagicBits : 0) + cs0;
            cinit[nt][1] = (GROUPED ? (int)kMagicBits : 0) + cs1;
        }
#pragma unroll
        for (int b = 0; b < BPG; ++b) {
            const int blk = gi * BPG + b;
            uint32_t b0[NT], b1[NT];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                // columns past the pass's rows read stale shared memory: their results are never stored
                const uint8_t *xr = xst + (8 * nt + g) * kXqChunkRowBytes + blk * 32 + 4 * t;
                b0[nt] = *reinterpret_cast<const uint32_t *>(xr);
                b1[nt] = *reinterpret_cast<const uint32_t *>(xr + 16);
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint8_t *wp = wst + h * kChunkMaxBytes + blk * kSlabBytes + t * 4;
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
                const float *sp = reinterpret_cast<const float *>(wst + h * kChunkMaxBytes + kChunkSlabBytes);
                const float sc_lo = sp[g * GPC + gi], sc_hi = sp[(g + 8) * GPC + gi];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    fold_pair(acc[h][nt][0], acc[h][nt][1], c[h][nt][0], c[h][nt][1], sc_lo, kMagicF, neg_zero);
                    fold_pair(acc[h][nt][2], acc[h][nt][3], c[h][nt][2], c[h][nt][3], sc_hi, kMagicF, neg_zero);
                }
            }
        } else {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int i = 0; i < 4; ++i) iacc[h][nt][i] += c[h][nt][i];
        }
    }
}

// Activations in the chunk-major layout (qrow_i8_kernel): P.xq[chunk][pcap][272], P.csum[chunk][pcap][8],
// P.sx[row]; rows are pair rows (row0 + i); P.rowmap is not used.  Grid: one CTA per SM.
template <bool GROUPED, int BPG>
__global__ void __launch_bounds__(kBlkThreads, 1) gemv_w4a8_block_kernel(const GemvParams P) {
    constexpr int GPC = kChunkBlocks / BPG;
    constexpr int CHUNK_BYTES = kChunkSlabBytes + (GROUPED ? GPC * 64 : 0);
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t smem_u = smem_u32(smem);
    const uint32_t full_b = smem_u + kBlkBarOff, empty_b = full_b + kBlkStages * 8;
    int *cum = reinterpret_cast<int *>(smem + kBlkCumOff);

    const int n_slots = min(*P.n_slots, kBlkMaxSlots);
    const int n_tb = (P.warp_tiles + kBlkW - 1) / kBlkW;
    // Slots in order of falling row count (ties by index): an item of an expert with 32 rows costs four
    // times the tensor-core and fold work of one with 8, so the items are dealt heaviest first and in
    // serpentine order over the CTAs (round 0: CTA b takes item b, round 1: item 2G - 1 - b, ...), which
    // evens out the sums without a shared counter.
    int *nrow_s = cum;                      // [n_slots] row counts
    int *order = cum + kBlkMaxSlots + 1;    // [n_active] slot of rank r
    for (int s = tid; s < n_slots; s += blockDim.x) nrow_s[s] = P.slots[s].nrows;
    if (tid == 0) {
        for (int s = 0; s < kBlkStages; ++s) {
            mbar_init(full_b + s * 8, 1);
            mbar_init(empty_b + s * 8, kBlkW);
        }
        fence_mbar_init();
        fence_proxy_async();
    }
    __syncthreads();
    for (int s = tid; s < n_slots; s += blockDim.x) {
        const int nr = nrow_s[s];
        if (nr > 0) {
            int rank = 0;
            for (int o = 0; o < n_slots; ++o) {
                const int no = nrow_s[o];
                rank += (no > nr || (no == nr && o < s)) ? 1 : 0;
            }
            order[rank] = s;
        }
    }
    __shared__ int s_active;
    if (tid == 0) {
        int n = 0;
        for (int s = 0; s < n_slots; ++s) n += nrow_s[s] > 0 ? 1 : 0;
        s_active = n;
    }
    __syncthreads();
    const int total = s_active * n_tb;

    // the k-th item of this CTA -> index in the dealing order -> (slot, tile block)
    const int G = gridDim.x;
    auto item_index = [&](int k) { return k * G + ((k & 1) ? G - 1 - (int)blockIdx.x : (int)blockIdx.x); };
    auto decode = [&](int i, BlkItem &it, int w) {
        const int r = i / n_tb;
        const int slot = order[r];
        const GemvSlot *s = P.slots + slot;
        it.slot = slot;
        it.tb = i - r * n_tb;
        it.nrows = s->nrows;
        it.npass = (s->nrows + kBlkRows - 1) / kBlkRows;
        it.row0 = s->row0;
        it.tile = it.tb * kBlkW + w;
        it.a = it.b = nullptr;
        it.a_rs = s->a_rs;
        it.b_rs = s->b_rs;
        if (it.tile < P.warp_tiles) {
            if (P.mode == 0) {
                it.a = s->a + (unsigned long long)it.tile * P.tile_bytes;
                it.b = s->b + (unsigned long long)it.tile * P.tile_bytes;
            } else {
                it.a = s->a + (unsigned long long)(2 * it.tile) * P.tile_bytes;
                it.b = (2 * it.tile + 1 < P.ntile) ? s->a + (unsigned long long)(2 * it.tile + 1) * P.tile_bytes : nullptr;
            }
        }
    };

    if (warp == kBlkW) {
        // ======================================================= producer warp
        // lane w < 8: the chunk (pair) of consumer warp w; lane 8: the pass's activation rows of the
        // chunk; lane 9: their block sums
        uint32_t q = 0;
        bool ok = true;
        for (int k = 0; ok; ++k) {
            const int i = item_index(k);
            if (i >= total) {
                if (k * G >= total) break;
                continue;  // this round has fewer items than CTAs
            }
            BlkItem it;
            decode(i, it, lane < kBlkW ? lane : 0);
            const int my_bytes = (lane < kBlkW && it.a) ? (it.b ? 2 : 1) * CHUNK_BYTES : 0;
            int wbytes = my_bytes;
            for (int o = 16; o > 0; o >>= 1) wbytes += __shfl_xor_sync(0xffffffffu, wbytes, o);
            for (int pc = 0; pc < it.npass * P.nchunk; ++pc, ++q) {
                const int pass = pc / P.nchunk, chunk = pc - pass * P.nchunk;
                const int first = it.row0 + pass * kBlkRows, nr = min(kBlkRows, it.nrows - pass * kBlkRows);
                const uint32_t stage = q % kBlkStages;
                if (q >= kBlkStages) {
                    const bool fine = mbar_wait_bounded(empty_b + stage * 8, ((q / kBlkStages) + 1) & 1u);
                    if (__any_sync(0xffffffffu, !fine)) {
                        if (lane == 0) report_error(P.err, kErrBarrierTimeout);
                        ok = false;
                        break;
                    }
                }
                const uint32_t bar = full_b + stage * 8;
                const uint32_t dst = smem_u + stage * kBlkStageBytes;
                if (lane == 0) {
                    fence_proxy_async();
                    mbar_expect_tx(bar, wbytes + nr * (kXqChunkRowBytes + kChunkBlocks * 4));
                }
                __syncwarp();
                const size_t off = (size_t)chunk * CHUNK_BYTES;
                const long long cr = (long long)chunk * P.pcap + first;
                if (lane < kBlkW) {
                    if (it.a) bulk_g2s(dst + lane * kStageBytes, it.a + off, CHUNK_BYTES, bar);
                    if (it.a && it.b) bulk_g2s(dst + lane * kStageBytes + kChunkMaxBytes, it.b + off, CHUNK_BYTES, bar);
                } else if (lane == kBlkW) {
                    bulk_g2s(dst + kBlkXOff, P.xq + cr * kXqChunkRowBytes, nr * kXqChunkRowBytes, bar);
                } else if (lane == kBlkW + 1) {
                    bulk_g2s(dst + kBlkCsOff, P.csum + cr * kChunkBlocks, nr * kChunkBlocks * 4, bar);
                }
            }
        }
        return;
    }
    // =========================================================== consumer warps
    uint32_t q = 0;
    float acc[2][4][4];
    int iacc[2][4][4];
    bool ok = true;
    for (int k = 0; ok; ++k) {
        const int i = item_index(k);
        if (i >= total) {
            if (k * G >= total) break;
            continue;
        }
        BlkItem it;
        decode(i, it, warp);
        for (int pass = 0; pass < it.npass && ok; ++pass) {
            const int row0 = it.row0 + pass * kBlkRows, nr = min(kBlkRows, it.nrows - pass * kBlkRows);
            const int nt_n = (nr + 7) >> 3;
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        acc[h][nt][j] = 0.0f;
                        iacc[h][nt][j] = 0;
                    }
            for (int chunk = 0; chunk < P.nchunk; ++chunk, ++q) {
                const uint32_t stage = q % kBlkStages;
                const bool fine = mbar_wait_bounded(full_b + stage * 8, (q / kBlkStages) & 1u);
                if (__any_sync(0xffffffffu, !fine)) {
                    if (lane == 0) report_error(P.err, kErrBarrierTimeout);
                    ok = false;
                    break;
                }
                if (it.a) {
                    const uint8_t *st = smem + stage * kBlkStageBytes;
                    const uint8_t *wst = st + warp * kStageBytes, *xst = st + kBlkXOff, *cst = st + kBlkCsOff;
                    switch (nt_n) {
                        case 1: blk_chunk<1, GROUPED, BPG>(wst, xst, cst, g, t, acc, iacc, P.neg_zero); break;
                        case 2: blk_chunk<2, GROUPED, BPG>(wst, xst, cst, g, t, acc, iacc, P.neg_zero); break;
                        case 3: blk_chunk<3, GROUPED, BPG>(wst, xst, cst, g, t, acc, iacc, P.neg_zero); break;
                        default: blk_chunk<4, GROUPED, BPG>(wst, xst, cst, g, t, acc, iacc, P.neg_zero); break;
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_b + stage * 8);
            }
            if (!ok || !it.a) continue;
            // ---- epilogue of the pass: activation scale, SwiGLU (mode 0), stores, row maxima
            auto value = [&](int h, int nt, int j, int o) -> float {
                const int rr = min(8 * nt + 2 * t + (j & 1), nr - 1);
                const float sxa = P.sx[row0 + rr];
                if (GROUPED) return __fmul_rn(acc[h][nt][j], sxa);
                const float *rsp = (P.mode == 0 && h) ? it.b_rs : it.a_rs;
                const float rs = (o < P.ntile * 16) ? rsp[o] : 0.0f;
                return __fmul_rn(__fmul_rn((float)iacc[h][nt][j], rs), sxa);  // block corrections rode in the MMA start values
            };
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                if (nt >= nt_n) break;
                float amax2[2] = {0.0f, 0.0f};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int ridx = 8 * nt + 2 * t + (j & 1);
                    const bool valid = ridx < nr;
                    const int r = g + 8 * (j >> 1);
                    if (P.mode == 0) {
                        const int o = it.tile * 16 + r;
                        const float vg = value(0, nt, j, o), vu = value(1, nt, j, o);
                        if (valid && o < P.O) {
                            const float hval = __fmul_rn(silu32(vg), vu);
                            P.out[(long long)(row0 + ridx) * P.out_stride + o] = hval;
                            const float a = fabsf(hval);
                            if (a == a) amax2[j & 1] = fmaxf(amax2[j & 1], a);  // NaN never becomes the maximum
                        }
                    } else {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const int o = (2 * it.tile + h) * 16 + r;
                            const float v = value(h, nt, j, o);
                            if (valid && o < P.O && (h == 0 || it.b))
                                P.out[(long long)(row0 + ridx) * P.out_stride + o] = v;
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
                        const int ridx = 8 * nt + 2 * t + j;
                        if (g == 0 && ridx < nr && a > 0.0f) atomicMax(P.amax_out + row0 + ridx, __float_as_uint(a));
                    }
                }
            }
        }
        // the same warp ran every pass of this (expert, tile pair): its arrival completes the expert's share
        if (ok && it.a && P.mode == 1 && P.comb.col_done != nullptr) ordered_combine_tile(P, it.tile, lane, n_slots);
    }
}

}  // namespace pgb
