// Batched-decode variant of the int4 x int8 expert matmul for experts with 9 to ~32 (and more)
// activation rows: the warps of a CTA work on ONE expert at a time and share its activation rows.
//
// gemv_w4a8_mma_kernel (kernels_mma.cuh) gives every warp a ring of its own, weights and activation
// rows alike; beyond 8 rows per expert the rows of a 256-element chunk (272 bytes each) weigh as much
// as the chunk's packed weights (5 KB for a tile pair), the traffic from L2 into the SM doubles and
// an expert with more than 16 rows is streamed once per 16 rows.  Here a work item is (expert, block
// of up to 32 rows, block of up to 8 tile pairs): four producer warps fill a CTA-wide ring stage by stage with
// the pairs' weight chunks, ONE copy of the item's activation rows of that chunk and their block
// sums; 16 consumer warps take one 16-row tile each (warp 2p + h: half h of pair p), multiply it with
// all rows of the item (m16n8k32 int8 MMAs, 1 to 4 column groups of 8 rows, chosen per item) and fold
// the group dots into fp32 in the reference's order (crates/peregrine-kernels/src/idot.rs:98-110,
// matmul.rs:75-106): the same arithmetic, accumulator presets and packed fold as
// gemv_w4a8_mma_kernel.  One tile per warp rather than a pair keeps four warps on every scheduler: a
// chunk is a chain of shared-memory loads, MMAs and a sequential fold, and with two warps per
// scheduler the issue slots stood empty two thirds of the time (measured as fast as the pair version,
// not faster: the SM's rate goes with the consumer warps it runs).  In a gate/up launch the up warp hands
// its values to the gate warp of the pair through shared memory for the SwiGLU.  An expert's weights
// are fetched once per 32 rows, the activation rows once per CTA instead of once per warp.  The
// ordered combine is not fused here (at these batch sizes it is a launch of its own).
#pragma once
#include "kernels_mma.cuh"

namespace pgb {

constexpr int kBlkW = 8;                  // tile pairs per work item
constexpr int kBlkCW = 2 * kBlkW;         // consumer warps: one tile each
constexpr int kBlkPW = 4;                 // producer warps: two tile pairs each (the first also the rows)
constexpr int kBlkThreads = (kBlkCW + kBlkPW) * 32;
constexpr int kBlkRows = 32;              // activation rows per work item, at most
constexpr int kBlkStages = 4;
constexpr int kBlkXOff = kBlkW * kStageBytes;
constexpr int kBlkCsOff = kBlkXOff + kBlkRows * kXqChunkRowBytes;
constexpr int kBlkStageBytes = kBlkCsOff + kBlkRows * kChunkBlocks * 4;
constexpr int kBlkBarOff = kBlkStages * kBlkStageBytes;
constexpr int kBlkCumOff = kBlkBarOff + 256;   // barriers: full[4], empty[4], then ready[8] and free[8] of the pairs
constexpr int kBlkMaxSlots = 320;         // slots of a launch (experts of a layer + the shared one)
constexpr int kBlkXchOff = kBlkCumOff + 2 * (kBlkMaxSlots + 1) * 4 + 64;   // up -> gate hand-over: [pair][nt][j][lane]
constexpr int kBlkMaxUnits = 1024;        // (slot, row block) units of a launch
constexpr int kBlkQueue = 8;              // item numbers in flight between producer and consumers
constexpr int kBlkQueueOff = kBlkXchOff + kBlkW * 4 * 4 * 32 * 4;
constexpr int kBlkUnitOff = kBlkQueueOff + kBlkQueue * 4 + 32;   // (queue, then the producers' item count)
constexpr int kBlkSmemBytes = kBlkUnitOff + kBlkMaxUnits * 4;

// Work items of a launch are handed out through one counter in device memory (first word: next item,
// second word: CTAs that have finished; the last one to finish clears both), so launches that use it
// must not overlap on a device.  Zero when the module is loaded.
__device__ unsigned g_blk_dyn[2];

struct BlkItem {
    int slot, tb, row0, nrows;  // rows [row0, row0 + nrows) of the slot: at most 32
    const uint8_t *a, *b;  // this warp's tile streams (nullptr: no tile for this warp)
    const float *a_rs, *b_rs;
    int tile;              // this warp's tile pair index
};

// One chunk of one item for one consumer warp (one 16-row tile): NT column groups of 8 rows.
// `wst` points at the tile's chunk in the stage.
template <int NT, bool GROUPED, int BPG>
__device__ __forceinline__ void blk_chunk(const uint8_t *wst, const uint8_t *xst, const uint8_t *cst, int g, int t,
                                          float (&acc)[4][4], int (&iacc)[4][4], float neg_zero) {
    constexpr int GPC = kChunkBlocks / BPG;
#pragma unroll
    for (int gi = 0; gi < GPC; ++gi) {
        int c[NT][4];
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
            const uint8_t *wp = wst + blk * kSlabBytes + t * 4;
            const uint32_t w0 = *reinterpret_cast<const uint32_t *>(wp + g * 16);
            const uint32_t w1 = *reinterpret_cast<const uint32_t *>(wp + (g + 8) * 16);
            const uint32_t a0 = w0 & 0x0F0F0F0Fu, a2 = (w0 >> 4) & 0x0F0F0F0Fu;
            const uint32_t a1 = w1 & 0x0F0F0F0Fu, a3 = (w1 >> 4) & 0x0F0F0F0Fu;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                // columns past the pass's rows read stale shared memory: their results are never stored
                const uint8_t *xr = xst + (8 * nt + g) * kXqChunkRowBytes + blk * 32 + 4 * t;
                const uint32_t b0 = *reinterpret_cast<const uint32_t *>(xr);
                const uint32_t b1 = *reinterpret_cast<const uint32_t *>(xr + 16);
                if (b == 0)
                    mma_u8s8_c(c[nt], a0, a1, a2, a3, b0, b1, cinit[nt][0], cinit[nt][1]);
                else
                    mma_u8s8(c[nt], a0, a1, a2, a3, b0, b1);
            }
        }
        if (GROUPED) {
            const float *sp = reinterpret_cast<const float *>(wst + kChunkSlabBytes);
            const float sc_lo = sp[g * GPC + gi], sc_hi = sp[(g + 8) * GPC + gi];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                fold_pair(acc[nt][0], acc[nt][1], c[nt][0], c[nt][1], sc_lo, kMagicF, neg_zero);
                fold_pair(acc[nt][2], acc[nt][3], c[nt][2], c[nt][3], sc_hi, kMagicF, neg_zero);
            }
        } else {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) iacc[nt][i] += c[nt][i];
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
    // Work is cut into units (slot, block of `rpp` rows) times tile blocks.  Smaller row blocks let several
    // CTAs share the tensor-core and fold work of an expert with many rows at the price of streaming its
    // weights once per block; whenever that made some CTA take a second item it cost more than it saved
    // (an expert-parallel rank with 7 experts: experts phase 151 us at 32 rows per unit, 162 at 16, 186 at
    // 8), so rpp is 32 unless every item of the finer cut still gets a CTA to itself.  Units are numbered
    // heaviest first (full units, then the ragged ends by falling row count) and handed out through a
    // counter: a CTA takes the next number when it has room in its ring, whatever the others hold.
    int *nrow_s = cum;                      // [n_slots] row counts
    int *units = reinterpret_cast<int *>(smem + kBlkUnitOff);   // [n_units] slot | first row << 16
    __shared__ int s_rpp, s_nfull, s_units, s_tbw;
    for (int s = tid; s < n_slots; s += blockDim.x) nrow_s[s] = P.slots[s].nrows;
    if (tid == 0) {
        for (int s = 0; s < kBlkStages; ++s) {
            mbar_init(full_b + s * 8, 1);
            mbar_init(empty_b + s * 8, kBlkCW);
        }
        for (int p = 0; p < 2 * kBlkW; ++p) mbar_init(full_b + 64 + p * 8, 1);
        reinterpret_cast<volatile int *>(smem + kBlkQueueOff)[kBlkQueue] = 0;  // items published so far
        fence_mbar_init();
        fence_proxy_async();
    }
    __syncthreads();
    if (warp == 0) {
        int u32 = 0, u16 = 0, u8 = 0;
        for (int s = lane; s < n_slots; s += 32) {
            const int nr = nrow_s[s];
            u32 += (nr + 31) >> 5;
            u16 += (nr + 15) >> 4;
            u8 += (nr + 7) >> 3;
        }
        for (int o = 16; o > 0; o >>= 1) {
            u32 += __shfl_xor_sync(0xffffffffu, u32, o);
            u16 += __shfl_xor_sync(0xffffffffu, u16, o);
            u8 += __shfl_xor_sync(0xffffffffu, u8, o);
        }
        // rows per unit: 32, unless the launch is so small that even with 16 (8) rows per unit every item
        // finds a CTA of its own at once: then the column groups of an expert with many rows run side by
        // side instead of one after the other inside one CTA (its weights come from L2 for all but one)
        int rpp = 32;
        if (P.blk_rpp == 8 || P.blk_rpp == 16 || P.blk_rpp == 32) {
            rpp = P.blk_rpp;
        } else {
            const int ntb8 = (P.warp_tiles + 7) / 8;
            if (u16 * ntb8 <= (int)gridDim.x) rpp = 16;
            if (u8 * ntb8 <= (int)gridDim.x) rpp = 8;
        }
        if (((rpp == 8) ? u8 : (rpp == 16 ? u16 : u32)) > kBlkMaxUnits) rpp = 32;  // (never at these batch sizes)
        // full units first, in slot order: an exclusive scan of nrows / rpp over the slots
        int base = 0;
        for (int s0 = 0; s0 < n_slots; s0 += 32) {
            const int s = s0 + lane;
            const int nf = s < n_slots ? nrow_s[s] / rpp : 0;
            int inc = nf;
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += v;
            }
            const int first = base + inc - nf;
            for (int p = 0; p < nf; ++p)
                if (first + p < kBlkMaxUnits) units[first + p] = s | ((p * rpp) << 16);
            base += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (lane == 0) {
            s_rpp = rpp;
            s_nfull = min(base, kBlkMaxUnits);
            // Tile pairs per item: 8 (all 16 consumer warps) unless the launch then has items for less
            // than half (a quarter) of the CTAs: with 4 (2) pairs per item twice (four times) as many
            // SMs share the work and no weight byte is fetched twice.  Not earlier: the consumer warps
            // are bound by their own instruction latencies, so an SM's rate falls with the warps it runs
            // (an expert-parallel rank with 112 items ran 10 % longer when they were cut into 224).
            const int units_n = (rpp == 8) ? u8 : (rpp == 16 ? u16 : u32);
            const int items8 = units_n * ((P.warp_tiles + 7) / 8);
            int tbw = kBlkW;
            if (2 * items8 <= (int)gridDim.x) tbw = 4;
            if (4 * items8 <= (int)gridDim.x) tbw = 2;
            s_tbw = tbw;
        }
    }
    __syncthreads();
    {
        const int rpp = s_rpp, nfull = s_nfull;
        for (int s = tid; s < n_slots; s += blockDim.x) {
            const int nr = nrow_s[s], rem = nr % rpp;
            if (rem > 0) {
                int rank = 0;
                for (int o = 0; o < n_slots; ++o) {
                    const int ro = nrow_s[o] % rpp;
                    rank += (ro > rem || (ro == rem && o < s)) ? 1 : 0;
                }
                if (nfull + rank < kBlkMaxUnits) units[nfull + rank] = s | ((nr - rem) << 16);
            }
        }
        if (warp == 0) {
            int n = 0;
            for (int s = lane; s < n_slots; s += 32) n += (nrow_s[s] % rpp) > 0 ? 1 : 0;
            for (int o = 16; o > 0; o >>= 1) n += __shfl_xor_sync(0xffffffffu, n, o);
            if (lane == 0) s_units = min(nfull + n, kBlkMaxUnits);
        }
    }
    __syncthreads();
    // (rows per unit, pairs per item and the item count stay in shared memory: they are needed once per
    // item, and the consumers' inner loop has no register to spare for them)
    __shared__ int s_ntb, s_total;
    if (tid == 0) {
        s_ntb = (P.warp_tiles + s_tbw - 1) / s_tbw;
        s_total = s_units * s_ntb;
    }
    __syncthreads();

    volatile int *queue = reinterpret_cast<volatile int *>(smem + kBlkQueueOff);
    auto decode = [&](int i, BlkItem &it, int w) {
        const int n_tb = s_ntb, tbw = s_tbw;
        const int u = i / n_tb;
        const int unit = units[u];
        const int slot = unit & 0xffff, r0 = unit >> 16;
        const GemvSlot *s = P.slots + slot;
        it.slot = slot;
        it.tb = i - u * n_tb;
        it.nrows = min(s_rpp, s->nrows - r0);
        it.row0 = s->row0 + r0;
        it.tile = it.tb * tbw + w;
        it.a = it.b = nullptr;
        it.a_rs = s->a_rs;
        it.b_rs = s->b_rs;
        if (w < tbw && it.tile < P.warp_tiles) {
            if (P.mode == 0) {
                it.a = s->a + (unsigned long long)it.tile * P.tile_bytes;
                it.b = s->b + (unsigned long long)it.tile * P.tile_bytes;
            } else {
                it.a = s->a + (unsigned long long)(2 * it.tile) * P.tile_bytes;
                it.b = (2 * it.tile + 1 < P.ntile) ? s->a + (unsigned long long)(2 * it.tile + 1) * P.tile_bytes : nullptr;
            }
        }
    };

    if (warp >= kBlkCW) {
        // ======================================================= producer warps
        // Issuing a bulk copy costs the issuing warp ~130 cycles, one copy after the other; one warp
        // issuing a stage's 18 copies took longer than the consumers needed for the stage.  So four
        // warps share them: producer p issues the chunks of tile pairs 2p and 2p + 1 (lanes 0-3: pair,
        // half), producer 0 also the item's activation rows and block sums, the byte count of the
        // stage and the item numbers (counter -> queue; `item_seq` tells the other producers how many
        // items have been published).
        const int p = warp - kBlkCW;
        volatile int *item_seq = queue + kBlkQueue;
        uint32_t q = 0;
        bool ok = true;
        for (int n = 0; ok; ++n) {
            int i = 0;
            if (p == 0) {
                if (lane == 0) {
                    i = (int)atomicAdd(&g_blk_dyn[0], 1u);
                    if (i >= s_total) i = -1;
                    queue[n % kBlkQueue] = i;  // the consumers read it once the item's first stage is full
                    __threadfence_block();
                    *item_seq = n + 1;
                }
            } else if (lane == 0) {
                const long long t0 = clock64();
                while (*item_seq <= n) {
                    if (clock64() - t0 > 2000000000LL) {
                        i = -2;
                        break;
                    }
                }
                __threadfence_block();
                if (i != -2) i = queue[n % kBlkQueue];
            }
            i = __shfl_sync(0xffffffffu, i, 0);
            if (i == -2) {
                if (lane == 0) report_error(P.err, kErrBarrierTimeout);
                break;
            }
            if (i < 0) {
                // end marker (producer 0): an empty stage whose queue entry is -1
                if (p == 0) {
                    const uint32_t stage = q % kBlkStages;
                    if (q >= kBlkStages) {
                        const bool fine = mbar_wait_bounded(empty_b + stage * 8, ((q / kBlkStages) + 1) & 1u);
                        if (__any_sync(0xffffffffu, !fine)) {
                            if (lane == 0) report_error(P.err, kErrBarrierTimeout);
                            break;
                        }
                    }
                    if (lane == 0) mbar_arrive(full_b + stage * 8);
                }
                break;
            }
            // producer 0: lane w < 8 looks at pair w for the stage's byte count; every producer: lanes 0-3
            // hold (pair 2p + lane / 2, half lane & 1)
            BlkItem it;
            int wbytes = 0;
            if (p == 0) {
                decode(i, it, lane < kBlkW ? lane : 0);
                wbytes = (lane < kBlkW && it.a) ? (it.b ? 2 : 1) * CHUNK_BYTES : 0;
                for (int o = 16; o > 0; o >>= 1) wbytes += __shfl_xor_sync(0xffffffffu, wbytes, o);
            }
            const int my_pair = 2 * p + ((lane & 3) >> 1);
            decode(i, it, my_pair);
            const uint8_t *my_src = (lane < 4) ? ((lane & 1) ? ((it.a != nullptr) ? it.b : nullptr) : it.a) : nullptr;
            const uint32_t my_dst = my_pair * kStageBytes + (lane & 1) * kChunkMaxBytes;
            for (int pc = 0; pc < P.nchunk; ++pc, ++q) {
                const int first = it.row0, nr = it.nrows;
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
                    // (copies of the other producers may land before this count is set: the phase cannot
                    // complete before this arrival)
                    if (p == 0) mbar_expect_tx(bar, wbytes + nr * (kXqChunkRowBytes + kChunkBlocks * 4));
                }
                __syncwarp();
                const size_t off = (size_t)pc * CHUNK_BYTES;
                if (my_src) bulk_g2s(dst + my_dst, my_src + off, CHUNK_BYTES, bar);
                if (p == 0) {
                    const long long cr = (long long)pc * P.pcap + first;
                    if (lane == 4)
                        bulk_g2s(dst + kBlkXOff, P.xq + cr * kXqChunkRowBytes, nr * kXqChunkRowBytes, bar);
                    else if (lane == 5)
                        bulk_g2s(dst + kBlkCsOff, P.csum + cr * kChunkBlocks, nr * kChunkBlocks * 4, bar);
                }
            }
        }
    } else {
    // =========================================================== consumer warps
    const int pair = warp >> 1, half = warp & 1;
    float *xch = reinterpret_cast<float *>(smem + kBlkXchOff) + pair * (4 * 4 * 32);
    const uint32_t ready_b = full_b + 64 + pair * 8, free_b = full_b + 64 + (kBlkW + pair) * 8;
    uint32_t q = 0, n_epi = 0;  // n_epi: hand-overs of this pair so far
    float acc[4][4];
    int iacc[4][4];
    bool ok = true;
    for (int n = 0; ok; ++n) {
        // the first stage of the next item (or the end marker) tells which item it is
        {
            const bool fine = mbar_wait_bounded(full_b + (q % kBlkStages) * 8, (q / kBlkStages) & 1u);
            if (__any_sync(0xffffffffu, !fine)) {
                if (lane == 0) report_error(P.err, kErrBarrierTimeout);
                break;
            }
        }
        const int i = queue[n % kBlkQueue];
        if (i < 0) break;
        bool first_stage = true;
        BlkItem it;
        decode(i, it, pair);
        // this warp's tile: gate / up tile of the pair (mode 0), down tiles 2t / 2t + 1 (mode 1)
        const bool have = half ? (it.a != nullptr && it.b != nullptr) : (it.a != nullptr);
        do {  // (one pass; `continue` leaves it)
            const int row0 = it.row0, nr = it.nrows;
            const int nt_n = (nr + 7) >> 3;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[nt][j] = 0.0f;
                    iacc[nt][j] = 0;
                }
            for (int chunk = 0; chunk < P.nchunk && ok; ++chunk, ++q) {
                const uint32_t stage = q % kBlkStages;
                if (!first_stage) {
                    const bool fine = mbar_wait_bounded(full_b + stage * 8, (q / kBlkStages) & 1u);
                    if (__any_sync(0xffffffffu, !fine)) {
                        if (lane == 0) report_error(P.err, kErrBarrierTimeout);
                        ok = false;
                        break;
                    }
                }
                first_stage = false;
                if (have) {
                    const uint8_t *st = smem + stage * kBlkStageBytes;
                    const uint8_t *wst = st + pair * kStageBytes + half * kChunkMaxBytes;
                    const uint8_t *xst = st + kBlkXOff, *cst = st + kBlkCsOff;
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
            if (!ok) continue;
            // ---- epilogue of the pass: activation scale, SwiGLU (mode 0), stores, row maxima
            auto value = [&](int nt, int j, int o) -> float {
                const int rr = min(8 * nt + 2 * t + (j & 1), nr - 1);
                const float sxa = P.sx[row0 + rr];
                if (GROUPED) return __fmul_rn(acc[nt][j], sxa);
                const float *rsp = (P.mode == 0 && half) ? it.b_rs : it.a_rs;
                const float rs = (o < P.ntile * 16) ? rsp[o] : 0.0f;
                return __fmul_rn(__fmul_rn((float)iacc[nt][j], rs), sxa);  // block corrections rode in the MMA start values
            };
            if (P.mode == 0) {
                // the up warp hands its values to the gate warp of the pair (bounded waits on both sides:
                // a warp that gave up leaves its partner to run out of patience, not to hang)
                if (half == 1) {
                    if (n_epi > 0) {
                        const bool fine = mbar_wait_bounded(free_b, (n_epi + 1) & 1u);
                        if (__any_sync(0xffffffffu, !fine)) {
                            if (lane == 0) report_error(P.err, kErrBarrierTimeout);
                            ok = false;
                            continue;
                        }
                    }
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt) {
                        if (nt >= nt_n) break;
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            xch[(nt * 4 + j) * 32 + lane] = have ? value(nt, j, it.tile * 16 + g + 8 * (j >> 1)) : 0.0f;
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(ready_b);
                } else {
                    const bool fine = mbar_wait_bounded(ready_b, n_epi & 1u);
                    if (__any_sync(0xffffffffu, !fine)) {
                        if (lane == 0) report_error(P.err, kErrBarrierTimeout);
                        ok = false;
                        continue;
                    }
                }
                ++n_epi;
                if (half == 0 && have) {
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt) {
                        if (nt >= nt_n) break;
                        float amax2[2] = {0.0f, 0.0f};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int ridx = 8 * nt + 2 * t + (j & 1);
                            const int o = it.tile * 16 + g + 8 * (j >> 1);
                            const float vg = value(nt, j, o), vu = xch[(nt * 4 + j) * 32 + lane];
                            if (ridx < nr && o < P.O) {
                                const float hval = __fmul_rn(silu32(vg), vu);
                                P.out[(long long)(row0 + ridx) * P.out_stride + o] = hval;
                                const float a = fabsf(hval);
                                if (a == a) amax2[j & 1] = fmaxf(amax2[j & 1], a);  // NaN never becomes the maximum
                            }
                        }
                        if (P.amax_out != nullptr) {
                            // row maxima of |h|: reduce over the 8 lanes that share this lane's two columns
#pragma unroll
                            for (int j = 0; j < 2; ++j) {
                                float a = amax2[j];
                                a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 4));
                                a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 8));
                                a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 16));
                                const int ridx = 8 * nt + 2 * t + j;
                                if (g == 0 && ridx < nr && a > 0.0f)
                                    atomicMax(P.amax_out + row0 + ridx, __float_as_uint(a));
                            }
                        }
                    }
                }
                if (half == 0) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(free_b);  // the hand-over area is free again
                }
            } else if (have) {
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    if (nt >= nt_n) break;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int ridx = 8 * nt + 2 * t + (j & 1);
                        const int o = (2 * it.tile + half) * 16 + g + 8 * (j >> 1);
                        const float v = value(nt, j, o);
                        if (ridx < nr && o < P.O) P.out[(long long)(row0 + ridx) * P.out_stride + o] = v;
                    }
                }
            }
        } while (false);
    }
    }
    // every CTA passes here, also after a failed wait: the last one re-arms the counter
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(&g_blk_dyn[1], 1u) == gridDim.x - 1) {
            g_blk_dyn[0] = 0u;
            g_blk_dyn[1] = 0u;
            __threadfence();
        }
    }
}

}  // namespace pgb