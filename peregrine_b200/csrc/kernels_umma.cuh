// Large-batch int4 x int8 expert matmul on the fifth-generation tensor cores (tcgen05.mma
// kind::i8, accumulators in tensor memory).  Tile, stream format and numerics are those of
// ffn_w4a8_tile_kernel (kernels_tile.cuh); what changes is who does the integer work:
//
//   warp 2          bulk copies (packed weight chunks, activation block, block sums), one per lane,
//                   into a 3-stage ring
//   warps 0, 1      each expands the packed nibbles of one half of every chunk into int8 rows laid
//                   out as 8x16-byte core matrices (byte p of a packed segment holds elements p and
//                   16+p, which are exactly the two 16-byte K halves of one MMA); warp 0 also
//                   transposes the chunk's scales
//   warp 3 lane 0   issues one 128 x 128 x 32 MMA per 32-element block: M = 128 activation rows
//                   (A, s8, copied from global memory already in core-matrix order), N = 64 gate +
//                   64 up weight rows (B, u8 = stored nibble)
//   warps 4-11      own one activation row each (TMEM lane) and 64 of the 128 columns: after every
//                   scale group they drain the group's int32 dots and fold them into fp32
//                   accumulators in reference order (crates/peregrine-kernels/src/idot.rs:98-110,
//                   matmul.rs:93-106), then run the SwiGLU / scale epilogue
//
// Exact int -> float without a conversion: the fold warps preset the TMEM accumulator to the
// bit pattern of 1.5 * 2^23, the tensor core adds the integer dot to it, and the drained word
// read as a float is 12582912 + dot; subtracting 12582912 + 8 * sum(q) (one constant per
// activation row and group) gives (float)(dot - 8 * sum(q)) exactly.
//
// Every wait is bounded; a wait that runs out sets the device error word and a CTA-wide flag that
// all roles poll, and every path reaches the common tail that frees the tensor memory.
#pragma once
#include "kernels_tile.cuh"

namespace pgb {

constexpr int kUmThreads = 384;
constexpr int kUmTok = 128;
constexpr int kUmStages = 3;
constexpr int kUmXOff = 8 * kChunkMaxBytes;                    // activations [16 k16][128 rows][16 B]
constexpr int kUmCsOff = kUmXOff + 16 * kUmTok * 16;           // block sums [128 rows][8]
constexpr int kUmScOff = kUmCsOff + kUmTok * kChunkBlocks * 4; // transposed scales [8 groups][128 cols]
constexpr int kUmStageBytes = kUmScOff + kChunkBlocks * 128 * 4;
constexpr int kUmBOff = kUmStages * kUmStageBytes;             // expanded weights: 2 x [8 k16][128 rows][16 B]
constexpr int kUmBHalfBytes = 8 * 128 * 16;
constexpr int kUmBarOff = kUmBOff + 2 * kUmBHalfBytes;
constexpr int kUmSmemBytes = kUmBarOff + 256;
// instruction descriptor: D = s32, A = s8, B = u8, both K-major, N = 128, M = 128
constexpr uint32_t kUmIdesc = (2u << 4) | (1u << 7) | (0u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    // K-major, no swizzle: 8 rows x 16 bytes per core matrix; LBO = distance between the two
    // 16-byte K halves, SBO = distance between 8-row groups; bit 46 = descriptor version 1
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) |
           ((uint64_t)(sbo_bytes >> 4) << 32) | (1ull << 46);
}
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, int (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
// store one value to 32 consecutive columns of this thread's lane
__device__ __forceinline__ void tmem_fill32(uint32_t taddr, int v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, "
        "%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};" ::"r"(taddr),
        "r"(v)
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// try_wait that lets the hardware park the thread for up to `ns` nanoseconds instead of
// returning at once: the waiting roles of this kernel share their schedulers with the fold warps
// and must not spend issue slots on polling
__device__ __forceinline__ uint32_t mbar_try_wait_park(uint32_t bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(ns)
        : "memory");
    return ok;
}

// fold_pair (kernels_mma.cuh) for two neighbouring columns of one activation row: the columns are
// different weight rows, so each has its own scale; the subtrahend is the row's constant.
__device__ __forceinline__ void fold_pair2(float &a0, float &a1, int c0, int c1, float s0, float s1, float K,
                                           float nz) {
    asm("{\n\t.reg .b64 cc, kk, ss, aa, ff, pp, zz;\n\t"
        "mov.b64 cc, {%2, %3};\n\tmov.b64 kk, {%6, %6};\n\tmov.b64 ss, {%4, %5};\n\t"
        "mov.b64 aa, {%0, %1};\n\tmov.b64 zz, {%7, %7};\n\t"
        "sub.rn.f32x2 ff, cc, kk;\n\tfma.rn.f32x2 pp, ff, ss, zz;\n\tadd.rn.f32x2 aa, aa, pp;\n\t"
        "mov.b64 {%0, %1}, aa;\n\t}"
        : "+f"(a0), "+f"(a1)
        : "r"(c0), "r"(c1), "f"(s0), "f"(s1), "f"(K), "f"(nz));
}

// bounded wait that also gives up when another role has already failed
__device__ __forceinline__ bool um_wait(uint32_t bar, uint32_t parity, volatile int *fail) {
    const long long t0 = clock64();
    while (!mbar_try_wait_park(bar, parity, 20000u)) {
        if (*fail) return false;
        if (clock64() - t0 > 2000000000LL) {
            *fail = 1;
            return false;
        }
    }
    return true;
}

// grid as ffn_w4a8_tile_kernel: x = block of weight rows (64 gate + 64 up rows, or 128 down rows),
// y = row block.  Activations: P.xq in core-matrix order [chunk][16][pcap][16 B]
// (qrow_i8_kernel with a negative capacity), P.csum [chunk][pcap][8], P.sx per pair row.
template <bool GROUPED, int BPG>
__global__ void __launch_bounds__(kUmThreads, 1) ffn_w4a8_umma_kernel(const GemvParams P) {
    constexpr int GPC = kChunkBlocks / BPG;
    constexpr int CHUNK_BYTES = kChunkSlabBytes + (GROUPED ? GPC * 64 : 0);
    constexpr int NACC = GROUPED ? 2 : 1;  // TMEM accumulator buffers of 128 columns
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int s_slot, s_first, s_per, s_fail;
    __shared__ uint32_t s_tmem;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t smem_u = smem_u32(smem);
    const uint32_t bar0 = smem_u + kUmBarOff;
    const uint32_t full_b = bar0, empty_b = bar0 + 24, bfree_b = bar0 + 48, accf_b = bar0 + 64, acce_b = bar0 + 80,
                   bready_b = bar0 + 96;

    // ---- row block of this CTA (same dealing of rows to blocks as ffn_w4a8_tile_kernel)
    const int n_slots = *P.n_slots;
    if (warp == 0) {
        int base = 0, found = -1, first = 0, per = kUmTok;
        for (int j0 = 0; j0 < n_slots && found < 0; j0 += 32) {
            const int j = j0 + lane;
            const int nrj = j < n_slots ? P.slots[j].nrows : 0;
            const int nb = (nrj + kUmTok - 1) / kUmTok;
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
            s_fail = 0;
            for (int s = 0; s < kUmStages; ++s) {
                mbar_init(full_b + s * 8, 1);
                // released by the MMA commit and, for grouped formats, by the eight fold warps
                mbar_init(empty_b + s * 8, 1 + 8);
            }
            for (int s = 0; s < 2; ++s) {
                mbar_init(bfree_b + s * 8, 1);
                mbar_init(accf_b + s * 8, 1);
                mbar_init(acce_b + s * 8, 8);
                mbar_init(bready_b + s * 8, 1);
            }
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
    const int prow0 = slot.row0 + first;
    const int ob = blockIdx.x;
    volatile int *fail = &s_fail;

    // ---- tensor memory: NACC x 128 columns, allocated (and later freed) by warp 3
    if (warp == 3) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)),
                     "r"((uint32_t)(NACC * 128))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tmem_fence_before();
    __syncthreads();
    tmem_fence_after();
    const uint32_t tmem = s_tmem;

    if (warp == 2) {
        // =============================================== loader: one bulk copy per lane
        const int s = lane - 16;  // lanes 16-23: weight tiles; lanes 0-15: activation units; lane 24: block sums
        const uint8_t *wsrc = nullptr;
        if (s >= 0 && s < 8) {
            const int half = s >> 2, i = s & 3;
            const int tile = (P.mode == 0) ? ob * 4 + i : ob * 8 + s;
            const uint8_t *mat = (P.mode == 0 && half) ? slot.b : slot.a;
            if (tile < P.ntile) wsrc = mat + (unsigned long long)tile * P.tile_bytes;
        }
        const int n_wt = __popc(__ballot_sync(0xffffffffu, wsrc != nullptr));
        for (int chunk = 0; chunk < P.nchunk; ++chunk) {
            const int stage = chunk % kUmStages;
            if (chunk >= kUmStages &&
                !__all_sync(0xffffffffu, um_wait(empty_b + stage * 8, ((chunk / kUmStages) + 1) & 1u, fail)))
                break;
            const uint32_t bar = full_b + stage * 8;
            const uint32_t dst = smem_u + stage * kUmStageBytes;
            if (lane == 0) {
                fence_proxy_async();
                mbar_expect_tx(bar, n_wt * CHUNK_BYTES + nr * (256 + kChunkBlocks * 4));
            }
            __syncwarp();
            if (lane < 16)
                bulk_g2s(dst + kUmXOff + lane * (kUmTok * 16),
                         P.xq + (((long long)chunk * 16 + lane) * P.pcap + prow0) * 16, nr * 16, bar);
            else if (wsrc)
                bulk_g2s(dst + s * kChunkMaxBytes, wsrc + (size_t)chunk * CHUNK_BYTES, CHUNK_BYTES, bar);
            else if (lane == 24)
                bulk_g2s(dst + kUmCsOff, P.csum + ((long long)chunk * P.pcap + prow0) * kChunkBlocks,
                         nr * kChunkBlocks * 4, bar);
        }
    } else if (warp < 2) {
        // =============================================== expander of half `warp` of every chunk
        const int hh = warp;
        uint8_t *bb = smem + kUmBOff + hh * kUmBHalfBytes;
        for (int chunk = 0; chunk < P.nchunk; ++chunk) {
            const int stage = chunk % kUmStages;
            if (!__all_sync(0xffffffffu, um_wait(full_b + stage * 8, (chunk / kUmStages) & 1u, fail))) break;
            const uint8_t *st = smem + stage * kUmStageBytes;
            if (GROUPED && hh == 0) {
                // scales of the chunk, transposed to [group][column] for the fold warps
                float *dstp = reinterpret_cast<float *>(const_cast<uint8_t *>(st) + kUmScOff);
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    const int col = cc * 32 + lane;
                    const float *sp =
                        reinterpret_cast<const float *>(st + (col >> 4) * kChunkMaxBytes + kChunkSlabBytes) + (col & 15) * GPC;
#pragma unroll
                    for (int gi = 0; gi < GPC; ++gi) dstp[gi * 128 + col] = sp[gi];
                }
            }
            // this buffer was last read by the MMAs of the previous chunk
            if (chunk >= 1 && !__all_sync(0xffffffffu, um_wait(bfree_b + hh * 8, (chunk + 1) & 1u, fail))) break;
#pragma unroll 4
            for (int it = 0; it < 16; ++it) {
                const int idx = it * 32 + lane;
                const int row = idx & 15, tile = (idx >> 4) & 7, bq = idx >> 7;
                const uint4 w = *reinterpret_cast<const uint4 *>(st + tile * kChunkMaxBytes + (4 * hh + bq) * kSlabBytes + row * 16);
                uint4 lo, hi;
                lo.x = w.x & 0x0F0F0F0Fu, lo.y = w.y & 0x0F0F0F0Fu, lo.z = w.z & 0x0F0F0F0Fu, lo.w = w.w & 0x0F0F0F0Fu;
                hi.x = (w.x >> 4) & 0x0F0F0F0Fu, hi.y = (w.y >> 4) & 0x0F0F0F0Fu;
                hi.z = (w.z >> 4) & 0x0F0F0F0Fu, hi.w = (w.w >> 4) & 0x0F0F0F0Fu;
                uint8_t *d = bb + (2 * bq) * 2048 + (tile * 16 + row) * 16;
                *reinterpret_cast<uint4 *>(d) = lo;
                *reinterpret_cast<uint4 *>(d + 2048) = hi;
            }
            fence_proxy_async();  // the expanded rows are read by the tensor core (async proxy)
            __syncwarp();
            if (lane == 0) mbar_arrive(bready_b + hh * 8);
        }
    } else if (warp == 3) {
        // =============================================== MMA issuer (one lane)
        if (lane == 0) {
            uint32_t group_no = 0;
            bool ok = true;
            for (int chunk = 0; chunk < P.nchunk && ok; ++chunk) {
                const int stage = chunk % kUmStages;
                ok = um_wait(full_b + stage * 8, (chunk / kUmStages) & 1u, fail);
                for (int hh = 0; hh < 2 && ok; ++hh) {
                    ok = um_wait(bready_b + hh * 8, chunk & 1u, fail);
                    if (!ok) break;
                    tmem_fence_after();
                    for (int j = 0; j < 4 && ok; ++j) {
                        const int blk = 4 * hh + j;
                        const uint64_t ad = umma_desc(smem_u + stage * kUmStageBytes + kUmXOff + (2 * blk) * 2048, 2048, 128);
                        const uint64_t bd = umma_desc(smem_u + kUmBOff + hh * kUmBHalfBytes + (2 * j) * 2048, 2048, 128);
                        if (GROUPED) {
                            const uint32_t ab = group_no & 1u;
                            if (blk % BPG == 0) {
                                ok = um_wait(acce_b + ab * 8, (group_no >> 1) & 1u, fail);
                                if (!ok) break;
                                tmem_fence_after();
                            }
                            umma_i8(tmem + ab * 128, ad, bd, kUmIdesc, 1u);  // adds to the preset accumulator
                            if (blk % BPG == BPG - 1) {
                                umma_commit(accf_b + ab * 8);
                                ++group_no;
                            }
                        } else {
                            umma_i8(tmem, ad, bd, kUmIdesc, (chunk > 0 || blk > 0) ? 1u : 0u);
                        }
                    }
                    umma_commit(bfree_b + hh * 8);
                    if (hh == 1) {
                        umma_commit(empty_b + stage * 8);
                        if (!GROUPED && chunk == P.nchunk - 1) umma_commit(accf_b);
                    }
                }
            }
        }
        __syncwarp();
    } else {
        // =============================================== fold / epilogue warps
        const int q = warp & 3, hf = (warp - 4) >> 2;
        const int row = 32 * q + lane;                       // activation row inside the block = TMEM lane
        const uint32_t tlane = tmem + ((uint32_t)(32 * q) << 16);
        const bool valid = row < nr;
        float acc[64];
        int csacc = 0;
#pragma unroll
        for (int i = 0; i < 64; ++i) acc[i] = 0.0f;
        if (GROUPED) {
            // preset both accumulator buffers, then hand them to the MMA issuer
#pragma unroll
            for (int ab = 0; ab < 2; ++ab) {
                tmem_fill32(tlane + ab * 128 + 32 * hf, (int)kMagicBits);
                tmem_fill32(tlane + ab * 128 + 64 + 32 * hf, (int)kMagicBits);
            }
            tmem_wait_st();
            tmem_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(acce_b);
                mbar_arrive(acce_b + 8);
            }
        }
        uint32_t group_no = 0;
        bool ok = true;
        for (int chunk = 0; chunk < P.nchunk && ok; ++chunk) {
            const int stage = chunk % kUmStages;
            ok = __all_sync(0xffffffffu, um_wait(full_b + stage * 8, (chunk / kUmStages) & 1u, fail));
            if (!ok) break;
            const uint8_t *st = smem + stage * kUmStageBytes;
            const int4 c0 = *reinterpret_cast<const int4 *>(st + kUmCsOff + row * 32);
            const int4 c1 = *reinterpret_cast<const int4 *>(st + kUmCsOff + row * 32 + 16);
            const int cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
            if (GROUPED) {
                const float *scT = reinterpret_cast<const float *>(st + kUmScOff);
#pragma unroll 1
                for (int gi = 0; gi < GPC; ++gi) {
                    int csum_g = 0;
#pragma unroll
                    for (int b = 0; b < BPG; ++b) csum_g += cs[(gi * BPG + b) & 7];
                    const float sub = kMagicF - (float)csum_g;
                    const uint32_t ab = group_no & 1u;
                    ok = __all_sync(0xffffffffu, um_wait(accf_b + ab * 8, (group_no >> 1) & 1u, fail));
                    if (!ok) break;
                    tmem_fence_after();
                    int d0[32], d1[32];
                    tmem_ld32(tlane + ab * 128 + 32 * hf, d0);
                    tmem_ld32(tlane + ab * 128 + 64 + 32 * hf, d1);
                    tmem_wait_ld();
                    tmem_fill32(tlane + ab * 128 + 32 * hf, (int)kMagicBits);
                    tmem_fill32(tlane + ab * 128 + 64 + 32 * hf, (int)kMagicBits);
                    tmem_wait_st();
                    tmem_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acce_b + ab * 8);
                    ++group_no;
                    const float4 *s0 = reinterpret_cast<const float4 *>(scT + gi * 128 + 32 * hf);
                    const float4 *s1 = reinterpret_cast<const float4 *>(scT + gi * 128 + 64 + 32 * hf);
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        const float4 a = s0[v], b = s1[v];
                        fold_pair2(acc[4 * v + 0], acc[4 * v + 1], d0[4 * v + 0], d0[4 * v + 1], a.x, a.y, sub, P.neg_zero);
                        fold_pair2(acc[4 * v + 2], acc[4 * v + 3], d0[4 * v + 2], d0[4 * v + 3], a.z, a.w, sub, P.neg_zero);
                        fold_pair2(acc[32 + 4 * v + 0], acc[32 + 4 * v + 1], d1[4 * v + 0], d1[4 * v + 1], b.x, b.y, sub, P.neg_zero);
                        fold_pair2(acc[32 + 4 * v + 2], acc[32 + 4 * v + 3], d1[4 * v + 2], d1[4 * v + 3], b.z, b.w, sub, P.neg_zero);
                    }
                }
            } else {
#pragma unroll
                for (int b = 0; b < 8; ++b) csacc += cs[b];
            }
            // this warp is done with the stage's block sums and scales
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_b + stage * 8);
        }
        int dint[64];
        if (!GROUPED && ok) {
            ok = __all_sync(0xffffffffu, um_wait(accf_b, 0u, fail));
            if (ok) {
                tmem_fence_after();
                int d0[32], d1[32];
                tmem_ld32(tlane + 32 * hf, d0);
                tmem_ld32(tlane + 64 + 32 * hf, d1);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    dint[i] = d0[i] + csacc;
                    dint[32 + i] = d1[i] + csacc;
                }
            }
        }
        if (ok) {
            // ---- epilogue: acc[0..31] = columns 32*hf.., acc[32..63] = columns 64 + 32*hf..
            const float sxa = P.sx[prow0 + (valid ? row : 0)];
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                float v[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int c = h * 64 + 32 * hf + i;  // column of the MMA = weight row inside the block
                    if (GROUPED) {
                        v[h] = __fmul_rn(acc[h * 32 + i], sxa);
                    } else {
                        const int tile = (P.mode == 0) ? ob * 4 + ((c & 63) >> 4) : ob * 8 + (c >> 4);
                        const float *rsp = (P.mode == 0 && h) ? slot.b_rs : slot.a_rs;
                        const float rs = (tile < P.ntile) ? rsp[tile * 16 + (c & 15)] : 0.0f;
                        v[h] = __fmul_rn(__fmul_rn((float)dint[h * 32 + i], rs), sxa);
                    }
                }
                if (P.mode == 0) {
                    const int o = ob * 64 + 32 * hf + i;
                    if (valid && o < P.O) {
                        const float hval = __fmul_rn(silu32(v[0]), v[1]);
                        P.out[(long long)(prow0 + row) * P.out_stride + o] = hval;
                        const float a = fabsf(hval);
                        if (a == a) amax = fmaxf(amax, a);
                    }
                } else {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int o = ob * 128 + h * 64 + 32 * hf + i;
                        if (valid && o < P.O) P.out[(long long)(prow0 + row) * P.out_stride + o] = v[h];
                    }
                }
            }
            if (P.mode == 0 && P.amax_out != nullptr && valid && amax > 0.0f)
                atomicMax(P.amax_out + prow0 + row, __float_as_uint(amax));
        }
    }
    // ---- common tail: wait for the tensor core to go quiet, then free the tensor memory
    if (*fail && tid == 0) report_error(P.err, kErrBarrierTimeout);
    if (*fail && tid == 96) {
        // MMAs may still be running: a commit on a barrier of its own arrives when they are done
        const uint32_t drain_b = bar0 + 112;
        mbar_init(drain_b, 1);
        fence_mbar_init();
        umma_commit(drain_b);
        const long long t0 = clock64();
        while (!mbar_try_wait(drain_b, 0u))
            if (clock64() - t0 > 2000000000LL) break;
    }
    tmem_fence_before();
    __syncthreads();
    if (warp == 3) {
        tmem_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)(NACC * 128))
                     : "memory");
    }
}

// ---------------------------------------------------------------- int8 tensor peak probe
// The denominator of the prefill roofline, measured instead of quoted: one CTA per SM issues
// `iters` back-to-back 128 x 256 x 32 tcgen05.mma kind::i8 (s8 x u8 -> s32) on operands that stay
// in shared memory, alternating between two 256-column accumulators in tensor memory; nothing else
// runs.  ops = iters * 2 * 128 * 256 * 32 per CTA.
constexpr int kPeakABytes = 2 * 128 * 16, kPeakBBytes = 2 * 256 * 16;
constexpr uint32_t kPeakIdesc = (2u << 4) | (1u << 7) | (0u << 10) | ((256u >> 3) << 17) | ((128u >> 4) << 24);
__global__ void __launch_bounds__(128, 1) int8_peak_probe_kernel(int iters, int *err) {
    __shared__ __align__(128) uint8_t ops[kPeakABytes + kPeakBBytes];
    __shared__ __align__(8) unsigned long long bar;
    __shared__ uint32_t s_tmem;
    const int tid = threadIdx.x, warp = tid >> 5;
    for (int i = tid; i < kPeakABytes + kPeakBBytes; i += blockDim.x)
        ops[i] = i < kPeakABytes ? (uint8_t)(int8_t)(((i * 37 + 11) % 7) - 3) : (uint8_t)((i * 29 + 5) & 15);
    const uint32_t b = smem_u32(&bar);
    if (tid == 0) {
        mbar_init(b, 1);
        fence_mbar_init();
    }
    fence_proxy_async();  // operands written by threads, read by the tensor core
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)),
                     "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tmem_fence_before();
    __syncthreads();
    tmem_fence_after();
    const uint32_t tmem = s_tmem;
    if (tid == 0) {
        const uint64_t adesc = umma_desc(smem_u32(ops), 128 * 16, 128);
        const uint64_t bdesc = umma_desc(smem_u32(ops + kPeakABytes), 256 * 16, 128);
        for (int i = 0; i < iters; ++i) umma_i8(tmem + (i & 1) * 256, adesc, bdesc, kPeakIdesc, i >= 2 ? 1u : 0u);
        umma_commit(b);
        const long long t0 = clock64();
        while (!mbar_try_wait_park(b, 0u, 20000u))
            if (clock64() - t0 > 20000000000LL) {
                report_error(err, kErrBarrierTimeout);
                break;
            }
        tmem_fence_after();
    }
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
}

}  // namespace pgb
