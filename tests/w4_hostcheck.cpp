// Host-only mirror of the device-side walk over a tile stream.  Built into a
// separate helper library that the CPU test-suite loads: it lets the stream
// layout, the repacker and the per-lane integer arithmetic of the GEMV kernel
// (mask split, 16x upper half, -8*sum correction, group fold order) be checked
// against the oracle on a machine without a GPU.  Never linked into the backend.
#include <cmath>
#include <cstring>
#include <vector>

#include "w4_host.h"

using namespace pgb;

#define HC_API extern "C" __attribute__((visibility("default")))

static inline int dp4a_us(uint32_t a, uint32_t b, int c) {
    for (int i = 0; i < 4; ++i) c += (int)((a >> (8 * i)) & 0xFF) * (int)(int8_t)((b >> (8 * i)) & 0xFF);
    return c;
}

// out[0..13] = fields of W4Layout in declaration order (size_t fields as two ints)
HC_API int pgb_hc_layout(int O, int K, int grouped, int gs, long long *out) {
    W4Layout L;
    if (!w4_layout_make(&L, O, K, grouped, gs)) return 0;
    long long v[] = {L.O,    L.K,     L.grouped,     L.gs,  L.bpg,    L.ng_src,
                     L.nblk, L.ntile, L.chunk_bytes, L.gpc, L.nchunk, L.kp,
                     (long long)L.tile_bytes, (long long)L.total_bytes};
    std::memcpy(out, v, sizeof(v));
    return 1;
}

HC_API int pgb_hc_repack(const uint8_t *q, const float *scales, int O, int K, int grouped, int gs, uint8_t *stream,
                         float *row_scales, int threads) {
    W4Layout L;
    if (!w4_layout_make(&L, O, K, grouped, gs)) return 0;
    w4_repack(L, q, scales, stream, row_scales, threads);
    return 1;
}

HC_API int pgb_hc_nibble(const uint8_t *stream, int O, int K, int grouped, int gs, int o, int k) {
    W4Layout L;
    if (!w4_layout_make(&L, O, K, grouped, gs)) return -1;
    return w4_stream_nibble(L, stream, o, k);
}

// The activation side as qrow_i8_kernel produces it: int8 row padded to kp, scale, -8*sum per block.
HC_API void pgb_hc_qrow(const float *x, int K, int kp, int nblk, int8_t *xq, float *sx, int *csum) {
    float amax = 0.0f;
    for (int i = 0; i < K; ++i) {
        float a = std::fabs(x[i]);
        if (a > amax) amax = a;
    }
    float s = amax / 127.0f;
    if (s < 1e-12f) s = 1e-12f;
    *sx = s;
    const float inv = 1.0f / s;
    for (int b = 0; b < nblk; ++b) {
        int sum = 0;
        for (int l = 0; l < 32; ++l) {
            const int i = b * 32 + l;
            int q = 0;
            if (i < K) {
                q = (int)std::nearbyintf(x[i] * inv);
                q = q < -128 ? -128 : (q > 127 ? 127 : q);
            }
            xq[i] = (int8_t)q;
            sum += q;
        }
        csum[b] = -8 * sum;
    }
    (void)kp;
}

// y[r, o] for nrows activation rows against one matrix, walking the stream chunk
// by chunk the way one half-warp of gemv_w4a8_kernel does (mode 1 addressing).
// tap (may be NULL): [nrows][O][ng_src] per-group int32 (grouped) or [nrows][O] (per-row).
HC_API int pgb_hc_walk(const uint8_t *stream, const float *row_scales, int O, int K, int grouped, int gs,
                       const int8_t *xq, const int *csum, const float *sx, int nrows, float *y, int *tap) {
    W4Layout L;
    if (!w4_layout_make(&L, O, K, grouped, gs)) return 0;
    const int GPC = L.gpc, BPG = L.bpg;
    for (int tile = 0; tile < L.ntile; ++tile) {
        const uint8_t *tbase = stream + (size_t)tile * L.tile_bytes;
        for (int r16 = 0; r16 < kTileRows; ++r16) {
            const int o = tile * kTileRows + r16;
            for (int r = 0; r < nrows; ++r) {
                float acc = 0.0f;
                int iacc = 0;
                for (int chunk = 0; chunk < L.nchunk; ++chunk) {
                    const uint8_t *wp = tbase + (size_t)chunk * L.chunk_bytes + r16 * 16;
                    const float *sp = reinterpret_cast<const float *>(tbase + (size_t)chunk * L.chunk_bytes +
                                                                      kChunkSlabBytes) + r16 * GPC;
                    const int8_t *xr = xq + (size_t)r * L.kp + chunk * kChunkElems;
                    const int *cp = csum + (size_t)r * L.nblk + chunk * kChunkBlocks;
                    for (int gi = 0; gi < GPC; ++gi) {
                        int dsum = 0;
                        for (int b = 0; b < BPG; ++b) {
                            const int blk = gi * BPG + b;
                            uint32_t w[4], x0[4], x1[4];
                            std::memcpy(w, wp + blk * kSlabBytes, 16);
                            std::memcpy(x0, xr + blk * 32, 16);
                            std::memcpy(x1, xr + blk * 32 + 16, 16);
                            int lo = cp[blk], hi = 0;
                            for (int j = 0; j < 4; ++j) {
                                lo = dp4a_us(w[j] & 0x0F0F0F0Fu, x0[j], lo);
                                hi = dp4a_us(w[j] & 0xF0F0F0F0u, x1[j], hi);
                            }
                            dsum += lo + (hi >> 4);
                        }
                        if (L.grouped) {
                            float sc;
                            std::memcpy(&sc, sp + gi, 4);
                            acc = acc + sc * (float)dsum;
                            const int g = chunk * GPC + gi;
                            if (tap && o < O && g < L.ng_src) tap[((size_t)r * O + o) * L.ng_src + g] = dsum;
                        } else {
                            iacc += dsum;
                        }
                    }
                }
                if (o >= O) continue;
                if (L.grouped) {
                    y[(size_t)r * O + o] = acc * sx[r];
                } else {
                    if (tap) tap[(size_t)r * O + o] = iacc;
                    y[(size_t)r * O + o] = (float)iacc * row_scales[o] * sx[r];
                }
            }
        }
    }
    return 1;
}
