#include "w4_host.h"

#include <algorithm>
#include <cstring>
#include <thread>
#include <vector>
#if defined(__SSE2__)
#include <emmintrin.h>
#endif

namespace pgb {

static inline uint8_t src_nibble(const uint8_t *q, size_t row_bytes, int O, int K, int o, int k) {
    if (o >= O || k >= K) return 8;  // stored 8 == value 0
    uint8_t byte = q[(size_t)o * row_bytes + (size_t)(k >> 1)];
    return (k & 1) ? (uint8_t)(byte >> 4) : (uint8_t)(byte & 0x0F);
}

// 16 source bytes (elements 0..31 as (even, odd) nibble pairs) -> 16 stream bytes
// (byte p = elem[p] | elem[16+p] << 4).
static inline void repack_block16(const uint8_t *src, uint8_t *dst) {
#if defined(__SSE2__)
    const __m128i m = _mm_set1_epi8(0x0F);
    const __m128i v = _mm_loadu_si128(reinterpret_cast<const __m128i *>(src));
    const __m128i even = _mm_and_si128(v, m);                     // elements 0,2,4,...,30
    const __m128i odd = _mm_and_si128(_mm_srli_epi16(v, 4), m);   // elements 1,3,5,...,31
    // low 8 bytes = first half (elements 0..15), high 8 bytes = second half (16..31)
    const __m128i e = _mm_or_si128(even, _mm_slli_epi16(_mm_srli_si128(even, 8), 4));
    const __m128i o = _mm_or_si128(odd, _mm_slli_epi16(_mm_srli_si128(odd, 8), 4));
    _mm_storeu_si128(reinterpret_cast<__m128i *>(dst), _mm_unpacklo_epi8(e, o));
#else
    for (int p = 0; p < 16; ++p) {
        uint8_t lo = (p & 1) ? (uint8_t)(src[p >> 1] >> 4) : (uint8_t)(src[p >> 1] & 0x0F);
        uint8_t hi = (p & 1) ? (uint8_t)(src[8 + (p >> 1)] >> 4) : (uint8_t)(src[8 + (p >> 1)] & 0x0F);
        dst[p] = (uint8_t)(lo | (hi << 4));
    }
#endif
}

static void repack_tiles(const W4Layout &L, const uint8_t *q, const float *scales, uint8_t *stream, int t0, int t1) {
    const size_t row_bytes = (size_t)(L.K + 1) / 2;
    for (int t = t0; t < t1; ++t) {
        uint8_t *tile = stream + (size_t)t * L.tile_bytes;
        for (int blk = 0; blk < L.nblk; ++blk) {
            const int k0 = blk * kBlockElems;
            for (int r = 0; r < kTileRows; ++r) {
                const int o = t * kTileRows + r;
                uint8_t *dst = tile + w4_seg_offset(L, blk, r);
                if (o < L.O && k0 + kBlockElems <= L.K) {
                    repack_block16(q + (size_t)o * row_bytes + (size_t)(k0 >> 1), dst);
                } else {
                    for (int p = 0; p < 16; ++p) {
                        uint8_t lo = src_nibble(q, row_bytes, L.O, L.K, o, k0 + p);
                        uint8_t hi = src_nibble(q, row_bytes, L.O, L.K, o, k0 + 16 + p);
                        dst[p] = (uint8_t)(lo | (hi << 4));
                    }
                }
            }
        }
        if (L.grouped) {
            const int ng_pad = L.nchunk * L.gpc;
            for (int g = 0; g < ng_pad; ++g)
                for (int r = 0; r < kTileRows; ++r) {
                    const int o = t * kTileRows + r;
                    float s = (o < L.O && g < L.ng_src) ? scales[(size_t)o * L.ng_src + g] : 0.0f;
                    std::memcpy(tile + w4_scale_offset(L, g, r), &s, 4);
                }
        }
    }
}

void w4_repack(const W4Layout &L, const uint8_t *q, const float *scales, uint8_t *stream, float *row_scales,
               int threads) {
    if (!L.grouped && row_scales) {
        for (int i = 0; i < L.ntile * kTileRows; ++i) row_scales[i] = (i < L.O) ? scales[i] : 0.0f;
    }
    int hw = (int)std::thread::hardware_concurrency();
    if (threads <= 0) threads = hw > 0 ? hw : 1;
    threads = std::min(threads, 32);
    // small matrices are not worth a thread spawn
    if (L.total_bytes < (1u << 20) || threads == 1 || L.ntile < 2 * threads) {
        repack_tiles(L, q, scales, stream, 0, L.ntile);
        return;
    }
    std::vector<std::thread> pool;
    const int per = (L.ntile + threads - 1) / threads;
    for (int i = 0; i < threads; ++i) {
        int t0 = i * per, t1 = std::min(L.ntile, t0 + per);
        if (t0 >= t1) break;
        pool.emplace_back(repack_tiles, std::cref(L), q, scales, stream, t0, t1);
    }
    for (auto &th : pool) th.join();
}

int w4_stream_nibble(const W4Layout &L, const uint8_t *stream, int o, int k) {
    const int t = o / kTileRows, r = o % kTileRows;
    const int blk = k / kBlockElems, e = k % kBlockElems;
    const uint8_t byte = stream[(size_t)t * L.tile_bytes + w4_seg_offset(L, blk, r) + (size_t)(e & 15)];
    return (e < 16) ? (byte & 0x0F) : (byte >> 4);
}

}  // namespace pgb
