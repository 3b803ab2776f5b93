// Tile-stream layout of a resident int4 weight matrix, shared by the host
// repacker, the CUDA kernels and the CPU walk used by the host-side tests.
//
// The caller hands over the reference's container layout
// (crates/peregrine-core/src/pack.rs:492-542): row-major [O, ceil(K/2)] bytes,
// element i of a row in the low (i even) or high (i odd) nibble of byte i/2,
// stored value = v + 8, with either one fp32 scale per row (fmt 2) or one per
// group of `gs` elements along K (fmt 4, scale[o*ng + g]).
//
// On the device the matrix is re-laid as a sequence of 16-row tiles, each tile
// one contiguous byte stream that a half-warp consumes front to back:
//
//   tile t  = rows 16t .. 16t+15
//   stream  = group 0 | group 1 | ... | group ng-1
//   group g = bpg slabs of 256 B  (+ 64 B of scales when the format is grouped)
//   slab b  = 16 rows x 16 B; row r at byte r*16 holds the 32 elements
//             [32*(g*bpg+b), +32) of row 16t+r
//   byte p of a row's 16 B = elem[p] | elem[16+p] << 4   (stored nibbles, v+8)
//   scales  = 16 fp32, row r at byte r*4
//
// With this split a 32-bit word masked with 0x0F0F0F0F is four consecutive
// elements [4j, 4j+4) and masked with 0xF0F0F0F0 is 16x the elements
// [16+4j, 16+4j+4): both feed dp4a against the activation row in natural order.
// Rows beyond O and elements beyond K are stored as nibble 8 (value 0) with
// scale 0, so padding never contributes.
#pragma once
#include <stddef.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define PGB_HD __host__ __device__ __forceinline__
#else
#define PGB_HD inline
#endif

namespace pgb {

constexpr int kTileRows = 16;        // rows per tile (one half-warp)
constexpr int kBlockElems = 32;      // elements per 16-byte row segment
constexpr int kSlabBytes = 256;      // 16 rows x 16 B
constexpr int kScaleBytes = 64;      // 16 rows x 4 B
constexpr int kChunkMaxBytes = 2176; // one bulk copy never exceeds this (gs<=256)

struct W4Layout {
    int O;           // logical rows
    int K;           // logical columns
    int grouped;     // 1: group scales inside the stream, 0: one scale per row (separate array)
    int gs;          // group size in elements (grouped only; multiple of 32)
    int bpg;         // 32-element blocks per group (1 when not grouped)
    int ng;          // groups per row as stored (not grouped: number of 32-blocks)
    int nblk;        // ng * bpg: 32-element blocks per padded row
    int ntile;       // ceil(O / 16)
    int group_bytes; // bpg*256 (+64 when grouped)
    int gpc;         // groups per bulk-copy chunk
    int nchunk;      // ceil(ng / gpc)
    int kp;          // padded row length in elements = nblk*32 (activation row stride)
    size_t tile_bytes;
    size_t total_bytes;
};

// Returns false for shapes the stream cannot hold (gs not a multiple of 32 or > 256).
PGB_HD bool w4_layout_make(W4Layout *L, int O, int K, int grouped, int gs) {
    if (O <= 0 || K <= 0) return false;
    L->O = O;
    L->K = K;
    L->grouped = grouped ? 1 : 0;
    if (grouped) {
        if (gs <= 0 || gs % kBlockElems != 0 || gs > 256) return false;
        L->gs = gs;
        L->bpg = gs / kBlockElems;
        L->ng = (K + gs - 1) / gs;
    } else {
        L->gs = 0;
        L->bpg = 1;
        L->ng = (K + kBlockElems - 1) / kBlockElems;
    }
    L->nblk = L->ng * L->bpg;
    L->ntile = (O + kTileRows - 1) / kTileRows;
    L->group_bytes = L->bpg * kSlabBytes + (L->grouped ? kScaleBytes : 0);
    L->gpc = kChunkMaxBytes / L->group_bytes;
    if (L->gpc < 1) return false;
    if (L->gpc > L->ng) L->gpc = L->ng;
    L->nchunk = (L->ng + L->gpc - 1) / L->gpc;
    L->kp = L->nblk * kBlockElems;
    L->tile_bytes = (size_t)L->ng * (size_t)L->group_bytes;
    L->total_bytes = L->tile_bytes * (size_t)L->ntile;
    return true;
}

// Byte offset, inside one tile's stream, of row r's 16-byte segment for block b of group g.
PGB_HD size_t w4_seg_offset(const W4Layout &L, int g, int b, int r) {
    return (size_t)g * L.group_bytes + (size_t)b * kSlabBytes + (size_t)r * 16;
}
// Byte offset, inside one tile's stream, of row r's scale for group g (grouped only).
PGB_HD size_t w4_scale_offset(const W4Layout &L, int g, int r) {
    return (size_t)g * L.group_bytes + (size_t)L.bpg * kSlabBytes + (size_t)r * 4;
}

}  // namespace pgb
