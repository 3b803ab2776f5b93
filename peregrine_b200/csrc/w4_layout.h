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
// one contiguous byte stream that a half-warp consumes front to back in chunks
// of 256 elements of K (one bulk copy each):
//
//   tile t  = rows 16t .. 16t+15
//   stream  = chunk 0 | chunk 1 | ... | chunk nchunk-1        (K padded to 256)
//   chunk c = 8 slabs of 256 B, then (group-scaled format only) gpc*64 B of scales
//   slab b  = 16 rows x 16 B; row r at byte r*16 holds the 32 elements
//             [256c + 32b, +32) of row 16t+r
//   byte p of a row's 16 B = elem[p] | elem[16+p] << 4   (stored nibbles, v+8)
//   scales  = 16 rows x gpc fp32, row-major: row r's scales for the chunk's
//             gpc = 256/gs groups are contiguous at byte r*gpc*4
//
// With this split a 32-bit word masked with 0x0F0F0F0F is four consecutive
// elements [4j, 4j+4) and masked with 0xF0F0F0F0 is 16x the elements
// [16+4j, 16+4j+4): both feed dp4a against the activation row in natural order.
// Rows beyond O, elements beyond K and groups beyond ceil(K/gs) are stored as
// nibble 8 (value 0) with scale 0, so padding never contributes.
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
constexpr int kChunkBlocks = 8;      // 32-element blocks per chunk
constexpr int kChunkElems = 256;     // elements of K per chunk
constexpr int kChunkSlabBytes = kChunkBlocks * kSlabBytes;  // 2048
constexpr int kChunkMaxBytes = kChunkSlabBytes + 8 * 64;    // 2560 (gs = 32)

struct W4Layout {
    int O;            // logical rows
    int K;            // logical columns
    int grouped;      // 1: group scales inside the stream, 0: one scale per row (separate array)
    int gs;           // group size in elements (grouped only): 32, 64, 128 or 256
    int bpg;          // 32-element blocks per group (1 when not grouped)
    int gpc;          // groups per chunk = 8 / bpg
    int ng_src;       // groups per row in the caller's scale array = ceil(K/gs) (0 when not grouped)
    int nchunk;       // ceil(K / 256)
    int nblk;         // nchunk * 8: 32-element blocks per padded row
    int ntile;        // ceil(O / 16)
    int chunk_bytes;  // 2048 (+ gpc*64 when grouped)
    int kp;           // padded row length in elements = nchunk*256 (activation row stride)
    size_t tile_bytes;
    size_t total_bytes;
};

// Returns false for shapes the stream cannot hold (gs not one of 32/64/128/256).
PGB_HD bool w4_layout_make(W4Layout *L, int O, int K, int grouped, int gs) {
    if (O <= 0 || K <= 0) return false;
    L->O = O;
    L->K = K;
    L->grouped = grouped ? 1 : 0;
    if (grouped) {
        if (gs != 32 && gs != 64 && gs != 128 && gs != 256) return false;
        L->gs = gs;
        L->bpg = gs / kBlockElems;
        L->ng_src = (K + gs - 1) / gs;
    } else {
        L->gs = 0;
        L->bpg = 1;
        L->ng_src = 0;
    }
    L->gpc = kChunkBlocks / L->bpg;
    L->nchunk = (K + kChunkElems - 1) / kChunkElems;
    L->nblk = L->nchunk * kChunkBlocks;
    L->ntile = (O + kTileRows - 1) / kTileRows;
    L->chunk_bytes = kChunkSlabBytes + (L->grouped ? L->gpc * 64 : 0);
    L->kp = L->nchunk * kChunkElems;
    L->tile_bytes = (size_t)L->nchunk * (size_t)L->chunk_bytes;
    L->total_bytes = L->tile_bytes * (size_t)L->ntile;
    return true;
}

// Byte offset, inside one tile's stream, of row r's 16-byte segment for 32-block `blk` (0 .. nblk-1).
PGB_HD size_t w4_seg_offset(const W4Layout &L, int blk, int r) {
    return (size_t)(blk / kChunkBlocks) * L.chunk_bytes + (size_t)(blk % kChunkBlocks) * kSlabBytes + (size_t)r * 16;
}
// Byte offset, inside one tile's stream, of row r's scale for padded group g (grouped only).
PGB_HD size_t w4_scale_offset(const W4Layout &L, int g, int r) {
    return (size_t)(g / L.gpc) * L.chunk_bytes + kChunkSlabBytes + (size_t)r * L.gpc * 4 + (size_t)(g % L.gpc) * 4;
}

}  // namespace pgb
