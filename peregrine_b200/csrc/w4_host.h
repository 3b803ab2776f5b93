// Host-side producer of the tile stream described in w4_layout.h.
#pragma once
#include "w4_layout.h"

namespace pgb {

// Re-lays a reference-format int4 matrix (row-major packed nibbles) into the
// tile stream.  `scales` is [O] (not grouped) or [O*ceil(K/gs)] (grouped).
// `stream` must hold L.total_bytes; `row_scales` (not grouped only) must hold
// L.ntile*16 floats and receives the per-row scales padded with zeros.
// Uses up to `threads` host threads (0 = hardware concurrency).
void w4_repack(const W4Layout &L, const uint8_t *q, const float *scales, uint8_t *stream, float *row_scales,
               int threads);

// Inverse of w4_repack for one element: the stored nibble (0..15) of (row o, element k).
int w4_stream_nibble(const W4Layout &L, const uint8_t *stream, int o, int k);

}  // namespace pgb
