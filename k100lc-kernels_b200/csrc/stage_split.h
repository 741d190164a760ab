// Which rows of a layer a CTA of the stream kernels takes when whole stages are dealt out (host and device: the
// kernels call it with their own block index, fm_stream_rows answers the same question on the host).
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define FM_HOST_DEVICE __host__ __device__
#else
#define FM_HOST_DEVICE
#endif

namespace fm {

// Rows [r0, r1) of a layer of `rows` rows for CTA `cta` of `grid`.  The layer is ceil(rows / stage_rows) stages; every
// CTA gets floor(stages / grid) of them and `stages mod grid` CTAs one more.  Those CTAs are the ones from a position
// that moves with `first` (the table index of the layer, or of the first chunk of the weight matrix it belongs to): the
// fractional part of first / golden ratio, scaled to the grid, so that consecutive layers start far apart and the
// starts of any run of layers cover the grid evenly.  The ranges of the CTAs of a layer are disjoint, ascending in the
// rotated CTA order, and cover [0, rows); only the last stage of a layer can be a partial one.
FM_HOST_DEVICE inline void stage_split(int rows, int first, int grid, int cta, int stage_rows, int* r0, int* r1) {
    const int S = (rows + stage_rows - 1) / stage_rows;
    const int base = S / grid, extra = S - base * grid;
    const int rot = (int)((((uint32_t)first * 2654435769u) >> 16) * (uint32_t)grid >> 16);
    int b = cta - rot;
    b += b < 0 ? grid : 0;
    const int s0 = b * base + (b < extra ? b : extra), s1 = s0 + base + (b < extra ? 1 : 0);
    const int a0 = s0 * stage_rows, a1 = s1 * stage_rows;
    *r0 = a0 < rows ? a0 : rows;
    *r1 = a1 < rows ? a1 : rows;
}

}  // namespace fm
