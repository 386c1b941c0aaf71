// Work split of the fused GEMV ("stream-K"), shared by the kernel and by the host-side probe
// that lets the split be checked without a GPU.  The weights are `units` consecutive units
// (column block major, `hblocks` units per 128-column block); CTA c of `grid` owns the
// contiguous range [units*c/grid, units*(c+1)/grid).
#pragma once

#ifndef __CUDACC__
#define ST_HD
#else
#define ST_HD __host__ __device__
#endif

namespace st {

struct Range { long long begin, end; };
ST_HD inline Range cta_range(long long units, int grid, int c) {
    return Range{units * c / grid, units * (c + 1) / grid};
}
// CTAs whose ranges intersect the units [lo, hi) of one column block: first..last.  `first`
// is the one whose range holds unit `lo` (it begins at or before the block), every other
// contributor begins inside the block.
ST_HD inline void contributors(long long units, int grid, long long lo, long long hi, int& first, int& last) {
    int c = (int)(lo * grid / units);
    if (c >= grid) c = grid - 1;
    while (c > 0 && cta_range(units, grid, c).begin > lo) --c;
    while (cta_range(units, grid, c).end <= lo) ++c;
    first = c;
    c = (int)((hi - 1) * grid / units);
    if (c >= grid) c = grid - 1;
    while (c + 1 < grid && cta_range(units, grid, c + 1).begin < hi) ++c;
    while (cta_range(units, grid, c).begin >= hi) --c;
    last = c;
}

}  // namespace st
