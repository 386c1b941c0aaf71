// Work split of the fused GEMV ("stream-K"), shared by the kernel and by the host-side probe
// that lets the split be checked without a GPU.  The weights are `units` consecutive units
// (column block major, `hblocks` units per 128-column block); with units = q*grid + r, CTA c
// owns q+1 consecutive units when c < r and q units otherwise.  q and r come from the host,
// so the kernel needs no division to find its range.
#pragma once

#ifndef __CUDACC__
#define ST_HD
#else
#define ST_HD __host__ __device__
#endif

namespace st {

struct Split { int q, r; };  // units / grid, units % grid; 1 <= grid <= units < 2^31
struct Range { int begin, end; };

ST_HD inline Split make_split(int units, int grid) { return Split{units / grid, units % grid}; }
ST_HD inline Range cta_range(Split s, int c) {
    const int begin = s.q * c + (c < s.r ? c : s.r);
    return Range{begin, begin + s.q + (c < s.r ? 1 : 0)};
}
// The CTA whose range holds unit u.
ST_HD inline int owner(Split s, int u) {
    const int wide = (s.q + 1) * s.r;  // units held by the r CTAs of q+1 units
    return u < wide ? u / (s.q + 1) : s.r + (u - wide) / s.q;
}
// CTAs whose ranges intersect the units [lo, hi) of one column block: first..last.  `first`
// is the one whose range holds unit `lo` (it begins at or before the block), every other
// contributor begins inside the block.
ST_HD inline void contributors(Split s, int lo, int hi, int& first, int& last) {
    first = owner(s, lo);
    last = owner(s, hi - 1);
}

}  // namespace st
