"""Invariants of the fused GEMV's work split, checked on the CPU through the library's own
arithmetic (strix_b200_gemv_partition): the unit ranges tile the weight stream, every shared
column block has exactly one folding CTA, that CTA waits only for CTAs above it (so the
bounded waits of the fold cannot form a cycle), it reaches the block at the very end of its
own range, and no CTA ever publishes more than one partial plane per launch."""
import ctypes as C

import pytest

from strix_trellis_b200 import native as N

SHAPES = [(4096, 4096), (5120, 5120), (1152, 4096), (4096, 14336), (16384, 4096), (4096, 129280),
          (128, 128), (128, 4096), (8192, 256), (2048, 1152)]


def split(lib, inputs, outputs, grid):
    hblocks, nblocks = inputs // 128, outputs // 128
    out = (N.u64 * 4)()
    ranges = []
    for cta in range(grid):
        assert lib.strix_b200_gemv_partition(inputs, outputs, grid, cta, 0, out) == N.SUCCESS
        ranges.append((out[0], out[1]))
    blocks = []
    for nb in range(nblocks):
        assert lib.strix_b200_gemv_partition(inputs, outputs, grid, 0, nb, out) == N.SUCCESS
        blocks.append((out[2], out[3]))
    return hblocks, nblocks, ranges, blocks


@pytest.mark.parametrize("sm_count", [148, 132, 7])
@pytest.mark.parametrize("shape", SHAPES)
def test_split_invariants(shape, sm_count):
    lib = N.load()
    inputs, outputs = shape
    units = (inputs // 128) * (outputs // 128)
    grid = min(sm_count, units)
    hblocks, nblocks, ranges, blocks = split(lib, inputs, outputs, grid)
    # contiguous, ordered, balanced to one unit, covering every unit once
    assert ranges[0][0] == 0 and ranges[-1][1] == units
    assert all(ranges[c][1] == ranges[c + 1][0] for c in range(grid - 1))
    sizes = [e - b for b, e in ranges]
    assert min(sizes) >= 1 and max(sizes) - min(sizes) <= 1
    planes = [0] * grid
    for nb, (first, last) in enumerate(blocks):
        lo, hi = nb * hblocks, (nb + 1) * hblocks
        touching = [c for c, (b, e) in enumerate(ranges) if b < hi and e > lo]
        assert touching == list(range(first, last + 1))
        assert ranges[first][0] <= lo < ranges[first][1]          # the folding CTA holds the block's first unit
        if first == last:
            continue                                                # finished locally, no plane
        assert ranges[first][1] < hi                                # ... and the block is the END of its range
        for c in range(first + 1, last + 1):                        # it waits only for CTAs above it
            assert ranges[c][0] > lo                                # which begin inside the block
            planes[c] += 1
    assert max(planes) <= 1                                         # one plane per CTA is enough


def test_partition_rejects_bad_arguments():
    lib = N.load()
    out = (N.u64 * 4)()
    assert lib.strix_b200_gemv_partition(4096, 4096, 148, 148, 0, out) == N.INVALID_ARGUMENT
    assert lib.strix_b200_gemv_partition(4096, 4100, 148, 0, 0, out) == N.INVALID_ARGUMENT
    assert lib.strix_b200_gemv_partition(4096, 4096, 148, 0, 32, out) == N.INVALID_ARGUMENT
    assert lib.strix_b200_gemv_partition(128, 128, 2, 0, 0, out) == N.INVALID_ARGUMENT
    assert lib.strix_b200_gemv_partition(4096, 4096, 148, 0, 0, None) == N.INVALID_ARGUMENT
