// Rate codes of a trellis tensor, shared by host and device code (plain C++).
// A rate code names the bits per weight: 1..8 are the integer rates; 9, 10 and 11 stand for 1.5,
// 2.5 and 3.5, where stream positions alternate between floor(rate) bits (even positions) and
// one bit more (odd positions) -- reference python/strix_trellis/codec.py:12-20, mul1 only.
// Everything that depends on the size of a tile goes through tile_words().
#pragma once

#ifdef __CUDACC__
#define ST_RATE_FN __host__ __device__ constexpr
#else
#define ST_RATE_FN constexpr
#endif

namespace st {

constexpr int kRateCodes = 11;
ST_RATE_FN int rate_x2(int code) { return code <= 8 ? 2 * code : 2 * (code - 8) + 1; }  // twice the bits per weight
ST_RATE_FN int tile_words(int code) { return 4 * rate_x2(code); }    // uint32 words per 16x16 tile
ST_RATE_FN int unit_bytes(int code) { return 256 * tile_words(code); }  // 64 tiles: one column block x one H128 block
ST_RATE_FN bool rate_is_half(int code) { return code > 8; }
// rate code of bits_x2 (twice the rate): 2, 4, ..., 16 -> 1..8; 3, 5, 7 -> 9, 10, 11; else 0
ST_RATE_FN int rate_code(unsigned bits_x2) {
    return (bits_x2 >= 2 && bits_x2 <= 16 && bits_x2 % 2 == 0) ? (int)(bits_x2 / 2)
           : (bits_x2 == 3 || bits_x2 == 5 || bits_x2 == 7) ? (int)(8 + bits_x2 / 2)
           : 0;
}
// of two rate codes, the one with the larger tiles
ST_RATE_FN int heavier_rate(int a, int b) { return tile_words(a) >= tile_words(b) ? a : b; }

}  // namespace st
