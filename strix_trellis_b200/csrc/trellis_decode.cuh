// Device-side EXL3 trellis decoder for sm_100a.
//
// One warp decodes one 16x16 tile: lane l owns stream positions 8l..8l+7, i.e. the
// eight 16-bit states whose windows end at ring bits (8l+1)K ... (8l+8)K (reference
// python/strix_trellis/codec.py:58-85, docs/FORMAT.md:44-66).  The states go through
// the procedural codebook (codec.py:27-47) and leave as four half2 registers that
// are, without any shuffle, the A fragment of mma.sync.m16n8k16 for the transposed
// tile (m = output column, k = input row):
//     frag[0] = positions 0,1   (col l/4,   rows 2(l%4), +1)
//     frag[1] = positions 4,5   (col l/4+8, rows 2(l%4), +1)
//     frag[2] = positions 2,3   (col l/4,   rows 2(l%4)+8, +9)
//     frag[3] = positions 6,7   (col l/4+8, rows 2(l%4)+8, +9)
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

#include "rates.h"

namespace st {

enum : int { CB_3INST = 0, CB_MCG = 1, CB_MUL1 = 2 };

// ---- ring geometry of a lane's window (all compile-time in K, run-time in lane) ---
template <int K> struct Ring {
    static constexpr bool kHalf = rate_is_half(K);
    static constexpr int kLow = kHalf ? K - 8 : K;  // bits of an even stream position
    static constexpr int kWords = tile_words(K);    // uint32 words per tile
    static constexpr int kBits = 32 * kWords;       // ring length
    static constexpr int kLaneBits = kBits / 32;    // bits the eight positions of one lane consume
    // Offset of state j's window from state 0's: j positions of kLow bits plus one extra bit for
    // every odd position passed (half rates).
    __host__ __device__ static constexpr int field_pos(int j) { return j * kLow + (kHalf ? (j + 1) / 2 : 0); }
    // A lane's eight windows span field_pos(7)+16 bits starting at bit (lane*kLaneBits + kLow - 16)
    // mod ring.  Two ring words suffice when the largest in-word offset any lane has plus that span
    // stays within 64 bits (rates 1..4, 1.5 and 2.5); the others need three.
    static constexpr int kSpan = field_pos(7) + 16;
    __host__ __device__ static constexpr int start_bit(int lane) {
        return (lane * kLaneBits + kLow - 16 + kBits) % kBits;
    }
    __host__ __device__ static constexpr int max_offset() {
        int most = 0;
        for (int lane = 0; lane < 32; ++lane) most = (start_bit(lane) & 31) > most ? (start_bit(lane) & 31) : most;
        return most;
    }
    static constexpr int kLoadWords = (max_offset() + kSpan <= 64) ? 2 : 3;
};
static_assert(Ring<1>::kLoadWords == 2 && Ring<3>::kLoadWords == 2 && Ring<4>::kLoadWords == 2 &&
              Ring<5>::kLoadWords == 3 && Ring<8>::kLoadWords == 3 && Ring<9>::kLoadWords == 2 &&
              Ring<10>::kLoadWords == 2 && Ring<11>::kLoadWords == 3, "window words");

// Per-lane constants of the window: word indices (with ring wrap) and the in-word bit
// offset.  Computed once per thread, outside every loop.
template <int K> struct LaneGeom {
    int i0, i1, i2, shift;
    __device__ __forceinline__ explicit LaneGeom(int lane) {
        const int s = Ring<K>::start_bit(lane);
        i0 = s >> 5;
        i1 = (i0 + 1 == Ring<K>::kWords) ? 0 : i0 + 1;
        i2 = (i1 + 1 == Ring<K>::kWords) ? 0 : i1 + 1;
        shift = s & 31;
    }
};

// The three (or two) ring words of a lane, read from a tile that starts at `tile`
// (shared or global memory, 4-byte aligned).
template <int K>
__device__ __forceinline__ void load_window(const uint32_t* tile, const LaneGeom<K>& g, uint32_t (&w)[3]) {
    w[0] = tile[g.i0];
    w[1] = tile[g.i1];
    if constexpr (Ring<K>::kLoadWords == 3) w[2] = tile[g.i2];
    else w[2] = 0;
}

// ---- state extraction ---------------------------------------------------------
// After alignment the lane's first window starts at bit 0 (MSB) of a[0]; state j is
// the 16 bits at offset j*K of the big-endian bit string a[0]:a[1]:a[2].
template <int K>
__device__ __forceinline__ void align_window(const uint32_t (&w)[3], const LaneGeom<K>& g, uint32_t (&a)[3]) {
    // In-word offsets: K=4 -> 20 and K=8 -> 24 for every lane; other rates depend on
    // lane%4 (odd K) or lane%2 (K=2,6).
    const int o = (K == 4) ? 20 : (K == 8) ? 24 : g.shift;
    a[0] = __funnelshift_l(w[1], w[0], o);
    if constexpr (Ring<K>::kLoadWords == 3) {
        a[1] = __funnelshift_l(w[2], w[1], o);
        a[2] = w[2] << o;
    } else {
        a[1] = w[1] << o;
        a[2] = 0;
    }
}

// 16-bit field at big-endian bit offset P of a[0]:a[1]:a[2], zero-extended.
template <int P>
__device__ __forceinline__ uint32_t field16(const uint32_t (&a)[3]) {
    constexpr int idx = P >> 5, sh = P & 31;
    if constexpr (sh == 0) return a[idx] >> 16;
    else if constexpr (sh == 16) return a[idx] & 0xFFFFu;
    else if constexpr (sh == 8) return __byte_perm(a[idx], 0, 0x4421);
    else if constexpr (sh < 16) return (a[idx] >> (16 - sh)) & 0xFFFFu;
    else return __funnelshift_l(a[idx + 1], a[idx], sh) >> 16;
}

template <int K>
__device__ __forceinline__ void extract_states(const uint32_t (&w)[3], const LaneGeom<K>& g, uint32_t (&s)[8]) {
    if constexpr (K == 4) {
        // Every lane's window is bits [20, 64) of w0:w1.  With U = bits [16,48) of the
        // pair, three shifts make all eight states byte aligned: 11 integer ops in all.
        const uint32_t u = __funnelshift_r(w[1], w[0], 16), u4 = u >> 4, v = w[1] >> 4;
        s[7] = w[1] & 0xFFFFu;
        s[6] = v & 0xFFFFu;
        s[5] = __byte_perm(w[1], 0, 0x4421);
        s[4] = __byte_perm(v, 0, 0x4421);
        s[3] = w[1] >> 16;
        s[2] = u4 & 0xFFFFu;
        s[1] = __byte_perm(u, 0, 0x4421);
        s[0] = __byte_perm(u4, 0, 0x4421);
        return;
    }
    uint32_t a[3];
    align_window<K>(w, g, a);
    if constexpr (K == 2 || K == 6) {
        // Even rates: states at the same bit residue mod 8 share one pre-shifted copy
        // of the window, after which every state is a single byte permute.
        constexpr int step = 2;  // distinct residues {0,2,4,6}
#pragma unroll
        for (int r = 0; r < 8; r += step) {
            uint32_t b[3];
            if (r == 0) { b[0] = a[0]; b[1] = a[1]; b[2] = a[2]; }
            else {
                b[0] = __funnelshift_l(a[1], a[0], r);
                b[1] = __funnelshift_l(a[2], a[1], r);
                b[2] = a[2] << r;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if ((j * K) % 8 == r) {
                    const int p = j * K - r;  // byte aligned in b
                    const int idx = p >> 5, sh = p & 31;
                    // sh == 24 straddles two words: a byte permute has no zero source
                    // left, so that one case costs a funnel shift plus a shift.
                    s[j] = sh == 0 ? b[idx] >> 16
                         : sh == 8 ? __byte_perm(b[idx], 0, 0x4421)
                         : sh == 16 ? (b[idx] & 0xFFFFu)
                         : __funnelshift_l(b[idx + 1 > 2 ? 2 : idx + 1], b[idx], 24) >> 16;
                }
        }
    } else {
        using R = Ring<K>;
        s[0] = field16<R::field_pos(0)>(a); s[1] = field16<R::field_pos(1)>(a);
        s[2] = field16<R::field_pos(2)>(a); s[3] = field16<R::field_pos(3)>(a);
        s[4] = field16<R::field_pos(4)>(a); s[5] = field16<R::field_pos(5)>(a);
        s[6] = field16<R::field_pos(6)>(a); s[7] = field16<R::field_pos(7)>(a);
    }
}

__device__ __forceinline__ __half2 as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ uint32_t as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }

// ---- codebooks ------------------------------------------------------------------
// mul1: p = s*0x83DCD12D, b = byte sum, value = fma(half(1024+b), 0x1EEE, 0xC931) with
// ONE rounding.  A byte sum with accumulator 0x6400 yields the bit pattern of half(1024+b)
// directly (b <= 1020).  The multiply, dp4a, the packing multiply-add and HFMA2 all issue on
// the same half-rate pipe, so one of the two byte sums of a pair goes through the video
// instruction vabsdiff4 (sum of |byte - 0|), which issues on the other integer pipe:
// measured 49.6 against 52.0 clocks per K4 tile per scheduler.  Two states share one HFMA2.
__device__ __forceinline__ uint32_t bytesum_alu(uint32_t p) {
    uint32_t d;
    asm("vabsdiff4.u32.u32.u32.add %0, %1, %2, %3;" : "=r"(d) : "r"(p), "r"(0u), "r"(0x6400u));
    return d;
}
__device__ __forceinline__ uint32_t mul1_pair(uint32_t s0, uint32_t s1) {
    const uint32_t d0 = bytesum_alu(s0 * 0x83DCD12Du);
    const uint32_t d1 = __dp4a(s1 * 0x83DCD12Du, 0x01010101u, 0x6400u);
    // d0, d1 < 2^16: d1*65536 + d0 packs them
    uint32_t packed;
    asm("mad.lo.u32 %0, %1, 65536, %2;" : "=r"(packed) : "r"(d1), "r"(d0));
    const __half2 v = __hfma2(as_h2(packed), as_h2(0x1EEE1EEEu), as_h2(0xC931C931u));
    return as_u32(v);
}
// 3inst / mcg: q = (p & 0x8FFF8FFF) ^ 0x3B603B60, value = RN16(half(lo q) + half(hi q)).
// Both halves have exponent field 0b011xx, so a binary16 add is the single rounding.
template <int CB>
__device__ __forceinline__ uint32_t mix_pair(uint32_t s0, uint32_t s1) {
    const uint32_t p0 = CB == CB_MCG ? s0 * 0xCBAC1FEDu : s0 * 89226354u + 64248484u;
    const uint32_t p1 = CB == CB_MCG ? s1 * 0xCBAC1FEDu : s1 * 89226354u + 64248484u;
    const uint32_t q0 = (p0 & 0x8FFF8FFFu) ^ 0x3B603B60u;
    const uint32_t q1 = (p1 & 0x8FFF8FFFu) ^ 0x3B603B60u;
    const uint32_t lo = __byte_perm(q0, q1, 0x5410);  // (lo16 q0, lo16 q1)
    const uint32_t hi = __byte_perm(q0, q1, 0x7632);  // (hi16 q0, hi16 q1)
    return as_u32(__hadd2(as_h2(lo), as_h2(hi)));
}
template <int CB>
__device__ __forceinline__ uint32_t codebook_pair(uint32_t s0, uint32_t s1) {
    if constexpr (CB == CB_MUL1) return mul1_pair(s0, s1);
    else return mix_pair<CB>(s0, s1);
}

// Decode the lane's eight weights of one tile into mma A-fragment order.
template <int K, int CB>
__device__ __forceinline__ void decode_tile_frag(const uint32_t* tile, const LaneGeom<K>& g, uint32_t (&frag)[4]) {
    uint32_t w[3], s[8];
    load_window<K>(tile, g, w);
    extract_states<K>(w, g, s);
    frag[0] = codebook_pair<CB>(s[0], s[1]);
    frag[2] = codebook_pair<CB>(s[2], s[3]);
    frag[1] = codebook_pair<CB>(s[4], s[5]);
    frag[3] = codebook_pair<CB>(s[6], s[7]);
}

// The same from ring words that are already in registers (software-pipelined callers).
template <int K, int CB>
__device__ __forceinline__ void decode_words_frag(const uint32_t (&w)[3], const LaneGeom<K>& g, uint32_t (&frag)[4]) {
    uint32_t s[8];
    extract_states<K>(w, g, s);
    frag[0] = codebook_pair<CB>(s[0], s[1]);
    frag[2] = codebook_pair<CB>(s[2], s[3]);
    frag[1] = codebook_pair<CB>(s[4], s[5]);
    frag[3] = codebook_pair<CB>(s[6], s[7]);
}

template <int K, int CB>
__device__ __forceinline__ void decode_tile_frag(const uint32_t* tile, int lane, uint32_t (&frag)[4]) {
    const LaneGeom<K> g(lane);
    decode_tile_frag<K, CB>(tile, g, frag);
}

// Logical coordinates of stream position 8*lane+j (docs/FORMAT.md:61-66).
__device__ __forceinline__ int frag_row(int lane, int j) { return 2 * (lane & 3) + (j & 1) + 8 * ((j >> 1) & 1); }
__device__ __forceinline__ int frag_col(int lane, int j) { return (lane >> 2) + 8 * (j >> 2); }

}  // namespace st
