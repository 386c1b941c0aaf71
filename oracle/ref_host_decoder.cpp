// Thin C wrapper that compiles the reference's OWN plain-C++ host decoder
// (src/host_reference.hpp in the reference tree: host_state :5-14, host_codebook
// :22-36) where it lies, so the oracle's ring windows and codebooks can be checked
// against code the reference authors wrote.  Test infrastructure only; the output
// goes to oracle/_ref/ and is never linked into the shipped library.  The header
// is included by path at build time (see Makefile, REFERENCE_ROOT); no reference
// source is copied into this repository.
#include <cstdint>
#include "host_reference.hpp"

extern "C" {
uint16_t ref_host_state(const uint32_t* tile_words, int bits, int position) {
    return host_state(tile_words, bits, position);
}
uint16_t ref_host_codebook(uint16_t state, int codebook) { return host_codebook(state, codebook); }
}
