// E2M1 nibble -> E4M3 byte dequantisation, 8 values per 32-bit word.
//
// Every E2M1 value {0,.5,1,1.5,2,3,4,6} is exactly representable in E4M3; the byte of code
// 0..7 is 00 30 38 3C 40 44 48 4C and the nibble's sign (bit 3) becomes the byte's bit 7.
// Element order: low nibble of byte 0 is element 0 (reference tests/test_cute_dsl_mla_fp4.py:76-84).
#pragma once
#include <stdint.h>

namespace mla {

// word = 8 packed E2M1 codes (elements 0..7, low nibble first) ->
// lo = E4M3 bytes of elements 0..3, hi = elements 4..7.  Nine integer instructions.
__device__ __forceinline__ void e2m1x8_to_e4m3x8(uint32_t word, uint32_t& lo, uint32_t& hi) {
  constexpr uint32_t kLutA = 0x3C383000u;  // codes 0..3
  constexpr uint32_t kLutB = 0x4C484440u;  // codes 4..7
  const uint32_t mag = word & 0x77777777u;
  const uint32_t mag_lo = __byte_perm(kLutA, kLutB, mag);
  const uint32_t mag_hi = __byte_perm(kLutA, kLutB, mag >> 16);
  // bit 7 of byte j: sign of nibble 2j in (word << 4), sign of nibble 2j+1 in word
  const uint32_t even = word << 4;
  const uint32_t sgn_lo = __byte_perm(even, word, 0x5140u);
  const uint32_t sgn_hi = __byte_perm(even, word, 0x7362u);
  lo = mag_lo | (sgn_lo & 0x80808080u);
  hi = mag_hi | (sgn_hi & 0x80808080u);
}

}  // namespace mla
