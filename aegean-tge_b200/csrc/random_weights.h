// Counter-based random weights: every element is a function of (key, element index) alone, so a tensor
// drawn on the device, on the host and by an independent reimplementation is the same bit for bit,
// whatever the order, the thread count or the chunking.  Only integer arithmetic decides the value; the
// one floating-point step at the end is a single correctly rounded operation (an int-to-float
// conversion followed by one multiplication, by a power of two in the uniform case), so no compiler's
// contraction or library's transcendental can make two implementations differ.
//
//   mix(z)      : z ^= z >> 30; z *= 0xBF58476D1CE4E5B9; z ^= z >> 27; z *= 0x94D049BB133111EB; z ^= z >> 31
//   word(k, c)  : mix(k + 0x9E3779B97F4A7C15 * (c + 1))                       (all modulo 2^64)
//   key         : mix(fnv1a64(tensor name) ^ mix(seed + 0x9E3779B97F4A7C15))   (formed by the caller)
//   normal  i   : s = sum of the eight 16-bit fields of word(k, 2i) and word(k, 2i+1);
//                 value = float(2 s - 8 * 65535) * scale          scale = std / (2 sqrt(8 (65536^2 - 1) / 12))
//                 (a sum of eight uniform integers: mean 0, the asked deviation, support +-4.9 deviations)
//   uniform i   : m = base + ((word(k, i) >> 32) * span >> 32);  value = float(m) * 2^-24
//                 base = round(lo 2^24), span = round((hi - lo) 2^24), both below 2^31
//
// The reference has no random model at all (its test fixture is zeros, tests/test_gguf.cpp:962-1018).
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#define TGE_RW_INLINE __host__ __device__ __forceinline__
#else
#define TGE_RW_INLINE inline
#endif

enum TgeRandomKind : int { TGE_RANDOM_NORMAL = 0, TGE_RANDOM_UNIFORM = 1 };

TGE_RW_INLINE uint64_t tge_rw_mix(uint64_t z) {
  z ^= z >> 30;
  z *= 0xBF58476D1CE4E5B9ull;
  z ^= z >> 27;
  z *= 0x94D049BB133111EBull;
  z ^= z >> 31;
  return z;
}

TGE_RW_INLINE uint64_t tge_rw_word(uint64_t key, uint64_t counter) {
  return tge_rw_mix(key + 0x9E3779B97F4A7C15ull * (counter + 1ull));
}

// the sum of the four 16-bit fields of a word
TGE_RW_INLINE uint32_t tge_rw_fields(uint64_t w) {
  const uint64_t pairs = (w & 0x0000FFFF0000FFFFull) + ((w >> 16) & 0x0000FFFF0000FFFFull);
  return (uint32_t)(pairs & 0xFFFFFFFFull) + (uint32_t)(pairs >> 32);
}

// the integer behind element `index` of a normal tensor: 2 s - 8 * 65535, magnitude below 2^20
TGE_RW_INLINE int32_t tge_rw_normal_int(uint64_t key, uint64_t index) {
  const uint32_t s = tge_rw_fields(tge_rw_word(key, 2ull * index)) + tge_rw_fields(tge_rw_word(key, 2ull * index + 1ull));
  return (int32_t)(2u * s) - 8 * 65535;
}

// the integer behind element `index` of a uniform tensor: value * 2^24
TGE_RW_INLINE int32_t tge_rw_uniform_int(uint64_t key, uint64_t index, int32_t base, uint32_t span) {
  const uint64_t high = tge_rw_word(key, index) >> 32;
  return base + (int32_t)((high * (uint64_t)span) >> 32);
}
