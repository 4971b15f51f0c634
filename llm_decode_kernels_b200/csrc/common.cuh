// Device helpers shared by every kernel of the decode step. Target: sm_100a (B200), fp16 storage,
// fp32 accumulation, no tensor-core instructions (the batch-1 step is a stream of GEMVs).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define DEVI __device__ __forceinline__

// Status codes returned by every extern "C" entry point (see include/b200decode.h).
#define B200_OK 0
#define B200_ERR_ARG (-1)     // null pointer, non-positive size, value out of range
#define B200_ERR_ALIGN (-2)   // a pointer that must be 16-byte aligned is not
#define B200_ERR_SHAPE (-3)   // a shape this library has no kernel for
#define B200_ERR_LAUNCH (-4)  // the CUDA runtime refused the launch
#define B200_ERR_LIMIT (-5)   // a size beyond a fixed capacity of the entry point

namespace b200 {

constexpr int kNumSMs = 148;

DEVI float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
DEVI float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

DEVI half2 as_h2(uint32_t u) { return *reinterpret_cast<half2*>(&u); }
DEVI uint32_t as_u32(half2 h) { return *reinterpret_cast<uint32_t*>(&h); }

// 128-bit streaming load for bytes that are used exactly once (packed weights, KV rows): read-only
// path, no L1 allocation, so the small reused vectors (activations, scales) keep the L1.
DEVI uint4 ld_stream(const uint4* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

// ---- INT4 nibble decoding -------------------------------------------------------------------
// A packed word holds elements 2i (bits [4i,4i+4)) and 2i+1 (bits [16+4i,16+4i+4)), i = 0..3.
// OR-ing a nibble into the mantissa of fp16 1024.0 (0x6400) gives 1024 + q when the nibble sits in
// bits 0..3 and 1024 + 16 q when it sits in bits 4..7, so one shift by 8 and four mask-or
// operations decode all eight nibbles of a word with no integer-to-float conversion:
//   lo(w)      -> 1024 +    (q0, q1)        hi(w)      -> 1024 + 16 (q2, q3)
//   lo(w >> 8) -> 1024 +    (q4, q5)        hi(w >> 8) -> 1024 + 16 (q6, q7)
// Subtracting 1024 + z (or 1024 + 16 z) is exact in fp16 because every value is an integer < 2048.
DEVI half2 nib_lo(uint32_t w) { return as_h2((w & 0x000F000Fu) | 0x64006400u); }
DEVI half2 nib_hi(uint32_t w) { return as_h2((w & 0x00F000F0u) | 0x64006400u); }

// Multiply-accumulate the 8 weights of one packed word against 8 activations held as 4 half2.
// zl = (1024 + z, 1024 + z), zh = (1024 + 16 z, 1024 + 16 z). The activations for the two "hi"
// pairs must already carry a factor 1/16 (see stage_x_scaled): the result is then
// sum_k (q_k - z) * x_k * c with one common factor c for all eight terms.
DEVI half2 dot_word(uint32_t w, uint32_t x01, uint32_t x23, uint32_t x45, uint32_t x67, half2 zl, half2 zh,
                    half2 acc) {
  const uint32_t w8 = w >> 8;
  acc = __hfma2(__hsub2(nib_lo(w), zl), as_h2(x01), acc);
  acc = __hfma2(__hsub2(nib_hi(w), zh), as_h2(x23), acc);
  acc = __hfma2(__hsub2(nib_lo(w8), zl), as_h2(x45), acc);
  acc = __hfma2(__hsub2(nib_hi(w8), zh), as_h2(x67), acc);
  return acc;
}

// Activation pre-scaling that goes with dot_word. Element pairs (2i, 2i+1) of each group of 8 with
// i even ("lo" nibbles) are multiplied by 1/16, pairs with i odd ("hi" nibbles, decoded as 16 q) by
// 1/256, so that every product is (q - z) * x / 16: the half2 partial sums stay 16x further away
// from fp16 overflow than plain (q - z) * x would, and the caller multiplies the fp32 sum by
// 16 * scale. Both factors are powers of two, so the scaling itself is exact for normal numbers.
DEVI uint4 scale_x8(uint4 v) {
  const half2 c_lo = __float2half2_rn(1.0f / 16.0f), c_hi = __float2half2_rn(1.0f / 256.0f);
  v.x = as_u32(__hmul2(as_h2(v.x), c_lo));
  v.y = as_u32(__hmul2(as_h2(v.y), c_hi));
  v.z = as_u32(__hmul2(as_h2(v.z), c_lo));
  v.w = as_u32(__hmul2(as_h2(v.w), c_hi));
  return v;
}
constexpr float kDotWordRescale = 16.0f;

DEVI void unpack8(uint4 v, float* f) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __half22float2(as_h2(w[i]));
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

// Order key for greedy argmax over fp16 logits: larger value wins, then the lower index. One max-reduction
// over these keys settles value and tie-break together.
DEVI unsigned long long argmax_key(half v, int idx) {
  uint32_t b = (uint32_t)__half_as_ushort(v);
  b = (b & 0x8000u) ? (~b & 0xFFFFu) : (b | 0x8000u);  // monotone map of fp16 bits to unsigned order
  return ((unsigned long long)b << 32) | (uint32_t)(0x7FFFFFFF - idx);
}

}  // namespace b200
