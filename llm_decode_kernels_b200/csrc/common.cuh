// Device helpers shared by the kernels of the library. Target: sm_100a (B200), fp16 storage, fp32 (or exact integer)
// accumulation. The GEMV and the persistent step feed the warp-level integer mma.sync.m16n8k32 with operands taken
// straight from the packed format (see "tensor-core operands" below), attention the fp16 m16n8k16; the 64-row-and-up
// tcgen05 MMAs, which a batch-1 step cannot fill, are used by the prompt's GEMM only (prefill_gemm.cu).
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

// ---- programmatic dependent launch ------------------------------------------------------------------------
// The decode step is a chain of small kernels, each waiting for the one before it; between two ordinary launches the
// GPU drains, flushes and only then schedules the next grid. Launched with launch_pdl(), a kernel may be scheduled
// while its predecessor still runs: every kernel says "my dependents may be scheduled" at its top
// (pdl_launch_dependents) and then blocks in pdl_wait() until the predecessor has completed and its writes are
// visible. Nothing that another kernel produced may be read before pdl_wait(); what does not depend on the
// predecessor (weights) may be fetched before it. Both are no-ops in a kernel launched the ordinary way.
DEVI void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
DEVI void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) is a per-device setting: launchers remember, per device, the size
// they have already allowed. `state` is a function-local static array of kMaxDevices zeros.
constexpr int kMaxDevices = 64;
template <typename Kern>
inline cudaError_t allow_dynamic_smem(Kern kern, size_t bytes, size_t* state) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const bool tracked = dev >= 0 && dev < kMaxDevices;
  if (bytes <= 48 * 1024 || (tracked && bytes <= state[dev])) return cudaSuccess;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e == cudaSuccess && tracked) state[dev] = bytes;
  return e;
}

// launch_pdl(...) inside a function that returns cudaError_t: a refused launch is returned at once
#define B200_LAUNCH(...)                               \
  do {                                                 \
    const cudaError_t pe_ = launch_pdl(__VA_ARGS__);   \
    if (pe_ != cudaSuccess) return pe_;                \
  } while (0)

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

// ---- inner product on masked nibbles (used by the persistent step kernel and the segmented GEMV) ------------------
// A nibble masked in place is an fp16 SUBNORMAL: bits 0..3 of a half are q * 2^-24, bits 4..7 are q * 2^-20. So
// (word & 0x000F000F) and (word & 0x00F000F0) are ready-made half2 operands and one shift by 8 exposes the other four
// nibbles. x is staged multiplied by 2^s (pairs under the low mask) or 2^(s-4) (pairs under the high mask), s chosen
// from max|x| so nothing overflows; every product is then q * x * 2^(s-24). With xs = sum of x over a 32-weight chunk,
//     sum (q - z) * scale * x = scale * (2^(24-s) * sum q x'  -  z * xs),
// so the zero point costs one FMA per chunk instead of one subtraction per weight.
// 16-byte chunk ci of x lives at swz(ci): a lane of the GEMV reads the four consecutive chunks 4u..4u+3 for its
// weight chunk u = lane, and without the swizzle those reads would be 64 bytes apart across lanes (4-way conflicts).
DEVI int swz(int ci) { return (ci & ~3) | ((ci & 3) ^ ((ci >> 3) & 3)); }

struct XScale { half2 lo, hi; float resc; };
// Power-of-two staging scale from max|x|: x * 2^s stays below 2^15.
DEVI XScale scale_for(float xmax) {
  int s = 14 - ilogbf(fmaxf(xmax, 1e-30f));
  s = max(-10, min(15, s));
  XScale r;
  r.lo = __float2half2_rn(exp2f((float)s));
  r.hi = __float2half2_rn(exp2f((float)(s - 4)));
  r.resc = exp2f((float)(24 - s));
  return r;
}

// One packed word (8 weights) of each of two rows against the 8 staged activations x = (x01, x23, x45, x67).
// Four independent half2 accumulators per row (one per nibble position): short chains, so fp16 rounding stays small
// and the FMAs of one word do not wait on each other.
DEVI void fma_word2(uint32_t wa, uint32_t wb, uint4 x, half2* a, half2* b) {
  const uint32_t wa8 = wa >> 8, wb8 = wb >> 8;
  a[0] = __hfma2(as_h2(wa & 0x000F000Fu), as_h2(x.x), a[0]);
  b[0] = __hfma2(as_h2(wb & 0x000F000Fu), as_h2(x.x), b[0]);
  a[1] = __hfma2(as_h2(wa & 0x00F000F0u), as_h2(x.y), a[1]);
  b[1] = __hfma2(as_h2(wb & 0x00F000F0u), as_h2(x.y), b[1]);
  a[2] = __hfma2(as_h2(wa8 & 0x000F000Fu), as_h2(x.z), a[2]);
  b[2] = __hfma2(as_h2(wb8 & 0x000F000Fu), as_h2(x.z), b[2]);
  a[3] = __hfma2(as_h2(wa8 & 0x00F000F0u), as_h2(x.w), a[3]);
  b[3] = __hfma2(as_h2(wb8 & 0x00F000F0u), as_h2(x.w), b[3]);
}

// The 32 staged activations of one weight chunk, held in registers, plus their unscaled sum.
struct XChunk { uint4 x0, x1, x2, x3; float xs; };

// One 32-weight chunk of two rows (packed words wa, wb; (scale, zero) sa, sb) against x: this lane's share of both
// dot products.
DEVI void chunk_two_rows(uint4 wa, uint4 wb, half2 sza, half2 szb, const XChunk& x, float resc, float& p0, float& p1) {
  const half2 zero2 = __float2half2_rn(0.f);
  const float2 sa = __half22float2(sza), sb = __half22float2(szb);
  half2 a[4] = {zero2, zero2, zero2, zero2}, b[4] = {zero2, zero2, zero2, zero2};
  fma_word2(wa.x, wb.x, x.x0, a, b);
  fma_word2(wa.y, wb.y, x.x1, a, b);
  fma_word2(wa.z, wb.z, x.x2, a, b);
  fma_word2(wa.w, wb.w, x.x3, a, b);
  const float2 fa0 = __half22float2(__hadd2(a[0], a[2])), fa1 = __half22float2(__hadd2(a[1], a[3]));
  const float2 fb0 = __half22float2(__hadd2(b[0], b[2])), fb1 = __half22float2(__hadd2(b[1], b[3]));
  p0 = fmaf(sa.x, fmaf((fa0.x + fa0.y) + (fa1.x + fa1.y), resc, -sa.y * x.xs), p0);
  p1 = fmaf(sb.x, fmaf((fb0.x + fb0.y) + (fb1.x + fb1.y), resc, -sb.y * x.xs), p1);
}

// ---- tensor-core operands ------------------------------------------------------------------------------------------
// mma.sync.m16n8k32, unsigned bytes x signed bytes, int32 accumulators (C += A B). Lane (g, t) holds
//   A: a0 = A[g][4t .. 4t+3], a1 = A[g+8][4t .. 4t+3], a2 = A[g][16+4t ..], a3 = A[g+8][16+4t ..]   (one byte per k)
//   B: b0 = B[4t .. 4t+3][g], b1 = B[16+4t ..][g]                       C: c0, c1 = C[g][2t, 2t+1], c2, c3 = C[g+8][2t, 2t+1].
// Native on this part: it issues every 8 cycles per SM sub-core like the fp16 m16n8k16, for twice the k. (The e4m3
// form of the same shape is emulated: measured with live operands it is slower than the fp16 one.)
DEVI void mma16832_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Bytes of one (16-row tile, 128-column unit) block of the tile layout (gemv_tile_repack_kernel): 512 B for row
// slots 0-7 (lane l's 16 bytes at 16 l), 512 B for row slots 8-15, 16 x (scale, zero).
constexpr int kTileUnitBytes = 1088;

// Order key for greedy argmax over fp16 logits: larger value wins, then the lower index. One max-reduction
// over these keys settles value and tie-break together.
DEVI unsigned long long argmax_key(half v, int idx) {
  uint32_t b = (uint32_t)__half_as_ushort(v);
  b = (b & 0x8000u) ? (~b & 0xFFFFu) : (b | 0x8000u);  // monotone map of fp16 bits to unsigned order
  return ((unsigned long long)b << 32) | (uint32_t)(0x7FFFFFFF - idx);
}

}  // namespace b200
