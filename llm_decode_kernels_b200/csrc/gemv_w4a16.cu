// W4A16 GEMV with fused nibble unpack and per-group scale/zero:  y[N] = dequant(W)[N,K] . x[K]
//
// Replaces the launcher gemv_w4a16_launch of the reference (kernels/gemv_w4a16.cu:111-130, called from
// kernels/bindings.cpp:27-38). Same data layout: packed int32 [N, K/8], (scale, zero) half2 [N, K/G],
// x fp16 [K], y fp16 [N]; fp32 accumulation across 32-weight chunks.
//
// Work split: one warp owns R consecutive rows over the whole K, lane l owns the 16-byte chunks
// l, l+32, ... of each row (one chunk = 32 weights, always inside one group because G >= 32). The block
// first stages x into shared memory, pre-scaled as dot_word() wants it, so the inner loop needs no
// activation arithmetic and x is read from L2 once per block instead of once per row. All weight
// loads of an unrolled step (R rows x UNR chunks, 16 bytes each) are issued before any is consumed.
//
// Arithmetic per 32-weight chunk: four packed words -> 16 half2 FMAs of exact integers (q - z) times
// pre-scaled activations into four independent half2 accumulators, summed, converted to fp32 and
// multiplied by the group scale once. The scale is therefore applied to the group's partial sum and
// not to each weight; `dequant_w4a16` below materialises the per-element weights for the bit-exact
// check of the format.
#include "common.cuh"

namespace b200 {

// Rows-per-warp R and weight chunks in flight UNR are compile-time; warps per block is the block size.
template <int R, int UNR>
__global__ void __launch_bounds__(256)
gemv_w4a16_kernel(const uint4* __restrict__ Wp, const half2* __restrict__ SZ, const uint4* __restrict__ X,
                  half* __restrict__ y, int N, int K, int log2G) {
  extern __shared__ uint4 xs[];  // K/8 chunks of 8 pre-scaled activations
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int U = K >> 5;          // 16-byte weight chunks per row
  const int ng = K >> log2G;     // groups per row
  for (int i = threadIdx.x; i < (K >> 3); i += blockDim.x) xs[i] = scale_x8(__ldg(X + i));
  __syncthreads();

  const int row0 = (blockIdx.x * nwarps + warp) * R;
  if (row0 >= N) return;
  const uint4* wrow[R];
  const half2* szrow[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int rr = min(row0 + r, N - 1);  // rows past the end repeat the last row; their result is dropped
    wrow[r] = Wp + (size_t)rr * U;
    szrow[r] = SZ + (size_t)rr * ng;
  }
  const half2 k1024 = __float2half2_rn(1024.f), k16 = __float2half2_rn(16.f);
  float acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = 0.f;

  for (int u0 = lane; u0 < U; u0 += 32 * UNR) {
    uint4 wv[UNR][R];
#pragma unroll
    for (int j = 0; j < UNR; ++j) {
      const int u = min(u0 + 32 * j, U - 1);
#pragma unroll
      for (int r = 0; r < R; ++r) wv[j][r] = ld_stream(wrow[r] + u);
    }
#pragma unroll
    for (int j = 0; j < UNR; ++j) {
      const int u = u0 + 32 * j;
      if (u < U) {
        const int g = (u << 5) >> log2G;
        const uint4 xa = xs[4 * u], xb = xs[4 * u + 1], xc = xs[4 * u + 2], xd = xs[4 * u + 3];
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const half2 sz = __ldg(szrow[r] + g);
          const half2 z2 = __half2half2(__high2half(sz));
          const half2 zl = __hadd2(z2, k1024), zh = __hfma2(z2, k16, k1024);
          const half2 zero2 = __float2half2_rn(0.f);
          const half2 a0 = dot_word(wv[j][r].x, xa.x, xa.y, xa.z, xa.w, zl, zh, zero2);
          const half2 a1 = dot_word(wv[j][r].y, xb.x, xb.y, xb.z, xb.w, zl, zh, zero2);
          const half2 a2 = dot_word(wv[j][r].z, xc.x, xc.y, xc.z, xc.w, zl, zh, zero2);
          const half2 a3 = dot_word(wv[j][r].w, xd.x, xd.y, xd.z, xd.w, zl, zh, zero2);
          const float2 f = __half22float2(__hadd2(__hadd2(a0, a1), __hadd2(a2, a3)));
          acc[r] = fmaf(f.x + f.y, __low2float(sz), acc[r]);
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const float v = warp_sum(acc[r]) * kDotWordRescale;
    if (lane == 0 && row0 + r < N) y[row0 + r] = __float2half(v);
  }
}

// One thread per weight, one warp per row, scalar nibble extraction, fp32 products of the fp16-rounded
// weight: the slow, obviously-correct form kept in-tree as a second opinion (API stage 0).
__global__ void gemv_w4a16_plain_kernel(const uint32_t* __restrict__ Wp, const half2* __restrict__ SZ,
                                        const half* __restrict__ x, half* __restrict__ y, int N, int K,
                                        int log2G) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= N) return;
  const int words = K >> 3, ng = K >> log2G;
  float acc = 0.f;
  for (int j = lane; j < words; j += 32) {
    const uint32_t w = Wp[(size_t)row * words + j];
    const half2 sz = SZ[(size_t)row * ng + ((j << 3) >> log2G)];
    const float s = __low2float(sz), z = __high2float(sz);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int q = (w >> (4 * (e >> 1) + 16 * (e & 1))) & 0xF;
      acc = fmaf(__half2float(__float2half(((float)q - z) * s)), __half2float(x[(j << 3) + e]), acc);
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) y[row] = __float2half(acc);
}

// out[N, K] fp16 = hmul(hsub(1024 + q, 1024 + z), scale): the per-element weight every kernel of
// this library stands for, bit-identical to quant.dequantize (reference runtime/quant.py:93-97).
// One thread per packed word.
__global__ void dequant_w4a16_kernel(const uint32_t* __restrict__ Wp, const half2* __restrict__ SZ,
                                     uint4* __restrict__ out, int N, int K, int log2G) {
  const int words = K >> 3, ng = K >> log2G;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)N * words) return;
  const int row = (int)(i / words), j = (int)(i % words);
  const uint32_t w = Wp[i];
  const half2 sz = SZ[(size_t)row * ng + ((j << 3) >> log2G)];
  const half2 s2 = __half2half2(__low2half(sz));
  const half2 zl = __hadd2(__half2half2(__high2half(sz)), __float2half2_rn(1024.f));
  uint4 o;
  o.x = as_u32(__hmul2(__hsub2(nib_lo(w), zl), s2));
  o.y = as_u32(__hmul2(__hsub2(nib_lo(w >> 4), zl), s2));
  o.z = as_u32(__hmul2(__hsub2(nib_lo(w >> 8), zl), s2));
  o.w = as_u32(__hmul2(__hsub2(nib_lo(w >> 12), zl), s2));
  out[i] = o;
}

template <int R, int UNR>
static cudaError_t launch_rows(const void* Wp, const void* SZ, const void* x, void* y, int N, int K, int log2G,
                               int warps, cudaStream_t st) {
  const int rows_per_block = R * warps;
  const int blocks = (N + rows_per_block - 1) / rows_per_block;
  const size_t smem = (size_t)K * 2;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(gemv_w4a16_kernel<R, UNR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return e;
  }
  gemv_w4a16_kernel<R, UNR><<<blocks, 32 * warps, smem, st>>>((const uint4*)Wp, (const half2*)SZ, (const uint4*)x,
                                                              (half*)y, N, K, log2G);
  return cudaPeekAtLastError();
}

// stage 0: plain kernel. stage >= 1 with R in {1,2,4,8} and warps in 1..8: that configuration.
// Anything else (R == 0): a shape-based choice - enough warps to cover 148 SMs several times over for
// small N, more rows per warp (fewer reads of x from shared memory per weight byte) for large N.
cudaError_t gemv_w4a16_dispatch(int stage, int R, int warps, const void* Wp, const void* SZ, const void* x, void* y,
                                int N, int K, int log2G, cudaStream_t st) {
  if (stage == 0) {
    const int w = (warps >= 1 && warps <= 8) ? warps : 4;
    gemv_w4a16_plain_kernel<<<(N + w - 1) / w, 32 * w, 0, st>>>((const uint32_t*)Wp, (const half2*)SZ,
                                                                 (const half*)x, (half*)y, N, K, log2G);
    return cudaPeekAtLastError();
  }
  if (!(R == 1 || R == 2 || R == 4 || R == 8) || warps < 1 || warps > 8) {
    if (N >= 16384) { R = 4; warps = 8; }
    else if (N >= 4096) { R = 2; warps = 8; }
    else { R = 2; warps = 4; }
  }
  switch (R) {
    case 1: return launch_rows<1, 4>(Wp, SZ, x, y, N, K, log2G, warps, st);
    case 2: return launch_rows<2, 4>(Wp, SZ, x, y, N, K, log2G, warps, st);
    case 4: return launch_rows<4, 2>(Wp, SZ, x, y, N, K, log2G, warps, st);
    default: return launch_rows<8, 1>(Wp, SZ, x, y, N, K, log2G, warps, st);
  }
}

cudaError_t dequant_w4a16_dispatch(const void* Wp, const void* SZ, void* out, int N, int K, int log2G,
                                   cudaStream_t st) {
  const size_t words = (size_t)N * (K >> 3);
  dequant_w4a16_kernel<<<(unsigned)((words + 255) / 256), 256, 0, st>>>((const uint32_t*)Wp, (const half2*)SZ,
                                                                        (uint4*)out, N, K, log2G);
  return cudaPeekAtLastError();
}

}  // namespace b200
