// W4A16 GEMV with fused nibble unpack and per-group scale/zero:  y[N] = dequant(W)[N,K] . x[K]
//
// Replaces the launcher gemv_w4a16_launch of the reference (kernels/gemv_w4a16.cu:111-130, called from
// kernels/bindings.cpp:27-38). Same data layout: packed int32 [N, K/8], (scale, zero) half2 [N, K/G],
// x fp16 [K], y fp16 [N]; fp32 accumulation across 32-weight chunks.
//
// Four kernels, in the order they were written; each later one exists because a measurement said so:
//   gemv_w4a16_plain_kernel  (stage 0)   one thread per weight, the readable baseline
//   gemv_w4a16_kernel<R,UNR> (R 1..8)    rows per warp, magic-number nibble decode, described next
//   gemv_w4a16_seg_kernel    (R = 16)    segmented, x in registers, nibbles multiplied as fp16 subnormals
//   gemv_w4a16_mma_kernel    (R = 0)     the default: masked nibbles as tensor-core operands, optional tile layout,
//                                        SwiGLU epilogue and residual add + RMSNorm prologue
//
// Rows-per-warp kernel. Work split: one warp owns R consecutive rows over the whole K, lane l owns the 16-byte chunks
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
#include "tp_comm.cuh"

namespace b200 {

// Rows-per-warp R and weight chunks in flight UNR are compile-time; warps per block is the block size.
template <int R, int UNR>
__global__ void __launch_bounds__(256)
gemv_w4a16_kernel(const uint4* __restrict__ Wp, const half2* __restrict__ SZ, const uint4* __restrict__ X,
                  half* __restrict__ y, int N, int K, int log2G) {
  pdl_launch_dependents();
  pdl_wait();
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
  pdl_launch_dependents();
  pdl_wait();
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

// ---- segmented GEMV (R = 16): the fastest CUDA-core kernel ---------------------------------------------------------------
// Same arithmetic as the GEMV phases of the persistent step kernel (masked nibbles as fp16 subnormals, zero point
// folded into one FMA per chunk; see common.cuh), laid out for one launch per matrix:
//   * a CTA of 8 warps owns a tile of consecutive units (unit = two consecutive rows);
//   * a row is cut into segments of 32 chunks (1024 weights); warp w works on segment w mod segs for the whole tile,
//     lane l on chunk l of it, so the lane's 32 activations are read from shared memory once per tile and stay in
//     registers; the warps sharing a segment take the tile's units round robin, two units (four rows) per trip;
//   * weights come straight from global memory with 128-bit streaming loads, the next trip's four loads issued before
//     the current trip's arithmetic; (scale, zero) words through the read-only cache;
//   * four partial sums per trip are reduced with 7 shuffles into shared memory; after one barrier per tile a thread
//     per unit adds the segments in order and stores two fp16 results.
// x is staged by every CTA itself: max|x| -> power-of-two scale -> scaled copy + per-chunk sums (4-16 KB from L2).
constexpr int kSegWarps = 8, kSegThreads = kSegWarps * 32;

struct SegRows { uint4 a0, a1, b0, b1; half2 za0, za1, zb0, zb1; };

__global__ void __launch_bounds__(kSegThreads)
gemv_w4a16_seg_kernel(const uint4* __restrict__ Wp, const half2* __restrict__ SZ, const uint2* __restrict__ X,
                      half* __restrict__ y, int N, int K, int log2G, int tile_units) {
  extern __shared__ __align__(16) uint8_t seg_smem[];
  const int U = K >> 5, ng = K >> log2G, segs = (U + 31) >> 5;
  uint4* xin = reinterpret_cast<uint4*>(seg_smem);                       // [K/8] scaled, swizzled
  float* xsum = reinterpret_cast<float*>(seg_smem + (size_t)K * 2);      // [U]
  float* part = xsum + U;                                                 // [tile_units * 2][segs]
  __shared__ float red[kSegWarps];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  pdl_launch_dependents();

  // ---- this CTA's tile and this warp's share of it
  const int units = (N + 1) >> 1;
  const int ub = blockIdx.x * tile_units, ue = min(units, ub + tile_units);
  if (ub >= ue) return;   // (CTA-uniform: taken by all threads or none, before any barrier)
  const int seg_first = warp % segs;                     // segs <= 8: one segment per warp; else several, strided
  const bool resident = segs <= kSegWarps;
  const int group = resident ? (kSegWarps - seg_first + segs - 1) / segs : 1;
  const int rank = resident ? warp / segs : 0;
  const size_t rowU = (size_t)U;

  auto x_of = [&](int u) {
    const int sw = (u >> 1) & 3;
    XChunk r;
    r.x0 = xin[4 * u + (0 ^ sw)]; r.x1 = xin[4 * u + (1 ^ sw)]; r.x2 = xin[4 * u + (2 ^ sw)]; r.x3 = xin[4 * u + (3 ^ sw)];
    r.xs = xsum[u];
    return r;
  };
  // ---- staging of x (run by the whole CTA, once, after the first weight loads have been issued)
  XScale sc;
  auto stage_x_all = [&]() {
    uint2* raw = reinterpret_cast<uint2*>(xin);
    float mx = 0.f;
    for (int g = tid; g < (K >> 2); g += kSegThreads) {
      const uint2 v = __ldg(X + g);
      raw[2 * swz(g >> 1) + (g & 1)] = v;
      const float2 a = __half22float2(__habs2(as_h2(v.x))), b = __half22float2(__habs2(as_h2(v.y)));
      mx = fmaxf(mx, fmaxf(fmaxf(a.x, a.y), fmaxf(b.x, b.y)));
    }
    mx = warp_max(mx);
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    float xmax = 0.f;
  #pragma unroll
    for (int k = 0; k < kSegWarps; ++k) xmax = fmaxf(xmax, red[k]);
    sc = scale_for(xmax);
    const int ngran = K >> 2;
    for (int g0 = 0; g0 < ngran; g0 += kSegThreads) {   // whole warps take part in the shuffles below
      const int g = g0 + tid;
      const bool live = g < ngran;
      const uint2 v = live ? raw[2 * swz(g >> 1) + (g & 1)] : make_uint2(0u, 0u);
      const float2 a = __half22float2(as_h2(v.x)), b = __half22float2(as_h2(v.y));
      float sm = (a.x + a.y) + (b.x + b.y);
      sm += __shfl_xor_sync(0xffffffffu, sm, 1);
      sm += __shfl_xor_sync(0xffffffffu, sm, 2);
      sm += __shfl_xor_sync(0xffffffffu, sm, 4);
      if (live && (tid & 7) == 0) xsum[g >> 3] = sm;
      uint2 o;
      o.x = as_u32(__hmul2(as_h2(v.x), sc.lo));
      o.y = as_u32(__hmul2(as_h2(v.y), sc.hi));
      if (live) raw[2 * swz(g >> 1) + (g & 1)] = o;
    }
    __syncthreads();

  };

  const int nu = ue - ub;
  bool staged = false;
  for (int seg = seg_first; seg < segs; seg += kSegWarps) {
    const int u = 32 * seg + lane;
    const bool act = u < U;
    const int uc = act ? u : U - 1, g = (uc << 5) >> log2G;
    // Running pointers to row 0 of the trip's two units; a trip advances them by 2 * group units = 4 * group rows.
    // Loads are predicated on the unit being inside the tile (and the odd row inside the matrix), so no clamping.
    const size_t wstep = (size_t)4 * group * rowU, zstep = (size_t)4 * group * ng;
    const uint4* wa = Wp + (size_t)(2 * (ub + rank)) * rowU + uc;
    const half2* za = SZ + (size_t)(2 * (ub + rank)) * ng + g;
    const uint4* wb = wa + (size_t)2 * group * rowU;
    const half2* zb = za + (size_t)2 * group * ng;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    const half2 zeroh = __float2half2_rn(0.f);
    const int last_row = N - 1;

#define SEG_LOAD(R, j)                                                                           \
  {                                                                                              \
    const bool ua_ = (j) < nu, ub_ = (j) + group < nu;                                           \
    const bool ua1_ = ua_ && 2 * (ub + (j)) + 1 <= last_row;                                     \
    const bool ub1_ = ub_ && 2 * (ub + (j) + group) + 1 <= last_row;                             \
    R.a0 = ua_ ? ld_stream(wa) : zero4;                                                          \
    R.a1 = ua1_ ? ld_stream(wa + rowU) : zero4;                                                  \
    R.b0 = ub_ ? ld_stream(wb) : zero4;                                                          \
    R.b1 = ub1_ ? ld_stream(wb + rowU) : zero4;                                                  \
    R.za0 = ua_ ? __ldg(za) : zeroh;                                                             \
    R.za1 = ua1_ ? __ldg(za + ng) : zeroh;                                                       \
    R.zb0 = ub_ ? __ldg(zb) : zeroh;                                                             \
    R.zb1 = ub1_ ? __ldg(zb + ng) : zeroh;                                                       \
    wa += wstep; wb += wstep; za += zstep; zb += zstep;                                          \
  }
#define SEG_TRIP(R, j)                                                                           \
  {                                                                                              \
    float p0 = 0.f, p1 = 0.f, q0 = 0.f, q1 = 0.f;                                                \
    if (act) {                                                                                   \
      chunk_two_rows(R.a0, R.a1, R.za0, R.za1, x, sc.resc, p0, p1);                              \
      if ((j) + group < nu) chunk_two_rows(R.b0, R.b1, R.zb0, R.zb1, x, sc.resc, q0, q1);        \
    }                                                                                            \
    const int qd = lane >> 3; /* 4 sums with 7 shuffles: quarter qd of the warp ends up holding value qd */ \
    float v0 = (qd & 2) ? q0 : p0, v1 = (qd & 2) ? q1 : p1;                                      \
    const float o0 = (qd & 2) ? p0 : q0, o1 = (qd & 2) ? p1 : q1;                                \
    v0 += __shfl_xor_sync(0xffffffffu, o0, 16);                                                  \
    v1 += __shfl_xor_sync(0xffffffffu, o1, 16);                                                  \
    float v = (qd & 1) ? v1 : v0;                                                                \
    v += __shfl_xor_sync(0xffffffffu, (qd & 1) ? v0 : v1, 8);                                    \
    v += __shfl_xor_sync(0xffffffffu, v, 4);                                                     \
    v += __shfl_xor_sync(0xffffffffu, v, 2);                                                     \
    v += __shfl_xor_sync(0xffffffffu, v, 1);                                                     \
    const int jj = (j) + ((qd & 2) ? group : 0);                                                 \
    if ((lane & 7) == 0 && jj < nu) part[(jj * 2 + (qd & 1)) * segs + seg] = v;                  \
  }

    // two register buffers used alternately: the loads of the next trip are in flight during the arithmetic of this
    // one, and no buffer is ever copied
    SegRows r0, r1;
    int j = rank;
    if (j < nu) SEG_LOAD(r0, j);
    if (!staged) {   // the weights just requested travel while x is staged (two barriers, one L2 round trip)
      pdl_wait();    // weights do not depend on the previous kernel, x does: from here on it may be read
      stage_x_all();
      staged = true;
    }
    const XChunk x = x_of(uc);
    for (; j < nu; j += 4 * group) {
      const int j1 = j + 2 * group;
      if (j1 < nu) SEG_LOAD(r1, j1);
      SEG_TRIP(r0, j);
      if (j1 < nu) {
        if (j1 + 2 * group < nu) SEG_LOAD(r0, j1 + 2 * group);
        SEG_TRIP(r1, j1);
      }
    }
#undef SEG_LOAD
#undef SEG_TRIP
  }
  __syncthreads();
  for (int i = tid; i < nu; i += kSegThreads) {
    float y0 = 0.f, y1 = 0.f;
    for (int k = 0; k < segs; ++k) { y0 += part[(2 * i) * segs + k]; y1 += part[(2 * i + 1) * segs + k]; }
    const int row0 = 2 * (ub + i);
    if (row0 + 1 < N) *reinterpret_cast<half2*>(y + row0) = __floats2half2_rn(y0, y1);
    else y[row0] = __float2half(y0);
  }
}

static cudaError_t launch_seg(const void* Wp, const void* SZ, const void* x, void* y, int N, int K, int log2G,
                              cudaStream_t st) {
  const int units = (N + 1) / 2, U = K >> 5, segs = (U + 31) / 32;
  int tile = (units + 2 * kNumSMs - 1) / (2 * kNumSMs);   // one wave of two CTAs per SM ...
  tile = tile < 8 ? 8 : (tile > 512 ? 512 : tile);          // ... but at least 16 rows
  const int blocks = (units + tile - 1) / tile;
  const size_t smem = (size_t)K * 2 + (size_t)U * 4 + (size_t)tile * 2 * segs * 4;
  static size_t allowed[kMaxDevices] = {};
  const cudaError_t e = allow_dynamic_smem(gemv_w4a16_seg_kernel, smem, allowed);
  if (e != cudaSuccess) return e;
  return launch_pdl(gemv_w4a16_seg_kernel, dim3(blocks), dim3(kSegThreads), smem, st, (const uint4*)Wp, (const half2*)SZ,
                    (const uint2*)x, (half*)y, N, K, log2G, tile);
}

// ---- tensor-core GEMV: the library's default where the shape allows -------------------------------------------------------
// The CUDA-core kernels above spend ~3.6 issued instructions per weight (mask, shift, half2 FMA, conversions, shuffles)
// and are bound by instruction issue at 45-60 % of the HBM bandwidth of this part. This kernel does the inner product
// on the INTEGER tensor cores. (word & 0x0F0F0F0F) and ((word >> 4) & 0x0F0F0F0F) are registers of four unsigned-byte
// weights each - three integer instructions for 8 weights - so a 16-row x 128-weight block of W is four
// mma.m16n8k32 (u8 x s8 -> s32) whose A registers are masked words. The activations go in as 15-bit fixed point:
// staging scales a 128-element unit of x by 2^s (s from the unit's max|x|), rounds to an integer X, |X| < 2^14, and
// splits it into two signed byte digits, X = 256 hi + lo, which ride in columns 0 and 1 of the B operand (a batch-1
// GEMV leaves the B columns idle anyway). The accumulation is exact, and scale and zero point are applied once per
// unit:
//     y += scale * (2^-s * (256 C[.][0] + C[.][1]) - zero * sum_unit(x)).
// Rounding x to 2^-14 of its unit's maximum is finer than the fp16 rounding x already carries, except for elements
// far below the maximum, whose absolute error it bounds by 2^-15 of the maximum. A NaN or infinity in a unit of x
// turns that unit's factor 2^-s into NaN, so every row's output is NaN as in the reference's arithmetic.
// An earlier form fed the masked nibbles to mma.m16n8k16 as fp16 subnormals (q * 2^-24, q * 2^-20): five mask/shift
// instructions per 8 weights on the half-rate integer pipe, which bound it at 0.72 of the copy bandwidth on the 70B
// gate|up matrix; this form reaches 0.82 there and waits for memory instead.
//   lane (g = lane / 4, t = lane % 4) loads 16 bytes (32 weights: words 4t .. 4t+3 of the unit) of row g and of row
//   g + 8; lanes (0, t) carry the hi digits of the matching 32 activations as the B operand, lanes (1, t) the lo
//   digits, the other lanes zeros.
// A block of 8 warps stages x once and walks row tiles of 16 rows; `ksplit` warps share a tile by splitting K (small
// matrices need the parallelism) and meet in shared memory, with ksplit = 1 a warp owns its tile and there is no
// barrier in the loop. Needs K % 128 == 0 and a group size that is a multiple of 128.
constexpr int kMmaGemvWarps = 8, kMmaGemvThreads = kMmaGemvWarps * 32;

// A batch = 4 consecutive 128-weight units of two rows and their (scale, zero). A lane's four 16-byte loads per row
// are 64 bytes apart, so the warp's loads of a batch cover 256 contiguous bytes of each of its 16 rows, issued back to
// back (row-buffer locality in DRAM), and 8 loads per lane are in flight per batch.
constexpr int kMmaBatch = 4;
struct MmaBatchRegs { uint4 wa[kMmaBatch], wb[kMmaBatch]; half2 sa[kMmaBatch], sb[kMmaBatch]; };

//
// TILED = true reads the weights from the tile layout made by gemv_tile_repack_kernel instead of the quantizer's
// row-major tensors. Row-major, the 16 rows of a tile are K/2 bytes apart and every load instruction of a warp touches
// 16 separate 64-byte pieces; measured on 134 MB matrices the kernel then moves 4.6 TB/s with 512-byte rows but only
// 3.4 TB/s with 8 KB rows (DRAM sees scattered short bursts). In the tile layout the bytes of a tile are stored in
// the order the warp consumes them: per 128-weight unit 512 bytes for rows g (lane l at 16 l), 512 bytes for rows
// g + 8, then the 16 rows' (scale, zero) - 1088 bytes, units and tiles back to back - so every warp load is one
// contiguous 512-byte read and a warp streams through memory in address order.

//
// SWIGLU = true (tile layout only): the matrix is [gate; up] and the repack has put gate row i and up row i into the
// same tile (slots g and g + 8), so the lane that ends up with gate_i also holds up_i and the epilogue stores
// half(silu(gate_i)) * up_i - the rounding of swiglu_kernel - instead of the two sums: one launch and 3/4 of the
// output traffic less per layer. N is then the number of OUTPUTS (the matrix has 2 N rows).
//
// NORM = true: the residual add and RMSNorm that precede the GEMV in a decoder layer run inside the staging of x,
// in every block (K values: nothing next to the weights the block streams), with the rounding of add_rmsnorm_kernel:
//     r = X +_fp16 delta (delta may be null);  x = nw *_fp16 half(float(r) * rsqrt(mean(r^2) + eps));  y = W x
// Block 0 also stores r to x_out, the residual stream for the rest of the layer. x_out must not alias X: the other
// blocks are still reading X. One launch less in front of the qkv, the gate|up and the LM-head GEMV.
struct NormArgs {
  const uint2* delta;   // [K] fp16 or null
  const uint2* nw;      // [K] fp16 norm weight
  uint2* x_out;         // [K] fp16
  float eps;
};

//
// ALLRED = true (tile layout, tensor-parallel row-split projections o_proj / down_proj): the kernel's rows are this
// rank's PARTIAL sums, and they leave the kernel over NVLink instead of through y. The block that has computed a tile
// group's rows rounds them to fp16 and stores them as 32-bit words (tag << 16 | row), tag = the slot's call number,
// into words[rank][row] of EVERY rank's exchange region (its own included): plain 16-byte peer stores. A word that
// carries the call's tag is its own arrival flag - no flag round, no fence. Then either
//   * tagged = 1 (b200_gemv_w4a16_tiled_push): the kernel is done; tp_pushed_add_rmsnorm_kernel on every rank polls
//     its own region, sums and goes on with residual add + RMSNorm; or
//   * tagged = 0 (b200_gemv_w4a16_tiled_allreduce): after its last round the block collects the rows of its own
//     tile groups from its OWN region - the peers' blocks of the same index push exactly those (the ranks launch the
//     same grid) -, polling each word until it carries the tag (bounded), adds the W copies in rank order with fp32
//     accumulation, rounds once and stores the sums to y: bit-identical on all ranks. The last block of the grid
//     moves the slot's call counter on.
// Slot reuse: a rank reaches call c + 1 on a slot only after another exchange has completed in between (the o_proj
// and down_proj slots alternate, and the logits gather follows the last layer), which every peer can only have joined
// after it was done reading this slot. N % 8 == 0. A wait that runs out sets the block's error word and leaves y's
// rows alone.
template <bool TILED, bool SWIGLU, bool NORM, bool ALLRED>
__global__ void __launch_bounds__(kMmaGemvThreads, 2)
gemv_w4a16_mma_kernel(const uint4* __restrict__ Wp, const half2* __restrict__ SZ, const uint2* __restrict__ X,
                      half* __restrict__ y, int N, int K, int log2G, int ksplit, int rounds, const NormArgs na,
                      const AllReduceArgs ar) {
  extern __shared__ __align__(16) uint8_t mma_smem[];
  const int nunit = K >> 7;                                                // 128-weight units per row
  uint4* xin = reinterpret_cast<uint4*>(mma_smem);                         // [K/8]: per unit 256 bytes of byte digits
  float* part = reinterpret_cast<float*>(xin + (K >> 3) + 4);              // [kMmaGemvWarps][16]
  float* xsg = part + kMmaGemvWarps * 16;                                  // [nunit][2]: 2^-s sum X and 2^-s per unit
  __shared__ float red2[kMmaGemvWarps];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  pdl_launch_dependents();

  const int ntiles = SWIGLU ? (N + 7) >> 3 : (N + 15) >> 4, tiles_per_round = kMmaGemvWarps / ksplit;
  const int kpart = warp % ksplit, tslot = warp / ksplit;
  const int ub = (int)(((long long)nunit * kpart) / ksplit), ue = (int)(((long long)nunit * (kpart + 1)) / ksplit);
  const int ng = K >> log2G, rowU4 = K >> 5;   // (scale, zero) entries and 16-byte pieces per row
  const int last = N - 1;

  const int tile_step = gridDim.x * tiles_per_round;   // round r: tile groups r * gridDim.x + blockIdx.x
  int tile = blockIdx.x * tiles_per_round + tslot;
  // Running pointers of the batch that will be loaded next: rows g and g + 8 of a tile (rows past the end repeat the
  // last one), this lane's 16-byte piece of unit u. `full` batches need no predicate; the host gives every warp a
  // K range that is a whole number of batches whenever K allows.
  const uint4 *pa, *pb;
  const half2 *za, *zb;
  auto seek = [&](int tl) {
    if (TILED) {   // Wp is the tile layout; SZ is unused
      const uint8_t* base = reinterpret_cast<const uint8_t*>(Wp) + ((size_t)tl * nunit + ub) * kTileUnitBytes;
      pa = reinterpret_cast<const uint4*>(base) + lane;
      pb = pa + 32;
      za = reinterpret_cast<const half2*>(base + 1024) + g;
      zb = za + 8;
    } else {
      const int ra = min(16 * tl + g, last), rb = min(16 * tl + g + 8, last);
      pa = Wp + (size_t)ra * rowU4 + 4 * ub + t;
      pb = Wp + (size_t)rb * rowU4 + 4 * ub + t;
      za = SZ + (size_t)ra * ng;
      zb = SZ + (size_t)rb * ng;
    }
  };
  auto load = [&](int u0, MmaBatchRegs& d) {
    constexpr int step = TILED ? kTileUnitBytes / 16 : 4;   // 16-byte pieces from one unit to the next
#pragma unroll
    for (int i = 0; i < kMmaBatch; ++i) {
      if (u0 + i < ue) {
        d.wa[i] = ld_stream(pa + step * i);
        d.wb[i] = ld_stream(pb + step * i);
        if (TILED) {
          d.sa[i] = __ldg(za + (kTileUnitBytes / 4) * i);
          d.sb[i] = __ldg(zb + (kTileUnitBytes / 4) * i);
        } else {
          const int gi = ((u0 + i) << 7) >> log2G;
          d.sa[i] = __ldg(za + gi);
          d.sb[i] = __ldg(zb + gi);
        }
      }
    }
    pa += step * kMmaBatch;
    pb += step * kMmaBatch;
    if (TILED) {
      za += (kTileUnitBytes / 4) * kMmaBatch;
      zb += (kTileUnitBytes / 4) * kMmaBatch;
    }
  };
  // the first weights travel while x is staged: they do not depend on the previous kernel, x does
  MmaBatchRegs cur, nxt;
  if (tile < ntiles) {
    seek(tile);
    load(ub, cur);
  }
  pdl_wait();

  // ---- stage x: (residual add + RMSNorm ->) per 128-element unit: 15-bit fixed point X = round(x 2^s), s from the
  // unit's max|x|, split into two signed byte digits laid out as the B fragments of the integer MMAs, and the unit's
  // 2^-s sum X and 2^-s. One warp per unit, lane = granule of 4 activations; no block-wide maximum, no barrier before
  // the units can be written.
  // xin words [unit][digit n = 0 (hi), 1 (lo)][t = 0..3][MMA m = 0..3][register r = 0..1]: lane (n, t) of the MMA loop
  // loads its eight registers with two 16-byte reads. Register r of MMA m pairs with word 2 (m / 2) + r of the lane's
  // four weight words, low nibbles (m even: elements e0 e4 e1 e5 of the word, in byte order) or high nibbles (m odd:
  // e2 e6 e3 e7). Granule l = 4 elements of word (l % 8) / 2: e0..e3 on even lanes, e4..e7 on odd ones.
  auto put_unit = [&](int u, uint2 v) {
    const uint32_t m2 = __vmaxu2(v.x & 0x7FFF7FFFu, v.y & 0x7FFF7FFFu);   // max |x| from the fp16 bit patterns
    const uint32_t mxb = __reduce_max_sync(0xffffffffu, max(m2 & 0xFFFFu, m2 >> 16));
    const bool finite = mxb < 0x7C00u;
    const int sh = 28 - max((int)(mxb >> 10), 1);             // 2^sh max|x| in [2^13, 2^14)
    const float scl = __int_as_float((sh + 127) << 23);
    constexpr float kMagic = 12582912.f + 128.f;              // 1.5 2^23 + 128: rounds to an integer, offset for the lo digit
    const float2 a = __half22float2(as_h2(v.x)), b = __half22float2(as_h2(v.y));
    const uint32_t w0 = __float_as_uint(fmaf(a.x, scl, kMagic)), w1 = __float_as_uint(fmaf(a.y, scl, kMagic));
    const uint32_t w2 = __float_as_uint(fmaf(b.x, scl, kMagic)), w3 = __float_as_uint(fmaf(b.y, scl, kMagic));
    const uint32_t kM = __float_as_uint(kMagic);
    const int xsum_i = __reduce_add_sync(0xffffffffu, (int)(w0 - kM) + (int)(w1 - kM) + (int)(w2 - kM) + (int)(w3 - kM));
    const float resc = finite ? __int_as_float((127 - sh) << 23) : __int_as_float(0x7fc00000);   // 2^-sh, or NaN
    if (lane == 0) {
      xsg[2 * u] = (float)xsum_i * resc;
      xsg[2 * u + 1] = resc;
    }
    const uint32_t lo = __byte_perm(__byte_perm(w0, w1, 0x0040), __byte_perm(w2, w3, 0x0040), 0x5410) ^ 0x80808080u;
    const uint32_t hi = __byte_perm(__byte_perm(w0, w1, 0x0051), __byte_perm(w2, w3, 0x0051), 0x5410);
    const int tt = lane >> 3, wd = (lane & 7) >> 1, odd = lane & 1;
    uint32_t* dst = reinterpret_cast<uint32_t*>(xin) + (size_t)u * 64 + tt * 8 + ((wd >> 1) * 2 + odd) * 2 + (wd & 1);
    const uint32_t hi_o = __shfl_xor_sync(0xffffffffu, hi, 1), lo_o = __shfl_xor_sync(0xffffffffu, lo, 1);
    dst[0] = odd ? __byte_perm(hi, hi_o, 0x3726) : __byte_perm(hi, hi_o, 0x5140);
    dst[32] = odd ? __byte_perm(lo, lo_o, 0x3726) : __byte_perm(lo, lo_o, 0x5140);
  };
  if (NORM) {
    float ss = 0.f;
    for (int i = tid; i < (K >> 2); i += kMmaGemvThreads) {
      uint2 v = __ldg(X + i);
      if (na.delta) {
        const uint2 d = __ldg(na.delta + i);
        v.x = as_u32(__hadd2(as_h2(v.x), as_h2(d.x)));
        v.y = as_u32(__hadd2(as_h2(v.y), as_h2(d.y)));
      }
      reinterpret_cast<uint2*>(xin)[i] = v;
      if (blockIdx.x == 0) na.x_out[i] = v;
      const float2 a = __half22float2(as_h2(v.x)), b = __half22float2(as_h2(v.y));
      ss = fmaf(a.x, a.x, fmaf(a.y, a.y, fmaf(b.x, b.x, fmaf(b.y, b.y, ss))));
    }
    ss = warp_sum(ss);
    if (lane == 0) red2[warp] = ss;
    __syncthreads();   // the residual values of every unit are in xin; the sum of squares is complete
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < kMmaGemvWarps; ++k) tot += red2[k];
    const float rinv = rsqrtf(tot / (float)K + na.eps);
    for (int u = warp; u < nunit; u += kMmaGemvWarps) {   // the unit's fp16 residual -> normalised x -> digits, in place
      const uint2 r = reinterpret_cast<uint2*>(xin)[32 * u + lane], w = __ldg(na.nw + 32 * u + lane);
      const float2 a = __half22float2(as_h2(r.x)), b = __half22float2(as_h2(r.y));
      uint2 v;
      v.x = as_u32(__hmul2(as_h2(w.x), __floats2half2_rn(a.x * rinv, a.y * rinv)));
      v.y = as_u32(__hmul2(as_h2(w.y), __floats2half2_rn(b.x * rinv, b.y * rinv)));
      __syncwarp();   // every lane has read its granule before the unit's 256 bytes are overwritten
      put_unit(u, v);
    }
  } else {
    for (int u = warp; u < nunit; u += kMmaGemvWarps) put_unit(u, __ldg(X + 32 * u + lane));
  }
  __syncthreads();

  // ALLRED: the tag of this call (the slot's call counter was last written by the kernel that closed the previous
  // call on this slot, which this stream has waited for)
  uint32_t push_tag = 0u;
  if (ALLRED)
    push_tag = comm_tag(*reinterpret_cast<const volatile uint32_t*>(ar.P.p[ar.rank] + ar.off) + 1u);
  for (int r = 0; r < rounds; ++r, tile += tile_step) {
    float ya = 0.f, yb = 0.f;
    if (tile < ntiles) {
      for (int u0 = ub; u0 < ue; u0 += kMmaBatch) {
        // the next batch's loads (this tile's, or the first of the warp's next tile) fly during this batch's arithmetic
        if (u0 + kMmaBatch < ue) {
          load(u0 + kMmaBatch, nxt);
        } else if (r + 1 < rounds && tile + tile_step < ntiles) {
          seek(tile + tile_step);
          load(ub, nxt);
        }
#pragma unroll
        for (int i = 0; i < kMmaBatch; ++i) {
          const int u = u0 + i;
          if (u < ue) {   // warp-uniform
            // B: lanes (0, t) carry the hi digits of the 32 activations that match the lane's 32 weights, lanes (1, t)
            // the lo digits, the other lanes zeros; four integer MMAs in two independent chains
            uint4 x0 = make_uint4(0u, 0u, 0u, 0u), x1 = x0;
            if (g < 2) {
              const uint4* xp = xin + (size_t)u * 16 + (g * 4 + t) * 2;
              x0 = xp[0];
              x1 = xp[1];
            }
            const uint4 wa = cur.wa[i], wb = cur.wb[i];
            constexpr uint32_t kNib = 0x0F0F0F0Fu;
            int c0[4] = {0, 0, 0, 0}, c1[4] = {0, 0, 0, 0};
            mma16832_u8s8(c0, wa.x & kNib, wb.x & kNib, wa.y & kNib, wb.y & kNib, x0.x, x0.y);
            mma16832_u8s8(c1, (wa.x >> 4) & kNib, (wb.x >> 4) & kNib, (wa.y >> 4) & kNib, (wb.y >> 4) & kNib, x0.z, x0.w);
            mma16832_u8s8(c0, wa.z & kNib, wb.z & kNib, wa.w & kNib, wb.w & kNib, x1.x, x1.y);
            mma16832_u8s8(c1, (wa.z >> 4) & kNib, (wb.z >> 4) & kNib, (wa.w >> 4) & kNib, (wb.w >> 4) & kNib, x1.z, x1.w);
            // lanes t == 0: C columns 0 (hi digits) and 1 (lo digits) of rows g (c[0], c[1]) and g + 8 (c[2], c[3])
            const float2 sa = __half22float2(cur.sa[i]), sb = __half22float2(cur.sb[i]);
            const float xs = xsg[2 * u], resc = xsg[2 * u + 1];
            const float va = (float)(((c0[0] + c1[0]) << 8) + (c0[1] + c1[1]));
            const float vb = (float)(((c0[2] + c1[2]) << 8) + (c0[3] + c1[3]));
            ya = fmaf(sa.x, fmaf(va, resc, -sa.y * xs), ya);
            yb = fmaf(sb.x, fmaf(vb, resc, -sb.y * xs), yb);
          }
        }
        cur = nxt;
      }
    }
    // SWIGLU: slot g = gate row, slot g + 8 = its up row, 8 outputs per tile
    auto gated = [](float ga, float up) {
      const half hg = __float2half(ga), hu = __float2half(up);
      const float gf = __half2float(hg);
      return __hmul(__float2half(gf / (1.f + expf(-gf))), hu);
    };
    __shared__ __align__(16) half rowbuf[kMmaGemvWarps * 16];   // ALLRED: the round's rows, in row order
    if (ksplit == 1) {
      if (t == 0 && tile < ntiles) {
        if (SWIGLU) {
          if (8 * tile + g < N) y[8 * tile + g] = gated(ya, yb);
        } else if (ALLRED) {
          rowbuf[16 * warp + g] = __float2half(ya);
          rowbuf[16 * warp + g + 8] = __float2half(yb);
        } else {
          const int ra = 16 * tile + g, rb = ra + 8;
          if (ra < N) y[ra] = __float2half(ya);
          if (rb < N) y[rb] = __float2half(yb);
        }
      }
    } else {
      if (t == 0) { part[warp * 16 + g] = ya; part[warp * 16 + g + 8] = yb; }
      __syncthreads();
      if (tid < tiles_per_round * 16) {
        const int ts = tid >> 4, row = tid & 15, tl = tile - tslot + ts;   // tile - tslot: first tile of the round
        float v = 0.f, v8 = 0.f;
        for (int k = 0; k < ksplit; ++k) {
          v += part[(ts * ksplit + k) * 16 + row];
          if (SWIGLU) v8 += part[(ts * ksplit + k) * 16 + (row | 8)];
        }
        if (SWIGLU) {
          if (row < 8 && tl < ntiles && 8 * tl + row < N) y[8 * tl + row] = gated(v, v8);
        } else if (ALLRED) {
          rowbuf[tid] = __float2half(v);
        } else if (tl < ntiles && 16 * tl + row < N) {
          y[16 * tl + row] = __float2half(v);
        }
      }
      if (!ALLRED) __syncthreads();
    }
    if (ALLRED) {
      // the tile group of pass r: tiles [gidx * tpr, (gidx + 1) * tpr), rows from row0 on, `nchunk` pieces of 8 rows:
      // pushed to every rank now; the collecting and the sum follow once, after the block's last pass
      const int gidx = r * gridDim.x + blockIdx.x, row0 = 16 * gidx * tiles_per_round;
      const int nrows = max(0, min(N - row0, 16 * tiles_per_round)), nchunk = nrows >> 3;
      __syncthreads();   // rowbuf complete
      {
        // tagged words: 8 rows = 32 bytes = two 16-byte stores per peer; a word with this call's tag is its own flag
        const size_t data_off = ar.off + kGemvSlotCtrlBytes + kGemvSlotFlagBytes + ((size_t)ar.rank * N + row0) * 4;
        for (int i = tid; i < 2 * nchunk * ar.W; i += kMmaGemvThreads) {
          const int p = i / (2 * nchunk), c = i - p * 2 * nchunk;   // c: 16-byte piece = 4 rows
          const uint2 h4 = reinterpret_cast<const uint2*>(rowbuf)[c];
          const uint4 wv = make_uint4(push_tag | (h4.x & 0xFFFFu), push_tag | (h4.x >> 16), push_tag | (h4.y & 0xFFFFu),
                                      push_tag | (h4.y >> 16));
          st_peer16(ar.P.p[p] + data_off + 16 * (size_t)c, wv);
        }
      }
      __syncthreads();   // rowbuf and part are free for the next round
    }
  }
  if (ALLRED && ar.tagged) return;   // push only: the sum happens where the rows are consumed (tp_pushed_add_rmsnorm_kernel)
  if (ALLRED) {
    // The sum inside the GEMV: block b of every rank handles the same tile groups (same grid, same rounds on all
    // ranks), so the rows this block has pushed are the rows it now collects - from its OWN region, where the peers'
    // copies are arriving. A word that carries the call's tag has arrived; no flag, no fence. Round after round, the
    // early rounds' rows are there long before the poll gets to them: one NVLink flight is exposed per GEMV.
    __shared__ int failed_s;
    uint8_t* mine = ar.P.p[ar.rank] + ar.off;
    if (tid == 0) failed_s = 0;
    __syncthreads();
    const uint32_t set_limit = *reinterpret_cast<const uint32_t*>(ar.P.p[ar.rank] + kCommLimitOff);
    const int limit = set_limit ? (int)set_limit : kCommSpinLimit;
    for (int r = 0; r < rounds; ++r) {
      const int gidx = r * gridDim.x + blockIdx.x, row0 = 16 * gidx * tiles_per_round;
      const int nrows = max(0, min(N - row0, 16 * tiles_per_round)), nchunk = nrows >> 3;
      const uint8_t* base = mine + kGemvSlotCtrlBytes + kGemvSlotFlagBytes + (size_t)row0 * 4;
      for (int c = tid; c < nchunk; c += kMmaGemvThreads) {
        float acc[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] = 0.f;
        bool bad = false;
        for (int q = 0; q < ar.W && !bad; ++q) {   // rank order, fp32, one rounding: the same bits on every rank
          const uint8_t* src = base + ((size_t)q * N + 8 * (size_t)c) * 4;
          uint4 v0 = ld_peer16(src), v1 = ld_peer16(src + 16);
          int spins = 0;
          while (((((v0.x ^ push_tag) | (v0.y ^ push_tag) | (v0.z ^ push_tag) | (v0.w ^ push_tag) | (v1.x ^ push_tag) |
                    (v1.y ^ push_tag) | (v1.z ^ push_tag) | (v1.w ^ push_tag)) >> 16) != 0)) {
            if (++spins > limit) { bad = true; break; }
            if (spins > 256) __nanosleep(200);
            v0 = ld_peer16(src);
            v1 = ld_peer16(src + 16);
          }
          const uint32_t wd[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
          for (int k = 0; k < 8; ++k) acc[k] += __half2float(__ushort_as_half((unsigned short)(wd[k] & 0xFFFFu)));
        }
        if (bad) {   // a peer's rows never came: say so and leave y's rows alone
          failed_s = 1;
          atomicExch(reinterpret_cast<uint32_t*>(ar.P.p[ar.rank] + kCommErrorOff), COMM_ERR_PEER_WAIT);
        } else {
          uint4 o;
          o.x = as_u32(__floats2half2_rn(acc[0], acc[1]));
          o.y = as_u32(__floats2half2_rn(acc[2], acc[3]));
          o.z = as_u32(__floats2half2_rn(acc[4], acc[5]));
          o.w = as_u32(__floats2half2_rn(acc[6], acc[7]));
          reinterpret_cast<uint4*>(y + row0)[c] = o;
        }
      }
      if (failed_s) break;   // do not spend a whole bounded wait on every further row
    }
    // the last block to finish closes the call: the slot's call counter moves on, the ticket goes back to zero
    uint32_t* ctrl = reinterpret_cast<uint32_t*>(mine);
    __syncthreads();
    if (tid == 0) {
      __threadfence();
      if (atomicAdd(ctrl + 1, 1u) == gridDim.x - 1) {
        ctrl[1] = 0u;
        __threadfence();
        *reinterpret_cast<volatile uint32_t*>(ctrl) = *reinterpret_cast<volatile uint32_t*>(ctrl) + 1u;
      }
    }
  }
}

// Launch shapes found by measurement (llm_decode_kernels_b200/autotune.py) override the heuristic of launch_mma for
// the matrix shapes they name. A small host-side table, filled at set-up time (not thread-safe against launches).
struct MmaTune { int mode, N, K, ksplit, blocks; };
constexpr int kMaxTunes = 128;
static MmaTune g_tunes[kMaxTunes];
static int g_ntunes = 0;

// ksplit in {1, 2, 4, 8}; blocks > 0. ksplit == 0 removes the entry. Returns false when the table is full.
bool gemv_mma_tune(int mode, int N, int K, int ksplit, int blocks) {
  for (int i = 0; i < g_ntunes; ++i) {
    if (g_tunes[i].mode == mode && g_tunes[i].N == N && g_tunes[i].K == K) {
      if (ksplit == 0) g_tunes[i] = g_tunes[--g_ntunes];
      else { g_tunes[i].ksplit = ksplit; g_tunes[i].blocks = blocks; }
      return true;
    }
  }
  if (ksplit == 0) return true;
  if (g_ntunes == kMaxTunes) return false;
  g_tunes[g_ntunes++] = MmaTune{mode, N, K, ksplit, blocks};
  return true;
}

// mode 0: row-major tensors; 1: tile layout; 2: tile layout of a [gate; up] matrix with the SwiGLU epilogue (N outputs)
static cudaError_t launch_mma(int mode, const void* Wp, const void* SZ, const void* x, void* y, int N, int K,
                              int log2G, cudaStream_t st, const NormArgs* norm = nullptr,
                              const AllReduceArgs* allred = nullptr) {
  const int ntiles = mode == 2 ? (N + 7) / 8 : (N + 15) / 16, nunit = K / 128;
  // ksplit warps share a row tile: the smallest split that gives the chip enough warps (measured: with enough tiles
  // a warp per tile, no barrier, is as fast as any split; short of tiles, splitting K wins), as long as a warp keeps
  // at least two units. Blocks: at most two per SM (register limit); with more tile groups than blocks every block
  // takes `rounds` of them, interleaved over the grid so the last round is spread over all SMs.
  const int max_blocks = 2 * kNumSMs, want_warps = (kNumSMs * 16 * 4) / 5;
  int ksplit = 1;
  while (ksplit < kMmaGemvWarps && ntiles * ksplit < want_warps && nunit / (2 * ksplit) >= 2) ksplit *= 2;
  int want_blocks = max_blocks;
  for (int i = 0; i < g_ntunes; ++i) {
    if (g_tunes[i].mode == mode && g_tunes[i].N == N && g_tunes[i].K == K && g_tunes[i].ksplit <= nunit) {
      ksplit = g_tunes[i].ksplit;
      want_blocks = g_tunes[i].blocks;
      break;
    }
  }
  const int tpr = kMmaGemvWarps / ksplit;
  const int groups = (ntiles + tpr - 1) / tpr;
  const int blocks = groups < want_blocks ? groups : want_blocks;
  const int rounds = (groups + blocks - 1) / blocks;
  const size_t smem = (size_t)K * 2 + (size_t)nunit * 8 + kMmaGemvWarps * 16 * 4 + 64;
  {
    static size_t allowed[kMaxDevices] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const bool tracked = dev >= 0 && dev < kMaxDevices;
    if (smem > 48 * 1024 && !(tracked && smem <= allowed[dev])) {   // all variants share one per-device record
      void (*all[])(const uint4*, const half2*, const uint2*, half*, int, int, int, int, int, const NormArgs,
                    const AllReduceArgs) = {
          gemv_w4a16_mma_kernel<false, false, false, false>, gemv_w4a16_mma_kernel<true, false, false, false>,
          gemv_w4a16_mma_kernel<true, true, false, false>,   gemv_w4a16_mma_kernel<true, false, true, false>,
          gemv_w4a16_mma_kernel<true, true, true, false>,    gemv_w4a16_mma_kernel<true, false, false, true>};
      for (auto k : all)
        if (e == cudaSuccess) e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
      if (tracked) allowed[dev] = smem;
    }
  }
  const NormArgs na = norm ? *norm : NormArgs{nullptr, nullptr, nullptr, 0.f};
  const AllReduceArgs ar = allred ? *allred : AllReduceArgs{};
  if (allred && (mode != 1 || norm || blocks > kCommMaxGroups || N % 8)) return cudaErrorInvalidValue;
  auto kern = mode == 0 ? gemv_w4a16_mma_kernel<false, false, false, false>
              : allred  ? gemv_w4a16_mma_kernel<true, false, false, true>
              : norm    ? (mode == 2 ? gemv_w4a16_mma_kernel<true, true, true, false>
                                     : gemv_w4a16_mma_kernel<true, false, true, false>)
                        : (mode == 2 ? gemv_w4a16_mma_kernel<true, true, false, false>
                                     : gemv_w4a16_mma_kernel<true, false, false, false>);
  // Dependent launch pays for the small matrices of a step and costs on large ones (the kernel then runs slower than
  // with an ordinary launch): matrices beyond 64 MB are launched the ordinary way.
  constexpr size_t pdl_max_mb = 64;
  const size_t weight_bytes = (size_t)(mode == 2 ? 2 * N : N) * K / 2;
  if (weight_bytes > (pdl_max_mb << 20)) {
    kern<<<blocks, kMmaGemvThreads, smem, st>>>((const uint4*)Wp, (const half2*)SZ, (const uint2*)x, (half*)y, N, K,
                                                log2G, ksplit, rounds, na, ar);
    return cudaPeekAtLastError();
  }
  return launch_pdl(kern, dim3(blocks), dim3(kMmaGemvThreads), smem, st, (const uint4*)Wp, (const half2*)SZ,
                    (const uint2*)x, (half*)y, N, K, log2G, ksplit, rounds, na, ar);
}

// ---- tile layout -------------------------------------------------------------------------------------------------------
// One thread per 16-byte piece of the output: 68 pieces per (tile, unit), see gemv_w4a16_mma_kernel. Rows past N are
// stored as zero weights with scale 0, so they add nothing.
__global__ void gemv_tile_repack_kernel(const uint4* __restrict__ Wp, const half2* __restrict__ SZ,
                                        uint4* __restrict__ out, int N, int K, int log2G, int pair) {
  // pair = 0: slot r of tile T is row 16 T + r. pair = I > 0 ([gate; up] of I rows each): slot r < 8 is gate row
  // 8 T + r, slot r >= 8 is up row I + 8 T + (r - 8).
  const int nunit = K >> 7, u = blockIdx.x, tile = blockIdx.y, idx = threadIdx.x;
  if (idx >= kTileUnitBytes / 16) return;
  auto row_of = [&](int slot) {
    if (!pair) return 16 * tile + slot < N ? 16 * tile + slot : -1;
    const int i = 8 * tile + (slot & 7);
    return i < pair ? i + (slot >= 8 ? pair : 0) : -1;
  };
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  if (idx < 64) {
    const int lane = idx & 31, g = lane >> 2, t = lane & 3, row = row_of(g + 8 * (idx >> 5));
    if (row >= 0) v = Wp[(size_t)row * (K >> 5) + 4 * u + t];
  } else {
    uint32_t e[4] = {0u, 0u, 0u, 0u};
    for (int k = 0; k < 4; ++k) {
      const int row = row_of(4 * (idx - 64) + k);
      if (row >= 0) e[k] = as_u32(SZ[(size_t)row * (K >> log2G) + ((u << 7) >> log2G)]);
    }
    v = make_uint4(e[0], e[1], e[2], e[3]);
  }
  out[((size_t)tile * nunit + u) * (kTileUnitBytes / 16) + idx] = v;
}

// gate_up != 0: N = 2 I rows [gate; up], paired layout (I / 8 tiles, rounded up)
size_t gemv_tiled_bytes(int N, int K, int gate_up) {
  const int tiles = gate_up ? (N / 2 + 7) / 8 : (N + 15) / 16;
  return (size_t)tiles * (K / 128) * kTileUnitBytes;
}

cudaError_t gemv_tile_repack_dispatch(const void* Wp, const void* SZ, void* out, int N, int K, int log2G, int gate_up,
                                      cudaStream_t st) {
  const int tiles = gate_up ? (N / 2 + 7) / 8 : (N + 15) / 16;
  gemv_tile_repack_kernel<<<dim3(K / 128, tiles), 96, 0, st>>>((const uint4*)Wp, (const half2*)SZ, (uint4*)out, N, K,
                                                               log2G, gate_up ? N / 2 : 0);
  return cudaPeekAtLastError();
}

// swiglu != 0: Wt is the paired layout of a [gate; up] matrix and y receives N = I values silu(gate) * up
cudaError_t gemv_w4a16_tiled_dispatch(const void* Wt, const void* x, void* y, int N, int K, int swiglu,
                                      cudaStream_t st) {
  return launch_mma(swiglu ? 2 : 1, Wt, nullptr, x, y, N, K, 7, st);
}

// y = all-reduce over the W ranks of (this rank's W x): the ALLRED form of the kernel. peers[r] = rank r's exchange
// block as this process sees it, slot_off = offset of a GEMV slot (gemv_slot_bytes) inside every block.
cudaError_t gemv_w4a16_tiled_allreduce_dispatch(const void* Wt, const void* x, void* y, int N, int K,
                                                const void* const* peers, int rank, int W, size_t slot_off,
                                                int tagged, cudaStream_t st) {
  AllReduceArgs ar = {};
  for (int r = 0; r < W; ++r) ar.P.p[r] = (uint8_t*)peers[r];
  ar.rank = rank;
  ar.W = W;
  ar.off = slot_off;
  ar.tagged = tagged;
  return launch_mma(1, Wt, nullptr, x, y, N, K, 7, st, nullptr, &ar);
}
size_t gemv_allreduce_slot_bytes(int N, int W) { return gemv_slot_bytes(N, W); }

// residual add + RMSNorm + GEMV (+ SwiGLU) in one launch: see NormArgs
cudaError_t gemv_w4a16_tiled_norm_dispatch(const void* Wt, const void* x_in, const void* delta, const void* norm_w,
                                           float eps, void* x_out, void* y, int N, int K, int swiglu, cudaStream_t st) {
  const NormArgs na = {(const uint2*)delta, (const uint2*)norm_w, (uint2*)x_out, eps};
  return launch_mma(swiglu ? 2 : 1, Wt, nullptr, x_in, y, N, K, 7, st, &na);
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
  return launch_pdl(gemv_w4a16_kernel<R, UNR>, dim3(blocks), dim3(32 * warps), smem, st, (const uint4*)Wp,
                    (const half2*)SZ, (const uint4*)x, (half*)y, N, K, log2G);
}

// stage 0: plain kernel. stage >= 1 with R in {1,2,4,8} and warps in 1..8: the row-per-warp kernel in that
// configuration. R == 16: the segmented kernel. Anything else (R == 0): the tensor-core kernel, or the segmented one
// where the shape rules it out.
cudaError_t gemv_w4a16_dispatch(int stage, int R, int warps, const void* Wp, const void* SZ, const void* x, void* y,
                                int N, int K, int log2G, cudaStream_t st) {
  if (stage == 0) {
    const int w = (warps >= 1 && warps <= 8) ? warps : 4;
    return launch_pdl(gemv_w4a16_plain_kernel, dim3((N + w - 1) / w), dim3(32 * w), 0, st, (const uint32_t*)Wp,
                      (const half2*)SZ, (const half*)x, (half*)y, N, K, log2G);
  }
  if (!(R == 1 || R == 2 || R == 4 || R == 8) || warps < 1 || warps > 8) {
    const bool x_ok = (reinterpret_cast<uintptr_t>(x) & 7u) == 0;
    // the library's own choice: the tensor-core kernel where the shape allows (R == 16 asks for the segmented one)
    if (R != 16 && x_ok && K % 128 == 0 && log2G >= 7) return launch_mma(0, Wp, SZ, x, y, N, K, log2G, st);
    if ((reinterpret_cast<uintptr_t>(y) & 3u) == 0 && x_ok)
      return launch_seg(Wp, SZ, x, y, N, K, log2G, st);   // the segmented kernel
    R = 2;   // y not 4-byte aligned (the segmented kernel stores row pairs): row-per-warp kernel
    warps = 4;
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
