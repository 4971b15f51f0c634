// Paged split-K decode attention (one query token per sequence, grouped-query heads) and its combine step.
//
// Replaces paged_attention_launch of the reference (kernels/paged_attention.cu:429-461, bound at
// kernels/bindings.cpp:45-62), generalised to a batch of sequences and to head_dim 64 or 128.
//
// Layout: caches [pages, n_kv, P, D] fp16 (P = 2^log2P tokens per page); block table bt[b, i] = physical page
// of tokens [i P, (i+1) P) of sequence b; context length of sequence b = pos[b] + 1, read on the device so one
// captured graph serves every step. Split s of a sequence owns tokens [s PS, min(ctx, (s+1) PS)).
//
// Grid (n_kv, max_splits, B), 128 threads. A block handles ALL heads of one kv group, so every K/V byte is
// fetched from HBM once. Inside a block each warp walks its own 32-token tiles with a private online-softmax
// state (no block barrier in the loop):
//   scores : lane t owns token t of the tile, holds that K row in registers and dots it with every head's
//            query (pre-scaled by 1/sqrt(D), fp32, broadcast reads from shared memory) - no shuffles;
//   p      : exp(score - running max) goes to a per-warp shared tile [32 tokens][HPG heads];
//   output : lane l owns D/32 consecutive output dims of every head and walks the tile's V rows
//            (each row one coalesced 128- or 256-byte read), acc[h][d] += p[t][h] * v[t][d].
// The four warps are merged once through shared memory with the max-rescale rule; a block that is the
// only live split of its sequence normalises and writes fp16 `out` itself, otherwise it writes
// un-normalised fp32 partials (o, m, l) and the combine kernel finishes:
//   M = max_s m_s,  L = sum_s l_s e^(m_s - M),  O = sum_s o_s e^(m_s - M) / L.
#include "common.cuh"
#include <math_constants.h>

namespace b200 {

constexpr int kAttnThreads = 128;
constexpr int kAttnWarps = kAttnThreads / 32;

template <int D, int HPG>
__global__ void __launch_bounds__(kAttnThreads)
paged_attn_partial_kernel(const half* __restrict__ q, const half* __restrict__ kc, const half* __restrict__ vc,
                          const int* __restrict__ bt, int bt_stride, const int* __restrict__ pos_ptr, int n_kv,
                          int log2P, int PS, float scale, float* __restrict__ o_part, float* __restrict__ m_part,
                          float* __restrict__ l_part, half* __restrict__ out, int max_splits) {
  constexpr int DPL = D / 32;      // output dims owned by one lane
  constexpr int CHUNKS = D / 8;    // 16-byte chunks per K/V row
  __shared__ __align__(16) float q_s[HPG][D];
  __shared__ __align__(16) float p_s[kAttnWarps][32][HPG];
  __shared__ long long row_s[kAttnWarps][32];  // element offset of each tile token's row in the caches
  __shared__ float wm[kAttnWarps][HPG], wl[kAttnWarps][HPG];
  __shared__ float wo[kAttnWarps][HPG][D];

  const int kvh = blockIdx.x, split = blockIdx.y, b = blockIdx.z;
  const int n_q = n_kv * HPG;
  const int ctx = pos_ptr[b] + 1;
  const int nsplit = min((ctx + PS - 1) / PS, max_splits);
  if (split >= nsplit) return;
  const int t0 = split * PS, t1 = min(ctx, t0 + PS);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int* btb = bt + (size_t)b * bt_stride;
  const int pmask = (1 << log2P) - 1;

  for (int i = tid; i < HPG * D; i += kAttnThreads)
    q_s[i / D][i % D] = __half2float(q[((size_t)b * n_q + kvh * HPG) * D + i]) * scale;
  __syncthreads();

  float m[HPG], l[HPG], acc[HPG][DPL];
#pragma unroll
  for (int h = 0; h < HPG; ++h) {
    m[h] = -CUDART_INF_F;
    l[h] = 0.f;
#pragma unroll
    for (int d = 0; d < DPL; ++d) acc[h][d] = 0.f;
  }

  for (int tile = t0 + 32 * warp; tile < t1; tile += 32 * kAttnWarps) {
    const int t = tile + lane;
    const bool valid = t < t1;
    const int tc = valid ? t : t1 - 1;
    const long long row = ((((long long)btb[tc >> log2P] * n_kv + kvh) << log2P) + (tc & pmask)) * D;
    row_s[warp][lane] = row;

    // ---- scores: this lane's token against every head of the group
    float s[HPG];
#pragma unroll
    for (int h = 0; h < HPG; ++h) s[h] = 0.f;
    const uint4* kp = reinterpret_cast<const uint4*>(kc + row);
#pragma unroll
    for (int c0 = 0; c0 < CHUNKS; c0 += 8) {
      uint4 kv[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) kv[c] = __ldg(kp + c0 + c);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float kf[8];
        unpack8(kv[c], kf);
#pragma unroll
        for (int h = 0; h < HPG; ++h) {
          const float4 qa = *reinterpret_cast<const float4*>(&q_s[h][(c0 + c) * 8]);
          const float4 qb = *reinterpret_cast<const float4*>(&q_s[h][(c0 + c) * 8 + 4]);
          s[h] = fmaf(kf[0], qa.x, fmaf(kf[1], qa.y, fmaf(kf[2], qa.z, fmaf(kf[3], qa.w, s[h]))));
          s[h] = fmaf(kf[4], qb.x, fmaf(kf[5], qb.y, fmaf(kf[6], qb.z, fmaf(kf[7], qb.w, s[h]))));
        }
      }
    }

    // ---- online softmax update (m uniform across the warp, l kept as per-lane partial sums)
#pragma unroll
    for (int h = 0; h < HPG; ++h) {
      const float sv = valid ? s[h] : -CUDART_INF_F;
      const float mn = fmaxf(m[h], warp_max(sv));
      const float alpha = __expf(m[h] - mn);  // first tile: e^(-inf) = 0
      const float p = __expf(sv - mn);        // masked lane: 0
      l[h] = l[h] * alpha + p;
      m[h] = mn;
#pragma unroll
      for (int d = 0; d < DPL; ++d) acc[h][d] *= alpha;
      p_s[warp][lane][h] = p;
    }
    __syncwarp();

    // ---- output: walk the tile's V rows, 4 rows in flight
    const int nt = min(32, t1 - tile);
    for (int j0 = 0; j0 < nt; j0 += 4) {
      float vf[4][DPL];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int jj = min(j0 + j, nt - 1);
        const half* vp = vc + row_s[warp][jj] + lane * DPL;
        if (DPL == 2) {
          const float2 f = __half22float2(*reinterpret_cast<const half2*>(vp));
          vf[j][0] = f.x; vf[j][1] = f.y;
        } else {
          const uint2 u = *reinterpret_cast<const uint2*>(vp);
          const float2 f0 = __half22float2(as_h2(u.x)), f1 = __half22float2(as_h2(u.y));
          vf[j][0] = f0.x; vf[j][1] = f0.y; vf[j][DPL - 2] = f1.x; vf[j][DPL - 1] = f1.y;
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (j0 + j < nt) {
#pragma unroll
          for (int h0 = 0; h0 < HPG; h0 += 4) {
            float ph[4];
            if (HPG >= 4) {
              const float4 p4 = *reinterpret_cast<const float4*>(&p_s[warp][j0 + j][h0]);
              ph[0] = p4.x; ph[1] = p4.y; ph[2] = p4.z; ph[3] = p4.w;
            } else {
#pragma unroll
              for (int k = 0; k < 4; ++k) ph[k] = k < HPG ? p_s[warp][j0 + j][k < HPG ? k : 0] : 0.f;
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              if (h0 + k < HPG) {
#pragma unroll
                for (int d = 0; d < DPL; ++d) acc[h0 + k][d] = fmaf(ph[k], vf[j][d], acc[h0 + k][d]);
              }
            }
          }
        }
      }
    }
    __syncwarp();  // p_s / row_s are rewritten by the next tile
  }

  // ---- merge the warps
#pragma unroll
  for (int h = 0; h < HPG; ++h) {
    const float lw = warp_sum(l[h]);
    if (lane == 0) { wm[warp][h] = m[h]; wl[warp][h] = lw; }
#pragma unroll
    for (int d = 0; d < DPL; ++d) wo[warp][h][lane * DPL + d] = acc[h][d];
  }
  __syncthreads();
  for (int i = tid; i < HPG * D; i += kAttnThreads) {
    const int h = i / D, d = i % D, head = kvh * HPG + h;
    float M = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) M = fmaxf(M, wm[w][h]);
    float o = 0.f, L = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float a = __expf(wm[w][h] - M);  // a warp that had no tile: e^(-inf) = 0
      o = fmaf(a, wo[w][h][d], o);
      L = fmaf(a, wl[w][h], L);
    }
    const size_t hq = (size_t)b * n_q + head;
    if (nsplit == 1) {
      out[hq * D + d] = __float2half(o / L);
    } else {
      o_part[(hq * max_splits + split) * D + d] = o;
      if (d == 0) { m_part[hq * max_splits + split] = M; l_part[hq * max_splits + split] = L; }
    }
  }
}

// Grid (n_q, B), D threads: thread d merges dim d of one head over the live splits.
__global__ void paged_attn_combine_kernel(const float* __restrict__ o_part, const float* __restrict__ m_part,
                                          const float* __restrict__ l_part, const int* __restrict__ pos_ptr, int PS,
                                          int max_splits, int D, half* __restrict__ out) {
  const int head = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const int ctx = pos_ptr[b] + 1;
  const int nsplit = min((ctx + PS - 1) / PS, max_splits);
  if (nsplit <= 1) return;  // the partial kernel already wrote `out`
  const size_t hq = (size_t)b * gridDim.x + head;
  const float* m = m_part + hq * max_splits;
  const float* l = l_part + hq * max_splits;
  const float* o = o_part + hq * max_splits * D + d;
  float M = -CUDART_INF_F;
  for (int s = 0; s < nsplit; ++s) M = fmaxf(M, __ldg(m + s));
  float L = 0.f, acc = 0.f;
#pragma unroll 4
  for (int s = 0; s < nsplit; ++s) {
    const float a = __expf(__ldg(m + s) - M);
    L = fmaf(a, __ldg(l + s), L);
    acc = fmaf(a, o[(size_t)s * D], acc);
  }
  out[hq * D + d] = __float2half(acc / L);
}

template <int D>
static cudaError_t launch_partial(int hpg, dim3 grid, cudaStream_t st, const half* q, const half* kc, const half* vc,
                                  const int* bt, int bt_stride, const int* pos, int n_kv, int log2P, int PS,
                                  float scale, float* o_part, float* m_part, float* l_part, half* out,
                                  int max_splits) {
#define B200_ATTN_CASE(H)                                                                                   \
  case H:                                                                                                   \
    paged_attn_partial_kernel<D, H><<<grid, kAttnThreads, 0, st>>>(q, kc, vc, bt, bt_stride, pos, n_kv,     \
                                                                   log2P, PS, scale, o_part, m_part, l_part, \
                                                                   out, max_splits);                        \
    break;
  switch (hpg) {
    B200_ATTN_CASE(1) B200_ATTN_CASE(2) B200_ATTN_CASE(4) B200_ATTN_CASE(8)
    default: return cudaErrorInvalidValue;
  }
#undef B200_ATTN_CASE
  return cudaPeekAtLastError();
}

cudaError_t paged_attention_dispatch(const void* q, const void* kc, const void* vc, const int* bt, int bt_stride,
                                     const int* pos, int B, int n_q, int n_kv, int D, int log2P, int PS,
                                     int max_splits, float* o_part, float* m_part, float* l_part, void* out,
                                     cudaStream_t st) {
  const int hpg = n_q / n_kv;
  const float scale = 1.0f / sqrtf((float)D);
  const dim3 grid(n_kv, max_splits, B);
  cudaError_t e;
  if (D == 64)
    e = launch_partial<64>(hpg, grid, st, (const half*)q, (const half*)kc, (const half*)vc, bt, bt_stride, pos, n_kv,
                           log2P, PS, scale, o_part, m_part, l_part, (half*)out, max_splits);
  else
    e = launch_partial<128>(hpg, grid, st, (const half*)q, (const half*)kc, (const half*)vc, bt, bt_stride, pos,
                            n_kv, log2P, PS, scale, o_part, m_part, l_part, (half*)out, max_splits);
  if (e != cudaSuccess) return e;
  if (max_splits > 1) {
    paged_attn_combine_kernel<<<dim3(n_q, B), D, 0, st>>>(o_part, m_part, l_part, pos, PS, max_splits, D,
                                                          (half*)out);
    e = cudaPeekAtLastError();
  }
  return e;
}

}  // namespace b200

// ---- attention without any allocation by the caller --------------------------------------------------------------------
// b200_paged_attention needs three scratch arrays for the split-K partials, and its callers get them from
// cudaMalloc (or torch). Some callers cannot allocate device memory at all: a plugin running inside a host
// application that owns the allocator and hands out nothing, code on a latency-critical path where an allocation may
// synchronise the device, a process whose memory budget was fixed at start-up. For them the partials live in this
// file-scope device array instead. Every GPU that loads the library holds it until the process exits.
//   capacity: 64 query heads x 32 splits x head_dim 128 (about 1 MB), one sequence per call.
// The array is shared by every call on the device and keeps whatever the previous call left; nothing in it has to
// start at zero (the combine step reads only the slots the partial kernel of the same call has just written), so it
// is never cleared. Two calls that overlap on the GPU (different streams) would overwrite each other's partials.
#include "../../include/b200decode.h"

namespace {
constexpr int kNoAllocMaxHeads = 64, kNoAllocMaxSplits = 32, kNoAllocMaxD = 128;
constexpr size_t kNoAllocO = (size_t)kNoAllocMaxHeads * kNoAllocMaxSplits * kNoAllocMaxD;
constexpr size_t kNoAllocML = (size_t)kNoAllocMaxHeads * kNoAllocMaxSplits;
static __device__ __align__(256) float g_attn_scratch[kNoAllocO + 2 * kNoAllocML];

constexpr int kMaxDevices = 64;
float* g_attn_scratch_ptr[kMaxDevices] = {};   // device address of the array, per device, filled on first use
}  // namespace

extern "C" int b200_paged_attention_noalloc(const void* q, const void* kc, const void* vc, const int* bt, const int* pos,
                                            int n_q, int n_kv, int D, int log2P, int PS, int max_splits, void* out,
                                            void* stream) {
  if (!q || !kc || !vc || !bt || !pos || !out || n_q <= 0 || n_kv <= 0 || PS <= 0 || max_splits <= 0 || log2P < 0 ||
      log2P >= 16)
    return B200_ERR_ARG;
  if ((D != 64 && D != 128) || n_q % n_kv) return B200_ERR_SHAPE;
  const int hpg = n_q / n_kv;
  if (hpg != 1 && hpg != 2 && hpg != 4 && hpg != 8) return B200_ERR_SHAPE;
  if (n_q > kNoAllocMaxHeads || max_splits > kNoAllocMaxSplits || D > kNoAllocMaxD) return B200_ERR_LIMIT;
  if ((reinterpret_cast<uintptr_t>(kc) & 15u) || (reinterpret_cast<uintptr_t>(vc) & 15u)) return B200_ERR_ALIGN;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return B200_ERR_LAUNCH;
  if (!g_attn_scratch_ptr[dev]) {
    // In host code `g_attn_scratch` is only a handle for the symbol, not a device address: ask the runtime for the
    // address on the current device, once per device.
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_attn_scratch) != cudaSuccess || !p) return B200_ERR_LAUNCH;
    g_attn_scratch_ptr[dev] = p;
  }
  float* o_part = g_attn_scratch_ptr[dev];
  float* m_part = o_part + (size_t)n_q * max_splits * D;
  float* l_part = m_part + (size_t)n_q * max_splits;
  const cudaError_t e = b200::paged_attention_dispatch(q, kc, vc, bt, 1 << 30, pos, 1, n_q, n_kv, D, log2P, PS,
                                                       max_splits, o_part, m_part, l_part, out,
                                                       reinterpret_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}
